// The engine: a model, its cache, and the one step function that everything else drives.
//
// Engine::step(items) runs the tokens it is given, as one batch, from the cache that earlier steps
// left, and returns the float32 logits at the wanted places.  A step may hold prompts of unequal
// lengths (all their tokens at once), single next tokens, or both; a sequence's start position is
// the cache's own record of its length.  The generation loop, the command line, the programming
// entry point and the trace replay program all go through this function.
//
// The reference's counterpart is Graph::execute(tokens, logits, nr_past, prefill)
// (src/core/graph.cpp:166-197): one sequence, the caller passes the past length, logits of the last
// token only or none at all.
#pragma once
#include <map>
#include <memory>
#include <string>
#include <vector>

#include "cache/cache.h"
#include "config/config.h"
#include "engine/step_context.h"
#include "models/decoder.h"

namespace illm {

struct EngineOptions {
    std::string dtype = "bfloat16";     // "bfloat16": serving kernels; "float32": everything in true 32-bit
    int device_id = 0;
    long long max_tokens = 4096;        // tokens that live sequences may hold together (sizes the cache);
                                        // <= 0: what mem_fraction of the memory left beside the weights holds
    double mem_fraction = 0.9;
    long long max_seq_len = 0;          // longest sequence; 0: the model's max positions
    int max_batch = 0;                  // slots; 0: max_tokens / page_size
    int page_size = 64;
    bool cuda_graphs = true;            // replay one-token-per-sequence steps and single prompts from captured CUDA graphs
    std::string gemm = "auto";          // bfloat16 products: "auto" | "tc" | "library" (see ops::GemmBackend)
    bool poison_freed_pages = false;    // fill pages that go back to the pool with NaN (a check, not for serving)
    void* stream = nullptr;             // the CUDA stream to work on; nullptr: one of the engine's own

    static EngineOptions from_json(const Json& j);
};

struct Limits {
    int max_batch;          // sequences that can be live together (slots)
    int num_pages;          // pages of the cache
    int page_size;
    long long max_seq_len;
};

struct StepItem {
    int slot = 0;
    std::vector<int> tokens;
    std::vector<int> want;      // places among `tokens` whose logits are asked for
};

// Logits of a step on the device: float32 [rows, vocab], valid until the engine's next step.
struct LogitsRef {
    const float* p = nullptr;
    long long rows = 0, vocab = 0;
};

constexpr int kPromptBucket = 64;               // tokens; also the rows the library's products are rounded up to
constexpr int kPromptGraphMaxTokens = 1024;     // longer prompts keep the GPU busy longer than the host needs to issue them

class Engine {
public:
    Engine(std::unique_ptr<ArchConfig> config, const EngineOptions& options);
    ~Engine();
    static std::unique_ptr<Engine> from_folder(const std::string& folder, const EngineOptions& options, const std::string& model_name = "");
    // Random weights made on the device, without a file.
    static std::unique_ptr<Engine> from_config(std::unique_ptr<ArchConfig> config, const EngineOptions& options, unsigned long long seed);
    void load_folder(const std::string& folder);
    void load_random(unsigned long long seed);

    int new_sequence();
    void end_sequence(int slot);
    long long sequence_length(int slot) const;
    Limits limits() const;

    // Run one step; float32 logits [number of wanted places, vocab] on the device, in the order of the
    // items and of each item's `want`.  `device_ids` (int32 on the device, one id per item) gives the
    // tokens of a one-token-per-sequence step without a round trip through the host, e.g. straight from
    // the sampling kernel; the items' tokens are then placeholders of length one.
    LogitsRef step(const std::vector<StepItem>& items, const int* device_ids = nullptr);

    // Pay what is paid once, before the first request: prompt steps for every bucket of 64 tokens up to
    // prompt_tokens (the library chooses its kernels per shape of a product, about 10 ms each at 7B
    // size; the second step of a bucket of up to 1,024 tokens captures its CUDA graph), and for every
    // batch size a few one-token steps, of which the second captures the graph that later steps of that
    // size replay.  Uses free slots and pages only and gives them back; sizes that do not fit the cache
    // are left out.
    void warm_up(long long prompt_tokens, const std::vector<int>& batch_sizes);
    // Read the kernels' error words (synchronises); EngineError naming what a kernel reported.
    void check_device_errors();

    // Copy a step's logits to host memory (synchronises).
    void read_logits(const LogitsRef& logits, float* host);
    // Sampled token ids (int32 on the device) on their way to the host: the copy starts behind what the
    // stream holds now and is waited for alone, not for work queued later.
    int read_tokens_async(const int* toks, int n);      // returns a ticket
    std::vector<int> finish_read(int ticket);

    Device& device() { return *device_; }
    Runtime& runtime() { return rt_; }
    DecoderModel& model() { return *model_; }
    SequenceCache& cache() { return *cache_; }
    const ArchConfig& config() const { return *config_; }
    const EngineOptions& options() const { return options_; }
    long long vocab_size() const { return model_->spec.vocab_size; }
    size_t last_upload_bytes() const { return last_upload_bytes_; }
    int graphs_captured() const;
    void forget_graphs() { drop_graphs(false); }     // e.g. after a change of which kernels run the products
    bool loaded() const { return loaded_; }

private:
    struct GraphEntry;
    long long tokens_that_fit(double fraction) const;
    StepContext make_context(const StepPlan& plan, const std::vector<int>& ids, const std::vector<int>& want_rows, int* into,
                             std::vector<const int*>* tables_dev);
    LogitsRef run_forward(const StepContext& ctx, const std::vector<const int*>& tables);
    bool prompt_step_graphed(int slot, const std::vector<int>& ids, const std::vector<int>& want_rows, LogitsRef* out);
    LogitsRef decode_step_graphed(const StepPlan& plan, const std::vector<int>& ids, const std::vector<int>& want_rows,
                                  const int* device_ids);
    LogitsRef capture_and_run(const std::string& key, const StepPlan& plan, const std::vector<int>& ids,
                              const std::vector<int>& want_rows, const int* device_ids);
    LogitsRef replay(GraphEntry& e, const StepPlan& plan, const std::vector<int>& ids, const std::vector<int>& want_rows,
                     const int* device_ids);
    void drop_graphs(bool keep_seen);
    size_t context_ints(int T, int B, int K) const;

    std::unique_ptr<ArchConfig> config_;
    EngineOptions options_;
    std::unique_ptr<Device> device_;
    Runtime rt_;
    std::unique_ptr<DecoderModel> model_;
    std::unique_ptr<SequenceCache> cache_;
    bool loaded_ = false;
    int pad_safe_ = -1, graph_safe_ = -1;
    size_t last_upload_bytes_ = 0;

    std::unique_ptr<StepContextBuilder> builder_;
    struct TokRead { int* host = nullptr; int cap = 0; int n = 0; cudaEvent_t done = nullptr; };
    TokRead tok_reads_[4];
    int tok_next_ = 0;
    std::map<std::string, std::unique_ptr<GraphEntry>> graphs_;
};

}  // namespace illm
