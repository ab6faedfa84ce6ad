// The programming entry point, in the manner of the reference's inferllm::Model (include/model.h:14-59):
// a ModelConfig, then load, init, prefill, decode, decode_iter, get_remain_token, reset_token,
// decode_summary, with the same names and meanings.  Differences that the scope of this library
// brings: prompts are lists of token ids (there is no tokenizer here), the model folder holds
// config.json and safetensors, the model class is chosen by config.json unless `model_name` names a
// registered one, and generate() adds batches of requests on top of the reference's single
// conversation.
#pragma once
#include <memory>
#include <string>
#include <vector>

#include "engine/engine.h"
#include "engine/generate.h"
#include "sampling/sampler.h"

namespace illm {

// Fields of the reference's ModelConfig (include/model.h:14-23).  compt_type: "bfloat16" or "float32";
// device_type must be "gpu"; nr_thread and enable_mmap are accepted and have no effect (no CPU threads
// compute here, and weight files are always memory-mapped); nr_ctx is the longest sequence; device_id
// the GPU ordinal.  max_tokens (not in the reference) sizes the cache for batches; 0: nr_ctx.
struct ModelConfig {
    std::string compt_type = "bfloat16";
    std::string device_type = "gpu";
    unsigned nr_thread = 1;
    unsigned nr_ctx = 2048;
    int device_id = 0;
    bool enable_mmap = true;
    long long max_tokens = 0;
    int max_batch = 0;
    // further engine options (not in the reference)
    int page_size = 64;
    bool cuda_graphs = true;
    std::string gemm = "auto";
    bool poison_freed_pages = false;
    void* stream = nullptr;
};

class Model {
public:
    explicit Model(const ModelConfig& config, const std::string& model_name = "");
    ~Model();

    // Load config.json and the safetensors weights of a model folder.
    void load(const std::string& model_path);
    // Random weights for a typed configuration, made on the device.
    void load_random(std::unique_ptr<ArchConfig> config, unsigned long long seed);
    // Sampling parameters of the conversation (include/model.h:38-39); seed < 0: from the clock.
    void init(unsigned top_k, float top_p, float temp, float repeat_penalty, int repeat_last_n, long long seed, int end_token);

    // ---- the single conversation of the reference's API
    unsigned get_remain_token();
    void reset_token();
    // Run a prompt into the cache without producing a token (src/core/model_imp.cpp:22-34).
    void prefill(const std::vector<int>& prompt);
    // Run further input tokens and return the first answer token (:37-52).
    int decode(const std::vector<int>& user_input);
    // Feed the previous answer token and return the next one (:55-64); timed.
    int decode_iter();
    // Totals in the reference's wording (src/core/model_imp.cpp:133-142).
    std::string decode_summary() const;

    // ---- batches of requests
    // stop_ids == nullptr: the end token given to init(); where that is one of the configuration's end
    // tokens (or init() was given none), all of them: the reference ends a turn on its one end token
    // (application/llama/llama.cpp:237), a config.json may name several.
    GenerationResult generate(const std::vector<std::vector<int>>& prompts, long long max_new_tokens = 128,
                              const std::vector<int>* stop_ids = nullptr, const TokenCallback& on_token = nullptr);
    void warm_up(long long prompt_tokens, const std::vector<int>& batch_sizes);

    Engine& engine();
    bool has_end_token() const { return has_end_token_; }
    int end_token() const { return end_token_; }
    const std::vector<int>& end_tokens() const { return end_tokens_; }
    const SamplingParams& sampling() const { return sampling_; }

private:
    EngineOptions options() const;
    void take_end_tokens();
    int sample(const LogitsRef& logits);
    ModelConfig config_;
    std::string model_name_;
    std::unique_ptr<Engine> engine_;
    SamplingParams sampling_;
    std::unique_ptr<Sampler> single_sampler_;
    bool has_end_token_ = false;
    int end_token_ = 0;
    std::vector<int> end_tokens_;
    int slot_ = -1;
    std::vector<int> history_;
    int n_generated_ = 0;
    bool has_pre_token_ = false;
    int pre_token_ = 0;
    double decode_s_ = 0;
    long long decode_tokens_ = 0;
};

}  // namespace illm
