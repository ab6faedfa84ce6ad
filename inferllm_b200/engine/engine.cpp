#include "engine/engine.h"

#include <algorithm>
#include <cstring>
#include <set>

#include "util/log.h"
#include "weights/loader.h"

namespace illm {

EngineOptions EngineOptions::from_json(const Json& j) {
    EngineOptions o;
    if (!j.is_object()) return o;
    if (j.at("dtype").is_string()) o.dtype = j.at("dtype").as_string();
    if (j.at("device_id").is_int()) o.device_id = (int)j.at("device_id").as_int();
    if (j.has("max_tokens")) o.max_tokens = j.at("max_tokens").is_int() ? j.at("max_tokens").as_int() : 0;
    if (j.at("mem_fraction").is_number()) o.mem_fraction = j.at("mem_fraction").as_double();
    if (j.at("max_seq_len").is_int()) o.max_seq_len = j.at("max_seq_len").as_int();
    if (j.at("max_batch").is_int()) o.max_batch = (int)j.at("max_batch").as_int();
    if (j.at("page_size").is_int()) o.page_size = (int)j.at("page_size").as_int();
    if (j.at("cuda_graphs").is_bool()) o.cuda_graphs = j.at("cuda_graphs").as_bool();
    if (j.at("gemm").is_string()) o.gemm = j.at("gemm").as_string();
    if (j.at("poison_freed_pages").is_bool()) o.poison_freed_pages = j.at("poison_freed_pages").as_bool();
    if (j.at("stream").is_int()) o.stream = (void*)(uintptr_t)j.at("stream").as_int();
    return o;
}

struct Engine::GraphEntry {
    cudaGraphExec_t exec = nullptr;     // nullptr: the shape has been seen once and is captured the next time
    cudaGraph_t graph = nullptr;
    int* ctx_buf = nullptr;             // the step's index arrays: the static input of the graph
    LogitsRef out;
    long long launches = 0;
};

static DType engine_dtype(const std::string& name) {
    if (name == "bfloat16" || name == "bf16") return DType::BF16;
    if (name == "float32" || name == "fp32") return DType::F32;
    throw EngineError("dtype '" + name + "' is not supported (bfloat16 or float32)");
}

static long long ceil_div(long long a, long long b) { return (a + b - 1) / b; }

Engine::Engine(std::unique_ptr<ArchConfig> config, const EngineOptions& options) : config_(std::move(config)), options_(options) {
    const DType dtype = engine_dtype(options.dtype);
    if (options.page_size <= 0) throw EngineError("page_size must be positive");
    device_.reset(new Device(options.device_id, (cudaStream_t)options.stream));
    rt_.dev = device_.get();
    rt_.dtype = dtype;
    rt_.page_size = options.page_size;
    rt_.gemm = ops::gemm_backend_from_name(options.gemm);
    model_.reset(new DecoderModel(config_->model_spec(), &rt_));
    const ModelSpec& spec = model_->spec;
    const long long max_seq = std::min(options.max_seq_len > 0 ? options.max_seq_len : spec.max_positions, spec.max_positions);
    long long max_tokens = options.max_tokens;
    if (max_tokens <= 0) max_tokens = tokens_that_fit(options.mem_fraction);
    const int num_pages = (int)std::max<long long>(1, ceil_div(max_tokens, options.page_size));
    const int num_slots = options.max_batch > 0 ? options.max_batch : num_pages;
    cache_.reset(new SequenceCache(model_->cache_requests(), num_slots, num_pages, options.page_size, max_seq, device_.get(), dtype,
                                   options.poison_freed_pages));
    builder_.reset(new StepContextBuilder(device_.get(), &rt_));
    for (TokRead& t : tok_reads_) check_cuda(cudaEventCreateWithFlags(&t.done, cudaEventDisableTiming), "cudaEventCreate");
    // say once which attention kernels the model's layers get: a head size that the tensor-core kernels
    // do not take falls to the general kernel, which is right but far slower on prompts
    std::set<std::string> said;
    for (const LayerSpec& ls : spec.layers) {
        if (ls.mixer.kind != "attention" || !ls.mixer.has("n_heads")) continue;
        const int nh = (int)ls.mixer.get_int("n_heads"), nkv = (int)ls.mixer.get_int("n_kv_heads", nh), d = (int)ls.mixer.get_int("head_dim", 0);
        const std::string what = ops::attention_kernels_for(dtype, nh, nkv, d, options.page_size);
        const std::string line = std::to_string(nh) + " heads over " + std::to_string(nkv) + " of size " + std::to_string(d) + ", pages of " +
                                 std::to_string(options.page_size) + ": " + what;
        if (!said.insert(line).second) continue;
        const bool slow = dtype == DType::BF16 && what.find("prompts: generic") != std::string::npos;
        log_line(slow ? LogLevel::Warning : LogLevel::Info, "attention, %s%s", line.c_str(),
                 slow ? " (head sizes 64 and 128 get the tensor-core kernels)" : "");
    }
}

Engine::~Engine() {
    if (device_) {
        cudaSetDevice(device_->ordinal());
        cudaStreamSynchronize(device_->stream());
    }
    drop_graphs(false);
    builder_.reset();
    for (TokRead& t : tok_reads_) {
        if (t.host) device_->free_pinned(t.host);
        if (t.done) cudaEventDestroy(t.done);
    }
    cache_.reset();
    model_.reset();
}

std::unique_ptr<Engine> Engine::from_folder(const std::string& folder, const EngineOptions& options, const std::string& model_name) {
    std::unique_ptr<Engine> e(new Engine(config_from_folder(folder, model_name), options));
    e->load_folder(folder);
    return e;
}
std::unique_ptr<Engine> Engine::from_config(std::unique_ptr<ArchConfig> config, const EngineOptions& options, unsigned long long seed) {
    std::unique_ptr<Engine> e(new Engine(std::move(config), options));
    e->load_random(seed);
    return e;
}
void Engine::load_folder(const std::string& folder) {
    device_->make_current();
    load_model_weights(*model_, folder);
    loaded_ = true;
}
void Engine::load_random(unsigned long long seed) {
    device_->make_current();
    init_random_weights(*model_, seed);
    loaded_ = true;
}

long long Engine::tokens_that_fit(double fraction) const {
    const size_t elem = dtype_size(rt_.dtype);
    size_t weights = 0;
    for (auto& d : model_->tensor_decls()) weights += (size_t)d.second.numel() * elem;
    const size_t per_token = SequenceCache::bytes_per_token(model_->cache_requests(), rt_.dtype);
    const size_t free_b = device_->mem_free();
    if (per_token == 0) return options_.page_size;
    const double room = ((double)free_b - (double)weights) * fraction;
    if (room < (double)per_token * options_.page_size) {
        char msg[200];
        snprintf(msg, sizeof msg, "the weights (%.1f GiB) leave no room for a cache on this device (%.1f GiB free)",
                 weights / 1073741824.0, free_b / 1073741824.0);
        throw EngineError(msg);
    }
    return (long long)(room / (double)per_token);
}

int Engine::new_sequence() {
    device_->make_current();
    return cache_->alloc_slot();
}
void Engine::end_sequence(int slot) {
    device_->make_current();
    cache_->free_slot(slot);
}
long long Engine::sequence_length(int slot) const {
    if (!cache_->slots.is_held(slot)) throw CacheError("slot " + std::to_string(slot) + " is not live");
    return cache_->seq_len[(size_t)slot];
}
Limits Engine::limits() const { return Limits{cache_->num_slots, cache_->num_pages, cache_->page_size, cache_->max_seq_len}; }
int Engine::graphs_captured() const {
    int n = 0;
    for (auto& g : graphs_)
        if (g.second->exec) n++;
    return n;
}

size_t Engine::context_ints(int T, int B, int K) const {
    return StepContextBuilder::ints(T, B, K, cache_->paged.size(), cache_->width);
}

StepContext Engine::make_context(const StepPlan& plan, const std::vector<int>& ids, const std::vector<int>& want_rows, int* into,
                                 std::vector<const int*>* tables_dev) {
    StepContext ctx = builder_->build(*cache_, plan, ids, want_rows, into, tables_dev);
    last_upload_bytes_ = builder_->last_upload_bytes;
    return ctx;
}

LogitsRef Engine::run_forward(const StepContext& ctx, const std::vector<const int*>& tables) {
    Mat logits = model_->forward(ctx, *cache_, tables);
    return LogitsRef{(const float*)logits.p, ctx.K, model_->spec.vocab_size};
}

// ---- the step

LogitsRef Engine::step(const std::vector<StepItem>& items, const int* device_ids) {
    if (!loaded_) throw EngineError("the model has no weights yet");
    if (items.empty()) throw EngineError("a step needs at least one sequence");
    device_->make_current();
    const long long V = vocab_size();
    std::vector<int> ids, want_rows, slots, q_lens;
    int off = 0;
    for (const StepItem& it : items) {
        const int n = (int)it.tokens.size();
        if (n == 0) throw EngineError("slot " + std::to_string(it.slot) + ": a step must bring at least one token");
        for (int tok : it.tokens)
            if (tok < 0 || tok >= V)
                throw EngineError("slot " + std::to_string(it.slot) + ": token id " + std::to_string(tok) + " is outside the vocabulary [0, " +
                                  std::to_string(V) + ")");
        for (int w : it.want) {
            if (w < 0 || w >= n)
                throw EngineError("slot " + std::to_string(it.slot) + ": wanted place " + std::to_string(w) + " is outside its " +
                                  std::to_string(n) + " tokens");
            want_rows.push_back(off + w);
        }
        ids.insert(ids.end(), it.tokens.begin(), it.tokens.end());
        slots.push_back(it.slot);
        q_lens.push_back(n);
        off += n;
    }
    if (device_ids && ids.size() != items.size()) throw EngineError("device_ids needs one int32 id per item and items of one token each");
    if (graph_safe_ < 0) graph_safe_ = model_->graph_safe() ? 1 : 0;
    if (options_.cuda_graphs && items.size() == 1 && ids.size() > 1 && ids.size() <= (size_t)kPromptGraphMaxTokens) {
        if (pad_safe_ < 0) pad_safe_ = model_->pad_safe() ? 1 : 0;
        LogitsRef out;
        if (pad_safe_ && prompt_step_graphed(items[0].slot, ids, want_rows, &out)) return out;
    }
    StepPlan plan = cache_->plan_step(slots, q_lens);
    LogitsRef logits;
    try {
        if (options_.cuda_graphs && ids.size() == items.size() && graph_safe_) {
            logits = decode_step_graphed(plan, ids, want_rows, device_ids);
        } else {
            device_->arena_rewind();
            std::vector<const int*> tables;
            StepContext ctx = make_context(plan, ids, want_rows, nullptr, &tables);
            if (device_ids)
                check_cuda(cudaMemcpyAsync((void*)ctx.ids, device_ids, ids.size() * sizeof(int), cudaMemcpyDeviceToDevice, device_->stream()),
                           "copying the step's token ids");
            logits = run_forward(ctx, tables);
        }
    } catch (...) {
        cache_->abandon_step(plan);     // the pages reserved for the step go back
        throw;
    }
    cache_->commit_step(plan);
    return logits;
}

void Engine::drop_graphs(bool keep_seen) {
    if (device_) cudaStreamSynchronize(device_->stream());
    for (auto it = graphs_.begin(); it != graphs_.end();) {
        GraphEntry& e = *it->second;
        if (!e.exec && keep_seen) {
            ++it;
            continue;
        }
        if (e.exec) cudaGraphExecDestroy(e.exec);
        if (e.graph) cudaGraphDestroy(e.graph);
        if (e.ctx_buf) device_->free_persistent(e.ctx_buf);
        it = graphs_.erase(it);
    }
}

LogitsRef Engine::capture_and_run(const std::string& key, const StepPlan& plan, const std::vector<int>& ids,
                                  const std::vector<int>& want_rows, const int* device_ids) {
    if (graphs_.size() > 64) drop_graphs(true);
    std::unique_ptr<GraphEntry> e(new GraphEntry);
    int T = 0;
    for (int q : plan.q_lens) T += q;
    e->ctx_buf = (int*)device_->alloc_persistent(context_ints(T, (int)plan.slots.size(), (int)want_rows.size()) * sizeof(int),
                                                 "the inputs of a captured step");
    device_->arena_rewind();
    std::vector<const int*> tables;
    StepContext ctx = make_context(plan, ids, want_rows, e->ctx_buf, &tables);
    if (device_ids)
        check_cuda(cudaMemcpyAsync((void*)ctx.ids, device_ids, ids.size() * sizeof(int), cudaMemcpyDeviceToDevice, device_->stream()),
                   "copying the step's token ids");
    device_->synchronize();
    const long long before = ops::launch_count();
    cudaError_t rc = cudaStreamBeginCapture(device_->stream(), cudaStreamCaptureModeRelaxed);
    if (rc != cudaSuccess) {
        device_->free_persistent(e->ctx_buf);
        check_cuda(rc, "cudaStreamBeginCapture");
    }
    try {
        e->out = run_forward(ctx, tables);
    } catch (...) {
        cudaGraph_t broken = nullptr;
        cudaStreamEndCapture(device_->stream(), &broken);
        if (broken) cudaGraphDestroy(broken);
        cudaGetLastError();
        device_->free_persistent(e->ctx_buf);
        throw;
    }
    rc = cudaStreamEndCapture(device_->stream(), &e->graph);
    if (rc == cudaSuccess) rc = cudaGraphInstantiate(&e->exec, e->graph, 0);
    if (rc != cudaSuccess) {
        if (e->graph) cudaGraphDestroy(e->graph);
        device_->free_persistent(e->ctx_buf);
        cudaGetLastError();
        check_cuda(rc, "capturing a step in a CUDA graph");
    }
    e->launches = ops::launch_count() - before;
    check_cuda(cudaGraphLaunch(e->exec, device_->stream()), "cudaGraphLaunch");
    LogitsRef out = e->out;
    graphs_[key] = std::move(e);
    return out;
}

LogitsRef Engine::replay(GraphEntry& e, const StepPlan& plan, const std::vector<int>& ids, const std::vector<int>& want_rows,
                         const int* device_ids) {
    std::vector<const int*> tables;
    StepContext ctx = make_context(plan, ids, want_rows, e.ctx_buf, &tables);
    if (device_ids)
        check_cuda(cudaMemcpyAsync((void*)ctx.ids, device_ids, ids.size() * sizeof(int), cudaMemcpyDeviceToDevice, device_->stream()),
                   "copying the step's token ids");
    check_cuda(cudaGraphLaunch(e.exec, device_->stream()), "cudaGraphLaunch");
    ops::count_replayed_launches(e.launches);
    return e.out;
}

// A single prompt (or a further piece of one sequence) of up to 1,024 tokens: the host needs longer to
// issue the step's launches than the GPU to run them, so the step is padded to whole buckets of 64
// tokens, with tokens behind the real ones that no real token sees (what they leave in the sequence's
// pages lies behind its length and is overwritten by the tokens that follow), and the launches of a
// bucket are captured in a CUDA graph the second time it is seen.  Only where the padding needs no
// page that the step would not need anyway and stays within the longest sequence; false otherwise (the
// caller then runs the step as it is).  The logits of the real tokens do not depend on the padding
// beyond rounding, and in float32 not at all.
bool Engine::prompt_step_graphed(int slot, const std::vector<int>& ids_in, const std::vector<int>& want_rows, LogitsRef* out) {
    SequenceCache& c = *cache_;
    const int T = (int)ids_in.size();
    const int padded = (int)ceil_div(T, kPromptBucket) * kPromptBucket;
    if (!c.slots.is_held(slot)) return false;
    const long long past = c.seq_len[(size_t)slot];
    if (past + padded > c.max_seq_len) return false;
    for (auto& g : c.paged)
        if (g.ledger->pages_needed(slot, past + padded) != g.ledger->pages_needed(slot, past + T)) return false;
    StepPlan plan = c.plan_step({slot}, {padded});
    std::vector<int> ids = ids_in;
    ids.resize((size_t)padded, 0);
    const std::string key = "p/" + std::to_string(padded) + "/" + std::to_string(want_rows.size());
    try {
        auto it = graphs_.find(key);
        if (it == graphs_.end()) {
            graphs_[key].reset(new GraphEntry);       // seen once
            device_->arena_rewind();
            std::vector<const int*> tables;
            StepContext ctx = make_context(plan, ids, want_rows, nullptr, &tables);
            *out = run_forward(ctx, tables);
        } else if (!it->second->exec) {
            *out = capture_and_run(key, plan, ids, want_rows, nullptr);
        } else {
            *out = replay(*it->second, plan, ids, want_rows, nullptr);
        }
    } catch (...) {
        c.abandon_step(plan);
        throw;
    }
    plan.q_lens = {T};          // the sequence grows by its real tokens only
    c.commit_step(plan);
    return true;
}

// One token per sequence: the launches of such a step are the same every time (all that changes lies
// in device memory), so the step is captured in a CUDA graph the second time a batch size is seen and
// replayed from then on.
LogitsRef Engine::decode_step_graphed(const StepPlan& plan, const std::vector<int>& ids, const std::vector<int>& want_rows,
                                      const int* device_ids) {
    const std::string key = "d/" + std::to_string(ids.size()) + "/" + std::to_string(want_rows.size());
    auto it = graphs_.find(key);
    if (it == graphs_.end()) {
        graphs_[key].reset(new GraphEntry);
        device_->arena_rewind();
        std::vector<const int*> tables;
        StepContext ctx = make_context(plan, ids, want_rows, nullptr, &tables);
        if (device_ids)
            check_cuda(cudaMemcpyAsync((void*)ctx.ids, device_ids, ids.size() * sizeof(int), cudaMemcpyDeviceToDevice, device_->stream()),
                       "copying the step's token ids");
        return run_forward(ctx, tables);
    }
    if (!it->second->exec) return capture_and_run(key, plan, ids, want_rows, device_ids);
    return replay(*it->second, plan, ids, want_rows, device_ids);
}

void Engine::read_logits(const LogitsRef& logits, float* host) {
    if (logits.rows <= 0) return;
    check_cuda(cudaMemcpyAsync(host, logits.p, (size_t)logits.rows * logits.vocab * sizeof(float), cudaMemcpyDeviceToHost, device_->stream()),
               "reading the logits");
    device_->synchronize();
}

int Engine::read_tokens_async(const int* toks, int n) {
    const int ticket = tok_next_;
    tok_next_ = (tok_next_ + 1) % 4;
    TokRead& r = tok_reads_[ticket];
    if (r.cap < n) {
        if (r.host) device_->free_pinned(r.host);
        r.cap = std::max(n, 256);
        r.host = (int*)device_->alloc_pinned((size_t)r.cap * sizeof(int));
    }
    r.n = n;
    check_cuda(cudaMemcpyAsync(r.host, toks, (size_t)n * sizeof(int), cudaMemcpyDeviceToHost, device_->stream()), "reading sampled tokens");
    check_cuda(cudaEventRecord(r.done, device_->stream()), "cudaEventRecord");
    return ticket;
}
std::vector<int> Engine::finish_read(int ticket) {
    TokRead& r = tok_reads_[ticket & 3];
    check_cuda(cudaEventSynchronize(r.done), "waiting for sampled tokens");
    return std::vector<int>(r.host, r.host + r.n);
}

void Engine::warm_up(long long prompt_tokens, const std::vector<int>& batch_sizes) {
    const Limits lim = limits();
    const long long longest = std::min<long long>({prompt_tokens, lim.max_seq_len, (long long)lim.num_pages * lim.page_size});
    for (long long n = ops::kLibraryRowBucket; n <= longest; n += ops::kLibraryRowBucket) {
        bool full = false;
        for (int round = 0; round < (n <= kPromptGraphMaxTokens ? 2 : 1) && !full; round++) {     // the second sight of a bucket captures its graph
            int slot;
            try {
                slot = new_sequence();
            } catch (const CacheError&) {
                full = true;
                break;
            }
            try {
                StepItem it;
                it.slot = slot;
                it.tokens.assign((size_t)n, 0);
                it.want = {(int)n - 1};
                step({it});
            } catch (const CacheError&) {          // live sequences hold the pages: no larger size fits either
                full = true;
            }
            end_sequence(slot);
        }
        if (full) break;
    }
    for (int b : batch_sizes) {
        if (b < 1 || b > lim.max_batch || b > lim.num_pages || cache_->slots.n_free() < b) continue;
        std::vector<int> slots;
        for (int i = 0; i < b; i++) slots.push_back(new_sequence());
        try {
            for (int round = 0; round < 4; round++) {
                std::vector<StepItem> items;
                for (int s : slots) {
                    StepItem it;
                    it.slot = s;
                    it.tokens = {0};
                    it.want = {0};
                    items.push_back(it);
                }
                step(items);
            }
        } catch (const CacheError&) {
        }
        for (int s : slots) end_sequence(s);
    }
    device_->synchronize();
}

void Engine::check_device_errors() {
    auto words = device_->take_error_words();
    if (words.first) {
        const char* what;
        switch (words.first) {
            case 4: what = "a wait inside the tensor-core matrix product (gemm_tc, gemm_tc2) timed out"; break;
            case 5: what = "a wait inside the tensor-core prompt attention (attention_prefill_tc) timed out"; break;
            case 6: what = "a tensor-core kernel found its shared memory misaligned and did not run"; break;
            case 7: what = "a wait inside the decode attention (attention_decode_ring) timed out"; break;
            default: what = nullptr;
        }
        throw EngineError((what ? std::string(what) : "a tensor-core kernel reported error " + std::to_string(words.first)) +
                          ": the step's results are not valid");
    }
    if (words.second) {
        const char* what;
        switch (words.second) {
            case 1: what = "a token id outside the embedding table"; break;
            case 2: what = "a cache write to a page that the sequence does not hold"; break;
            case 3: what = "a position beyond the position table"; break;
            default: what = nullptr;
        }
        throw EngineError("a kernel reported " + (what ? std::string(what) : "error " + std::to_string(words.second)));
    }
}

}  // namespace illm
