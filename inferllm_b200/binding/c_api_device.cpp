// C entry points of the engine, the model API, the sampler, and of what the GPU tests need beside
// them: single kernels through their C++ faces, parts alone in a sandbox, and parts written in
// another language.  Bound by inferllm_b200/binding.py with ctypes.
#include <map>
#include <memory>

#include "binding/common.h"
#include "csrc/kernels.h"
#include "engine/engine.h"
#include "engine/generate.h"
#include "engine/model_api.h"
#include "sampling/sampler.h"
#include "weights/loader.h"

using namespace illm;
using namespace illm::binding;

static std::vector<StepItem> items_from(int n_items, const int* slots, const int* n_tokens, const int* tokens, const int* n_want,
                                        const int* want) {
    std::vector<StepItem> items;
    size_t to = 0, wo = 0;
    for (int i = 0; i < n_items; i++) {
        StepItem it;
        it.slot = slots[i];
        it.tokens.assign(tokens + to, tokens + to + n_tokens[i]);
        it.want.assign(want + wo, want + wo + n_want[i]);
        to += (size_t)n_tokens[i];
        wo += (size_t)n_want[i];
        items.push_back(std::move(it));
    }
    return items;
}

// ---- engine

ILLM_API int illm_engine_create(void* cfg, const char* options_json, void** out) {
    return guard([&] {
        // the engine takes a configuration of its own: a second typed copy of the same keys
        std::unique_ptr<ArchConfig> copy = config_from_json(((ArchConfig*)cfg)->to_json(), ((ArchConfig*)cfg)->architecture());
        *out = new Engine(std::move(copy), EngineOptions::from_json(parse_json_arg(options_json, "engine options")));
    });
}
ILLM_API int illm_engine_from_folder(const char* folder, const char* options_json, const char* model_name, void** out) {
    return guard([&] {
        *out = Engine::from_folder(folder, EngineOptions::from_json(parse_json_arg(options_json, "engine options")), model_name ? model_name : "")
                       .release();
    });
}
ILLM_API void illm_engine_free(void* e) { delete (Engine*)e; }
ILLM_API int illm_engine_load_folder(void* e, const char* folder) {
    return guard([&] { ((Engine*)e)->load_folder(folder); });
}
ILLM_API int illm_engine_load_random(void* e, unsigned long long seed) {
    return guard([&] { ((Engine*)e)->load_random(seed); });
}
ILLM_API int illm_engine_new_sequence(void* e, int* slot) {
    return guard([&] { *slot = ((Engine*)e)->new_sequence(); });
}
ILLM_API int illm_engine_end_sequence(void* e, int slot) {
    return guard([&] { ((Engine*)e)->end_sequence(slot); });
}
ILLM_API int illm_engine_sequence_length(void* e, int slot, long long* n) {
    return guard([&] { *n = ((Engine*)e)->sequence_length(slot); });
}
ILLM_API int illm_engine_limits(void* e, long long out[4]) {
    return guard([&] {
        Limits l = ((Engine*)e)->limits();
        out[0] = l.max_batch;
        out[1] = l.num_pages;
        out[2] = l.page_size;
        out[3] = l.max_seq_len;
    });
}
// A caller's stream as the binding passes it: 0 means none; the legacy default stream is given as
// cudaStreamLegacy (1).
static cudaStream_t caller_stream(void* s) { return (cudaStream_t)s; }

// Runs one step.  The logits [sum of n_want, vocab] are copied to `logits_out` (device, float32) if it
// is not null; *logits_dev gets the engine's own copy (valid until its next step).  `caller`: the
// stream on which the caller made device_ids and will read logits_out (nullptr: none): the engine's
// stream waits for it before the step, and it waits for the engine's stream after the step; the host
// waits for neither.
ILLM_API int illm_engine_step(void* e, int n_items, const int* slots, const int* n_tokens, const int* tokens, const int* n_want,
                              const int* want, const int* device_ids, float* logits_out, const float** logits_dev, void* caller) {
    return guard([&] {
        Engine* eng = (Engine*)e;
        eng->device().make_current();
        // the step itself waits for the caller only if it reads the caller's memory; the copy into the
        // caller's buffer waits in any case (the buffer may still be in use on the caller's stream)
        if (caller && device_ids) eng->device().wait_for(caller_stream(caller));
        LogitsRef lg = eng->step(items_from(n_items, slots, n_tokens, tokens, n_want, want), device_ids);
        if (logits_dev) *logits_dev = lg.p;
        if (caller && !device_ids && logits_out && lg.rows > 0) eng->device().wait_for(caller_stream(caller));
        if (logits_out && lg.rows > 0)
            check_cuda(cudaMemcpyAsync(logits_out, lg.p, (size_t)lg.rows * lg.vocab * sizeof(float), cudaMemcpyDeviceToDevice,
                                       eng->device().stream()),
                       "copying the logits");
        if (caller) eng->device().signal_to(caller_stream(caller));
    });
}
// Orders the engine's stream against a caller's: direction 0: the engine waits for the caller;
// 1: the caller waits for the engine.
ILLM_API int illm_engine_order(void* e, void* caller, int direction) {
    return guard([&] {
        Engine* eng = (Engine*)e;
        eng->device().make_current();
        if (!caller) return;
        if (direction == 0) eng->device().wait_for(caller_stream(caller));
        else eng->device().signal_to(caller_stream(caller));
    });
}
ILLM_API int illm_engine_warm_up(void* e, long long prompt_tokens, const int* batch_sizes, int n) {
    return guard([&] { ((Engine*)e)->warm_up(prompt_tokens, std::vector<int>(batch_sizes, batch_sizes + n)); });
}
ILLM_API int illm_engine_check_device_errors(void* e) {
    return guard([&] { ((Engine*)e)->check_device_errors(); });
}
ILLM_API void* illm_engine_cache(void* e) { return &((Engine*)e)->cache(); }
ILLM_API int illm_engine_info(void* e, char** out) {
    return guard([&] {
        Engine* eng = (Engine*)e;
        Json j = Json::object();
        j.set("vocab_size", eng->vocab_size());
        j.set("graphs_captured", eng->graphs_captured());
        j.set("last_upload_bytes", (long long)eng->last_upload_bytes());
        j.set("dtype", dtype_word(eng->runtime().dtype));
        j.set("device", eng->device().ordinal());
        j.set("n_sms", eng->device().n_sms());
        j.set("gemm", ops::gemm_backend_name(eng->runtime().gemm));
        j.set("arena_bytes", (long long)eng->device().arena_bytes());
        j.set("loaded", eng->loaded());
        j.set("graph_safe", eng->model().graph_safe());
        j.set("pad_safe", eng->model().pad_safe());
        j.set("spec", eng->model().spec.to_json());
        j.set("config", eng->config().to_json());
        j.set("stream", (long long)(uintptr_t)eng->device().stream());
        j.set("tc_error_word", (long long)(uintptr_t)eng->device().tc_error_word());
        j.set("step_error_word", (long long)(uintptr_t)eng->device().step_error_word());
        *out = dup_string(j.dump());
    });
}
ILLM_API int illm_engine_set_gemm(void* e, const char* name) {
    return guard([&] {
        Engine* eng = (Engine*)e;
        const ops::GemmBackend b = ops::gemm_backend_from_name(name);
        if (b != eng->runtime().gemm) {
            eng->runtime().gemm = b;
            eng->forget_graphs();       // which kernels run the products is part of what a graph captured
        }
    });
}
ILLM_API long long illm_launch_count_total() { return ops::launch_count(); }
ILLM_API void illm_set_pdl_enabled(int on) { ops::set_pdl(on != 0); }

// ---- sampler

ILLM_API float illm_uniform_for(long long seed, long long request, long long step) { return uniform_for(seed, request, step); }

static SamplingParams params_from(const Json& j) {
    SamplingParams p;
    if (j.at("temp").is_number()) p.temp = (float)j.at("temp").as_double();
    if (j.at("top_k").is_int()) p.top_k = (int)j.at("top_k").as_int();
    if (j.at("top_p").is_number()) p.top_p = (float)j.at("top_p").as_double();
    if (j.at("repeat_penalty").is_number()) p.repeat_penalty = (float)j.at("repeat_penalty").as_double();
    if (j.at("repeat_last_n").is_int()) p.repeat_last_n = (int)j.at("repeat_last_n").as_int();
    if (j.at("seed").is_int()) p.seed = j.at("seed").as_int();
    return p;
}
ILLM_API int illm_sampling_params_validate(const char* params_json) {
    return guard([&] { params_from(parse_json_arg(params_json, "sampling parameters")).validate(); });
}
ILLM_API int illm_sampler_create(void* engine, const char* params_json, void** out) {
    return guard([&] { *out = new Sampler(&((Engine*)engine)->device(), params_from(parse_json_arg(params_json, "sampling parameters"))); });
}
ILLM_API void illm_sampler_free(void* s) { delete (Sampler*)s; }
// logits: float32 [B, V] on the device; hist_lens == nullptr: no histories.  *tokens: int32 [B] on the
// device, valid for the sampler's next three calls.
ILLM_API int illm_sampler_choose(void* s, const float* logits, int B, long long V, const int* requests, const int* steps,
                                 const int* hist_lens, const int* hist, const int** tokens) {
    return guard([&] {     // (the caller orders the streams with illm_engine_order around this call)
        std::vector<std::vector<int>> hs;
        if (hist_lens) {
            size_t off = 0;
            for (int i = 0; i < B; i++) {
                hs.emplace_back(hist + off, hist + off + hist_lens[i]);
                off += (size_t)hist_lens[i];
            }
        }
        TokensRef t = ((Sampler*)s)->choose(LogitsRef{logits, B, V}, std::vector<int>(requests, requests + B),
                                            std::vector<int>(steps, steps + B), hist_lens ? &hs : nullptr);
        *tokens = t.p;
    });
}

// ---- the model API

ILLM_API int illm_model_create(const char* config_json, const char* model_name, void** out) {
    return guard([&] {
        const Json j = parse_json_arg(config_json, "model configuration");
        ModelConfig c;
        if (j.at("compt_type").is_string()) c.compt_type = j.at("compt_type").as_string();
        if (j.at("device_type").is_string()) c.device_type = j.at("device_type").as_string();
        if (j.at("nr_thread").is_int()) c.nr_thread = (unsigned)j.at("nr_thread").as_int();
        if (j.at("nr_ctx").is_int()) c.nr_ctx = (unsigned)j.at("nr_ctx").as_int();
        if (j.at("device_id").is_int()) c.device_id = (int)j.at("device_id").as_int();
        if (j.at("enable_mmap").is_bool()) c.enable_mmap = j.at("enable_mmap").as_bool();
        if (j.at("max_tokens").is_int()) c.max_tokens = j.at("max_tokens").as_int();
        if (j.at("max_batch").is_int()) c.max_batch = (int)j.at("max_batch").as_int();
        if (j.at("page_size").is_int()) c.page_size = (int)j.at("page_size").as_int();
        if (j.at("cuda_graphs").is_bool()) c.cuda_graphs = j.at("cuda_graphs").as_bool();
        if (j.at("gemm").is_string()) c.gemm = j.at("gemm").as_string();
        if (j.at("poison_freed_pages").is_bool()) c.poison_freed_pages = j.at("poison_freed_pages").as_bool();
        if (j.at("stream").is_int()) c.stream = (void*)(uintptr_t)j.at("stream").as_int();
        *out = new Model(c, model_name ? model_name : "");
    });
}
ILLM_API void illm_model_free(void* m) { delete (Model*)m; }
ILLM_API int illm_model_load(void* m, const char* path) {
    return guard([&] { ((Model*)m)->load(path); });
}
ILLM_API int illm_model_load_random(void* m, void* cfg, unsigned long long seed) {
    return guard([&] {
        ((Model*)m)->load_random(config_from_json(((ArchConfig*)cfg)->to_json(), ((ArchConfig*)cfg)->architecture()), seed);
    });
}
ILLM_API int illm_model_init(void* m, unsigned top_k, float top_p, float temp, float repeat_penalty, int repeat_last_n, long long seed,
                             int end_token) {
    return guard([&] { ((Model*)m)->init(top_k, top_p, temp, repeat_penalty, repeat_last_n, seed, end_token); });
}
ILLM_API int illm_model_engine(void* m, void** engine) {
    return guard([&] { *engine = &((Model*)m)->engine(); });
}
ILLM_API int illm_model_end_tokens(void* m, char** out) {
    return guard([&] {
        Model* mm = (Model*)m;
        Json j = Json::object(), a = Json::array();
        for (int t : mm->end_tokens()) a.push(t);
        j.set("end_tokens", a);
        j.set("end_token", mm->has_end_token() ? Json(mm->end_token()) : Json());
        *out = dup_string(j.dump());
    });
}
ILLM_API int illm_model_get_remain_token(void* m, unsigned* n) {
    return guard([&] { *n = ((Model*)m)->get_remain_token(); });
}
ILLM_API int illm_model_reset_token(void* m) {
    return guard([&] { ((Model*)m)->reset_token(); });
}
ILLM_API int illm_model_prefill(void* m, const int* tokens, int n) {
    return guard([&] { ((Model*)m)->prefill(std::vector<int>(tokens, tokens + n)); });
}
ILLM_API int illm_model_decode(void* m, const int* tokens, int n, int* token) {
    return guard([&] { *token = ((Model*)m)->decode(std::vector<int>(tokens, tokens + n)); });
}
ILLM_API int illm_model_decode_iter(void* m, int* token) {
    return guard([&] { *token = ((Model*)m)->decode_iter(); });
}
ILLM_API int illm_model_decode_summary(void* m, char** out) {
    return guard([&] { *out = dup_string(((Model*)m)->decode_summary()); });
}
ILLM_API int illm_model_warm_up(void* m, long long prompt_tokens, const int* batch_sizes, int n) {
    return guard([&] { ((Model*)m)->warm_up(prompt_tokens, std::vector<int>(batch_sizes, batch_sizes + n)); });
}
typedef void (*illm_token_fn)(void* user, int request, int token);
// stop_ids == nullptr: the default stop set (see Model::generate).
ILLM_API int illm_model_generate(void* m, int n_prompts, const int* prompt_lens, const int* prompts, long long max_new_tokens,
                                 const int* stop_ids, int n_stop, illm_token_fn on_token, void* user, char** result_json) {
    return guard([&] {
        std::vector<std::vector<int>> ps;
        size_t off = 0;
        for (int i = 0; i < n_prompts; i++) {
            ps.emplace_back(prompts + off, prompts + off + prompt_lens[i]);
            off += (size_t)prompt_lens[i];
        }
        std::vector<int> stop;
        if (stop_ids) stop.assign(stop_ids, stop_ids + n_stop);
        TokenCallback cb;
        if (on_token) cb = [&](int r, int t) { on_token(user, r, t); };
        GenerationResult res = ((Model*)m)->generate(ps, max_new_tokens, stop_ids ? &stop : nullptr, cb);
        *result_json = dup_string(res.to_json().dump());
    });
}

// ---- single kernels through their C++ faces (tests and kernel benchmarks)

namespace {
std::map<std::pair<int, uintptr_t>, std::unique_ptr<Device>>& test_devices() {
    static std::map<std::pair<int, uintptr_t>, std::unique_ptr<Device>> d;
    return d;
}
}  // namespace
// A device context for calls outside an engine, on the given stream of the current device.  Results of
// the illm_op_* calls live in its step arena until illm_test_device_rewind.
ILLM_API int illm_test_device(void* stream, void** out) {
    return guard([&] {
        int ordinal = 0;
        check_cuda(cudaGetDevice(&ordinal), "cudaGetDevice");
        auto key = std::make_pair(ordinal, (uintptr_t)stream);
        auto& slot = test_devices()[key];
        if (!slot) slot.reset(new Device(ordinal, (cudaStream_t)stream));
        *out = slot.get();
    });
}
ILLM_API int illm_test_device_rewind(void* dev) {
    return guard([&] { ((Device*)dev)->arena_rewind(); });
}
ILLM_API int illm_test_device_info(void* dev, int* n_sms, int** tc_err, int** step_err) {
    Device* d = (Device*)dev;
    *n_sms = d->n_sms();
    *tc_err = d->tc_error_word();
    *step_err = d->step_error_word();
    return 0;
}
ILLM_API int illm_copy_device(void* dev, void* dst, const void* src, long long bytes) {
    return guard([&] {
        check_cuda(cudaMemcpyAsync(dst, src, (size_t)bytes, cudaMemcpyDeviceToDevice, ((Device*)dev)->stream()), "copying device memory");
    });
}
static Mat mat_of(const void* p, long long rows, long long cols, int dtype) {
    Mat m;
    m.p = (void*)p;
    m.rows = m.rows_held = rows;
    m.cols = cols;
    m.dtype = (DType)dtype;
    return m;
}
// x [M, K] . w [N, K]^T by the engine's choice of kernel for `backend`.  dtype / out_dtype: 0 float32, 1
// bfloat16.  *out: the result [M, N] (arena) unless the product came back as unreduced slices, in which
// case *ws [*splits, M, N] float32 holds them and *out is null.
ILLM_API int illm_op_linear(void* dev, const char* backend, const void* x, long long M, long long K, const void* w, long long N, int dtype,
                            int out_dtype, int defer_reduce, void** out, float** ws, int* splits) {
    return guard([&] {
        MatOrPartials r = ops::linear(*(Device*)dev, ops::gemm_backend_from_name(backend), mat_of(x, M, K, dtype), mat_of(w, N, K, dtype),
                                      (DType)out_dtype, defer_reduce != 0);
        *out = r.is_partials() ? nullptr : r.m.p;
        *ws = r.is_partials() ? r.part.ws : nullptr;
        *splits = r.is_partials() ? r.part.splits : 0;
    });
}
ILLM_API int illm_op_linear_gated(void* dev, const char* backend, const void* x, long long M, long long K, const void* w, long long N,
                                  int dtype, void** out) {
    return guard([&] {
        *out = ops::linear_gated(*(Device*)dev, ops::gemm_backend_from_name(backend), mat_of(x, M, K, dtype), mat_of(w, N, K, dtype)).p;
    });
}
ILLM_API int illm_policy_gemm_tc_splits(long long M, long long N, long long K, int n_sms) { return ops::gemm_tc_splits(M, N, K, n_sms); }
ILLM_API int illm_policy_ring_splits(long long T, int n_kv_heads, long long max_len, int head_dim, int n_sms) {
    return ops::attention_decode_ring_splits(T, n_kv_heads, max_len, head_dim, n_sms);
}
// which: 0 decode_ring, 1 decode (split keys), 2 decode_gqa, 3 prefill (mma.sync), 4 prefill_tc
ILLM_API int illm_policy_attention_supported(int which, int dtype, int nh, int nkv, int d, int page_size) {
    const DType t = (DType)dtype;
    switch (which) {
        case 0: return ops::attention_decode_ring_supported(t, nh, nkv, d, page_size);
        case 1: return ops::attention_decode_supported(t, nh, nkv, d, page_size);
        case 2: return ops::attention_decode_gqa_supported(t, nh, nkv, d);
        case 3: return ops::attention_prefill_supported(t, nh, nkv, d);
        case 4: return ops::attention_prefill_tc_supported(t, nh, nkv, d, page_size);
    }
    return 0;
}
ILLM_API int illm_policy_attention_kernels(int dtype, int nh, int nkv, int d, int page_size, char** out) {
    return guard([&] { *out = dup_string(ops::attention_kernels_for((DType)dtype, nh, nkv, d, page_size)); });
}
