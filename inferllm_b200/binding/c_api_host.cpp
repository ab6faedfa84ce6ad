// C entry points of the parts of the library that need no device: configuration and registry,
// weight files, random model folders, the cache's bookkeeping, the generation loop over stand-ins.
// The Python package binds them with ctypes (inferllm_b200/binding.py); any other language can do the
// same.  The reference exposes a C++ class only (include/model.h).
#include <map>
#include <memory>
#include <mutex>

#include "binding/common.h"
#include "cache/cache.h"
#include "config/config.h"
#include "engine/generate.h"
#include "models/decoder.h"
#include "weights/loader.h"

using namespace illm;
using namespace illm::binding;

namespace illm {
namespace binding {

static thread_local int g_code = 0;
static thread_local std::string g_message;

void set_last_error(int code, const std::string& message) {
    g_code = code;
    g_message = message;
}
char* dup_string(const std::string& s) {
    char* p = (char*)malloc(s.size() + 1);
    memcpy(p, s.c_str(), s.size() + 1);
    return p;
}
Json parse_json_arg(const char* text, const char* what) {
    try {
        return Json::parse(text ? text : "null");
    } catch (const std::runtime_error& e) {
        throw ConfigError(std::string(what) + ": not valid JSON (" + e.what() + ")");
    }
}

}  // namespace binding
}  // namespace illm

ILLM_API const char* illm_last_error(int* code) {
    if (code) *code = g_code;
    return g_message.c_str();
}
ILLM_API void illm_free(void* p) { free(p); }

// ---- configuration and registry

ILLM_API int illm_config_from_json(const char* json, const char* model_name, void** out) {
    return guard([&] { *out = config_from_json(parse_json_arg(json, "config"), model_name ? model_name : "").release(); });
}
ILLM_API int illm_config_from_folder(const char* folder, const char* model_name, void** out) {
    return guard([&] { *out = config_from_folder(folder, model_name ? model_name : "").release(); });
}
ILLM_API void illm_config_free(void* cfg) { delete (ArchConfig*)cfg; }
ILLM_API int illm_config_to_json(void* cfg, char** out) {
    return guard([&] { *out = dup_string(((ArchConfig*)cfg)->to_json().dump()); });
}
ILLM_API int illm_config_architecture(void* cfg, char** out) {
    return guard([&] { *out = dup_string(((ArchConfig*)cfg)->architecture()); });
}
ILLM_API int illm_config_model_spec(void* cfg, char** out) {
    return guard([&] { *out = dup_string(((ArchConfig*)cfg)->model_spec().to_json().dump()); });
}
ILLM_API int illm_model_spec_validate(const char* spec_json) {
    return guard([&] { ModelSpec::from_json(parse_json_arg(spec_json, "model spec")).validate(); });
}
ILLM_API int illm_registered_architectures(char** out) {
    return guard([&] {
        Json a = Json::array();
        for (auto& n : registered_architectures()) a.push(n);
        *out = dup_string(a.dump());
    });
}
ILLM_API int illm_resolve_architecture(const char* name, char** out) {
    return guard([&] { *out = dup_string(resolve_architecture(name)); });
}
ILLM_API int illm_registered_parts(const char* family, char** out) {
    return guard([&] {
        Json a = Json::array();
        for (auto& n : registered_parts(family)) a.push(n);
        *out = dup_string(a.dump());
    });
}

// An architecture written in another language: `describe(user, config_json)` returns a JSON text
// {"config": {... the configuration's own keys ...}, "spec": {... a ModelSpec ...}} that stays valid
// until its next call, or {"error": "..."}.
typedef const char* (*illm_arch_describe_fn)(void* user, const char* config_json);
namespace {
struct ForeignConfig : ArchConfig {
    std::string name;
    Json config, spec;
    std::string architecture() const override { return name; }
    Json to_json() const override { return config; }
    ModelSpec model_spec() const override { return ModelSpec::from_json(spec); }
};
}  // namespace
ILLM_API int illm_register_architecture(const char* name, const char* aliases_json, illm_arch_describe_fn describe, void* user) {
    return guard([&] {
        std::vector<std::string> aliases;
        const Json alias_list = parse_json_arg(aliases_json, "aliases");
        for (const Json& a : alias_list.items()) aliases.push_back(a.as_string());
        const std::string arch = name;
        register_architecture(arch, [arch, describe, user](const Json& d) -> std::unique_ptr<ArchConfig> {
            const char* text = describe(user, d.dump().c_str());
            Json j = parse_json_arg(text, "the description of a registered architecture");
            if (j.at("error").is_string()) throw ConfigError(j.at("error").as_string());
            std::unique_ptr<ForeignConfig> c(new ForeignConfig);
            c->name = arch;
            c->config = j.at("config");
            c->spec = j.at("spec");
            c->model_spec();       // checked here, in words
            return std::unique_ptr<ArchConfig>(c.release());
        }, aliases);
    });
}
ILLM_API int illm_unregister_architecture(const char* name) {
    return guard([&] { unregister_architecture(name); });
}

// ---- weights

ILLM_API int illm_tensor_decls(void* cfg, char** out) {
    return guard([&] {
        DecoderModel model(((ArchConfig*)cfg)->model_spec(), nullptr);
        Json a = Json::array();
        for (auto& d : model.tensor_decls()) {
            Json e = Json::array(), shape = Json::array();
            for (long long s : d.second.shape) shape.push(s);
            e.push(d.first);
            e.push(shape);
            e.push(d.second.init);
            a.push(e);
        }
        *out = dup_string(a.dump());
    });
}
ILLM_API int illm_check_model_folder(void* cfg, const char* folder) {
    return guard([&] {
        DecoderModel model(((ArchConfig*)cfg)->model_spec(), nullptr);
        check_model_folder(model, folder);
    });
}
static DType dtype_arg(const char* name) {
    const std::string s = name ? name : "";
    if (s == "bfloat16" || s == "bf16") return DType::BF16;
    if (s == "float32" || s == "fp32") return DType::F32;
    if (s == "float16" || s == "fp16") return DType::F16;
    if (s == "float64") return DType::F64;
    if (s == "int64") return DType::I64;
    if (s == "int32") return DType::I32;
    if (s == "int16") return DType::I16;
    if (s == "int8") return DType::I8;
    if (s == "uint8") return DType::U8;
    if (s == "bool") return DType::BOOL;
    DType t;
    if (dtype_from_name(s, &t)) return t;
    throw WeightError("unknown dtype '" + s + "'");
}
ILLM_API int illm_write_random_model(void* cfg, const char* folder, unsigned long long seed, const char* dtype) {
    return guard([&] { write_random_model(*(ArchConfig*)cfg, folder, seed, dtype_arg(dtype)); });
}
ILLM_API int illm_storage_dtype(const char* stored, const char* runtime, const char* init, char** out) {
    return guard([&] { *out = dup_string(dtype_word(storage_dtype(dtype_arg(stored), dtype_arg(runtime), init ? init : "matrix"))); });
}
ILLM_API int illm_random_values(unsigned long long seed, const char* name, long long n, const char* init, float* out) {
    return guard([&] {
        for (long long i = 0; i < n; i++) out[i] = random_value(seed, name, i, init ? init : "matrix");
    });
}
// All tensor records of a model folder as JSON {name: {"dtype", "shape", "file", "bytes"}}.
ILLM_API int illm_model_files(const char* folder, char** out) {
    return guard([&] {
        ModelFiles files = open_model_files(folder);
        Json o = Json::object();
        for (auto& r : files.records) {
            Json e = Json::object(), shape = Json::array();
            for (long long s : r.second.shape) shape.push(s);
            e.set("dtype", dtype_name(r.second.dtype));
            e.set("shape", shape);
            e.set("file", r.second.file->path());
            e.set("bytes", (long long)(r.second.end - r.second.begin));
            o.set(r.first, e);
        }
        *out = dup_string(o.dump());
    });
}
ILLM_API int illm_model_files_read(const char* folder, const char* name, void* dst, long long capacity) {
    return guard([&] {
        ModelFiles files = open_model_files(folder);
        auto it = files.records.find(name);
        if (it == files.records.end()) throw WeightError(std::string("no tensor '") + name + "' in " + folder);
        const long long bytes = (long long)(it->second.end - it->second.begin);
        if (bytes > capacity) throw WeightError("the destination is too small for the tensor");
        memcpy(dst, it->second.data(), (size_t)bytes);
    });
}
// tensors_json: [[name, dtype, shape], ...]; data[i]: the bytes of tensor i.
ILLM_API int illm_write_safetensors(const char* path, const char* tensors_json, const void** data, const char* metadata_json) {
    return guard([&] {
        std::vector<TensorToWrite> ts;
        const Json tensor_list = parse_json_arg(tensors_json, "tensors");
        for (const Json& t : tensor_list.items()) {
            TensorToWrite w;
            w.name = t[0].as_string();
            w.dtype = dtype_arg(t[1].as_string().c_str());
            for (const Json& s : t[2].items()) w.shape.push_back(s.as_int());
            ts.push_back(w);
        }
        write_safetensors(path, ts, [&](size_t i, void* dst, size_t bytes) { memcpy(dst, data[i], bytes); },
                          parse_json_arg(metadata_json, "metadata"));
    });
}

// ---- the cache's bookkeeping (host only)

ILLM_API int illm_pool_create(int n, const char* what, void** out) {
    return guard([&] { *out = new IndexPool(n, what ? what : "item"); });
}
ILLM_API void illm_pool_free_handle(void* p) { delete (IndexPool*)p; }
ILLM_API int illm_pool_alloc(void* p, int count, int* out) {
    return guard([&] {
        std::vector<int> got = ((IndexPool*)p)->alloc(count);
        std::copy(got.begin(), got.end(), out);
    });
}
ILLM_API int illm_pool_release(void* p, const int* items, int n) {
    return guard([&] { ((IndexPool*)p)->free(std::vector<int>(items, items + n)); });
}
ILLM_API int illm_pool_check(void* p) {
    return guard([&] { ((IndexPool*)p)->check(); });
}
ILLM_API int illm_pool_stats(void* p, int* n_free, int* n_held) {
    *n_free = ((IndexPool*)p)->n_free();
    *n_held = ((IndexPool*)p)->n_held();
    return 0;
}
ILLM_API int illm_pool_is_held(void* p, int i) { return ((IndexPool*)p)->is_held(i) ? 1 : 0; }

ILLM_API int illm_ledger_create(int num_pages, int page_size, int num_slots, int window, void** out) {
    return guard([&] { *out = new PageLedger(num_pages, page_size, num_slots, window); });
}
ILLM_API void illm_ledger_free_handle(void* p) { delete (PageLedger*)p; }
ILLM_API int illm_ledger_pages_needed(void* p, int slot, long long new_len) { return ((PageLedger*)p)->pages_needed(slot, new_len); }
ILLM_API int illm_ledger_reserve(void* p, int slot, long long new_len) {
    return guard([&] { ((PageLedger*)p)->reserve(slot, new_len); });
}
ILLM_API int illm_ledger_release_outside_window(void* p, int slot, long long seq_len) {
    return guard([&] { ((PageLedger*)p)->release_outside_window(slot, seq_len); });
}
ILLM_API int illm_ledger_release_all(void* p, int slot) {
    return guard([&] { ((PageLedger*)p)->release_all(slot); });
}
ILLM_API int illm_ledger_release_beyond(void* p, int slot, long long seq_len) {
    return guard([&] { ((PageLedger*)p)->release_beyond(slot, seq_len); });
}
ILLM_API int illm_ledger_row(void* p, int slot, int width, int* out) {
    return guard([&] { ((PageLedger*)p)->row(slot, width, out); });
}
ILLM_API int illm_ledger_check(void* p) {
    return guard([&] { ((PageLedger*)p)->check(); });
}
ILLM_API void* illm_ledger_pool(void* p) { return &((PageLedger*)p)->pool; }
// The logical page numbers a slot holds, ascending; returns their count.
ILLM_API int illm_ledger_pages(void* p, int slot, int* logical, int* physical, int capacity) {
    int n = 0;
    for (auto& e : ((PageLedger*)p)->pages[(size_t)slot]) {
        if (n < capacity) {
            logical[n] = e.first;
            physical[n] = e.second;
        }
        n++;
    }
    return n;
}

namespace {
struct CacheHandle {
    std::unique_ptr<SequenceCache> own;
    SequenceCache* cache = nullptr;
    std::map<int, StepPlan> plans;
    int next_plan = 1;
};
}  // namespace

ILLM_API int illm_cache_create(const char* requests_json, int num_slots, int num_pages, int page_size, long long max_seq_len, void** out) {
    return guard([&] {
        std::map<int, CacheRequest> reqs;
        const Json request_map = parse_json_arg(requests_json, "cache requests");
        for (auto& m : request_map.members()) reqs[atoi(m.first.c_str())] = CacheRequest::from_json(m.second);
        std::unique_ptr<CacheHandle> h(new CacheHandle);
        h->own.reset(new SequenceCache(reqs, num_slots, num_pages, page_size, max_seq_len, nullptr, DType::BF16));
        h->cache = h->own.get();
        *out = h.release();
    });
}
// A handle on a cache that somebody else owns (an engine's).
ILLM_API void* illm_cache_wrap(void* sequence_cache) {
    CacheHandle* h = new CacheHandle;
    h->cache = (SequenceCache*)sequence_cache;
    return h;
}
ILLM_API void illm_cache_free_handle(void* h) { delete (CacheHandle*)h; }
ILLM_API int illm_cache_alloc_slot(void* h, int* slot) {
    return guard([&] { *slot = ((CacheHandle*)h)->cache->alloc_slot(); });
}
ILLM_API int illm_cache_free_slot(void* h, int slot) {
    return guard([&] { ((CacheHandle*)h)->cache->free_slot(slot); });
}
ILLM_API int illm_cache_reset(void* h) {
    return guard([&] { ((CacheHandle*)h)->cache->reset(); });
}
ILLM_API int illm_cache_check(void* h) {
    return guard([&] { ((CacheHandle*)h)->cache->check(); });
}
// Plans a step; the page tables go to tables_out (groups x B x width) and the lengths before the step
// to past_out; *plan is a ticket for commit or abandon.
ILLM_API int illm_cache_plan_step(void* hh, const int* slots, const int* q_lens, int n, int* tables_out, long long* past_out, int* plan) {
    return guard([&] {
        CacheHandle* h = (CacheHandle*)hh;
        StepPlan p = h->cache->plan_step(std::vector<int>(slots, slots + n), std::vector<int>(q_lens, q_lens + n));
        size_t off = 0;
        for (auto& t : p.tables) {
            if (tables_out) std::copy(t.begin(), t.end(), tables_out + off);
            off += t.size();
        }
        if (past_out) std::copy(p.past.begin(), p.past.end(), past_out);
        *plan = h->next_plan++;
        h->plans[*plan] = std::move(p);
    });
}
ILLM_API int illm_cache_commit_step(void* hh, int plan) {
    return guard([&] {
        CacheHandle* h = (CacheHandle*)hh;
        auto it = h->plans.find(plan);
        if (it == h->plans.end()) throw CacheError("no such planned step");
        h->cache->commit_step(it->second);
        h->plans.erase(it);
    });
}
ILLM_API int illm_cache_abandon_step(void* hh, int plan) {
    return guard([&] {
        CacheHandle* h = (CacheHandle*)hh;
        auto it = h->plans.find(plan);
        if (it == h->plans.end()) throw CacheError("no such planned step");
        h->cache->abandon_step(it->second);
        h->plans.erase(it);
    });
}
// The cache's state as JSON: sizes, free slots, lengths, and per group its entries, request, free
// pages and the pages of every slot.
ILLM_API int illm_cache_stats(void* hh, char** out) {
    return guard([&] {
        SequenceCache& c = *((CacheHandle*)hh)->cache;
        Json j = Json::object(), lens = Json::array(), paged = Json::array(), states = Json::array();
        j.set("num_slots", c.num_slots);
        j.set("num_pages", c.num_pages);
        j.set("page_size", c.page_size);
        j.set("width", c.width);
        j.set("max_seq_len", c.max_seq_len);
        j.set("slots_free", c.slots.n_free());
        Json held = Json::array();
        for (int s = 0; s < c.num_slots; s++) {
            lens.push(c.seq_len[(size_t)s]);
            if (c.slots.is_held(s)) held.push(s);
        }
        j.set("slots_held", held);
        j.set("seq_len", lens);
        for (auto& g : c.paged) {
            Json o = Json::object(), entries = Json::array(), pages = Json::array();
            for (int e : g.entries) entries.push(e);
            o.set("entries", entries);
            o.set("request", g.request.to_json());
            o.set("pages_free", g.ledger->pool.n_free());
            o.set("pages_held", g.ledger->pool.n_held());
            for (auto& per_slot : g.ledger->pages) {
                Json m = Json::object();
                for (auto& e : per_slot) m.set(std::to_string(e.first), e.second);
                pages.push(m);
            }
            o.set("pages", pages);
            o.set("k", (long long)(uintptr_t)g.k);
            o.set("v", (long long)(uintptr_t)g.v);
            paged.push(o);
        }
        for (auto& g : c.states) {
            Json o = Json::object(), entries = Json::array();
            for (int e : g.entries) entries.push(e);
            o.set("entries", entries);
            o.set("request", g.request.to_json());
            o.set("state", (long long)(uintptr_t)g.state);
            states.push(o);
        }
        j.set("paged", paged);
        j.set("states", states);
        j.set("storage_bytes", (long long)c.storage_bytes());
        *out = dup_string(j.dump());
    });
}

// ---- the generation loop over stand-ins

// The loop's backend and chooser as callbacks, so that its decisions can be tested without a device
// (or driven from another language).  Logits and token lists are opaque 64-bit handles of the callee.
// Callbacks return 0, or non-zero after having recorded their own error (the loop then ends with an
// EngineError and every live slot is given back).
struct illm_loop_callbacks {
    void* user;
    int (*limits)(void* user, long long out[4]);       // max_batch, num_pages, page_size, max_seq_len
    int (*new_sequence)(void* user, int* slot);
    int (*end_sequence)(void* user, int slot);
    int (*step)(void* user, int n_items, const int* slots, const int* n_tokens, const int* tokens, const int* n_want, const int* want,
                long long device_ids, long long* logits);
    int (*choose)(void* user, long long logits, int n, const int* requests, const int* steps, int has_histories, const int* hist_lens,
                  const int* hist, long long* tokens);
    int (*read_async)(void* user, long long tokens, int* ticket);
    int (*finish_read)(void* user, int ticket, int* out, int capacity, int* n);
    int (*select)(void* user, long long tokens, const int* idx, int n, long long* out);
    double (*clock)(void* user);
    void (*on_token)(void* user, int request, int token);
};

namespace {
[[noreturn]] void callback_failed(const char* which) { throw EngineError(std::string("the ") + which + " callback reported an error"); }

struct CallbackBackend : GenBackend, Chooser {
    illm_loop_callbacks cb;
    Limits limits() override {
        long long v[4];
        if (cb.limits(cb.user, v)) callback_failed("limits");
        return Limits{(int)v[0], (int)v[1], (int)v[2], v[3]};
    }
    int new_sequence() override {
        int s = -1;
        if (cb.new_sequence(cb.user, &s)) callback_failed("new_sequence");
        return s;
    }
    void end_sequence(int slot) override {
        if (cb.end_sequence(cb.user, slot)) callback_failed("end_sequence");
    }
    LogitsRef step(const std::vector<StepItem>& items, const TokensRef* ids) override {
        std::vector<int> slots, nt, toks, nw, want;
        for (auto& it : items) {
            slots.push_back(it.slot);
            nt.push_back((int)it.tokens.size());
            toks.insert(toks.end(), it.tokens.begin(), it.tokens.end());
            nw.push_back((int)it.want.size());
            want.insert(want.end(), it.want.begin(), it.want.end());
        }
        long long h = 0;
        if (cb.step(cb.user, (int)items.size(), slots.data(), nt.data(), toks.data(), nw.data(), want.data(),
                    ids ? (long long)(intptr_t)ids->p : -1, &h))
            callback_failed("step");
        return LogitsRef{(const float*)(intptr_t)h, (long long)want.size(), 0};
    }
    TokensRef choose(const LogitsRef& logits, const std::vector<int>& requests, const std::vector<int>& steps,
                     const std::vector<std::vector<int>>* histories) override {
        std::vector<int> lens, flat;
        if (histories)
            for (auto& h : *histories) {
                lens.push_back((int)h.size());
                flat.insert(flat.end(), h.begin(), h.end());
            }
        long long t = 0;
        if (cb.choose(cb.user, (long long)(intptr_t)logits.p, (int)requests.size(), requests.data(), steps.data(), histories ? 1 : 0,
                      lens.data(), flat.data(), &t))
            callback_failed("choose");
        return TokensRef{(const int*)(intptr_t)t, (int)requests.size()};
    }
    int read_tokens_async(const TokensRef& t) override {
        int ticket = 0;
        if (cb.read_async(cb.user, (long long)(intptr_t)t.p, &ticket)) callback_failed("read_async");
        return ticket;
    }
    std::vector<int> finish_read(int ticket) override {
        std::vector<int> out(65536);
        int n = 0;
        if (cb.finish_read(cb.user, ticket, out.data(), (int)out.size(), &n)) callback_failed("finish_read");
        out.resize((size_t)n);
        return out;
    }
    TokensRef select(const TokensRef& toks, const std::vector<int>& idx) override {
        long long h = 0;
        if (cb.select(cb.user, (long long)(intptr_t)toks.p, idx.data(), (int)idx.size(), &h)) callback_failed("select");
        return TokensRef{(const int*)(intptr_t)h, (int)idx.size()};
    }
};
}  // namespace

ILLM_API int illm_generate_with_callbacks(const illm_loop_callbacks* cb, int n_prompts, const int* prompt_lens, const int* prompts,
                                          long long max_new_tokens, const int* stop_ids, int n_stop, char** result_json) {
    return guard([&] {
        CallbackBackend b;
        b.cb = *cb;
        std::vector<std::vector<int>> ps;
        size_t off = 0;
        for (int i = 0; i < n_prompts; i++) {
            ps.emplace_back(prompts + off, prompts + off + prompt_lens[i]);
            off += (size_t)prompt_lens[i];
        }
        TokenCallback on_token;
        if (cb->on_token) on_token = [&](int r, int t) { cb->on_token(cb->user, r, t); };
        std::function<double()> clock;
        if (cb->clock) clock = [&] { return cb->clock(cb->user); };
        GenerationResult res = generate(b, ps, b, max_new_tokens, std::vector<int>(stop_ids, stop_ids + n_stop), on_token, clock);
        *result_json = dup_string(res.to_json().dump());
    });
}
ILLM_API int illm_plan_batches(const int* prompt_lens, int n, long long max_new_tokens, int max_batch, int num_pages, int page_size,
                               long long max_seq_len, char** out) {
    return guard([&] {
        Json a = Json::array();
        for (auto& b : plan_batches(std::vector<int>(prompt_lens, prompt_lens + n), max_new_tokens,
                                    Limits{max_batch, num_pages, page_size, max_seq_len})) {
            Json e = Json::array();
            for (int r : b) e.push(r);
            a.push(e);
        }
        *out = dup_string(a.dump());
    });
}
