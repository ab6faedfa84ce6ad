// Parts written in another language (binding/foreign.h), and a sandbox in which a single part is
// built, loaded and run without a model: a device, a cache for the part's request and step contexts
// made the way the engine makes them.
#include <map>
#include <memory>

#include "binding/common.h"
#include "binding/foreign.h"
#include "engine/step_context.h"
#include "parts/parts.h"

using namespace illm;
using namespace illm::binding;

// ---- foreign parts

namespace {

void fill_step(const StepContext& ctx, illm_step_info* s) {
    s->T = ctx.T;
    s->B = ctx.B;
    s->K = ctx.K;
    s->max_q = ctx.max_q;
    s->is_decode = ctx.is_decode ? 1 : 0;
    s->max_len = ctx.max_len;
    s->max_seq_len = ctx.max_seq_len;
    s->ids = ctx.ids;
    s->token_pos = ctx.token_pos;
    s->token_seq = ctx.token_seq;
    s->want_rows = ctx.want_rows;
    s->slots = ctx.slots;
    s->seq_lens = ctx.seq_lens;
    s->cu_q = ctx.cu_q;
    s->q_lens = ctx.q_lens.data();
    s->host_slots = ctx.host_slots.data();
    s->past = ctx.past.data();
    s->err = ctx.err;
    s->stream = ctx.dev ? ctx.dev->stream() : nullptr;
    s->dtype = ctx.rt ? (int)ctx.rt->dtype : 1;
    s->page_size = ctx.rt ? ctx.rt->page_size : 0;
}
void fill_kv(const KVView& kv, illm_cache_info* c) {
    memset(c, 0, sizeof *c);
    c->kind = 1;
    c->k = kv.k;
    c->v = kv.v;
    c->block_table = kv.block_table;
    c->width = kv.width;
    c->num_pages = kv.num_pages;
    c->page_size = kv.page_size;
    c->window = kv.window;
    c->n_kv_heads = kv.n_kv_heads;
    c->head_dim = kv.head_dim;
    c->dtype = (int)kv.dtype;
    c->writes = kv.writes ? 1 : 0;
}
void fill_cache(const CacheView& v, illm_cache_info* c) {
    memset(c, 0, sizeof *c);
    if (v.kind == CacheView::KV) {
        fill_kv(v.kv, c);
    } else if (v.kind == CacheView::State) {
        c->kind = 2;
        c->state = v.st.state;
        c->slots = v.st.slots;
        c->num_slots = v.st.num_slots;
        c->elements = v.st.elements;
        c->state_dtype = (int)v.st.dtype;
    }
}

// What all foreign parts share: the description, the instance, the tensors the library holds for it.
struct ForeignCore {
    illm_foreign_part t;
    std::string kind;
    Json desc;
    long long instance = 0;
    bool created = false;
    std::vector<DeviceBuffer> tensors;

    ForeignCore(const illm_foreign_part& table, const PartSpec& spec, Runtime* rt) : t(table), kind(spec.kind) {
        const std::string spec_json = spec.to_json().dump();
        desc = parse_json_arg(t.describe(t.user, spec_json.c_str()), "the description of a part");
        if (desc.at("error").is_string()) throw ConfigError(kind + ": " + desc.at("error").as_string());
        if (t.create(t.user, spec_json.c_str(), rt ? (int)rt->dtype : 1, rt ? 1 : 0, &instance))
            throw ConfigError(kind + ": the part could not be created");
        created = true;
    }
    ~ForeignCore() {
        if (created && t.destroy) t.destroy(t.user, instance);
    }
    TensorDecls decls() const {
        TensorDecls out;
        for (const Json& e : desc.at("tensors").items()) {
            TensorDecl d;
            for (const Json& s : e[1].items()) d.shape.push_back(s.as_int());
            d.init = e.size() > 2 && e[2].is_string() ? e[2].as_string() : "matrix";
            out.emplace_back(e[0].as_string(), d);
        }
        return out;
    }
    void load(Runtime* rt, TensorSource& src) {
        for (auto& d : decls()) {
            const DType keep = src.kept_dtype(d.first);
            tensors.emplace_back(rt->dev, (size_t)d.second.numel() * dtype_size(keep), "a tensor of a registered part");
            src.fetch_into(d.first, tensors.back().get(), keep, 0);
            if (t.load(t.user, instance, d.first.c_str(), tensors.back().get(), (int)keep, d.second.shape.data(), (int)d.second.shape.size()))
                throw WeightError(kind + ": the part refused its tensor '" + d.first + "'");
        }
    }
    bool flag(const char* name, bool fallback) const { return desc.at(name).is_bool() ? desc.at(name).as_bool() : fallback; }
};

struct ForeignMixer : Mixer {
    ForeignCore core;
    ForeignMixer(const illm_foreign_part& t, const PartSpec& s, Runtime* rt) : Mixer(s, rt), core(t, s, rt) {}
    TensorDecls tensors() const override { return core.decls(); }
    void load(TensorSource& src) override { core.load(rt, src); }
    bool graph_safe() const override { return core.flag("graph_safe", false); }
    bool pad_safe() const override { return core.flag("pad_safe", false); }
    CacheRequest cache_request() const override { return CacheRequest::from_json(core.desc.at("cache")); }
    MatOrPartials forward(const Mat& h, const StepContext& ctx, const CacheView& cache, bool writes, bool) override {
        if (!core.t.mixer_forward) throw EngineError(core.kind + ": the part has no mixer_forward");
        MatOrPartials out;
        out.m = ops::new_mat(*rt->dev, h.rows, h.cols, h.dtype);
        illm_step_info si;
        illm_cache_info ci;
        fill_step(ctx, &si);
        fill_cache(cache, &ci);
        ci.writes = writes ? 1 : 0;
        if (core.t.mixer_forward(core.t.user, core.instance, &si, &ci, h.p, out.m.p, h.rows, h.cols, writes ? 1 : 0))
            throw EngineError(core.kind + ": the part's forward reported an error");
        return out;
    }
};

struct ForeignFeedForward : FeedForward {
    ForeignCore core;
    ForeignFeedForward(const illm_foreign_part& t, const PartSpec& s, Runtime* rt) : FeedForward(s, rt), core(t, s, rt) {}
    TensorDecls tensors() const override { return core.decls(); }
    void load(TensorSource& src) override { core.load(rt, src); }
    bool graph_safe() const override { return core.flag("graph_safe", false); }
    MatOrPartials forward(const Mat& h, const StepContext& ctx, bool) override {
        if (!core.t.ffn_forward) throw EngineError(core.kind + ": the part has no ffn_forward");
        MatOrPartials out;
        out.m = ops::new_mat(*rt->dev, h.rows, h.cols, h.dtype);
        illm_step_info si;
        fill_step(ctx, &si);
        if (core.t.ffn_forward(core.t.user, core.instance, &si, h.p, out.m.p, h.rows, h.cols))
            throw EngineError(core.kind + ": the part's forward reported an error");
        return out;
    }
};

struct ForeignPosition : PositionEncoding {
    ForeignCore core;
    ForeignPosition(const illm_foreign_part& t, const PartSpec& s, Runtime* rt) : PositionEncoding(s, rt), core(t, s, rt) {}
    TensorDecls tensors() const override { return core.decls(); }
    Mat encode_and_store(const MatOrPartials& qkv, ops::Geometry g, const StepContext& ctx, const KVView& kv) override {
        if (!core.t.encode_and_store) throw EngineError(core.kind + ": the part has no encode_and_store");
        Mat m = qkv.is_partials() ? ops::materialize(*rt->dev, qkv.part, rt->dtype) : qkv.m;
        illm_step_info si;
        illm_cache_info ci;
        fill_step(ctx, &si);
        fill_kv(kv, &ci);
        if (core.t.encode_and_store(core.t.user, core.instance, &si, &ci, m.p, m.rows, m.cols, g.n_heads, g.n_kv_heads, g.head_dim))
            throw EngineError(core.kind + ": the part's encode_and_store reported an error");
        return m;
    }
};

}  // namespace

ILLM_API int illm_register_foreign_part(const char* family, const char* kind, const illm_foreign_part* table) {
    return guard([&] {
        const illm_foreign_part t = *table;
        const std::string fam = family;
        if (fam == "mixer")
            register_mixer(kind, [t](const PartSpec& s, Runtime* rt) { return std::unique_ptr<Mixer>(new ForeignMixer(t, s, rt)); });
        else if (fam == "feed_forward")
            register_feed_forward(kind, [t](const PartSpec& s, Runtime* rt) { return std::unique_ptr<FeedForward>(new ForeignFeedForward(t, s, rt)); });
        else if (fam == "position")
            register_position(kind, [t](const PartSpec& s, Runtime* rt) { return std::unique_ptr<PositionEncoding>(new ForeignPosition(t, s, rt)); });
        else
            throw ConfigError("parts of the family '" + fam + "' cannot be registered through callbacks (mixer, feed_forward, position)");
    });
}
ILLM_API int illm_unregister_part(const char* family, const char* kind) {
    return guard([&] { unregister_part(family, kind); });
}

// ---- the sandbox

namespace {

struct PartHandle {
    std::string family;
    std::unique_ptr<Mixer> mixer;
    std::unique_ptr<FeedForward> ffn;
    std::unique_ptr<Norm> norm;
    std::unique_ptr<PositionEncoding> position;
    std::unique_ptr<EmbeddingPart> embedding;
    std::unique_ptr<HeadPart> head;
    Part* part() {
        if (mixer) return mixer.get();
        if (ffn) return ffn.get();
        if (norm) return norm.get();
        if (position) return position.get();
        if (embedding) return embedding.get();
        return head.get();
    }
};

struct Sandbox {
    std::unique_ptr<Device> dev;
    Runtime rt;
    std::unique_ptr<SequenceCache> cache;
    std::unique_ptr<StepContextBuilder> builder;
    StepContext ctx;
    StepPlan plan;
    std::vector<const int*> tables;
    bool in_step = false;
};

struct BlockHandle {
    std::unique_ptr<Block> block;
};

// Tensors handed over as device pointers.
class MemorySource : public TensorSource {
public:
    MemorySource(Runtime* rt, const Json& tensors, const TensorDecls& decls) : rt_(rt), tensors_(tensors) {
        for (auto& d : decls) inits_[d.first] = d.second.init;
    }
    const Json& rec(const std::string& name) const {
        if (!tensors_.has(name)) throw WeightError("the part needs a tensor '" + name + "' that was not given");
        return tensors_.at(name);
    }
    static DType dt(const Json& r) {
        const std::string s = r.at("dtype").as_string();
        if (s == "float32") return DType::F32;
        if (s == "bfloat16") return DType::BF16;
        if (s == "float16") return DType::F16;
        if (s == "int32") return DType::I32;
        if (s == "int64") return DType::I64;
        throw WeightError("tensors of dtype '" + s + "' cannot be handed to a part");
    }
    DType kept_dtype(const std::string& name) override {
        const DType stored = dt(rec(name));
        const std::string init = inits_.count(name) ? inits_[name] : "matrix";
        if (init == "int" || !dtype_is_float(stored)) return DType::I32;
        if (rt_->is_f32() || stored == DType::F32) return DType::F32;
        return DType::BF16;
    }
    std::vector<long long> shape(const std::string& name) override {
        std::vector<long long> s;
        for (const Json& d : rec(name).at("shape").items()) s.push_back(d.as_int());
        return s;
    }
    void fetch_into(const std::string& name, void* dst, DType want, long long dst_row_elems) override {
        const Json& r = rec(name);
        const DType have = dt(r);
        const void* src = (const void*)(uintptr_t)r.at("ptr").as_int();
        std::vector<long long> sh = shape(name);
        long long cols = sh.empty() ? 1 : sh.back(), rows = 1;
        for (size_t i = 0; i + 1 < sh.size(); i++) rows *= sh[i];
        Device& dev = *rt_->dev;
        const void* conv = src;
        if (have != want) {
            void* tmp = dev.alloc((size_t)rows * cols * dtype_size(want));
            ops::convert(dev, src, have, tmp, want, rows * cols);
            conv = tmp;
        }
        const size_t es = dtype_size(want);
        const size_t pitch = (size_t)(dst_row_elems ? dst_row_elems : cols) * es;
        check_cuda(cudaMemcpy2DAsync(dst, pitch, conv, (size_t)cols * es, (size_t)cols * es, (size_t)rows, cudaMemcpyDeviceToDevice, dev.stream()),
                   "copying a tensor");
    }

private:
    Runtime* rt_;
    Json tensors_;
    std::map<std::string, std::string> inits_;
};

}  // namespace

ILLM_API int illm_sandbox_create(const char* requests_json, const char* dtype, int num_slots, int num_pages, int page_size,
                                 long long max_seq_len, void* stream, void** out) {
    return guard([&] {
        std::unique_ptr<Sandbox> sb(new Sandbox);
        int ordinal = 0;
        check_cuda(cudaGetDevice(&ordinal), "cudaGetDevice");
        sb->dev.reset(new Device(ordinal, (cudaStream_t)stream));
        sb->rt.dev = sb->dev.get();
        const std::string d = dtype ? dtype : "bfloat16";
        if (d != "bfloat16" && d != "float32") throw EngineError("dtype '" + d + "' is not supported (bfloat16 or float32)");
        sb->rt.dtype = d == "float32" ? DType::F32 : DType::BF16;
        sb->rt.page_size = page_size;
        std::map<int, CacheRequest> reqs;
        const Json request_map = parse_json_arg(requests_json, "cache requests");
        for (auto& m : request_map.members()) reqs[atoi(m.first.c_str())] = CacheRequest::from_json(m.second);
        sb->cache.reset(new SequenceCache(reqs, num_slots, num_pages, page_size, max_seq_len, sb->dev.get(), sb->rt.dtype));
        sb->builder.reset(new StepContextBuilder(sb->dev.get(), &sb->rt));
        *out = sb.release();
    });
}
ILLM_API void illm_sandbox_free(void* sb) { delete (Sandbox*)sb; }
ILLM_API void* illm_sandbox_cache(void* sb) { return ((Sandbox*)sb)->cache.get(); }
ILLM_API void* illm_sandbox_device(void* sb) { return ((Sandbox*)sb)->dev.get(); }

ILLM_API int illm_sandbox_build(void* sbp, const char* family, const char* spec_json, void** out) {
    return guard([&] {
        Sandbox* sb = (Sandbox*)sbp;
        const PartSpec spec = PartSpec::from_json(parse_json_arg(spec_json, "part spec"), "part spec");
        std::unique_ptr<PartHandle> h(new PartHandle);
        h->family = family;
        if (h->family == "mixer") h->mixer = build_mixer(spec, &sb->rt);
        else if (h->family == "feed_forward") h->ffn = build_feed_forward(spec, &sb->rt);
        else if (h->family == "norm") h->norm = build_norm(spec, &sb->rt);
        else if (h->family == "position") {
            h->position = build_position(spec, &sb->rt);
            h->position->prepare();
        } else if (h->family == "embedding") h->embedding = build_embedding(spec, &sb->rt);
        else if (h->family == "head") h->head = build_head(spec, &sb->rt);
        else throw ConfigError("unknown family of parts '" + h->family + "'");
        *out = h.release();
    });
}
ILLM_API void illm_part_free(void* p) { delete (PartHandle*)p; }
ILLM_API int illm_part_describe(void* p, char** out) {
    return guard([&] {
        PartHandle* h = (PartHandle*)p;
        Json j = Json::object(), ts = Json::array();
        for (auto& d : h->part()->tensors()) {
            Json e = Json::array(), shape = Json::array();
            for (long long s : d.second.shape) shape.push(s);
            e.push(d.first);
            e.push(shape);
            e.push(d.second.init);
            ts.push(e);
        }
        j.set("tensors", ts);
        if (h->mixer) {
            j.set("cache", h->mixer->cache_request().to_json());
            j.set("graph_safe", h->mixer->graph_safe());
            j.set("pad_safe", h->mixer->pad_safe());
        }
        if (h->position) {
            const float* t = nullptr;
            int rot = 0;
            long long n = 0;
            const bool is_table = h->position->rotation_table(&t, &rot, &n);
            j.set("rotation_table", is_table ? Json((long long)(uintptr_t)t) : Json());
            j.set("rot_dim", rot);
            j.set("positions", n);
            j.set("takes_partials", h->position->takes_partials());
        }
        *out = dup_string(j.dump());
    });
}
// tensors_json: {name: {"ptr": device address, "dtype": "bfloat16", "shape": [...]}}
ILLM_API int illm_sandbox_load(void* sbp, void* p, const char* tensors_json) {
    return guard([&] {
        Sandbox* sb = (Sandbox*)sbp;
        PartHandle* h = (PartHandle*)p;
        sb->dev->arena_rewind();
        MemorySource src(&sb->rt, parse_json_arg(tensors_json, "tensors"), h->part()->tensors());
        h->part()->load(src);
        sb->dev->synchronize();
    });
}
ILLM_API int illm_sandbox_tie(void* head, void* embedding) {
    return guard([&] { ((PartHandle*)head)->head->tie(*((PartHandle*)embedding)->embedding); });
}
// Plans a step for the given slots and lengths and uploads its description; the arena is rewound.
ILLM_API int illm_sandbox_begin_step(void* sbp, const int* slots, const int* q_lens, int n, const int* ids, const int* want, int n_want) {
    return guard([&] {
        Sandbox* sb = (Sandbox*)sbp;
        if (sb->in_step) throw EngineError("the sandbox's last step was neither committed nor abandoned");
        sb->plan = sb->cache->plan_step(std::vector<int>(slots, slots + n), std::vector<int>(q_lens, q_lens + n));
        int T = 0;
        for (int i = 0; i < n; i++) T += q_lens[i];
        std::vector<int> id_list = ids ? std::vector<int>(ids, ids + T) : std::vector<int>((size_t)T, 0);
        sb->dev->arena_rewind();
        sb->ctx = sb->builder->build(*sb->cache, sb->plan, id_list, std::vector<int>(want, want + n_want), nullptr, &sb->tables);
        sb->in_step = true;
    });
}
ILLM_API int illm_sandbox_commit_step(void* sbp) {
    return guard([&] {
        Sandbox* sb = (Sandbox*)sbp;
        if (!sb->in_step) throw EngineError("the sandbox has no step to commit");
        sb->cache->commit_step(sb->plan);
        sb->in_step = false;
    });
}
ILLM_API int illm_sandbox_abandon_step(void* sbp) {
    return guard([&] {
        Sandbox* sb = (Sandbox*)sbp;
        if (sb->in_step) sb->cache->abandon_step(sb->plan);
        sb->in_step = false;
    });
}
ILLM_API int illm_sandbox_step_info(void* sbp, illm_step_info* out) {
    return guard([&] { fill_step(((Sandbox*)sbp)->ctx, out); });
}
static CacheView view_of(Sandbox* sb, int entry, bool writes) {
    CacheView v;
    switch (sb->cache->kind_of(entry)) {
        case SequenceCache::KV:
            v.kind = CacheView::KV;
            v.kv = sb->cache->kv_view(entry, sb->tables[(size_t)sb->cache->group_of(entry)]);
            v.kv.writes = writes;
            break;
        case SequenceCache::State:
            v.kind = CacheView::State;
            v.st = sb->cache->state_view(entry, sb->ctx.slots);
            break;
        default: break;
    }
    return v;
}
ILLM_API int illm_sandbox_cache_info(void* sbp, int entry, int writes, illm_cache_info* out) {
    return guard([&] { fill_cache(view_of((Sandbox*)sbp, entry, writes != 0), out); });
}
static Mat mat_arg(const void* p, long long rows, long long cols, DType dt) {
    Mat m;
    m.p = (void*)p;
    m.rows = m.rows_held = rows;
    m.cols = cols;
    m.dtype = dt;
    return m;
}
// h [T, H] in the sandbox's dtype -> *out [T, *out_cols] in the arena.
ILLM_API int illm_sandbox_mixer_forward(void* sbp, void* p, const void* h, long long T, long long H, int entry, int writes, void** out,
                                        long long* out_cols) {
    return guard([&] {
        Sandbox* sb = (Sandbox*)sbp;
        MatOrPartials r = ((PartHandle*)p)->mixer->forward(mat_arg(h, T, H, sb->rt.dtype), sb->ctx, view_of(sb, entry, writes != 0), writes != 0, false);
        Mat m = r.is_partials() ? ops::materialize(*sb->dev, r.part, sb->rt.dtype) : r.m;
        *out = m.p;
        *out_cols = m.cols;
    });
}
ILLM_API int illm_sandbox_ffn_forward(void* sbp, void* p, const void* h, long long T, long long H, void** out, long long* out_cols) {
    return guard([&] {
        Sandbox* sb = (Sandbox*)sbp;
        StepContext ctx = sb->ctx;
        ctx.dev = sb->dev.get();
        ctx.rt = &sb->rt;
        MatOrPartials r = ((PartHandle*)p)->ffn->forward(mat_arg(h, T, H, sb->rt.dtype), ctx, false);
        Mat m = r.is_partials() ? ops::materialize(*sb->dev, r.part, sb->rt.dtype) : r.m;
        *out = m.p;
        *out_cols = m.cols;
    });
}
ILLM_API int illm_stream_create(void* sbp, void* x, long long T, long long H, void** out) {
    return guard([&] {
        ResidualStream* s = new ResidualStream;
        s->dev = ((Sandbox*)sbp)->dev.get();
        s->x = mat_arg(x, T, H, DType::F32);
        *out = s;
    });
}
ILLM_API void illm_stream_free(void* s) { delete (ResidualStream*)s; }
ILLM_API int illm_stream_add(void* s, const void* delta, int dtype) {
    return guard([&] {
        ResidualStream* rs = (ResidualStream*)s;
        MatOrPartials d;
        d.m = mat_arg(delta, rs->x.rows, rs->x.cols, (DType)dtype);
        rs->add(d);
    });
}
ILLM_API int illm_stream_flush(void* s) {
    return guard([&] { ((ResidualStream*)s)->flush(); });
}
ILLM_API int illm_stream_has_pending(void* s) { return ((ResidualStream*)s)->has_pending ? 1 : 0; }
ILLM_API int illm_sandbox_norm_forward(void* sbp, void* p, void* stream, const int* rows, long long n_rows, void** out) {
    return guard([&] { *out = ((PartHandle*)p)->norm->forward(*(ResidualStream*)stream, rows, n_rows).p; });
}
// norms_json: {"norm1": address of a part handle, ...}
ILLM_API int illm_sandbox_block(void* sbp, const char* kind, void* mixer, void* ffn, const char* norms_json, void** out) {
    return guard([&] {
        const BlockKind& bk = lookup_block(kind);
        std::unique_ptr<BlockHandle> b(new BlockHandle);
        b->block = bk.make();
        b->block->mixer = ((PartHandle*)mixer)->mixer.get();
        b->block->ffn = ((PartHandle*)ffn)->ffn.get();
        const Json norms = parse_json_arg(norms_json, "norms");
        for (const std::string& role : bk.norm_roles) {
            if (!norms.at(role).is_int()) throw ConfigError("the block arrangement '" + std::string(kind) + "' needs a norm for the role '" + role + "'");
            b->block->norms[role] = ((PartHandle*)(uintptr_t)norms.at(role).as_int())->norm.get();
        }
        *out = b.release();
    });
}
ILLM_API void illm_block_free(void* b) { delete (BlockHandle*)b; }
ILLM_API int illm_block_norm_roles(const char* kind, char** out) {
    return guard([&] {
        Json a = Json::array();
        for (auto& r : lookup_block(kind).norm_roles) a.push(r);
        *out = dup_string(a.dump());
    });
}
ILLM_API int illm_sandbox_block_forward(void* sbp, void* block, void* stream, int entry, int writes) {
    return guard([&] {
        Sandbox* sb = (Sandbox*)sbp;
        ((BlockHandle*)block)->block->forward(*(ResidualStream*)stream, sb->ctx, view_of(sb, entry, writes != 0), writes != 0);
    });
}
