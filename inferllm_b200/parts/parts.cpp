#include "parts/parts.h"

#include <cmath>

namespace illm {

// ---- registries

namespace {
template <typename T> std::map<std::string, PartFactory<T>>& reg() {
    static std::map<std::string, PartFactory<T>> r;
    return r;
}
std::map<std::string, BlockKind>& block_reg() {
    static std::map<std::string, BlockKind> r;
    return r;
}
void register_builtin_parts();
void ensure_builtin() {
    static bool done = false;
    if (!done) {
        done = true;
        register_builtin_parts();
    }
}
template <typename T> std::unique_ptr<T> build(const char* family, const PartSpec& s, Runtime* rt) {
    ensure_builtin();
    auto it = reg<T>().find(s.kind);
    if (it == reg<T>().end()) {
        std::string known;
        for (auto& k : reg<T>()) known += (known.empty() ? "" : ", ") + k.first;
        throw ConfigError(std::string("unknown ") + family + " kind '" + s.kind + "'; registered: " + known);
    }
    return it->second(s, rt);
}
}  // namespace

void register_mixer(const std::string& kind, PartFactory<Mixer> f) { ensure_builtin(); reg<Mixer>()[kind] = std::move(f); }
void register_feed_forward(const std::string& kind, PartFactory<FeedForward> f) { ensure_builtin(); reg<FeedForward>()[kind] = std::move(f); }
void register_norm(const std::string& kind, PartFactory<Norm> f) { ensure_builtin(); reg<Norm>()[kind] = std::move(f); }
void register_position(const std::string& kind, PartFactory<PositionEncoding> f) { ensure_builtin(); reg<PositionEncoding>()[kind] = std::move(f); }
void register_embedding(const std::string& kind, PartFactory<EmbeddingPart> f) { ensure_builtin(); reg<EmbeddingPart>()[kind] = std::move(f); }
void register_head(const std::string& kind, PartFactory<HeadPart> f) { ensure_builtin(); reg<HeadPart>()[kind] = std::move(f); }
void register_block(const std::string& kind, BlockKind k) { ensure_builtin(); block_reg()[kind] = std::move(k); }

void unregister_part(const std::string& family, const std::string& kind) {
    ensure_builtin();
    if (family == "mixer") reg<Mixer>().erase(kind);
    else if (family == "feed_forward") reg<FeedForward>().erase(kind);
    else if (family == "norm") reg<Norm>().erase(kind);
    else if (family == "position") reg<PositionEncoding>().erase(kind);
    else if (family == "embedding") reg<EmbeddingPart>().erase(kind);
    else if (family == "head") reg<HeadPart>().erase(kind);
    else if (family == "block") block_reg().erase(kind);
    else throw ConfigError("unknown family of parts '" + family + "'");
}
std::vector<std::string> registered_parts(const std::string& family) {
    ensure_builtin();
    std::vector<std::string> out;
    auto names = [&](auto& m) { for (auto& k : m) out.push_back(k.first); };
    if (family == "mixer") names(reg<Mixer>());
    else if (family == "feed_forward") names(reg<FeedForward>());
    else if (family == "norm") names(reg<Norm>());
    else if (family == "position") names(reg<PositionEncoding>());
    else if (family == "embedding") names(reg<EmbeddingPart>());
    else if (family == "head") names(reg<HeadPart>());
    else if (family == "block") names(block_reg());
    else throw ConfigError("unknown family of parts '" + family + "'");
    return out;
}

std::unique_ptr<Mixer> build_mixer(const PartSpec& s, Runtime* rt) { return build<Mixer>("mixer", s, rt); }
std::unique_ptr<FeedForward> build_feed_forward(const PartSpec& s, Runtime* rt) { return build<FeedForward>("feed_forward", s, rt); }
std::unique_ptr<Norm> build_norm(const PartSpec& s, Runtime* rt) { return build<Norm>("norm", s, rt); }
std::unique_ptr<PositionEncoding> build_position(const PartSpec& s, Runtime* rt) { return build<PositionEncoding>("position", s, rt); }
std::unique_ptr<EmbeddingPart> build_embedding(const PartSpec& s, Runtime* rt) { return build<EmbeddingPart>("embedding", s, rt); }
std::unique_ptr<HeadPart> build_head(const PartSpec& s, Runtime* rt) { return build<HeadPart>("head", s, rt); }
const BlockKind& lookup_block(const std::string& kind) {
    ensure_builtin();
    auto it = block_reg().find(kind);
    if (it == block_reg().end()) {
        std::string known;
        for (auto& k : block_reg()) known += (known.empty() ? "" : ", ") + k.first;
        throw ConfigError("unknown block kind '" + kind + "'; registered: " + known);
    }
    return it->second;
}

OwnedMat fetch_owned(Runtime* rt, TensorSource& src, const std::string& name, DType want, const char* what) {
    std::vector<long long> shape = src.shape(name);
    OwnedMat o;
    o.m.rows = shape.size() >= 2 ? shape[0] : 1;
    o.m.cols = shape.empty() ? 1 : shape.back();
    if (shape.size() > 2)
        for (size_t i = 1; i + 1 < shape.size(); i++) o.m.rows *= shape[i];
    o.m.rows_held = o.m.rows;
    o.m.dtype = want;
    o.buf = DeviceBuffer(rt->dev, (size_t)o.m.rows * o.m.cols * dtype_size(want), what);
    o.m.p = o.buf.get();
    src.fetch_into(name, o.m.p, want, 0);
    return o;
}

std::shared_ptr<PositionTable> shared_position_table(Runtime* rt, double theta, int rot_dim, long long positions) {
    char key[96];
    snprintf(key, sizeof key, "%.17g/%d/%lld", theta, rot_dim, positions);
    auto it = rt->position_tables.find(key);
    if (it != rt->position_tables.end()) return it->second;
    const int half = rot_dim / 2;
    std::vector<float> host((size_t)positions * half * 2);
    std::vector<double> inv((size_t)half);
    for (int j = 0; j < half; j++) inv[j] = std::pow(theta, -2.0 * j / rot_dim);
    for (long long p = 0; p < positions; p++)
        for (int j = 0; j < half; j++) {
            const double ang = (double)p * inv[j];
            host[((size_t)p * half + j) * 2] = (float)std::cos(ang);
            host[((size_t)p * half + j) * 2 + 1] = (float)std::sin(ang);
        }
    auto t = std::make_shared<PositionTable>();
    t->positions = positions;
    t->rot_dim = rot_dim;
    t->buf = DeviceBuffer(rt->dev, host.size() * sizeof(float), "a position table");
    check_cuda(cudaMemcpyAsync(t->buf.get(), host.data(), host.size() * sizeof(float), cudaMemcpyHostToDevice, rt->dev->stream()),
               "uploading a position table");
    rt->dev->synchronize();        // `host` goes away
    rt->position_tables[key] = t;
    return t;
}

// ---- the parts of the LLaMA decoder

namespace {

// RMSNorm with a weight, fused with the residual addition that precedes it.  Formula of the reference
// (src/kern/naive/naive.cpp:186-207, weight multiply :138-149): y = x / sqrt(mean(x^2) + eps) * w.  The
// reference fixes eps in code (1e-6 in the layers, src/graph/llama_like.cpp:77-78; 1e-5 in the head,
// src/core/graph.h:160-163); here it is a parameter of the part.
struct RMSNorm : Norm {
    long long size;
    float eps;
    OwnedMat weight;
    RMSNorm(const PartSpec& s, Runtime* rt) : Norm(s, rt), size(s.get_int("size")), eps((float)s.get_double("eps")) {
        if (size <= 0 || !(eps > 0)) throw ConfigError("rmsnorm: size and eps must be positive");
    }
    TensorDecls tensors() const override { return {{"weight", TensorDecl{{size}, "norm"}}}; }
    void load(TensorSource& src) override {
        // a weight stored in 32-bit stays 32-bit; bfloat16 stays bfloat16 (the kernel takes both)
        weight = fetch_owned(rt, src, "weight", src.kept_dtype("weight"), "a norm weight");
    }
    Mat forward(ResidualStream& stream, const int* rows, long long n_rows) override {
        Mat y = ops::add_rmsnorm(*rt->dev, stream.x, stream.has_pending ? &stream.pending : nullptr, weight.m, eps, rt->dtype, rows, n_rows,
                                 rows == nullptr);
        if (rows == nullptr) stream.has_pending = false;
        return y;
    }
};

// "rope_half" is the reference's RotMode::ModelRotHalf (src/kern/naive/naive.cpp:389-414): pair
// (j, j + rot/2) of every Q and K head is rotated by the angle p * theta^(-2j/rot).  The reference
// computes the trigonometry per element (in double on the CPU, with powf/sinf/cosf on the GPU,
// src/kern/gpu/kernel_gpu.cu:343-371); here a table [position, rot/2, (cos, sin)] is computed once in
// float64 and stored in float32, and the rotation is done in float32 inside the kernel that also
// writes K and V into the cache.  theta (fixed to 10000 in the reference) and rot_dim are parameters.
struct RopeHalf : PositionEncoding {
    int head_dim, rot_dim;
    double theta;
    long long max_positions;
    std::shared_ptr<PositionTable> table;
    RopeHalf(const PartSpec& s, Runtime* rt)
            : PositionEncoding(s, rt), head_dim((int)s.get_int("head_dim")), rot_dim((int)s.get_int("rot_dim", s.get_int("head_dim"))),
              theta(s.get_double("theta")), max_positions(s.get_int("max_positions")) {
        if (rot_dim % 2 || rot_dim <= 0 || rot_dim > head_dim)
            throw ConfigError("rope_half: rot_dim " + std::to_string(rot_dim) + " must be even and in (0, head_dim]");
        if (!(theta > 0) || max_positions <= 0) throw ConfigError("rope_half: theta and max_positions must be positive");
    }
    bool takes_partials() const override { return true; }
    void prepare() override { table = shared_position_table(rt, theta, rot_dim, max_positions); }
    bool rotation_table(const float** t, int* rot, long long* n_pos) const override {
        *t = table ? table->data() : nullptr;
        *rot = rot_dim;
        *n_pos = max_positions;
        return true;
    }
    Mat encode_and_store(const MatOrPartials& qkv, ops::Geometry g, const StepContext& ctx, const KVView& kv) override {
        return ops::rope_kv_write(*rt->dev, qkv, table->data(), rot_dim, max_positions, ctx, kv, g);
    }
};

// "none" encodes nothing and only stores K and V.
struct NoPosition : PositionEncoding {
    using PositionEncoding::PositionEncoding;
    bool takes_partials() const override { return true; }
    bool rotation_table(const float** t, int* rot, long long* n_pos) const override {
        *t = nullptr;
        *rot = 0;
        *n_pos = 0;
        return true;
    }
    Mat encode_and_store(const MatOrPartials& qkv, ops::Geometry g, const StepContext& ctx, const KVView& kv) override {
        if (kv.writes) return ops::rope_kv_write(*rt->dev, qkv, nullptr, 0, 0, ctx, kv, g);
        return qkv.is_partials() ? ops::materialize(*rt->dev, qkv.part, rt->dtype) : qkv.m;
    }
};

// Causal self-attention with grouped heads over the paged cache: the mixer of LLaMA.
//
// Order of operations of the reference's LlamaAttention::execute (src/core/op.cpp:348-500): Q, K, V
// projections without bias; position encoding of Q and of the new K rows; K and V go into the cache;
// scores of every query against all cached keys of its sequence, scaled by 1/sqrt(head size) (:488)
// and masked causally; softmax; weighted values; then the output projection (AttentionModule,
// src/core/graph.h:106-111).  The reference has separate [H, H] matrices and one KV head per query
// head (src/core/op.h:327-332); here the three matrices are stacked into one
// [(heads + 2 kv heads) * d, H] at load so that one product feeds the rotation kernel, and the number
// of KV heads, the head size and an optional window are parameters.
struct Attention : Mixer {
    long long hidden;
    int n_heads, n_kv_heads, head_dim, window;
    float scale;
    std::unique_ptr<PositionEncoding> position;
    DeviceBuffer qkv_buf, o_buf;
    Mat w_qkv, w_o;
    Attention(const PartSpec& s, Runtime* rt)
            : Mixer(s, rt), hidden(s.get_int("hidden_size")), n_heads((int)s.get_int("n_heads")), n_kv_heads((int)s.get_int("n_kv_heads")),
              head_dim((int)s.get_int("head_dim")), window((int)s.get_int("window", 0)) {
        if (hidden <= 0 || n_heads <= 0 || n_kv_heads <= 0 || head_dim <= 0 || window < 0)
            throw ConfigError("attention: sizes must be positive");
        if (n_heads % n_kv_heads) throw ConfigError("attention: n_heads must be a multiple of n_kv_heads");
        // the attention kernels read heads 16 bytes at a time: said when the model is built, not at its first step
        if (rt && head_dim % 8)
            throw ConfigError("attention: head size " + std::to_string(head_dim) +
                              " is not supported by the kernels (multiples of 8 up to " + std::to_string(ops::kMaxHeadDimGeneric) + ")");
        if (rt && head_dim > ops::kMaxHeadDimGeneric && !(head_dim == 64 || head_dim == 128))
            throw ConfigError("attention: head size " + std::to_string(head_dim) + " is not supported by the kernels (up to " +
                              std::to_string(ops::kMaxHeadDimGeneric) + ")");
        scale = s.has("scale") ? (float)s.get_double("scale") : (float)(1.0 / std::sqrt((double)head_dim));
        position = build_position(s.get_part("position"), rt);
        if (rt) position->prepare();
    }
    bool graph_safe() const override { return true; }     // a decode step's launches depend only on the batch size
    // Causal attention: tokens behind a sequence's real ones are seen by none of them.  Said only for
    // the plain case: no window, and a position encoding that is nothing but the table rotation (any
    // other runs code of its own, which is not known to launch the same kernels).
    bool pad_safe() const override {
        const float* t;
        int rot;
        long long n;
        return window == 0 && position->rotation_table(&t, &rot, &n);
    }
    TensorDecls tensors() const override {
        const long long q = (long long)n_heads * head_dim, kv = (long long)n_kv_heads * head_dim;
        return {{"q_proj.weight", TensorDecl{{q, hidden}}}, {"k_proj.weight", TensorDecl{{kv, hidden}}},
                {"v_proj.weight", TensorDecl{{kv, hidden}}}, {"o_proj.weight", TensorDecl{{hidden, q}}}};
    }
    void load(TensorSource& src) override {
        const long long q = (long long)n_heads * head_dim, kv = (long long)n_kv_heads * head_dim;
        const size_t es = dtype_size(rt->dtype);
        qkv_buf = DeviceBuffer(rt->dev, (size_t)(q + 2 * kv) * hidden * es, "the packed Q/K/V matrix");
        w_qkv = Mat{qkv_buf.get(), q + 2 * kv, hidden, rt->dtype, q + 2 * kv};
        src.fetch_into("q_proj.weight", w_qkv.p, rt->dtype);
        src.fetch_into("k_proj.weight", (char*)w_qkv.p + (size_t)q * hidden * es, rt->dtype);
        src.fetch_into("v_proj.weight", (char*)w_qkv.p + (size_t)(q + kv) * hidden * es, rt->dtype);
        o_buf = DeviceBuffer(rt->dev, (size_t)hidden * q * es, "the output matrix of an attention layer");
        w_o = Mat{o_buf.get(), hidden, q, rt->dtype, hidden};
        src.fetch_into("o_proj.weight", w_o.p, rt->dtype);
    }
    CacheRequest cache_request() const override { return CacheRequest::paged(n_kv_heads, head_dim, window); }

    MatOrPartials forward(const Mat& h, const StepContext& ctx, const CacheView& cache, bool writes, bool may_defer) override {
        if (cache.kind != CacheView::KV) throw EngineError("attention: the layer's cache entry holds no keys and values");
        Device& dev = *rt->dev;
        KVView kv = cache.kv;
        kv.writes = writes;
        const ops::Geometry g{n_heads, n_kv_heads, head_dim};
        const float* table = nullptr;
        int rot = 0;
        long long n_pos = 0;
        const bool rotation = position->rotation_table(&table, &rot, &n_pos);
        if (ctx.is_decode && rotation && rot % 16 == 0 && ops::attention_decode_ring_supported(h.dtype, n_heads, n_kv_heads, head_dim, kv.page_size)) {
            // one token per sequence: the attention kernel itself adds up the K slices of the projection,
            // rotates Q and the new K row and writes K and V into the cache
            MatOrPartials qkv = ops::linear(dev, rt->gemm, h, w_qkv, rt->dtype, true);
            ops::FusedRope fr{table, rot, n_pos, writes, ctx.err};
            Mat o = ops::attention_decode_ring(dev, qkv, kv, ctx, g, scale, ctx.max_seq_len, 0, &fr);
            return ops::linear(dev, rt->gemm, o, w_o, rt->dtype, may_defer);
        }
        // the packed projection may stay in K slices if the position encoding's kernel adds them up
        MatOrPartials qkv = ops::linear(dev, rt->gemm, h, w_qkv, rt->dtype, position->takes_partials());
        Mat q = position->encode_and_store(qkv, g, ctx, kv);
        Mat o = ops::attention(dev, q, kv, ctx, g, scale);
        return ops::linear(dev, rt->gemm, o, w_o, rt->dtype, may_defer);
    }
};

// Gated feed-forward (SwiGLU): down( act(gate(h)) * up(h) ), no biases.  The reference's
// LlamaFFNModule (src/core/graph.cpp:57-79) runs w3 (up), w1 (gate), Silu, Mul, w2 (down) as five
// operators; silu(x) = x / (1 + exp(-x)) (src/kern/naive/naive.cpp:80-89).  Here gate and up are packed
// into one [2I, H] matrix at load, row 2i the gate row and row 2i + 1 the up row of output i, so that
// one product feeds the activation, and where the package's own kernels run that product the
// activation is their epilogue (ops::linear_gated).
struct GatedMLP : FeedForward {
    long long hidden, inter;
    DeviceBuffer gu_buf, down_buf;
    Mat w_gate_up, w_down;
    GatedMLP(const PartSpec& s, Runtime* rt) : FeedForward(s, rt), hidden(s.get_int("hidden_size")), inter(s.get_int("intermediate_size")) {
        const std::string act = s.get_string("activation", "silu");
        if (act != "silu") throw ConfigError("gated_mlp: activation '" + act + "' is not supported (only 'silu')");
        if (hidden <= 0 || inter <= 0) throw ConfigError("gated_mlp: sizes must be positive");
    }
    TensorDecls tensors() const override {
        return {{"gate_proj.weight", TensorDecl{{inter, hidden}}}, {"up_proj.weight", TensorDecl{{inter, hidden}}},
                {"down_proj.weight", TensorDecl{{hidden, inter}}}};
    }
    void load(TensorSource& src) override {
        const size_t es = dtype_size(rt->dtype);
        gu_buf = DeviceBuffer(rt->dev, (size_t)2 * inter * hidden * es, "the packed gate/up matrix");
        w_gate_up = Mat{gu_buf.get(), 2 * inter, hidden, rt->dtype, 2 * inter};
        src.fetch_into("gate_proj.weight", w_gate_up.p, rt->dtype, 2 * hidden);
        src.fetch_into("up_proj.weight", (char*)w_gate_up.p + (size_t)hidden * es, rt->dtype, 2 * hidden);
        down_buf = DeviceBuffer(rt->dev, (size_t)hidden * inter * es, "the down matrix of a feed-forward layer");
        w_down = Mat{down_buf.get(), hidden, inter, rt->dtype, hidden};
        src.fetch_into("down_proj.weight", w_down.p, rt->dtype);
    }
    MatOrPartials forward(const Mat& h, const StepContext&, bool may_defer) override {
        Device& dev = *rt->dev;
        return ops::linear(dev, rt->gemm, ops::linear_gated(dev, rt->gemm, h, w_gate_up), w_down, rt->dtype, may_defer);
    }
};

// Token embedding: x[t] = W[id[t]] (src/kern/naive/naive.cpp:43-54; EmbdModule, src/core/graph.cpp:143-151),
// written as the float32 residual stream.
struct Embedding : EmbeddingPart {
    long long vocab, hidden;
    OwnedMat weight;
    Embedding(const PartSpec& s, Runtime* rt) : EmbeddingPart(s, rt), vocab(s.get_int("vocab_size")), hidden(s.get_int("hidden_size")) {}
    TensorDecls tensors() const override { return {{"weight", TensorDecl{{vocab, hidden}}}}; }
    void load(TensorSource& src) override { weight = fetch_owned(rt, src, "weight", rt->dtype, "the embedding table"); }
    ResidualStream forward(const StepContext& ctx) override {
        ResidualStream s;
        s.dev = rt->dev;
        s.x = ops::embedding(*rt->dev, ctx.ids, ctx.T, weight.m, ctx.err);
        return s;
    }
    const Mat* table() const override { return &weight.m; }
};

// Output head: logits = y . W_out^T in float32 (src/core/op.cpp:230-247 computes it for the last row
// only and not at all on prefill, src/core/graph.cpp:132-141; here for the rows the caller wants).  A
// tied head uses the embedding table (the reference has no tying).
struct LMHead : HeadPart {
    long long vocab, hidden;
    bool is_tied;
    OwnedMat own;
    Mat weight;
    LMHead(const PartSpec& s, Runtime* rt)
            : HeadPart(s, rt), vocab(s.get_int("vocab_size")), hidden(s.get_int("hidden_size")), is_tied(s.get_bool("tied", false)) {}
    TensorDecls tensors() const override {
        if (is_tied) return {};
        return {{"weight", TensorDecl{{vocab, hidden}}}};
    }
    void load(TensorSource& src) override {
        if (is_tied) return;
        own = fetch_owned(rt, src, "weight", rt->dtype, "the output matrix");
        weight = own.m;
    }
    bool tied() const override { return is_tied; }
    void tie(const EmbeddingPart& e) override {
        if (!e.table()) throw ConfigError("lm_head: tied to an embedding that has no table");
        weight = *e.table();
    }
    Mat forward(const Mat& y, const StepContext&) override { return ops::linear(*rt->dev, rt->gemm, y, weight, DType::F32, false).m; }
};

// "prenorm" is the reference's layer (src/graph/llama_like.cpp:69-105):
//     x = x + mixer(norm1(x));  x = x + ffn(norm2(x))
// with the residual taken from the un-normed stream.
struct PreNormBlock : Block {
    void forward(ResidualStream& stream, const StepContext& ctx, const CacheView& cache, bool writes) override {
        // the outputs only go into the residual stream, so they may stay unreduced: the next norm adds
        // the slices while it reads the row anyway
        Mat h = norms.at("norm1")->forward(stream, nullptr, 0);
        stream.add(mixer->forward(h, ctx, cache, writes, true));
        h = norms.at("norm2")->forward(stream, nullptr, 0);
        stream.add(ffn->forward(h, ctx, true));
    }
};

void register_builtin_parts() {
    reg<Norm>()["rmsnorm"] = [](const PartSpec& s, Runtime* rt) { return std::unique_ptr<Norm>(new RMSNorm(s, rt)); };
    reg<PositionEncoding>()["rope_half"] = [](const PartSpec& s, Runtime* rt) { return std::unique_ptr<PositionEncoding>(new RopeHalf(s, rt)); };
    reg<PositionEncoding>()["none"] = [](const PartSpec& s, Runtime* rt) { return std::unique_ptr<PositionEncoding>(new NoPosition(s, rt)); };
    reg<Mixer>()["attention"] = [](const PartSpec& s, Runtime* rt) { return std::unique_ptr<Mixer>(new Attention(s, rt)); };
    reg<FeedForward>()["gated_mlp"] = [](const PartSpec& s, Runtime* rt) { return std::unique_ptr<FeedForward>(new GatedMLP(s, rt)); };
    reg<EmbeddingPart>()["embedding"] = [](const PartSpec& s, Runtime* rt) { return std::unique_ptr<EmbeddingPart>(new Embedding(s, rt)); };
    reg<HeadPart>()["lm_head"] = [](const PartSpec& s, Runtime* rt) { return std::unique_ptr<HeadPart>(new LMHead(s, rt)); };
    block_reg()["prenorm"] = BlockKind{{"norm1", "norm2"}, [] { return std::unique_ptr<Block>(new PreNormBlock); }};
}

}  // namespace

}  // namespace illm
