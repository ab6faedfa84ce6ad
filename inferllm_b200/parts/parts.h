// Interfaces and registries of the parts that a layer is put together from.
//
// A part is built from a PartSpec (its sizes and constants) and a Runtime (device, compute dtype,
// which kernels run the products); it never learns which model it is in.  It declares the tensors it
// needs under names of its own (tensors()), receives them (load()), and runs on the tokens of one
// step (forward()).  The kinds are looked up by name in the registries below, so a mixer,
// feed-forward, norm, position encoding, block arrangement, embedding or head is added without
// touching this library:
//
//     struct MyMixer : illm::Mixer { ... };
//     illm::register_mixer("my_mixer", [](const PartSpec& s, Runtime* rt) { return std::unique_ptr<Mixer>(new MyMixer(s, rt)); });
//
// (or through the C entry points of binding/c_api.h, which let a part be written in another language).
// The reference has the same seam one level lower: modules take their sizes as constructor arguments
// and own their weights by name (AttentionModule, LlamaFFNModule, src/core/graph.h:84-123,
// src/core/graph.cpp:57-79).
#pragma once
#include <functional>
#include <map>
#include <memory>
#include <string>
#include <vector>

#include "cache/cache.h"
#include "config/config.h"
#include "kernels/ops.h"

namespace illm {

struct PositionTable;

// Where and in which precision a model runs.  `dtype` is the dtype of activations, matrices and
// cache pages: bfloat16 (serving) or float32 (everything in true 32-bit).
struct Runtime {
    Device* dev = nullptr;
    DType dtype = DType::BF16;
    int page_size = 64;
    ops::GemmBackend gemm = ops::GemmBackend::Auto;
    bool is_f32() const { return dtype == DType::F32; }
    // cos/sin tables of rotary encodings, one per distinct (theta, rot_dim, positions) of the model:
    // layers with the same encoding share a table
    std::map<std::string, std::shared_ptr<PositionTable>> position_tables;
};

// A tensor that a part needs.  init: "matrix" -> N(0, 0.02); "norm" -> 1 + N(0, 0.02); "int" -> an
// integer table (kept int32).  Used by the loader to check shapes and by the random-weights writer.
struct TensorDecl {
    std::vector<long long> shape;
    std::string init = "matrix";
    long long numel() const { long long n = 1; for (long long s : shape) n *= s; return n; }
};
using TensorDecls = std::vector<std::pair<std::string, TensorDecl>>;     // in the part's own order

// Persistent device memory owned by a part.
class DeviceBuffer {
public:
    DeviceBuffer() {}
    DeviceBuffer(Device* dev, size_t bytes, const char* what) : dev_(dev), p_(dev->alloc_persistent(bytes, what)), bytes_(bytes) {}
    ~DeviceBuffer() { reset(); }
    DeviceBuffer(DeviceBuffer&& o) noexcept : dev_(o.dev_), p_(o.p_), bytes_(o.bytes_) { o.p_ = nullptr; }
    DeviceBuffer& operator=(DeviceBuffer&& o) noexcept {
        if (this != &o) { reset(); dev_ = o.dev_; p_ = o.p_; bytes_ = o.bytes_; o.p_ = nullptr; }
        return *this;
    }
    void reset() { if (p_ && dev_) dev_->free_persistent(p_); p_ = nullptr; }
    void* get() const { return p_; }
    size_t bytes() const { return bytes_; }
private:
    Device* dev_ = nullptr;
    void* p_ = nullptr;
    size_t bytes_ = 0;
};

// Where a part's tensors come from at load: a weight file or the random generator.  Names are the
// part's own (the model adds the prefix).
class TensorSource {
public:
    virtual ~TensorSource() {}
    // The dtype the tensor is kept in by the storage rule: 16-bit floats -> bfloat16, a tensor stored
    // in 32-bit stays so, integers -> int32; in the float32 mode every float is widened to float32.
    virtual DType kept_dtype(const std::string& name) = 0;
    // Bring the tensor to the device as `want` (float32 or bfloat16 for floats, int32 for integer
    // tables) into dst, whose rows are `dst_row_elems` elements apart (0: contiguous).
    virtual void fetch_into(const std::string& name, void* dst, DType want, long long dst_row_elems = 0) = 0;
    virtual std::vector<long long> shape(const std::string& name) = 0;
};

// A matrix owned by a part: a fresh persistent buffer filled from the source.
struct OwnedMat {
    DeviceBuffer buf;
    Mat m;
};
OwnedMat fetch_owned(Runtime* rt, TensorSource& src, const std::string& name, DType want, const char* what);

class Part {
public:
    Part(PartSpec s, Runtime* runtime) : spec(std::move(s)), rt(runtime) {}
    virtual ~Part() {}
    virtual TensorDecls tensors() const { return {}; }
    // Receive the declared tensors and bring them into the form the kernels want.
    virtual void load(TensorSource&) {}
    PartSpec spec;
    Runtime* rt;      // nullptr: the part only declares its tensors (checking a folder, writing a random one)
};

// The step as the parts see it: the device-side arrays (StepView) and, for parts that need them on
// the host, the step's lengths.  A part that reads the host fields cannot be replayed from a graph
// (see Mixer::graph_safe).
struct StepContext : StepView {
    Device* dev = nullptr;
    Runtime* rt = nullptr;
    std::vector<int> q_lens, host_slots;
    std::vector<long long> past;
};

// What a mixer gets of its cache entry for the step.
struct CacheView {
    enum Kind { None, KV, State } kind = None;
    KVView kv;
    StateView st;
};

// The float32 residual stream [T, H] with at most one addition pending.  A part's output is not added
// at once: the next norm adds it while it reads the row anyway (one kernel for add + norm), which is
// also where the sum is rounded: never, it stays float32.
struct ResidualStream {
    Device* dev = nullptr;
    Mat x;
    bool has_pending = false;
    MatOrPartials pending;
    void add(const MatOrPartials& delta) {
        if (has_pending) flush();
        pending = delta;
        has_pending = true;
    }
    Mat& flush() {
        if (has_pending) {
            ops::residual_add(*dev, x, pending);
            has_pending = false;
        }
        return x;
    }
};

class Norm : public Part {
public:
    using Part::Part;
    // Fold the stream's pending addition in and return the normed rows in the compute dtype; `rows`
    // (int32, device) restricts it to those rows (the stream itself is then left as it is).
    virtual Mat forward(ResidualStream& stream, const int* rows, long long n_rows) = 0;
};

class PositionEncoding : public Part {
public:
    using Part::Part;
    // true: encode_and_store also takes the packed projection as unreduced slices of a split matrix
    // product and adds them up itself.  false (default): it always gets a finished matrix.
    virtual bool takes_partials() const { return false; }
    virtual void prepare() {}     // build device tables; called once after construction on a device
    // true if all this encoding does is the rotate-half rotation of the first rot_dim channels of every
    // Q and K head by angles from a cos/sin table float32 [positions, rot_dim / 2, 2] (rot_dim 0: nothing
    // at all), so that a mixer whose kernel can do that itself may skip encode_and_store.
    virtual bool rotation_table(const float** table, int* rot_dim, long long* n_pos) const { return false; }
    // Encode positions into the Q and K heads of the packed projection and store the new K and V in the
    // cache (if kv.writes).  Returns the matrix that holds the encoded queries in its first
    // heads * head_dim columns: qkv itself (encoded in place) or, for unreduced slices, a new one.
    virtual Mat encode_and_store(const MatOrPartials& qkv, ops::Geometry g, const StepContext& ctx, const KVView& kv) = 0;
};

class Mixer : public Part {
public:
    using Part::Part;
    // true promises that a one-token-per-sequence step launches the same kernels with the same
    // arguments whenever the batch size is the same (everything that varies is read from device
    // memory), so the engine may capture it in a CUDA graph.  A mixer that reads host-side fields of
    // the step context (q_lens, past, ...) says false.
    virtual bool graph_safe() const { return false; }
    // true when tokens appended behind a sequence's real tokens in a step change nothing that is kept
    // (they may leave keys and values behind the sequence's length in its own pages, which the next
    // tokens overwrite) and nothing the real tokens get back, and when a step of many tokens of one
    // sequence launches the same kernels whenever the token count is the same.  The engine then pads
    // single prompts to whole buckets of tokens and replays them from captured graphs.
    virtual bool pad_safe() const { return false; }
    virtual CacheRequest cache_request() const { return CacheRequest(); }
    // h [T, H] in the compute dtype -> [T, H].  `may_defer`: the result may be the unreduced slices of
    // a split matrix product, for a caller that only adds it to the residual stream.
    virtual MatOrPartials forward(const Mat& h, const StepContext& ctx, const CacheView& cache, bool writes, bool may_defer) = 0;
};

class FeedForward : public Part {
public:
    using Part::Part;
    virtual bool graph_safe() const { return true; }
    virtual MatOrPartials forward(const Mat& h, const StepContext& ctx, bool may_defer) = 0;
};

class EmbeddingPart : public Part {
public:
    using Part::Part;
    virtual ResidualStream forward(const StepContext& ctx) = 0;     // ctx.ids -> the float32 stream [T, H]
    virtual const Mat* table() const { return nullptr; }            // what a tied head may use
};

class HeadPart : public Part {
public:
    using Part::Part;
    virtual bool tied() const { return false; }
    virtual void tie(const EmbeddingPart&) {}
    virtual Mat forward(const Mat& y, const StepContext& ctx) = 0;  // normed rows -> float32 logits [rows, vocab]
};

// An arrangement of norms, a mixer and a feed-forward around the residual stream.
class Block {
public:
    virtual ~Block() {}
    Mixer* mixer = nullptr;
    FeedForward* ffn = nullptr;
    std::map<std::string, Norm*> norms;
    virtual void forward(ResidualStream& stream, const StepContext& ctx, const CacheView& cache, bool writes) = 0;
};
struct BlockKind {
    std::vector<std::string> norm_roles;                   // keys of LayerSpec::norms and LayerSpec::names
    std::function<std::unique_ptr<Block>()> make;
};

// ---- registries

template <typename T> using PartFactory = std::function<std::unique_ptr<T>(const PartSpec&, Runtime*)>;
void register_mixer(const std::string& kind, PartFactory<Mixer> f);
void register_feed_forward(const std::string& kind, PartFactory<FeedForward> f);
void register_norm(const std::string& kind, PartFactory<Norm> f);
void register_position(const std::string& kind, PartFactory<PositionEncoding> f);
void register_embedding(const std::string& kind, PartFactory<EmbeddingPart> f);
void register_head(const std::string& kind, PartFactory<HeadPart> f);
void register_block(const std::string& kind, BlockKind k);
void unregister_part(const std::string& family, const std::string& kind);
std::vector<std::string> registered_parts(const std::string& family);

// ConfigError "unknown <family> kind '...'; registered: ..." for a kind that is not there.
std::unique_ptr<Mixer> build_mixer(const PartSpec& s, Runtime* rt);
std::unique_ptr<FeedForward> build_feed_forward(const PartSpec& s, Runtime* rt);
std::unique_ptr<Norm> build_norm(const PartSpec& s, Runtime* rt);
std::unique_ptr<PositionEncoding> build_position(const PartSpec& s, Runtime* rt);
std::unique_ptr<EmbeddingPart> build_embedding(const PartSpec& s, Runtime* rt);
std::unique_ptr<HeadPart> build_head(const PartSpec& s, Runtime* rt);
const BlockKind& lookup_block(const std::string& kind);

// A cos/sin table of a rotate-half encoding on the device: float32 [positions, rot_dim / 2, 2],
// angles p * theta^(-2j / rot_dim) computed in float64 on the host.
struct PositionTable {
    DeviceBuffer buf;
    long long positions = 0;
    int rot_dim = 0;
    const float* data() const { return (const float*)buf.get(); }
};
std::shared_ptr<PositionTable> shared_position_table(Runtime* rt, double theta, int rot_dim, long long positions);

}  // namespace illm
