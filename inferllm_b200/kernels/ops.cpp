#include "kernels/ops.h"

#include <algorithm>
#include <cmath>

#include "csrc/kernels.h"

namespace illm {
namespace ops {

static long long g_replayed = 0;
long long launch_count() { return illm_launch_count() + g_replayed; }
void count_replayed_launches(long long n) { g_replayed += n; }
void set_pdl(bool on) { illm_set_pdl(on ? 1 : 0); }

GemmBackend gemm_backend_from_name(const std::string& name) {
    if (name == "auto") return GemmBackend::Auto;
    if (name == "tc") return GemmBackend::TC;
    if (name == "library") return GemmBackend::Library;
    throw EngineError("gemm backend must be 'tc', 'library' or 'auto', found '" + name + "'");
}
const char* gemm_backend_name(GemmBackend b) { return b == GemmBackend::Auto ? "auto" : b == GemmBackend::TC ? "tc" : "library"; }

static int code_of(DType t, const char* what) {
    if (t == DType::F32) return 0;
    if (t == DType::BF16) return 1;
    throw KernelError(std::string(what) + ": unsupported dtype " + dtype_word(t) + ": the kernels take float32 and bfloat16");
}
static long long ceil_div(long long a, long long b) { return (a + b - 1) / b; }
static void need(const Mat& m, const char* name, bool want_dtype = false, DType dtype = DType::BF16) {
    if (m.p == nullptr && m.rows * m.cols > 0) throw KernelError(std::string(name) + " has no storage");
    if (want_dtype && m.dtype != dtype)
        throw KernelError(std::string(name) + " must be " + dtype_word(dtype) + ", found " + dtype_word(m.dtype));
    // rows of a multiple of 16 bytes are read 16 bytes at a time
    if (((uintptr_t)m.p & 15) && (m.cols * (long long)dtype_size(m.dtype)) % 16 == 0 && m.rows * m.cols > 0)
        throw KernelError(std::string(name) + " must start on a 16-byte boundary");
}
static void* row_ptr(const Mat& m, long long row) { return (char*)m.p + (size_t)row * m.cols * dtype_size(m.dtype); }

Mat new_mat(Device& dev, long long rows, long long cols, DType dtype) {
    Mat m;
    m.rows = rows;
    m.cols = cols;
    m.dtype = dtype;
    m.rows_held = rows;
    if (dtype == DType::BF16 && rows > kLibraryRowBucket && rows % kLibraryRowBucket)
        m.rows_held = ceil_div(rows, kLibraryRowBucket) * kLibraryRowBucket;
    m.p = dev.alloc((size_t)m.rows_held * cols * dtype_size(dtype));
    return m;
}
static Mat new_mat_exact(Device& dev, long long rows, long long cols, DType dtype) {
    Mat m;
    m.rows = m.rows_held = rows;
    m.cols = cols;
    m.dtype = dtype;
    m.p = dev.alloc((size_t)rows * cols * dtype_size(dtype));
    return m;
}

// ---- policies

int gemm_tc_splits(long long M, long long N, long long K, int n_sms) {
    if (M > 64) return 1;
    const long long tiles = ceil_div(N, 128), k_iters = ceil_div(K, 64);
    long long splits = std::max<long long>(1, std::min<long long>({2LL * n_sms / tiles, k_iters / 8, 8}));   // (more than 8 slices cost their readers more than they win)
    const long long per = ceil_div(k_iters, splits);
    return (int)ceil_div(k_iters, per);          // every slice owns at least one 64-wide piece of K
}

int attention_decode_ring_splits(long long T, int n_kv_heads, long long max_len, int head_dim, int n_sms, double stream_bytes_per_us) {
    const long long pairs = std::max<long long>(1, T * n_kv_heads), tiles = std::max<long long>(1, ceil_div(max_len, 64));
    const long long slots = 2LL * n_sms;
    const double stream_us = (double)pairs * (double)max_len * head_dim * 4 / stream_bytes_per_us;
    int best = 1;
    double best_us = INFINITY;
    for (long long n = 1; n <= std::min<long long>(tiles, kRingDecodeMaxSplits); n++) {
        const long long blocks = pairs * n;
        const double waves = (double)blocks / slots;
        double stretch;
        if (blocks <= slots) {
            stretch = 1.0 / std::min(1.0, blocks / 160.0);
        } else {
            const long long full = blocks / slots, rest = blocks % slots;
            stretch = (full + (rest ? std::max((double)rest / slots, 0.43) : 0.0)) / waves;
        }
        const double us = stream_us * stretch + (n > 1 ? 2.5 + 0.7 * n : 0.0) + 1.0 * ceil_div(blocks, slots);
        if (us < best_us - 1e-9) {
            best = (int)n;
            best_us = us;
        }
    }
    return best;
}

bool attention_decode_ring_supported(DType dtype, int nh, int nkv, int d, int page_size) {
    return dtype == DType::BF16 && (d == 64 || d == 128) && nkv > 0 && nh % nkv == 0 && nh / nkv <= 16 && page_size % 64 == 0;
}
bool attention_decode_supported(DType dtype, int nh, int nkv, int d, int page_size) {
    return dtype == DType::BF16 && nkv > 0 && nh % nkv == 0 && illm_attention_decode_supported(d, nh / nkv, page_size) != 0;
}
bool attention_decode_gqa_supported(DType dtype, int nh, int nkv, int d) {
    return dtype == DType::BF16 && (d == 64 || d == 128) && nkv > 0 && nh % nkv == 0 && nh / nkv >= 2 && nh / nkv <= 16;
}
bool attention_prefill_supported(DType dtype, int nh, int nkv, int d) {
    return dtype == DType::BF16 && (d == 64 || d == 128) && nkv > 0 && nh % nkv == 0;
}
bool attention_prefill_tc_supported(DType dtype, int nh, int nkv, int d, int page_size) {
    return dtype == DType::BF16 && (d == 64 || d == 128) && nkv > 0 && nh % nkv == 0 && page_size % 64 == 0;
}
std::string attention_kernels_for(DType dtype, int nh, int nkv, int d, int page_size) {
    const int group = nkv ? nh / nkv : 0;
    std::string prompt = attention_prefill_tc_supported(dtype, nh, nkv, d, page_size) ? "prefill_tc (tcgen05)"
                         : attention_prefill_supported(dtype, nh, nkv, d)             ? "prefill (mma.sync)"
                                                                                      : "generic (float32 SIMT, O(T^2) global reads)";
    std::string decode;
    if (attention_decode_ring_supported(dtype, nh, nkv, d, page_size)) decode = "decode_ring (TMA ring)";
    else if ((group >= kGqaDecodeMinGroup || !attention_decode_supported(dtype, nh, nkv, d, page_size)) &&
             attention_decode_gqa_supported(dtype, nh, nkv, d)) decode = "decode_gqa (mma.sync)";
    else if (attention_decode_supported(dtype, nh, nkv, d, page_size)) decode = "decode (split keys)";
    else decode = "generic (float32 SIMT)";
    return "prompts: " + prompt + "; single tokens: " + decode;
}

// ---- element-wise kernels

Mat embedding(Device& dev, const int* ids, long long T, const Mat& table, int* err) {
    need(table, "table");
    Mat out = new_mat_exact(dev, T, table.cols, DType::F32);
    check_kernel(illm_embedding(ids, table.p, code_of(table.dtype, "embedding"), (float*)out.p, (int)T, (int)table.cols, (int)table.rows,
                                err, dev.stream()),
                 "embedding");
    return out;
}

Mat materialize(Device& dev, const Partials& p, DType dtype) {
    Mat out = new_mat_exact(dev, p.rows, p.cols, dtype);
    check_kernel(illm_splitk_reduce(p.ws, out.p, code_of(dtype, "splitk_reduce"), p.rows * p.cols, p.splits, dev.stream()), "splitk_reduce");
    return out;
}

Mat add_rmsnorm(Device& dev, const Mat& resid, const MatOrPartials* delta, const Mat& weight, float eps, DType out_dtype,
                const int* rows, long long n_rows, bool write_resid) {
    need(resid, "resid", true, DType::F32);
    const long long H = resid.cols;
    if (H > kMaxNormWidth)
        throw KernelError("rmsnorm: width " + std::to_string(H) + " exceeds the " + std::to_string(kMaxNormWidth) +
                          " that one block's shared memory holds");
    const Partials* partials = nullptr;
    Mat d;
    bool has_delta = false;
    if (delta && delta->is_partials()) {
        if (out_dtype == DType::BF16 && H % 8 == 0 && H <= 16384 && delta->part.rows == resid.rows && delta->part.cols == resid.cols) {
            partials = &delta->part;
        } else {
            d = materialize(dev, delta->part, out_dtype);
            has_delta = true;
        }
    } else if (delta) {
        d = delta->m;
        has_delta = true;
    }
    if (has_delta) {
        need(d, "delta", true, out_dtype);
        if (d.rows != resid.rows || d.cols != resid.cols)
            throw KernelError("delta [" + std::to_string(d.rows) + ", " + std::to_string(d.cols) + "] does not match resid [" +
                              std::to_string(resid.rows) + ", " + std::to_string(resid.cols) + "]");
    }
    need(weight, "norm weight");
    if (weight.rows * weight.cols != H)
        throw KernelError("norm weight has " + std::to_string(weight.rows * weight.cols) + " elements, the rows have " + std::to_string(H));
    const long long n = rows ? n_rows : resid.rows;
    Mat y = new_mat(dev, n, H, out_dtype);
    if (partials)
        check_kernel(illm_add_rmsnorm_partials((float*)resid.p, partials->ws, partials->splits, partials->rows * partials->cols, weight.p,
                                               code_of(weight.dtype, "rmsnorm"), y.p, code_of(out_dtype, "rmsnorm"), rows, (int)n, (int)H, eps,
                                               write_resid ? 1 : 0, dev.stream()),
                     "add_rmsnorm_partials");
    else
        check_kernel(illm_add_rmsnorm((float*)resid.p, has_delta ? d.p : nullptr, weight.p, code_of(weight.dtype, "rmsnorm"), y.p,
                                      code_of(out_dtype, "rmsnorm"), rows, (int)n, (int)H, eps, write_resid ? 1 : 0, dev.stream()),
                     "add_rmsnorm");
    return y;
}

void residual_add(Device& dev, const Mat& resid, const MatOrPartials& delta) {
    Mat d = delta.is_partials() ? materialize(dev, delta.part, DType::BF16) : delta.m;
    need(resid, "resid", true, DType::F32);
    need(d, "delta");
    if (d.rows != resid.rows || d.cols != resid.cols) throw KernelError("residual_add: shapes differ");
    check_kernel(illm_residual_add((float*)resid.p, d.p, code_of(d.dtype, "residual_add"), resid.rows * resid.cols, dev.stream()),
                 "residual_add");
}

Mat swiglu(Device& dev, const MatOrPartials& gu_in) {
    Mat gu;
    if (gu_in.is_partials()) {
        const Partials& p = gu_in.part;
        if (p.cols % 16 == 0) {
            Mat out = new_mat(dev, p.rows, p.cols / 2, DType::BF16);
            check_kernel(illm_swiglu_partials(p.ws, p.splits, p.rows * p.cols, out.p, (int)p.rows, (int)(p.cols / 2), dev.stream()),
                         "swiglu_partials");
            return out;
        }
        gu = materialize(dev, p, DType::BF16);
    } else {
        gu = gu_in.m;
    }
    need(gu, "gu");
    if (gu.cols % 2) throw KernelError("swiglu: the packed projection must have an even number of columns");
    Mat out = new_mat(dev, gu.rows, gu.cols / 2, gu.dtype);
    check_kernel(illm_swiglu(gu.p, out.p, code_of(gu.dtype, "swiglu"), (int)gu.rows, (int)(gu.cols / 2), dev.stream()), "swiglu");
    return out;
}

// ---- matrix products

Mat gemm_f32(Device& dev, const Mat& x, const Mat& w) {
    need(x, "x", true, DType::F32);
    need(w, "w", true, DType::F32);
    const long long M = x.rows, K = x.cols, N = w.rows;
    if (w.cols != K)
        throw KernelError("gemm: x is [" + std::to_string(M) + ", " + std::to_string(K) + "] but w is [" + std::to_string(w.rows) + ", " +
                          std::to_string(w.cols) + "]");
    Mat out = new_mat_exact(dev, M, N, DType::F32);
    for (long long m0 = 0; m0 < M; m0 += 65535LL * 64) {
        const long long m1 = std::min(M, m0 + 65535LL * 64);
        check_kernel(illm_gemm_f32_nt((const float*)row_ptr(x, m0), (const float*)w.p, (float*)row_ptr(out, m0), (int)(m1 - m0), (int)N, (int)K,
                                      (int)K, (int)K, (int)N, dev.tc_error_word(), dev.stream()),
                     "gemm_f32");
    }
    return out;
}

static void check_product(const Mat& x, const Mat& w, const char* what, bool gated = false) {
    need(x, "x", true, DType::BF16);
    need(w, "w", true, DType::BF16);
    if (w.cols != x.cols)
        throw KernelError("gemm: x is [" + std::to_string(x.rows) + ", " + std::to_string(x.cols) + "] but w is [" + std::to_string(w.rows) +
                          ", " + std::to_string(w.cols) + "]");
    if (x.cols % 8 || ((uintptr_t)x.p & 15) || ((uintptr_t)w.p & 15) || (gated && w.rows % 2))
        throw KernelError(std::string(what) + ": K = " + std::to_string(x.cols) +
                          " must be a multiple of 8, the operands 16-byte aligned and a gated weight an even number of rows");
}

MatOrPartials gemm_bf16_tc(Device& dev, const Mat& x, const Mat& w, DType out_dtype, int splits, bool defer_reduce) {
    check_product(x, w, "gemm_bf16_tc");
    const long long M = x.rows, K = x.cols, N = w.rows;
    MatOrPartials r;
    r.m = new_mat_exact(dev, M, N, out_dtype);
    if (splits <= 0) {
        splits = gemm_tc_splits(M, N, K, dev.n_sms());
    } else {
        const long long k_iters = ceil_div(K, 64);
        long long s = std::max<long long>(1, std::min<long long>(splits, k_iters));
        splits = (int)ceil_div(k_iters, ceil_div(k_iters, s));
    }
    if (M > 64) splits = 1;
    float* ws = splits > 1 ? dev.alloc_n<float>((size_t)splits * M * N) : nullptr;
    const bool defer = defer_reduce && splits > 1;
    check_kernel(illm_gemm_bf16_tc(x.p, w.p, r.m.p, code_of(out_dtype, "gemm_bf16_tc"), (int)M, (int)N, (int)K, ws, splits, dev.tc_error_word(),
                                   dev.stream(), defer ? 1 : 0),
                 "gemm_bf16_tc");
    if (defer) {
        r.part.ws = ws;
        r.part.splits = splits;
        r.part.rows = M;
        r.part.cols = N;
    }
    return r;
}

Mat gemm_bf16_tc2(Device& dev, const Mat& x, const Mat& w, DType out_dtype, bool gated) {
    check_product(x, w, "gemm_bf16_tc2", gated);
    const long long M = x.rows, K = x.cols, N = w.rows;
    Mat out = new_mat(dev, M, gated ? N / 2 : N, out_dtype);
    check_kernel(illm_gemm_bf16_tc2(x.p, w.p, out.p, code_of(out_dtype, "gemm_bf16_tc2"), gated ? 1 : 0, (int)M, (int)N, (int)K,
                                    dev.tc_error_word(), dev.stream()),
                 "gemm_bf16_tc2");
    return out;
}

MatOrPartials linear(Device& dev, GemmBackend backend, const Mat& x, const Mat& w, DType out_dtype, bool defer_reduce) {
    MatOrPartials r;
    if (x.dtype == DType::F32) {
        r.m = gemm_f32(dev, x, w);
        return r;
    }
    need(x, "x", true, DType::BF16);
    need(w, "w", true, DType::BF16);
    const long long M = x.rows, K = x.cols, N = w.rows;
    if (M > 0 && K % 8 == 0 && (backend == GemmBackend::TC || (backend == GemmBackend::Auto && M <= kGemmTcMaxTokensAuto))) {
        if (M > 128 && N >= 256) {
            r.m = gemm_bf16_tc2(dev, x, w, out_dtype, false);     // prompts: pairs of SMs
            return r;
        }
        return gemm_bf16_tc(dev, x, w, out_dtype, 0, defer_reduce);
    }
    if (w.cols != K) throw KernelError("gemm: the operands' inner sizes differ");
    // the library sees whole buckets of rows where the activation was allocated so (see Mat::rows_held);
    // the rows beyond M are never initialised and never read back: a row of a product depends on its
    // own row of the input only
    long long Mlib = M;
    if (M > kLibraryRowBucket && M % kLibraryRowBucket && x.rows_held >= ceil_div(M, kLibraryRowBucket) * kLibraryRowBucket)
        Mlib = ceil_div(M, kLibraryRowBucket) * kLibraryRowBucket;
    r.m = new_mat_exact(dev, Mlib, N, out_dtype);
    r.m.rows = M;
    if (M > 0) dev.library_gemm_bf16(x.p, w.p, r.m.p, out_dtype, (int)Mlib, (int)N, (int)K);
    return r;
}

Mat linear_gated(Device& dev, GemmBackend backend, const Mat& x, const Mat& w) {
    const long long M = x.rows, K = x.cols, N = w.rows;
    if (x.dtype == DType::BF16 && w.dtype == DType::BF16 && M > 0 && K % 8 == 0 && N % 2 == 0 && !((uintptr_t)x.p & 15) &&
        !((uintptr_t)w.p & 15)) {
        const bool tc = backend == GemmBackend::TC || (backend == GemmBackend::Auto && M <= kGemmTcMaxTokensAuto);
        if (tc && M <= 64 && gemm_tc_splits(M, N, K, dev.n_sms()) == 1) {
            check_product(x, w, "gemm_bf16_tc_gated", true);
            Mat out = new_mat_exact(dev, M, N / 2, DType::BF16);
            check_kernel(illm_gemm_bf16_tc_gated(x.p, w.p, out.p, (int)M, (int)N, (int)K, dev.tc_error_word(), dev.stream()),
                         "gemm_bf16_tc_gated");
            return out;
        }
        if (N >= 256 && ((backend == GemmBackend::TC && M > 128) || (backend == GemmBackend::Auto && M >= kGatedPromptsOnTcMinTokens)))
            return gemm_bf16_tc2(dev, x, w, DType::BF16, true);
    }
    return swiglu(dev, linear(dev, backend, x, w, x.dtype, true));
}

// ---- rotation and attention

static void check_cache(const KVView& kv, DType want, Geometry g, const char* what) {
    if (kv.k == nullptr || kv.v == nullptr) throw KernelError(std::string(what) + ": the cache entry has no storage");
    if (kv.dtype != want)
        throw KernelError(std::string(what) + ": the cache pages must be " + dtype_word(want) + ", found " + dtype_word(kv.dtype));
    if (kv.n_kv_heads != g.n_kv_heads || kv.head_dim != g.head_dim)
        throw KernelError(std::string(what) + ": cache pages of " + std::to_string(kv.n_kv_heads) + " heads of " + std::to_string(kv.head_dim) +
                          " do not match the layer's " + std::to_string(g.n_kv_heads) + " heads of " + std::to_string(g.head_dim));
    if (((uintptr_t)kv.k & 15) || ((uintptr_t)kv.v & 15)) throw KernelError(std::string(what) + ": the cache pages must be 16-byte aligned");
}

Mat rope_kv_write(Device& dev, const MatOrPartials& in, const float* cos_sin, int rot_dim, long long n_pos, const StepView& ctx,
                  const KVView& kv, Geometry g) {
    const Partials* partials = nullptr;
    Mat qkv;
    if (in.is_partials()) {
        if (g.head_dim % 8 == 0 && rot_dim % 16 == 0 && kv.writes && kv.k && kv.dtype == DType::BF16) {
            partials = &in.part;
            qkv = new_mat_exact(dev, in.part.rows, in.part.cols, DType::BF16);
        } else {
            qkv = materialize(dev, in.part, DType::BF16);
        }
    } else {
        qkv = in.m;
    }
    need(qkv, "qkv");
    const long long T = qkv.rows;
    if (qkv.cols != (long long)(g.n_heads + 2 * g.n_kv_heads) * g.head_dim)
        throw KernelError("qkv width " + std::to_string(qkv.cols) + " is not (heads + 2 kv heads) * head_dim");
    if (kv.writes) check_cache(kv, qkv.dtype, g, "rope_kv_write");
    if (rot_dim && !cos_sin) throw KernelError("rope_kv_write: a rotation needs its cos/sin table");
    void* kc = kv.writes ? kv.k : nullptr;
    void* vc = kv.writes ? kv.v : nullptr;
    const int code = code_of(qkv.dtype, "rope_kv_write");
    if (partials)
        check_kernel(illm_rope_kv_write_partials(qkv.p, partials->ws, partials->splits, partials->rows * partials->cols, rot_dim ? cos_sin : nullptr,
                                                 ctx.token_pos, ctx.token_seq, kv.block_table, kv.width, kc, vc, code, (int)T, g.n_heads,
                                                 g.n_kv_heads, g.head_dim, rot_dim, kv.page_size, kv.writes ? 1 : 0, (int)(rot_dim ? n_pos : 0),
                                                 ctx.err, dev.stream()),
                     "rope_kv_write_partials");
    else
        check_kernel(illm_rope_kv_write(qkv.p, rot_dim ? cos_sin : nullptr, ctx.token_pos, ctx.token_seq, kv.block_table, kv.width, kc, vc, code,
                                        (int)T, g.n_heads, g.n_kv_heads, g.head_dim, rot_dim, kv.page_size, kv.writes ? 1 : 0,
                                        (int)(rot_dim ? n_pos : 0), ctx.err, dev.stream()),
                     "rope_kv_write");
    return qkv;
}

Mat attention_generic(Device& dev, const Mat& qkv, const KVView& kv, const StepView& ctx, Geometry g, float scale) {
    if (g.head_dim % 8 || g.head_dim > kMaxHeadDimGeneric)
        throw KernelError("attention: head size " + std::to_string(g.head_dim) + " is not supported (multiples of 8 up to " +
                          std::to_string(kMaxHeadDimGeneric) + ")");
    if (g.n_kv_heads <= 0 || g.n_heads % g.n_kv_heads) throw KernelError("attention: heads must be a multiple of kv heads");
    need(qkv, "qkv");
    check_cache(kv, qkv.dtype, g, "attention_generic");
    Mat out = new_mat(dev, qkv.rows, (long long)g.n_heads * g.head_dim, qkv.dtype);
    check_kernel(illm_attention_generic(qkv.p, (int)qkv.cols, kv.k, kv.v, kv.block_table, kv.width, ctx.token_pos, ctx.token_seq, out.p,
                                        code_of(qkv.dtype, "attention_generic"), (int)qkv.rows, g.n_heads, g.n_kv_heads, g.head_dim, kv.page_size,
                                        kv.window, scale, dev.stream()),
                 "attention_generic");
    return out;
}

typedef int (*DecodeFn)(const void*, int, const void*, const void*, const int*, int, const int*, const int*, float*, float*, void*, int, int,
                        int, int, int, int, float, int, void*);

static Mat decode_chunked(Device& dev, DecodeFn fn, const char* what, int chunk_keys, const Mat& qkv, const KVView& kv, const StepView& ctx,
                          Geometry g, float scale, long long max_len) {
    need(qkv, "qkv", true, DType::BF16);
    check_cache(kv, DType::BF16, g, what);
    const long long T = qkv.rows;
    const int n_chunks = (int)std::max<long long>(1, ceil_div(max_len, chunk_keys));
    float* part_acc = dev.alloc_n<float>((size_t)T * g.n_heads * n_chunks * g.head_dim);
    float* part_ml = dev.alloc_n<float>((size_t)T * g.n_heads * n_chunks * 2);
    Mat out = new_mat(dev, T, (long long)g.n_heads * g.head_dim, DType::BF16);
    for (long long t0 = 0; t0 < T; t0 += 65535) {
        const long long t1 = std::min(T, t0 + 65535);
        check_kernel(fn(row_ptr(qkv, t0), (int)qkv.cols, kv.k, kv.v, kv.block_table, kv.width, ctx.token_pos + t0, ctx.token_seq + t0,
                        part_acc + (size_t)t0 * g.n_heads * n_chunks * g.head_dim, part_ml + (size_t)t0 * g.n_heads * n_chunks * 2, row_ptr(out, t0),
                        (int)(t1 - t0), g.n_heads, g.n_kv_heads, g.head_dim, kv.page_size, kv.window, scale, n_chunks, dev.stream()),
                     what);
    }
    return out;
}

Mat attention_decode(Device& dev, const Mat& qkv, const KVView& kv, const StepView& ctx, Geometry g, float scale, long long max_len) {
    return decode_chunked(dev, illm_attention_decode, "attention_decode", kDecodeChunk, qkv, kv, ctx, g, scale, max_len);
}
Mat attention_decode_gqa(Device& dev, const Mat& qkv, const KVView& kv, const StepView& ctx, Geometry g, float scale, long long max_len) {
    return decode_chunked(dev, illm_attention_decode_gqa, "attention_decode_gqa", kGqaDecodeChunk, qkv, kv, ctx, g, scale, max_len);
}

Mat attention_decode_ring(Device& dev, const MatOrPartials& in, const KVView& kv, const StepView& ctx, Geometry g, float scale,
                          long long max_len, int splits, const FusedRope* rope) {
    long long T, width;
    if (in.is_partials()) {
        if (!rope) throw KernelError("attention_decode_ring: unreduced slices need the fused position encoding");
        T = in.part.rows;
        width = in.part.cols;
    } else {
        need(in.m, "qkv", true, DType::BF16);
        T = in.m.rows;
        width = in.m.cols;
    }
    check_cache(kv, DType::BF16, g, "attention_decode_ring");
    if (rope && width != (long long)(g.n_heads + 2 * g.n_kv_heads) * g.head_dim)
        throw KernelError("qkv width " + std::to_string(width) + " is not (heads + 2 kv heads) * head_dim");
    Mat out = new_mat_exact(dev, T, (long long)g.n_heads * g.head_dim, DType::BF16);
    for (long long t0 = 0; t0 < T; t0 += 65535) {
        const long long t1 = std::min(T, t0 + 65535);
        const int n = splits > 0 ? splits : attention_decode_ring_splits(t1 - t0, g.n_kv_heads, max_len, g.head_dim, dev.n_sms(), dev.stream_bytes_per_us());
        float *part_acc = nullptr, *part_ml = nullptr;
        if (n > 1) {
            part_acc = dev.alloc_n<float>((size_t)(t1 - t0) * g.n_heads * n * g.head_dim);
            part_ml = dev.alloc_n<float>((size_t)(t1 - t0) * g.n_heads * n * 2);
        }
        if (!rope) {
            check_kernel(illm_attention_decode_ring(row_ptr(in.m, t0), (int)width, kv.k, kv.v, kv.num_pages, kv.block_table, kv.width,
                                                    ctx.token_pos + t0, ctx.token_seq + t0, part_acc, part_ml, row_ptr(out, t0), (int)(t1 - t0),
                                                    g.n_heads, g.n_kv_heads, g.head_dim, kv.page_size, kv.window, scale, n, dev.tc_error_word(),
                                                    dev.stream()),
                         "attention_decode_ring");
            continue;
        }
        if (rope->rot_dim && !rope->cos_sin) throw KernelError("attention_decode_ring: a rotation needs its cos/sin table");
        if (T > 65535) throw KernelError("attention_decode_ring with the position encoding inside takes at most 65535 tokens");
        check_kernel(illm_attention_decode_ring_rope(in.is_partials() ? nullptr : in.m.p, in.is_partials() ? in.part.ws : nullptr,
                                                     in.is_partials() ? in.part.splits : 0, in.is_partials() ? T * width : 0,
                                                     rope->rot_dim ? rope->cos_sin : nullptr, rope->rot_dim, (int)(rope->rot_dim ? rope->n_pos : 0),
                                                     rope->write_kv ? 1 : 0, kv.k, kv.v, kv.num_pages, kv.block_table, kv.width, ctx.token_pos,
                                                     ctx.token_seq, part_acc, part_ml, out.p, (int)T, g.n_heads, g.n_kv_heads, g.head_dim,
                                                     kv.page_size, kv.window, scale, n, dev.tc_error_word(), rope->step_err, dev.stream()),
                     "attention_decode_ring_rope");
    }
    return out;
}

Mat attention_prefill(Device& dev, const Mat& qkv, const KVView& kv, const StepView& ctx, Geometry g, float scale) {
    need(qkv, "qkv", true, DType::BF16);
    check_cache(kv, DType::BF16, g, "attention_prefill");
    Mat out = new_mat(dev, qkv.rows, (long long)g.n_heads * g.head_dim, DType::BF16);
    check_kernel(illm_attention_prefill(qkv.p, (int)qkv.cols, kv.k, kv.v, kv.block_table, kv.width, ctx.cu_q, ctx.seq_lens, out.p, ctx.B, ctx.max_q,
                                        g.n_heads, g.n_kv_heads, g.head_dim, kv.page_size, kv.window, scale, dev.stream()),
                 "attention_prefill");
    return out;
}

Mat attention_prefill_tc(Device& dev, const Mat& qkv, const KVView& kv, const StepView& ctx, Geometry g, float scale) {
    need(qkv, "qkv", true, DType::BF16);
    check_cache(kv, DType::BF16, g, "attention_prefill_tc");
    Mat out = new_mat(dev, qkv.rows, (long long)g.n_heads * g.head_dim, DType::BF16);
    check_kernel(illm_attention_prefill_tc(qkv.p, (int)qkv.cols, (int)qkv.rows, kv.k, kv.v, kv.num_pages, kv.block_table, kv.width, ctx.cu_q,
                                           ctx.seq_lens, out.p, ctx.B, ctx.max_q, g.n_heads, g.n_kv_heads, g.head_dim, kv.page_size, kv.window,
                                           scale, dev.tc_error_word(), dev.stream()),
                 "attention_prefill_tc");
    return out;
}

Mat attention(Device& dev, const Mat& qkv, const KVView& kv, const StepView& ctx, Geometry g, float scale) {
    const int nh = g.n_heads, nkv = g.n_kv_heads, d = g.head_dim, group = nkv ? nh / nkv : 0;
    // grids and scratch of the decode kernels are sized for the longest sequence the cache allows, so
    // that the launch is the same at every step
    if (ctx.is_decode && attention_decode_ring_supported(qkv.dtype, nh, nkv, d, kv.page_size)) {
        MatOrPartials in;
        in.m = qkv;
        return attention_decode_ring(dev, in, kv, ctx, g, scale, ctx.max_seq_len, 0, nullptr);
    }
    if (ctx.is_decode && (group >= kGqaDecodeMinGroup || !attention_decode_supported(qkv.dtype, nh, nkv, d, kv.page_size)) &&
        attention_decode_gqa_supported(qkv.dtype, nh, nkv, d))
        return attention_decode_gqa(dev, qkv, kv, ctx, g, scale, ctx.max_seq_len);
    if (ctx.is_decode && attention_decode_supported(qkv.dtype, nh, nkv, d, kv.page_size))
        return attention_decode(dev, qkv, kv, ctx, g, scale, ctx.max_seq_len);
    if (!ctx.is_decode && attention_prefill_tc_supported(qkv.dtype, nh, nkv, d, kv.page_size))
        return attention_prefill_tc(dev, qkv, kv, ctx, g, scale);
    if (!ctx.is_decode && attention_prefill_supported(qkv.dtype, nh, nkv, d)) return attention_prefill(dev, qkv, kv, ctx, g, scale);
    return attention_generic(dev, qkv, kv, ctx, g, scale);
}

// ---- sampling and utilities

int* argmax(Device& dev, const float* logits, long long B, long long V, int* out) {
    if (!out) out = dev.alloc_n<int>((size_t)std::max<long long>(B, 1));
    const long long n_chunks = ceil_div(V, 2048);
    for (long long b0 = 0; b0 < B; b0 += 65535) {
        const long long b1 = std::min(B, b0 + 65535);
        float* sv = dev.alloc_n<float>((size_t)(b1 - b0) * n_chunks);
        int* si = dev.alloc_n<int>((size_t)(b1 - b0) * n_chunks);
        check_kernel(illm_argmax(logits + (size_t)b0 * V, (int)(b1 - b0), (int)V, (int)V, out + b0, sv, si, dev.stream()), "argmax");
    }
    return out;
}

int* sample(Device& dev, const float* logits, long long B, long long V, const float* uniforms, float temp, int top_k, float top_p,
            float repeat_penalty, const int* last_tokens, int n_last, int* out) {
    if (!out) out = dev.alloc_n<int>((size_t)std::max<long long>(B, 1));
    float* z = dev.alloc_n<float>((size_t)B * V);
    for (long long b0 = 0; b0 < B; b0 += 65535) {
        const long long b1 = std::min(B, b0 + 65535);
        // temperature alone and top_k <= 64 run in two passes over chunks of the row and need scratch
        const long long n_scratch = illm_sample_scratch_elems((int)(b1 - b0), (int)V, top_k, top_p);
        int* scratch = n_scratch ? dev.alloc_n<int>((size_t)n_scratch) : nullptr;
        check_kernel(illm_sample(logits + (size_t)b0 * V, (int)(b1 - b0), (int)V, (int)V, z + (size_t)b0 * V,
                                 last_tokens ? last_tokens + (size_t)b0 * n_last : nullptr, last_tokens ? n_last : 0, temp, repeat_penalty, top_k,
                                 top_p, uniforms + b0, out + b0, scratch, dev.stream()),
                     "sample");
    }
    return out;
}

void fill_random(Device& dev, void* out, DType dtype, long long n, unsigned long long key, float std, float mean) {
    check_kernel(illm_fill_random(out, code_of(dtype, "fill_random"), n, key, std, mean, dev.stream()), "fill_random");
}

void convert(Device& dev, const void* src, DType src_dtype, void* dst, DType dst_dtype, long long n) {
    const int rc = illm_convert(src, (int)src_dtype, dst, (int)dst_dtype, n, dev.stream());
    if (rc == 10001)
        throw KernelError(std::string("a tensor stored as ") + dtype_word(src_dtype) + " cannot be brought to " + dtype_word(dst_dtype));
    check_kernel(rc, "convert");
}

}  // namespace ops
}  // namespace illm
