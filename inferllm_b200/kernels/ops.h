// The C++ faces of the CUDA kernels: argument checks, the choice of a kernel for the sizes at
// hand, scratch and results from the step arena, the launch.
//
// Every function launches on the device's stream and returns without synchronising.  A size that a
// kernel cannot take is refused with a KernelError that names it; nothing falls back to another
// implementation, except that the plain matrix product of the bfloat16 mode is the library's
// (cuBLAS), as the reference's is (cublasSgemm, src/kern/gpu/kernel_gpu.cu:420-435).  Results are cut
// from the device's step arena and live until the next step rewinds it.
#pragma once
#include <cstdint>
#include <string>

#include "cache/cache.h"
#include "device/device.h"

namespace illm {

// A row-major matrix on the device: rows x cols elements of `dtype`, rows contiguous.
struct Mat {
    void* p = nullptr;
    long long rows = 0, cols = 0;
    DType dtype = DType::BF16;
    // Rows that the allocation really holds (>= rows): prompt-sized bfloat16 activations are allocated
    // in whole buckets of 64 rows, so that the library's products only ever see multiples of 64 rows
    // (it chooses a kernel per shape, which costs milliseconds the first time a shape is seen).
    long long rows_held = 0;
    size_t bytes() const { return (size_t)rows * cols * dtype_size(dtype); }
};

// The K slices of a split matrix product that have not been added up yet: float32
// [splits, rows, cols].  The norm, the rotation and the decode attention kernels take it in place of
// the finished matrix and do the addition themselves (ascending order of the slice, as the
// stand-alone reduction does), which saves a kernel per product in a decode step.
struct Partials {
    float* ws = nullptr;
    int splits = 0;
    long long rows = 0, cols = 0;
};

// Either a finished matrix or unreduced slices.
struct MatOrPartials {
    Mat m;
    Partials part;
    bool is_partials() const { return part.ws != nullptr; }
    long long rows() const { return is_partials() ? part.rows : m.rows; }
    long long cols() const { return is_partials() ? part.cols : m.cols; }
};

// What every part sees of a step, on the device: int32 arrays in one buffer.
struct StepView {
    const int* ids = nullptr;         // [T] token id
    const int* token_pos = nullptr;   // [T] absolute position
    const int* token_seq = nullptr;   // [T] index of the token's sequence within the step
    const int* want_rows = nullptr;   // [K] rows (among the T tokens) whose logits are wanted
    const int* slots = nullptr;       // [B]
    const int* seq_lens = nullptr;    // [B] length after the step
    const int* cu_q = nullptr;        // [B + 1] token offsets of the sequences
    int T = 0, B = 0, K = 0;
    int max_q = 0;                    // the most tokens one sequence brings
    long long max_len = 0;            // the longest sequence after the step
    long long max_seq_len = 0;        // the longest sequence the cache allows (sizes decode grids and scratch)
    bool is_decode = false;           // one token per sequence
    int* err = nullptr;               // the step's error word
};

namespace ops {

enum class GemmBackend { Auto, TC, Library };
// Which kernel runs the bfloat16 matrix products.  TC: the package's tcgen05 kernels for every
// product they can take (K a multiple of 8): gemm_tc.cu up to 128 tokens, the SM-pair kernel
// gemm_tc2.cu above; Library: cuBLAS; Auto (default): the tcgen05 kernel for small decode batches (at
// most 16 tokens), where its swapped, split-K form with weight prefetch across kernel boundaries is
// faster than the library (74.8 against 89.5 us for the four products of a 7B layer at batch 1, 78.1
// against 79.4 at batch 16), and the library for larger ones.  From 17 to 64 tokens the kernel alone
// still matches the library (85.0 against 88.1 us at 64 tokens, back to back), but its float32 K
// slices grow with the tokens and their readers (the norms, the fused attention) pay for them: whole
// 7B decode steps at context 600 take 4.35 ms with the library and 4.47 ms with the kernel at batch
// 24, 4.77 and 5.01 at batch 32, 5.86 and 6.17 at batch 48.  Gate/up products of prompts from 512
// tokens on run on the SM-pair kernel with the activation as their epilogue.
GemmBackend gemm_backend_from_name(const std::string& name);
const char* gemm_backend_name(GemmBackend b);

constexpr int kLibraryRowBucket = 64;
constexpr int kGemmTcMaxTokensAuto = 16;
constexpr int kGatedPromptsOnTcMinTokens = 512;
constexpr int kMaxHeadDimGeneric = 256;
constexpr int kMaxNormWidth = 200 * 1024 / 4;
constexpr int kDecodeChunk = 256, kGqaDecodeChunk = 128, kGqaDecodeMinGroup = 4, kRingDecodeMaxSplits = 32;

// An uninitialised [rows, cols] activation from the step arena; for prompt-sized bfloat16 rows the
// head of a buffer of whole buckets.
Mat new_mat(Device& dev, long long rows, long long cols, DType dtype);

// ---- policies (pure functions, tested on the CPU)

// How many slices of K a decode-sized product (M <= 64) is cut into, so that about two blocks per SM
// stream the weights; 1 for larger M.
int gemm_tc_splits(long long M, long long N, long long K, int n_sms);
// Blocks per (token, kv head) of the ring decode attention, by a small model of the kernel's time
// fitted to measurements (13B size, batch 8, context 4096, 320 pairs: 1 split 129 us, 6 splits 106 us;
// 160 pairs: 1 split 56 us, 2 splits 69 us).  Two blocks fit an SM, so 2 * n_sms run at once.  Up to
// that number the kernel streams at the memory rate once about 160 blocks are at work.  Beyond it the
// blocks run in waves, and a last wave of few blocks still takes 0.43 of a full one (a block alone is
// bound by what one SM can take in), so a grid a little larger than one wave is the worst and one of
// many waves is fine again.  Splits cost their partial results and the merge (2.5 us and 0.7 us per
// split), every wave about 1 us of start-up.  At most one split per 64-key tile and at most 32.
int attention_decode_ring_splits(long long T, int n_kv_heads, long long max_len, int head_dim, int n_sms,
                                 double stream_bytes_per_us = 6.6e6);
bool attention_decode_ring_supported(DType dtype, int nh, int nkv, int d, int page_size);
bool attention_decode_supported(DType dtype, int nh, int nkv, int d, int page_size);
bool attention_decode_gqa_supported(DType dtype, int nh, int nkv, int d);
bool attention_prefill_supported(DType dtype, int nh, int nkv, int d);
bool attention_prefill_tc_supported(DType dtype, int nh, int nkv, int d, int page_size);
// Which attention kernel a configuration gets for prompts and for single tokens (for the log line at
// engine start): "prefill_tc/decode_ring", "generic/generic", ...
std::string attention_kernels_for(DType dtype, int nh, int nkv, int d, int page_size);

// ---- kernels

Mat embedding(Device& dev, const int* ids, long long T, const Mat& table, int* err);
// y = rmsnorm(resid (+ delta)) * weight; resid is updated in place when write_resid.  rows (int32
// [n_rows], device) gathers: only those rows are normed and y is [n_rows, H].
Mat add_rmsnorm(Device& dev, const Mat& resid, const MatOrPartials* delta, const Mat& weight, float eps, DType out_dtype,
                const int* rows, long long n_rows, bool write_resid);
void residual_add(Device& dev, const Mat& resid, const MatOrPartials& delta);
Mat materialize(Device& dev, const Partials& p, DType dtype);
Mat swiglu(Device& dev, const MatOrPartials& gu);
Mat gemm_f32(Device& dev, const Mat& x, const Mat& w);
MatOrPartials gemm_bf16_tc(Device& dev, const Mat& x, const Mat& w, DType out_dtype, int splits /* 0: by policy */, bool defer_reduce);
Mat gemm_bf16_tc2(Device& dev, const Mat& x, const Mat& w, DType out_dtype, bool gated);
// x [M, K] . w [N, K]^T.  defer_reduce allows the result to come back as unreduced slices (only a
// caller that hands it to add_rmsnorm, the rotation or the fused decode attention asks).
MatOrPartials linear(Device& dev, GemmBackend backend, const Mat& x, const Mat& w, DType out_dtype, bool defer_reduce);
// silu(gate) * up of x . w^T, where w's rows 2i, 2i + 1 are the gate and the up row of output i.
Mat linear_gated(Device& dev, GemmBackend backend, const Mat& x, const Mat& w);

struct Geometry { int n_heads, n_kv_heads, head_dim; };
// Rotate Q (and K) of the packed projection and store K, V in the cache pages.  cos_sin: float32
// [positions, rot_dim / 2, 2] or nullptr with rot_dim 0.  Returns the matrix whose first
// n_heads * head_dim columns hold the rotated queries: qkv itself (rotated in place), or, if qkv came
// as unreduced slices, a new one (the slices are added up on the way).
Mat rope_kv_write(Device& dev, const MatOrPartials& qkv, const float* cos_sin, int rot_dim, long long n_pos, const StepView& ctx,
                  const KVView& kv, Geometry g);
Mat attention_generic(Device& dev, const Mat& qkv, const KVView& kv, const StepView& ctx, Geometry g, float scale);
Mat attention_decode(Device& dev, const Mat& qkv, const KVView& kv, const StepView& ctx, Geometry g, float scale, long long max_len);
Mat attention_decode_gqa(Device& dev, const Mat& qkv, const KVView& kv, const StepView& ctx, Geometry g, float scale, long long max_len);
struct FusedRope { const float* cos_sin; int rot_dim; long long n_pos; bool write_kv; int* step_err; };
Mat attention_decode_ring(Device& dev, const MatOrPartials& qkv, const KVView& kv, const StepView& ctx, Geometry g, float scale,
                          long long max_len, int splits /* 0: by policy */, const FusedRope* rope);
Mat attention_prefill(Device& dev, const Mat& qkv, const KVView& kv, const StepView& ctx, Geometry g, float scale);
Mat attention_prefill_tc(Device& dev, const Mat& qkv, const KVView& kv, const StepView& ctx, Geometry g, float scale);
// Attention of the step's tokens over a cache entry: picks the kernel for the dtype, head size and kind of step.
Mat attention(Device& dev, const Mat& qkv, const KVView& kv, const StepView& ctx, Geometry g, float scale);

// float32 [B, V] -> int32 [B], the lowest id among equal maxima.
int* argmax(Device& dev, const float* logits, long long B, long long V, int* out /* nullptr: from the arena */);
// Temperature / repetition penalty / top-k / top-p sampling, one draw per row (the reference's chain,
// src/utils.cpp:31-115).  uniforms float32 [B] in [0, 1); last_tokens int32 [B, n_last] (-1 pads) or nullptr.
int* sample(Device& dev, const float* logits, long long B, long long V, const float* uniforms, float temp, int top_k, float top_p,
            float repeat_penalty, const int* last_tokens, int n_last, int* out /* nullptr: from the arena */);
void fill_random(Device& dev, void* out, DType dtype, long long n, unsigned long long key, float std, float mean);
void convert(Device& dev, const void* src, DType src_dtype, void* dst, DType dst_dtype, long long n);

long long launch_count();               // kernels of this package launched so far (graph replays counted by the engine)
void count_replayed_launches(long long n);
void set_pdl(bool on);

}  // namespace ops
}  // namespace illm
