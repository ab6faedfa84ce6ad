// Position encoding of Q and K (rotate-half) fused with the write of K and V into the paged
// cache.
//
// The reference rotates Q and the new K rows in place (src/kern/gpu/kernel_gpu.cu:343-401,
// formula src/kern/naive/naive.cpp:389-414: pair (j, j + rot/2), angle p * theta^(-2j/rot)),
// after the K and V projections have written straight into the cache rows
// (src/core/op.cpp:414-416).  Here one launch reads the packed projection
// qkv[t] = [q heads | k heads | v heads], rotates Q in place, and stores rotated K and plain V
// at the token's place in the cache: page block_table[seq, p / page_size], offset p % page_size
// of a cache laid out [page, kv head, offset, d].  cos and sin come from a float32 table
// [position, rot/2] that the host computed in float64; the rotation itself is float32.
// rot = 0 turns the rotation off (the launch is then only the cache write); write_kv = 0
// leaves the cache alone (a layer that reads another layer's keys and values).
#include "common.cuh"

#define RK_WARPS 4
#define RK_SLOTS_PER_WARP 4         // scalar kernel: each warp takes its head slots one after the other
#define RK_VEC_THREADS 256

// x / d and x % d for a divisor that the host found to be a power of two (shift >= 0) or not
__device__ __forceinline__ int rk_div(int x, int d, int shift) { return shift >= 0 ? x >> shift : x / d; }

// The 16-byte path (d, rot and rot/2 multiples of 8): one work item per thread.  A token's items
// are, for each Q and K head, its rot/16 rotated pairs of 8-channel chunks and its chunks outside the
// rotated part, then the d/8 chunks of each V head; block (t, y) takes items y*256 .. y*256+255 of
// token t.  The loads of the projection are issued first (they need only the item), the token's
// position, its cos/sin row and, for K and V items only, its page are looked up behind them.
// PARTIALS: the projection comes as `splits` float32 slices of a split-K matrix product; a chunk is
// then the sum of its slices in ascending order, Q is written to `qkv` for the attention kernel and
// K and V go to the cache only.
template <typename TA, bool PARTIALS>
__global__ void __launch_bounds__(RK_VEC_THREADS)
rope_kv_vec_kernel(TA* __restrict__ qkv, const float2* __restrict__ cs, const int* __restrict__ token_pos,
                   const int* __restrict__ token_seq, const int* __restrict__ block_table, int max_pages,
                   TA* __restrict__ kc, TA* __restrict__ vc, int nh, int nkv, int d, int rot, int page_size,
                   int write_kv, int table_positions, int* __restrict__ err, const float* __restrict__ partials,
                   int splits, long long split_stride, int ipc_shift, int cpd_shift) {
    pdl_grid_sync();
    const int t = blockIdx.x;
    const int half = rot >> 1, cpd = d >> 3, hc = half >> 3, ipc = cpd - hc;
    const int n_rot_items = (nh + nkv) * ipc, n_items = n_rot_items + nkv * cpd;
    const int idx = blockIdx.y * RK_VEC_THREADS + threadIdx.x;
    if (idx >= n_items) return;
    int slot, c;
    if (idx < n_rot_items) {
        slot = rk_div(idx, ipc, ipc_shift);
        c = idx - slot * ipc;
        if (c >= hc) c += hc;                 // behind the rotated part
    } else {
        const int i2 = idx - n_rot_items, s2 = rk_div(i2, cpd, cpd_shift);
        slot = nh + nkv + s2;
        c = i2 - s2 * cpd;
    }
    const bool is_q = slot < nh, is_k = !is_q && slot < nh + nkv;
    const bool rotate = (is_q || is_k) && c < hc;
    if (is_q && !rotate && !PARTIALS) return;          // Q outside the rotated part stays where it is
    if (!is_q && !write_kv) return;
    const size_t off = (size_t)t * (nh + 2 * nkv) * d + (size_t)slot * d + c * 8;
    auto fetch = [&](size_t o, float* out8) {
        if (PARTIALS) {
#pragma unroll
            for (int k = 0; k < 8; k++) out8[k] = 0.f;
            for (int z = 0; z < splits; z++) {
                float p8[8];
                load8(partials + (size_t)z * split_stride + o, p8);
#pragma unroll
                for (int k = 0; k < 8; k++) out8[k] += p8[k];
            }
        } else {
            load8(qkv + o, out8);
        }
    };
    float a[8], b[8];
    fetch(off, a);
    if (rotate) fetch(off + half, b);
    const int p = token_pos[t];
    if (half > 0 && p >= table_positions) {
        atomicExch(err, 3);
        return;
    }
    TA* dst = qkv + off;
    if (!is_q) {
        const int page = block_table[(size_t)token_seq[t] * max_pages + p / page_size];
        if (page < 0) {
            atomicExch(err, 2);
            return;
        }
        const int hk = is_k ? slot - nh : slot - nh - nkv;
        dst = (is_k ? kc : vc) + (((size_t)page * nkv + hk) * page_size + (p % page_size)) * d + c * 8;
    }
    if (rotate) {
        const float2* cst = cs + (size_t)p * half + c * 8;
        float ra[8], rb[8];
#pragma unroll
        for (int k = 0; k < 8; k += 2) {
            const float4 cc = *reinterpret_cast<const float4*>(cst + k);   // (cos, sin) x 2
            ra[k] = a[k] * cc.x - b[k] * cc.y;
            rb[k] = a[k] * cc.y + b[k] * cc.x;
            ra[k + 1] = a[k + 1] * cc.z - b[k + 1] * cc.w;
            rb[k + 1] = a[k + 1] * cc.w + b[k + 1] * cc.z;
        }
        store8(dst, ra);
        store8(dst + half, rb);
    } else {
        store8(dst, a);
    }
}

// Any other sizes: element by element, a warp per group of head slots.
template <typename TA>
__global__ void rope_kv_write_kernel(TA* __restrict__ qkv, const float2* __restrict__ cs,
                                     const int* __restrict__ token_pos,
                                     const int* __restrict__ token_seq,
                                     const int* __restrict__ block_table, int max_pages,
                                     TA* __restrict__ kc, TA* __restrict__ vc, int nh, int nkv, int d,
                                     int rot, int page_size, int write_kv, int table_positions,
                                     int* __restrict__ err) {
    pdl_grid_sync();
    const int t = blockIdx.x;
    const int p = token_pos[t];
    const int half = rot >> 1;
    TA* row = qkv + (size_t)t * (nh + 2 * nkv) * d;
    TA* kdst = nullptr;
    TA* vdst = nullptr;
    if (write_kv) {
        const int page = block_table[(size_t)token_seq[t] * max_pages + p / page_size];
        if (page < 0) {
            if (threadIdx.x == 0) atomicExch(err, 2);
            write_kv = 0;
        } else {
            size_t base = ((size_t)page * nkv * page_size + (p % page_size)) * d;
            kdst = kc + base;
            vdst = vc + base;
        }
    }
    if (half > 0 && p >= table_positions) {
        if (threadIdx.x == 0) atomicExch(err, 3);
        return;
    }
    const size_t head_stride = (size_t)page_size * d;  // between kv heads inside a page
    // this block's share of the head slots: [q heads | k heads | v heads]
    const int n_slots = nh + 2 * nkv;
    const int lane = threadIdx.x & 31;
    const int s0 = blockIdx.y * RK_WARPS * RK_SLOTS_PER_WARP + (threadIdx.x >> 5) * RK_SLOTS_PER_WARP;
    const int s1 = min(n_slots, s0 + RK_SLOTS_PER_WARP);
    const float2* cst = cs + (size_t)p * half;
    const int rest = d - rot;
    for (int slot = s0; slot < s1; slot++) {
        TA* src = row + (size_t)slot * d;
        if (slot < nh + nkv) {
            const bool is_k = slot >= nh;
            if (is_k && !write_kv) continue;
            TA* dst = is_k ? kdst + (size_t)(slot - nh) * head_stride : src;
            for (int j = lane; j < half; j += 32) {
                const float a = to_f32(src[j]), b = to_f32(src[j + half]);
                const float2 c = cst[j];
                dst[j] = from_f32<TA>(a * c.x - b * c.y);
                dst[j + half] = from_f32<TA>(a * c.y + b * c.x);
            }
            if (is_k)   // K channels outside the rotated part
                for (int c = rot + lane; c < rot + rest; c += 32) dst[c] = src[c];
        } else if (write_kv) {
            TA* dst = vdst + (size_t)(slot - nh - nkv) * head_stride;
            for (int c = lane; c < d; c += 32) dst[c] = src[c];
        }
    }
}

static int rope_launch(void* qkv, const float* cos_sin, const int* token_pos, const int* token_seq,
                       const int* block_table, int max_pages, void* kc, void* vc, int act_dtype, int T, int nh,
                       int nkv, int d, int rot, int page_size, int write_kv, int table_positions, int* err,
                       void* stream, const float* partials, int splits, long long split_stride);

extern "C" int illm_rope_kv_write(void* qkv, const float* cos_sin, const int* token_pos,
                                  const int* token_seq, const int* block_table, int max_pages,
                                  void* kc, void* vc, int act_dtype, int T, int nh, int nkv, int d,
                                  int rot, int page_size, int write_kv, int table_positions,
                                  int* err, void* stream) {
    return rope_launch(qkv, cos_sin, token_pos, token_seq, block_table, max_pages, kc, vc, act_dtype, T, nh, nkv, d,
                       rot, page_size, write_kv, table_positions, err, stream, nullptr, 0, 0);
}

// The same with the packed projection given as `splits` float32 slices [splits][T][(nh+2nkv)*d] of a
// split-K matrix product; `qkv` receives the rotated Q heads (its K and V columns stay unwritten).
// Needs the 16-byte path: d, rot and rot/2 multiples of 8.
extern "C" int illm_rope_kv_write_partials(void* qkv, const float* partials, int splits, long long split_stride,
                                           const float* cos_sin, const int* token_pos, const int* token_seq,
                                           const int* block_table, int max_pages, void* kc, void* vc,
                                           int act_dtype, int T, int nh, int nkv, int d, int rot, int page_size,
                                           int write_kv, int table_positions, int* err, void* stream) {
    if (!partials || splits < 1 || (d & 7) || (rot & 15)) return ILLM_ERR_BAD_ARG;
    return rope_launch(qkv, cos_sin, token_pos, token_seq, block_table, max_pages, kc, vc, act_dtype, T, nh, nkv, d,
                       rot, page_size, write_kv, table_positions, err, stream, partials, splits, split_stride);
}

static int rk_shift(int d) { return (d > 0 && (d & (d - 1)) == 0) ? __builtin_ctz((unsigned)d) : -1; }

static int rope_launch(void* qkv, const float* cos_sin, const int* token_pos, const int* token_seq,
                       const int* block_table, int max_pages, void* kc, void* vc, int act_dtype, int T, int nh,
                       int nkv, int d, int rot, int page_size, int write_kv, int table_positions, int* err,
                       void* stream, const float* partials, int splits, long long split_stride) {
    if (T <= 0) return 0;
    if (rot < 0 || rot > d || (rot & 1) || (rot > 0 && cos_sin == nullptr)) return ILLM_ERR_BAD_ARG;
    if (act_dtype != ILLM_BF16 && act_dtype != ILLM_F32) return ILLM_ERR_BAD_ARG;
    cudaStream_t s = (cudaStream_t)stream;
    const int n_slots = nh + 2 * nkv;
    if (T > 2147483647 / 2) return ILLM_ERR_BAD_ARG;
    const bool vec = ((rot & 15) == 0) && ((d & 7) == 0);
    if (vec) {
        const int cpd = d / 8, ipc = cpd - rot / 16;
        const int n_items = (nh + nkv) * ipc + nkv * cpd;
        dim3 grid(T, (n_items + RK_VEC_THREADS - 1) / RK_VEC_THREADS);
        if (grid.y > 65535) return ILLM_ERR_BAD_ARG;
#define RK_VEC(TA, PART)                                                                                          \
    illm_launch(rope_kv_vec_kernel<TA, PART>, grid, dim3(RK_VEC_THREADS), 0, s, (TA*)qkv, (const float2*)cos_sin,  \
                token_pos, token_seq, block_table, max_pages, (TA*)kc, (TA*)vc, nh, nkv, d, rot, page_size,      \
                write_kv, table_positions, err, partials, splits, split_stride, rk_shift(ipc), rk_shift(cpd))
        if (act_dtype == ILLM_BF16 && partials) RK_VEC(bf16, true);
        else if (act_dtype == ILLM_BF16) RK_VEC(bf16, false);
        else if (partials) return ILLM_ERR_BAD_ARG;
        else RK_VEC(float, false);
#undef RK_VEC
        return illm_launch_status();
    }
    if (partials) return ILLM_ERR_BAD_ARG;
    dim3 grid(T, (n_slots + RK_WARPS * RK_SLOTS_PER_WARP - 1) / (RK_WARPS * RK_SLOTS_PER_WARP));
    if (grid.y > 65535) return ILLM_ERR_BAD_ARG;
    if (act_dtype == ILLM_BF16)
        illm_launch(rope_kv_write_kernel<bf16>, grid, dim3(RK_WARPS * 32), 0, s, (bf16*)qkv, (const float2*)cos_sin,
                    token_pos, token_seq, block_table, max_pages, (bf16*)kc, (bf16*)vc, nh, nkv, d, rot, page_size,
                    write_kv, table_positions, err);
    else
        illm_launch(rope_kv_write_kernel<float>, grid, dim3(RK_WARPS * 32), 0, s, (float*)qkv, (const float2*)cos_sin,
                    token_pos, token_seq, block_table, max_pages, (float*)kc, (float*)vc, nh, nkv, d, rot, page_size,
                    write_kv, table_positions, err);
    return illm_launch_status();
}
