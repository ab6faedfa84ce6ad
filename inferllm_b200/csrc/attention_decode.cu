// Attention of single tokens over long paged caches, bfloat16, bound by reading K and V once.
//
// One decode step must read every cached key and value of every live sequence; nothing else of
// the attention costs anything.  So the work is cut for bandwidth: a block owns one
// (token, kv head, chunk of 256 keys) and handles all query heads of that kv head together, so a
// key or value is fetched once however many query heads share it (the reference's only grouped
// attention loops over the query heads and re-reads K and V for each,
// src/kern/gpu/kernel_gpu.cu:688-756).  Inside a block every key row is read by D/8 neighbouring
// lanes with one 16-byte load each (fully coalesced), eight keys per lane group in flight, and
// each lane group keeps a running maximum, sum and weighted value sum of its own (scores and
// softmax in float32; formulas src/kern/naive/naive.cpp:606-632, :531-553, :209-240, :664-691).
// Partial results go to a scratch buffer [token, head, chunk] and a second kernel merges the
// chunks of a token in ascending order.  Which keys fall into which chunk and lane group depends
// only on the token's own position, so the result does not depend on the rest of the batch.
// The grid covers the chunks of the longest possible sequence; blocks beyond a token's own
// length return at once, which keeps the launch identical from step to step (CUDA graphs).
#include <math.h>

#include "common.cuh"

#define AD_THREADS 128
#define AD_CHUNK 256   // keys per block
#define AD_U 8         // keys per lane group and iteration

// 16-byte load that does not linger in L1 (every key and value is used once per step)
__device__ __forceinline__ uint4 ld_stream16(const bf16* p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}
__device__ __forceinline__ void unpack8(const uint4& u, float* f) {
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
    for (int i = 0; i < 4; i++) {
        const float2 t = __bfloat1622float2(h[i]);
        f[2 * i] = t.x;
        f[2 * i + 1] = t.y;
    }
}

template <int D, int G>
__global__ void __launch_bounds__(AD_THREADS)
attention_decode_kernel(const bf16* __restrict__ q, int q_stride, const bf16* __restrict__ kc,
                        const bf16* __restrict__ vc, const int* __restrict__ block_table, int max_pages,
                        const int* __restrict__ token_pos, const int* __restrict__ token_seq,
                        float* __restrict__ part_acc, float* __restrict__ part_ml, int n_chunks, int nh,
                        int nkv, int page_size, int window, float scale_log2e) {
    pdl_grid_sync();
    constexpr int LPK = D / 8;                 // lanes per key
    constexpr int GROUPS = AD_THREADS / LPK;   // independent softmax streams in the block
    const int chunk = blockIdx.x, hk = blockIdx.y, t = blockIdx.z;
    const int p = token_pos[t];
    const int lo = (window > 0 && p - window + 1 > 0) ? p - window + 1 : 0;
    const int c0 = chunk * AD_CHUNK;
    if (c0 > p || c0 + AD_CHUNK <= lo) return;
    const int first = c0 > lo ? c0 : lo;                       // first key of this block
    const int last = (c0 + AD_CHUNK - 1 < p) ? c0 + AD_CHUNK - 1 : p;  // last key, inclusive

    const int tid = threadIdx.x;
    const int grp = tid / LPK, sub = tid % LPK;
    const int* bt = block_table + (size_t)token_seq[t] * max_pages;

    float qr[G][8];
#pragma unroll
    for (int g = 0; g < G; g++) load8(q + (size_t)t * q_stride + (size_t)(hk * G + g) * D + sub * 8, qr[g]);

    float m[G], l[G], acc[G][8];
#pragma unroll
    for (int g = 0; g < G; g++) {
        m[g] = -INFINITY;
        l[g] = 0.f;
#pragma unroll
        for (int i = 0; i < 8; i++) acc[g][i] = 0.f;
    }

    // lane group `grp` takes keys base + grp*AD_U + u of every stretch of GROUPS*AD_U keys
    const int aligned = first - (first % AD_U);   // AD_U keys never straddle a page (page_size % AD_U == 0)
    // (the trip count is the same for every lane of a warp: the shuffles below need all of them)
    for (int base0 = aligned; base0 <= last; base0 += GROUPS * AD_U) {
        const int base = base0 + grp * AD_U;
        const int page = base <= last ? bt[base / page_size] : 0;
        const size_t row0 = (((size_t)page * nkv + hk) * page_size + (base % page_size)) * D + sub * 8;
        // all loads of the stretch are issued before anything is computed: 2 * AD_U 16-byte loads
        // in flight per thread, kept as raw bits until they are used
        uint4 kraw[AD_U], vraw[AD_U];
        bool ok[AD_U];
#pragma unroll
        for (int u = 0; u < AD_U; u++) {
            ok[u] = (base + u >= first) && (base + u <= last);
            kraw[u] = make_uint4(0u, 0u, 0u, 0u);
            vraw[u] = make_uint4(0u, 0u, 0u, 0u);
            if (ok[u]) {
                kraw[u] = ld_stream16(kc + row0 + (size_t)u * D);
                vraw[u] = ld_stream16(vc + row0 + (size_t)u * D);
            }
        }
        float s[G][AD_U];
#pragma unroll
        for (int u = 0; u < AD_U; u++) {
            float kf[8];
            unpack8(kraw[u], kf);
#pragma unroll
            for (int g = 0; g < G; g++) {
                float d = 0.f;
#pragma unroll
                for (int i = 0; i < 8; i++) d = fmaf(qr[g][i], kf[i], d);
#pragma unroll
                for (int o = LPK / 2; o > 0; o >>= 1) d += __shfl_xor_sync(0xffffffffu, d, o);
                s[g][u] = ok[u] ? d * scale_log2e : -INFINITY;
            }
        }
        float pe[G][AD_U];
#pragma unroll
        for (int g = 0; g < G; g++) {
            float mn = m[g];
#pragma unroll
            for (int u = 0; u < AD_U; u++) mn = fmaxf(mn, s[g][u]);
            const float mu = (mn == -INFINITY) ? 0.f : mn;      // nothing valid yet: all weights 0
            const float corr = exp2f(m[g] - mu);                // m = -inf gives 0
            float ps = 0.f;
#pragma unroll
            for (int u = 0; u < AD_U; u++) {
                pe[g][u] = exp2f(s[g][u] - mu);
                ps += pe[g][u];
            }
            l[g] = l[g] * corr + ps;
#pragma unroll
            for (int i = 0; i < 8; i++) acc[g][i] *= corr;
            m[g] = mn;
        }
#pragma unroll
        for (int u = 0; u < AD_U; u++) {
            float vf[8];
            unpack8(vraw[u], vf);
#pragma unroll
            for (int g = 0; g < G; g++)
#pragma unroll
                for (int i = 0; i < 8; i++) acc[g][i] = fmaf(pe[g][u], vf[i], acc[g][i]);
        }
    }

    // merge the lane groups of the block, in ascending order of group, through shared memory
    __shared__ float sm_m[GROUPS][G], sm_l[GROUPS][G];
    __shared__ float sm_acc[GROUPS][G][D];
#pragma unroll
    for (int g = 0; g < G; g++) {
        if (sub == 0) {
            sm_m[grp][g] = m[g];
            sm_l[grp][g] = l[g];
        }
#pragma unroll
        for (int i = 0; i < 8; i++) sm_acc[grp][g][sub * 8 + i] = acc[g][i];
    }
    __syncthreads();
    for (int idx = tid; idx < G * D; idx += AD_THREADS) {
        const int g = idx / D, c = idx - g * D;
        float M = -INFINITY;
#pragma unroll
        for (int r = 0; r < GROUPS; r++) M = fmaxf(M, sm_m[r][g]);
        float num = 0.f, den = 0.f;
#pragma unroll
        for (int r = 0; r < GROUPS; r++) {
            const float w = (sm_m[r][g] == -INFINITY) ? 0.f : exp2f(sm_m[r][g] - M);
            num += sm_acc[r][g][c] * w;
            den += sm_l[r][g] * w;
        }
        const size_t o = ((size_t)t * nh + hk * G + g) * n_chunks + chunk;
        part_acc[o * D + c] = num;
        if (c == 0) {
            part_ml[o * 2] = M;
            part_ml[o * 2 + 1] = den;
        }
    }
}

template <int D>
__global__ void attention_decode_merge_kernel(const float* __restrict__ part_acc,
                                              const float* __restrict__ part_ml,
                                              const int* __restrict__ token_pos, bf16* __restrict__ out,
                                              int n_chunks, int nh, int window, int chunk_keys) {
    pdl_grid_sync();
    const int h = blockIdx.x, t = blockIdx.y, c = threadIdx.x;
    const int p = token_pos[t];
    const int lo = (window > 0 && p - window + 1 > 0) ? p - window + 1 : 0;
    const int cfirst = lo / chunk_keys;
    int clast = p / chunk_keys;
    if (clast >= n_chunks) {
        // a position beyond what the caller sized the partial results for (token_pos < max_len is the
        // contract): the keys behind chunk n_chunks - 1 were never looked at, so the row is marked
        // as not a number instead of read from another head's partial results
        out[((size_t)t * nh + h) * D + c] = __float2bfloat16_rn(NAN);
        return;
    }
    const size_t o = ((size_t)t * nh + h) * n_chunks;
    float M = -INFINITY;
    for (int ch = cfirst; ch <= clast; ch++) M = fmaxf(M, part_ml[(o + ch) * 2]);
    float num = 0.f, den = 0.f;
    for (int ch = cfirst; ch <= clast; ch++) {
        const float w = exp2f(part_ml[(o + ch) * 2] - M);
        den += part_ml[(o + ch) * 2 + 1] * w;
        num += part_acc[(o + ch) * D + c] * w;
    }
    out[((size_t)t * nh + h) * D + c] = __float2bfloat16_rn(num / den);
}

template <int D, int G>
static int launch(const void* q, int q_stride, const void* kc, const void* vc, const int* block_table,
                  int max_pages, const int* token_pos, const int* token_seq, float* part_acc,
                  float* part_ml, void* out, int T, int nh, int nkv, int page_size, int window,
                  float scale, int n_chunks, cudaStream_t s) {
    dim3 grid(n_chunks, nkv, T);
    illm_launch(attention_decode_kernel<D, G>, dim3(grid), dim3(AD_THREADS), 0, s, 
        (const bf16*)q, q_stride, (const bf16*)kc, (const bf16*)vc, block_table, max_pages, token_pos,
        token_seq, part_acc, part_ml, n_chunks, nh, nkv, page_size, window, scale * 1.4426950408889634f);
    illm_launch(attention_decode_merge_kernel<D>, dim3(dim3(nh, T)), dim3(D), 0, s, part_acc, part_ml, token_pos, (bf16*)out,
                                                             n_chunks, nh, window, AD_CHUNK);
    return illm_launch_status();
}

// Scratch: part_acc float [T, nh, n_chunks, D], part_ml float [T, nh, n_chunks, 2], with
// n_chunks = ceil(max_len / 256) for the longest sequence the launch may meet.
extern "C" int illm_attention_decode(const void* q, int q_stride, const void* kc, const void* vc,
                                     const int* block_table, int max_pages, const int* token_pos,
                                     const int* token_seq, float* part_acc, float* part_ml, void* out,
                                     int T, int nh, int nkv, int d, int page_size, int window,
                                     float scale, int n_chunks, void* stream) {
    if (T <= 0) return 0;
    if (nkv <= 0 || nh % nkv || page_size % AD_U || T > 65535 || nkv > 65535 || d <= 0 || n_chunks <= 0)
        return ILLM_ERR_BAD_ARG;
    // the kernel reads q, the pages and writes out 16 bytes at a time
    if ((q_stride & 7) || ((uintptr_t)q & 15) || ((uintptr_t)kc & 15) || ((uintptr_t)vc & 15) || ((uintptr_t)out & 15))
        return ILLM_ERR_BAD_ARG;
    cudaStream_t s = (cudaStream_t)stream;
    const int g = nh / nkv;
#define AD_CASE(DD, GG)                                                                            \
    if (d == DD && g == GG)                                                                        \
        return launch<DD, GG>(q, q_stride, kc, vc, block_table, max_pages, token_pos, token_seq,  \
                              part_acc, part_ml, out, T, nh, nkv, page_size, window, scale, n_chunks, s);
    AD_CASE(128, 1) AD_CASE(128, 2) AD_CASE(128, 4) AD_CASE(128, 8)
    AD_CASE(64, 1) AD_CASE(64, 2) AD_CASE(64, 3) AD_CASE(64, 4) AD_CASE(64, 8)
#undef AD_CASE
    return ILLM_ERR_BAD_ARG;
}

// The merge alone, for kernels that write the same partial layout with chunks of another size
// (attention_decode_gqa.cu).
extern "C" int illm_attention_decode_merge(const float* part_acc, const float* part_ml, const int* token_pos,
                                           void* out, int T, int nh, int d, int n_chunks, int chunk_keys, int window,
                                           void* stream) {
    if (T <= 0) return 0;
    cudaStream_t s = (cudaStream_t)stream;
    if (d == 128)
        illm_launch(attention_decode_merge_kernel<128>, dim3(nh, T), dim3(128), 0, s, part_acc, part_ml, token_pos,
                    (bf16*)out, n_chunks, nh, window, chunk_keys);
    else if (d == 64)
        illm_launch(attention_decode_merge_kernel<64>, dim3(nh, T), dim3(64), 0, s, part_acc, part_ml, token_pos,
                    (bf16*)out, n_chunks, nh, window, chunk_keys);
    else
        return ILLM_ERR_BAD_ARG;
    return illm_launch_status();
}

extern "C" int illm_attention_decode_supported(int d, int g, int page_size) {
    if (page_size % AD_U) return 0;
    if (d == 128) return g == 1 || g == 2 || g == 4 || g == 8;
    if (d == 64) return g == 1 || g == 2 || g == 3 || g == 4 || g == 8;
    return 0;
}

// ---- the entry point that allocates nothing (declared and described in no_alloc.h)

#include <stdio.h>

#include <mutex>

#include "no_alloc.h"

// Scratch of the static entry point: lives in the device image of this library on every GPU that
// loads it.  In host code this name is only a handle for cudaGetSymbolAddress, not an address.
static __device__ __align__(256) float g_static_scratch[ILLM_STATIC_SCRATCH_BYTES / sizeof(float)];

#define ILLM_MAX_DEVICES 64
static float* g_static_scratch_addr[ILLM_MAX_DEVICES];  // per device, filled at its first call
static std::mutex g_static_scratch_mutex;

static int static_scratch_for_current_device(float** ptr) {
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return (int)e;
    if (dev < 0 || dev >= ILLM_MAX_DEVICES) return ILLM_ERR_BAD_ARG;
    std::lock_guard<std::mutex> lock(g_static_scratch_mutex);
    if (g_static_scratch_addr[dev] == nullptr) {
        void* p = nullptr;
        e = cudaGetSymbolAddress(&p, g_static_scratch);   // the address on the current device
        if (e != cudaSuccess) return (int)e;
        g_static_scratch_addr[dev] = (float*)p;
    }
    *ptr = g_static_scratch_addr[dev];
    return 0;
}

extern "C" int illm_attention_decode_static(const void* q, int q_stride, const void* kc, const void* vc,
                                            const int* block_table, int max_pages, const int* token_pos,
                                            const int* token_seq, void* out, int T, int nh, int nkv, int d,
                                            int page_size, int window, float scale, int max_len,
                                            char* err_msg, int err_len, void* stream) {
    if (err_msg && err_len > 0) err_msg[0] = 0;
    if (T <= 0) return 0;
    if (max_len <= 0 || nh <= 0 || d <= 0) return ILLM_ERR_BAD_ARG;
    const long long n_chunks = (max_len + AD_CHUNK - 1) / AD_CHUNK;
    const long long need = (long long)T * nh * n_chunks * (d + 2) * (long long)sizeof(float);
    if (need > (long long)ILLM_STATIC_SCRATCH_BYTES) {
        if (err_msg && err_len > 0)
            snprintf(err_msg, (size_t)err_len,
                     "illm_attention_decode_static: %d tokens x %d heads x %lld chunks of keys need %lld "
                     "bytes of scratch, the built-in array holds %u; split the call or use "
                     "illm_attention_decode with scratch of your own",
                     T, nh, n_chunks, need, (unsigned)ILLM_STATIC_SCRATCH_BYTES);
        return ILLM_ERR_SCRATCH_TOO_SMALL;
    }
    float* scratch = nullptr;
    int rc = static_scratch_for_current_device(&scratch);
    if (rc != 0) return rc;
    float* part_acc = scratch;
    float* part_ml = scratch + (size_t)T * nh * n_chunks * d;
    return illm_attention_decode(q, q_stride, kc, vc, block_table, max_pages, token_pos, token_seq,
                                 part_acc, part_ml, out, T, nh, nkv, d, page_size, window, scale,
                                 (int)n_chunks, stream);
}
