// Attention of single tokens over long paged caches for grouped heads (several query heads per
// KV head), bfloat16.
//
// With G query heads sharing a KV head, the SIMT kernel of attention_decode.cu spends most of its
// time on the G dot products per key and their cross-lane sums, and falls far below the memory
// rate (2.4 TB/s at G = 4).  Here the G heads of one token become the rows of a 16-row MMA tile
// (rows beyond G are zero), so one warp-level MMA (m16n8k16) does all of them at once and the
// kernel is bound by reading K and V again.  A block of 4 warps owns one (token, kv head, chunk of
// 128 keys): each warp brings its 32 keys and values into shared memory with cp.async (16-byte
// chunks, XOR-swizzled rows), computes S = Q K^T, the softmax weights in float32, and P V, all for
// its 32 keys; the four warps are merged through shared memory and the partial result goes to the
// same scratch layout as the SIMT kernel's, [token, head, chunk], which the merge kernel of
// attention_decode.cu adds up in ascending order of the chunk.  Any group size up to 16.
// Formulas: src/kern/naive/naive.cpp:576-604 (scores with key head h / G), :531-553 (mask),
// :209-240 (softmax), :634-662 (values); the reference's GPU code loops over the G heads with one
// library call each (src/kern/gpu/kernel_gpu.cu:688-756).
#include <math.h>

#include "common.cuh"

#define GD_WARPS 4
#define GD_BN 32                       // keys per warp
#define GD_CHUNK (GD_WARPS * GD_BN)    // keys per block

namespace {

__device__ __forceinline__ unsigned gd_smem(const void* p) { return (unsigned)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void gd_cp16(unsigned dst, const void* src, int bytes) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(dst), "l"(src), "r"(bytes));
}
__device__ __forceinline__ void gd_ldm(unsigned& r0, unsigned& r1, unsigned& r2, unsigned& r3, unsigned addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void gd_ldm_t(unsigned& r0, unsigned& r1, unsigned& r2, unsigned& r3, unsigned addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void gd_mma(float* c, const unsigned* a, unsigned b0, unsigned b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ unsigned gd_pack(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<unsigned*>(&v);
}
template <int D> __device__ __forceinline__ int gd_swz(int r, int c) { return r * D + ((c ^ (r & 7)) << 3); }

}  // namespace

template <int D>
__global__ void __launch_bounds__(GD_WARPS * 32)
attention_decode_gqa_kernel(const bf16* __restrict__ q, int q_stride, const bf16* __restrict__ kc,
                            const bf16* __restrict__ vc, const int* __restrict__ block_table, int max_pages,
                            const int* __restrict__ token_pos, const int* __restrict__ token_seq,
                            float* __restrict__ part_acc, float* __restrict__ part_ml, int n_chunks, int nh,
                            int nkv, int G, int page_size, int window, float scale_log2e) {
    pdl_grid_sync();
    constexpr int CH = D / 8, KS = D / 16, NT_D = D / 8;
    extern __shared__ __align__(128) unsigned char smem_raw[];
    bf16* Qs = reinterpret_cast<bf16*>(smem_raw);            // [16][D]
    bf16* KVs = Qs + 16 * D;                                  // per warp: K [64][D], V [64][D]

    const int chunk = blockIdx.x, hk = blockIdx.y, t = blockIdx.z;
    const int p = token_pos[t];
    const int lo = (window > 0 && p - window + 1 > 0) ? p - window + 1 : 0;
    const int c0 = chunk * GD_CHUNK;
    if (c0 > p || c0 + GD_CHUNK <= lo) return;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int g = lane >> 2, t4 = lane & 3, mtx = lane >> 3;
    const int* bt = block_table + (size_t)token_seq[t] * max_pages;

    // ---- Q: the G heads of this kv head as rows 0..G-1, zero rows above
    for (int i = tid; i < 16 * CH; i += GD_WARPS * 32) {
        const int r = i / CH, c = i % CH;
        const bool ok = r < G;
        const bf16* src = ok ? q + (size_t)t * q_stride + (size_t)(hk * G + r) * D + c * 8 : q;
        gd_cp16(gd_smem(Qs + gd_swz<D>(r, c)), src, ok ? 16 : 0);
    }
    // ---- this warp's 64 keys and values (rows beyond the token's position are zero)
    const int key0 = c0 + warp * GD_BN;
    bf16* Kw = KVs + (size_t)warp * 2 * GD_BN * D;
    bf16* Vw = Kw + GD_BN * D;
    for (int i = lane; i < GD_BN * CH; i += 32) {
        const int r = i / CH, c = i % CH;
        const int key = key0 + r;
        const bool ok = key <= p && key >= lo;
        size_t off = 0;
        if (ok) {
            const int page = bt[key / page_size];
            off = (((size_t)page * nkv + hk) * page_size + (key % page_size)) * D + c * 8;
        }
        gd_cp16(gd_smem(Kw + gd_swz<D>(r, c)), kc + off, ok ? 16 : 0);
        gd_cp16(gd_smem(Vw + gd_swz<D>(r, c)), vc + off, ok ? 16 : 0);
    }
    asm volatile("cp.async.commit_group;\n" ::);
    asm volatile("cp.async.wait_group 0;\n" ::);
    __syncthreads();

    float m_w[2] = {-INFINITY, -INFINITY}, l_w[2] = {0.f, 0.f};
    float o[NT_D][4];
#pragma unroll
    for (int i = 0; i < NT_D; i++) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
    const bool warp_has_keys = key0 <= p && key0 + GD_BN > lo;
    if (warp_has_keys) {
        float s[GD_BN / 8][4];
#pragma unroll
        for (int i = 0; i < GD_BN / 8; i++) s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.f;
#pragma unroll
        for (int ks = 0; ks < KS; ks++) {
            unsigned qf[4];
            gd_ldm(qf[0], qf[1], qf[2], qf[3], gd_smem(Qs + gd_swz<D>((mtx & 1) * 8 + (lane & 7), ks * 2 + (mtx >> 1))));
#pragma unroll
            for (int np = 0; np < GD_BN / 16; np++) {
                const int r = np * 16 + (mtx >> 1) * 8 + (lane & 7);
                unsigned b0, b1, b2, b3;
                gd_ldm(b0, b1, b2, b3, gd_smem(Kw + gd_swz<D>(r, ks * 2 + (mtx & 1))));
                gd_mma(s[np * 2], qf, b0, b1);
                gd_mma(s[np * 2 + 1], qf, b2, b3);
            }
        }
        // scale, mask (only keys outside [lo, p] are hidden: one token, no causal triangle), max
        float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
        for (int nt = 0; nt < GD_BN / 8; nt++)
#pragma unroll
            for (int e = 0; e < 4; e++) {
                const int key = key0 + nt * 8 + t4 * 2 + (e & 1);
                const float v = (key > p || key < lo) ? -INFINITY : s[nt][e] * scale_log2e;
                s[nt][e] = v;
                mx[e >> 1] = fmaxf(mx[e >> 1], v);
            }
        unsigned pf[GD_BN / 16][4];
#pragma unroll
        for (int e = 0; e < 2; e++) {
            mx[e] = fmaxf(mx[e], __shfl_xor_sync(0xffffffffu, mx[e], 1));
            mx[e] = fmaxf(mx[e], __shfl_xor_sync(0xffffffffu, mx[e], 2));
            m_w[e] = mx[e];                       // finite: the warp has at least one valid key
        }
#pragma unroll
        for (int nt = 0; nt < GD_BN / 8; nt++) {
            const float p0 = fast_exp2(s[nt][0] - m_w[0]), p1 = fast_exp2(s[nt][1] - m_w[0]);
            const float p2 = fast_exp2(s[nt][2] - m_w[1]), p3 = fast_exp2(s[nt][3] - m_w[1]);
            l_w[0] += p0 + p1;
            l_w[1] += p2 + p3;
            pf[nt >> 1][(nt & 1) * 2] = gd_pack(p0, p1);
            pf[nt >> 1][(nt & 1) * 2 + 1] = gd_pack(p2, p3);
        }
#pragma unroll
        for (int e = 0; e < 2; e++) {
            l_w[e] += __shfl_xor_sync(0xffffffffu, l_w[e], 1);
            l_w[e] += __shfl_xor_sync(0xffffffffu, l_w[e], 2);
        }
#pragma unroll
        for (int ks = 0; ks < GD_BN / 16; ks++)
#pragma unroll
            for (int np = 0; np < NT_D / 2; np++) {
                const int r = ks * 16 + (mtx & 1) * 8 + (lane & 7);
                unsigned b0, b1, b2, b3;
                gd_ldm_t(b0, b1, b2, b3, gd_smem(Vw + gd_swz<D>(r, np * 2 + (mtx >> 1))));
                gd_mma(o[np * 2], pf[ks], b0, b1);
                gd_mma(o[np * 2 + 1], pf[ks], b2, b3);
            }
    }
    __syncthreads();     // all warps are done with their K/V tiles: the memory is reused for the merge

    // ---- merge the warps (ascending) and write the chunk's partial result for heads 0..G-1
    float* mrg = reinterpret_cast<float*>(KVs);              // [GD_WARPS][16][D + 2]
    constexpr int ROW = D + 2;
#pragma unroll
    for (int e = 0; e < 2; e++) {
        const int r = g + e * 8;
        float* dst = mrg + ((size_t)warp * 16 + r) * ROW;
#pragma unroll
        for (int i = 0; i < NT_D; i++) {
            dst[i * 8 + t4 * 2] = o[i][e * 2];
            dst[i * 8 + t4 * 2 + 1] = o[i][e * 2 + 1];
        }
        if (t4 == 0) {
            dst[D] = m_w[e];
            dst[D + 1] = l_w[e];
        }
    }
    __syncthreads();
    for (int idx = tid; idx < G * D; idx += GD_WARPS * 32) {
        const int r = idx / D, c = idx - r * D;
        float M = -INFINITY;
#pragma unroll
        for (int w = 0; w < GD_WARPS; w++) M = fmaxf(M, mrg[((size_t)w * 16 + r) * ROW + D]);
        float num = 0.f, den = 0.f;
#pragma unroll
        for (int w = 0; w < GD_WARPS; w++) {
            const float mw = mrg[((size_t)w * 16 + r) * ROW + D];
            const float wgt = (mw == -INFINITY) ? 0.f : fast_exp2(mw - M);
            num += mrg[((size_t)w * 16 + r) * ROW + c] * wgt;
            den += mrg[((size_t)w * 16 + r) * ROW + D + 1] * wgt;
        }
        const size_t oidx = ((size_t)t * nh + hk * G + r) * n_chunks + chunk;
        part_acc[oidx * D + c] = num;
        if (c == 0) {
            part_ml[oidx * 2] = M;
            part_ml[oidx * 2 + 1] = den;
        }
    }
}

// merges chunks of `chunk_keys` keys (the kernel of attention_decode.cu, with the chunk size as an
// argument); declared there
extern "C" int illm_attention_decode_merge(const float* part_acc, const float* part_ml, const int* token_pos,
                                           void* out, int T, int nh, int d, int n_chunks, int chunk_keys, int window,
                                           void* stream);

template <int D>
static int gd_launch(const void* q, int q_stride, const void* kc, const void* vc, const int* block_table,
                     int max_pages, const int* token_pos, const int* token_seq, float* part_acc, float* part_ml,
                     void* out, int T, int nh, int nkv, int page_size, int window, float scale, int n_chunks,
                     cudaStream_t s) {
    const size_t smem = (size_t)16 * D * 2 + (size_t)GD_WARPS * 2 * GD_BN * D * 2;
    auto kern = attention_decode_gqa_kernel<D>;
    if (smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
    }
    dim3 grid(n_chunks, nkv, T);
    illm_launch(kern, grid, dim3(GD_WARPS * 32), smem, s, (const bf16*)q, q_stride, (const bf16*)kc, (const bf16*)vc,
                block_table, max_pages, token_pos, token_seq, part_acc, part_ml, n_chunks, nh, nkv, nh / nkv, page_size,
                window, scale * 1.4426950408889634f);
    int rc = illm_launch_status();
    if (rc != 0) return rc;
    return illm_attention_decode_merge(part_acc, part_ml, token_pos, out, T, nh, D, n_chunks, GD_CHUNK, window, s);
}

// Scratch: part_acc float [T, nh, n_chunks, d], part_ml float [T, nh, n_chunks, 2] with
// n_chunks = ceil(max_len / 128).
extern "C" int illm_attention_decode_gqa(const void* q, int q_stride, const void* kc, const void* vc,
                                         const int* block_table, int max_pages, const int* token_pos,
                                         const int* token_seq, float* part_acc, float* part_ml, void* out, int T,
                                         int nh, int nkv, int d, int page_size, int window, float scale, int n_chunks,
                                         void* stream) {
    if (T <= 0) return 0;
    if (nkv <= 0 || nh % nkv || nh / nkv > 16 || T > 65535 || nkv > 65535 || (q_stride & 7)) return ILLM_ERR_BAD_ARG;
    cudaStream_t s = (cudaStream_t)stream;
    if (d == 128)
        return gd_launch<128>(q, q_stride, kc, vc, block_table, max_pages, token_pos, token_seq, part_acc, part_ml, out,
                              T, nh, nkv, page_size, window, scale, n_chunks, s);
    if (d == 64)
        return gd_launch<64>(q, q_stride, kc, vc, block_table, max_pages, token_pos, token_seq, part_acc, part_ml, out,
                             T, nh, nkv, page_size, window, scale, n_chunks, s);
    return ILLM_ERR_BAD_ARG;
}
