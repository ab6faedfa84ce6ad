// Causal attention of every token of a step over the paged cache: the generic kernel.
//
// It takes any head size that is a multiple of 8 up to 256, any number of heads and groups,
// any page size, float32 or bfloat16 storage, prompts and single tokens alike, and does all
// arithmetic in float32.  It is the whole attention of the float32 mode and the fall-back of
// the bfloat16 mode for head sizes that the tensor-core kernels do not take.
//
// The reference materialises the score matrix and runs four launches over it: a batched
// product Q K^T (src/kern/gpu/kernel_gpu.cu:576-591), scale + causal mask (:504-536), a
// three-pass row softmax (:78-125) and the batched product with V (:593-609); formulas
// src/kern/naive/naive.cpp:606-632, :531-553, :209-240, :664-691, grouped heads :576-604.
// Here one block owns one (token, head): its sixteen warps walk the keys lo..p in blocks of 32
// (a key per lane for the scores, a channel per lane for the values) with a running maximum
// and sum, and are merged in a fixed order.  The split of the keys depends only on the
// token's own position and window, so its result does not depend on the step it is part of.
//   score = (q . k) * scale;  keys lo..p with lo = max(0, p - window + 1) (window 0 = all)
#include <math.h>

#include "common.cuh"

#define AG_WARPS 16
#define AG_MAX_D 256

template <typename TA>
__global__ void __launch_bounds__(AG_WARPS * 32)
attention_generic_kernel(const TA* __restrict__ q, int q_stride, const TA* __restrict__ kc,
                         const TA* __restrict__ vc, const int* __restrict__ block_table,
                         int max_pages, const int* __restrict__ token_pos,
                         const int* __restrict__ token_seq, TA* __restrict__ out, int nh, int nkv,
                         int d, int page_size, int window, float scale) {
    pdl_grid_sync();
    extern __shared__ float smem[];
    float* qs = smem;                 // [d]
    float* acc_s = smem + d;          // [AG_WARPS][d]
    __shared__ float m_s[AG_WARPS], l_s[AG_WARPS];

    const int t = blockIdx.x, h = blockIdx.y;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int hk = h / (nh / nkv);
    const int p = token_pos[t];
    const int lo = (window > 0 && p - window + 1 > 0) ? p - window + 1 : 0;
    const int* bt = block_table + (size_t)token_seq[t] * max_pages;

    const TA* qrow = q + (size_t)t * q_stride + (size_t)h * d;
    for (int c = threadIdx.x; c < d; c += blockDim.x) qs[c] = to_f32(qrow[c]);
    __syncthreads();

    float m = -INFINITY, l = 0.f;
    float acc[AG_MAX_D / 32];
#pragma unroll
    for (int i = 0; i < AG_MAX_D / 32; i++) acc[i] = 0.f;

    for (int kb = lo + warp * 32; kb <= p; kb += AG_WARPS * 32) {
        const int key = kb + lane;
        const bool valid = key <= p;
        float s = -INFINITY;
        long long off = 0;
        if (valid) {
            const int page = bt[key / page_size];
            off = (((long long)page * nkv + hk) * page_size + (key % page_size)) * d;
            const TA* kr = kc + off;
            float dot = 0.f;
#pragma unroll 4
            for (int c = 0; c < d; c += 8) {
                float f[8];
                load8(kr + c, f);
#pragma unroll
                for (int i = 0; i < 8; i++) dot = fmaf(qs[c + i], f[i], dot);
            }
            s = dot * scale;
        }
        const float m_new = fmaxf(m, warp_max(s));
        const float pe = valid ? expf(s - m_new) : 0.f;
        const float corr = (m == -INFINITY) ? 0.f : expf(m - m_new);
        l = l * corr + warp_sum(pe);
#pragma unroll
        for (int i = 0; i < AG_MAX_D / 32; i++) acc[i] *= corr;
        const int nk = (p - kb + 1 < 32) ? p - kb + 1 : 32;
#pragma unroll 4
        for (int j = 0; j < nk; j++) {
            const float pj = __shfl_sync(0xffffffffu, pe, j);
            const long long oj = __shfl_sync(0xffffffffu, off, j);
            const TA* vr = vc + oj;
#pragma unroll
            for (int i = 0; i < AG_MAX_D / 32; i++) {
                const int c = lane + 32 * i;
                if (c < d) acc[i] = fmaf(pj, to_f32(vr[c]), acc[i]);
            }
        }
        m = m_new;
    }

    if (lane == 0) {
        m_s[warp] = m;
        l_s[warp] = l;
    }
#pragma unroll
    for (int i = 0; i < AG_MAX_D / 32; i++) {
        const int c = lane + 32 * i;
        if (c < d) acc_s[warp * d + c] = acc[i];
    }
    __syncthreads();
    float M = m_s[0];
#pragma unroll
    for (int w = 1; w < AG_WARPS; w++) M = fmaxf(M, m_s[w]);
    float wgt[AG_WARPS], den = 0.f;
#pragma unroll
    for (int w = 0; w < AG_WARPS; w++) {
        wgt[w] = (m_s[w] == -INFINITY) ? 0.f : expf(m_s[w] - M);
        den += l_s[w] * wgt[w];
    }
    const float inv = 1.0f / den;
    TA* o = out + ((size_t)t * nh + h) * d;
    for (int c = threadIdx.x; c < d; c += blockDim.x) {
        float num = 0.f;
#pragma unroll
        for (int w = 0; w < AG_WARPS; w++) num += acc_s[w * d + c] * wgt[w];
        o[c] = from_f32<TA>(num * inv);
    }
}

extern "C" int illm_attention_generic(const void* q, int q_stride, const void* kc, const void* vc,
                                      const int* block_table, int max_pages, const int* token_pos,
                                      const int* token_seq, void* out, int act_dtype, int T, int nh,
                                      int nkv, int d, int page_size, int window, float scale,
                                      void* stream) {
    if (T <= 0) return 0;
    if (d <= 0 || d > AG_MAX_D || (d & 7) || nkv <= 0 || nh % nkv || nh > 65535) return ILLM_ERR_BAD_ARG;
    cudaStream_t s = (cudaStream_t)stream;
    dim3 grid(T, nh);
    size_t smem = (size_t)(1 + AG_WARPS) * d * sizeof(float);
    if (act_dtype == ILLM_BF16)
        illm_launch(attention_generic_kernel<bf16>, dim3(grid), dim3(AG_WARPS * 32), smem, s, 
            (const bf16*)q, q_stride, (const bf16*)kc, (const bf16*)vc, block_table, max_pages,
            token_pos, token_seq, (bf16*)out, nh, nkv, d, page_size, window, scale);
    else if (act_dtype == ILLM_F32)
        illm_launch(attention_generic_kernel<float>, dim3(grid), dim3(AG_WARPS * 32), smem, s, 
            (const float*)q, q_stride, (const float*)kc, (const float*)vc, block_table, max_pages,
            token_pos, token_seq, (float*)out, nh, nkv, d, page_size, window, scale);
    else
        return ILLM_ERR_BAD_ARG;
    return illm_launch_status();
}
