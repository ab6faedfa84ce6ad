// True float32 matrix product C[M, N] = A[M, K] . W[N, K]^T with float32 FMA accumulation:
// the contraction of the float32 mode.  No tensor cores, no TF32, no split of K: every
// element of C is one thread's sum over k in ascending order, so a row of C is bit-identical
// whatever M is and wherever the row lies.  That makes the float32 mode show faults of the
// cache or the batching that rounding would otherwise excuse.
// The reference calls cublasSgemm here (src/kern/gpu/kernel_gpu.cu:420-435), formula
// src/kern/naive/naive.cpp:363-379 (weight row-major [out, in], no bias).
// 64x64 tile of C per block, 16-wide slices of K through shared memory, 4x4 outputs a thread.
#include "common.cuh"

#define GF_BM 64
#define GF_BN 64
#define GF_BK 16

__global__ void __launch_bounds__(256)
gemm_f32_nt_kernel(const float* __restrict__ A, const float* __restrict__ W, float* __restrict__ C,
                   int M, int N, int K, int lda, int ldw, int ldc) {
    pdl_grid_sync();
    __shared__ __align__(16) float As[GF_BK][GF_BM + 4];
    __shared__ __align__(16) float Ws[GF_BK][GF_BN + 4];
    const int tid = threadIdx.x;
    const int m0 = blockIdx.y * GF_BM, n0 = blockIdx.x * GF_BN;
    const int lr = tid >> 2, lk = (tid & 3) * 4;  // loader: row within the tile, k offset
    const int ty = tid >> 4, tx = tid & 15;
    const bool vec = ((K & 3) == 0) && ((lda & 3) == 0) && ((ldw & 3) == 0) &&
                     ((reinterpret_cast<uintptr_t>(A) | reinterpret_cast<uintptr_t>(W)) & 15) == 0;
    float acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; i++)
#pragma unroll
        for (int j = 0; j < 4; j++) acc[i][j] = 0.f;

    for (int k0 = 0; k0 < K; k0 += GF_BK) {
        float a[4] = {0.f, 0.f, 0.f, 0.f}, w[4] = {0.f, 0.f, 0.f, 0.f};
        const int k = k0 + lk;
        if (m0 + lr < M) {
            const float* src = A + (size_t)(m0 + lr) * lda + k;
            if (vec && k + 3 < K) {
                float4 v = *reinterpret_cast<const float4*>(src);
                a[0] = v.x; a[1] = v.y; a[2] = v.z; a[3] = v.w;
            } else {
#pragma unroll
                for (int i = 0; i < 4; i++)
                    if (k + i < K) a[i] = src[i];
            }
        }
        if (n0 + lr < N) {
            const float* src = W + (size_t)(n0 + lr) * ldw + k;
            if (vec && k + 3 < K) {
                float4 v = *reinterpret_cast<const float4*>(src);
                w[0] = v.x; w[1] = v.y; w[2] = v.z; w[3] = v.w;
            } else {
#pragma unroll
                for (int i = 0; i < 4; i++)
                    if (k + i < K) w[i] = src[i];
            }
        }
        __syncthreads();
#pragma unroll
        for (int i = 0; i < 4; i++) {
            As[lk + i][lr] = a[i];
            Ws[lk + i][lr] = w[i];
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < GF_BK; kk++) {
            const float4 av = *reinterpret_cast<const float4*>(&As[kk][ty * 4]);
            const float4 wv = *reinterpret_cast<const float4*>(&Ws[kk][tx * 4]);
            const float ar[4] = {av.x, av.y, av.z, av.w};
            const float wr[4] = {wv.x, wv.y, wv.z, wv.w};
#pragma unroll
            for (int i = 0; i < 4; i++)
#pragma unroll
                for (int j = 0; j < 4; j++) acc[i][j] = fmaf(ar[i], wr[j], acc[i][j]);
        }
    }
#pragma unroll
    for (int i = 0; i < 4; i++) {
        const int m = m0 + ty * 4 + i;
        if (m >= M) continue;
#pragma unroll
        for (int j = 0; j < 4; j++) {
            const int n = n0 + tx * 4 + j;
            if (n < N) C[(size_t)m * ldc + n] = acc[i][j];
        }
    }
}

extern "C" int illm_gemm_f32_nt(const float* A, const float* W, float* C, int M, int N, int K,
                                int lda, int ldw, int ldc, void* stream) {
    if (M <= 0 || N <= 0) return 0;
    if (K <= 0) return ILLM_ERR_BAD_ARG;
    dim3 grid((N + GF_BN - 1) / GF_BN, (M + GF_BM - 1) / GF_BM);
    if (grid.y > 65535) return ILLM_ERR_BAD_ARG;
    illm_launch(gemm_f32_nt_kernel, dim3(grid), dim3(256), 0, (cudaStream_t)stream, A, W, C, M, N, K, lda, ldw, ldc);
    return illm_launch_status();
}
