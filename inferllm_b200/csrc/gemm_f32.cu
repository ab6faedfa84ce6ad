// True float32 matrix product C[M, N] = A[M, K] . W[N, K]^T with float32 FMA accumulation:
// the contraction of the float32 mode.  No tensor cores, no TF32, no split of K: every
// element of C is one thread's sum over k in ascending order, so a row of C is bit-identical
// whatever M is and wherever the row lies.  That makes the float32 mode show faults of the
// cache or the batching that rounding would otherwise excuse.
// The reference calls cublasSgemm here (src/kern/gpu/kernel_gpu.cu:420-435), formula
// src/kern/naive/naive.cpp:363-379 (weight row-major [out, in], no bias).
// 64x64 tile of C per block, 16-wide slices of K through shared memory, 4x4 outputs a thread.
#include "tc_common.cuh"

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

// The same product for at most 8 rows (single tokens of a few sequences), where the tile kernel above
// leaves most of the GPU idle (N / 64 blocks that each wait for one 16-wide slice of K at a time).
// One warp per 32 outputs of a row: the warp streams its [32, K] slab of W through a ring of
// shared-memory stages of 128 values of k, each fetched as four TMA boxes of [32 rows x 32 floats]
// (128-byte rows, 128-byte swizzle) plus one box [MR x 128] of the activations, completion counted
// on the stage's mbarrier; rows past N and columns past K arrive as zeros.  (Earlier forms, with
// 16-byte cp.async or one 512-byte bulk copy per row, reached a quarter of the memory rate: the
// first is bounded by the load/store unit's miss queue, the second by the copy unit's rate of
// requests.)  Every lane owns one output column, whose sum it forms over k in ascending order with
// one fused multiply-add per k, starting from zero: the chain of the tile kernel, so the result is
// the same bits.  A lane reads its own row of a box, 16 bytes at a time, at the swizzled place
// (chunk c of row r lies at chunk c ^ (r & 7)): eight lanes then touch all 32 banks once.  The
// weights are requested before the wait for the kernels ahead (they are nobody's result), the
// activations after it.  The waits are bounded like those of the tensor-core kernels.
#define GS_STAGES(MR) ((MR) > 4 ? 5 : 6)             // two blocks per SM: at most 113 KB each
#define GS_KT 128                                   // values of k per stage
#define GS_W_BYTES (32 * GS_KT * 4)                 // 16 KB: four boxes of 4 KB
#define GS_SMEM(MR) (GS_STAGES(MR) * (GS_W_BYTES + (MR) * GS_KT * 4) + 1024)

template <int MR>
__global__ void __launch_bounds__(32)
gemm_f32_small_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_a,
                      float* __restrict__ C, int M, int N, int K, int ldc, int* __restrict__ err) {
    constexpr int S = GS_STAGES(MR);
    extern __shared__ unsigned char gs_raw[];
    __shared__ __align__(8) unsigned long long gs_full[S];
    constexpr unsigned X_BYTES = MR * GS_KT * 4, STAGE_TX = GS_W_BYTES + X_BYTES;
    const unsigned w_base = (tc_smem_u32(gs_raw) + 1023u) & ~1023u, x_base = w_base + S * GS_W_BYTES;
    const unsigned char* w_gen = gs_raw + (w_base - tc_smem_u32(gs_raw));
    const int lane = threadIdx.x, n0 = blockIdx.x * 32;
    const int n_tiles = (K + GS_KT - 1) / GS_KT;
    if (lane == 0) {
        for (int s = 0; s < S; s++) mbar_init(tc_smem_u32(&gs_full[s]), 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    __syncwarp();
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    auto issue_w = [&](int t) {
        const int s = t % S;
        const unsigned bar = tc_smem_u32(&gs_full[s]);
        mbar_expect_tx(bar, STAGE_TX);
#pragma unroll
        for (int q = 0; q < 4; q++) tma_load_2d(w_base + s * GS_W_BYTES + q * 4096, &map_w, t * GS_KT + q * 32, n0, bar);
    };
    auto issue_x = [&](int t) {
        const int s = t % S;
        tma_load_2d(x_base + s * X_BYTES, &map_a, t * GS_KT, 0, tc_smem_u32(&gs_full[s]));
    };
    const int n_pre = n_tiles < S - 1 ? n_tiles : S - 1;
    if (lane == 0)
        for (int t = 0; t < n_pre; t++) issue_w(t);
    asm volatile("griddepcontrol.wait;" ::: "memory");
    if (lane == 0)
        for (int t = 0; t < n_pre; t++) issue_x(t);
    float acc[MR];
#pragma unroll
    for (int m = 0; m < MR; m++) acc[m] = 0.f;
    bool alive = true;
    int t = 0;
    for (; t < n_tiles; t++) {
        // the stage that was read in the round before is free (the __syncwarp below)
        if (lane == 0 && t + S - 1 < n_tiles) {
            issue_w(t + S - 1);
            issue_x(t + S - 1);
        }
        alive = __all_sync(0xffffffffu, mbar_wait(tc_smem_u32(&gs_full[t % S]), (t / S) & 1, err));
        if (!alive) break;
        const unsigned char* wst = w_gen + (size_t)(t % S) * GS_W_BYTES + lane * 128;
        const float* xs = reinterpret_cast<const float*>(w_gen + (size_t)S * GS_W_BYTES + (size_t)(t % S) * X_BYTES);
#pragma unroll
        for (int q = 0; q < 4; q++) {
#pragma unroll
            for (int c = 0; c < 8; c++) {
                const float4 w = *reinterpret_cast<const float4*>(wst + q * 4096 + ((c ^ (lane & 7)) << 4));
#pragma unroll
                for (int m = 0; m < MR; m++) {
                    const float4 x = *reinterpret_cast<const float4*>(xs + m * GS_KT + q * 32 + c * 4);
                    acc[m] = fmaf(x.x, w.x, acc[m]);
                    acc[m] = fmaf(x.y, w.y, acc[m]);
                    acc[m] = fmaf(x.z, w.z, acc[m]);
                    acc[m] = fmaf(x.w, w.w, acc[m]);
                }
            }
        }
        __syncwarp();      // the stage is refilled by the next round's requests
    }
    if (!alive) {
        // a wait ran out (the error word is set): no result; the copies still in flight are waited
        // for, each with a short limit, before the block gives its shared memory back
        for (int u = t + 1; u < n_tiles && u < t + S; u++)
            mbar_wait(tc_smem_u32(&gs_full[u % S]), (u / S) & 1, err, TC_ERR_TIMEOUT, 1LL << 24);
        return;
    }
    const int n = n0 + lane;
    if (n < N) {
#pragma unroll
        for (int m = 0; m < MR; m++)
            if (m < M) C[(size_t)m * ldc + n] = acc[m];
    }
}

typedef CUresult (*GsEncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                    const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                    CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// Tensor map of a row-major float32 matrix [rows, K] with row stride ld; boxes of [box_rows, box_k].
static int gs_make_map(CUtensorMap* map, const float* ptr, long long rows, long long K, long long ld, int box_rows, int box_k,
                       CUtensorMapSwizzle swizzle) {
    static GsEncodeTiledFn fn = nullptr;
    if (!fn) {
        void* q = nullptr;
        cudaDriverEntryPointQueryResult r;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &q, cudaEnableDefault, &r) != cudaSuccess ||
            r != cudaDriverEntryPointSuccess)
            return ILLM_ERR_BAD_ARG;
        fn = (GsEncodeTiledFn)q;
    }
    cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)ld * 4};
    cuuint32_t box[2] = {(cuuint32_t)box_k, (cuuint32_t)box_rows};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, const_cast<float*>(ptr), dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? 0 : ILLM_ERR_BAD_ARG;
}

template <int MR>
static int launch_gemm_f32_small(const float* A, const float* W, float* C, int M, int N, int K, int lda, int ldw, int ldc,
                                 int* err, cudaStream_t s) {
    CUtensorMap mw, ma;
    int rc;
    if ((rc = gs_make_map(&mw, W, N, K, ldw, 32, 32, CU_TENSOR_MAP_SWIZZLE_128B)) != 0) return rc;
    if ((rc = gs_make_map(&ma, A, M, K, lda, MR, GS_KT, CU_TENSOR_MAP_SWIZZLE_NONE)) != 0) return rc;
    auto kern = gemm_f32_small_kernel<MR>;
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, GS_SMEM(MR));
    if (e != cudaSuccess) return (int)e;
    illm_launch(kern, dim3((N + 31) / 32), dim3(32), (size_t)GS_SMEM(MR), s, mw, ma, C, M, N, K, ldc, err);
    return illm_launch_status();
}

// err: the device's error word for the bounded waits of the few-rows kernel (null: that kernel is
// not used and every size takes the tile kernel).
extern "C" int illm_gemm_f32_nt(const float* A, const float* W, float* C, int M, int N, int K,
                                int lda, int ldw, int ldc, int* err, void* stream) {
    if (M <= 0 || N <= 0) return 0;
    if (K <= 0) return ILLM_ERR_BAD_ARG;
    if (err != nullptr && M <= 8 && (K & 3) == 0 && (lda & 3) == 0 && (ldw & 3) == 0 &&
        ((reinterpret_cast<uintptr_t>(A) | reinterpret_cast<uintptr_t>(W)) & 15) == 0) {
        cudaStream_t s = (cudaStream_t)stream;
        if (M == 1) return launch_gemm_f32_small<1>(A, W, C, M, N, K, lda, ldw, ldc, err, s);
        if (M == 2) return launch_gemm_f32_small<2>(A, W, C, M, N, K, lda, ldw, ldc, err, s);
        if (M <= 4) return launch_gemm_f32_small<4>(A, W, C, M, N, K, lda, ldw, ldc, err, s);
        return launch_gemm_f32_small<8>(A, W, C, M, N, K, lda, ldw, ldc, err, s);
    }
    dim3 grid((N + GF_BN - 1) / GF_BN, (M + GF_BM - 1) / GF_BM);
    if (grid.y > 65535) return ILLM_ERR_BAD_ARG;
    illm_launch(gemm_f32_nt_kernel, dim3(grid), dim3(256), 0, (cudaStream_t)stream, A, W, C, M, N, K, lda, ldw, ldc);
    return illm_launch_status();
}
