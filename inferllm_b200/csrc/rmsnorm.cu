// Residual add + RMSNorm in one pass over the row.
//
//   x = resid[r] (+ delta[r]);  resid[r] = x (if write_resid);
//   y[i] = (x * rsqrt(mean(x^2) + eps)) * w
//
// The reference runs three launches for this (the add src/kern/gpu/kernel_gpu.cu:183-258,
// the norm :260-294 with one warp per row, the weight multiply :33-75), formula
// src/kern/naive/naive.cpp:186-207.  The residual stream is float32 in every mode; the sum
// of squares, the scale and the product with the weight are float32 and y is rounded once.
// `rows` (optional) gathers: block i reads row rows[i] and writes output row i, which is how
// the final norm touches only the positions whose logits are wanted.
// One block per row; the row is kept in shared memory between the two passes, so H is
// bounded by the shared memory a block can have (checked on the host side of the call).
#include "common.cuh"

template <typename TA, typename TW>
__global__ void add_rmsnorm_kernel(float* __restrict__ resid, const TA* __restrict__ delta,
                                   const TW* __restrict__ w, TA* __restrict__ y,
                                   const int* __restrict__ rows, int H, float eps,
                                   int write_resid) {
    pdl_grid_sync();
    extern __shared__ float row[];
    __shared__ float scratch[32];
    const int r = rows ? rows[blockIdx.x] : blockIdx.x;
    float* x = resid + (size_t)r * H;
    const TA* dl = delta ? delta + (size_t)r * H : nullptr;
    float ss = 0.f;
    for (int c = threadIdx.x; c < H; c += blockDim.x) {
        float v = x[c];
        if (dl) v += to_f32(dl[c]);
        row[c] = v;
        ss += v * v;
    }
    if (dl && write_resid)
        for (int c = threadIdx.x; c < H; c += blockDim.x) x[c] = row[c];
    ss = block_sum(ss, scratch);
    const float scale = rsqrtf(ss / (float)H + eps);
    TA* o = y + (size_t)blockIdx.x * H;
    for (int c = threadIdx.x; c < H; c += blockDim.x)
        o[c] = from_f32<TA>((row[c] * scale) * to_f32(w[c]));
}

// Rows of up to 2 * 8 * 1024 elements (H a multiple of 8): the row stays in registers, 8
// elements per thread and iteration with 16-byte accesses; same arithmetic as above.  The block
// has one thread per 8 elements up to 1024 threads (a function of H alone: the order of the sums,
// and with it every bit of the result, is the same for one row and for thousands).
#define RN_MAX_THREADS 1024
template <typename TA, typename TW, int ITERS, int MAXT>
__global__ void __launch_bounds__(MAXT)
add_rmsnorm_reg_kernel(float* __restrict__ resid, const TA* __restrict__ delta, const TW* __restrict__ w,
                       TA* __restrict__ y, const int* __restrict__ rows, int H, float eps, int write_resid,
                       const float* __restrict__ partials, int splits, long long split_stride) {
    // the norm's weight is no result of the previous kernel: it is read while that kernel drains
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    float wv[ITERS][8];
#pragma unroll
    for (int i = 0; i < ITERS; i++) {
        const int c = (threadIdx.x + i * (int)blockDim.x) * 8;
        if (c < H) load8(w + c, wv[i]);
    }
    asm volatile("griddepcontrol.wait;" ::: "memory");
    __shared__ float scratch[32];
    const int r = rows ? rows[blockIdx.x] : blockIdx.x;
    float* x = resid + (size_t)r * H;
    const TA* dl = delta ? delta + (size_t)r * H : nullptr;
    float v[ITERS][8];
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < ITERS; i++) {
        const int c = (threadIdx.x + i * (int)blockDim.x) * 8;
        if (c < H) {
            load8(x + c, v[i]);
            if (dl) {
                float d8[8];
                load8(dl + c, d8);
#pragma unroll
                for (int k = 0; k < 8; k++) v[i][k] += d8[k];
                if (write_resid) store8(x + c, v[i]);
            } else if (partials) {
                // the addend is still in K slices (float32, from a split matrix product): they are
                // summed here, in ascending order, instead of by a kernel of their own
                float d8[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
                const float* pz = partials + (size_t)r * H + c;
                int z = 0;
                constexpr int FLY = MAXT <= 512 ? 8 : 4;   // slices in flight (registers allowing), added in order
                for (; z + FLY <= splits; z += FLY) {
                    float p8[FLY][8];
#pragma unroll
                    for (int q = 0; q < FLY; q++) load8(pz + (size_t)(z + q) * split_stride, p8[q]);
#pragma unroll
                    for (int q = 0; q < FLY; q++)
#pragma unroll
                        for (int k = 0; k < 8; k++) d8[k] += p8[q][k];
                }
                if (FLY == 8 && z + 4 <= splits) {
                    float p8[4][8];
#pragma unroll
                    for (int q = 0; q < 4; q++) load8(pz + (size_t)(z + q) * split_stride, p8[q]);
#pragma unroll
                    for (int q = 0; q < 4; q++)
#pragma unroll
                        for (int k = 0; k < 8; k++) d8[k] += p8[q][k];
                    z += 4;
                }
                for (; z < splits; z++) {
                    float p8[8];
                    load8(pz + (size_t)z * split_stride, p8);
#pragma unroll
                    for (int k = 0; k < 8; k++) d8[k] += p8[k];
                }
#pragma unroll
                for (int k = 0; k < 8; k++) v[i][k] += d8[k];
                if (write_resid) store8(x + c, v[i]);
            }
#pragma unroll
            for (int k = 0; k < 8; k++) ss += v[i][k] * v[i][k];
        }
    }
    ss = block_sum(ss, scratch);
    const float scale = rsqrtf(ss / (float)H + eps);
    TA* o = y + (size_t)blockIdx.x * H;
#pragma unroll
    for (int i = 0; i < ITERS; i++) {
        const int c = (threadIdx.x + i * (int)blockDim.x) * 8;
        if (c < H) {
            float r8[8];
#pragma unroll
            for (int k = 0; k < 8; k++) r8[k] = (v[i][k] * scale) * wv[i][k];
            store8(o + c, r8);
        }
    }
}

template <typename TA, typename TW>
static int launch(float* resid, const void* delta, const void* w, void* y, const int* rows,
                  int n_rows, int H, float eps, int write_resid, cudaStream_t s,
                  const float* partials = nullptr, int splits = 0, long long split_stride = 0) {
    if (partials && !((H & 7) == 0 && H <= 2 * 8 * RN_MAX_THREADS)) return ILLM_ERR_BAD_ARG;
    if ((H & 7) == 0 && H <= 2 * 8 * RN_MAX_THREADS) {
        const int chunks = H / 8;
        int threads = (chunks + 31) / 32 * 32;
        if (threads > RN_MAX_THREADS) threads = RN_MAX_THREADS;
        if (threads < 64) threads = 64;
        const int iters = (chunks + threads - 1) / threads;
#define RN_CASE(N, MT)                                                                               \
    illm_launch(add_rmsnorm_reg_kernel<TA, TW, N, MT>, dim3(n_rows), dim3(threads), 0, s, resid, (const TA*)delta, (const TW*)w, \
                                                                   (TA*)y, rows, H, eps, write_resid, partials, splits, split_stride)
        if (iters <= 1 && threads <= 512) RN_CASE(1, 512);
        else if (iters <= 1) RN_CASE(1, RN_MAX_THREADS);
        else RN_CASE(2, RN_MAX_THREADS);
#undef RN_CASE
        return illm_launch_status();
    }
    size_t smem = (size_t)H * sizeof(float);
    if (smem > 200 * 1024) return ILLM_ERR_BAD_ARG;
    auto kern = add_rmsnorm_kernel<TA, TW>;
    if (smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
    }
    int threads = H >= 4096 ? 512 : (H >= 1024 ? 256 : 128);
    illm_launch(kern, dim3(n_rows), dim3(threads), smem, s, resid, (const TA*)delta, (const TW*)w, (TA*)y, rows, H, eps,
                                       write_resid);
    return illm_launch_status();
}

extern "C" int illm_add_rmsnorm(float* resid, const void* delta, const void* w, int w_dtype,
                                void* y, int act_dtype, const int* rows, int n_rows, int H,
                                float eps, int write_resid, void* stream) {
    if (n_rows <= 0) return 0;
    cudaStream_t s = (cudaStream_t)stream;
    if (act_dtype == ILLM_BF16 && w_dtype == ILLM_BF16)
        return launch<bf16, bf16>(resid, delta, w, y, rows, n_rows, H, eps, write_resid, s);
    if (act_dtype == ILLM_BF16 && w_dtype == ILLM_F32)
        return launch<bf16, float>(resid, delta, w, y, rows, n_rows, H, eps, write_resid, s);
    if (act_dtype == ILLM_F32 && w_dtype == ILLM_F32)
        return launch<float, float>(resid, delta, w, y, rows, n_rows, H, eps, write_resid, s);
    if (act_dtype == ILLM_F32 && w_dtype == ILLM_BF16)
        return launch<float, bf16>(resid, delta, w, y, rows, n_rows, H, eps, write_resid, s);
    return ILLM_ERR_BAD_ARG;
}

// The same with the addend given as `splits` float32 slices [splits][rows][H] of a split-K matrix
// product (slice z at partials + z * split_stride): saves the kernel that would add them up.
extern "C" int illm_add_rmsnorm_partials(float* resid, const float* partials, int splits, long long split_stride,
                                         const void* w, int w_dtype, void* y, int act_dtype, const int* rows,
                                         int n_rows, int H, float eps, int write_resid, void* stream) {
    if (n_rows <= 0) return 0;
    if (!partials || splits < 1) return ILLM_ERR_BAD_ARG;
    cudaStream_t s = (cudaStream_t)stream;
    if (act_dtype == ILLM_BF16 && w_dtype == ILLM_BF16)
        return launch<bf16, bf16>(resid, nullptr, w, y, rows, n_rows, H, eps, write_resid, s, partials, splits, split_stride);
    if (act_dtype == ILLM_BF16 && w_dtype == ILLM_F32)
        return launch<bf16, float>(resid, nullptr, w, y, rows, n_rows, H, eps, write_resid, s, partials, splits, split_stride);
    return ILLM_ERR_BAD_ARG;
}

// resid[r] += delta[r] without a norm (flushes a pending addition of the residual stream).
template <typename TA>
__global__ void residual_add_kernel(float* __restrict__ resid, const TA* __restrict__ delta, size_t n) {
    pdl_grid_sync();
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) resid[i] += to_f32(delta[i]);
}

extern "C" int illm_residual_add(float* resid, const void* delta, int act_dtype, long long n,
                                 void* stream) {
    if (n <= 0) return 0;
    cudaStream_t s = (cudaStream_t)stream;
    unsigned blocks = (unsigned)((n + 255) / 256);
    if (act_dtype == ILLM_BF16)
        illm_launch(residual_add_kernel<bf16>, dim3(blocks), dim3(256), 0, s, resid, (const bf16*)delta, (size_t)n);
    else if (act_dtype == ILLM_F32)
        illm_launch(residual_add_kernel<float>, dim3(blocks), dim3(256), 0, s, resid, (const float*)delta, (size_t)n);
    else
        return ILLM_ERR_BAD_ARG;
    return illm_launch_status();
}
