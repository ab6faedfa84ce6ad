// Gated activation of the feed-forward: out[t, i] = silu(gu[t, 2i]) * gu[t, 2i + 1]: the packed
// projection holds gate and up of an output next to each other (the weight's rows are interleaved at
// load), so that a matrix-product epilogue that sees a few neighbouring columns can apply the same
// formula without this kernel.
// silu(x) = x / (1 + exp(-x)) as in the reference (src/kern/gpu/kernel_gpu.cu:183-258 runs it
// as two launches, Silu and Mul; formula src/kern/naive/naive.cpp:80-89), in float32.
#include "common.cuh"

template <typename TA>
__global__ void swiglu_kernel(const TA* __restrict__ gu, TA* __restrict__ out, int I) {
    pdl_grid_sync();
    const int t = blockIdx.y;
    const TA* g = gu + (size_t)t * 2 * I;
    TA* o = out + (size_t)t * I;
    for (int c = blockIdx.x * blockDim.x + threadIdx.x; c < I; c += gridDim.x * blockDim.x) {
        float a = to_f32(g[2 * c]);
        float b = to_f32(g[2 * c + 1]);
        float sv = a / (1.0f + expf(-a));
        o[c] = from_f32<TA>(sv * b);
    }
}

// 8 outputs per thread from 16 consecutive inputs with 16-byte loads (I a multiple of 8).
template <typename TA>
__global__ void swiglu_vec_kernel(const TA* __restrict__ gu, TA* __restrict__ out, int I, long long n_vec) {
    pdl_grid_sync();
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n_vec) return;
    const int per_row = I / 8;
    const long long t = i / per_row;
    const int c = (int)(i - t * per_row) * 8;
    float x[16];
    load8(gu + t * 2 * I + 2 * c, x);
    load8(gu + t * 2 * I + 2 * c + 8, x + 8);
    float r[8];
#pragma unroll
    for (int k = 0; k < 8; k++) r[k] = (x[2 * k] / (1.0f + expf(-x[2 * k]))) * x[2 * k + 1];
    store8(out + t * I + c, r);
}

// The same with the packed projection still in `P` float32 slices of a split matrix product
// (slice z at slices + z * stride): they are added in ascending order first.
__global__ void swiglu_partials_kernel(const float* __restrict__ slices, int P, long long stride,
                                       bf16* __restrict__ out, int I, long long n_vec) {
    pdl_grid_sync();
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n_vec) return;
    const int per_row = I / 8;
    const long long t = i / per_row;
    const int c = (int)(i - t * per_row) * 8;
    float x[16];
#pragma unroll
    for (int k = 0; k < 16; k++) x[k] = 0.f;
    for (int z = 0; z < P; z++) {
        float px[16];
        load8(slices + (size_t)z * stride + t * 2 * I + 2 * c, px);
        load8(slices + (size_t)z * stride + t * 2 * I + 2 * c + 8, px + 8);
#pragma unroll
        for (int k = 0; k < 16; k++) x[k] += px[k];
    }
    float r[8];
#pragma unroll
    for (int k = 0; k < 8; k++) r[k] = (x[2 * k] / (1.0f + expf(-x[2 * k]))) * x[2 * k + 1];
    store8(out + t * I + c, r);
}

extern "C" int illm_swiglu_partials(const float* slices, int P, long long stride, void* out, int T, int I,
                                    void* stream) {
    if (T <= 0 || I <= 0) return 0;
    if ((I & 7) || P < 1) return ILLM_ERR_BAD_ARG;
    const long long n_vec = (long long)T * (I / 8);
    illm_launch(swiglu_partials_kernel, dim3((unsigned)((n_vec + 255) / 256)), dim3(256), 0, (cudaStream_t)stream,
                slices, P, stride, (bf16*)out, I, n_vec);
    return illm_launch_status();
}

extern "C" int illm_swiglu(const void* gu, void* out, int act_dtype, int T, int I, void* stream) {
    if (T <= 0 || I <= 0) return 0;
    if (T > 65535 * 32) return ILLM_ERR_BAD_ARG;
    cudaStream_t s = (cudaStream_t)stream;
    if ((I & 7) == 0) {
        const long long n_vec = (long long)T * (I / 8);
        const unsigned blocks = (unsigned)((n_vec + 255) / 256);
        if (act_dtype == ILLM_BF16)
            illm_launch(swiglu_vec_kernel<bf16>, dim3(blocks), dim3(256), 0, s, (const bf16*)gu, (bf16*)out, I, n_vec);
        else if (act_dtype == ILLM_F32)
            illm_launch(swiglu_vec_kernel<float>, dim3(blocks), dim3(256), 0, s, (const float*)gu, (float*)out, I, n_vec);
        else
            return ILLM_ERR_BAD_ARG;
        return illm_launch_status();
    }
    // grid.y is limited to 65535: fold larger T into several launches
    for (int t0 = 0; t0 < T; t0 += 65535) {
        int n = T - t0 < 65535 ? T - t0 : 65535;
        dim3 grid((I + 255) / 256 > 64 ? 64 : (I + 255) / 256, n);
        if (act_dtype == ILLM_BF16)
            illm_launch(swiglu_kernel<bf16>, dim3(grid), dim3(256), 0, s, (const bf16*)gu + (size_t)t0 * 2 * I,
                                                     (bf16*)out + (size_t)t0 * I, I);
        else if (act_dtype == ILLM_F32)
            illm_launch(swiglu_kernel<float>, dim3(grid), dim3(256), 0, s, (const float*)gu + (size_t)t0 * 2 * I,
                                                      (float*)out + (size_t)t0 * I, I);
        else
            return ILLM_ERR_BAD_ARG;
    }
    return illm_launch_status();
}
