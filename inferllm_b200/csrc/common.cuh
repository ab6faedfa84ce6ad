// Shared device helpers of the sm_100a kernels: element conversion, warp and block
// reductions with a fixed order (so that a row's result never depends on what else is in
// the launch), and the C ABI conventions.
//
// C ABI: every entry point is `extern "C" int illm_<name>(..., void* stream)`; it returns 0
// or a cudaError_t of the launch, never aborts.  dtype codes: 0 = float32, 1 = bfloat16.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#define ILLM_F32 0
#define ILLM_BF16 1
#define ILLM_ERR_BAD_ARG 10001  // outside cudaError_t's range: an argument the kernel refuses

typedef __nv_bfloat16 bf16;

__device__ __forceinline__ float to_f32(float v) { return v; }
__device__ __forceinline__ float to_f32(bf16 v) { return __bfloat162float(v); }
template <typename T> __device__ __forceinline__ T from_f32(float v);
template <> __device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ bf16 from_f32<bf16>(float v) { return __float2bfloat16_rn(v); }

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// Sum over the block; every thread gets the result.  `scratch` holds 32 floats.
__device__ __forceinline__ float block_sum(float v, float* scratch) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int nwarp = (blockDim.x + 31) >> 5;
    v = warp_sum(v);
    __syncthreads();
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    float t = (lane < nwarp) ? scratch[lane] : 0.f;
    return warp_sum(t);
}

// 16-byte loads of 8 bf16 or 4 float into float registers.
__device__ __forceinline__ void load8(const bf16* p, float* f) {
    uint4 u = *reinterpret_cast<const uint4*>(p);
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
    for (int i = 0; i < 4; i++) {
        float2 t = __bfloat1622float2(h[i]);
        f[2 * i] = t.x;
        f[2 * i + 1] = t.y;
    }
}
__device__ __forceinline__ void load8(const float* p, float* f) {
    float4 a = *reinterpret_cast<const float4*>(p);
    float4 b = *reinterpret_cast<const float4*>(p + 4);
    f[0] = a.x; f[1] = a.y; f[2] = a.z; f[3] = a.w;
    f[4] = b.x; f[5] = b.y; f[6] = b.z; f[7] = b.w;
}

__device__ __forceinline__ void store8(bf16* p, const float* f) {
    uint4 u;
    __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&u);
#pragma unroll
    for (int i = 0; i < 4; i++) h[i] = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
    *reinterpret_cast<uint4*>(p) = u;
}
__device__ __forceinline__ void store8(float* p, const float* f) {
    *reinterpret_cast<float4*>(p) = make_float4(f[0], f[1], f[2], f[3]);
    *reinterpret_cast<float4*>(p + 4) = make_float4(f[4], f[5], f[6], f[7]);
}

// 2^x by the special-function unit (one instruction, relative error about 2^-22, -inf gives 0):
// for softmax weights that are rounded to bfloat16 or summed in float32 afterwards.
__device__ __forceinline__ float fast_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

// Programmatic dependent launch.  Every kernel of the package starts with pdl_grid_sync(): it
// lets the kernel after it in the stream begin to launch, then waits until the kernels before
// it have finished and their writes are visible.  With the launch attribute below, a kernel's
// blocks are therefore scheduled and set up (shared memory, barriers, and in the matrix product
// the first weight tiles) while its predecessors are still running, which hides most of the gap
// between the many short kernels of a decode step.  A kernel still touches no activation before
// its own wait, and a kernel's wait covers everything before it in the stream, so the order of
// reads and writes is the stream's.  Without the attribute both instructions do nothing.
__device__ __forceinline__ void pdl_grid_sync() {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
}

inline int g_illm_pdl = 1;   // illm_set_pdl() switches the launch attribute off (e.g. for profilers)
inline long long g_illm_launches = 0;   // kernels launched by this library (illm_launch_count())

template <typename... KArgs, typename... Args>
static inline void illm_launch(void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t s,
                               Args&&... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = s;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = g_illm_pdl ? 1 : 0;
    g_illm_launches++;
    cudaLaunchKernelEx(&cfg, kern, static_cast<KArgs>(args)...);
}

static inline int illm_launch_status() { return (int)cudaGetLastError(); }
