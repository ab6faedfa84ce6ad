// Token embedding: x[t, :] = table[ids[t], :], written as the float32 residual stream.
// Replaces the reference's row gather (src/kern/gpu/kernel_gpu.cu:127-148,
// src/kern/naive/naive.cpp:43-54).  One block per token; 16-byte loads where the row
// allows it.  An id outside [0, V) writes zeros and raises the error word instead of
// reading outside the table.
#include "common.cuh"

template <typename TW>
__global__ void embedding_kernel(const int* __restrict__ ids, const TW* __restrict__ table,
                                 float* __restrict__ out, int H, int V, int* __restrict__ err) {
    pdl_grid_sync();
    const int t = blockIdx.x;
    const int id = ids[t];
    float* o = out + (size_t)t * H;
    if (id < 0 || id >= V) {
        if (threadIdx.x == 0) atomicExch(err, 1);
        for (int c = threadIdx.x; c < H; c += blockDim.x) o[c] = 0.f;
        return;
    }
    const TW* row = table + (size_t)id * H;
    if ((H & 7) == 0) {
        for (int c = threadIdx.x * 8; c < H; c += blockDim.x * 8) {
            float f[8];
            load8(row + c, f);
            *reinterpret_cast<float4*>(o + c) = make_float4(f[0], f[1], f[2], f[3]);
            *reinterpret_cast<float4*>(o + c + 4) = make_float4(f[4], f[5], f[6], f[7]);
        }
    } else {
        for (int c = threadIdx.x; c < H; c += blockDim.x) o[c] = to_f32(row[c]);
    }
}

extern "C" int illm_embedding(const int* ids, const void* table, int table_dtype, float* out,
                              int T, int H, int V, int* err, void* stream) {
    if (T <= 0) return 0;
    cudaStream_t s = (cudaStream_t)stream;
    int threads = H >= 2048 ? 256 : 128;
    if (table_dtype == ILLM_BF16)
        illm_launch(embedding_kernel<bf16>, dim3(T), dim3(threads), 0, s, ids, (const bf16*)table, out, H, V, err);
    else if (table_dtype == ILLM_F32)
        illm_launch(embedding_kernel<float>, dim3(T), dim3(threads), 0, s, ids, (const float*)table, out, H, V, err);
    else
        return ILLM_ERR_BAD_ARG;
    return illm_launch_status();
}

// Switches programmatic dependent launch of all kernels of the library on (1, default) or off (0).
extern "C" int illm_set_pdl(int on) {
    g_illm_pdl = on ? 1 : 0;
    return 0;
}

// How many kernels the library has launched in this process (a launch into a stream capture counts
// once; replays of the captured graph are the caller's to count).
extern "C" long long illm_launch_count() { return g_illm_launches; }
