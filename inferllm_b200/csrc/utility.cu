// Utility kernels: random weights from a counter-based generator, poisoning of cache pages that
// went back to the pool, and a self-test of the bounded mbarrier wait.
//
// The reference has no counterpart of the first two (its tests randomise tensors per operator on
// the host, test/checker.cpp:162-204, and its one KV tensor per layer is never given back); where
// it meets a condition it cannot handle it aborts (src/utils.h:120-130), where the kernels of this
// package set an error word and return.
#include "random_init.h"
#include "tc_common.cuh"

// ---- random weights -------------------------------------------------------------------------------

template <typename T>
__global__ void fill_random_kernel(T* __restrict__ out, long long n, unsigned long long base, float scale, float mean) {
    pdl_grid_sync();
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
        // one multiplication and one addition, each rounded once: what the host twins do
        const float v = __fadd_rn(__fmul_rn((float)illm_random_centered_sum(base, (unsigned long long)i), scale), mean);
        out[i] = from_f32<T>(v);
    }
}

// out[i] = mean + std * z_i for i in [0, n), z_i the approximately normal number i of the stream
// `key` (illm_random_key(seed, tensor name)); see random_init.h for the exact definition.
// dtype: 0 float32, 1 bfloat16 (rounded to nearest even from the float32 value).
extern "C" int illm_fill_random(void* out, int dtype, long long n, unsigned long long key, float std, float mean,
                                void* stream) {
    if (n <= 0) return 0;
    if (out == nullptr || (dtype != ILLM_F32 && dtype != ILLM_BF16)) return ILLM_ERR_BAD_ARG;
    const unsigned long long base = illm_random_base(key);
    const float scale = std / 65536.0f;          // exact: a power of two
    const int threads = 256;
    long long blocks = (n + threads - 1) / threads;
    if (blocks > 148 * 16) blocks = 148 * 16;
    if (dtype == ILLM_F32)
        illm_launch(fill_random_kernel<float>, dim3((unsigned)blocks), dim3(threads), 0, (cudaStream_t)stream,
                    (float*)out, n, base, scale, mean);
    else
        illm_launch(fill_random_kernel<bf16>, dim3((unsigned)blocks), dim3(threads), 0, (cudaStream_t)stream,
                    (bf16*)out, n, base, scale, mean);
    return illm_launch_status();
}

// ---- poisoned pages -------------------------------------------------------------------------------

// Fills pages of a paged group with all-ones bits, which is a NaN in bfloat16 and in float32: a
// kernel that reads a page its sequence no longer holds (or does not hold yet) then gives NaN
// instead of a plausible number.  k, v: [entries, pages, page_bytes]; pages: the pages to fill.
__global__ void poison_pages_kernel(uint4* __restrict__ k, uint4* __restrict__ v, long long entry_vec, long long page_vec,
                                    const int* __restrict__ pages) {
    pdl_grid_sync();
    const long long off = (long long)blockIdx.y * entry_vec + (long long)pages[blockIdx.x] * page_vec;
    uint4* dst = (blockIdx.z ? v : k) + off;
    const uint4 ones = make_uint4(0xFFFFFFFFu, 0xFFFFFFFFu, 0xFFFFFFFFu, 0xFFFFFFFFu);
    for (long long i = threadIdx.x; i < page_vec; i += blockDim.x) dst[i] = ones;
}

extern "C" int illm_poison_pages(void* k, void* v, long long entry_stride_bytes, int n_entries, long long page_bytes,
                                 const int* pages, int n_pages, void* stream) {
    if (n_pages <= 0 || n_entries <= 0) return 0;
    if (k == nullptr || v == nullptr || pages == nullptr || (page_bytes & 15) || (entry_stride_bytes & 15) ||
        ((uintptr_t)k & 15) || ((uintptr_t)v & 15) || n_pages > 65535 * 32767 || n_entries > 65535)
        return ILLM_ERR_BAD_ARG;
    for (int p0 = 0; p0 < n_pages; p0 += 1 << 20) {
        const int n = n_pages - p0 < (1 << 20) ? n_pages - p0 : (1 << 20);
        illm_launch(poison_pages_kernel, dim3(n, n_entries, 2), dim3(256), 0, (cudaStream_t)stream, (uint4*)k, (uint4*)v,
                    entry_stride_bytes / 16, page_bytes / 16, pages + p0);
    }
    return illm_launch_status();
}

// ---- self-test of the bounded wait ----------------------------------------------------------------

// One thread waits, through the same mbar_wait as the tensor-core kernels, for a phase of an mbarrier
// at which nobody ever arrives, with a limit of `limit_clocks` instead of the kernels' second.  The
// wait gives up, the error word gets `code`, and the kernel returns: result[0] = 1 if the wait
// reported the time-out to its caller, result[1] = the clocks it waited.  Nothing else of the device
// is touched: no copy is in flight and no tensor memory is held when the wait ends.
__global__ void selftest_wait_timeout_kernel(int* err, long long* result, long long limit_clocks, int code) {
    __shared__ __align__(8) unsigned long long bar;
    if (threadIdx.x == 0) {
        mbar_init(tc_smem_u32(&bar), 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        const long long t0 = clock64();
        const bool done = mbar_wait(tc_smem_u32(&bar), 0, err, code, limit_clocks);
        result[0] = done ? 0 : 1;
        result[1] = clock64() - t0;
    }
}

extern "C" int illm_selftest_wait_timeout(int* err, long long* result, long long limit_clocks, int code, void* stream) {
    if (err == nullptr || result == nullptr || limit_clocks <= 0 || limit_clocks > TC_WAIT_CLOCKS) return ILLM_ERR_BAD_ARG;
    selftest_wait_timeout_kernel<<<1, 32, 0, (cudaStream_t)stream>>>(err, result, limit_clocks, code);
    return illm_launch_status();
}
