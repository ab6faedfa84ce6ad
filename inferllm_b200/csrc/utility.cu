// Utility kernels: random weights from a counter-based generator, poisoning of cache pages that
// went back to the pool, and a self-test of the bounded mbarrier wait.
//
// The reference has no counterpart of the first two (its tests randomise tensors per operator on
// the host, test/checker.cpp:162-204, and its one KV tensor per layer is never given back); where
// it meets a condition it cannot handle it aborts (src/utils.h:120-130), where the kernels of this
// package set an error word and return.
#include <cuda_fp16.h>

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

// ---- conversions and small index kernels ------------------------------------------------------------

template <typename TIn> __device__ __forceinline__ float load_as_f32(const TIn* p, long long i) { return (float)p[i]; }
template <> __device__ __forceinline__ float load_as_f32<bf16>(const bf16* p, long long i) { return __bfloat162float(p[i]); }
template <> __device__ __forceinline__ float load_as_f32<__half>(const __half* p, long long i) { return __half2float(p[i]); }

template <typename TIn, typename TOut>
__global__ void convert_kernel(const TIn* __restrict__ src, TOut* __restrict__ dst, long long n) {
    pdl_grid_sync();
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x)
        dst[i] = from_f32<TOut>(load_as_f32<TIn>(src, i));
}
template <typename TIn>
__global__ void convert_int_kernel(const TIn* __restrict__ src, int* __restrict__ dst, long long n) {
    pdl_grid_sync();
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x)
        dst[i] = (int)src[i];
}

// Element-wise conversion of a stored tensor into an engine dtype.  src codes: 0 float32, 1 bfloat16,
// 2 float16, 3 float64, 4 int64, 5 int32, 6 int16, 7 int8, 8 uint8; dst codes: 0 float32, 1 bfloat16,
// 5 int32 (floating point to floating point, integers to int32).  bfloat16 results are rounded to
// nearest even from the float32 value of the source.
extern "C" int illm_convert(const void* src, int src_dtype, void* dst, int dst_dtype, long long n, void* stream) {
    if (n <= 0) return 0;
    cudaStream_t s = (cudaStream_t)stream;
    long long blocks = (n + 255) / 256;
    if (blocks > 148 * 16) blocks = 148 * 16;
    const dim3 grid((unsigned)blocks), block(256);
#define CONV(SC, TIN, DC, TOUT)                                                                         \
    if (src_dtype == SC && dst_dtype == DC) {                                                            \
        illm_launch(convert_kernel<TIN, TOUT>, grid, block, 0, s, (const TIN*)src, (TOUT*)dst, n);       \
        return illm_launch_status();                                                                     \
    }
    CONV(0, float, 0, float) CONV(0, float, 1, bf16) CONV(1, bf16, 0, float) CONV(1, bf16, 1, bf16)
    CONV(2, __half, 0, float) CONV(2, __half, 1, bf16) CONV(3, double, 0, float) CONV(3, double, 1, bf16)
#undef CONV
#define CONVI(SC, TIN)                                                                          \
    if (src_dtype == SC && dst_dtype == 5) {                                                     \
        illm_launch(convert_int_kernel<TIN>, grid, block, 0, s, (const TIN*)src, (int*)dst, n);  \
        return illm_launch_status();                                                             \
    }
    CONVI(4, long long) CONVI(5, int) CONVI(6, short) CONVI(7, signed char) CONVI(8, unsigned char)
#undef CONVI
    return ILLM_ERR_BAD_ARG;
}

// dst[i] = src[idx[i]] for i < n (int32): the sampled tokens of the sequences that go on.
__global__ void gather_i32_kernel(const int* __restrict__ src, const int* __restrict__ idx, int* __restrict__ dst, int n) {
    pdl_grid_sync();
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) dst[i] = src[idx[i]];
}
extern "C" int illm_gather_i32(const int* src, const int* idx, int* dst, int n, void* stream) {
    if (n <= 0) return 0;
    illm_launch(gather_i32_kernel, dim3((n + 255) / 256), dim3(256), 0, (cudaStream_t)stream, src, idx, dst, n);
    return illm_launch_status();
}

// The windows of last tokens of the repetition penalty, int32 [rows of the batch, n_last].
// gather: dst[i, :] = window[rows[i], :];  put: window[rows[i], col] = toks[i]  (rows == nullptr: row i).
__global__ void window_gather_kernel(const int* __restrict__ window, int n_last, const int* __restrict__ rows,
                                     int* __restrict__ dst, int n) {
    pdl_grid_sync();
    const int i = blockIdx.x;
    if (i >= n) return;
    const int r = rows ? rows[i] : i;
    for (int c = threadIdx.x; c < n_last; c += blockDim.x) dst[(size_t)i * n_last + c] = window[(size_t)r * n_last + c];
}
__global__ void window_put_kernel(int* __restrict__ window, int n_last, const int* __restrict__ rows, int col,
                                  const int* __restrict__ toks, int n) {
    pdl_grid_sync();
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) window[(size_t)(rows ? rows[i] : i) * n_last + col] = toks[i];
}
extern "C" int illm_window_gather(const int* window, int n_last, const int* rows, int* dst, int n, void* stream) {
    if (n <= 0 || n_last <= 0) return 0;
    illm_launch(window_gather_kernel, dim3(n), dim3(64), 0, (cudaStream_t)stream, window, n_last, rows, dst, n);
    return illm_launch_status();
}
extern "C" int illm_window_put(int* window, int n_last, const int* rows, int col, const int* toks, int n, void* stream) {
    if (n <= 0 || n_last <= 0) return 0;
    if (col < 0 || col >= n_last) return ILLM_ERR_BAD_ARG;
    illm_launch(window_put_kernel, dim3((n + 255) / 256), dim3(256), 0, (cudaStream_t)stream, window, n_last, rows, col, toks, n);
    return illm_launch_status();
}
