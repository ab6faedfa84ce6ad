#include "device/device.h"

#include <cublas_v2.h>

#include <algorithm>
#include <cstring>

namespace illm {

void check_kernel(int code, const char* what) {
    if (code == 0) return;
    if (code == 10001) throw KernelError(std::string(what) + ": the kernel refused its arguments");
    throw KernelError(std::string(what) + ": CUDA error " + std::to_string(code) + " (" +
                      cudaGetErrorString((cudaError_t)code) + ")");
}

void check_cuda(cudaError_t e, const char* what) {
    if (e != cudaSuccess) throw EngineError(std::string(what) + ": " + cudaGetErrorString(e));
}

Device::Device(int ordinal, cudaStream_t stream) : ordinal_(ordinal) {
    int count = 0;
    if (cudaGetDeviceCount(&count) != cudaSuccess || count == 0)
        throw EngineError("inferllm_b200 needs a CUDA device: there is no CPU path");
    if (ordinal < 0 || ordinal >= count)
        throw EngineError("GPU " + std::to_string(ordinal) + " does not exist (" + std::to_string(count) + " visible)");
    check_cuda(cudaSetDevice(ordinal), "cudaSetDevice");
    cudaDeviceProp prop;
    check_cuda(cudaGetDeviceProperties(&prop, ordinal), "cudaGetDeviceProperties");
    n_sms_ = prop.multiProcessorCount;
    int mem_khz = 0, bus_bits = 0;
    if (cudaDeviceGetAttribute(&mem_khz, cudaDevAttrMemoryClockRate, ordinal) == cudaSuccess &&
        cudaDeviceGetAttribute(&bus_bits, cudaDevAttrGlobalMemoryBusWidth, ordinal) == cudaSuccess && mem_khz > 0 && bus_bits > 0)
        stream_bytes_per_us_ = 0.86 * 2.0 * (double)mem_khz * 1e3 * ((double)bus_bits / 8.0) / 1e6;
    if (prop.major != 10)
        throw EngineError(std::string("GPU ") + prop.name + " has compute capability " + std::to_string(prop.major) + "." +
                          std::to_string(prop.minor) + ": the kernels of inferllm_b200 are built for sm_100a (B200) only");
    if (stream) {
        stream_ = stream;
    } else {
        check_cuda(cudaStreamCreateWithFlags(&stream_, cudaStreamNonBlocking), "cudaStreamCreate");
        own_stream_ = true;
    }
    tc_err_ = (int*)alloc_persistent(256, "the error words", true);
    step_err_ = tc_err_ + 32;
    cublasHandle_t h;
    if (cublasCreate(&h) != CUBLAS_STATUS_SUCCESS) throw EngineError("cublasCreate failed");
    cublas_ = h;
    // a workspace of its own: the library then allocates nothing during a step or a capture
    cublas_ws_ = alloc_persistent(32u << 20, "the library's workspace");
    cublasSetWorkspace(h, cublas_ws_, 32u << 20);
    cublasSetStream(h, stream_);
}

Device::~Device() {
    cudaSetDevice(ordinal_);
    cudaStreamSynchronize(stream_);
    if (order_event_) cudaEventDestroy(order_event_);
    for (SmallStage& st : small_) {
        if (st.host) cudaFreeHost(st.host);
        if (st.done) cudaEventDestroy(st.done);
    }
    if (cublas_) cublasDestroy((cublasHandle_t)cublas_);
    if (cublas_ws_) cudaFree(cublas_ws_);
    if (tc_err_) cudaFree(tc_err_);
    for (Lane& lane : lanes_)
        for (Block& b : lane.blocks) cudaFree(b.base);
    if (own_stream_) cudaStreamDestroy(stream_);
}

void Device::set_stream(cudaStream_t s) {
    if (s == stream_) return;
    cudaStreamSynchronize(stream_);
    if (own_stream_) cudaStreamDestroy(stream_);
    own_stream_ = false;
    stream_ = s;
    cublasSetStream((cublasHandle_t)cublas_, stream_);
}

void Device::wait_for(cudaStream_t other) {
    if (other == stream_) return;
    if (!order_event_) check_cuda(cudaEventCreateWithFlags(&order_event_, cudaEventDisableTiming), "cudaEventCreate");
    check_cuda(cudaEventRecord(order_event_, other), "cudaEventRecord");
    check_cuda(cudaStreamWaitEvent(stream_, order_event_, 0), "cudaStreamWaitEvent");
}
void Device::signal_to(cudaStream_t other) {
    if (other == stream_) return;
    if (!order_event_) check_cuda(cudaEventCreateWithFlags(&order_event_, cudaEventDisableTiming), "cudaEventCreate");
    check_cuda(cudaEventRecord(order_event_, stream_), "cudaEventRecord");
    check_cuda(cudaStreamWaitEvent(other, order_event_, 0), "cudaStreamWaitEvent");
}

void Device::make_current() const { check_cuda(cudaSetDevice(ordinal_), "cudaSetDevice"); }
void Device::synchronize() const { check_cuda(cudaStreamSynchronize(stream_), "cudaStreamSynchronize"); }

size_t Device::mem_free() const {
    size_t free_b = 0, total = 0;
    make_current();
    check_cuda(cudaMemGetInfo(&free_b, &total), "cudaMemGetInfo");
    return free_b;
}

void* Device::alloc_persistent(size_t bytes, const char* what, bool zero) {
    make_current();
    void* p = nullptr;
    if (bytes == 0) bytes = 256;
    cudaError_t e = cudaMalloc(&p, bytes);
    if (e != cudaSuccess) {
        cudaGetLastError();
        size_t free_b = 0, total = 0;
        cudaMemGetInfo(&free_b, &total);
        char msg[256];
        snprintf(msg, sizeof msg, "%s needs %.2f GiB, the device has %.2f GiB free", what, bytes / 1073741824.0,
                 free_b / 1073741824.0);
        throw EngineError(msg);
    }
    if (zero) check_cuda(cudaMemsetAsync(p, 0, bytes, stream_), "cudaMemset");
    return p;
}

void Device::free_persistent(void* p) {
    if (!p) return;
    cudaStreamSynchronize(stream_);
    cudaFree(p);
}

void* Device::alloc(size_t bytes) {
    bytes = (bytes + 255) & ~(size_t)255;
    if (bytes == 0) bytes = 256;
    Lane& lane = lanes_[lane_];
    while (lane.cur < lane.blocks.size()) {
        Block& b = lane.blocks[lane.cur];
        if (b.used + bytes <= b.size) {
            void* p = b.base + b.used;
            b.used += bytes;
            return p;
        }
        lane.cur++;
        if (lane.cur < lane.blocks.size()) lane.blocks[lane.cur].used = 0;
    }
    // a new block: at least 64 MiB, and at least half of what the lane holds (so the blocks stay few)
    size_t held = 0;
    for (Block& b : lane.blocks) held += b.size;
    const size_t size = std::max<size_t>({bytes, held / 2, (size_t)64 << 20});
    Block nb;
    nb.base = (char*)alloc_persistent(size, "the step's working memory");
    nb.size = size;
    nb.used = bytes;
    lane.blocks.push_back(nb);
    lane.cur = lane.blocks.size() - 1;
    arena_generation_++;
    return nb.base;
}

void Device::set_lane(int lane, bool rewind) {
    lane_ = lane;
    if (rewind) {
        lanes_[lane].cur = 0;
        if (!lanes_[lane].blocks.empty()) lanes_[lane].blocks[0].used = 0;
    }
}

void Device::arena_rewind() {
    for (int l = 0; l < kLanes; l++) set_lane(l, true);
    lane_ = 0;
}

void Device::arena_release() {
    synchronize();
    for (Lane& lane : lanes_) {
        for (Block& b : lane.blocks) cudaFree(b.base);
        lane.blocks.clear();
        lane.cur = 0;
    }
    lane_ = 0;
}

size_t Device::arena_bytes() const {
    size_t held = 0;
    for (const Lane& lane : lanes_)
        for (const Block& b : lane.blocks) held += b.size;
    return held;
}

std::pair<int, int> Device::take_error_words() {
    int host[64];
    make_current();
    check_cuda(cudaMemcpyAsync(host, tc_err_, sizeof host, cudaMemcpyDeviceToHost, stream_), "reading the error words");
    synchronize();
    if (host[0] || host[32]) {
        check_cuda(cudaMemsetAsync(tc_err_, 0, 256, stream_), "clearing the error words");
        synchronize();
    }
    return {host[0], host[32]};
}

void Device::library_gemm_bf16(const void* x, const void* w, void* out, DType out_dtype, int M, int N, int K) {
    const float alpha = 1.f, beta = 0.f;
    // row-major out [M, N] is column-major [N, M] = w (column-major [K, N], transposed) . x (column-major [K, M])
    cublasStatus_t st = cublasGemmEx((cublasHandle_t)cublas_, CUBLAS_OP_T, CUBLAS_OP_N, N, M, K, &alpha, w, CUDA_R_16BF, K, x,
                                     CUDA_R_16BF, K, &beta, out, out_dtype == DType::F32 ? CUDA_R_32F : CUDA_R_16BF, N,
                                     CUBLAS_COMPUTE_32F, CUBLAS_GEMM_DEFAULT_TENSOR_OP);
    if (st != CUBLAS_STATUS_SUCCESS)
        throw KernelError("the library's matrix product failed with status " + std::to_string((int)st) + " for [" +
                          std::to_string(M) + ", " + std::to_string(K) + "] x [" + std::to_string(N) + ", " + std::to_string(K) + "]^T");
}

void Device::upload_small(void* dst, const void* src, size_t bytes) {
    if (bytes == 0) return;
    SmallStage& st = small_[small_next_];
    small_next_ = (small_next_ + 1) % 8;
    if (!st.done) check_cuda(cudaEventCreateWithFlags(&st.done, cudaEventDisableTiming), "cudaEventCreate");
    if (st.used) check_cuda(cudaEventSynchronize(st.done), "waiting for a staging buffer");
    if (st.cap < bytes) {
        if (st.host) cudaFreeHost(st.host);
        st.cap = std::max<size_t>(bytes, 65536);
        st.host = (char*)alloc_pinned(st.cap);
    }
    memcpy(st.host, src, bytes);
    check_cuda(cudaMemcpyAsync(dst, st.host, bytes, cudaMemcpyHostToDevice, stream_), "uploading a small array");
    check_cuda(cudaEventRecord(st.done, stream_), "cudaEventRecord");
    st.used = true;
}

void* Device::alloc_pinned(size_t bytes) {
    void* p = nullptr;
    check_cuda(cudaMallocHost(&p, bytes ? bytes : 64), "cudaMallocHost");
    return p;
}
void Device::free_pinned(void* p) {
    if (p) cudaFreeHost(p);
}

}  // namespace illm
