// One GPU as the engine sees it: a stream, memory, the library's matrix product and the kernels'
// error words.
//
// Memory comes in two kinds.  Persistent blocks (weights, cache pages, tables, inputs and outputs of
// captured graphs) are taken from the driver one by one and live until they are freed.  Everything a
// step computes on its way (activations, partial results, scratch of kernels) comes from the step
// arena: lists of large blocks from which allocations are cut off in order and which are rewound,
// not freed.  The same sequence of allocations therefore gets the same addresses every time, which
// is what lets a step be captured in a CUDA graph and replayed, and no step pays the driver for
// memory once the arena has seen its size.  The arena has three lanes: lane 0 holds what lives for
// the whole step (its index arrays, the residual stream, the logits); lanes 1 and 2 take turns
// layer by layer, and a lane is rewound when its turn comes again, so a step holds the activations
// of two layers, not of all (what a layer hands to the next one, its last product's output, is read
// by the next layer's first norm, before that layer's own lane comes round again).  The arena only
// grows while steps run: a block is never given back or moved, so addresses inside captured graphs
// stay valid.  The reference's counterpart is its Device with a free-list pool per size
// (src/core/device.cpp: allocate / free_device) and a workspace that is re-sized when the token
// count changes (src/core/graph.cpp:169-180).
#pragma once
#include <cuda_runtime.h>

#include <cstddef>
#include <string>
#include <vector>

#include "util/dtype.h"
#include "util/error.h"

namespace illm {

// Raises KernelError for a non-zero status of a kernel entry point (`what` names it).
void check_kernel(int code, const char* what);
// Raises EngineError for a CUDA runtime error.
void check_cuda(cudaError_t e, const char* what);

class Device {
public:
    // `stream`: the stream all work is issued to; nullptr creates one (the Python binding passes the
    // stream of the framework whose tensors it exchanges).
    explicit Device(int ordinal, cudaStream_t stream = nullptr);
    ~Device();
    Device(const Device&) = delete;

    int ordinal() const { return ordinal_; }
    int n_sms() const { return n_sms_; }
    // Bytes per microsecond that a streaming kernel reads from device memory: 0.86 of the product of the
    // memory clock, the bus width and the double data rate, which is what a copy reaches on this kind of
    // memory (6.6e6 on a B200).  The policies that weigh a kernel's stream against its fixed costs use it.
    double stream_bytes_per_us() const { return stream_bytes_per_us_; }
    cudaStream_t stream() const { return stream_; }
    void set_stream(cudaStream_t s);
    // Ordering against another stream of the same device (a caller that exchanges device memory with
    // the engine works on its own stream): this stream waits for what `other` holds now / `other` waits
    // for what this stream holds now.  Neither blocks the host.
    void wait_for(cudaStream_t other);
    void signal_to(cudaStream_t other);
    void make_current() const;
    void synchronize() const;
    size_t mem_free() const;

    // persistent memory (zeroed when `zero`); `what` goes into the error message when the device is full
    void* alloc_persistent(size_t bytes, const char* what, bool zero = false);
    void free_persistent(void* p);

    // the step arena
    static constexpr int kLanes = 3;
    void* alloc(size_t bytes);                 // from the current lane; 256-byte aligned; valid until that lane is rewound
    template <typename T> T* alloc_n(size_t n) { return (T*)alloc(n * sizeof(T)); }
    void arena_rewind();                       // a new step begins: all lanes rewound, lane 0 current
    void set_lane(int lane, bool rewind);      // allocate from this lane from now on (rewound first if asked)
    void arena_release();                      // give all blocks back to the driver (only while no captured graph uses them)
    size_t arena_bytes() const;                // what the arena holds from the driver
    unsigned long long arena_generation() const { return arena_generation_; }   // grows whenever a block was added

    int* tc_error_word() const { return tc_err_; }       // bounded waits of the tensor-core kernels
    int* step_error_word() const { return step_err_; }   // ids outside the table, writes to unheld pages, ...
    // Read and clear both words (synchronises); returns {tensor-core word, step word}.
    std::pair<int, int> take_error_words();

    // bfloat16 x [M, K] . w [N, K]^T -> out [M, N] (bfloat16 or float32) with float32 accumulation by
    // the library (cuBLAS), as the reference uses cublasSgemm for its float32 products
    // (src/kern/gpu/kernel_gpu.cu:420-435).
    void library_gemm_bf16(const void* x, const void* w, void* out, DType out_dtype, int M, int N, int K);

    // Copy a small host array to the device without making the host wait for the work already queued:
    // through a ring of pinned staging buffers, each reused only when its copy has left.
    void upload_small(void* dst, const void* src, size_t bytes);

    // pinned host memory (staging of a step's index arrays and of sampled tokens)
    void* alloc_pinned(size_t bytes);
    void free_pinned(void* p);

private:
    struct Block { char* base; size_t size, used; };
    struct Lane { std::vector<Block> blocks; size_t cur = 0; };
    int ordinal_, n_sms_ = 148;
    double stream_bytes_per_us_ = 6.6e6;
    cudaStream_t stream_ = nullptr;
    bool own_stream_ = false;
    Lane lanes_[kLanes];
    int lane_ = 0;
    unsigned long long arena_generation_ = 0;
    int *tc_err_ = nullptr, *step_err_ = nullptr;
    void* cublas_ = nullptr;
    void* cublas_ws_ = nullptr;
    cudaEvent_t order_event_ = nullptr;
    struct SmallStage { char* host = nullptr; size_t cap = 0; cudaEvent_t done = nullptr; bool used = false; };
    SmallStage small_[8];
    int small_next_ = 0;
};

}  // namespace illm
