// A decode-attention entry point for callers that cannot allocate device memory.
//
// This has no counterpart in MegEngine/InferLLM: the reference allocates its attention
// workspace from its device pool on every step (src/core/op.cpp:289-329, src/core/device.cpp).
//
// Who needs it: code that runs where cudaMalloc is off limits.  Examples are a host program that
// has handed all device memory to its own pool up front and must not let a library take more, a
// real-time loop in which an allocation's latency or failure is not acceptable, and callers that
// issue work while a stream capture is open, where cudaMalloc would invalidate the capture.
// The regular entry point, illm_attention_decode, leaves the scratch to its caller (the Python
// face takes it from torch's allocator); this one brings its own.
//
//   int illm_attention_decode_static(q, q_stride, kc, vc, block_table, max_pages, token_pos,
//                                    token_seq, out, T, nh, nkv, d, page_size, window, scale,
//                                    max_len, err_msg, err_len, stream)
//
// Arguments are those of illm_attention_decode (bfloat16 q, cache pages and out; int32 tables),
// without the two scratch pointers; `max_len` bounds the sequence lengths of the call and decides
// how much scratch it needs: T * nh * ceil(max_len / 256) * (d + 2) floats.  Every token_pos must be
// below max_len: a token at or beyond it gets a row of NaN instead of a result.  q, the cache pages
// and out must start on 16-byte boundaries and q_stride must be a multiple of 8 elements, else the
// call is refused with ILLM_ERR_BAD_ARG.
//
// The scratch is one array in the library's device image, ILLM_STATIC_SCRATCH_BYTES (32 MiB)
// large and 256-byte aligned.  Every GPU on which this library is loaded holds those 32 MiB until
// the process exits.  A call that needs more is refused: the function returns
// ILLM_ERR_SCRATCH_TOO_SMALL and, if `err_msg` is not NULL, writes a sentence with both sizes
// into it (at most err_len bytes, NUL-terminated).  32 MiB is enough for 64 tokens x 32 heads at
// 4096 positions with head size 128.
//
// The function calls no cudaMalloc, cudaFree or allocating library routine.  The first call on
// each device looks up the array's device address (cudaGetSymbolAddress, with that device
// current) and keeps it; make that first call before any stream capture begins, since the lookup
// may load the module.  All calls share the one array and it keeps what the last call left.  The
// kernels write every partial result they later read, so nothing has to be cleared between
// calls; but two calls whose kernels overlap on the GPU (different streams, or a captured graph
// replayed next to a live call) race on the array and give wrong results.  Run them one after
// another on one stream.
//
// Returns 0, a cudaError_t of the launch, ILLM_ERR_BAD_ARG (10001) for sizes the kernel does not
// take, or ILLM_ERR_SCRATCH_TOO_SMALL (10002).
#pragma once

#define ILLM_STATIC_SCRATCH_BYTES (32u * 1024u * 1024u)
#define ILLM_ERR_SCRATCH_TOO_SMALL 10002

#ifdef __cplusplus
extern "C" {
#endif

int illm_attention_decode_static(const void* q, int q_stride, const void* kc, const void* vc,
                                 const int* block_table, int max_pages, const int* token_pos,
                                 const int* token_seq, void* out, int T, int nh, int nkv, int d,
                                 int page_size, int window, float scale, int max_len, char* err_msg,
                                 int err_len, void* stream);

#ifdef __cplusplus
}
#endif
