// The C interface through which a part is written in another language (the Python package offers base
// classes over it, inferllm_b200/extend.py): a table of callbacks per family, registered under a kind
// like any part of the library.  Tensors, activations and cache storage are device pointers; the
// library allocates a part's tensors and its outputs, the callbacks fill or read them on the stream
// of the step.
#pragma once

#ifdef __cplusplus
extern "C" {
#endif

// What a part sees of a step.  Device arrays are int32; the host arrays have B entries.
typedef struct illm_step_info {
    int T, B, K, max_q, is_decode;
    long long max_len, max_seq_len;
    const int *ids, *token_pos, *token_seq, *want_rows, *slots, *seq_lens, *cu_q;     /* device */
    const int* q_lens;                                                             /* host */
    const int* host_slots;                                                         /* host */
    const long long* past;                                                         /* host */
    int* err;           /* the step's error word (device) */
    void* stream;       /* cudaStream_t of the step */
    int dtype;          /* compute dtype: 0 float32, 1 bfloat16 */
    int page_size;
} illm_step_info;

// A mixer's cache entry for the step.  kind: 0 none, 1 keys and values, 2 fixed state.
typedef struct illm_cache_info {
    int kind;
    void *k, *v;                /* [pages, kv heads, page_size, head_dim] */
    const int* block_table;     /* device int32 [B, width] */
    int width, num_pages, page_size, window, n_kv_heads, head_dim, dtype, writes;
    void* state;                /* [slots, elements] */
    const int* slots;           /* device int32 [B] */
    int num_slots;
    long long elements;
    int state_dtype;
} illm_cache_info;

// Callbacks return 0, or non-zero after having recorded their own error.
typedef struct illm_foreign_part {
    void* user;
    // JSON text, valid until the next call: {"tensors": [[name, [shape], init], ...], "cache": null |
    // {"kind": "kv", "n_kv_heads", "head_dim", "window"} | {"kind": "state", "shape", "dtype"},
    // "graph_safe": bool, "pad_safe": bool, "takes_partials": bool} or {"error": "..."}
    const char* (*describe)(void* user, const char* spec_json);
    int (*create)(void* user, const char* spec_json, int dtype, int on_device, long long* instance);
    void (*destroy)(void* user, long long instance);
    // one of the part's tensors: on the device, in the dtype the storage rule keeps it in; the memory
    // stays valid as long as the instance lives
    int (*load)(void* user, long long instance, const char* name, void* ptr, int dtype, const long long* shape, int ndim);
    // mixer: h [T, H] -> out [T, H], both in the compute dtype
    int (*mixer_forward)(void* user, long long instance, const illm_step_info* step, const illm_cache_info* cache, const void* h, void* out,
                         long long T, long long H, int writes);
    // feed-forward: h [T, H] -> out [T, H]
    int (*ffn_forward)(void* user, long long instance, const illm_step_info* step, const void* h, void* out, long long T, long long H);
    // position encoding: encode Q and K heads of qkv [T, width] in place and store K, V (if cache->writes)
    int (*encode_and_store)(void* user, long long instance, const illm_step_info* step, const illm_cache_info* cache, void* qkv, long long T,
                            long long width, int n_heads, int n_kv_heads, int head_dim);
} illm_foreign_part;

// family: "mixer", "feed_forward" or "position".
int illm_register_foreign_part(const char* family, const char* kind, const illm_foreign_part* table);
int illm_unregister_part(const char* family, const char* kind);

#ifdef __cplusplus
}
#endif
