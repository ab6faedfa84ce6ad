// C prototypes of every kernel entry point of csrc/*.cu, for the C++ core (the kernels themselves
// are documented where they are defined).  Conventions: device pointers, dtype codes 0 = float32 and
// 1 = bfloat16, the last argument is the cudaStream_t; the result is 0, a cudaError_t of the launch or
// ILLM_ERR_BAD_ARG (10001) for sizes the kernel refuses.  Nothing here allocates or synchronises.
#pragma once

#ifdef __cplusplus
extern "C" {
#endif

// attention_decode.cu
int illm_attention_decode(const void* q, int q_stride, const void* kc, const void* vc, const int* block_table, int max_pages, const int* token_pos, const int* token_seq, float* part_acc, float* part_ml, void* out, int T, int nh, int nkv, int d, int page_size, int window, float scale, int n_chunks, void* stream);
int illm_attention_decode_merge(const float* part_acc, const float* part_ml, const int* token_pos, void* out, int T, int nh, int d, int n_chunks, int chunk_keys, int window, void* stream);
int illm_attention_decode_supported(int d, int g, int page_size);
int illm_attention_decode_static(const void* q, int q_stride, const void* kc, const void* vc, const int* block_table, int max_pages, const int* token_pos, const int* token_seq, void* out, int T, int nh, int nkv, int d, int page_size, int window, float scale, int max_len, char* err_msg, int err_len, void* stream);

// attention_decode_gqa.cu
int illm_attention_decode_gqa(const void* q, int q_stride, const void* kc, const void* vc, const int* block_table, int max_pages, const int* token_pos, const int* token_seq, float* part_acc, float* part_ml, void* out, int T, int nh, int nkv, int d, int page_size, int window, float scale, int n_chunks, void* stream);

// attention_decode_ring.cu
int illm_attention_decode_ring(const void* q, int q_stride, const void* kc, const void* vc, long long n_pages, const int* block_table, int max_pages, const int* token_pos, const int* token_seq, float* part_acc, float* part_ml, void* out, int T, int nh, int nkv, int d, int page_size, int window, float scale, int n_splits, int* err, void* stream);
int illm_attention_decode_ring_rope(const void* qkv, const float* partials, int splits, long long split_stride, const float* cos_sin, int rot, int table_positions, int write_kv, void* kc, void* vc, long long n_pages, const int* block_table, int max_pages, const int* token_pos, const int* token_seq, float* part_acc, float* part_ml, void* out, int T, int nh, int nkv, int d, int page_size, int window, float scale, int n_splits, int* err, int* step_err, void* stream);

// attention_generic.cu
int illm_attention_generic(const void* q, int q_stride, const void* kc, const void* vc, const int* block_table, int max_pages, const int* token_pos, const int* token_seq, void* out, int act_dtype, int T, int nh, int nkv, int d, int page_size, int window, float scale, void* stream);

// attention_prefill.cu
int illm_attention_prefill(const void* q, int q_stride, const void* kc, const void* vc, const int* block_table, int max_pages, const int* cu_q, const int* seq_lens, void* out, int B, int max_q, int nh, int nkv, int d, int page_size, int window, float scale, void* stream);

// attention_prefill_tc.cu
int illm_attention_prefill_tc(const void* q, int q_stride, int T, const void* kc, const void* vc, long long n_pages, const int* block_table, int max_pages, const int* cu_q, const int* seq_lens, void* out, int B, int max_q, int nh, int nkv, int d, int page_size, int window, float scale, int* err, void* stream);

// embedding.cu
int illm_embedding(const int* ids, const void* table, int table_dtype, float* out, int T, int H, int V, int* err, void* stream);
int illm_set_pdl(int on);
long long illm_launch_count();

// gemm_f32.cu
int illm_gemm_f32_nt(const float* A, const float* W, float* C, int M, int N, int K, int lda, int ldw, int ldc, int* err, void* stream);

// gemm_tc.cu
int illm_gemm_bf16_tc_tune(int stages);
int illm_gemm_bf16_tc(const void* X, const void* W, void* out, int out_dtype, int M, int N, int K, float* ws, int splits, int* err, void* stream, int skip_reduce);
int illm_gemm_bf16_tc_gated(const void* X, const void* W, void* out, int M, int N, int K, int* err, void* stream);
int illm_splitk_reduce(const float* ws, void* out, int out_dtype, long long n, int splits, void* stream);

// gemm_tc2.cu
int illm_gemm_bf16_tc2(const void* X, const void* W, void* out, int out_dtype, int epi, int M, int N, int K, int* err, void* stream);

// rmsnorm.cu
int illm_add_rmsnorm(float* resid, const void* delta, const void* w, int w_dtype, void* y, int act_dtype, const int* rows, int n_rows, int H, float eps, int write_resid, void* stream);
int illm_add_rmsnorm_partials(float* resid, const float* partials, int splits, long long split_stride, const void* w, int w_dtype, void* y, int act_dtype, const int* rows, int n_rows, int H, float eps, int write_resid, void* stream);
int illm_residual_add(float* resid, const void* delta, int act_dtype, long long n, void* stream);

// rope_kv.cu
int illm_rope_kv_write(void* qkv, const float* cos_sin, const int* token_pos, const int* token_seq, const int* block_table, int max_pages, void* kc, void* vc, int act_dtype, int T, int nh, int nkv, int d, int rot, int page_size, int write_kv, int table_positions, int* err, void* stream);
int illm_rope_kv_write_partials(void* qkv, const float* partials, int splits, long long split_stride, const float* cos_sin, const int* token_pos, const int* token_seq, const int* block_table, int max_pages, void* kc, void* vc, int act_dtype, int T, int nh, int nkv, int d, int rot, int page_size, int write_kv, int table_positions, int* err, void* stream);

// sampling.cu
int illm_argmax(const float* logits, int B, int V, int ld, int* out, float* scratch_v, int* scratch_i, void* stream);
long long illm_sample_scratch_elems(int B, int V, int top_k, float top_p);
int illm_sample(const float* logits, int B, int V, int ld, float* z_scratch, const int* last_tokens, int n_last, float temp, float penalty, int top_k, float top_p, const float* uniforms, int* out, int* scratch, void* stream);

// swiglu.cu
int illm_swiglu_partials(const float* slices, int P, long long stride, void* out, int T, int I, void* stream);
int illm_swiglu(const void* gu, void* out, int act_dtype, int T, int I, void* stream);

// utility.cu
int illm_fill_random(void* out, int dtype, long long n, unsigned long long key, float std, float mean, void* stream);
int illm_poison_pages(void* k, void* v, long long entry_stride_bytes, int n_entries, long long page_bytes, const int* pages, int n_pages, void* stream);
int illm_selftest_wait_timeout(int* err, long long* result, long long limit_clocks, int code, void* stream);
int illm_convert(const void* src, int src_dtype, void* dst, int dst_dtype, long long n, void* stream);
int illm_gather_i32(const int* src, const int* idx, int* dst, int n, void* stream);
int illm_window_gather(const int* window, int n_last, const int* rows, int* dst, int n, void* stream);
int illm_window_put(int* window, int n_last, const int* rows, int col, const int* toks, int n, void* stream);

#ifdef __cplusplus
}
#endif
