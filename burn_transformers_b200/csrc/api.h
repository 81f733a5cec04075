// C interface of the kernel library.  Every function returns 0 on success; otherwise
// bt_last_error() holds the reason.  dtype codes: 0 = float32, 1 = bfloat16.
#pragma once
#include <cuda_runtime.h>

extern "C" {
const char* bt_last_error();
int bt_abi_version();
long long bt_launch_count();

// Fills `out` (128 bytes) with a tensor map of a rows x cols bfloat16 tensor (rows `row_stride` elements apart)
// that is copied in boxes of box_rows x 64 columns with the 128-byte swizzle.
int bt_tensor_map_2d_bf16(void* out, const void* base, unsigned long long rows, unsigned long long cols,
                          unsigned long long row_stride, unsigned box_rows);

int bt_embed(const int* tokens, const int* positions, const void* wte, const void* wpe, float* out, int n_tokens,
             int width, int vocab, int n_positions, int dtype, int* status, cudaStream_t stream);

int bt_layernorm(const float* x, const int* rows, const float* gamma, const float* beta, void* out, int n_rows,
                 int width, float eps, int out_dtype, cudaStream_t stream);

int bt_linear_simt(const void* A, const void* W, const float* bias, const float* residual, void* out, int M, int N,
                   int K, int w_is_nk, int act, int in_dtype, int out_dtype, cudaStream_t stream);

int bt_kv_append(const void* proj, long long row_stride, int k_offset, int v_offset, const int* positions,
                 const int* token_seq, const int* ctx_len, const int* table, int table_stride, int table_len,
                 int page_size, void* k_pool, void* v_pool, int n_tokens, int n_kv_heads, int head_dim, int dtype,
                 cudaStream_t stream);

int bt_attention_prefill_simt(const void* q, long long q_row_stride, const void* k, const void* v,
                              const int* kv_table, int table_stride, int table_len, int page_size,
                              long long kv_row_stride, void* out, const int* seq_start, const int* past_len,
                              int n_seqs, int max_new, int n_heads, int n_kv_heads, int head_dim, float scale,
                              int causal, int window, int dtype, cudaStream_t stream);

int bt_attention_prefill_tcgen05_supports(int head_dim, int page_size);
int bt_attention_prefill_tcgen05(const void* q, long long q_rows, long long q_row_stride, const void* k, const void* v,
                                 long long pool_pages, const int* kv_table, int table_stride, int table_len, int page_size,
                                 void* out, int* status, const int* seq_start, const int* past_len, int n_seqs, int max_new,
                                 int n_heads, int n_kv_heads, int head_dim, float scale, int causal, int window,
                                 cudaStream_t stream);

long long bt_attention_decode_scratch_floats(int n_seqs, int n_heads, int head_dim, int n_splits);
// out[M, N] = act(a[M, K] @ w[N, K]^T + bias) (+ residual) for at most 64 bfloat16 rows (made for 17..64).
int bt_linear_mid_supports(int M, int N, int K);
int bt_linear_mid(const void* a, const void* w, const float* bias, const float* residual, void* out, int* status, int M, int N,
                  int K, int act, int out_is_f32, int split, cudaStream_t stream);

// Decode attention on tensor cores (bfloat16, head sizes 16..128 in steps of 16): arguments as bt_attention_decode,
// plus the number of pages of the pools.
int bt_attention_decode_mma_supports(int head_dim);
int bt_attention_decode_mma(const void* q, long long q_row_stride, const void* new_k, const void* new_v, void* k_pool,
                            void* v_pool, long long pool_pages, const int* kv_table, int table_stride, int table_len,
                            void* out, float* scratch, int* tickets, int* status, const int* ctx_len, int n_seqs,
                            int n_heads, int n_kv_heads, int head_dim, float scale, int window, int n_splits, int max_ctx,
                            int merge, cudaStream_t stream);

int bt_attention_decode(const void* q, long long q_row_stride, const void* new_k, const void* new_v, void* k_pool,
                        void* v_pool, const int* kv_table, int table_stride, int table_len, int page_size, void* out,
                        float* scratch, int* tickets, int* status, const int* ctx_len, int n_seqs, int n_heads,
                        int n_kv_heads, int head_dim, float scale, int window, int n_splits, int max_ctx, int merge,
                        int dtype, cudaStream_t stream);

int bt_sample(const float* logits, long long row_stride, int n_rows, int vocab, int do_sample, float temperature,
              int top_k, float top_p, float min_p, const float* uniforms, const unsigned long long* stream_seeds,
              const int* counters, int* out_ids, float* out_logp, cudaStream_t stream);
int bt_advance(const int* ids, int* tokens, int* positions, int* past_len, int* ctx_len, int* counters, int n,
               cudaStream_t stream);
int bt_linear_tcgen05_supports(int M, int N, int K);
int bt_linear_tcgen05(const void* a, const void* w, const float* bias, const float* residual, void* out, int* status,
                      int M, int N, int K, int act, int out_is_f32, cudaStream_t stream);
// out[M, N] = act(x[M, K] @ w[N, K]^T + bias) (+ residual) for at most 128 bfloat16 rows over large weights, on the
// tcgen05 tensor cores with the weights on their M side; split: blocks per cluster along K (0: chosen from the shape).
int bt_linear_few_tcgen05_supports(int M, int N, int K);
int bt_linear_few_tcgen05(const void* x, const void* w, const float* bias, const float* residual, void* out, int* status,
                          int M, int N, int K, int act, int out_is_f32, int split, cudaStream_t stream);
int bt_linear_stream_supports(int M, int N, int K, int fuse_ln);
int bt_linear_stream(const void* a, const float* x32, const int* rows, const float* gamma, const float* beta, float eps,
                     const void* w, const float* bias, const float* residual, void* out, int M, int N, int K, int act,
                     int out_is_f32, int warps_k, cudaStream_t stream);
int bt_linear_skinny_supports(int M, int N, int K, int w_is_nk, int fuse_ln);
int bt_linear_skinny(const void* a, const float* x32, const int* rows, const float* gamma, const float* beta, float eps,
                     const void* w, const float* bias, const float* residual, void* out, int M, int N, int K,
                     int w_is_nk, int act, int out_is_f32, int split, cudaStream_t stream);
int bt_logit_edits(float* logits, long long row_stride, const int* rows, const int* tokens, const float* vals,
                   int n_edits, int vocab, cudaStream_t stream);
}
