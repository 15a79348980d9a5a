// C entry points of this library's kernels, as the native step executor calls them.
//
// Every function launches on the given stream without synchronising and returns 0 or one of the MM_ERR_* codes
// (common.cuh); the message of the last error is mm_last_error().  The Python binding declares the same
// prototypes for ctypes (kernels/lib.py, kernels/attention_bf16.py).
#pragma once

extern "C" {
const char* mm_last_error();

// elementwise.cu
int mm_embedding(const void* ids, const void* table, int table_dtype, void* out, int n_tokens, int vocab, int d, float scale,
                 void* stream);
int mm_add_rmsnorm(void* residual, const void* delta, const void* rows, const void* weight, int weight_dtype, void* out,
                   int act_dtype, int n_rows, int d, float eps, void* stream);
int mm_add_residual(void* residual, const void* delta, int act_dtype, long long n, void* stream);
int mm_silu_mul(const void* gu, void* out, int act_dtype, int n, int F, int interleave, void* stream);
int mm_qkv_rope_tables(const void* qkv, const void* bias, int bias_dtype, void* q_out, void* k_pages, void* v_pages,
                       const void* rope_table, const void* slots, int page_size, int n_tokens, int H, int G, int hd,
                       int interleave, void* stream);
int mm_qkv_rope_kvwrite(const void* qkv, const void* bias, int bias_dtype, void* q_out, void* k_pages, void* v_pages,
                        int act_dtype, const void* positions, const void* token_req, const void* block_table, int table_width,
                        int page_size, int n_tokens, int H, int G, int hd, int rotary_dim, float theta_base, int interleave,
                        void* stream);
int mm_rope_table(const void* positions, void* out, int n_tokens, int dim, float theta_base, void* stream);
int mm_slot_mapping(const void* positions, const void* token_req, const void* block_table, int table_width, int page_size,
                    int n_tokens, void* out, void* stream);

// matrix products
int mm_gemm_simt(const void* A, int a_dtype, const void* W, int w_dtype, const void* bias, int bias_dtype, void* C, int c_dtype,
                 int M, int N, int K, int lda, int ldc, void* stream);
int mm_gemv_bf16(const void* W, const void* x, const void* bias, int bias_dtype, void* out, int out_dtype, int M, int N, int K,
                 int ldx, int ldo, int rt, int ks, int swiglu, const void* in_ss, int in_tiles, int in_dim, float in_eps,
                 void* stream);
int mm_gemv_bf16_residual(const void* W, const void* x, void* residual, const void* norm_w, int norm_w_dtype, void* xw_out,
                          void* out_ss, int M, int N, int K, int ldx, int rt, int ks, const void* in_ss, int in_tiles,
                          int in_dim, float in_eps, void* stream);
int mm_gemv_bf16_qkv_rope(const void* W, const void* x, const void* bias, int bias_dtype, void* q_out, void* k_pages,
                          void* v_pages, const void* rope_table, const void* slots, int page_size, int H, int G, int hd, int M,
                          int K, int ldx, int rt, int ks, const void* in_ss, int in_tiles, int in_dim, float in_eps,
                          void* stream);
int mm_gemm_skinny(const void* W, const void* x, const void* bias, int bias_dtype, void* out, int out_dtype, int M, int N,
                   int K, int ldx, int ldo, int splits, int swiglu, const void* in_ss, int in_tiles, int in_dim, int in_ld,
                   float in_eps, void* err, void* stream);
int mm_gemm_skinny_residual(const void* W, const void* x, void* residual, const void* norm_w, int norm_w_dtype, void* xw_out,
                            void* out_ss, int out_ld, int M, int N, int K, int ldx, int splits, const void* in_ss,
                            int in_tiles, int in_dim, int in_ld, float in_eps, void* err, void* stream);
int mm_gemm_skinny_qkv_rope(const void* W, const void* x, const void* bias, int bias_dtype, void* q_out, void* k_pages,
                            void* v_pages, const void* rope_table, const void* slots, int page_size, int H, int G, int hd,
                            int M, int K, int ldx, int splits, const void* in_ss, int in_tiles, int in_dim, int in_ld,
                            float in_eps, void* err, void* stream);
int mm_gemm_tcgen05(const void* A, const void* W, const void* bias, int bias_dtype, void* out, int epilogue, int M, int N,
                    int K, int lda, int ldo, void* err, void* stream);
int mm_gemm_tcgen05_pair(const void* A, const void* W, const void* bias, int bias_dtype, void* out, int epilogue, int M, int N,
                         int K, int lda, int ldo, void* err, void* stream);

// attention
int mm_attention_generic(const void* q, const void* k_pages, const void* v_pages, void* out, int dtype, const void* positions,
                         const void* token_req, const void* block_table, int table_width, int page_size, int n_tokens, int H,
                         int G, int hd, int window, float scale, void* stream);
int mm_attention_prefill_bf16(const void* q, const void* k_pages, const void* v_pages, void* out, const void* tiles,
                              int n_tiles, const void* block_table, int table_width, int page_size, int H, int G, int hd,
                              int window, float scale, void* stream);
int mm_attention_prefill_tcgen05(const void* q, const void* k_pages, const void* v_pages, void* out, const void* tiles,
                                 int n_tiles, const void* block_table, int table_width, int page_size, int num_pages,
                                 int n_tokens, int H, int G, int hd, int window, float scale, void* err, void* stream);
int mm_attention_decode_tma_bf16(const void* q, const void* k_pages, const void* v_pages, void* out, void* part_o, void* part_ml,
                                 const void* items, int n_items, const void* positions, const void* token_req,
                                 const void* block_table, int table_width, int page_size, int num_pages, int H, int G, int hd,
                                 int window, float scale, int split_len, int max_splits, int stages, int cluster, void* err,
                                 void* stream);
int mm_attention_decode_tma_max_clusters(int hd, int cluster_size, int* out);
int mm_attention_decode_bf16(const void* q, const void* k_pages, const void* v_pages, void* out, void* part_o, void* part_ml,
                             const void* items, int n_items, const void* positions, const void* token_req,
                             const void* block_table, int table_width, int page_size, int H, int G, int hd, int window,
                             float scale, int split_len, int max_splits, void* stream);
int mm_attention_decode_merge_bf16(void* out, const void* part_o, const void* part_ml, const void* items, int n_items,
                                   const void* positions, int H, int hd, int window, int split_len, int max_splits,
                                   void* stream);

// sampling.cu
int mm_argmax_rows(const void* logits, void* out, int R, int V, void* stream);
int mm_argmax_rows_split(const void* logits, void* out, void* part_val, void* part_idx, int R, int V, int P, void* stream);
int mm_sample_rows(const void* logits, void* out, int R, int V, const void* temperature, const void* top_k, const void* top_p,
                   const void* seeds, const void* counters, void* stream);
int mm_window_push(void* recent, int R, int W, const void* widths, void* lengths, const void* tokens, void* stream);
int mm_advance_step(void* positions, void* counters, void* next_ids, const void* tokens, int n, void* stream);
int mm_apply_penalties(void* logits, int R, int V, const void* recent, int W, const void* rep, const void* freq,
                       const void* pres, const void* softcap, void* stream);
}
