// C entry points of the kernel library.  Pointers are device pointers; `stream` is
// the CUDA stream the caller works on.  Each returns 0 on success, a cudaError_t
// (> 0) if the launch failed, or -1 if it refuses the sizes, with the reason in
// zi_last_error().  dtype tags: 0 = float32, 1 = bfloat16.
#pragma once
#include <cuda_runtime.h>

#ifdef __cplusplus
extern "C" {
#endif

const char* zi_last_error();

int zi_embed_gather(float* h, const void* table, int table_dtype, const int* ids, int T, int H, int V,
                    cudaStream_t stream);
int zi_add_rmsnorm(float* h, const void* delta, int delta_dtype, const float* delta_partials, int splits,
                   long long split_stride, const float* w, float eps, void* out, int out_dtype, const int* rows,
                   int n_rows, int H, cudaStream_t stream);
int zi_residual_add(float* h, const void* delta, int delta_dtype, long long n, cudaStream_t stream);
int zi_residual_add_partials(float* h, const float* partials, int splits, long long split_stride, long long n,
                             cudaStream_t stream);
int zi_patch_tokens(int* ids, const int* prev, const int* dst, const int* src, int n, cudaStream_t stream);
int zi_swiglu(void* out, const void* gu, int dtype, int T, int I, int interleave, cudaStream_t stream);
int zi_swiglu_partials(void* out, int dtype, const float* partials, int splits, long long split_stride, int T, int I,
                       int interleave, cudaStream_t stream);
int zi_gemm_tcgen05_swiglu(void* out, int out_dtype, const void* x, const void* w, int M, int N2, int K, int ldx,
                           int ldw, int ldo, int sm_count, cudaStream_t stream);
int zi_gemm_argmax_units(int N);
int zi_gemm_tcgen05_argmax(float* out, const void* x, const void* w, int M, int N, int K, int ldx, int ldw, int ldo,
                           float* cand_val, int* cand_idx, int sm_count, cudaStream_t stream);
int zi_rope_table(float* cos_t, float* sin_t, int n_pos, int d, float theta, cudaStream_t stream);
int zi_qk_norm_rope_store(const void* src, int dtype, int T, int src_stride, const float* partials, int splits,
                          long long split_stride, void* q_out, int q_stride, int nq, int nkv, int d, const float* qw,
                          const float* kw, float eps, const float* cos_t, const float* sin_t, int n_table_pos,
                          const int* positions, void* kcache, void* vcache, const int* slots, int page_size,
                          int write_kv, cudaStream_t stream);

int zi_gemm_simt(void* out, int out_dtype, const void* x, int x_dtype, const void* w, int w_dtype, int M, int N,
                 int K, int ldx, int ldw, int ldo, cudaStream_t stream);

int zi_gemm_tcgen05_supported(const void* x, const void* w, int K, int ldx, int ldw);
long long zi_gemm_tcgen05_plan(int M, int N, int K, int sm_count, int* plan);
int zi_gemm_tcgen05(void* out, int out_dtype, const void* x, const void* w, int M, int N, int K, int ldx, int ldw,
                    int ldo, float* workspace, long long workspace_bytes, int sm_count, int defer_reduce,
                    cudaStream_t stream);
int zi_gemm_tcgen05_status();
int zi_gemm_tcgen05_pair_enable(int on);

int zi_paged_attention_tile_rows();
int zi_paged_attention(void* out, int out_stride, const void* q, int q_stride, int dtype, const void* kcache,
                       const void* vcache, const int* block_tables, int bt_stride, const int* cu_q,
                       const int* kv_lens, const int* tile_seq, const int* tile_q0, int n_tiles, int nq, int nkv,
                       int d, int page_size, int window, float scale, cudaStream_t stream);

int zi_attention_prefill_tile_rows();
int zi_attention_mma_supported(int nq, int nkv, int d, int decode);
int zi_attention_prefill_mma(void* out, int out_stride, const void* q, int q_stride, const void* kcache,
                             const void* vcache, const int* block_tables, int bt_stride, const int* cu_q,
                             const int* kv_lens, const int* tile_seq, const int* tile_q0, int n_tiles, int nq, int nkv,
                             int d, int page_size, int window, float scale, cudaStream_t stream);
int zi_attention_prefill_tcgen05_supported(int nq, int nkv, int d, int page_size, const void* q, int q_stride,
                                           const void* kcache, const void* vcache);
int zi_attention_prefill_tcgen05(void* out, int out_stride, const void* q, int q_stride, int n_tokens,
                                 const void* kcache, const void* vcache, long long n_pages, const int* block_tables,
                                 int bt_stride, const int* cu_q, const int* kv_lens, const int* tile_seq,
                                 const int* tile_q0, int n_tiles, int nq, int nkv, int d, int page_size, int window,
                                 float scale, cudaStream_t stream);
long long zi_attention_decode_workspace_floats(int n_dec, int nq, int nkv, int d, int splits);
int zi_attention_decode_mma(void* out, int out_stride, float* workspace, const void* q, int q_stride,
                            const void* kcache, const void* vcache, long long n_pages, const int* block_tables, int bt_stride,
                            const int* cu_q, const int* kv_lens, const int* dec_seq, int n_dec, int nq, int nkv, int d,
                            int page_size, int window, float scale, int splits, cudaStream_t stream);

int zi_attention_decode_fused(void* out, int out_stride, float* workspace, const void* qkv, int qkv_stride,
                              const float* partials, int part_splits, long long part_zstride, const float* qw,
                              const float* kw, float eps, const float* cos_t, const float* sin_t, int n_table_pos,
                              const int* positions, const int* slots, void* kcache, void* vcache, long long n_pages,
                              const int* block_tables, int bt_stride, const int* cu_q, const int* kv_lens,
                              const int* dec_seq, int n_dec, int nq, int nkv, int d, int page_size, int window,
                              float scale, int splits, cudaStream_t stream);

int zi_argmax_chunks(int R, int V);
int zi_argmax(int* out, const float* logits, int R, int V, int ld, void* workspace, cudaStream_t stream);
int zi_argmax_candidates(int* out, const float* cand_val, const int* cand_idx, int R, int units, cudaStream_t stream);
int zi_sample_ctas_per_row(int R, int sm_count);
int zi_sample(int* out, const float* logits, int R, int V, int ld, const float* temperature, const int* top_k,
              const float* top_p, const float* min_p, const float* rep, const float* pres, const float* freq,
              const int* count_rows, int* counts, const unsigned long long* seeds, const int* draw_index,
              cudaStream_t stream);
int zi_count_tokens(int* counts, const int* tokens, int n, int V, cudaStream_t stream);

#ifdef __cplusplus
}
#endif
