// C launchers exported by the CUDA sources (one declaration per entry point).
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

extern "C" {
// gemm_tcgen05.cu
int vb_gemm_bf16(const void* A, const void* B, void* D, const void* bias, int M, int N, int K, long long lda,
                 long long ldb, long long ldd, int a_mn, int b_mn, int out_f32, int accumulate, int max_ctas,
                 cudaStream_t stream);
int vb_gemm_bf16_ex(const void* A, const void* B, void* D, const void* bias, int M, int N, int K, long long lda,
                    long long ldb, long long ldd, int a_mn, int b_mn, int out_f32, int accumulate, int max_ctas, int k_splits,
                    float* splitk_ws, cudaStream_t stream);
int vb_gemm_bf16_fetch(const void* A, const void* B, void* D, const void* bias, int M, int N, int K, long long lda,
                       long long ldb, long long ldd, int a_mn, int b_mn, int out_f32, int accumulate,
                       const unsigned long long* src_ptrs, int world, unsigned long long dst, long long total_bytes,
                       long long slice_bytes, int chunk_begin, int chunk_end, long long b_off_bytes,
                       unsigned int* panel_counters, double limit_s, cudaStream_t stream);
int vb_gemm_bf16_splitk_allreduce(const void* A, const void* B, void* D, const void* bias, int M, int N, int K, long long lda,
                                  long long ldb, long long ldd, const unsigned long long* part_ptrs,
                                  const unsigned long long* flag_ptrs, unsigned int* epoch, long long buf_elems, int world, int rank,
                                  double limit_s, int k_splits, float* splitk_ws, int skinny, cudaStream_t stream);
int vb_gemm_skinny_splits(int M, int N, int K);
int vb_gemm_skinny_seg_splits(int M, int K, int nseg, const int* seg_w0, const int* seg_rows);
int vb_gemm_skinny_seg(const void* X, const void* W, void* D, const void* bias, int M, int K, int w_rows, long long ldx, long long ldw,
                       long long ldd, int nseg, const int* seg_w0, const int* seg_rows, int splits, float* ws, int ws_rows,
                       int partials_only, cudaStream_t stream);
int vb_gemm_skinny_status();
int vb_gemm_skinny(const void* X, const void* W, void* D, const void* bias, int M, int N, int K, long long ldx, long long ldw,
                   long long ldd, int splits, float* ws, int ws_rows, int partials_only, cudaStream_t stream);
int vb_gemm_bf16_allreduce_ex(const void* A, const void* B, void* D, const void* bias, int M, int N, int K, long long lda,
                             long long ldb, long long ldd, int b_mn, int rs_rows, const unsigned long long* part_ptrs,
                             const unsigned long long* flag_ptrs, unsigned int* epoch, long long buf_elems, int world, int rank,
                             double limit_s, cudaStream_t stream);
int vb_gemm_bf16_allreduce(const void* A, const void* B, void* D, const void* bias, int M, int N, int K, long long lda,
                           long long ldb, long long ldd, const unsigned long long* part_ptrs,
                           const unsigned long long* flag_ptrs, unsigned int* epoch, long long buf_elems, int world, int rank,
                           double limit_s, cudaStream_t stream);
int vb_gemm_grouped(int mode, const void* A, const void* B, void* D, int rows_cap, int M, int N, int K, long long lda, long long ldb,
                    long long ldd, int b_mn, int accumulate, int E, const int* tile_expert, const int* num_mtiles,
                    const int* seg_start, cudaStream_t stream);
int vb_gemm_bf16_swiglu(const void* A, const void* W, void* act, void* gu_out, int M, int I, int K, long long lda, long long ldw,
                        long long ldd, long long gu_ld, cudaStream_t stream);
int vb_gemm_suggest_splits(int M, int N, int K);
int vb_gemm_fold_in_kernel();
int vb_gemm_status();
int vb_lmhead_num_tiles(int V);
int vb_lmhead_fwd(const void* hidden, const void* weight, const long long* labels, float inv_temp, float* partial,
                  float* label_logit, float* logprob, float* entropy, float* lse, int T, int V, int H, long long ldh,
                  long long ldw, cudaStream_t stream);
int vb_lmhead_dlogits(const void* hidden, const void* weight_chunk, const long long* labels, int v0, float inv_temp,
                      const float* lse, const float* ex, const float* g_lp, const float* g_ent, void* dlogits, int T,
                      int Vc, int H, long long ldh, long long ldw, long long ldd, cudaStream_t stream);
// elementwise.cu
int vb_rmsnorm_fwd(const void* x, const void* residual, const void* w, void* y, void* res_out, float* rstd, int T,
                   int H, float eps, cudaStream_t s);
int vb_rmsnorm_bwd_blocks(int T);
int vb_rmsnorm_bwd(const void* dy, const void* x, const void* w, const float* rstd, const void* dres_in, void* dx,
                   float* dw, float* scratch, int T, int H, int accumulate_dw, cudaStream_t s);
int vb_rope(void* x, const int* pos, const float* cos_t, const float* sin_t, int T, int nheads, int hd, long long ld,
            int backward, cudaStream_t s);
int vb_swiglu_fwd(const void* gu, void* out, long long T, int I, cudaStream_t s);
int vb_swiglu_bwd(const void* dout, const void* gu, void* dgu, long long T, int I, cudaStream_t s);
int vb_embedding_fwd(const long long* ids, const void* w, void* out, int T, int H, int V, cudaStream_t s);
int vb_embedding_bwd(const long long* ids, const void* dout, float* dw, int T, int H, int V, cudaStream_t s);
int vb_sumsq(const float* g, long long n, float* ctrl, cudaStream_t s);
int vb_clip_coef(float* ctrl, float max_norm, cudaStream_t s);
int vb_adamw(float* master, float* grad, float* m, float* v, void* out_bf16, long long n, const float* ctrl, float lr,
             float beta1, float beta2, float eps, float wd, int step, float grad_scale, int zero_grad, cudaStream_t s);
int vb_cast_f32_bf16(const float* in, void* out, long long n, float scale, cudaStream_t s);
int vb_accum_bf16_f32(const void* in, float* out, long long n, float scale, int accumulate, cudaStream_t s);
// rollout_kernels.cu
int vb_kv_append(const void* k, const void* v, long long ldk, long long ldv, const long long* slot, void* kc, void* vc,
                 int T, int nkv, int hd, cudaStream_t s);
int vb_paged_decode(const void* q, long long ldq, const void* kc, const void* vc, const int* block_table,
                    int max_blocks, const int* ctx_len, void* out, long long ldo, int B, int nh, int nkv, int hd,
                    int block_size, float scale, cudaStream_t s);
int vb_paged_decode_grouped(const void* q, long long ldq, const void* kc, const void* vc, long long num_slots, const int* block_table,
                            int max_blocks, const int* ctx_len, const int* members, const int* grp_pages, const int* skip, int NG,
                            void* out, long long ldo, int B, int nh, int nkv, int hd, int block_size, float scale, int psplit,
                            int nsplit, float* part_o, float* part_ml, cudaStream_t stream);
int vb_rope_kv_append(void* qkv, long long ld, const int* pos, const float* cos_t, const float* sin_t, const long long* slot,
                      void* kc, void* vc, int T, int nh, int nkv, int hd, cudaStream_t s);
int vb_sample(const void* logits, long long ld, int B, int V, int valid_vocab, float inv_temp, const long long* seeds,
              long long step, long long* tokens, float* logprobs, cudaStream_t s);
int vb_sample_topkp(const void* logits, long long ld, int B, int V, int valid_vocab, float inv_temp, int top_k, float top_p,
                    const long long* seeds, long long step, long long* tokens, float* logprobs, cudaStream_t s);
// attention_fwd_tcgen05.cu
int vb_attn_fwd(const void* q, const void* k, const void* v, long long ldq, long long ldk, long long ldv,
                const int* cu_seqlens, int num_seqs, int total_tokens, int nh, int nkv, int hd, float scale, void* out,
                long long ldo, float* lse, cudaStream_t stream);
int vb_attn_status();
// attention_bwd_tcgen05.cu
int vb_attn_bwd(const void* q, const void* k, const void* v, const void* out, const void* dout, long long ldq, long long ldk,
                long long ldv, long long ldo, long long lddo, const float* lse, const int* cu_seqlens, int num_seqs,
                int total_tokens, int nh, int nkv, int hd, float scale, void* dq, void* dk, void* dv, long long lddq,
                long long lddk, long long lddv, float* delta_ws, float* dq32_ws, int max_seqlen, cudaStream_t stream);
int vb_attn_bwd_status();
// paged_decode_tma.cu
int vb_paged_decode_v2(const void* q, long long ldq, const void* kc, const void* vc, long long num_slots,
                       const int* block_table, int max_blocks, const int* ctx_len, void* out, long long ldo, int B, int nh,
                       int nkv, int hd, int block_size, float scale, int nsplit, float* part_o, float* part_ml,
                       cudaStream_t stream);
int vb_pd_status();
// comm_fused.cu
int vb_peer_barrier(const unsigned long long* pad_ptrs, int rank, int W, unsigned int epoch, double limit_s,
                    float* poison_on_timeout, cudaStream_t s);
int vb_rs_sumsq(const unsigned long long* grad_ptrs, unsigned long long mc_ptr, float* out, long long lo, long long n, int W,
                int rank, float scale, float* ctrl, cudaStream_t s);
int vb_adamw_allgather(float* master, const float* grad, float* m, float* v, const unsigned long long* param_ptrs,
                       unsigned long long mc_ptr, long long lo, long long n, int W, int rank, const float* ctrl, float lr,
                       float beta1, float beta2, float eps, float wd, int step, cudaStream_t s);
int vb_peer_share(const unsigned long long* buf_ptrs, const unsigned long long* flag_ptrs, unsigned int* epoch, const void* src,
                  void* out, int n, int cap, int rank, int W, double limit_s, cudaStream_t s);
int vb_scatter_copy(const void* jobs, const int* block_start, int njobs, int total_blocks, cudaStream_t s);
int vb_allreduce_peer(const unsigned long long* buf_ptrs, void* out, long long n, int W, int rank, cudaStream_t s);
int vb_comm_status();
// gemm_fp8_blockscale.cu
int vb_nvfp4_fake_quant(const void* x, long long ldx, void* y, long long ldy, long long rows, int cols, float global_scale,
                        cudaStream_t s);
int vb_fp8_quant_1x128(const void* x, long long ldx, void* q, long long ldq, float* scales, int R, int C, cudaStream_t s);
int vb_gemm_fp8_blockscale(const void* Aq, const float* sa, const void* Bq, const float* sb, void* D, const void* bias, int M, int N,
                           int K, long long lda, long long ldb, long long ldd, cudaStream_t stream);
int vb_gemm_fp8_blockscale_grouped(const void* Aq, const float* sa, const void* Bq, const float* sb, void* D, int rows_cap, int N, int K,
                                   int E, long long lda, long long ldb, long long ldd, const int* tile_expert, const int* num_mtiles,
                                   cudaStream_t s);
int vb_fp8_quant_128x128(const void* w, long long ldw, void* q, long long ldq, float* scale_inv, int R, int C, cudaStream_t s);
int vb_fp8_status();
// moe_kernels.cu
int vb_moe_route_topk(const void* logits, long long ld, int T, int E, int k, int renorm, float* weights, int* experts, int* counts,
                      cudaStream_t s);
int vb_moe_gather_rows(const void* src, long long lds, const int* map, const float* scale, void* dst, long long ldd, int rows, int H,
                       cudaStream_t s);
int vb_moe_combine(const void* y, long long ldy, const int* slot, const float* w, void* out, long long ldo, int T, int H, int k,
                   cudaStream_t s);
int vb_moe_combine_bwd_w(const void* g, long long ldg, const void* y, long long ldy, const int* slot, float* gw, int T, int H, int k,
                         cudaStream_t s);
int vb_moe_dispatch_peer(const void* src, long long lds, const unsigned long long* dst_ptrs_dev, const int* dest_rank, const int* dest_row,
                         int pairs, int k, int H, cudaStream_t s);
int vb_moe_combine_peer(const unsigned long long* y_ptrs_dev, const int* src_rank, const int* src_row, const float* w, void* out,
                        long long ldo, int T, int H, int k, cudaStream_t s);
int vb_moe_publish_counts(const int* counts, const unsigned long long* table_ptrs_dev, int W, int rank, int E, cudaStream_t s);
// advantage.cu
int vb_grpo_advantage(const float* rewards, const float* mask, const int* group, int B, int L, int num_groups,
                      float eps, int norm_by_std, float* scores, float* stats, float* adv, cudaStream_t s);
int vb_gae(const float* rewards, const float* values, const float* mask, int B, int L, float gamma, float lam,
           int whiten, float* adv, float* ret, float* acc, cudaStream_t s);
}
