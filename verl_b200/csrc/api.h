// C entry points of the sm_100a kernel library (no libtorch dependency). All functions return 0 on success and a
// negative code for rejected arguments; kernels with device-side waits report run-time failures through `err_word`.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

void vb_gemm_plan(int M, int N, int K, int b_mn, int bn_req, int* bn, int* split_k);
int vb_gemm_bf16(const void* A, const void* B, void* C, const void* bias, int M, int N, int K, int lda, int ldb, int ldc,
                 int a_mn, int b_mn, int out_f32, int accumulate, int bn, int split_k, float* split_ws, int* err_word,
                 cudaStream_t stream);

int vb_rmsnorm_fwd(const void* x, const void* res, const void* w, void* y, void* res_out, float* rstd, int T, int H,
                   float eps, cudaStream_t st);
int vb_rmsnorm_bwd(const void* dy, const void* x, const void* w, const float* rstd, const void* dres, void* dx, float* dw,
                   int T, int H, cudaStream_t st);
int vb_rope(void* x, const int* pos, const float* cs, const float* sn, int T, int nheads, int D, long ld, float sign,
            cudaStream_t st);
int vb_segment_sum_rows(const void* g, const long* order, const long* offsets, void* out, long U, int C, cudaStream_t st);
int vb_swiglu_fwd(const void* gu, void* out, long T, int I, cudaStream_t st);
int vb_swiglu_bwd(const void* gu, const void* dout, void* dgu, long T, int I, cudaStream_t st);
int vb_adamw(float* p32, float* m, float* v, const void* g, int g_is_bf16, void* p16, long n, float lr, float b1, float b2,
             float eps, float wd, int step, const float* scalars, cudaStream_t st);
int vb_sqnorm(const void* g, int is_bf16, long n, float* out, cudaStream_t st);
int vb_clip_coef(const float* sumsq, float max_norm, float* scalars, cudaStream_t st);

int vb_kv_cache_write(const void* k, const void* v, long ld, const long* slots, void* cache, int n_kv_heads, long T,
                      cudaStream_t st);
int vb_sample(const void* logits, int is_bf16, long ld, int B, int V, float temperature, int top_k, float top_p,
              const long* rng, const int* row_ids, long* out_token, float* out_logprob, cudaStream_t st);

long vb_lmhead_scratch_floats(int M, int V);
int vb_lmhead_logprob_fwd(const void* h, const void* W, const long* labels, int M, int V, int K, int ldh, int ldw,
                          float inv_temp, float* scratch, float* logp, float* ent, float* lse, int* err_word,
                          cudaStream_t stream);
int vb_lmhead_dlogits(const void* h, const void* W, const long* labels, int M, int Vc, int K, int ldh, int ldw, float inv_temp,
                      int col_offset, const float* lse, const float* ent, const float* g_lp, const float* g_ent, void* dlogits,
                      int ldd, int* err_word, cudaStream_t stream);

int vb_attn_varlen_fwd(const void* q, const void* k, const void* v, long ld, int T, int n_q_heads, int n_kv_heads,
                       const void* tiles, int n_tiles, void* out, long ld_out, float* lse, long lse_stride, float scale,
                       int* err_word, cudaStream_t st);
int vb_attn_paged_decode(const void* q, long ld_q, const void* cache, long num_blocks, const int* block_table, int max_blocks,
                         const int* kv_lens, int B, int n_q_heads, int n_kv_heads, void* out, long ld_out, float scale,
                         int num_splits, int max_kv_len, float* part_o, float* part_ml, int* err_word, cudaStream_t st);
int vb_attn_decode_gqa(const void* q, long ld_q, const void* cache, long num_blocks, const int* block_table, int max_blocks,
                       const int* kv_lens, int B, int n_q_heads, int n_kv_heads, void* out, long ld_out, float scale,
                       int num_splits, int max_kv_len, float* part_o, float* part_ml, int* err_word, cudaStream_t st);
int vb_attn_varlen_bwd(const void* q, const void* k, const void* v, long ld, const void* dO, const void* O, long ld_o, int T,
                       int n_q_heads, int n_kv_heads, const void* tiles, int n_tiles, const float* lse, float* delta,
                       long stat_stride, float* dq_acc, void* dq, void* dk, void* dv, long ld_d, float scale, int* err_word,
                       cudaStream_t st);

int vb_gemm_allgather(int which, const long* seg_ptrs, int world, int seg_rows, int ld_seg, const void* other, int ld_other, void* C,
                      const void* bias, int M, int N, int K, int ldc, int rank, void* stage, int* stage_flags, int stage_epoch, int b_mn,
                      int* err_word, cudaStream_t st);
int vb_gemm_peer_scatter(const void* A, const void* B, int M, int N, int K, int lda, int ldb, int ld_slot, const long* out_ptrs,
                         int rank, int world, int rows_per_owner, long slot_elems, int b_mn, int* err_word, cudaStream_t st);
int vb_slots_reduce(const void* slots, int world, long slot_elems, long rows, int cols, int ld, const void* residual, void* out,
                    int ld_out, cudaStream_t st);
long vb_symm_alloc(long nbytes);
int vb_symm_free(long ptr);
int vb_ipc_get_handle(long ptr, unsigned char* out64);
long vb_ipc_open_handle(const unsigned char* in64);
int vb_ipc_close(long ptr);
int vb_symm_barrier(const long* pad_ptrs, int rank, int world, int epoch, int* err_word, cudaStream_t st);
int vb_symm_barrier_auto(const long* pad_ptrs, int rank, int world, int* err_word, cudaStream_t st);
int vb_symm_reduce_scatter(const long* grad_ptrs, int world, long shard_off, long n, float scale, float* out, float* sumsq,
                           cudaStream_t st);
int vb_symm_adamw_allgather(float* p32, float* m, float* v, const float* g, const long* param_ptrs, int world, long shard_off,
                            long n, float lr, float b1, float b2, float eps, float wd, int step, const float* scalars,
                            cudaStream_t st);

int vb_gemm_bf16_pair(const void* A, const void* B, void* C, const void* bias, int M, int N, int K, int lda, int ldb, int ldc, int a_mn,
                      int b_mn, int out_f32, int accumulate, int* err_word, cudaStream_t stream);
int vb_fp8_block_cast(const void* x, long ldx, void* y, long ldy, float* scale, int M, int N, cudaStream_t st);
int vb_gemm_head_scatter(const void* A, const void* B, const void* bias, int M, int N, int K, int lda, int ldb, int ld_out, const long* out_ptrs,
                         int world, int row_off, int head_dim, const int* head_rank, const int* head_slot, int b_mn, int* err_word, cudaStream_t st);
int vb_gemm_kseg(const long* seg_ptrs, int world, int k_per_rank, int ld_seg, int rows_total, int row_off, const void* B, int ldb, void* C,
                 const void* bias, int M, int N, int ldc, int rank, void* stage, int* stage_flags, int stage_epoch, int b_mn,
                 int* err_word, cudaStream_t st);
int vb_fp8_row_cast(const void* x, long ldx, void* y, long ldy, float* scale, long M, int K, cudaStream_t st);
int vb_gemm_fp8_pair(const void* A, const void* B, void* C, const void* bias, const float* a_scale, const float* b_scale, int M, int N, int K,
                     int lda, int ldb, int ldc, int out_f32, int* err_word, cudaStream_t stream);
int vb_gemm_fp8_block(const void* A, const void* B, void* C, const float* a_scale, const float* b_scale, const void* bias, int M, int N, int K,
                      int lda, int ldb, int ldc, int out_f32, int* err_word, cudaStream_t stream);
int vb_gemm_pair_plan(int M, int N, int K);
int vb_gemm_pair512_ok(const void* C, int ldc, int out_f32, int accumulate);
int vb_gemm_bf16_pair512(const void* A, const void* B, void* C, const void* bias, int M, int N, int K, int lda, int ldb, int ldc, int a_mn,
                         int b_mn, int out_f32, int accumulate, int* err_word, cudaStream_t stream);
int vb_gemm_bf16_pair_splitk(const void* A, const void* B, void* C, const void* bias, int M, int N, int K, int lda, int ldb, int ldc, int out_f32,
                             int accumulate, int split_k, float* split_ws, int* err_word, cudaStream_t stream);
void vb_allreduce_plan(int M, int N, int K, int* bn, int* split_k);
int vb_gemm_allreduce_sig(const void* A, const void* B, int M, int N, int K, int lda, int ldb, const long* out_ptrs, const long* sig_ptrs,
                          int rank, int world, long slot_elems, long half_elems, int bn, int split_k, int* err_word, cudaStream_t st);
int vb_slots_reduce_sig(const long* slot_ptrs, const void* sig, int rank, int world, int split_k, long slot_elems, long half_elems, long rows,
                        int cols, const void* residual, void* out, int ld_out, int* err_word, cudaStream_t st);
int vb_gemm_grouped(const void* A, const void* B, void* C, const int* blk_expert, int R, int N, int K, int E, int lda, int ldc, int b_mn,
                    int* err_word, cudaStream_t stream);
int vb_gemm_grouped_dispatch(const long* src_ptrs, int world, int ld_src, const int* row_src, const void* B, void* C, const int* blk_expert,
                             int R, int N, int K, int E, int ldc, int b_mn, void* stage, int* stage_flags, int* err_word, cudaStream_t stream);
int vb_gemm_grouped_combine(const void* A, const void* B, const int* blk_expert, const int* row_dst, const float* row_w, const long* out_ptrs,
                            int world, int R, int N, int K, int E, int lda, int ld_out, int b_mn, int* err_word, cudaStream_t stream);
int vb_gemm_grouped_wgrad(const void* dY, const void* X, void* dW, const void* expert_rng, int R, int M, int N, int E, int ld_dy, int ld_x,
                          int out_f32, int accumulate, int* err_word, cudaStream_t stream);
int vb_ppo_loss(const float* lp, const float* old_lp, const float* ref_lp, const float* adv, const float* weight, const float* mask,
                const float* is_w, long n, float clip_lo, float clip_hi, float clip_c, int kl_type, float kl_coef, float* grad,
                float* loss_out, float* stats, cudaStream_t st);
int vb_ep_count(const int* idx_all, long n_total, int lo, int e_local, int* counts, cudaStream_t st);
int vb_ep_fill(const int* idx_all, const float* w_all, long n_total, int Tc, int k, int lo, int e_local, const int* counts, int n_blocks, int* scratch,
               int* row_src, int* row_dst, float* row_w, int* blk_expert, int* expert_rng, cudaStream_t st);
int vb_gae(const float* rewards, const float* values, const float* mask, int B, int R, float gamma, float lam, int whiten, float* adv, float* ret,
           float* stats, cudaStream_t st);
int vb_value_loss(const float* v, const float* v_old, const float* ret, const float* weight, const float* mask, long n, float clip, float* grad,
                  float* stats, cudaStream_t st);
int vb_grpo_advantage(const float* scores, const int* group, int B, int G, const float* mask, int R, float eps, int norm_by_std,
                      float* mean, float* stdv, float* adv, cudaStream_t st);
int vb_reshard_quant(const long* src_ptrs, int world, int rows_per_rank, long ld_src, int row_begin, void* y, long ldy, float* scale,
                     void* out_bf16, long ld_bf16, int M_out, int N, cudaStream_t st);
int vb_fp8_act_cast(const void* x, long ldx, void* y, long ldy, float* scale, long M, int K, cudaStream_t st);
int vb_fp4_fake_quant(const void* x, void* y, long n, const float* global_amax, cudaStream_t st);
int vb_delta_compact16(const void* cur, void* snap, long n, int* pos_out, void* val_out, unsigned long long* counter, long cap,
                       cudaStream_t st);
int vb_delta_apply16(void* dst, const int* pos, const void* val, long count, cudaStream_t st);

#ifdef __cplusplus
}
#endif
