// C entry points of the sm_100a kernels (one launcher per op).  Every function
// returns 0 on success, a cudaError_t value or a negative argument-check code
// otherwise, launches on `stream` and allocates nothing.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

int rb_gemm(const void* A, const void* B, void* C, const void* bias, int M, int N, int K, int lda, int ldb, int ldc,
            int a_mn_major, int b_mn_major, int out_fp32, int accumulate, int is_fp16, int force_bn, int lbo_a,
            int sbo_a, int lbo_b, int sbo_b, int* err_flag, cudaStream_t stream);

int rb_gemm_pair(const void* A, const void* B, void* C, int M, int N, int K, int lda, int ldb, int ldc, int a_mn_major,
                 int b_mn_major, int out_fp32, int accumulate, int force_bn, int* err_flag, cudaStream_t stream);

int rb_rmsnorm_fwd(const void* x, const void* res, const void* w, void* y, void* r_out, int rows, int cols, float eps,
                   int dtype, cudaStream_t st);
int rb_rmsnorm_bwd_parts(int rows, int cols);
int rb_rmsnorm_bwd(const void* x, const void* w, const void* dy, void* dx, void* dw, float* scratch, int rows, int cols,
                   float eps, int dtype, cudaStream_t st);
int rb_rope(const void* x, void* y, const float* cos_t, const float* sin_t, long long tokens, int H, int D, int backward,
            int dtype, cudaStream_t st);
int rb_swiglu_fwd(const void* in, void* out, long long rows, int F, int dtype, cudaStream_t st);
int rb_swiglu_bwd(const void* in, const void* dout, void* din, long long rows, int F, int dtype, cudaStream_t st);
int rb_adam(void* p, void* master, const void* g, float* m, float* v, long long n, int step, float lr, float b1, float b2,
            float eps, float wd, float gscale, int split, int grad_fp32, cudaStream_t st);
int rb_sumsq(const void* g, long long n, float* out, int dtype, cudaStream_t st);
int rb_copy_table(const void* table, int n_desc, const int* chunk_start, int total_chunks, int chunk_rows, int elem_size,
                  cudaStream_t st);
int rb_kv_scatter(const void* k, const void* v, void* kc, void* vc, const long long* slots, int tokens, int row_elems,
                  long long k_stride, long long v_stride, int dtype, cudaStream_t st);
int rb_int4_fake_quant(const void* x, void* out, void* scale, void* zero, int M, int N, int bm, int bn, int sym, int dtype,
                       cudaStream_t st);
int rb_fp8_block_cast(const void* w, void* q, float* scale, int M, int N, int block, int ue8m0, int dtype, cudaStream_t st);
int rb_fp8_block_dequant(const void* q, const float* scale, void* out, int M, int N, int block, int dtype, cudaStream_t st);

#ifdef __cplusplus
}
#endif

#ifdef TORCH_EXTENSION_NAME
#include <pybind11/pybind11.h>
void register_more(pybind11::module_& m);
#endif

// ---- attention / decode / sampling / fused LM head (declared again for C callers)
#ifdef __cplusplus
extern "C" {
#endif
int rb_fa_fwd(const void* q, const void* k, const void* v, void* o, float* lse, const int* cu_q, const int* cu_k,
              int num_seqs, int Tq, int Tk, int Hq, int Hkv, long long q_tok, long long q_head, long long k_tok,
              long long k_head, long long v_tok, long long v_head, int causal, float scale, int max_q_blocks, int* err,
              cudaStream_t stream);
int rb_fa_bwd(const void* q, const void* k, const void* v, const void* o, const void* d_o, const float* lse, void* dq,
              void* dk, void* dv, float* delta, float* dq_acc, const int* cu_q, const int* cu_k, int num_seqs, int Tq,
              int Tk, int Hq, int Hkv, int causal, float scale, int max_kv_blocks, int* err, cudaStream_t stream);
int rb_decode_attn_splits(int B, int Hkv, int max_ctx);
int rb_decode_attn(const void* q, const void* kc, const void* vc, const int* block_tables, const int* ctx_lens, void* out,
                   float* part_o, float* part_ml, int B, int Hq, int Hkv, int block_size, int max_blocks, int max_ctx,
                   float scale, int splits, cudaStream_t st);
int rb_decode_attn_v1(const void* q, const void* kc, const void* vc, const int* block_tables, const int* ctx_lens, void* out,
                      float* part_o, float* part_ml, int B, int Hq, int Hkv, int block_size, int max_blocks, int max_ctx,
                      float scale, int splits, cudaStream_t st);
int rb_decode_attn_tc(const void* q, const void* kc, const void* vc, const int* block_tables, const int* ctx_lens, void* out,
                      float* part_o, float* part_ml, int B, int Hq, int Hkv, int num_blocks, int block_size, int max_blocks,
                      int max_ctx, float scale, int splits, int* err, cudaStream_t st);
int rb_sample(const float* logits, int B, int V, int ld, const float* temperature, const long long* top_k,
              const float* top_p, const float* uniform, long long* tok, float* logp, cudaStream_t st);
int rb_topk_router(const float* logits, int T, int E, int K, int norm, float* w, long long* idx, float* probs,
                   cudaStream_t st);
int rb_sample_v2(const void* logits, int is_bf16, int B, int V, long long ld, const float* temperature,
                 const long long* top_k, const float* top_p, const float* uniform, long long* tok, float* logp,
                 cudaStream_t st);
int rb_decode_advance(const long long* tok_new, const float* lp_new, long long* tok_in, long long* pos, int* ctx,
                      long long* slot, const int* block_table, int max_blocks, int block_size, int* active, int* remain,
                      const long long* eos, const long long* stop_ids, int n_stop, long long* out_tok, float* out_lp,
                      int* counter, int window, const float* u_all, float* u_next, int B, cudaStream_t st);
int rb_gemm_splitk_plan(int M, int N, int K, int* bn_out);
int rb_gemm_splitk(const void* A, const void* B, void* C, const void* bias, const void* residual, float* workspace, int M,
                   int N, int K, int lda, int ldb, int ldc, int splits, int bn, int is_fp16, int* err_flag,
                   cudaStream_t stream);
int rb_gemm_ar_plan(int M, int N, int K, int* bn_out);
int rb_gemm_ar_rmsnorm(const void* A, const void* B, int M, int N, int K, int lda, int ldb, int tp, int tp_rank,
                       float* const* peer_ws, unsigned* const* peer_sig, int* state, const void* residual,
                       const void* norm_w, void* out_h, void* out_x, float eps, int splits, int bn,
                       int reduce_scatter, int b_mn_major, unsigned long long wait_ns, unsigned long long* timeline,
                       int* err_flag, cudaStream_t stream);
int rb_ag_gemm(const void* x_shard, const void* B, void* C, int M, int N, int K, int ldb, int ldc, int tp, int tp_rank,
               void* const* peer_ag, unsigned* const* peer_sig, int* state, int bn, unsigned long long wait_ns,
               int* err_flag, cudaStream_t stream);
int rb_qkv_post(const void* qkv, int ld, const void* qw, const void* kw, const float* cos_t, const float* sin_t, void* q_out,
                void* k_out, void* v_out, void* k_cache, void* v_cache, const long long* slots, int T, int nq, int nkv,
                float eps, cudaStream_t st);
int rb_splitk_swiglu(const float* ws, void* out, int M, int F, int splits, cudaStream_t st);
int rb_dp_reduce_sumsq(float* const* peer_g, unsigned* const* peer_sig, int* state, int dp, int rank, long long lo, long long n,
                       float* out, float* sumsq, float scale, unsigned long long wait_ns, int* err, cudaStream_t st);
int rb_dp_adam_allgather(void* const* peer_p, unsigned* const* peer_sig, int* state, int dp, int rank, long long lo,
                         long long n, void* master, const float* g, float* m, float* v, int step, float lr, float b1,
                         float b2, float eps, float wd, float gscale, int split, unsigned long long wait_ns, int* err,
                         cudaStream_t st);
int rb_fa_bwd_ex(const void* q, const void* k, const void* v, const void* o, const void* d_o, const float* lse, void* dq,
                 void* dk, void* dv, float* delta, float* dq_acc, const int* cu_q, const int* cu_k, int num_seqs, int Tq,
                 int Tk, int Hq, int Hkv, int causal, float scale, int max_kv_blocks, int flags, int* err,
                 cudaStream_t stream);
int rb_fa_dq_convert(const float* dq_acc, void* dq, long long n, cudaStream_t stream);
int rb_peer_barrier(unsigned* const* peer_sig, int* state, int n, int rank, int slot, int state_idx,
                    unsigned long long wait_ns, int* err, cudaStream_t st);
int rb_peer_push(const void* src, void* const* dst, int n_dst, long long nbytes, cudaStream_t st);
int rb_gemm_fp8_blockscaled(const void* A, const float* sa, const void* B, const float* sb, void* C, int M, int N, int K,
                            int lda, int ldb, int ldc, int* err, cudaStream_t stream);
int rb_grouped_gemm_fwd(const void* X, const void* W, void* Y, const int* tile_expert, int rows_cap, int N, int K, int E,
                        int* err, cudaStream_t st);
int rb_grouped_gemm_dgrad(const void* dY, const void* W, void* dX, const int* tile_expert, int rows_cap, int Nw, int Kw,
                          int E, int* err, cudaStream_t st);
int rb_grouped_gemm_wgrad(const void* dY, const void* X, void* dW, const int* expert_rows, int rows_cap, int Nw, int Kw,
                          int E, int out_fp32, int accumulate, int* err, cudaStream_t st);
int rb_decode_gemm_splits(int tiles, int k_iters);
int rb_decode_gemm(const void* x, const void* W, void* y, int Mt, int N, int K, int ldx, int ldw, int swiglu, int splits,
                   int* err, cudaStream_t st);
int rb_policy_loss(const float* ppo_kl, const float* adv, float* loss, float* clipfrac, float* dkl, long long n, float eps_clip,
                   float eps_clip_high, float eps_clip_c, cudaStream_t st);
int rb_lm_head_splits(int M, int N);
int rb_lm_head_logprob(const void* h, const void* W, const long long* targets, float* partials, int M, int N, int K,
                       int ldh, int ldw, int vocab_start, float inv_temp, int n_splits, int* err, cudaStream_t stream);
int rb_lm_head_dlogits(const void* h, const void* W, const long long* targets, const float* row_stats, const float* g_lp,
                       const float* g_ent, void* dlogits, int M, int N, int K, int ldh, int ldw, int ldd, int vocab_start,
                       float inv_temp, int* err, cudaStream_t stream);
#ifdef __cplusplus
}
#endif
