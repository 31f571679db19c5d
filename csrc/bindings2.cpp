// Bindings of the attention / decode / sampling / fused-loss launchers.
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/extension.h>

#include "api.h"

namespace {
// Also clears this thread's "last error" slot: launchers report cudaGetLastError() after their
// launch, and an unrelated, already handled status left there by another library (for example
// cudaErrorNotReady from an event query) must not be mistaken for a launch failure.
inline cudaStream_t cur_stream() {
  (void)cudaGetLastError();
  return at::cuda::getCurrentCUDAStream().stream();
}
inline void check(int rc, const char* what) {
  if (rc != 0) {
    char buf[160];
    snprintf(buf, sizeof(buf), "%s failed with code %d (%s)", what, rc, rc > 0 ? cudaGetErrorString((cudaError_t)rc) : "argument check");
    fprintf(stderr, "[relax_b200] %s\n", buf);
    throw std::runtime_error(buf);
  }
}

void fa_fwd(torch::Tensor q, torch::Tensor k, torch::Tensor v, torch::Tensor o, torch::Tensor lse, torch::Tensor cu_q,
            torch::Tensor cu_k, int64_t max_q_blocks, bool causal, double scale, torch::Tensor err) {
  const c10::cuda::CUDAGuard guard(q.device());
  TORCH_CHECK(q.scalar_type() == at::kBFloat16 && q.size(2) == 128, "flash attention: bf16, head_dim 128");
  TORCH_CHECK(q.stride(2) == 1 && k.stride(2) == 1 && v.stride(2) == 1, "head dimension must be contiguous");
  check(rb_fa_fwd(q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(), lse.data_ptr<float>(), cu_q.data_ptr<int>(),
                  cu_k.data_ptr<int>(), (int)cu_q.numel() - 1, (int)q.size(0), (int)k.size(0), (int)q.size(1),
                  (int)k.size(1), q.stride(0), q.stride(1), k.stride(0), k.stride(1), v.stride(0), v.stride(1), causal,
                  (float)scale, (int)max_q_blocks, err.data_ptr<int>(), cur_stream()),
        "rb_fa_fwd");
}
void fa_bwd(torch::Tensor q, torch::Tensor k, torch::Tensor v, torch::Tensor o, torch::Tensor d_o, torch::Tensor lse,
            torch::Tensor dq, torch::Tensor dk, torch::Tensor dv, torch::Tensor delta, torch::Tensor dq_acc,
            torch::Tensor cu_q, torch::Tensor cu_k, int64_t max_kv_blocks, bool causal, double scale, torch::Tensor err) {
  const c10::cuda::CUDAGuard guard(q.device());
  check(rb_fa_bwd(q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(), d_o.data_ptr(), lse.data_ptr<float>(),
                  dq.data_ptr(), dk.data_ptr(), dv.data_ptr(), delta.data_ptr<float>(), dq_acc.data_ptr<float>(),
                  cu_q.data_ptr<int>(), cu_k.data_ptr<int>(), (int)cu_q.numel() - 1, (int)q.size(0), (int)k.size(0),
                  (int)q.size(1), (int)k.size(1), causal, (float)scale, (int)max_kv_blocks, err.data_ptr<int>(),
                  cur_stream()),
        "rb_fa_bwd");
}
int64_t decode_attn_splits(int64_t B, int64_t Hkv, int64_t max_ctx) {
  return rb_decode_attn_splits((int)B, (int)Hkv, (int)max_ctx);
}
void decode_attn(torch::Tensor q, torch::Tensor kc, torch::Tensor vc, torch::Tensor block_tables, torch::Tensor ctx_lens,
                 torch::Tensor out, c10::optional<torch::Tensor> part_o, c10::optional<torch::Tensor> part_ml,
                 int64_t max_ctx, double scale, int64_t splits, int64_t version, torch::Tensor err) {
  const c10::cuda::CUDAGuard guard(q.device());
  TORCH_CHECK(q.scalar_type() == at::kBFloat16 && q.size(2) == 128, "decode attention: bf16, head_dim 128");
  if (version == 3) {
    check(rb_decode_attn_tc(q.data_ptr(), kc.data_ptr(), vc.data_ptr(), block_tables.data_ptr<int>(), ctx_lens.data_ptr<int>(),
                            out.data_ptr(), part_o.has_value() ? part_o->data_ptr<float>() : nullptr,
                            part_ml.has_value() ? part_ml->data_ptr<float>() : nullptr, (int)q.size(0), (int)q.size(1),
                            (int)kc.size(2), (int)kc.size(0), (int)kc.size(1), (int)block_tables.size(1), (int)max_ctx,
                            (float)scale, (int)splits, err.data_ptr<int>(), cur_stream()),
          "rb_decode_attn_tc");
    return;
  }
  auto fn = version == 1 ? rb_decode_attn_v1 : rb_decode_attn;
  check(fn(q.data_ptr(), kc.data_ptr(), vc.data_ptr(), block_tables.data_ptr<int>(), ctx_lens.data_ptr<int>(),
                       out.data_ptr(), part_o.has_value() ? part_o->data_ptr<float>() : nullptr,
                       part_ml.has_value() ? part_ml->data_ptr<float>() : nullptr, (int)q.size(0), (int)q.size(1),
                       (int)kc.size(2), (int)kc.size(1), (int)block_tables.size(1), (int)max_ctx, (float)scale,
                       (int)splits, cur_stream()),
        "rb_decode_attn");
}
void sample(torch::Tensor logits, torch::Tensor temperature, torch::Tensor top_k, torch::Tensor top_p,
            torch::Tensor uniform, torch::Tensor tok, torch::Tensor logp, int64_t V) {
  const c10::cuda::CUDAGuard guard(logits.device());
  check(rb_sample(logits.data_ptr<float>(), (int)logits.size(0), (int)V, (int)logits.stride(0),
                  temperature.data_ptr<float>(), (const long long*)top_k.data_ptr<int64_t>(), top_p.data_ptr<float>(),
                  uniform.data_ptr<float>(), (long long*)tok.data_ptr<int64_t>(), logp.data_ptr<float>(), cur_stream()),
        "rb_sample");
}
void sample_v2(torch::Tensor logits, torch::Tensor temperature, torch::Tensor top_k, torch::Tensor top_p,
               torch::Tensor uniform, torch::Tensor tok, torch::Tensor logp, int64_t V) {
  const c10::cuda::CUDAGuard guard(logits.device());
  TORCH_CHECK(logits.dim() == 2 && logits.stride(1) == 1, "sample: logits rows must be contiguous");
  const bool bf = logits.scalar_type() == at::kBFloat16;
  TORCH_CHECK(bf || logits.scalar_type() == at::kFloat, "sample: bf16 or fp32 logits");
  check(rb_sample_v2(logits.data_ptr(), bf ? 1 : 0, (int)logits.size(0), (int)V, (long long)logits.stride(0),
                     temperature.data_ptr<float>(), (const long long*)top_k.data_ptr<int64_t>(), top_p.data_ptr<float>(),
                     uniform.data_ptr<float>(), (long long*)tok.data_ptr<int64_t>(), logp.data_ptr<float>(), cur_stream()),
        "rb_sample_v2");
}
void decode_advance(torch::Tensor tok_new, torch::Tensor lp_new, torch::Tensor tok_in, torch::Tensor pos, torch::Tensor ctx,
                    torch::Tensor slot, torch::Tensor block_table, int64_t block_size, torch::Tensor active,
                    torch::Tensor remain, torch::Tensor eos, torch::Tensor stop_ids, torch::Tensor out_tok,
                    torch::Tensor out_lp, torch::Tensor counter, torch::Tensor u_all, torch::Tensor u_next) {
  const c10::cuda::CUDAGuard guard(tok_new.device());
  const int B = (int)tok_in.size(0);
  TORCH_CHECK(block_table.dim() == 2 && block_table.size(0) == B && block_table.is_contiguous(), "block table [B, max_blocks]");
  TORCH_CHECK(out_tok.dim() == 2 && out_tok.size(1) == B && out_tok.is_contiguous() && out_lp.is_contiguous(), "window ring [W, B]");
  TORCH_CHECK(u_all.dim() == 2 && u_all.size(0) == out_tok.size(0) && u_all.size(1) == B && u_all.is_contiguous(), "u_all [W, B]");
  TORCH_CHECK(stop_ids.dim() == 2 && stop_ids.size(0) == B && stop_ids.is_contiguous(), "stop ids [B, n]");
  check(rb_decode_advance((const long long*)tok_new.data_ptr<int64_t>(), lp_new.data_ptr<float>(),
                          (long long*)tok_in.data_ptr<int64_t>(), (long long*)pos.data_ptr<int64_t>(), ctx.data_ptr<int>(),
                          (long long*)slot.data_ptr<int64_t>(), block_table.data_ptr<int>(), (int)block_table.size(1),
                          (int)block_size, active.data_ptr<int>(), remain.data_ptr<int>(),
                          (const long long*)eos.data_ptr<int64_t>(), (const long long*)stop_ids.data_ptr<int64_t>(),
                          (int)stop_ids.size(1), (long long*)out_tok.data_ptr<int64_t>(), out_lp.data_ptr<float>(),
                          counter.data_ptr<int>(), (int)out_tok.size(0), u_all.data_ptr<float>(), u_next.data_ptr<float>(), B,
                          cur_stream()),
        "rb_decode_advance");
}
void policy_loss(torch::Tensor ppo_kl, torch::Tensor adv, torch::Tensor loss, torch::Tensor clipfrac, torch::Tensor dkl,
                 double eps_clip, double eps_clip_high, double eps_clip_c) {
  const c10::cuda::CUDAGuard guard(ppo_kl.device());
  TORCH_CHECK(ppo_kl.scalar_type() == at::kFloat && adv.scalar_type() == at::kFloat, "fp32 inputs");
  TORCH_CHECK(ppo_kl.is_contiguous() && adv.is_contiguous() && adv.numel() == ppo_kl.numel(), "contiguous inputs of one size");
  check(rb_policy_loss(ppo_kl.data_ptr<float>(), adv.data_ptr<float>(), loss.data_ptr<float>(), clipfrac.data_ptr<float>(),
                       dkl.data_ptr<float>(), ppo_kl.numel(), (float)eps_clip, (float)eps_clip_high, (float)eps_clip_c,
                       cur_stream()),
        "rb_policy_loss");
}
// Weight-streaming decode GEMM; returns false when the shape is outside its range (the caller uses the split-K path).
bool decode_gemm(torch::Tensor x, torch::Tensor W, torch::Tensor y, bool swiglu, int64_t splits, torch::Tensor err) {
  const c10::cuda::CUDAGuard guard(x.device());
  TORCH_CHECK(x.scalar_type() == at::kBFloat16 && W.scalar_type() == at::kBFloat16 && y.scalar_type() == at::kBFloat16, "bf16 only");
  TORCH_CHECK(x.dim() == 2 && W.dim() == 2 && x.stride(1) == 1 && W.stride(1) == 1 && y.is_contiguous(), "row-major operands");
  const int rc = rb_decode_gemm(x.data_ptr(), W.data_ptr(), y.data_ptr(), (int)x.size(0), (int)W.size(0), (int)x.size(1),
                                (int)x.stride(0), (int)W.stride(0), swiglu, (int)splits, err.data_ptr<int>(), cur_stream());
  if (rc == -20) return false;
  check(rc, "rb_decode_gemm");
  return true;
}
void grouped_gemm_fwd(torch::Tensor X, torch::Tensor W, torch::Tensor Y, torch::Tensor tile_expert, torch::Tensor err) {
  const c10::cuda::CUDAGuard guard(X.device());
  TORCH_CHECK(X.scalar_type() == at::kBFloat16 && W.scalar_type() == at::kBFloat16 && Y.scalar_type() == at::kBFloat16, "bf16 only");
  TORCH_CHECK(X.is_contiguous() && W.is_contiguous() && Y.is_contiguous() && W.dim() == 3, "contiguous X [cap,K], W [E,N,K]");
  TORCH_CHECK(tile_expert.scalar_type() == at::kInt && tile_expert.numel() * 128 == X.size(0), "tile map: one int32 per 128 rows");
  check(rb_grouped_gemm_fwd(X.data_ptr(), W.data_ptr(), Y.data_ptr(), tile_expert.data_ptr<int>(), (int)X.size(0),
                            (int)W.size(1), (int)W.size(2), (int)W.size(0), err.data_ptr<int>(), cur_stream()),
        "rb_grouped_gemm_fwd");
}
void grouped_gemm_dgrad(torch::Tensor dY, torch::Tensor W, torch::Tensor dX, torch::Tensor tile_expert, torch::Tensor err) {
  const c10::cuda::CUDAGuard guard(dY.device());
  TORCH_CHECK(dY.scalar_type() == at::kBFloat16 && W.scalar_type() == at::kBFloat16 && dX.scalar_type() == at::kBFloat16, "bf16 only");
  TORCH_CHECK(dY.is_contiguous() && W.is_contiguous() && dX.is_contiguous() && W.dim() == 3, "contiguous dY [cap,N], W [E,N,K]");
  TORCH_CHECK(tile_expert.scalar_type() == at::kInt && tile_expert.numel() * 128 == dY.size(0), "tile map: one int32 per 128 rows");
  check(rb_grouped_gemm_dgrad(dY.data_ptr(), W.data_ptr(), dX.data_ptr(), tile_expert.data_ptr<int>(), (int)dY.size(0),
                              (int)W.size(1), (int)W.size(2), (int)W.size(0), err.data_ptr<int>(), cur_stream()),
        "rb_grouped_gemm_dgrad");
}
void grouped_gemm_wgrad(torch::Tensor dY, torch::Tensor X, torch::Tensor dW, torch::Tensor expert_rows, bool accumulate,
                        torch::Tensor err) {
  const c10::cuda::CUDAGuard guard(dY.device());
  TORCH_CHECK(dY.scalar_type() == at::kBFloat16 && X.scalar_type() == at::kBFloat16, "bf16 inputs");
  TORCH_CHECK(dY.is_contiguous() && X.is_contiguous() && dW.is_contiguous() && dW.dim() == 3, "contiguous dY, X, dW [E,N,K]");
  TORCH_CHECK(expert_rows.scalar_type() == at::kInt && expert_rows.numel() == dW.size(0) + 1, "expert_rows: int32 [E + 1]");
  const bool f32 = dW.scalar_type() == at::kFloat;
  TORCH_CHECK(f32 || dW.scalar_type() == at::kBFloat16, "dW must be fp32 or bf16");
  check(rb_grouped_gemm_wgrad(dY.data_ptr(), X.data_ptr(), dW.data_ptr(), expert_rows.data_ptr<int>(), (int)dY.size(0),
                              (int)dW.size(1), (int)dW.size(2), (int)dW.size(0), f32, accumulate, err.data_ptr<int>(),
                              cur_stream()),
        "rb_grouped_gemm_wgrad");
}
void topk_router(torch::Tensor logits, int64_t K, bool norm, torch::Tensor w, torch::Tensor idx, torch::Tensor probs) {
  const c10::cuda::CUDAGuard guard(logits.device());
  check(rb_topk_router(logits.data_ptr<float>(), (int)logits.size(0), (int)logits.size(1), (int)K, norm,
                       w.data_ptr<float>(), (long long*)idx.data_ptr<int64_t>(), probs.data_ptr<float>(), cur_stream()),
        "rb_topk_router");
}
std::tuple<int64_t, int64_t> gemm_splitk_plan(int64_t M, int64_t N, int64_t K) {
  int bn = 0;
  const int s = rb_gemm_splitk_plan((int)M, (int)N, (int)K, &bn);
  return {s, bn};
}
void gemm_splitk(torch::Tensor A, torch::Tensor B, torch::Tensor C, c10::optional<torch::Tensor> bias,
                 c10::optional<torch::Tensor> residual, torch::Tensor workspace, int64_t splits, int64_t bn,
                 torch::Tensor err) {
  const c10::cuda::CUDAGuard guard(A.device());
  check(rb_gemm_splitk(A.data_ptr(), B.data_ptr(), C.data_ptr(), bias.has_value() ? bias->data_ptr() : nullptr,
                       residual.has_value() ? residual->data_ptr() : nullptr, workspace.data_ptr<float>(), (int)A.size(0),
                       (int)B.size(0), (int)A.size(1), (int)A.stride(0), (int)B.stride(0), (int)C.stride(0), (int)splits,
                       (int)bn, A.scalar_type() == at::kHalf, err.data_ptr<int>(), cur_stream()),
        "rb_gemm_splitk");
}
int64_t lm_head_splits(int64_t M, int64_t N) { return rb_lm_head_splits((int)M, (int)N); }
void lm_head_logprob(torch::Tensor h, torch::Tensor W, torch::Tensor targets, torch::Tensor partials, int64_t vocab_start,
                     double inv_temp, int64_t n_splits, torch::Tensor err) {
  const c10::cuda::CUDAGuard guard(h.device());
  TORCH_CHECK(h.scalar_type() == at::kBFloat16 && W.scalar_type() == at::kBFloat16, "fused LM head: bf16");
  check(rb_lm_head_logprob(h.data_ptr(), W.data_ptr(), (const long long*)targets.data_ptr<int64_t>(),
                           partials.data_ptr<float>(), (int)h.size(0), (int)W.size(0), (int)h.size(1), (int)h.stride(0),
                           (int)W.stride(0), (int)vocab_start, (float)inv_temp, (int)n_splits, err.data_ptr<int>(),
                           cur_stream()),
        "rb_lm_head_logprob");
}
void lm_head_dlogits(torch::Tensor h, torch::Tensor W, torch::Tensor targets, torch::Tensor row_stats, torch::Tensor g_lp,
                     c10::optional<torch::Tensor> g_ent, torch::Tensor dlogits, int64_t vocab_start, double inv_temp,
                     torch::Tensor err) {
  const c10::cuda::CUDAGuard guard(h.device());
  check(rb_lm_head_dlogits(h.data_ptr(), W.data_ptr(), (const long long*)targets.data_ptr<int64_t>(),
                           row_stats.data_ptr<float>(), g_lp.data_ptr<float>(),
                           g_ent.has_value() ? g_ent->data_ptr<float>() : nullptr, dlogits.data_ptr(), (int)h.size(0),
                           (int)W.size(0), (int)h.size(1), (int)h.stride(0), (int)W.stride(0), (int)dlogits.stride(0),
                           (int)vocab_start, (float)inv_temp, err.data_ptr<int>(), cur_stream()),
        "rb_lm_head_dlogits");
}
}  // namespace

void register_symm(pybind11::module_& m);
void register_fused(pybind11::module_& m);
void register_vmm(pybind11::module_& m);

void register_more(pybind11::module_& m) {
  register_symm(m);
  register_fused(m);
  register_vmm(m);
  m.def("fa_fwd", &fa_fwd);
  m.def("fa_bwd", &fa_bwd);
  m.def("decode_attn_splits", &decode_attn_splits);
  m.def("decode_attn", &decode_attn);
  m.def("sample", &sample);
  m.def("sample_v2", &sample_v2);
  m.def("decode_advance", &decode_advance);
  m.def("policy_loss", &policy_loss);
  m.def("decode_gemm", &decode_gemm);
  m.def("grouped_gemm_fwd", &grouped_gemm_fwd);
  m.def("grouped_gemm_dgrad", &grouped_gemm_dgrad);
  m.def("grouped_gemm_wgrad", &grouped_gemm_wgrad);
  m.def("topk_router", &topk_router);
  m.def("gemm_splitk_plan", &gemm_splitk_plan);
  m.def("gemm_splitk", &gemm_splitk);
  m.def("lm_head_splits", &lm_head_splits);
  m.def("lm_head_logprob", &lm_head_logprob);
  m.def("lm_head_dlogits", &lm_head_dlogits);
}
