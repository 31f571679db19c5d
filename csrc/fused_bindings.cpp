// Bindings of the kernels that fuse a GEMM with its tensor-parallel collective over NVLink peer memory.
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/extension.h>

#include "api.h"

namespace {
inline cudaStream_t cur_stream() {
  (void)cudaGetLastError();
  return at::cuda::getCurrentCUDAStream().stream();
}
inline void check(int rc, const char* what) {
  if (rc != 0) {
    char buf[160];
    snprintf(buf, sizeof(buf), "%s failed with code %d (%s)", what, rc, rc > 0 ? cudaGetErrorString((cudaError_t)rc) : "argument check");
    throw std::runtime_error(buf);
  }
}

std::tuple<int64_t, int64_t> gemm_ar_plan(int64_t M, int64_t N, int64_t K) {
  int bn = 0;
  const int s = rb_gemm_ar_plan((int)M, (int)N, (int)K, &bn);
  return {s, bn};
}

// x [M,K] bf16, w [N,K] bf16 (this rank's K shard).  ws_ptrs / sig_ptrs: device addresses of every rank's
// workspace / counters as mapped in this process.  Writes out_h (and out_x when norm_w is given).
void gemm_ar_rmsnorm(torch::Tensor x, torch::Tensor w, std::vector<int64_t> ws_ptrs, std::vector<int64_t> sig_ptrs,
                     int64_t tp_rank, torch::Tensor state, c10::optional<torch::Tensor> residual,
                     c10::optional<torch::Tensor> norm_w, torch::Tensor out_h, c10::optional<torch::Tensor> out_x, double eps,
                     int64_t splits, int64_t bn, bool reduce_scatter, bool w_is_kn, int64_t wait_ns, torch::Tensor err,
                     c10::optional<torch::Tensor> timeline) {
  const c10::cuda::CUDAGuard guard(x.device());
  TORCH_CHECK(x.scalar_type() == at::kBFloat16 && w.scalar_type() == at::kBFloat16, "gemm_ar_rmsnorm: bf16");
  TORCH_CHECK(x.stride(1) == 1 && w.stride(1) == 1 && out_h.is_contiguous(), "gemm_ar_rmsnorm: contiguous rows");
  // w_is_kn: w is stored [K][N] (the dgrad form dy @ W); otherwise [N][K]
  const int N = (int)(w_is_kn ? w.size(1) : w.size(0));
  TORCH_CHECK(norm_w.has_value() == out_x.has_value(), "norm_w and out_x go together");
  const int tp = (int)ws_ptrs.size();
  TORCH_CHECK(tp >= 1 && tp <= 8 && sig_ptrs.size() == ws_ptrs.size());
  float* ws[8];
  unsigned* sg[8];
  for (int r = 0; r < tp; ++r) {
    ws[r] = reinterpret_cast<float*>(ws_ptrs[r]);
    sg[r] = reinterpret_cast<unsigned*>(sig_ptrs[r]);
  }
  check(rb_gemm_ar_rmsnorm(x.data_ptr(), w.data_ptr(), (int)x.size(0), N, (int)x.size(1), (int)x.stride(0),
                           (int)w.stride(0), tp, (int)tp_rank, ws, sg, state.data_ptr<int>(),
                           residual.has_value() ? residual->data_ptr() : nullptr,
                           norm_w.has_value() ? norm_w->data_ptr() : nullptr, out_h.data_ptr(),
                           out_x.has_value() ? out_x->data_ptr() : nullptr, (float)eps, (int)splits, (int)bn,
                           reduce_scatter ? 1 : 0, w_is_kn ? 1 : 0, (unsigned long long)wait_ns,
                           timeline.has_value() ? reinterpret_cast<unsigned long long*>(timeline->data_ptr<int64_t>()) : nullptr,
                           err.data_ptr<int>(), cur_stream()),
        "rb_gemm_ar_rmsnorm");
}

// x_shard [M/tp, K] bf16 contiguous, w [N, K] bf16; y [M, N].  ag_ptrs: every rank's gathered buffer ([2][M][K]).
void ag_gemm(torch::Tensor x_shard, torch::Tensor w, torch::Tensor y, std::vector<int64_t> ag_ptrs,
             std::vector<int64_t> sig_ptrs, int64_t tp_rank, torch::Tensor state, int64_t bn, int64_t wait_ns,
             torch::Tensor err) {
  const c10::cuda::CUDAGuard guard(x_shard.device());
  TORCH_CHECK(x_shard.scalar_type() == at::kBFloat16 && w.scalar_type() == at::kBFloat16, "ag_gemm: bf16");
  TORCH_CHECK(x_shard.is_contiguous() && w.stride(1) == 1 && y.stride(1) == 1, "ag_gemm: contiguous rows");
  const int tp = (int)ag_ptrs.size();
  TORCH_CHECK(tp >= 1 && tp <= 8 && sig_ptrs.size() == ag_ptrs.size() && state.numel() >= 12);
  void* ag[8];
  unsigned* sg[8];
  for (int r = 0; r < tp; ++r) {
    ag[r] = reinterpret_cast<void*>(ag_ptrs[r]);
    sg[r] = reinterpret_cast<unsigned*>(sig_ptrs[r]);
  }
  check(rb_ag_gemm(x_shard.data_ptr(), w.data_ptr(), y.data_ptr(), (int)x_shard.size(0) * tp, (int)w.size(0),
                   (int)x_shard.size(1), (int)w.stride(0), (int)y.stride(0), tp, (int)tp_rank, ag, sg,
                   state.data_ptr<int>(), (int)bn, (unsigned long long)wait_ns, err.data_ptr<int>(), cur_stream()),
        "rb_ag_gemm");
}

// Fused QKV post-processing (see qkv_post_sm100.cu).  k_out / v_out / cache / slots are optional.
void qkv_post(torch::Tensor qkv, c10::optional<torch::Tensor> qw, c10::optional<torch::Tensor> kw, torch::Tensor cos_t,
              torch::Tensor sin_t, torch::Tensor q_out, c10::optional<torch::Tensor> k_out,
              c10::optional<torch::Tensor> v_out, c10::optional<torch::Tensor> k_cache,
              c10::optional<torch::Tensor> v_cache, c10::optional<torch::Tensor> slots, int64_t nq, int64_t nkv, double eps) {
  const c10::cuda::CUDAGuard guard(qkv.device());
  TORCH_CHECK(qkv.scalar_type() == at::kBFloat16 && qkv.stride(1) == 1 && qkv.size(1) == (nq + 2 * nkv) * 128,
              "qkv_post: bf16 [T, (nq + 2 nkv) * 128]");
  TORCH_CHECK(cos_t.scalar_type() == at::kFloat && cos_t.is_contiguous() && sin_t.is_contiguous() && cos_t.size(1) == 64);
  TORCH_CHECK(q_out.is_contiguous() && (!k_out.has_value() || k_out->is_contiguous()) &&
              (!v_out.has_value() || v_out->is_contiguous()));
  TORCH_CHECK(slots.has_value() == k_cache.has_value() && slots.has_value() == v_cache.has_value());
  if (k_cache.has_value()) TORCH_CHECK(k_cache->is_contiguous() && v_cache->is_contiguous() && k_cache->size(2) == nkv);
  auto ptr = [](c10::optional<torch::Tensor>& t) -> void* { return t.has_value() ? t->data_ptr() : nullptr; };
  check(rb_qkv_post(qkv.data_ptr(), (int)qkv.stride(0), ptr(qw), ptr(kw), cos_t.data_ptr<float>(), sin_t.data_ptr<float>(),
                    q_out.data_ptr(), ptr(k_out), ptr(v_out), ptr(k_cache), ptr(v_cache),
                    slots.has_value() ? (const long long*)slots->data_ptr<int64_t>() : nullptr, (int)qkv.size(0), (int)nq,
                    (int)nkv, (float)eps, cur_stream()),
        "rb_qkv_post");
}

// Split-K partial sums of x @ w^T into ws ([splits][M][N] fp32); no reduction.
void gemm_splitk_partial(torch::Tensor A, torch::Tensor B, torch::Tensor workspace, int64_t splits, int64_t bn,
                         torch::Tensor err) {
  const c10::cuda::CUDAGuard guard(A.device());
  check(rb_gemm_splitk(A.data_ptr(), B.data_ptr(), nullptr, nullptr, nullptr, workspace.data_ptr<float>(), (int)A.size(0),
                       (int)B.size(0), (int)A.size(1), (int)A.stride(0), (int)B.stride(0), (int)B.size(0), (int)splits, (int)bn,
                       A.scalar_type() == at::kHalf, err.data_ptr<int>(), cur_stream()),
        "rb_gemm_splitk");
}
void splitk_swiglu(torch::Tensor workspace, torch::Tensor out, int64_t splits) {
  const c10::cuda::CUDAGuard guard(out.device());
  TORCH_CHECK(out.scalar_type() == at::kBFloat16 && out.is_contiguous());
  check(rb_splitk_swiglu(workspace.data_ptr<float>(), out.data_ptr(), (int)out.size(0), (int)out.size(1), (int)splits,
                         cur_stream()),
        "rb_splitk_swiglu");
}

// Distributed-optimizer kernels over peer memory (see dist_optim_sm100.cu).
void dp_reduce_sumsq(std::vector<int64_t> grad_ptrs, std::vector<int64_t> sig_ptrs, torch::Tensor state, int64_t rank,
                     int64_t lo, torch::Tensor out, torch::Tensor sumsq, double scale, int64_t wait_ns, torch::Tensor err) {
  const c10::cuda::CUDAGuard guard(out.device());
  const int dp = (int)grad_ptrs.size();
  TORCH_CHECK(dp >= 1 && dp <= 8 && sig_ptrs.size() == grad_ptrs.size() && state.numel() >= 16);
  TORCH_CHECK(out.scalar_type() == at::kFloat && out.is_contiguous() && sumsq.scalar_type() == at::kFloat);
  float* g[8];
  unsigned* sg[8];
  for (int r = 0; r < dp; ++r) {
    g[r] = reinterpret_cast<float*>(grad_ptrs[r]);
    sg[r] = reinterpret_cast<unsigned*>(sig_ptrs[r]);
  }
  check(rb_dp_reduce_sumsq(g, sg, state.data_ptr<int>(), dp, (int)rank, lo, out.numel(), out.data_ptr<float>(),
                           sumsq.data_ptr<float>(), (float)scale, (unsigned long long)wait_ns, err.data_ptr<int>(), cur_stream()),
        "rb_dp_reduce_sumsq");
}
void dp_adam_allgather(std::vector<int64_t> param_ptrs, std::vector<int64_t> sig_ptrs, torch::Tensor state, int64_t rank,
                       int64_t lo, torch::Tensor master, torch::Tensor g, torch::Tensor m, torch::Tensor v, int64_t step,
                       double lr, double b1, double b2, double eps, double wd, double gscale, bool split, int64_t wait_ns,
                       torch::Tensor err) {
  const c10::cuda::CUDAGuard guard(g.device());
  const int dp = (int)param_ptrs.size();
  TORCH_CHECK(dp >= 1 && dp <= 8 && sig_ptrs.size() == param_ptrs.size() && state.numel() >= 16);
  TORCH_CHECK(g.scalar_type() == at::kFloat && m.scalar_type() == at::kFloat && v.scalar_type() == at::kFloat);
  void* pp[8];
  unsigned* sg[8];
  for (int r = 0; r < dp; ++r) {
    pp[r] = reinterpret_cast<void*>(param_ptrs[r]);
    sg[r] = reinterpret_cast<unsigned*>(sig_ptrs[r]);
  }
  check(rb_dp_adam_allgather(pp, sg, state.data_ptr<int>(), dp, (int)rank, lo, g.numel(), master.data_ptr(),
                             g.data_ptr<float>(), m.data_ptr<float>(), v.data_ptr<float>(), (int)step, (float)lr, (float)b1,
                             (float)b2, (float)eps, (float)wd, (float)gscale, split ? 1 : 0, (unsigned long long)wait_ns,
                             err.data_ptr<int>(), cur_stream()),
        "rb_dp_adam_allgather");
}

void peer_barrier(std::vector<int64_t> sig_ptrs, torch::Tensor state, int64_t rank, int64_t slot, int64_t state_idx,
                  int64_t wait_ns, torch::Tensor err) {
  const c10::cuda::CUDAGuard guard(state.device());
  const int n = (int)sig_ptrs.size();
  unsigned* sg[8];
  TORCH_CHECK(n >= 1 && n <= 8);
  for (int r = 0; r < n; ++r) sg[r] = reinterpret_cast<unsigned*>(sig_ptrs[r]);
  check(rb_peer_barrier(sg, state.data_ptr<int>(), n, (int)rank, (int)slot, (int)state_idx, (unsigned long long)wait_ns,
                        err.data_ptr<int>(), cur_stream()),
        "rb_peer_barrier");
}

// Flash-attention backward with caller-controlled scratch handling (flags as in rb_fa_bwd_ex); tensors may alias
// peer memory.  dq may be an empty tensor when flag 4 is set.
void fa_bwd_ex(torch::Tensor q, torch::Tensor k, torch::Tensor v, torch::Tensor o, torch::Tensor d_o, torch::Tensor lse,
               torch::Tensor dq, torch::Tensor dk, torch::Tensor dv, torch::Tensor delta, torch::Tensor dq_acc,
               torch::Tensor cu_q, torch::Tensor cu_k, int64_t max_kv_blocks, bool causal, double scale, int64_t flags,
               torch::Tensor err) {
  const c10::cuda::CUDAGuard guard(k.device());
  check(rb_fa_bwd_ex(q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(), d_o.data_ptr(), lse.data_ptr<float>(),
                     dq.data_ptr(), dk.data_ptr(), dv.data_ptr(), delta.data_ptr<float>(), dq_acc.data_ptr<float>(),
                     cu_q.data_ptr<int>(), cu_k.data_ptr<int>(), (int)cu_q.numel() - 1, (int)q.size(0), (int)k.size(0),
                     (int)q.size(1), (int)k.size(1), causal, (float)scale, (int)max_kv_blocks, (int)flags,
                     err.data_ptr<int>(), cur_stream()),
        "rb_fa_bwd_ex");
}
void fa_dq_convert(torch::Tensor dq_acc, torch::Tensor dq) {
  const c10::cuda::CUDAGuard guard(dq.device());
  check(rb_fa_dq_convert(dq_acc.data_ptr<float>(), dq.data_ptr(), dq.numel(), cur_stream()), "rb_fa_dq_convert");
}

// src (contiguous) -> dst_ptrs[i] + offset_bytes for every destination.
void peer_push(torch::Tensor src, std::vector<int64_t> dst_ptrs, int64_t offset_bytes) {
  const c10::cuda::CUDAGuard guard(src.device());
  TORCH_CHECK(src.is_contiguous() && dst_ptrs.size() <= 8);
  void* d[8];
  for (size_t i = 0; i < dst_ptrs.size(); ++i) d[i] = reinterpret_cast<void*>(dst_ptrs[i] + offset_bytes);
  check(rb_peer_push(src.data_ptr(), d, (int)dst_ptrs.size(), (long long)src.numel() * src.element_size(), cur_stream()),
        "rb_peer_push");
}

// Block-scaled fp8 GEMM: a_q [M,K] e4m3 with a_scale [M, K/128]; b_q [N,K] e4m3 with b_scale [N/128, K/128]; out bf16.
void gemm_fp8(torch::Tensor a_q, torch::Tensor a_scale, torch::Tensor b_q, torch::Tensor b_scale, torch::Tensor out,
              torch::Tensor err) {
  const c10::cuda::CUDAGuard guard(a_q.device());
  TORCH_CHECK(a_q.element_size() == 1 && b_q.element_size() == 1 && a_q.stride(1) == 1 && b_q.stride(1) == 1, "fp8 operands");
  TORCH_CHECK(a_scale.scalar_type() == at::kFloat && b_scale.scalar_type() == at::kFloat && a_scale.is_contiguous() &&
              b_scale.is_contiguous() && out.scalar_type() == at::kBFloat16 && out.stride(1) == 1);
  const int M = (int)a_q.size(0), K = (int)a_q.size(1), N = (int)b_q.size(0);
  const int kb = (K + 127) / 128;
  TORCH_CHECK(a_scale.size(0) == M && a_scale.size(1) == kb && b_scale.size(0) == (N + 127) / 128 && b_scale.size(1) == kb,
              "scale shapes: a [M, K/128], b [N/128, K/128]");
  check(rb_gemm_fp8_blockscaled(a_q.data_ptr(), a_scale.data_ptr<float>(), b_q.data_ptr(), b_scale.data_ptr<float>(),
                                out.data_ptr(), M, N, K, (int)a_q.stride(0), (int)b_q.stride(0), (int)out.stride(0),
                                err.data_ptr<int>(), cur_stream()),
        "rb_gemm_fp8_blockscaled");
}
}  // namespace

void register_fused(pybind11::module_& m) {
  m.def("gemm_ar_plan", &gemm_ar_plan);
  m.def("ag_gemm", &ag_gemm);
  m.def("qkv_post", &qkv_post);
  m.def("gemm_fp8", &gemm_fp8);
  m.def("peer_barrier", &peer_barrier);
  m.def("peer_push", &peer_push);
  m.def("fa_bwd_ex", &fa_bwd_ex);
  m.def("fa_dq_convert", &fa_dq_convert);
  m.def("dp_reduce_sumsq", &dp_reduce_sumsq);
  m.def("dp_adam_allgather", &dp_adam_allgather);
  m.def("gemm_splitk_partial", &gemm_splitk_partial);
  m.def("splitk_swiglu", &splitk_swiglu);
  m.def("gemm_ar_rmsnorm", &gemm_ar_rmsnorm, pybind11::arg("x"), pybind11::arg("w"), pybind11::arg("ws_ptrs"),
        pybind11::arg("sig_ptrs"), pybind11::arg("tp_rank"), pybind11::arg("state"), pybind11::arg("residual"),
        pybind11::arg("norm_w"), pybind11::arg("out_h"), pybind11::arg("out_x"), pybind11::arg("eps"),
        pybind11::arg("splits"), pybind11::arg("bn"), pybind11::arg("reduce_scatter"), pybind11::arg("w_is_kn"),
        pybind11::arg("wait_ns"), pybind11::arg("err"), pybind11::arg("timeline") = c10::optional<torch::Tensor>());
}
