// Python bindings: thin tensor -> pointer adapters around the extern "C" kernel
// launchers.  No allocation policy lives here except output tensors requested by
// the Python wrappers; every launcher runs on the current CUDA stream.
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/extension.h>

#include "api.h"
#include "host_utils.h"

#include <execinfo.h>
#include <signal.h>
#include <unistd.h>

namespace {

// Debug aid: print a native backtrace when the process receives SIGSEGV/SIGABRT.
void crash_handler(int sig) {
  const char msg[] = "\n[relax_b200] fatal signal, native backtrace:\n";
  (void)!write(2, msg, sizeof(msg) - 1);
  void* frames[64];
  const int n = backtrace(frames, 64);
  backtrace_symbols_fd(frames, n, 2);
  signal(sig, SIG_DFL);
  raise(sig);
}
void install_crash_handler() {
  void* warm[4];
  (void)backtrace(warm, 4);  // loads the unwinder now, not inside the handler
  signal(SIGSEGV, crash_handler);
  signal(SIGBUS, crash_handler);
}

// Also clears this thread's "last error" slot: launchers report cudaGetLastError() after their
// launch, and an unrelated, already handled status left there by another library (for example
// cudaErrorNotReady from an event query) must not be mistaken for a launch failure.
inline cudaStream_t cur_stream() {
  (void)cudaGetLastError();
  return at::cuda::getCurrentCUDAStream().stream();
}

inline int dtype_code(const torch::Tensor& t) {
  switch (t.scalar_type()) {
    case at::kBFloat16: return 0;
    case at::kHalf: return 1;
    case at::kFloat: return 2;
    default: TORCH_CHECK(false, "unsupported dtype ", t.scalar_type());
  }
}
inline void check(int rc, const char* what) {
  if (rc != 0) {
    char buf[160];
    snprintf(buf, sizeof(buf), "%s failed with code %d (%s)", what, rc, rc > 0 ? cudaGetErrorString((cudaError_t)rc) : "argument check");
    fprintf(stderr, "[relax_b200] %s\n", buf);
    throw std::runtime_error(buf);
  }
}
inline const void* optptr(const c10::optional<torch::Tensor>& t) { return t.has_value() ? t->data_ptr() : nullptr; }

#define CHECK_CUDA_CONTIG(t) TORCH_CHECK((t).is_cuda() && (t).is_contiguous(), #t " must be a contiguous CUDA tensor")

void gemm(torch::Tensor A, torch::Tensor B, torch::Tensor C, c10::optional<torch::Tensor> bias, int64_t M, int64_t N,
          int64_t K, int64_t lda, int64_t ldb, int64_t ldc, bool a_mn, bool b_mn, bool accumulate, int64_t force_bn,
          int64_t lbo_a, int64_t sbo_a, int64_t lbo_b, int64_t sbo_b, torch::Tensor err) {
  const c10::cuda::CUDAGuard guard(A.device());
  TORCH_CHECK(A.scalar_type() == B.scalar_type(), "A/B dtype mismatch");
  const bool fp16 = A.scalar_type() == at::kHalf;
  TORCH_CHECK(fp16 || A.scalar_type() == at::kBFloat16, "gemm inputs must be bf16 or fp16");
  const bool out_fp32 = C.scalar_type() == at::kFloat;
  TORCH_CHECK(out_fp32 || C.scalar_type() == A.scalar_type(), "output must be fp32 or the input dtype");
  check(rb_gemm(A.data_ptr(), B.data_ptr(), C.data_ptr(), optptr(bias), (int)M, (int)N, (int)K, (int)lda, (int)ldb,
                (int)ldc, a_mn, b_mn, out_fp32, accumulate, fp16, (int)force_bn, (int)lbo_a, (int)sbo_a, (int)lbo_b,
                (int)sbo_b, err.data_ptr<int>(), cur_stream()),
        "rb_gemm");
}

// CTA-pair kernel; returns false when the problem does not qualify (the caller then uses `gemm`).
bool gemm_pair(torch::Tensor A, torch::Tensor B, torch::Tensor C, int64_t M, int64_t N, int64_t K, int64_t lda, int64_t ldb,
               int64_t ldc, bool a_mn, bool b_mn, bool accumulate, int64_t force_bn, torch::Tensor err) {
  const c10::cuda::CUDAGuard guard(A.device());
  TORCH_CHECK(A.scalar_type() == at::kBFloat16 && B.scalar_type() == at::kBFloat16, "gemm_pair inputs must be bf16");
  const bool out_fp32 = C.scalar_type() == at::kFloat;
  TORCH_CHECK(out_fp32 || C.scalar_type() == at::kBFloat16, "output must be fp32 or bf16");
  const int rc = rb_gemm_pair(A.data_ptr(), B.data_ptr(), C.data_ptr(), (int)M, (int)N, (int)K, (int)lda, (int)ldb, (int)ldc,
                              a_mn, b_mn, out_fp32, accumulate, (int)force_bn, err.data_ptr<int>(), cur_stream());
  if (rc == -20) return false;
  check(rc, "rb_gemm_pair");
  return true;
}

void rmsnorm_fwd(torch::Tensor x, c10::optional<torch::Tensor> res, torch::Tensor w, torch::Tensor y,
                 c10::optional<torch::Tensor> r_out, int64_t rows, int64_t cols, double eps) {
  const c10::cuda::CUDAGuard guard(x.device());
  check(rb_rmsnorm_fwd(x.data_ptr(), optptr(res), w.data_ptr(), y.data_ptr(),
                       r_out.has_value() ? r_out->data_ptr() : nullptr, (int)rows, (int)cols, (float)eps, dtype_code(x),
                       cur_stream()),
        "rb_rmsnorm_fwd");
}
int64_t rmsnorm_bwd_parts(int64_t rows, int64_t cols) { return rb_rmsnorm_bwd_parts((int)rows, (int)cols); }
void rmsnorm_bwd(torch::Tensor x, torch::Tensor w, torch::Tensor dy, torch::Tensor dx, torch::Tensor dw,
                 torch::Tensor scratch, int64_t rows, int64_t cols, double eps) {
  const c10::cuda::CUDAGuard guard(x.device());
  check(rb_rmsnorm_bwd(x.data_ptr(), w.data_ptr(), dy.data_ptr(), dx.data_ptr(), dw.data_ptr(), scratch.data_ptr<float>(),
                       (int)rows, (int)cols, (float)eps, dtype_code(x), cur_stream()),
        "rb_rmsnorm_bwd");
}
void rope(torch::Tensor x, torch::Tensor y, torch::Tensor cos_t, torch::Tensor sin_t, int64_t tokens, int64_t H,
          int64_t D, bool backward) {
  const c10::cuda::CUDAGuard guard(x.device());
  check(rb_rope(x.data_ptr(), y.data_ptr(), cos_t.data_ptr<float>(), sin_t.data_ptr<float>(), tokens, (int)H, (int)D,
                backward, dtype_code(x), cur_stream()),
        "rb_rope");
}
void swiglu_fwd(torch::Tensor in, torch::Tensor out, int64_t rows, int64_t F) {
  const c10::cuda::CUDAGuard guard(in.device());
  check(rb_swiglu_fwd(in.data_ptr(), out.data_ptr(), rows, (int)F, dtype_code(in), cur_stream()), "rb_swiglu_fwd");
}
void swiglu_bwd(torch::Tensor in, torch::Tensor dout, torch::Tensor din, int64_t rows, int64_t F) {
  const c10::cuda::CUDAGuard guard(in.device());
  check(rb_swiglu_bwd(in.data_ptr(), dout.data_ptr(), din.data_ptr(), rows, (int)F, dtype_code(in), cur_stream()),
        "rb_swiglu_bwd");
}
void adam(torch::Tensor p, torch::Tensor master, torch::Tensor g, torch::Tensor m, torch::Tensor v, int64_t step,
          double lr, double b1, double b2, double eps, double wd, double gscale, bool split) {
  const c10::cuda::CUDAGuard guard(p.device());
  TORCH_CHECK(p.scalar_type() == at::kBFloat16, "fused adam expects bf16 parameters");
  check(rb_adam(p.data_ptr(), master.data_ptr(), g.data_ptr(), m.data_ptr<float>(), v.data_ptr<float>(), p.numel(),
                (int)step, (float)lr, (float)b1, (float)b2, (float)eps, (float)wd, (float)gscale, split,
                g.scalar_type() == at::kFloat, cur_stream()),
        "rb_adam");
}
void sumsq(torch::Tensor g, torch::Tensor out) {
  const c10::cuda::CUDAGuard guard(g.device());
  check(rb_sumsq(g.data_ptr(), g.numel(), out.data_ptr<float>(), dtype_code(g), cur_stream()), "rb_sumsq");
}
void copy_table(torch::Tensor table, int64_t n_desc, torch::Tensor chunk_start, int64_t total_chunks, int64_t chunk_rows,
                int64_t elem_size) {
  const c10::cuda::CUDAGuard guard(table.device());
  check(rb_copy_table(table.data_ptr(), (int)n_desc, chunk_start.data_ptr<int>(), (int)total_chunks, (int)chunk_rows,
                      (int)elem_size, cur_stream()),
        "rb_copy_table");
}
void kv_scatter(torch::Tensor k, torch::Tensor v, torch::Tensor kc, torch::Tensor vc, torch::Tensor slots, int64_t tokens,
                int64_t row_elems, int64_t k_stride, int64_t v_stride) {
  const c10::cuda::CUDAGuard guard(k.device());
  check(rb_kv_scatter(k.data_ptr(), v.data_ptr(), kc.data_ptr(), vc.data_ptr(), (const long long*)slots.data_ptr<int64_t>(),
                      (int)tokens, (int)row_elems, k_stride, v_stride, dtype_code(k), cur_stream()),
        "rb_kv_scatter");
}
void int4_fake_quant(torch::Tensor x, torch::Tensor out, torch::Tensor scale, torch::Tensor zero, int64_t bm, int64_t bn,
                     bool sym) {
  const c10::cuda::CUDAGuard guard(x.device());
  check(rb_int4_fake_quant(x.data_ptr(), out.data_ptr(), scale.data_ptr(), zero.data_ptr(), (int)x.size(0), (int)x.size(1),
                           (int)bm, (int)bn, sym, dtype_code(x), cur_stream()),
        "rb_int4_fake_quant");
}
void fp8_block_cast(torch::Tensor w, torch::Tensor q, torch::Tensor scale, int64_t block, bool ue8m0) {
  const c10::cuda::CUDAGuard guard(w.device());
  check(rb_fp8_block_cast(w.data_ptr(), q.data_ptr(), scale.data_ptr<float>(), (int)w.size(0), (int)w.size(1), (int)block,
                          ue8m0, dtype_code(w), cur_stream()),
        "rb_fp8_block_cast");
}
void fp8_block_dequant(torch::Tensor q, torch::Tensor scale, torch::Tensor out, int64_t block) {
  const c10::cuda::CUDAGuard guard(q.device());
  check(rb_fp8_block_dequant(q.data_ptr(), scale.data_ptr<float>(), out.data_ptr(), (int)q.size(0), (int)q.size(1),
                             (int)block, dtype_code(out), cur_stream()),
        "rb_fp8_block_dequant");
}

}  // namespace

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m) {
  m.def("install_crash_handler", &install_crash_handler);
  m.def("launch_count", []() { return (int64_t)rb_launch_count(); });
  m.def("reset_launch_count", []() { rb_reset_launch_count(); });
  m.def("gemm", &gemm);
  m.def("gemm_pair", &gemm_pair);
  m.def("rmsnorm_fwd", &rmsnorm_fwd);
  m.def("rmsnorm_bwd_parts", &rmsnorm_bwd_parts);
  m.def("rmsnorm_bwd", &rmsnorm_bwd);
  m.def("rope", &rope);
  m.def("swiglu_fwd", &swiglu_fwd);
  m.def("swiglu_bwd", &swiglu_bwd);
  m.def("adam", &adam);
  m.def("sumsq", &sumsq);
  m.def("copy_table", &copy_table);
  m.def("kv_scatter", &kv_scatter);
  m.def("int4_fake_quant", &int4_fake_quant);
  m.def("fp8_block_cast", &fp8_block_cast);
  m.def("fp8_block_dequant", &fp8_block_dequant);
  register_more(m);
}
