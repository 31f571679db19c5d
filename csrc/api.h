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
