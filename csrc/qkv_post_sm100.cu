// Decode/prefill glue kernels of the rollout engine that replace chains of small launches.
//
// rb_qkv_post: one pass over the fused QKV projection output of a layer:
//   per-head RMSNorm of q and k (Qwen3 "qk layernorm", optional) -> rotary embedding (rotate-half)
//   -> q to a packed [T][nq][128] tensor, k/v to the paged KV cache rows slots[T] and, when asked
//   (prefill needs them for the varlen attention), to packed [T][nkv][128] tensors.
// It stands for five launches (q norm, k norm, rope q, rope k, cache scatter).  One warp handles one
// (token, head): 128 dims = 4 per lane, so the norm is a warp reduction and the rotation partner
// (dim +-64) sits 16 lanes away.
//
// rb_splitk_swiglu: the split-K reduction of the gate/up projection fused with SwiGLU:
//   out[m][f] = silu(sum_s ws[s][m][f]) * (sum_s ws[s][m][F+f]).
#include "common.cuh"
#include "host_utils.h"

namespace rb {

__device__ __forceinline__ float bf16_round(float x) { return __bfloat162float(__float2bfloat16(x)); }

template <bool NORM>
__global__ void qkv_post_kernel(const __nv_bfloat16* __restrict__ qkv, int ld, const __nv_bfloat16* __restrict__ qw,
                                const __nv_bfloat16* __restrict__ kw, const float* __restrict__ cos_t,
                                const float* __restrict__ sin_t, __nv_bfloat16* __restrict__ q_out,
                                __nv_bfloat16* __restrict__ k_out, __nv_bfloat16* __restrict__ v_out,
                                __nv_bfloat16* __restrict__ k_cache, __nv_bfloat16* __restrict__ v_cache,
                                const long long* __restrict__ slots, int T, int nq, int nkv, float eps) {
  const int heads = nq + 2 * nkv;
  const int lane = threadIdx.x & 31;
  const long long w = blockIdx.x * static_cast<long long>(blockDim.x >> 5) + (threadIdx.x >> 5);
  griddep_wait();                    // qkv comes from the GEMM before this kernel
  if (w >= static_cast<long long>(T) * heads) return;
  const int t = static_cast<int>(w / heads), h = static_cast<int>(w % heads);
  const uint2 raw = *reinterpret_cast<const uint2*>(qkv + static_cast<size_t>(t) * ld + h * 128 + lane * 4);
  uint2 outv = raw;
  if (h < nq + nkv) {
    const __nv_bfloat162 a0 = *reinterpret_cast<const __nv_bfloat162*>(&raw.x);
    const __nv_bfloat162 a1 = *reinterpret_cast<const __nv_bfloat162*>(&raw.y);
    float x[4] = {__low2float(a0), __high2float(a0), __low2float(a1), __high2float(a1)};
    if constexpr (NORM) {
      float ss = x[0] * x[0] + x[1] * x[1] + x[2] * x[2] + x[3] * x[3];
      ss = warp_sum(ss);
      const float rstd = rsqrtf(ss * (1.f / 128.f) + eps);
      const uint2 wr = *reinterpret_cast<const uint2*>((h < nq ? qw : kw) + lane * 4);
      const __nv_bfloat162 w0 = *reinterpret_cast<const __nv_bfloat162*>(&wr.x);
      const __nv_bfloat162 w1 = *reinterpret_cast<const __nv_bfloat162*>(&wr.y);
      // rounded to bf16 like the separate norm kernel, so both paths agree bit for bit
      x[0] = bf16_round(x[0] * rstd * __low2float(w0));
      x[1] = bf16_round(x[1] * rstd * __high2float(w0));
      x[2] = bf16_round(x[2] * rstd * __low2float(w1));
      x[3] = bf16_round(x[3] * rstd * __high2float(w1));
    }
    const int j = (lane & 15) * 4;  // frequency index of this lane's 4 dims
    const float4 c = *reinterpret_cast<const float4*>(cos_t + static_cast<size_t>(t) * 64 + j);
    const float4 s = *reinterpret_cast<const float4*>(sin_t + static_cast<size_t>(t) * 64 + j);
    const float cs[4] = {c.x, c.y, c.z, c.w}, sn[4] = {s.x, s.y, s.z, s.w};
    float y[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float other = __shfl_xor_sync(0xffffffffu, x[i], 16);
      y[i] = (lane < 16) ? x[i] * cs[i] - other * sn[i] : x[i] * cs[i] + other * sn[i];
    }
    outv.x = pack_bf16(y[0], y[1]);
    outv.y = pack_bf16(y[2], y[3]);
  }
  if (h < nq) {
    *reinterpret_cast<uint2*>(q_out + (static_cast<size_t>(t) * nq + h) * 128 + lane * 4) = outv;
    return;
  }
  const bool is_k = h < nq + nkv;
  const int hk = is_k ? h - nq : h - nq - nkv;
  __nv_bfloat16* dense = is_k ? k_out : v_out;
  if (dense) *reinterpret_cast<uint2*>(dense + (static_cast<size_t>(t) * nkv + hk) * 128 + lane * 4) = outv;
  if (slots) {
    const long long slot = slots[t];
    if (slot >= 0) {
      __nv_bfloat16* cache = is_k ? k_cache : v_cache;
      *reinterpret_cast<uint2*>(cache + (static_cast<size_t>(slot) * nkv + hk) * 128 + lane * 4) = outv;
    }
  }
}

__global__ void splitk_swiglu_kernel(const float* __restrict__ ws, __nv_bfloat16* __restrict__ out, int M, int F, int splits) {
  const long long total = static_cast<long long>(M) * (F / 4);
  const size_t slot = static_cast<size_t>(M) * 2 * F;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const int m = static_cast<int>(i / (F / 4)), f = static_cast<int>(i % (F / 4)) * 4;
    float4 g = make_float4(0.f, 0.f, 0.f, 0.f), u = g;
    for (int s = 0; s < splits; ++s) {
      const float* row = ws + s * slot + static_cast<size_t>(m) * 2 * F;
      const float4 a = *reinterpret_cast<const float4*>(row + f);
      const float4 b = *reinterpret_cast<const float4*>(row + F + f);
      g.x += a.x; g.y += a.y; g.z += a.z; g.w += a.w;
      u.x += b.x; u.y += b.y; u.z += b.z; u.w += b.w;
    }
    // the unfused path rounds the GEMM output to bf16 before the activation: keep that
    const float gx = bf16_round(g.x), gy = bf16_round(g.y), gz = bf16_round(g.z), gw = bf16_round(g.w);
    const float ux = bf16_round(u.x), uy = bf16_round(u.y), uz = bf16_round(u.z), uw = bf16_round(u.w);
    uint2 pk;
    pk.x = pack_bf16(gx / (1.f + __expf(-gx)) * ux, gy / (1.f + __expf(-gy)) * uy);
    pk.y = pack_bf16(gz / (1.f + __expf(-gz)) * uz, gw / (1.f + __expf(-gw)) * uw);
    *reinterpret_cast<uint2*>(out + static_cast<size_t>(m) * F + f) = pk;
  }
}

}  // namespace rb

extern "C" int rb_qkv_post(const void* qkv, int ld, const void* qw, const void* kw, const float* cos_t, const float* sin_t,
                           void* q_out, void* k_out, void* v_out, void* k_cache, void* v_cache, const long long* slots, int T,
                           int nq, int nkv, float eps, cudaStream_t st) {
  using namespace rb;
  if (T == 0) return 0;
  if ((ld % 4) || (qw == nullptr) != (kw == nullptr)) return -2;
  const long long warps = static_cast<long long>(T) * (nq + 2 * nkv);
  const int grid = static_cast<int>((warps + 7) / 8);
  auto* x = reinterpret_cast<const __nv_bfloat16*>(qkv);
  if (qw)
    launch_pdl(qkv_post_kernel<true>, dim3(grid), dim3(256), 0, st, x, ld, (const __nv_bfloat16*)qw, (const __nv_bfloat16*)kw,
               cos_t, sin_t, (__nv_bfloat16*)q_out, (__nv_bfloat16*)k_out, (__nv_bfloat16*)v_out, (__nv_bfloat16*)k_cache,
               (__nv_bfloat16*)v_cache, slots, T, nq, nkv, eps);
  else
    launch_pdl(qkv_post_kernel<false>, dim3(grid), dim3(256), 0, st, x, ld, (const __nv_bfloat16*)nullptr,
               (const __nv_bfloat16*)nullptr, cos_t, sin_t, (__nv_bfloat16*)q_out, (__nv_bfloat16*)k_out, (__nv_bfloat16*)v_out,
               (__nv_bfloat16*)k_cache, (__nv_bfloat16*)v_cache, slots, T, nq, nkv, eps);
  rb_note_launch(1);
  return static_cast<int>(cudaGetLastError());
}

extern "C" int rb_splitk_swiglu(const float* ws, void* out, int M, int F, int splits, cudaStream_t st) {
  using namespace rb;
  if (M == 0) return 0;
  if (F % 4) return -2;
  long long blocks = (static_cast<long long>(M) * (F / 4) + 255) / 256;
  if (blocks > num_sms() * 8LL) blocks = num_sms() * 8LL;
  splitk_swiglu_kernel<<<(int)blocks, 256, 0, st>>>(ws, (__nv_bfloat16*)out, M, F, splits);
  rb_note_launch(1);
  return static_cast<int>(cudaGetLastError());
}
