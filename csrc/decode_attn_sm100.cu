// Paged-KV decode attention, version 2: warp-private online softmax, 4-lane groups.
//
// q [B][Hq][128]; caches [num_blocks][block_size][Hkv][128] bf16.  One CTA per (sequence,
// kv head, split); its four warps each walk a quarter of the split's tokens, eight tokens
// at a time:
//   scores : a group of 4 lanes owns one token; each lane reads 64 contiguous bytes of the K
//            row (4 x 128-bit loads) and accumulates the dot products for the G query heads
//            of the group against q held in shared memory; 2 shuffles finish the dot.
//   softmax: running max / sum per head are warp-private (3 shuffles per head per 8 tokens).
//   P*V    : the eight tokens are visited in turn; the whole warp reads one V row coalesced
//            (8 bytes per lane) and each lane updates its 4 output dims for the G heads.
// The four warps are merged through shared memory at the end; with splits > 1 the partial
// (m, l, o) goes to scratch and a second kernel combines (same layout as version 1).
#include "common.cuh"
#include "host_utils.h"

namespace rb {

constexpr int DB_D = 128;
constexpr int DB_THREADS = 128;
constexpr int DB_WARPS = DB_THREADS / 32;

template <int G>
__global__ void __launch_bounds__(DB_THREADS)
decode_attn2_kernel(const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ kc,
                    const __nv_bfloat16* __restrict__ vc, const int* __restrict__ block_tables,
                    const int* __restrict__ ctx_lens, __nv_bfloat16* __restrict__ out, float* __restrict__ part_o,
                    float* __restrict__ part_ml, int Hq, int Hkv, int block_size, int max_blocks, float scale_log2,
                    int num_splits, int split_tokens) {
  __shared__ __align__(16) float sq[G][DB_D];
  __shared__ float s_m[DB_WARPS][G], s_l[DB_WARPS][G];
  __shared__ __align__(16) float s_o[DB_WARPS][G][DB_D];
  const int b = blockIdx.x, kvh = blockIdx.y, split = blockIdx.z;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int grp = lane >> 2, sub = lane & 3;
  const int ctx = ctx_lens[b];
  const int t_begin = split * split_tokens;
  const int t_end = min(ctx, t_begin + split_tokens);
  const int* bt = block_tables + static_cast<size_t>(b) * max_blocks;
  for (int i = tid; i < G * DB_D; i += DB_THREADS) {
    const int g = i / DB_D, d = i % DB_D;
    sq[g][d] = __bfloat162float(q[(static_cast<size_t>(b) * Hq + kvh * G + g) * DB_D + d]) * scale_log2;
  }
  __syncthreads();
  float m_run[G], l_run[G], acc[G][4];
#pragma unroll
  for (int g = 0; g < G; ++g) {
    m_run[g] = -1e30f; l_run[g] = 0.f;
    acc[g][0] = acc[g][1] = acc[g][2] = acc[g][3] = 0.f;
  }
  const size_t tok_stride = static_cast<size_t>(Hkv) * DB_D;
  // this warp's contiguous token range
  const int span = t_end > t_begin ? t_end - t_begin : 0;
  const int per_warp = ((span + DB_WARPS - 1) / DB_WARPS + 7) & ~7;
  const int w_begin = t_begin + warp * per_warp;
  const int w_end = min(t_end, w_begin + per_warp);
  for (int t0 = w_begin; t0 < w_end; t0 += 8) {
    const int tok = t0 + grp;
    const bool valid = tok < w_end;
    size_t row = 0;
    if (valid) row = (static_cast<size_t>(bt[tok / block_size]) * block_size + tok % block_size) * tok_stride + kvh * DB_D;
    float s[G];
#pragma unroll
    for (int g = 0; g < G; ++g) s[g] = 0.f;
    if (valid) {
      const uint4* kp = reinterpret_cast<const uint4*>(kc + row + sub * 32);
      uint4 kk[4];
#pragma unroll
      for (int v = 0; v < 4; ++v) kk[v] = kp[v];
#pragma unroll
      for (int v = 0; v < 4; ++v) {
        const __nv_bfloat162* k2 = reinterpret_cast<const __nv_bfloat162*>(&kk[v]);
        float kf[8];
#pragma unroll
        for (int u = 0; u < 4; ++u) { kf[2 * u] = __low2float(k2[u]); kf[2 * u + 1] = __high2float(k2[u]); }
#pragma unroll
        for (int g = 0; g < G; ++g) {
          const float4 qa = *reinterpret_cast<const float4*>(&sq[g][sub * 32 + v * 8]);
          const float4 qb = *reinterpret_cast<const float4*>(&sq[g][sub * 32 + v * 8 + 4]);
          s[g] += kf[0] * qa.x + kf[1] * qa.y + kf[2] * qa.z + kf[3] * qa.w + kf[4] * qb.x + kf[5] * qb.y + kf[6] * qb.z + kf[7] * qb.w;
        }
      }
    }
    // prefetch the V rows' addresses: the token of group j is t0 + j
#pragma unroll
    for (int g = 0; g < G; ++g) {
      s[g] += __shfl_xor_sync(0xffffffffu, s[g], 1);
      s[g] += __shfl_xor_sync(0xffffffffu, s[g], 2);
      if (!valid) s[g] = -1e30f;
    }
    float p[G];
#pragma unroll
    for (int g = 0; g < G; ++g) {
      float mx = s[g];
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 4));
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 8));
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 16));
      const float m_new = fmaxf(m_run[g], mx);
      const float alpha = exp2f(m_run[g] - m_new);
      m_run[g] = m_new;
      p[g] = valid ? exp2f(s[g] - m_new) : 0.f;
      float ps = (sub == 0) ? p[g] : 0.f;   // one lane per group contributes to the sum
      ps += __shfl_xor_sync(0xffffffffu, ps, 4);
      ps += __shfl_xor_sync(0xffffffffu, ps, 8);
      ps += __shfl_xor_sync(0xffffffffu, ps, 16);
      ps += __shfl_xor_sync(0xffffffffu, ps, 1);
      ps += __shfl_xor_sync(0xffffffffu, ps, 2);
      l_run[g] = l_run[g] * alpha + ps;
#pragma unroll
      for (int k = 0; k < 4; ++k) acc[g][k] *= alpha;
    }
    // ---- P*V: visit the eight tokens, whole warp reads one V row (8 bytes per lane)
    const int n_here = min(8, w_end - t0);
    uint2 vv[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const size_t rj = __shfl_sync(0xffffffffu, row, j * 4);
      if (j < n_here) vv[j] = reinterpret_cast<const uint2*>(vc + rj)[lane];
    }
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      float pj[G];
#pragma unroll
      for (int g = 0; g < G; ++g) pj[g] = __shfl_sync(0xffffffffu, p[g], j * 4);
      if (j < n_here) {
        const __nv_bfloat162 v01 = *reinterpret_cast<const __nv_bfloat162*>(&vv[j].x);
        const __nv_bfloat162 v23 = *reinterpret_cast<const __nv_bfloat162*>(&vv[j].y);
        const float f0 = __low2float(v01), f1 = __high2float(v01), f2 = __low2float(v23), f3 = __high2float(v23);
#pragma unroll
        for (int g = 0; g < G; ++g) {
          acc[g][0] += pj[g] * f0; acc[g][1] += pj[g] * f1; acc[g][2] += pj[g] * f2; acc[g][3] += pj[g] * f3;
        }
      }
    }
  }
  // ---- merge the four warps
#pragma unroll
  for (int g = 0; g < G; ++g) {
    if (lane == 0) { s_m[warp][g] = m_run[g]; s_l[warp][g] = l_run[g]; }
    *reinterpret_cast<float4*>(&s_o[warp][g][lane * 4]) = make_float4(acc[g][0], acc[g][1], acc[g][2], acc[g][3]);
  }
  __syncthreads();
  for (int i = tid; i < G * DB_D; i += DB_THREADS) {
    const int g = i / DB_D, d = i % DB_D;
    float m = -1e30f;
#pragma unroll
    for (int w = 0; w < DB_WARPS; ++w) m = fmaxf(m, s_m[w][g]);
    float l = 0.f, o = 0.f;
#pragma unroll
    for (int w = 0; w < DB_WARPS; ++w) {
      const float sc = exp2f(s_m[w][g] - m);
      l += sc * s_l[w][g];
      o += sc * s_o[w][g][d];
    }
    const int hq = kvh * G + g;
    if (num_splits == 1) {
      out[(static_cast<size_t>(b) * Hq + hq) * DB_D + d] = __float2bfloat16(l > 0.f ? o / l : 0.f);
    } else {
      const size_t pidx = (static_cast<size_t>(b) * Hq + hq) * num_splits + split;
      part_o[pidx * DB_D + d] = o;
      if (d == 0) { part_ml[pidx * 2] = m; part_ml[pidx * 2 + 1] = l; }
    }
  }
}

__global__ void decode_attn2_combine_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml,
                                            __nv_bfloat16* __restrict__ out, int num_splits) {
  const size_t bh = blockIdx.x;
  const int d = threadIdx.x;
  float m = -1e30f;
  for (int s = 0; s < num_splits; ++s) m = fmaxf(m, part_ml[(bh * num_splits + s) * 2]);
  float l = 0.f, o = 0.f;
  for (int s = 0; s < num_splits; ++s) {
    const float w = exp2f(part_ml[(bh * num_splits + s) * 2] - m);
    l += w * part_ml[(bh * num_splits + s) * 2 + 1];
    o += w * part_o[(bh * num_splits + s) * DB_D + d];
  }
  out[bh * DB_D + d] = __float2bfloat16(l > 0.f ? o / l : 0.f);
}

}  // namespace rb

using namespace rb;

// scratch (only when splits > 1): part_o fp32 [B*Hq*splits*128], part_ml fp32 [B*Hq*splits*2]
extern "C" int rb_decode_attn(const void* q, const void* kc, const void* vc, const int* block_tables, const int* ctx_lens,
                              void* out, float* part_o, float* part_ml, int B, int Hq, int Hkv, int block_size,
                              int max_blocks, int max_ctx, float scale, int splits, cudaStream_t st) {
  if (B == 0) return 0;
  const int G = Hq / Hkv;
  if (Hq % Hkv || G > 8) return -2;
  const int split_tokens = ((max_ctx + splits - 1) / splits + 31) / 32 * 32;
  dim3 grid(B, Hkv, splits);
  const float sl2 = scale * 1.4426950408889634f;
#define RB_DA(G_)                                                                                                     \
  decode_attn2_kernel<G_><<<grid, DB_THREADS, 0, st>>>((const __nv_bfloat16*)q, (const __nv_bfloat16*)kc,             \
                                                       (const __nv_bfloat16*)vc, block_tables, ctx_lens,              \
                                                       (__nv_bfloat16*)out, part_o, part_ml, Hq, Hkv, block_size,    \
                                                       max_blocks, sl2, splits, split_tokens)
  switch (G) {
    case 1: RB_DA(1); break;
    case 2: RB_DA(2); break;
    case 4: RB_DA(4); break;
    case 7: RB_DA(7); break;
    case 8: RB_DA(8); break;
    default: return -3;
  }
#undef RB_DA
  if (splits > 1) decode_attn2_combine_kernel<<<B * Hq, DB_D, 0, st>>>(part_o, part_ml, (__nv_bfloat16*)out, splits);
  rb_note_launch(splits > 1 ? 2 : 1);
  return (int)cudaGetLastError();
}
