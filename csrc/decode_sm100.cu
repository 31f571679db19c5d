// Rollout-side kernels: paged-KV decode attention (split-KV, GQA), token sampling
// (temperature / top-k / top-p with log-prob of the sampled token), MoE router
// softmax + top-k.  These are bandwidth- or latency-bound and use CUDA cores.
#include "common.cuh"
#include "host_utils.h"

namespace rb {

// ----------------------------------------------------------------------------- paged decode attention
// q [B][Hq][128]; caches [num_blocks][block_size][Hkv][128]; one CTA per (sequence, kv head, split).
// Phase A: thread-per-token scores for the G query heads of the group (q broadcast from shared memory).
// Phase B: lane-per-4-dims accumulation of P*V.  Partials (m, l, o) go to scratch when split > 1.
constexpr int DA_D = 128;
constexpr int DA_CHUNK = 256;    // tokens per inner iteration
constexpr int DA_THREADS = 128;
constexpr int DA_MAXG = 8;

template <int G>
__global__ void __launch_bounds__(DA_THREADS)
decode_attn_kernel(const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ kc,
                   const __nv_bfloat16* __restrict__ vc, const int* __restrict__ block_tables,
                   const int* __restrict__ ctx_lens, __nv_bfloat16* __restrict__ out, float* __restrict__ part_o,
                   float* __restrict__ part_ml, int Hq, int Hkv, int block_size, int max_blocks, float scale_log2,
                   int num_splits, int split_tokens) {
  __shared__ float sq[G][DA_D];
  __shared__ float sc[G][DA_CHUNK];
  __shared__ float red[G][DA_THREADS / 32];
  __shared__ float so[DA_THREADS / 32][G][DA_D];
  const int b = blockIdx.x, kvh = blockIdx.y, split = blockIdx.z;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int ctx = ctx_lens[b];
  const int t_begin = split * split_tokens;
  const int t_end = min(ctx, t_begin + split_tokens);
  const int* bt = block_tables + static_cast<size_t>(b) * max_blocks;
  for (int i = tid; i < G * DA_D; i += DA_THREADS) {
    const int g = i / DA_D, d = i % DA_D;
    sq[g][d] = __bfloat162float(q[(static_cast<size_t>(b) * Hq + kvh * G + g) * DA_D + d]) * scale_log2;
  }
  float m_run[G], l_run[G], acc[G][4];
#pragma unroll
  for (int g = 0; g < G; ++g) {
    m_run[g] = -1e30f; l_run[g] = 0.f;
    acc[g][0] = acc[g][1] = acc[g][2] = acc[g][3] = 0.f;
  }
  __syncthreads();
  const size_t tok_stride = static_cast<size_t>(Hkv) * DA_D;
  for (int c0 = t_begin; c0 < t_end; c0 += DA_CHUNK) {
    const int n = min(DA_CHUNK, t_end - c0);
    // ---- phase A: scores
    for (int tt = tid; tt < DA_CHUNK; tt += DA_THREADS) {
      float s[G];
#pragma unroll
      for (int g = 0; g < G; ++g) s[g] = 0.f;
      if (tt < n) {
        const int tok = c0 + tt;
        const size_t row = (static_cast<size_t>(bt[tok / block_size]) * block_size + tok % block_size) * tok_stride + kvh * DA_D;
        const uint4* kp = reinterpret_cast<const uint4*>(kc + row);
#pragma unroll 4
        for (int v = 0; v < DA_D / 8; ++v) {
          const uint4 kk = kp[v];
          const __nv_bfloat162* k2 = reinterpret_cast<const __nv_bfloat162*>(&kk);
#pragma unroll
          for (int u = 0; u < 4; ++u) {
            const float k0 = __low2float(k2[u]), k1 = __high2float(k2[u]);
#pragma unroll
            for (int g = 0; g < G; ++g) s[g] += k0 * sq[g][v * 8 + 2 * u] + k1 * sq[g][v * 8 + 2 * u + 1];
          }
        }
      }
#pragma unroll
      for (int g = 0; g < G; ++g) sc[g][tt] = (tt < n) ? s[g] : -1e30f;
    }
    __syncthreads();
    // ---- chunk max per head
    float mx[G];
#pragma unroll
    for (int g = 0; g < G; ++g) {
      float v = fmaxf(sc[g][tid], sc[g][tid + DA_THREADS]);
      v = warp_max(v);
      if (lane == 0) red[g][warp] = v;
    }
    __syncthreads();
#pragma unroll
    for (int g = 0; g < G; ++g) {
      float v = red[g][0];
#pragma unroll
      for (int w = 1; w < DA_THREADS / 32; ++w) v = fmaxf(v, red[g][w]);
      mx[g] = fmaxf(m_run[g], v);
    }
    __syncthreads();
    // ---- exponentiate in place, chunk sums
#pragma unroll
    for (int g = 0; g < G; ++g) {
      float s = 0.f;
      for (int tt = tid; tt < DA_CHUNK; tt += DA_THREADS) {
        const float e = (tt < n) ? exp2f(sc[g][tt] - mx[g]) : 0.f;
        sc[g][tt] = e;
        s += e;
      }
      s = warp_sum(s);
      if (lane == 0) red[g][warp] = s;
    }
    __syncthreads();
#pragma unroll
    for (int g = 0; g < G; ++g) {
      float s = 0.f;
#pragma unroll
      for (int w = 0; w < DA_THREADS / 32; ++w) s += red[g][w];
      const float alpha = exp2f(m_run[g] - mx[g]);
      l_run[g] = l_run[g] * alpha + s;
      m_run[g] = mx[g];
#pragma unroll
      for (int k = 0; k < 4; ++k) acc[g][k] *= alpha;
    }
    // ---- phase B: P*V, each warp takes every 4th token, lane owns dims [4*lane, 4*lane+4)
    for (int tt = warp; tt < n; tt += DA_THREADS / 32) {
      const int tok = c0 + tt;
      const size_t row = (static_cast<size_t>(bt[tok / block_size]) * block_size + tok % block_size) * tok_stride + kvh * DA_D;
      const uint2 vv = reinterpret_cast<const uint2*>(vc + row)[lane];
      const __nv_bfloat162 v01 = *reinterpret_cast<const __nv_bfloat162*>(&vv.x), v23 = *reinterpret_cast<const __nv_bfloat162*>(&vv.y);
      const float f0 = __low2float(v01), f1 = __high2float(v01), f2 = __low2float(v23), f3 = __high2float(v23);
#pragma unroll
      for (int g = 0; g < G; ++g) {
        const float pw = sc[g][tt];
        acc[g][0] += pw * f0; acc[g][1] += pw * f1; acc[g][2] += pw * f2; acc[g][3] += pw * f3;
      }
    }
    __syncthreads();
  }
  // ---- combine the four warps
#pragma unroll
  for (int g = 0; g < G; ++g) {
    so[warp][g][lane * 4 + 0] = acc[g][0]; so[warp][g][lane * 4 + 1] = acc[g][1];
    so[warp][g][lane * 4 + 2] = acc[g][2]; so[warp][g][lane * 4 + 3] = acc[g][3];
  }
  __syncthreads();
  for (int i = tid; i < G * DA_D; i += DA_THREADS) {
    const int g = i / DA_D, d = i % DA_D;
    float o = 0.f;
#pragma unroll
    for (int w = 0; w < DA_THREADS / 32; ++w) o += so[w][g][d];
    const int hq = kvh * G + g;
    if (num_splits == 1) {
      const float l = l_run[g];
      out[(static_cast<size_t>(b) * Hq + hq) * DA_D + d] = __float2bfloat16(l > 0.f ? o / l : 0.f);
    } else {
      const size_t pidx = (static_cast<size_t>(b) * Hq + hq) * num_splits + split;
      part_o[pidx * DA_D + d] = o;
      if (d == 0) { part_ml[pidx * 2] = m_run[g]; part_ml[pidx * 2 + 1] = l_run[g]; }
    }
  }
}

__global__ void decode_attn_combine_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml,
                                           __nv_bfloat16* __restrict__ out, int num_splits) {
  const size_t bh = blockIdx.x;
  const int d = threadIdx.x;
  float m = -1e30f;
  for (int s = 0; s < num_splits; ++s) m = fmaxf(m, part_ml[(bh * num_splits + s) * 2]);
  float l = 0.f, o = 0.f;
  for (int s = 0; s < num_splits; ++s) {
    const float w = exp2f(part_ml[(bh * num_splits + s) * 2] - m);
    l += w * part_ml[(bh * num_splits + s) * 2 + 1];
    o += w * part_o[(bh * num_splits + s) * DA_D + d];
  }
  out[bh * DA_D + d] = __float2bfloat16(l > 0.f ? o / l : 0.f);
}

// ----------------------------------------------------------------------------- sampling
// One CTA per row of fp32 logits.  Filters: top-k (k largest), then top-p (smallest prefix of the
// descending order whose mass reaches p), both realised as a probability threshold found by
// bisection; the token is then drawn by inverse CDF in vocabulary order over the kept entries.
// log-prob returned is that of the unfiltered temperature-scaled distribution.
constexpr int SM_THREADS = 1024;

__device__ __forceinline__ float block_reduce_sum(float v, float* sh) {
  v = warp_sum(v);
  if ((threadIdx.x & 31) == 0) sh[threadIdx.x >> 5] = v;
  __syncthreads();
  float s = 0.f;
  for (int i = 0; i < SM_THREADS / 32; ++i) s += sh[i];
  __syncthreads();
  return s;
}
__device__ __forceinline__ float block_reduce_max(float v, float* sh) {
  v = warp_max(v);
  if ((threadIdx.x & 31) == 0) sh[threadIdx.x >> 5] = v;
  __syncthreads();
  float s = -INFINITY;
  for (int i = 0; i < SM_THREADS / 32; ++i) s = fmaxf(s, sh[i]);
  __syncthreads();
  return s;
}

__global__ void __launch_bounds__(SM_THREADS)
sample_kernel(const float* __restrict__ logits, int V, int ld, const float* __restrict__ temperature,
              const long long* __restrict__ top_k, const float* __restrict__ top_p, const float* __restrict__ uniform,
              long long* __restrict__ tok_out, float* __restrict__ logp_out) {
  __shared__ float sh[SM_THREADS / 32];
  __shared__ float seg[SM_THREADS];
  __shared__ int pick;
  __shared__ float resid_sh;
  const int row = blockIdx.x, tid = threadIdx.x;
  const float* z = logits + static_cast<size_t>(row) * ld;
  const float temp = temperature[row];
  const bool greedy = temp <= 0.f;
  const float inv_t = 1.f / fmaxf(temp, 1e-6f);
  // contiguous segment per thread so that the CDF walks the vocabulary in order
  const int per = (V + SM_THREADS - 1) / SM_THREADS;
  const int lo = min(V, tid * per), hi = min(V, lo + per);
  float mx = -INFINITY;
  int amax = lo;
  for (int i = lo; i < hi; ++i) { const float v = z[i] * inv_t; if (v > mx) { mx = v; amax = i; } }
  const float gmax = block_reduce_max(mx, sh);
  float s = 0.f;
  for (int i = lo; i < hi; ++i) s += __expf(z[i] * inv_t - gmax);
  const float total = block_reduce_sum(s, sh);
  const float log_total = __logf(total);
  if (greedy) {
    // smallest index among the maxima
    seg[tid] = (mx == gmax) ? static_cast<float>(amax) : 3e38f;
    __syncthreads();
    for (int o = SM_THREADS / 2; o > 0; o >>= 1) { if (tid < o) seg[tid] = fminf(seg[tid], seg[tid + o]); __syncthreads(); }
    if (tid == 0) { const int t = static_cast<int>(seg[0]); tok_out[row] = t; logp_out[row] = z[t] * inv_t - gmax - log_total; }
    return;
  }
  // ---- threshold (in units of exp(z - gmax)) such that kept = {e >= thr}
  float thr = 0.f;
  const long long k = top_k[row];
  const float pp = top_p[row];
  if (k > 0 && k < V) {
    float a = 0.f, b = 1.f;  // count(e >= a) > k >= count(e >= b) is maintained; e in (0, 1]
    for (int itn = 0; itn < 32; ++itn) {
      const float mid = 0.5f * (a + b);
      float c = 0.f;
      for (int i = lo; i < hi; ++i) c += (__expf(z[i] * inv_t - gmax) >= mid) ? 1.f : 0.f;
      c = block_reduce_sum(c, sh);
      if (c > static_cast<float>(k)) a = mid; else b = mid;
    }
    thr = b;
  }
  if (pp < 1.f) {
    // largest threshold t >= thr whose kept mass (within the top-k set) is still >= p * mass(top-k set)
    float kept = 0.f;
    for (int i = lo; i < hi; ++i) { const float e = __expf(z[i] * inv_t - gmax); kept += (e >= thr) ? e : 0.f; }
    kept = block_reduce_sum(kept, sh);
    const float need = pp * kept;
    float a = thr, b = 1.0000001f;  // mass(e >= a) >= need > mass(e >= b)
    for (int itn = 0; itn < 32; ++itn) {
      const float mid = 0.5f * (a + b);
      float msum = 0.f;
      for (int i = lo; i < hi; ++i) { const float e = __expf(z[i] * inv_t - gmax); msum += (e >= mid) ? e : 0.f; }
      msum = block_reduce_sum(msum, sh);
      if (msum >= need) a = mid; else b = mid;
    }
    thr = a;
  }
  // ---- inverse CDF over kept entries in vocabulary order
  float mine = 0.f;
  for (int i = lo; i < hi; ++i) { const float e = __expf(z[i] * inv_t - gmax); mine += (e >= thr) ? e : 0.f; }
  seg[tid] = mine;
  __syncthreads();
  if (tid == 0) {
    float tot = 0.f;
    for (int i = 0; i < SM_THREADS; ++i) tot += seg[i];
    const float target = uniform[row] * tot;
    float run = 0.f;
    int t = -1, last = 0;
    for (int i = 0; i < SM_THREADS; ++i) {
      if (seg[i] > 0.f) {
        last = i;
        if (run + seg[i] > target) { t = i; break; }
      }
      run += seg[i];
    }
    if (t < 0) {  // rounding pushed the target past the end: take the last non-empty segment
      t = last;
      run = 0.f;
      for (int i = 0; i < t; ++i) run += seg[i];
    }
    pick = t;
    resid_sh = target - run;
  }
  __syncthreads();
  if (tid == pick) {
    const float resid = resid_sh;
    float run = 0.f;
    int t = -1, last = -1;
    for (int i = lo; i < hi; ++i) {
      const float e = __expf(z[i] * inv_t - gmax);
      if (e >= thr) { last = i; run += e; if (run > resid) { t = i; break; } }
    }
    if (t < 0) t = last;
    tok_out[row] = t;
    logp_out[row] = z[t] * inv_t - gmax - log_total;
  }
}

// ----------------------------------------------------------------------------- MoE router: softmax + top-k, one warp per token
__global__ void topk_router_kernel(const float* __restrict__ logits, int E, int K, int norm, float* __restrict__ w_out,
                                   long long* __restrict__ idx_out, float* __restrict__ probs_out, int T) {
  const int warps = blockDim.x >> 5, lane = threadIdx.x & 31;
  for (int t = blockIdx.x * warps + (threadIdx.x >> 5); t < T; t += gridDim.x * warps) {
    const float* z = logits + static_cast<size_t>(t) * E;
    float mx = -INFINITY;
    for (int e = lane; e < E; e += 32) mx = fmaxf(mx, z[e]);
    mx = warp_max(mx);
    float s = 0.f;
    for (int e = lane; e < E; e += 32) s += __expf(z[e] - mx);
    s = warp_sum(s);
    const float inv = 1.f / s;
    // each lane holds up to 8 experts (E <= 256)
    float pv[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const int e = lane + 32 * j;
      pv[j] = (e < E) ? __expf(z[e] - mx) * inv : -1.f;
      if (probs_out && e < E) probs_out[static_cast<size_t>(t) * E + e] = pv[j];
    }
    float wsum = 0.f;
    float wsel[8];
    int isel[8];
    for (int k = 0; k < K; ++k) {
      float best = -1.f;
      int bi = 0x7fffffff;
#pragma unroll
      for (int j = 0; j < 8; ++j) if (pv[j] > best) { best = pv[j]; bi = lane + 32 * j; }
      // warp arg-max, ties to the smaller expert index
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        const float ob = __shfl_xor_sync(0xffffffffu, best, o);
        const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
        if (ob > best || (ob == best && oi < bi)) { best = ob; bi = oi; }
      }
      if ((bi & 31) == lane) pv[bi >> 5] = -1.f;
      if (k < 8) { wsel[k] = best; isel[k] = bi; }
      wsum += best;
    }
    if (lane == 0) {
      for (int k = 0; k < K && k < 8; ++k) {
        w_out[static_cast<size_t>(t) * K + k] = norm ? wsel[k] / wsum : wsel[k];
        idx_out[static_cast<size_t>(t) * K + k] = isel[k];
      }
    }
  }
}

}  // namespace rb

using namespace rb;

extern "C" int rb_decode_attn_splits(int B, int Hkv, int max_ctx) {
  // enough CTAs to fill the machine twice, at least 512 tokens per split
  int splits = 1;
  const int base = B * Hkv;
  while (base * splits < 2 * num_sms() && (max_ctx + splits - 1) / splits > 512 && splits < 32) splits *= 2;
  return splits;
}

// scratch (only when splits > 1): part_o fp32 [B*Hq*splits*128], part_ml fp32 [B*Hq*splits*2]
extern "C" int rb_decode_attn_v1(const void* q, const void* kc, const void* vc, const int* block_tables, const int* ctx_lens,
                              void* out, float* part_o, float* part_ml, int B, int Hq, int Hkv, int block_size,
                              int max_blocks, int max_ctx, float scale, int splits, cudaStream_t st) {
  if (B == 0) return 0;
  const int G = Hq / Hkv;
  if (Hq % Hkv || G > DA_MAXG) return -2;
  const int split_tokens = ((max_ctx + splits - 1) / splits + DA_CHUNK - 1) / DA_CHUNK * DA_CHUNK;
  dim3 grid(B, Hkv, splits);
  const float sl2 = scale * 1.4426950408889634f;
#define RB_DA(G_)                                                                                                     \
  decode_attn_kernel<G_><<<grid, DA_THREADS, 0, st>>>((const __nv_bfloat16*)q, (const __nv_bfloat16*)kc,              \
                                                      (const __nv_bfloat16*)vc, block_tables, ctx_lens,               \
                                                      (__nv_bfloat16*)out, part_o, part_ml, Hq, Hkv, block_size,     \
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
  if (splits > 1) decode_attn_combine_kernel<<<B * Hq, DA_D, 0, st>>>(part_o, part_ml, (__nv_bfloat16*)out, splits);
  rb_note_launch(1);
  return (int)cudaGetLastError();
}

extern "C" int rb_sample(const float* logits, int B, int V, int ld, const float* temperature, const long long* top_k,
                         const float* top_p, const float* uniform, long long* tok, float* logp, cudaStream_t st) {
  if (B == 0) return 0;
  sample_kernel<<<B, SM_THREADS, 0, st>>>(logits, V, ld, temperature, top_k, top_p, uniform, tok, logp);
  rb_note_launch(1);
  return (int)cudaGetLastError();
}

extern "C" int rb_topk_router(const float* logits, int T, int E, int K, int norm, float* w, long long* idx, float* probs,
                              cudaStream_t st) {
  if (T == 0) return 0;
  if (E > 256 || K > 8) return -2;
  int blocks = (T + 7) / 8;
  if (blocks > num_sms() * 8) blocks = num_sms() * 8;
  topk_router_kernel<<<blocks, 256, 0, st>>>(logits, E, K, norm, w, idx, probs, T);
  rb_note_launch(1);
  return (int)cudaGetLastError();
}
