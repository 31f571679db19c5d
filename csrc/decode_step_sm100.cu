// Rollout decode-step tail: token sampling with coalesced vocabulary sweeps, and the device-side
// "advance" that turns the sampled tokens into the next step's inputs, so a CUDA graph of one decode step can
// be replayed several times in a row without the host in between.
//
// Sampling semantics (same as the first-generation kernel in decode_sm100.cu): temperature scaling, top-k, then
// top-p inside the top-k set, both realised as a probability threshold found by bisection; the token is drawn by
// inverse CDF in vocabulary order over the kept entries; the returned log-prob is that of the UNFILTERED
// temperature-scaled distribution (what the trainer recomputes).
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <math.h>
#include <stdint.h>

#include "host_utils.h"

namespace rb {

constexpr int SV_THREADS = 1024;
constexpr int SV_WARPS = SV_THREADS / 32;

__device__ __forceinline__ float sv_warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float sv_warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
__device__ __forceinline__ float sv_block_sum(float v, float* sh) {
  v = sv_warp_sum(v);
  if ((threadIdx.x & 31) == 0) sh[threadIdx.x >> 5] = v;
  __syncthreads();
  float s = 0.f;
#pragma unroll
  for (int i = 0; i < SV_WARPS; ++i) s += sh[i];
  __syncthreads();
  return s;
}
__device__ __forceinline__ float sv_block_max(float v, float* sh) {
  v = sv_warp_max(v);
  if ((threadIdx.x & 31) == 0) sh[threadIdx.x >> 5] = v;
  __syncthreads();
  float s = -INFINITY;
#pragma unroll
  for (int i = 0; i < SV_WARPS; ++i) s = fmaxf(s, sh[i]);
  __syncthreads();
  return s;
}

// VEC consecutive logits starting at element `i` of row `z` (i is a multiple of VEC and the row start is aligned
// to VEC elements when VEC > 1); entries at or past `hi` come back as -inf.
template <typename T, int VEC>
__device__ __forceinline__ void sv_load(const T* __restrict__ z, int i, int hi, float (&v)[VEC]) {
  if constexpr (VEC == 1) {
    v[0] = (i < hi) ? static_cast<float>(z[i]) : -INFINITY;
  } else if constexpr (sizeof(T) == 2) {
    static_assert(VEC == 8, "bf16 rows are read 16 bytes at a time");
    if (i + VEC <= hi) {
      const uint4 raw = *reinterpret_cast<const uint4*>(z + i);
      const __nv_bfloat162* p = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 f = __bfloat1622float2(p[j]);
        v[2 * j] = f.x;
        v[2 * j + 1] = f.y;
      }
    } else {
#pragma unroll
      for (int j = 0; j < VEC; ++j) v[j] = (i + j < hi) ? static_cast<float>(z[i + j]) : -INFINITY;
    }
  } else {
    static_assert(VEC == 4, "fp32 rows are read 16 bytes at a time");
    if (i + VEC <= hi) {
      const float4 raw = *reinterpret_cast<const float4*>(z + i);
      v[0] = raw.x; v[1] = raw.y; v[2] = raw.z; v[3] = raw.w;
    } else {
#pragma unroll
      for (int j = 0; j < VEC; ++j) v[j] = (i + j < hi) ? static_cast<float>(z[i + j]) : -INFINITY;
    }
  }
}

// One CTA per row.  Warp w owns the contiguous vocabulary chunk [w*C, (w+1)*C) and sweeps it with coalesced
// 16-byte loads; only the last step (inverse CDF inside the chosen chunk) depends on the order of the entries.
template <typename T, int VEC>
__global__ void __launch_bounds__(SV_THREADS)
sample_v2_kernel(const T* __restrict__ logits, int V, long long ld, const float* __restrict__ temperature,
                 const long long* __restrict__ top_k, const float* __restrict__ top_p, const float* __restrict__ uniform,
                 long long* __restrict__ tok_out, float* __restrict__ logp_out) {
  __shared__ float sh[SV_WARPS];
  __shared__ float seg[SV_WARPS];
  __shared__ int shi[SV_WARPS];
  __shared__ int pick_sh;
  __shared__ float resid_sh;
  const int row = blockIdx.x, tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const T* z = logits + static_cast<size_t>(row) * ld;
  const float temp = temperature[row];
  const bool greedy = temp <= 0.f;
  const float inv_t = 1.f / fmaxf(temp, 1e-6f);
  constexpr int STEP = 32 * VEC;
  const int C = ((V + SV_WARPS - 1) / SV_WARPS + STEP - 1) / STEP * STEP;
  const int lo = min(V, warp * C), hi = min(V, lo + C);

  // ---- pass 1: maximum (and its first index, for greedy rows)
  float mx = -INFINITY;
  int amax = V;
  for (int base = lo + lane * VEC; base < hi; base += STEP) {
    float v[VEC];
    sv_load<T, VEC>(z, base, hi, v);
#pragma unroll
    for (int j = 0; j < VEC; ++j) {
      const float s = v[j] * inv_t;
      if (s > mx) { mx = s; amax = base + j; }
    }
  }
  const float gmax = sv_block_max(mx, sh);
  // ---- pass 2: normaliser
  float s = 0.f;
  for (int base = lo + lane * VEC; base < hi; base += STEP) {
    float v[VEC];
    sv_load<T, VEC>(z, base, hi, v);
#pragma unroll
    for (int j = 0; j < VEC; ++j) s += __expf(v[j] * inv_t - gmax);   // exp(-inf) = 0 for masked entries
  }
  const float total = sv_block_sum(s, sh);
  const float log_total = __logf(total);
  if (greedy) {
    // smallest index among the maxima
    int cand = (mx == gmax) ? amax : V;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) cand = min(cand, __shfl_xor_sync(0xffffffffu, cand, o));
    if (lane == 0) shi[warp] = cand;
    __syncthreads();
    if (tid == 0) {
      int t = V;
      for (int i = 0; i < SV_WARPS; ++i) t = min(t, shi[i]);
      t = min(t, V - 1);
      tok_out[row] = t;
      logp_out[row] = static_cast<float>(z[t]) * inv_t - gmax - log_total;
    }
    return;
  }
  // ---- threshold (in units of exp(z - gmax)) such that kept = {e >= thr}
  float thr = 0.f;
  const long long k = top_k[row];
  const float pp = top_p[row];
  if (k > 0 && k < V) {
    float a = 0.f, b = 1.f;   // count(e >= a) > k >= count(e >= b); e in (0, 1]
    for (int itn = 0; itn < 32; ++itn) {
      const float mid = 0.5f * (a + b);
      float c = 0.f;
      for (int base = lo + lane * VEC; base < hi; base += STEP) {
        float v[VEC];
        sv_load<T, VEC>(z, base, hi, v);
#pragma unroll
        for (int j = 0; j < VEC; ++j) c += (__expf(v[j] * inv_t - gmax) >= mid) ? 1.f : 0.f;
      }
      c = sv_block_sum(c, sh);
      if (c > static_cast<float>(k)) a = mid; else b = mid;
    }
    thr = b;
  }
  if (pp < 1.f) {
    float kept = 0.f;
    for (int base = lo + lane * VEC; base < hi; base += STEP) {
      float v[VEC];
      sv_load<T, VEC>(z, base, hi, v);
#pragma unroll
      for (int j = 0; j < VEC; ++j) { const float e = __expf(v[j] * inv_t - gmax); kept += (e >= thr) ? e : 0.f; }
    }
    kept = sv_block_sum(kept, sh);
    const float need = pp * kept;
    float a = thr, b = 1.0000001f;   // mass(e >= a) >= need > mass(e >= b)
    for (int itn = 0; itn < 32; ++itn) {
      const float mid = 0.5f * (a + b);
      float msum = 0.f;
      for (int base = lo + lane * VEC; base < hi; base += STEP) {
        float v[VEC];
        sv_load<T, VEC>(z, base, hi, v);
#pragma unroll
        for (int j = 0; j < VEC; ++j) { const float e = __expf(v[j] * inv_t - gmax); msum += (e >= mid) ? e : 0.f; }
      }
      msum = sv_block_sum(msum, sh);
      if (msum >= need) a = mid; else b = mid;
    }
    thr = a;
  }
  // ---- kept mass per warp chunk, then the chunk that holds the target
  float mine = 0.f;
  for (int base = lo + lane * VEC; base < hi; base += STEP) {
    float v[VEC];
    sv_load<T, VEC>(z, base, hi, v);
#pragma unroll
    for (int j = 0; j < VEC; ++j) { const float e = __expf(v[j] * inv_t - gmax); mine += (e >= thr) ? e : 0.f; }
  }
  mine = sv_warp_sum(mine);
  if (lane == 0) seg[warp] = mine;
  __syncthreads();
  if (tid == 0) {
    float tot = 0.f;
    for (int i = 0; i < SV_WARPS; ++i) tot += seg[i];
    const float target = uniform[row] * tot;
    float run = 0.f;
    int t = -1, last = 0;
    for (int i = 0; i < SV_WARPS; ++i) {
      if (seg[i] > 0.f) {
        last = i;
        if (run + seg[i] > target) { t = i; break; }
      }
      run += seg[i];
    }
    if (t < 0) {   // rounding pushed the target past the end: take the last non-empty chunk
      t = last;
      run = 0.f;
      for (int i = 0; i < t; ++i) run += seg[i];
    }
    pick_sh = t;
    resid_sh = target - run;
  }
  __syncthreads();
  if (warp != pick_sh) return;
  // ---- inverse CDF inside the chosen chunk: 32*VEC entries per iteration, warp prefix sums
  const float resid = resid_sh;
  float run = 0.f;
  int found = -1, last_kept = -1;
  for (int base0 = lo; base0 < hi && found < 0; base0 += STEP) {
    const int base = base0 + lane * VEC;
    float v[VEC], e[VEC];
    sv_load<T, VEC>(z, base, hi, v);
    float lsum = 0.f;
    int llast = -1;
#pragma unroll
    for (int j = 0; j < VEC; ++j) {
      const float x = __expf(v[j] * inv_t - gmax);
      e[j] = (x >= thr && base + j < hi) ? x : 0.f;
      if (e[j] > 0.f) llast = base + j;
      lsum += e[j];
    }
    float incl = lsum;   // inclusive prefix over lanes
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const float n = __shfl_up_sync(0xffffffffu, incl, o);
      if (lane >= o) incl += n;
    }
    const bool cross = (lsum > 0.f) && (run + incl > resid);
    const unsigned ball = __ballot_sync(0xffffffffu, cross);
    int wl = llast;   // last kept index seen so far in this iteration (max over lanes)
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) wl = max(wl, __shfl_xor_sync(0xffffffffu, wl, o));
    if (ball) {
      const int src = __ffs(ball) - 1;
      int t = -1;
      if (lane == src) {
        float r = run + incl - lsum;
        int lk = -1;
#pragma unroll
        for (int j = 0; j < VEC; ++j) {
          if (e[j] > 0.f) { lk = base + j; r += e[j]; if (t < 0 && r > resid) t = base + j; }
        }
        if (t < 0) t = lk;
      }
      found = __shfl_sync(0xffffffffu, t, src);
    } else {
      run += __shfl_sync(0xffffffffu, incl, 31);
      if (wl >= 0) last_kept = wl;
    }
  }
  if (lane == 0) {
    int t = found >= 0 ? found : last_kept;
    if (t < 0) t = min(max(lo, 0), V - 1);   // an empty chunk cannot be picked; defensive
    tok_out[row] = t;
    logp_out[row] = static_cast<float>(z[t]) * inv_t - gmax - log_total;
  }
}

// ----------------------------------------------------------------------------- decode advance
// One CTA (B <= 1024 rows).  State of the running batch lives in device memory and is advanced in place:
//   tok_in[r]  next input token         pos[r]    its position          ctx[r]  context length incl. that token
//   slot[r]    KV-cache row of that token (block_table[r][pos / bs] * bs + pos % bs)
//   active[r]  0 once the row has stopped (EOS / stop id / length); stopped rows keep rewriting their last slot
//   remain[r]  tokens the row may still emit
// The sampled token and its log-prob are appended to the window ring at index *counter; rows that were already
// stopped append -1.  `u_next` (the uniform draws of the step after this one) is copied from u_all[counter + 1].
__global__ void __launch_bounds__(1024)
decode_advance_kernel(const long long* __restrict__ tok_new, const float* __restrict__ lp_new, long long* __restrict__ tok_in,
                      long long* __restrict__ pos, int* __restrict__ ctx, long long* __restrict__ slot,
                      const int* __restrict__ block_table, int max_blocks, int block_size, int* __restrict__ active,
                      int* __restrict__ remain, const long long* __restrict__ eos, const long long* __restrict__ stop_ids,
                      int n_stop, long long* __restrict__ out_tok, float* __restrict__ out_lp, int* __restrict__ counter,
                      int window, const float* __restrict__ u_all, float* __restrict__ u_next, int B) {
  const int r = threadIdx.x;
  const int c = *counter;
  __syncthreads();
  if (r < B && c < window) {
    long long emitted = -1;
    float lp = 0.f;
    if (active[r]) {
      const long long t = tok_new[r];
      emitted = t;
      lp = lp_new[r];
      int left = remain[r] - 1;
      bool stop = (eos[r] >= 0 && t == eos[r]);
      for (int j = 0; j < n_stop; ++j) {
        const long long sid = stop_ids[static_cast<size_t>(r) * n_stop + j];
        stop = stop || (sid >= 0 && t == sid);
      }
      if (stop || left <= 0) {
        active[r] = 0;
      } else {
        const long long p = pos[r] + 1;
        const long long blk = p / block_size;
        if (blk < max_blocks) {   // never index past the row's block table; the host sized it for the full length
          tok_in[r] = t;
          pos[r] = p;
          ctx[r] = static_cast<int>(p + 1);
          slot[r] = static_cast<long long>(block_table[static_cast<size_t>(r) * max_blocks + blk]) * block_size + p % block_size;
        } else {
          active[r] = 0;
        }
      }
      remain[r] = left;
    }
    out_tok[static_cast<size_t>(c) * B + r] = emitted;
    out_lp[static_cast<size_t>(c) * B + r] = lp;
    if (c + 1 < window) u_next[r] = u_all[static_cast<size_t>(c + 1) * B + r];
  }
  if (r == 0 && c < window) *counter = c + 1;
}

}  // namespace rb

// logits: [B][ld] rows of `V` valid entries, bf16 (is_bf16 = 1) or fp32.
extern "C" int rb_sample_v2(const void* logits, int is_bf16, int B, int V, long long ld, const float* temperature,
                            const long long* top_k, const float* top_p, const float* uniform, long long* tok, float* logp,
                            cudaStream_t st) {
  using namespace rb;
  if (B == 0) return 0;
  if (V <= 0) return -2;
  const uintptr_t addr = reinterpret_cast<uintptr_t>(logits);
  if (is_bf16) {
    const __nv_bfloat16* z = static_cast<const __nv_bfloat16*>(logits);
    if (addr % 16 == 0 && ld % 8 == 0)
      sample_v2_kernel<__nv_bfloat16, 8><<<B, SV_THREADS, 0, st>>>(z, V, ld, temperature, top_k, top_p, uniform, tok, logp);
    else
      sample_v2_kernel<__nv_bfloat16, 1><<<B, SV_THREADS, 0, st>>>(z, V, ld, temperature, top_k, top_p, uniform, tok, logp);
  } else {
    const float* z = static_cast<const float*>(logits);
    if (addr % 16 == 0 && ld % 4 == 0)
      sample_v2_kernel<float, 4><<<B, SV_THREADS, 0, st>>>(z, V, ld, temperature, top_k, top_p, uniform, tok, logp);
    else
      sample_v2_kernel<float, 1><<<B, SV_THREADS, 0, st>>>(z, V, ld, temperature, top_k, top_p, uniform, tok, logp);
  }
  rb_note_launch(1);
  return (int)cudaGetLastError();
}

extern "C" int rb_decode_advance(const long long* tok_new, const float* lp_new, long long* tok_in, long long* pos, int* ctx,
                                 long long* slot, const int* block_table, int max_blocks, int block_size, int* active,
                                 int* remain, const long long* eos, const long long* stop_ids, int n_stop,
                                 long long* out_tok, float* out_lp, int* counter, int window, const float* u_all,
                                 float* u_next, int B, cudaStream_t st) {
  if (B <= 0) return 0;
  if (B > 1024 || block_size <= 0 || max_blocks <= 0 || window <= 0 || n_stop < 0) return -2;
  rb::decode_advance_kernel<<<1, 1024, 0, st>>>(tok_new, lp_new, tok_in, pos, ctx, slot, block_table, max_blocks,
                                                block_size, active, remain, eos, stop_ids, n_stop, out_tok, out_lp,
                                                counter, window, u_all, u_next, B);
  rb_note_launch(1);
  return (int)cudaGetLastError();
}
