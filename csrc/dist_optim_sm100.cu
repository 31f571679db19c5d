// Distributed-optimizer step over NVLink peer memory (data-parallel ranks of one node).
//
// The unfused step is: NCCL reduce-scatter of the fp32 gradient buffer -> sum of squares -> (norm
// all-reduce, clip) -> Adam on this rank's shard -> NCCL all-gather of the updated bf16 parameters.
// Here the two collectives disappear into the two elementwise kernels that surround them:
//
//   rb_dp_reduce_sumsq   my_shard[i] = scale * sum_r grad_r[lo + i]   (peer loads), plus sum of squares of the result
//   rb_dp_adam_allgather Adam on my shard, the new bf16 parameters stored into EVERY rank's parameter buffer
//
// Gradient and parameter buffers live in symmetric memory (same layout on every rank).  Ordering between
// ranks uses two monotonic counters in every rank's signal pad: "my gradients are complete" (bumped at
// the start of the first kernel, which waits for all ranks before reading) and "my parameter stores have
// landed" (bumped at the end of the second kernel, which waits for all ranks before it ends, so the next
// forward pass on any rank sees every shard).  All waits are bounded; on expiry the kernel records error
// 3 and returns.
#include "common.cuh"
#include "host_utils.h"

namespace rb {

struct DpParams {
  int dp, rank;
  const float* peer_g[8];      // gradient buffer of rank r as mapped here (full buffer)
  __nv_bfloat16* peer_p[8];    // parameter buffer of rank r as mapped here (full buffer)
  unsigned* peer_sig[8];       // signal pad of rank r; this file uses words 32 (ready) and 33 (done)
  int* state;                  // local ints: [12] ready base, [13] done base, [14]/[15] block tickets
  long long lo, n;             // my shard = elements [lo, lo + n)
  unsigned long long wait_ns;
  int* err;
};

__global__ void __launch_bounds__(256)
dp_reduce_sumsq_kernel(const DpParams p, float* __restrict__ out, float* __restrict__ sumsq, float scale) {
  __shared__ int s_ok;
  __shared__ float s_red[8];
  if (threadIdx.x == 0) {
    if (blockIdx.x == 0)
      for (int r = 0; r < p.dp; ++r) sys_red_add(p.peer_sig[r] + 32, 1u);
    const unsigned target = static_cast<unsigned>(p.state[12]) + static_cast<unsigned>(p.dp);
    s_ok = sys_wait_ge(p.peer_sig[p.rank] + 32, target, p.wait_ns) ? 1 : 0;
    if (!s_ok) atomicExch(p.err, 3);
  }
  __syncthreads();
  float ss = 0.f;
  if (s_ok) {
    for (long long i = (blockIdx.x * (long long)blockDim.x + threadIdx.x) * 4; i < p.n; i += (long long)gridDim.x * blockDim.x * 4) {
      float4 a = make_float4(0.f, 0.f, 0.f, 0.f);
      for (int k = 0; k < p.dp; ++k) {
        const int r = (p.rank + k) % p.dp;  // start with the local copy, spread the peers over the links
        const float4 v = __ldcv(reinterpret_cast<const float4*>(p.peer_g[r] + p.lo + i));
        a.x += v.x; a.y += v.y; a.z += v.z; a.w += v.w;
      }
      a.x *= scale; a.y *= scale; a.z *= scale; a.w *= scale;
      *reinterpret_cast<float4*>(out + i) = a;
      ss += a.x * a.x + a.y * a.y + a.z * a.z + a.w * a.w;
    }
  }
  ss = warp_sum(ss);
  if ((threadIdx.x & 31) == 0) s_red[threadIdx.x >> 5] = ss;
  __syncthreads();
  if (threadIdx.x == 0) {
    float t = 0.f;
    for (int w = 0; w < 8; ++w) t += s_red[w];
    atomicAdd(sumsq, t);
    __threadfence();
    if (atomicAdd(p.state + 14, 1) == static_cast<int>(gridDim.x) - 1) {
      p.state[14] = 0;
      p.state[12] += p.dp;
      __threadfence();
    }
  }
}

template <bool SPLIT>
__global__ void __launch_bounds__(256)
dp_adam_allgather_kernel(const DpParams p, void* __restrict__ master, const float* __restrict__ g, float* __restrict__ m,
                         float* __restrict__ v, float lr, float b1, float b2, float eps, float wd, float gscale, float bc1,
                         float bc2) {
  const __nv_bfloat16* mine = p.peer_p[p.rank] + p.lo;
  for (long long i = (blockIdx.x * (long long)blockDim.x + threadIdx.x) * 4; i < p.n; i += (long long)gridDim.x * blockDim.x * 4) {
    const float4 g4 = *reinterpret_cast<const float4*>(g + i);
    float4 m4 = *reinterpret_cast<float4*>(m + i), v4 = *reinterpret_cast<float4*>(v + i);
    const float gv[4] = {g4.x, g4.y, g4.z, g4.w};
    float mv[4] = {m4.x, m4.y, m4.z, m4.w}, vv[4] = {v4.x, v4.y, v4.z, v4.w}, w[4];
    const uint2 praw = *reinterpret_cast<const uint2*>(mine + i);
    const uint16_t* ph = reinterpret_cast<const uint16_t*>(&praw);
    if constexpr (SPLIT) {
      const uint2 rraw = *reinterpret_cast<const uint2*>(reinterpret_cast<const int16_t*>(master) + i);
      const int16_t* rh = reinterpret_cast<const int16_t*>(&rraw);
#pragma unroll
      for (int k = 0; k < 4; ++k) w[k] = __int_as_float((static_cast<int>(static_cast<int16_t>(ph[k])) << 16) + static_cast<int>(rh[k]));
    } else {
      const float4 t = *reinterpret_cast<const float4*>(reinterpret_cast<const float*>(master) + i);
      w[0] = t.x; w[1] = t.y; w[2] = t.z; w[3] = t.w;
    }
    uint16_t hi[4];
    int16_t rem[4];
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const float gg = gv[k] * gscale;
      mv[k] = b1 * mv[k] + (1.f - b1) * gg;
      vv[k] = b2 * vv[k] + (1.f - b2) * gg * gg;
      const float denom = sqrtf(vv[k] / bc2) + eps;
      w[k] = w[k] * (1.f - lr * wd) - lr * (mv[k] / bc1) / denom;
      const __nv_bfloat16 h = __float2bfloat16_rn(w[k]);
      hi[k] = *reinterpret_cast<const uint16_t*>(&h);
      int r = __float_as_int(w[k]) - (static_cast<int>(static_cast<int16_t>(hi[k])) << 16);
      if (r == 32768) {  // exact tie: take the other bf16 neighbour so the remainder fits int16
        hi[k] = static_cast<uint16_t>(hi[k] + 1);
        r = -32768;
      }
      rem[k] = static_cast<int16_t>(r);
    }
    *reinterpret_cast<float4*>(m + i) = make_float4(mv[0], mv[1], mv[2], mv[3]);
    *reinterpret_cast<float4*>(v + i) = make_float4(vv[0], vv[1], vv[2], vv[3]);
    if constexpr (SPLIT) *reinterpret_cast<uint2*>(reinterpret_cast<int16_t*>(master) + i) = *reinterpret_cast<uint2*>(rem);
    else *reinterpret_cast<float4*>(reinterpret_cast<float*>(master) + i) = make_float4(w[0], w[1], w[2], w[3]);
    const uint2 pk = *reinterpret_cast<const uint2*>(hi);
    for (int k = 0; k < p.dp; ++k) {  // the all-gather: every rank's copy of my shard
      const int r = (p.rank + k) % p.dp;
      *reinterpret_cast<uint2*>(p.peer_p[r] + p.lo + i) = pk;
    }
  }
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) {
    if (atomicAdd(p.state + 15, 1) == static_cast<int>(gridDim.x) - 1) {
      // every block of this rank has stored and fenced: tell all ranks, then wait until all of them have
      for (int r = 0; r < p.dp; ++r) sys_red_add(p.peer_sig[r] + 33, 1u);
      const unsigned target = static_cast<unsigned>(p.state[13]) + static_cast<unsigned>(p.dp);
      if (!sys_wait_ge(p.peer_sig[p.rank] + 33, target, p.wait_ns)) atomicExch(p.err, 3);
      p.state[15] = 0;
      p.state[13] += p.dp;
      __threadfence();
    }
  }
}

// Barrier between the ranks of a group through their signal pads: every rank adds 1 to word `slot` of every
// rank's pad (a system-scope release, so its earlier stores - e.g. a buffer it just filled for the peers - are
// visible first) and waits, bounded, until its own word shows one arrival per rank.  One block, launched in
// stream order between the kernels it separates.
__global__ void peer_barrier_kernel(const DpParams p, int slot, int state_idx) {
  __shared__ int ok;
  if (threadIdx.x < p.dp) sys_red_add(p.peer_sig[threadIdx.x] + slot, 1u);
  __syncthreads();
  if (threadIdx.x == 0) {
    const unsigned target = static_cast<unsigned>(p.state[state_idx]) + static_cast<unsigned>(p.dp);
    ok = sys_wait_ge(p.peer_sig[p.rank] + slot, target, p.wait_ns) ? 1 : 0;
    if (!ok) atomicExch(p.err, 3);
    p.state[state_idx] += p.dp;
    __threadfence_system();
  }
}

// Copies a contiguous buffer into the same offset of up to 8 destinations (this GPU's or peers' memory mapped
// here): the push half of an all-gather.  16-byte vectors; completion is ordered by the barrier that follows.
struct PushParams {
  uint4* dst[8];
  int n_dst;
};
__global__ void peer_push_kernel(const uint4* __restrict__ src, const PushParams p, long long nvec) {
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < nvec; i += (long long)gridDim.x * blockDim.x) {
    const uint4 v = src[i];
    for (int d = 0; d < p.n_dst; ++d) p.dst[d][i] = v;
  }
}

}  // namespace rb

static void fill(rb::DpParams& p, int dp, int rank, float* const* peer_g, void* const* peer_p, unsigned* const* peer_sig,
                 int* state, long long lo, long long n, unsigned long long wait_ns, int* err) {
  p.dp = dp; p.rank = rank; p.state = state; p.lo = lo; p.n = n; p.wait_ns = wait_ns; p.err = err;
  for (int r = 0; r < dp; ++r) {
    p.peer_g[r] = peer_g ? peer_g[r] : nullptr;
    p.peer_p[r] = peer_p ? reinterpret_cast<__nv_bfloat16*>(peer_p[r]) : nullptr;
    p.peer_sig[r] = peer_sig[r];
  }
}

extern "C" int rb_dp_reduce_sumsq(float* const* peer_g, unsigned* const* peer_sig, int* state, int dp, int rank, long long lo,
                                  long long n, float* out, float* sumsq, float scale, unsigned long long wait_ns, int* err,
                                  cudaStream_t st) {
  using namespace rb;
  if (n == 0) return 0;
  if (dp < 1 || dp > 8 || (n % 4) || (lo % 4)) return -2;
  DpParams p{};
  fill(p, dp, rank, peer_g, nullptr, peer_sig, state, lo, n, wait_ns, err);
  long long blocks = (n / 4 + 255) / 256;
  if (blocks > num_sms() * 4LL) blocks = num_sms() * 4LL;
  dp_reduce_sumsq_kernel<<<(int)blocks, 256, 0, st>>>(p, out, sumsq, scale);
  rb_note_launch(1);
  return (int)cudaGetLastError();
}

extern "C" int rb_dp_adam_allgather(void* const* peer_p, unsigned* const* peer_sig, int* state, int dp, int rank, long long lo,
                                    long long n, void* master, const float* g, float* m, float* v, int step, float lr, float b1,
                                    float b2, float eps, float wd, float gscale, int split, unsigned long long wait_ns,
                                    int* err, cudaStream_t st) {
  using namespace rb;
  if (n == 0) return 0;
  if (dp < 1 || dp > 8 || (n % 4) || (lo % 4)) return -2;
  DpParams p{};
  fill(p, dp, rank, nullptr, peer_p, peer_sig, state, lo, n, wait_ns, err);
  const float bc1 = 1.f - powf(b1, (float)step), bc2 = 1.f - powf(b2, (float)step);
  long long blocks = (n / 4 + 255) / 256;
  if (blocks > num_sms() * 4LL) blocks = num_sms() * 4LL;
  if (split) dp_adam_allgather_kernel<true><<<(int)blocks, 256, 0, st>>>(p, master, g, m, v, lr, b1, b2, eps, wd, gscale, bc1, bc2);
  else dp_adam_allgather_kernel<false><<<(int)blocks, 256, 0, st>>>(p, master, g, m, v, lr, b1, b2, eps, wd, gscale, bc1, bc2);
  rb_note_launch(1);
  return (int)cudaGetLastError();
}

extern "C" int rb_peer_barrier(unsigned* const* peer_sig, int* state, int n, int rank, int slot, int state_idx,
                               unsigned long long wait_ns, int* err, cudaStream_t st) {
  using namespace rb;
  if (n < 1 || n > 8 || slot < 0 || slot >= 256 || state_idx < 0) return -2;
  DpParams p{};
  fill(p, n, rank, nullptr, nullptr, peer_sig, state, 0, 0, wait_ns, err);
  peer_barrier_kernel<<<1, 32, 0, st>>>(p, slot, state_idx);
  rb_note_launch(1);
  return (int)cudaGetLastError();
}

extern "C" int rb_peer_push(const void* src, void* const* dst, int n_dst, long long nbytes, cudaStream_t st) {
  using namespace rb;
  if (nbytes == 0 || n_dst == 0) return 0;
  if (n_dst < 0 || n_dst > 8 || (nbytes % 16) || (reinterpret_cast<uintptr_t>(src) % 16)) return -2;
  PushParams p{};
  p.n_dst = n_dst;
  for (int d = 0; d < n_dst; ++d) {
    if (reinterpret_cast<uintptr_t>(dst[d]) % 16) return -2;
    p.dst[d] = reinterpret_cast<uint4*>(dst[d]);
  }
  const long long nvec = nbytes / 16;
  long long blocks = (nvec + 255) / 256;
  if (blocks > num_sms() * 8LL) blocks = num_sms() * 8LL;
  peer_push_kernel<<<(int)blocks, 256, 0, st>>>(reinterpret_cast<const uint4*>(src), p, nvec);
  rb_note_launch(1);
  return (int)cudaGetLastError();
}
