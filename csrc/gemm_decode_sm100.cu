// Weight-streaming GEMM for decode (a few hundred token rows at most): y[Mt, N] = x[Mt, K] * W[N, K]^T, optionally
// followed by SwiGLU when W = [gate; up].
//
// A decode GEMM is bound by reading W once; everything in this kernel serves that stream:
//   * the WEIGHT tile (128 output features x 64 k) is the M operand of tcgen05.mma and all the tokens are its N
//     operand (up to 256), so W is read exactly once however many tokens there are;
//   * the reduction dimension is split over the CTAs of a thread-block cluster and the partial sums are added
//     through distributed shared memory - no fp32 workspace in global memory and no second kernel;
//   * CTAs are small (about 100 KB of shared memory) so two share an SM: while one is in its prologue or its
//     reduction the other keeps the TMA stream going;
//   * the SwiGLU variant loads 64 gate rows and the matching 64 up rows into one tile, so the activation is
//     applied in the same reduction pass and only [Mt, F] is written.
// Every wait (mbarrier, cluster hand-shake) is bounded.  No load uses cluster multicast.
#include "common.cuh"
#include "host_utils.h"

namespace rb {
namespace dg {

constexpr int BM = 128;     // output features per CTA tile
constexpr int BK = 64;
constexpr int THREADS = 192;
constexpr int CHUNK = 64;   // token columns reduced per pass

struct Params {
  int Mt, N, K;             // tokens, output features of W (rows), reduction length
  int S;                    // cluster size = k splits
  int swiglu;               // W rows are [gate (N/2); up (N/2)], output is [Mt, N/2]
  void* out;
  int* err;
};

template <int NT>
struct Cfg {
  static constexpr int kStages = NT <= 64 ? 4 : (NT <= 128 ? 3 : 2);
  static constexpr int kWBytes = BM * BK * 2;
  static constexpr int kXBytes = NT * BK * 2;
  static constexpr int kStageBytes = kWBytes + kXBytes;
  static constexpr int kPipeBytes = kStages * kStageBytes;           // >= 96 KB... reused as the reduction buffers
  static constexpr int kRedBytes = 2 * CHUNK * BM * 4;               // two buffers of [64 tokens][128 features] fp32
  static constexpr int kDataBytes = kPipeBytes > kRedBytes ? kPipeBytes : kRedBytes;
  static constexpr int kBarOffset = kDataBytes;
  static constexpr int kTotal = kBarOffset + 256 + 1024;
};

__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ uint32_t map_to_cta(uint32_t smem_addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(smem_addr), "r"(rank));
  return r;
}
__device__ __forceinline__ void mbar_arrive_remote(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
__device__ __forceinline__ float4 ld_cluster_f32x4(uint32_t cluster_addr) {
  float4 v;
  asm volatile("ld.shared::cluster.v4.f32 {%0, %1, %2, %3}, [%4];"
               : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w)
               : "r"(cluster_addr));
  return v;
}
__device__ __forceinline__ void store_bf16x4(__nv_bfloat16* dst, const float4& v) {   // dst 8-byte aligned
  const __nv_bfloat162 lo = __floats2bfloat162_rn(v.x, v.y), hi = __floats2bfloat162_rn(v.z, v.w);
  uint2 u;
  u.x = *reinterpret_cast<const uint32_t*>(&lo);
  u.y = *reinterpret_cast<const uint32_t*>(&hi);
  *reinterpret_cast<uint2*>(dst) = u;
}
__device__ __forceinline__ bool mbar_try_wait_cluster(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}
// bounded wait on a barrier that CTAs of the cluster arrive on
__device__ __forceinline__ bool mbar_wait_cluster(uint64_t* bar, uint32_t parity, volatile int* abort_flag, int* g_err) {
  for (uint32_t i = 0; i < kSpinLimit; ++i) {
    if (mbar_try_wait_cluster(bar, parity)) return true;
    if ((i & 1023u) == 1023u && *abort_flag) return false;
  }
  *abort_flag = 1;
  if (g_err) atomicCAS(g_err, kOk, kErrBarrierTimeout);
  return false;
}

template <int NT>
__global__ void __launch_bounds__(THREADS, 2)
decode_gemm_kernel(const __grid_constant__ CUtensorMap tma_w, const __grid_constant__ CUtensorMap tma_x, const Params p) {
  using C = Cfg<NT>;
  constexpr int kStages = C::kStages;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + C::kBarOffset);
  uint64_t* empty_bar = full_bar + kStages;
  uint64_t* tfull_bar = empty_bar + kStages;
  uint64_t* ready_bar = tfull_bar + 1;    // [2] every CTA of the cluster has published reduction buffer b
  uint64_t* done_bar = ready_bar + 2;     // [2] every CTA of the cluster has finished reading MY buffer b
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(done_bar + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  float* red = reinterpret_cast<float*>(smem);     // [2][CHUNK][BM]; aliases the pipeline stages (idle by then)

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int S = p.S;
  const int q = static_cast<int>(cluster_ctarank());
  const int tile = blockIdx.x / S;
  const int k_iters = (p.K + BK - 1) / BK;
  const int per = (k_iters + S - 1) / S;
  const int k_lo = q * per, k_hi = min(k_iters, k_lo + per);
  const bool has_work = k_lo < k_hi;
  const int F = p.N / 2;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) { mbar_init(&full_bar[s], 1); mbar_init(&empty_bar[s], 1); }
    mbar_init(tfull_bar, 1);
    for (int b = 0; b < 2; ++b) { mbar_init(&ready_bar[b], S); mbar_init(&done_bar[b], S); }
    *abort_flag = 0;
    fence_barrier_init();
  }
  if (warp == 1) {
    tmem_alloc<NT>(tmem_slot);
    tmem_relinquish();
  }
  tc_fence_before();
  // the barriers of every CTA of the cluster exist before anyone arrives on a peer's
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  if (!(warp == 0 && lane == 0)) griddep_wait();   // (the producer waits after it has started the weight stream)

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      tma_prefetch_desc(&tma_w);
      tma_prefetch_desc(&tma_x);
      auto load_w = [&](int s, int k) {
        uint8_t* sw = smem + s * C::kStageBytes;
        mbar_expect_tx(&full_bar[s], C::kStageBytes);
        if (!p.swiglu) {
          tma_load_2d(sw, &tma_w, &full_bar[s], k * BK, tile * BM);
        } else {   // 64 gate rows, then the 64 up rows of the same features
          tma_load_2d(sw, &tma_w, &full_bar[s], k * BK, tile * 64);
          tma_load_2d(sw + 64 * 128, &tma_w, &full_bar[s], k * BK, F + tile * 64);
        }
      };
      auto load_x = [&](int s, int k) {
        tma_load_2d(smem + s * C::kStageBytes + C::kWBytes, &tma_x, &full_bar[s], k * BK, 0);
      };
      // the weights do not depend on the kernel before this one: fill the ring with W tiles first, wait for the
      // predecessor, then add the token tiles (the stage's barrier counts both)
      const int pre = min(kStages, k_hi - k_lo);
      for (int i = 0; i < pre; ++i) load_w(i, k_lo + i);
      griddep_wait();
      for (int i = 0; i < pre; ++i) load_x(i, k_lo + i);
      int s = pre == kStages ? 0 : pre;
      uint32_t ph = pre == kStages ? 1 : 0;
      for (int k = k_lo + pre; k < k_hi; ++k) {
        if (!mbar_wait(&empty_bar[s], ph ^ 1, abort_flag, p.err)) break;
        load_w(s, k);
        load_x(s, k);
        if (++s == kStages) { s = 0; ph ^= 1; }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0 && has_work) {
      const uint32_t idesc = make_idesc_f16(BM, NT, true, false, false);
      int s = 0;
      uint32_t ph = 0;
      bool ok = true;
      for (int k = k_lo; k < k_hi; ++k) {
        if (!mbar_wait(&full_bar[s], ph, abort_flag, p.err)) { ok = false; break; }
        tc_fence_after();
        const uint32_t sw = smem_u32(smem + s * C::kStageBytes);
        const uint32_t sx = sw + C::kWBytes;
#pragma unroll
        for (int kk = 0; kk < BK / 16; ++kk) {
          const uint64_t da = make_smem_desc(sw + kk * 32, 16, 1024, kSwizzle128B);
          const uint64_t db = make_smem_desc(sx + kk * 32, 16, 1024, kSwizzle128B);
          umma_f16(tmem_base, da, db, idesc, (k > k_lo || kk > 0) ? 1u : 0u);
        }
        umma_commit(&empty_bar[s]);
        if (++s == kStages) { s = 0; ph ^= 1; }
      }
      if (ok) umma_commit(tfull_bar);
    }
  } else {
    // ------------------------------------------------------------------ epilogue: cluster reduction + store
    const int et = threadIdx.x - 64;          // 0..127
    const int lane_grp = warp & 3;
    const int row = lane_grp * 32 + lane;     // feature row of the tile = TMEM lane
    bool ok = true;
    if (has_work) {
      ok = mbar_wait(tfull_bar, 0, abort_flag, p.err);
      tc_fence_after();
    }
    const int nchunks = (p.Mt + CHUNK - 1) / CHUNK;
    const uint32_t taddr = tmem_base + (static_cast<uint32_t>(lane_grp * 32) << 16);
    // slice of the tile this CTA reduces: feature rows (plain) or gate/up pairs (SwiGLU).  S is a power of two, so
    // the slice is a power of two >= 8 and splits into float4 groups with shifts.
    const int lgS = 31 - __clz(S);
    const int units = p.swiglu ? 64 : BM;
    const int u_n = units >> lgS;
    const int u_lo = q * u_n;
    const int lgG = 31 - __clz(u_n >> 2);
    const int G = 1 << lgG;
    uint32_t peer[8];   // the reduction buffers of every CTA of the cluster, in cluster shared addresses
#pragma unroll
    for (int z = 0; z < 8; ++z) peer[z] = map_to_cta(smem_u32(red), z < S ? z : 0);
    for (int c = 0; c < nchunks; ++c) {
      const int buf = c & 1, use = c >> 1;
      float* mine = red + buf * (CHUNK * BM);
      if (c >= 2 && ok) ok = mbar_wait_cluster(&done_bar[buf], static_cast<uint32_t>(use - 1) & 1, abort_flag, p.err);
      {
        uint32_t r0[32], r1[32];
        if (has_work && ok) {
          tmem_ld_32x32b_x32(taddr + c * CHUNK, r0);
          tmem_ld_32x32b_x32(taddr + c * CHUNK + 32, r1);
          tmem_wait_ld();
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) { r0[i] = 0; r1[i] = 0; }
        }
#pragma unroll
        for (int j = 0; j < 32; ++j) {
          mine[j * BM + row] = __uint_as_float(r0[j]);
          mine[(32 + j) * BM + row] = __uint_as_float(r1[j]);
        }
      }
      named_bar_sync(1, 128);
      if (et < S) mbar_arrive_remote(map_to_cta(smem_u32(&ready_bar[buf]), et));
      if (ok) ok = mbar_wait_cluster(&ready_bar[buf], static_cast<uint32_t>(use) & 1, abort_flag, p.err);
      if (ok) {
        const uint32_t boff = static_cast<uint32_t>(buf * (CHUNK * BM) * 4);
        for (int idx = et; idx < CHUNK * G; idx += 128) {
          const int g = idx & (G - 1), j = idx >> lgG;
          const int tok = c * CHUNK + j;
          if (tok >= p.Mt) break;     // j grows with idx
          const uint32_t off = boff + static_cast<uint32_t>((j * BM + u_lo + 4 * g) * 4);
          float4 a[8];
#pragma unroll
          for (int z = 0; z < 8; ++z)
            if (z < S) a[z] = ld_cluster_f32x4(peer[z] + off);
          float4 acc = a[0];
#pragma unroll
          for (int z = 1; z < 8; ++z)
            if (z < S) { acc.x += a[z].x; acc.y += a[z].y; acc.z += a[z].z; acc.w += a[z].w; }
          if (!p.swiglu) {
            const int f = tile * BM + u_lo + 4 * g;
            __nv_bfloat16* o = reinterpret_cast<__nv_bfloat16*>(p.out) + static_cast<size_t>(tok) * p.N + f;
            if (f + 3 < p.N) {
              store_bf16x4(o, acc);
            } else {
              const float v[4] = {acc.x, acc.y, acc.z, acc.w};
              for (int e = 0; e < 4; ++e)
                if (f + e < p.N) o[e] = __float2bfloat16(v[e]);
            }
          } else {
            float4 b[8];
#pragma unroll
            for (int z = 0; z < 8; ++z)
              if (z < S) b[z] = ld_cluster_f32x4(peer[z] + off + 64 * 4);
            float4 up = b[0];
#pragma unroll
            for (int z = 1; z < 8; ++z)
              if (z < S) { up.x += b[z].x; up.y += b[z].y; up.z += b[z].z; up.w += b[z].w; }
            const int f = tile * 64 + u_lo + 4 * g;      // F is a multiple of 64: always inside
            float4 r;
            r.x = acc.x / (1.f + __expf(-acc.x)) * up.x;
            r.y = acc.y / (1.f + __expf(-acc.y)) * up.y;
            r.z = acc.z / (1.f + __expf(-acc.z)) * up.z;
            r.w = acc.w / (1.f + __expf(-acc.w)) * up.w;
            store_bf16x4(reinterpret_cast<__nv_bfloat16*>(p.out) + static_cast<size_t>(tok) * F + f, r);
          }
        }
      }
      named_bar_sync(1, 128);
      if (et < S) mbar_arrive_remote(map_to_cta(smem_u32(&done_bar[buf]), et));
    }
    // nobody may still be reading this CTA's buffers when it leaves
    for (int buf = 0; buf < 2; ++buf) {
      const int uses = (nchunks + 1 - buf) / 2;
      if (uses > 0 && ok) ok = mbar_wait_cluster(&done_bar[buf], static_cast<uint32_t>(uses - 1) & 1, abort_flag, p.err);
    }
  }

  if (*abort_flag) __nanosleep(50000);
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc<NT>(tmem_base);
  }
}

template <int NT>
static int launch(const CUtensorMap& tw, const CUtensorMap& tx, const Params& p, int tiles, cudaStream_t st) {
  using C = Cfg<NT>;
  static bool attr = false;
  auto kern = decode_gemm_kernel<NT>;
  if (!attr) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, C::kTotal);
    if (e != cudaSuccess) return static_cast<int>(e);
    attr = true;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(tiles * p.S);
  cfg.blockDim = dim3(THREADS);
  cfg.dynamicSmemBytes = C::kTotal;
  cfg.stream = st;
  cudaLaunchAttribute at[2];
  at[0].id = cudaLaunchAttributeClusterDimension;
  at[0].val.clusterDim.x = p.S;
  at[0].val.clusterDim.y = 1;
  at[0].val.clusterDim.z = 1;
  at[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  at[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = at;
  cfg.numAttrs = pdl_enabled() ? 2 : 1;
  cudaError_t e = cudaLaunchKernelEx(&cfg, kern, tw, tx, p);
  rb_note_launch(1);
  return e != cudaSuccess ? static_cast<int>(e) : static_cast<int>(cudaGetLastError());
}

}  // namespace dg
}  // namespace rb

// K splits (= cluster size: 1, 2, 4 or 8) for a decode GEMM with `tiles` weight tiles and `k_iters` 64-deep steps.
// Measured on B200 at 128 and 256 tokens: one CTA per SM is enough to keep the weight stream going as long as
// every CTA has a few k steps, a second wave costs more than it gains, and long reductions (k_iters / S >= 16
// after doubling) are worth a second CTA per SM.
extern "C" int rb_decode_gemm_splits(int tiles, int k_iters) {
  const int slots = 2 * rb::num_sms();
  int s = 1;
  while (s < 8 && tiles * s < 128 && k_iters / (2 * s) >= 4) s *= 2;
  if (s < 8 && tiles * 2 * s <= slots && k_iters / (2 * s) >= 16) s *= 2;
  return s;
}

// y = x W^T (swiglu = 0, y [Mt, N]) or y = silu(x Wg^T) * (x Wu^T) with W = [Wg; Wu] (swiglu = 1, y [Mt, N / 2]).
// x [Mt <= 256, K], W [N, K], all bf16 row-major; returns -20 when the shape is outside what this kernel covers.
extern "C" int rb_decode_gemm(const void* x, const void* W, void* y, int Mt, int N, int K, int ldx, int ldw, int swiglu,
                              int splits, int* err, cudaStream_t st) {
  using namespace rb;
  using namespace rb::dg;
  if (Mt <= 0 || N <= 0 || K <= 0) return 0;
  if (Mt > 256 || (ldx % 8) || (ldw % 8) || (K % 8)) return -20;
  if ((reinterpret_cast<uintptr_t>(x) % 16) || (reinterpret_cast<uintptr_t>(W) % 16)) return -20;
  if (swiglu && ((N / 2) % 64)) return -20;
  if ((N % 4) || (reinterpret_cast<uintptr_t>(y) % 8)) return -20;   // 4 features per store
  const int nt = Mt <= 64 ? 64 : (Mt <= 128 ? 128 : 256);
  const int tiles = swiglu ? (N / 2) / 64 : (N + BM - 1) / BM;
  const int k_iters = (K + BK - 1) / BK;
  Params p{};
  p.Mt = Mt; p.N = N; p.K = K; p.swiglu = swiglu; p.out = y; p.err = err;
  p.S = splits > 0 ? splits : rb_decode_gemm_splits(tiles, k_iters);
  if (p.S > 8) p.S = 8;
  while (p.S & (p.S - 1)) p.S &= p.S - 1;       // the reduction slices the tile in powers of two
  CUtensorMap tw, tx;
  int rc = encode_tma_2d_bf16(&tw, W, K, N, ldw, BK, swiglu ? 64 : BM);
  if (rc) return rc;
  rc = encode_tma_2d_bf16(&tx, x, K, Mt, ldx, BK, nt);
  if (rc) return rc;
  if (nt == 64) return launch<64>(tw, tx, p, tiles, st);
  if (nt == 128) return launch<128>(tw, tx, p, tiles, st);
  return launch<256>(tw, tx, p, tiles, st);
}
