// Persistent warp-specialised GEMM for sm_100a: TMA -> shared memory ring ->
// tcgen05.mma (accumulators in TMEM, double buffered) -> epilogue warps.
//
//   C[M,N] (+)= A_op[M,K] * B_op[N,K]^T        bf16/fp16 in, fp32 accumulate
//
// Operand storage (all row-major in global memory):
//   A K-major : A[M][K]  (lda >= K)        A MN-major : A[K][M]  (lda >= M)   ("transposed A")
//   B K-major : B[N][K]  (ldb >= K)        B MN-major : B[K][N]  (ldb >= N)
// which covers y = x W^T (K,K), dx = dy W (K,MN) and dW = dy^T x (MN,MN) without
// materialising a transpose.
//
// Roles (192 threads): warp 0 = TMA producer, warp 1 = MMA issuer + TMEM owner,
// warps 2..5 = epilogue (TMEM -> registers -> global).  One CTA per SM, static
// round-robin tile schedule with grouped ordering for L2 reuse.
#include "common.cuh"
#include "host_utils.h"
#include <type_traits>

namespace rb {

constexpr int BM = 128;
constexpr int BK = 64;  // 64 bf16 = 128 bytes = one swizzle row
constexpr int GEMM_THREADS = 192;
constexpr int kStagePitch = 36;                          // floats per staged row (32 + 4: conflict-free float4 access)
constexpr int kStageBytes4 = 4 * 32 * kStagePitch * 4;   // per-warp 32x32 fp32 staging of the peer-reduce epilogue

struct GemmParams {
  int M, N, K;
  int ldc;
  int tiles_m, tiles_n;
  int out_fp32, accumulate;
  int a_mn, b_mn;
  int k_splits, k_iters_per_split;  // split-K: partial sums go to fp32 workspace slices C + split*M*ldc
  uint32_t lbo_a, sbo_a, lbo_b, sbo_b;  // MN-major descriptor strides (bytes)
  void* C;
  const void* bias;  // optional [N], same dtype as inputs
  int* err;
  // ---- fused LM-head modes (MODE 1: log-prob/entropy partials, MODE 2: d(logits) tile)
  const long long* targets;  // [M] global vocabulary ids
  int vocab_start;           // first vocabulary id of this shard
  float inv_temp;
  int n_splits, tiles_per_split;
  float* partials;           // MODE 1 out: [M][n_splits][4] = (max, sum exp, sum exp*z, target logit or -inf)
  const float* row_stats;    // MODE 2 in:  [M][2] = (log Z, sum p*z) of the temperature-scaled logits
  const float* g_lp;         // MODE 2 in:  [M] upstream gradient of log-prob
  const float* g_ent;        // MODE 2 in:  [M] upstream gradient of entropy (may be null)
  // ---- MODE 3: row-parallel GEMM fused with its tensor-parallel all-reduce, the residual add and RMSNorm.
  // Every rank stores its fp32 partial tiles straight into slot (parity, rank, k split) of EVERY
  // rank's workspace through NVLink peer pointers, bumps a counter on every rank, waits (bounded)
  // until all tiles of all ranks have landed in its own workspace and then reduces its own copy.
  // Reduce-scatter form (rs != 0): row block r of the product belongs to rank r only, so a partial row
  // goes to its owner alone and every rank reduces rows_out = M / tp rows; tiles are visited starting
  // with the next rank's rows so that the transfers overlap the rest of the GEMM.
  int tp, tp_rank, rs, rows_out, tm_rot;
  float* peer_ws[8];         // workspace of rank r as mapped here: [2][tp][k_splits][rows_out][N] fp32
  unsigned* peer_sig[8];     // arrival counters of rank r as mapped here: [2], one per parity
  int* pr_state;             // local: [0] call sequence, [1..2] counter base per parity, [3] CTAs finished
  const void* residual;      // [M][N] bf16 (may be null)
  const void* norm_w;        // [N] bf16 (may be null: no norm output)
  void* out_h;               // [M][N] bf16: residual + sum over ranks
  void* out_x;               // [M][N] bf16: rmsnorm(out_h) * norm_w
  float eps;
  unsigned long long wait_ns;  // limit of the wait for the peers
  // ---- MODE 4: all-gather of the A row shards fused into the GEMM.  The epilogue warps first push this rank's
  // shard into every peer's gathered buffer (double buffered by call parity) and signal; the TMA producer
  // starts with this rank's own rows and waits (bounded) for a peer's arrival count before its rows.
  void* peer_ag[8];          // gathered buffer of rank r as mapped here: [2][M][K] bf16
  const void* ag_src;        // this rank's shard [M/tp][K], contiguous
  int ag_rows;               // M / tp
  unsigned long long* timeline;  // optional [grid][8] global-timer stamps of the phases (profiling aid)
};

enum : int { kEpiStore = 0, kEpiLogProb = 1, kEpiDLogits = 2, kEpiPeerReduce = 3, kEpiAllGather = 4 };

template <int BN>
struct GemmSmem {
  static constexpr int kStages = (BN >= 256) ? 4 : (BN >= 128 ? 6 : 8);
  static constexpr int kABytes = BM * BK * 2;
  static constexpr int kBBytes = BN * BK * 2;
  static constexpr int kStageBytes = kABytes + kBBytes;
  static constexpr int kBarOffset = kStages * kStageBytes;
  static constexpr int kTotal = kBarOffset + 256 + 1024;  // barriers + alignment slack
};

__device__ __forceinline__ void tile_coords(int t, int tiles_m, int tiles_n, int& tm, int& tn) {
  constexpr int GM = 8;
  const int per_group = GM * tiles_n;
  const int group = t / per_group;
  const int first_m = group * GM;
  const int gm = min(tiles_m - first_m, GM);
  const int r = t - group * per_group;
  tm = first_m + (r % gm);
  tn = r / gm;
}

// i-th tile of this CTA.  MODE 1 pins a CTA to one row block and a contiguous range of
// column tiles (so per-row softmax statistics stay in registers); the other modes use the
// persistent round-robin schedule.
template <int MODE>
__device__ __forceinline__ bool next_tile(const GemmParams& p, int i, int& tm, int& tn, int& split) {
  split = 0;
  if constexpr (MODE == kEpiLogProb) {
    tm = blockIdx.x / p.n_splits;
    tn = (blockIdx.x % p.n_splits) * p.tiles_per_split + i;
    return i < p.tiles_per_split && tn < p.tiles_n;
  } else {
    int t = blockIdx.x + i * gridDim.x;
    if (t >= p.tiles_m * p.tiles_n * p.k_splits) return false;
    split = t % p.k_splits;
    t /= p.k_splits;
    tile_coords(t, p.tiles_m, p.tiles_n, tm, tn);
    if constexpr (MODE == kEpiPeerReduce || MODE == kEpiAllGather) {
      tm += p.tm_rot;
      if (tm >= p.tiles_m) tm -= p.tiles_m;
    }
    return true;
  }
}

template <int BN, bool BF16, int MODE>
__global__ void __launch_bounds__(GEMM_THREADS, 1)
gemm_kernel(const __grid_constant__ CUtensorMap tma_a, const __grid_constant__ CUtensorMap tma_b,
            const __grid_constant__ CUtensorMap tma_g, const GemmParams p) {
  using S = GemmSmem<BN>;
  constexpr int kStages = S::kStages;
  constexpr int kTmemCols = (2 * BN <= 32) ? 32 : 2 * BN;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + S::kBarOffset);
  uint64_t* empty_bar = full_bar + kStages;
  uint64_t* tfull_bar = empty_bar + kStages;   // [2]
  uint64_t* tempty_bar = tfull_bar + 2;        // [2]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tempty_bar + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int k_iters_total = (p.K + BK - 1) / BK;
  // In the all-gather mode the TMA producer may wait (bounded by p.wait_ns) for another GPU; every other
  // role then waits on it through the pipeline barriers, so their limit has to be the longer one.
  auto pipe_wait = [&](uint64_t* bar, uint32_t parity) -> bool {
    if constexpr (MODE == kEpiAllGather) return mbar_wait_timed(bar, parity, abort_flag, p.err, p.wait_ns + 2000000000ull);
    else return mbar_wait(bar, parity, abort_flag, p.err);
  };

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&tfull_bar[a], 1);
      mbar_init(&tempty_bar[a], 4);
    }
    *abort_flag = 0;
    fence_barrier_init();
  }
  if (warp == 1) {
    tmem_alloc<kTmemCols>(tmem_slot);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      tma_prefetch_desc(&tma_a);
      tma_prefetch_desc(&tma_b);
      int s = 0;
      uint32_t ph = 0;
      bool ok = true;
      // MODE 4 state: parity of this call, arrival target, sources already seen complete
      int ag_parity = 0;
      unsigned ag_target = 0, ag_ready = 0;
      if constexpr (MODE == kEpiAllGather) {
        tma_prefetch_desc(&tma_g);
        ag_parity = p.pr_state[8] & 1;
        ag_target = static_cast<unsigned>(p.pr_state[9 + ag_parity]) + gridDim.x;
        ag_ready = 1u << p.tp_rank;
      }
      for (int ti = 0; ok; ++ti) {
        int tm, tn, split;
        if (!next_tile<MODE>(p, ti, tm, tn, split)) break;
        const int m0 = tm * BM, n0 = tn * BN;
        int ag_src_rank = 0;
        if constexpr (MODE == kEpiAllGather) {
          ag_src_rank = m0 / p.ag_rows;
          if (!((ag_ready >> ag_src_rank) & 1u)) {
            if (!sys_wait_ge(p.peer_sig[p.tp_rank] + 16 + ag_parity * 8 + ag_src_rank, ag_target, p.wait_ns)) {
              *abort_flag = 1;
              atomicExch(p.err, 3);
              break;
            }
            fence_proxy_async_global();
            ag_ready |= 1u << ag_src_rank;
          }
        }
        const int k_lo = split * p.k_iters_per_split, k_hi = min(k_iters_total, k_lo + p.k_iters_per_split);
        for (int k = k_lo; k < k_hi; ++k) {
          if (!pipe_wait(&empty_bar[s], ph ^ 1)) { ok = false; break; }
          uint8_t* sa = smem + s * S::kStageBytes;
          uint8_t* sb = sa + S::kABytes;
          mbar_expect_tx(&full_bar[s], S::kStageBytes);
          if constexpr (MODE == kEpiAllGather) {
            if (ag_src_rank == p.tp_rank) tma_load_2d(sa, &tma_a, &full_bar[s], k * BK, m0 - p.tp_rank * p.ag_rows);
            else tma_load_2d(sa, &tma_g, &full_bar[s], k * BK, ag_parity * p.M + m0);
          } else if (!p.a_mn) {
            tma_load_2d(sa, &tma_a, &full_bar[s], k * BK, m0);
          } else {
#pragma unroll
            for (int c = 0; c < BM / 64; ++c) tma_load_2d(sa + c * (BK * 128), &tma_a, &full_bar[s], m0 + c * 64, k * BK);
          }
          if (!p.b_mn) {
            tma_load_2d(sb, &tma_b, &full_bar[s], k * BK, n0);
          } else {
#pragma unroll
            for (int c = 0; c < (BN + 63) / 64; ++c) tma_load_2d(sb + c * (BK * 128), &tma_b, &full_bar[s], n0 + c * 64, k * BK);
          }
          if (++s == kStages) { s = 0; ph ^= 1; }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      const uint32_t idesc = make_idesc_f16(BM, BN, BF16, p.a_mn != 0, p.b_mn != 0);
      int s = 0;
      uint32_t ph = 0;
      int acc = 0;
      uint32_t acc_ph = 0;
      bool ok = true;
      for (int ti = 0; ok; ++ti) {
        int tm_, tn_, split;
        if (!next_tile<MODE>(p, ti, tm_, tn_, split)) break;
        const int k_lo = split * p.k_iters_per_split, k_hi = min(k_iters_total, k_lo + p.k_iters_per_split);
        if (!pipe_wait(&tempty_bar[acc], acc_ph ^ 1)) break;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int k = k_lo; k < k_hi; ++k) {
          if (!pipe_wait(&full_bar[s], ph)) { ok = false; break; }
          tc_fence_after();
          const uint32_t sa = smem_u32(smem + s * S::kStageBytes);
          const uint32_t sb = sa + S::kABytes;
#pragma unroll
          for (int kk = 0; kk < BK / 16; ++kk) {
            // K-major: 16 elements = 32 bytes inside the 128-byte swizzle row.
            // MN-major: 16 k-rows of 128 bytes.
            const uint64_t da = p.a_mn ? make_smem_desc(sa + kk * 2048, p.lbo_a, p.sbo_a, kSwizzle128B)
                                       : make_smem_desc(sa + kk * 32, 16, 1024, kSwizzle128B);
            const uint64_t db = p.b_mn ? make_smem_desc(sb + kk * 2048, p.lbo_b, p.sbo_b, kSwizzle128B)
                                       : make_smem_desc(sb + kk * 32, 16, 1024, kSwizzle128B);
            umma_f16(d_tmem, da, db, idesc, (k > k_lo || kk > 0) ? 1u : 0u);
          }
          umma_commit(&empty_bar[s]);  // frees the stage once these MMAs have read it
          if (++s == kStages) { s = 0; ph ^= 1; }
        }
        if (!ok) break;
        umma_commit(&tfull_bar[acc]);
        acc ^= 1;
        if (acc == 0) acc_ph ^= 1;
      }
    }
  } else {
    // ------------------------------------------------------------------ epilogue (warps 2..5)
    const int lane_grp = warp & 3;  // TMEM lanes [32*lane_grp, +32) are visible to this warp
    int acc = 0;
    uint32_t acc_ph = 0;
    // MODE 1 running statistics of this thread's row over the CTA's column range
    float st_m = -1e30f, st_s = 0.f, st_u = 0.f, st_t = -INFINITY;
    int st_row = -1;
    if constexpr (MODE == kEpiLogProb) st_row = (blockIdx.x / p.n_splits) * BM + lane_grp * 32 + lane;
    int pr_parity = 0;
    if constexpr (MODE == kEpiPeerReduce) {
      pr_parity = p.pr_state[0] & 1;
      if (p.timeline && threadIdx.x == 64) p.timeline[blockIdx.x * 8 + 0] = global_timer_ns();
    }
    if constexpr (MODE == kEpiAllGather) {
      // ---- push this rank's shard to the peers while the first tiles (own rows) are being computed
      const int et = threadIdx.x - 64;
      const int parity = p.pr_state[8] & 1;
      const long long total = static_cast<long long>(p.ag_rows) * p.K / 8;  // 16-byte vectors
      const long long per = (total + gridDim.x - 1) / gridDim.x;
      const long long lo = per * blockIdx.x, hi = (lo + per < total) ? lo + per : total;
      const uint4* src = reinterpret_cast<const uint4*>(p.ag_src);
      const long long dst_off = (static_cast<long long>(parity) * p.M + static_cast<long long>(p.tp_rank) * p.ag_rows) * p.K / 8;
      for (int rk = 1; rk < p.tp; ++rk) {
        const int dst_rank = (p.tp_rank + rk) % p.tp;
        uint4* dst = reinterpret_cast<uint4*>(p.peer_ag[dst_rank]) + dst_off;
        long long i = lo + et;
        for (; i + 3 * 128 < hi; i += 4 * 128) {
          const uint4 v0 = __ldg(src + i), v1 = __ldg(src + i + 128), v2 = __ldg(src + i + 256), v3 = __ldg(src + i + 384);
          dst[i] = v0; dst[i + 128] = v1; dst[i + 256] = v2; dst[i + 384] = v3;
        }
        for (; i < hi; i += 128) dst[i] = __ldg(src + i);
      }
      named_bar_sync(1, 128);
      if (et < p.tp && et != p.tp_rank) sys_red_add(p.peer_sig[et] + 16 + parity * 8 + p.tp_rank, 1u);
    }
    for (int ti = 0;; ++ti) {
      int tm, tn, split;
      if (!next_tile<MODE>(p, ti, tm, tn, split)) break;
      const int row = tm * BM + lane_grp * 32 + lane;
      st_row = row;
      const int n0 = tn * BN;
      if (!pipe_wait(&tfull_bar[acc], acc_ph)) break;
      tc_fence_after();
      const uint32_t taddr = tmem_base + acc * BN + (static_cast<uint32_t>(lane_grp * 32) << 16);
#pragma unroll 1
      for (int c = 0; c < BN / 32; ++c) {
        uint32_t r[32];
        tmem_ld_32x32b_x32(taddr + c * 32, r);
        tmem_wait_ld();
        const int col = n0 + c * 32;
        if constexpr (MODE == kEpiLogProb) {
          if (row < p.M && col < p.N) {
            const float l2e = 1.4426950408889634f;
            const long long tgt = p.targets[row] - p.vocab_start;
            float mx = st_m;
#pragma unroll
            for (int i = 0; i < 32; ++i) {
              const float z = (col + i < p.N) ? __uint_as_float(r[i]) * p.inv_temp : -1e30f;
              r[i] = __float_as_uint(z);
              mx = fmaxf(mx, z);
            }
            const float alpha = exp2f((st_m - mx) * l2e);
            st_s *= alpha;
            st_u *= alpha;
            st_m = mx;
#pragma unroll
            for (int i = 0; i < 32; ++i) {
              const float z = __uint_as_float(r[i]);
              const float e = exp2f((z - mx) * l2e);
              st_s += e;
              st_u += (col + i < p.N) ? e * z : 0.f;
              if (tgt == col + i) st_t = z;
            }
          }
          continue;
        }
        if constexpr (MODE == kEpiDLogits) {
          if (row < p.M && col < p.N) {
            const float l2e = 1.4426950408889634f;
            const long long tgt = p.targets[row] - p.vocab_start;
            const float logz = p.row_stats[2 * row], ez = p.row_stats[2 * row + 1];
            const float glp = p.g_lp[row];
            const float gen = p.g_ent ? p.g_ent[row] : 0.f;
#pragma unroll
            for (int i = 0; i < 32; ++i) {
              const float z = __uint_as_float(r[i]) * p.inv_temp;
              const float pr = exp2f((z - logz) * l2e);
              float g = -pr * glp + pr * (ez - z) * gen;
              if (tgt == col + i) g += glp;
              r[i] = __float_as_uint(g * p.inv_temp);
            }
          }
        }
        if constexpr (MODE == kEpiPeerReduce) {
          // fp32 partial tile -> slot (parity, my rank, k split) of EVERY rank's symmetric workspace
          // Transpose the warp's 32x32 fp32 block through shared memory so that every store instruction
          // writes whole 128-byte rows (4 rows x 8 lanes x 16 bytes): peer stores over NVLink need full lines.
          float* stg = reinterpret_cast<float*>(smem + S::kBarOffset + 256) + (warp - 2) * (32 * kStagePitch);
#pragma unroll
          for (int i = 0; i < 8; ++i)
            *reinterpret_cast<float4*>(stg + lane * kStagePitch + 4 * i) =
                make_float4(__uint_as_float(r[4 * i]), __uint_as_float(r[4 * i + 1]), __uint_as_float(r[4 * i + 2]),
                            __uint_as_float(r[4 * i + 3]));
          __syncwarp();
          if (col + 32 <= p.N) {
            const size_t slot = (static_cast<size_t>(pr_parity) * p.tp + p.tp_rank) * p.k_splits + split;
            const int row0 = tm * BM + lane_grp * 32;
            const int sub = lane >> 3, c4 = (lane & 7) * 4;
#pragma unroll
            for (int j = 0; j < 8; ++j) {
              const int rr = j * 4 + sub;
              const int grow = row0 + rr;
              if (grow < p.M) {
                const float4 val = *reinterpret_cast<const float4*>(stg + rr * kStagePitch + c4);
                const int owner = p.rs ? grow / p.rows_out : 0;
                const int lrow = p.rs ? grow - owner * p.rows_out : grow;
                const int r_hi = p.rs ? owner + 1 : p.tp;
                const size_t off = (slot * p.rows_out + lrow) * p.N + col + c4;
                for (int rk = owner; rk < r_hi; ++rk) *reinterpret_cast<float4*>(p.peer_ws[rk] + off) = val;
              }
            }
          }
          __syncwarp();
          continue;
        }
        if (row < p.M && col < p.N) {
          float v[32];
#pragma unroll
          for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]);
          if (p.bias) {
            if constexpr (BF16) {
              const __nv_bfloat16* b = reinterpret_cast<const __nv_bfloat16*>(p.bias) + col;
#pragma unroll
              for (int i = 0; i < 32; ++i) if (col + i < p.N) v[i] += __bfloat162float(b[i]);
            } else {
              const __half* b = reinterpret_cast<const __half*>(p.bias) + col;
#pragma unroll
              for (int i = 0; i < 32; ++i) if (col + i < p.N) v[i] += __half2float(b[i]);
            }
          }
          const size_t off = static_cast<size_t>(split) * p.M * p.ldc + static_cast<size_t>(row) * p.ldc + col;
          const bool full = (col + 32 <= p.N);
          if (p.out_fp32) {
            float* out = reinterpret_cast<float*>(p.C) + off;
            if (full && (p.ldc % 4 == 0)) {
#pragma unroll
              for (int i = 0; i < 8; ++i) {
                float4 o = make_float4(v[4 * i], v[4 * i + 1], v[4 * i + 2], v[4 * i + 3]);
                if (p.accumulate) {
                  const float4 old = reinterpret_cast<float4*>(out)[i];
                  o.x += old.x; o.y += old.y; o.z += old.z; o.w += old.w;
                }
                reinterpret_cast<float4*>(out)[i] = o;
              }
            } else {
              for (int i = 0; i < 32 && col + i < p.N; ++i) out[i] = p.accumulate ? out[i] + v[i] : v[i];
            }
          } else {
            uint16_t* out = reinterpret_cast<uint16_t*>(p.C) + off;
            if (full && (p.ldc % 8 == 0) && !p.accumulate) {
#pragma unroll
              for (int i = 0; i < 4; ++i) {
                uint4 o;
                if constexpr (BF16) {
                  o.x = pack_bf16(v[8 * i], v[8 * i + 1]);
                  o.y = pack_bf16(v[8 * i + 2], v[8 * i + 3]);
                  o.z = pack_bf16(v[8 * i + 4], v[8 * i + 5]);
                  o.w = pack_bf16(v[8 * i + 6], v[8 * i + 7]);
                } else {
                  __half2 h0 = __floats2half2_rn(v[8 * i], v[8 * i + 1]), h1 = __floats2half2_rn(v[8 * i + 2], v[8 * i + 3]);
                  __half2 h2 = __floats2half2_rn(v[8 * i + 4], v[8 * i + 5]), h3 = __floats2half2_rn(v[8 * i + 6], v[8 * i + 7]);
                  o.x = *reinterpret_cast<uint32_t*>(&h0); o.y = *reinterpret_cast<uint32_t*>(&h1);
                  o.z = *reinterpret_cast<uint32_t*>(&h2); o.w = *reinterpret_cast<uint32_t*>(&h3);
                }
                reinterpret_cast<uint4*>(out)[i] = o;
              }
            } else {
              for (int i = 0; i < 32 && col + i < p.N; ++i) {
                float x = v[i];
                if constexpr (BF16) {
                  __nv_bfloat16* o = reinterpret_cast<__nv_bfloat16*>(out) + i;
                  if (p.accumulate) x += __bfloat162float(*o);
                  *o = __float2bfloat16(x);
                } else {
                  __half* o = reinterpret_cast<__half*>(out) + i;
                  if (p.accumulate) x += __half2float(*o);
                  *o = __float2half(x);
                }
              }
            }
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&tempty_bar[acc]);
      acc ^= 1;
      if (acc == 0) acc_ph ^= 1;
    }
    if constexpr (MODE == kEpiPeerReduce) {
      // ---- publish: this CTA's partial tiles are on their way to every rank
      const int et = threadIdx.x - 64;  // 0..127 among the epilogue threads
      unsigned long long* tl = (p.timeline && et == 0) ? p.timeline + blockIdx.x * 8 : nullptr;
      if (tl) tl[1] = global_timer_ns();
      // All stores of the 128 epilogue threads are ordered before the barrier; the signalling threads
      // (one per destination, in parallel) then release at system scope, which is cumulative over them.
      named_bar_sync(1, 128);
      if (tl) tl[2] = global_timer_ns();
      if (et < p.tp && !*abort_flag) sys_red_add(p.peer_sig[et] + pr_parity, 1u);
      if (tl) tl[3] = global_timer_ns();
      // ---- wait until every CTA of every rank has published into THIS rank's workspace
      const unsigned target = static_cast<unsigned>(p.pr_state[1 + pr_parity]) + static_cast<unsigned>(p.tp) * gridDim.x;
      if (et == 0) {
        if (!sys_wait_ge(p.peer_sig[p.tp_rank] + pr_parity, target, p.wait_ns)) {
          *abort_flag = 1;
          atomicExch(p.err, 3);
        }
      }
      named_bar_sync(1, 128);
      if (tl) tl[4] = global_timer_ns();
      if (!*abort_flag) {
        __threadfence_system();  // order the reads below after the acquire seen by thread 0
        float* red = reinterpret_cast<float*>(smem);  // pipeline stages are idle by now (all tiles consumed)
        const int slots = p.tp * p.k_splits;
        const float* ws = p.peer_ws[p.tp_rank] + static_cast<size_t>(pr_parity) * slots * p.rows_out * p.N;
        const size_t slot_stride = static_cast<size_t>(p.rows_out) * p.N;
        for (int row = blockIdx.x; row < p.rows_out; row += gridDim.x) {
          const size_t base = static_cast<size_t>(row) * p.N;
          __nv_bfloat16* oh = reinterpret_cast<__nv_bfloat16*>(p.out_h) + base;
          float ss = 0.f;
          // 8 column chunks per pass so that 8 independent 16-byte loads are in flight per slot
          for (int c0 = et * 4; c0 < p.N; c0 += 512 * 8) {
            float4 a[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) a[j] = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll 2
            for (int s = 0; s < slots; ++s) {
              float4 v[8];
#pragma unroll
              for (int j = 0; j < 8; ++j) {
                const int c = c0 + j * 512;
                v[j] = (c < p.N) ? __ldcg(reinterpret_cast<const float4*>(ws + s * slot_stride + base + c))
                                 : make_float4(0.f, 0.f, 0.f, 0.f);
              }
#pragma unroll
              for (int j = 0; j < 8; ++j) { a[j].x += v[j].x; a[j].y += v[j].y; a[j].z += v[j].z; a[j].w += v[j].w; }
            }
#pragma unroll
            for (int j = 0; j < 8; ++j) {
              const int c = c0 + j * 512;
              if (c >= p.N) continue;
              if (p.residual) {
                const uint2 rr = *reinterpret_cast<const uint2*>(reinterpret_cast<const __nv_bfloat16*>(p.residual) + base + c);
                const __nv_bfloat162 r0 = *reinterpret_cast<const __nv_bfloat162*>(&rr.x);
                const __nv_bfloat162 r1 = *reinterpret_cast<const __nv_bfloat162*>(&rr.y);
                a[j].x += __low2float(r0); a[j].y += __high2float(r0); a[j].z += __low2float(r1); a[j].w += __high2float(r1);
              }
              uint2 pk;
              pk.x = pack_bf16(a[j].x, a[j].y);
              pk.y = pack_bf16(a[j].z, a[j].w);
              *reinterpret_cast<uint2*>(oh + c) = pk;
              const __nv_bfloat162 q0 = *reinterpret_cast<const __nv_bfloat162*>(&pk.x);
              const __nv_bfloat162 q1 = *reinterpret_cast<const __nv_bfloat162*>(&pk.y);
              const float h0 = __low2float(q0), h1 = __high2float(q0), h2 = __low2float(q1), h3 = __high2float(q1);
              ss += h0 * h0 + h1 * h1 + h2 * h2 + h3 * h3;
            }
          }
          if (p.norm_w) {
            ss = warp_sum(ss);
            if (lane == 0) red[warp - 2] = ss;
            named_bar_sync(1, 128);
            const float rstd = rsqrtf((red[0] + red[1] + red[2] + red[3]) / p.N + p.eps);
            named_bar_sync(1, 128);
            __nv_bfloat16* ox = reinterpret_cast<__nv_bfloat16*>(p.out_x) + base;
            const __nv_bfloat16* w = reinterpret_cast<const __nv_bfloat16*>(p.norm_w);
            for (int c = et * 4; c < p.N; c += 512) {
              const uint2 hh = *reinterpret_cast<const uint2*>(oh + c);  // this thread's own stores
              const uint2 ww = *reinterpret_cast<const uint2*>(w + c);
              const __nv_bfloat162 h0 = *reinterpret_cast<const __nv_bfloat162*>(&hh.x);
              const __nv_bfloat162 h1 = *reinterpret_cast<const __nv_bfloat162*>(&hh.y);
              const __nv_bfloat162 w0 = *reinterpret_cast<const __nv_bfloat162*>(&ww.x);
              const __nv_bfloat162 w1 = *reinterpret_cast<const __nv_bfloat162*>(&ww.y);
              uint2 pk;
              pk.x = pack_bf16(__low2float(h0) * rstd * __low2float(w0), __high2float(h0) * rstd * __high2float(w0));
              pk.y = pack_bf16(__low2float(h1) * rstd * __low2float(w1), __high2float(h1) * rstd * __high2float(w1));
              *reinterpret_cast<uint2*>(ox + c) = pk;
            }
          }
        }
      }
      // ---- the last CTA of this rank to finish advances the call state for the next launch
      named_bar_sync(1, 128);
      if (tl) tl[5] = global_timer_ns();
      if (et == 0) {
        __threadfence();
        if (atomicAdd(p.pr_state + 3, 1) == static_cast<int>(gridDim.x) - 1) {
          p.pr_state[3] = 0;
          p.pr_state[1 + pr_parity] = static_cast<int>(target);
          p.pr_state[0] = p.pr_state[0] + 1;
          __threadfence();
        }
      }
    }
    if constexpr (MODE == kEpiAllGather) {
      // the last CTA of this rank to finish advances the call state for the next launch
      named_bar_sync(1, 128);
      if (threadIdx.x == 64) {
        __threadfence();
        if (atomicAdd(p.pr_state + 11, 1) == static_cast<int>(gridDim.x) - 1) {
          const int parity = p.pr_state[8] & 1;
          p.pr_state[11] = 0;
          p.pr_state[9 + parity] += static_cast<int>(gridDim.x);
          p.pr_state[8] = p.pr_state[8] + 1;
          __threadfence();
        }
      }
    }
    if constexpr (MODE == kEpiLogProb) {
      if (st_row >= 0 && st_row < p.M) {
        float4 o = make_float4(st_m, st_s, st_u, st_t);
        reinterpret_cast<float4*>(p.partials)[static_cast<size_t>(st_row) * p.n_splits + (blockIdx.x % p.n_splits)] = o;
      }
    }
  }

  // ------------------------------------------------------------------ teardown
  if (*abort_flag) __nanosleep(50000);  // let any bulk copy still in flight land before shared memory is released
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc<kTmemCols>(tmem_base);
  }
}

// ----------------------------------------------------------------------------- host side

static int make_operand_map(CUtensorMap* map, const void* ptr, bool mn_major, int rows_op, int K, int ld, int box_rows) {
  // rows_op = M (for A) or N (for B).  K-major storage: [rows_op][K] -> dims {K, rows_op}, box {64, box_rows}.
  // MN-major storage: [K][rows_op] -> dims {rows_op, K}, box {64, 64}.
  if (!mn_major) return encode_tma_2d_bf16(map, ptr, K, rows_op, ld, BK, box_rows);
  return encode_tma_2d_bf16(map, ptr, rows_op, K, ld, 64, BK);
}

template <int BN, bool BF16, int MODE = kEpiStore>
static int launch(const CUtensorMap& ta, const CUtensorMap& tb, GemmParams p, cudaStream_t stream,
                  const CUtensorMap* tg = nullptr) {
  using S = GemmSmem<BN>;
  static bool attr_set = false;
  constexpr int kSmem = S::kTotal + (MODE == kEpiPeerReduce ? kStageBytes4 : 0);
  auto kern = gemm_kernel<BN, BF16, MODE>;
  if (!attr_set) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmem);
    if (e != cudaSuccess) return static_cast<int>(e);
    attr_set = true;
  }
  p.tiles_m = (p.M + BM - 1) / BM;
  p.tiles_n = (p.N + BN - 1) / BN;
  if (p.k_splits < 1) p.k_splits = 1;
  {
    const int kit = (p.K + BK - 1) / BK;
    p.k_iters_per_split = (kit + p.k_splits - 1) / p.k_splits;
  }
  const int tiles = p.tiles_m * p.tiles_n * p.k_splits;
  int grid = tiles < num_sms() ? tiles : num_sms();
  if (MODE == kEpiLogProb) {
    p.k_splits = 1;
    p.tiles_per_split = (p.tiles_n + p.n_splits - 1) / p.n_splits;
    grid = p.tiles_m * p.n_splits;
  }
  kern<<<grid, GEMM_THREADS, kSmem, stream>>>(ta, tb, tg ? *tg : ta, p);
  rb_note_launch(1);
  return static_cast<int>(cudaGetLastError());
}

}  // namespace rb

extern "C" int rb_gemm(const void* A, const void* B, void* C, const void* bias, int M, int N, int K, int lda, int ldb,
                       int ldc, int a_mn_major, int b_mn_major, int out_fp32, int accumulate, int is_fp16,
                       int force_bn, int lbo_a, int sbo_a, int lbo_b, int sbo_b, int* err_flag, cudaStream_t stream) {
  using namespace rb;
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  if ((lda % 8) || (ldb % 8) || (reinterpret_cast<uintptr_t>(A) % 16) || (reinterpret_cast<uintptr_t>(B) % 16)) return -2;
  int bn = force_bn;
  if (bn == 0) {
    // fill the machine: shrink the N tile while the tile count is below the SM count
    const int tm = (M + BM - 1) / BM;
    bn = 256;
    while (bn > 64 && tm * ((N + bn - 1) / bn) < num_sms()) bn >>= 1;
    if (!b_mn_major && bn == 64 && tm * ((N + 63) / 64) < num_sms() / 2) bn = 32;
  }
  if (b_mn_major && bn < 64) bn = 64;
  GemmParams p{};
  p.M = M; p.N = N; p.K = K; p.ldc = ldc;
  p.out_fp32 = out_fp32; p.accumulate = accumulate;
  p.a_mn = a_mn_major; p.b_mn = b_mn_major;
  // MN-major canonical layout (128-byte swizzle): 64-element chunks along M/N are
  // BK*128 bytes apart (one TMA box each), 8-row k groups are 1024 bytes apart.
  p.lbo_a = lbo_a ? lbo_a : BK * 128; p.sbo_a = sbo_a ? sbo_a : 1024;
  p.lbo_b = lbo_b ? lbo_b : BK * 128; p.sbo_b = sbo_b ? sbo_b : 1024;
  p.C = C; p.bias = bias; p.err = err_flag;
  CUtensorMap ta, tb;
  int rc = make_operand_map(&ta, A, a_mn_major, M, K, lda, BM);
  if (rc) return rc;
  rc = make_operand_map(&tb, B, b_mn_major, N, K, ldb, bn);
  if (rc) return rc;
#define RB_LAUNCH(BN_)                                                              \
  return is_fp16 ? launch<BN_, false>(ta, tb, p, stream) : launch<BN_, true>(ta, tb, p, stream);
  switch (bn) {
    case 256: RB_LAUNCH(256)
    case 128: RB_LAUNCH(128)
    case 64: RB_LAUNCH(64)
    case 32: RB_LAUNCH(32)
    default: return -3;
  }
#undef RB_LAUNCH
}


// Number of column splits the log-prob kernel uses for M rows (callers size `partials` with it).
extern "C" int rb_lm_head_splits(int M, int N) {
  using namespace rb;
  const int tm = (M + BM - 1) / BM;
  const int tn = (N + 255) / 256;
  int splits = (num_sms() + tm - 1) / tm;
  if (splits > tn) splits = tn;
  if (splits < 1) splits = 1;
  const int per = (tn + splits - 1) / splits;
  return (tn + per - 1) / per;  // every split owns at least one column tile
}

// Fused LM head, forward: partials[M][splits][4] of the temperature-scaled logits h W^T
// (never written to memory).  h [M][K], W [N][K] (bf16, K-major).
extern "C" int rb_lm_head_logprob(const void* h, const void* W, const long long* targets, float* partials, int M, int N,
                                  int K, int ldh, int ldw, int vocab_start, float inv_temp, int n_splits, int* err,
                                  cudaStream_t stream) {
  using namespace rb;
  if (M <= 0 || N <= 0) return 0;
  if ((ldh % 8) || (ldw % 8)) return -2;
  GemmParams p{};
  p.M = M; p.N = N; p.K = K; p.ldc = N; p.err = err;
  p.lbo_a = p.lbo_b = BK * 128; p.sbo_a = p.sbo_b = 1024;
  p.targets = targets; p.vocab_start = vocab_start; p.inv_temp = inv_temp; p.n_splits = n_splits; p.partials = partials;
  CUtensorMap ta, tb;
  int rc = make_operand_map(&ta, h, false, M, K, ldh, BM);
  if (rc) return rc;
  rc = make_operand_map(&tb, W, false, N, K, ldw, 256);
  if (rc) return rc;
  return launch<256, true, kEpiLogProb>(ta, tb, p, stream);
}

// Fused LM head, backward helper: dlogits[M][N] (bf16) from recomputed logits.
extern "C" int rb_lm_head_dlogits(const void* h, const void* W, const long long* targets, const float* row_stats,
                                  const float* g_lp, const float* g_ent, void* dlogits, int M, int N, int K, int ldh,
                                  int ldw, int ldd, int vocab_start, float inv_temp, int* err, cudaStream_t stream) {
  using namespace rb;
  if (M <= 0 || N <= 0) return 0;
  if ((ldh % 8) || (ldw % 8)) return -2;
  GemmParams p{};
  p.M = M; p.N = N; p.K = K; p.ldc = ldd; p.C = dlogits; p.err = err;
  p.lbo_a = p.lbo_b = BK * 128; p.sbo_a = p.sbo_b = 1024;
  p.targets = targets; p.vocab_start = vocab_start; p.inv_temp = inv_temp;
  p.row_stats = row_stats; p.g_lp = g_lp; p.g_ent = g_ent;
  CUtensorMap ta, tb;
  int rc = make_operand_map(&ta, h, false, M, K, ldh, BM);
  if (rc) return rc;
  rc = make_operand_map(&tb, W, false, N, K, ldw, 256);
  if (rc) return rc;
  return launch<256, true, kEpiDLogits>(ta, tb, p, stream);
}


namespace rb {
// out[m][n] = sum_s ws[s][m][n] (+ bias[n]) (+ residual[m][n]); 8 columns per thread
template <bool BF16>
__global__ void splitk_reduce_kernel(const float* __restrict__ ws, void* __restrict__ out, const void* __restrict__ bias,
                                     const void* __restrict__ residual, int M, int N, int splits, int ldo) {
  const long long total = static_cast<long long>(M) * (N / 4);
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const int m = static_cast<int>(i / (N / 4)), n = static_cast<int>(i % (N / 4)) * 4;
    float4 a = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int s = 0; s < splits; ++s) {
      const float4 v = *reinterpret_cast<const float4*>(ws + (static_cast<size_t>(s) * M + m) * N + n);
      a.x += v.x; a.y += v.y; a.z += v.z; a.w += v.w;
    }
    using T = typename std::conditional<BF16, __nv_bfloat16, __half>::type;
    auto tof = [](T v) { if constexpr (BF16) return __bfloat162float(v); else return __half2float(v); };
    if (bias) { const T* b = reinterpret_cast<const T*>(bias) + n; a.x += tof(b[0]); a.y += tof(b[1]); a.z += tof(b[2]); a.w += tof(b[3]); }
    if (residual) {
      const T* r = reinterpret_cast<const T*>(residual) + static_cast<size_t>(m) * ldo + n;
      a.x += tof(r[0]); a.y += tof(r[1]); a.z += tof(r[2]); a.w += tof(r[3]);
    }
    T* o = reinterpret_cast<T*>(out) + static_cast<size_t>(m) * ldo + n;
    if constexpr (BF16) {
      uint2 pk; pk.x = pack_bf16(a.x, a.y); pk.y = pack_bf16(a.z, a.w);
      *reinterpret_cast<uint2*>(o) = pk;
    } else {
      o[0] = __float2half(a.x); o[1] = __float2half(a.y); o[2] = __float2half(a.z); o[3] = __float2half(a.w);
    }
  }
}
}  // namespace rb

// Split-K plan for skinny problems (decode): returns the number of K splits (1 = do not split) and the N tile.
extern "C" int rb_gemm_splitk_plan(int M, int N, int K, int* bn_out) {
  using namespace rb;
  const int tm = (M + BM - 1) / BM;
  int bn = 128;
  if (N % 128 && N % 64 == 0) bn = 64;
  const int tiles = tm * ((N + bn - 1) / bn);
  const int kit = (K + BK - 1) / BK;
  int splits = 1;
  if (tiles < num_sms()) {
    splits = num_sms() / tiles;
    if (splits > kit / 8) splits = kit / 8;   // at least 8 k-iterations (512 elements) per split
    if (splits < 1) splits = 1;
    if (splits > 16) splits = 16;
  }
  *bn_out = bn;
  return splits;
}

// C[M,N] = A[M,K] * B[N,K]^T through split-K: workspace fp32 [splits][M][N] supplied by the caller.
extern "C" int rb_gemm_splitk(const void* A, const void* B, void* C, const void* bias, const void* residual, float* workspace,
                              int M, int N, int K, int lda, int ldb, int ldc, int splits, int bn, int is_fp16, int* err_flag,
                              cudaStream_t stream) {
  using namespace rb;
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  if ((lda % 8) || (ldb % 8) || (N % 4) || (reinterpret_cast<uintptr_t>(A) % 16) || (reinterpret_cast<uintptr_t>(B) % 16)) return -2;
  GemmParams p{};
  p.M = M; p.N = N; p.K = K; p.ldc = N;
  p.out_fp32 = 1; p.accumulate = 0;
  p.lbo_a = p.lbo_b = BK * 128; p.sbo_a = p.sbo_b = 1024;
  p.C = workspace; p.err = err_flag; p.k_splits = splits;
  CUtensorMap ta, tb;
  int rc = make_operand_map(&ta, A, false, M, K, lda, BM);
  if (rc) return rc;
  rc = make_operand_map(&tb, B, false, N, K, ldb, bn);
  if (rc) return rc;
  if (bn == 128) rc = is_fp16 ? launch<128, false>(ta, tb, p, stream) : launch<128, true>(ta, tb, p, stream);
  else if (bn == 64) rc = is_fp16 ? launch<64, false>(ta, tb, p, stream) : launch<64, true>(ta, tb, p, stream);
  else return -3;
  if (rc) return rc;
  if (C == nullptr) return 0;  // partial sums only: the caller runs its own fused reduction
  long long blocks = (static_cast<long long>(M) * (N / 4) + 255) / 256;
  if (blocks > num_sms() * 8LL) blocks = num_sms() * 8LL;
  if (is_fp16) splitk_reduce_kernel<false><<<(int)blocks, 256, 0, stream>>>(workspace, C, bias, residual, M, N, splits, ldc);
  else splitk_reduce_kernel<true><<<(int)blocks, 256, 0, stream>>>(workspace, C, bias, residual, M, N, splits, ldc);
  rb_note_launch(1);
  return static_cast<int>(cudaGetLastError());
}

// ----------------------------------------------------------------------------- GEMM + all-reduce + residual + RMSNorm
// Plan of the fused row-parallel GEMM (decode: M <= a few hundred rows): N tile and K splits.  Every rank
// calls it with the same shapes and so gets the same plan (the workspace slot layout depends on it).
extern "C" int rb_gemm_ar_plan(int M, int N, int K, int* bn_out) {
  using namespace rb;
  const int tm = (M + BM - 1) / BM;
  const int bn = (N % 64 == 0) ? 64 : 32;
  const int tiles = tm * (N / bn);
  const int kit = (K + BK - 1) / BK;
  int splits = num_sms() / (tiles > 0 ? tiles : 1);
  if (splits > kit / 8) splits = kit / 8;
  if (splits > 4) splits = 4;
  if (splits < 1) splits = 1;
  *bn_out = bn;
  return splits;
}

// out_h = residual + sum_r A_r B_r^T ; out_x = rmsnorm(out_h) * norm_w, with the sum over the `tp` ranks done
// inside the kernel over peer memory.  A [M][K] and B [N][K] are this rank's K shards (bf16, K-major).
// peer_ws / peer_sig: host arrays of `tp` device pointers (rank r's workspace / counters as mapped in this
// process).  The workspace holds 2*tp*splits*rows_out*N floats (rows_out = M, or M/tp when reduce_scatter).
// reduce_scatter: rank r keeps rows [r*M/tp, (r+1)*M/tp) only; out_h is then [M/tp][N].  state: 4 ints of this rank, zero at set-up.
extern "C" int rb_gemm_ar_rmsnorm(const void* A, const void* B, int M, int N, int K, int lda, int ldb, int tp, int tp_rank,
                                  float* const* peer_ws, unsigned* const* peer_sig, int* state, const void* residual,
                                  const void* norm_w, void* out_h, void* out_x, float eps, int splits, int bn,
                                  int reduce_scatter, int b_mn_major, unsigned long long wait_ns,
                                  unsigned long long* timeline, int* err_flag, cudaStream_t stream) {
  using namespace rb;
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  if (tp < 1 || tp > 8 || tp_rank < 0 || tp_rank >= tp) return -4;
  if (reduce_scatter && (M % tp)) return -5;
  if (b_mn_major && bn < 64) return -3;
  if ((lda % 8) || (ldb % 8) || (N % 32) || (reinterpret_cast<uintptr_t>(A) % 16) || (reinterpret_cast<uintptr_t>(B) % 16)) return -2;
  GemmParams p{};
  p.M = M; p.N = N; p.K = K; p.ldc = N;
  p.lbo_a = p.lbo_b = BK * 128; p.sbo_a = p.sbo_b = 1024;
  p.err = err_flag; p.k_splits = splits;
  p.tp = tp; p.tp_rank = tp_rank;
  p.rs = reduce_scatter; p.rows_out = reduce_scatter ? M / tp : M; p.b_mn = b_mn_major;
  if (reduce_scatter) {
    // start with the rows of rank+1, finish with this rank's own rows
    const int tiles_m = (M + BM - 1) / BM;
    p.tm_rot = static_cast<int>((static_cast<long long>((tp_rank + 1) % tp) * p.rows_out) / BM) % tiles_m;
  }
  for (int r = 0; r < tp; ++r) { p.peer_ws[r] = peer_ws[r]; p.peer_sig[r] = peer_sig[r]; }
  p.pr_state = state; p.residual = residual; p.norm_w = norm_w; p.out_h = out_h; p.out_x = out_x; p.eps = eps;
  p.wait_ns = wait_ns; p.timeline = timeline;
  CUtensorMap ta, tb;
  int rc = make_operand_map(&ta, A, false, M, K, lda, BM);
  if (rc) return rc;
  rc = make_operand_map(&tb, B, b_mn_major != 0, N, K, ldb, bn);
  if (rc) return rc;
  if (bn == 256) return launch<256, true, kEpiPeerReduce>(ta, tb, p, stream);
  if (bn == 128) return launch<128, true, kEpiPeerReduce>(ta, tb, p, stream);
  if (bn == 64) return launch<64, true, kEpiPeerReduce>(ta, tb, p, stream);
  if (bn == 32) return launch<32, true, kEpiPeerReduce>(ta, tb, p, stream);
  return -3;
}

// ----------------------------------------------------------------------------- all-gather + GEMM
// y[M][N] = all_gather_rows(x_shard)[M][K] * W[N][K]^T with the gather done by the kernel itself: peers' shards
// arrive in `peer_ag[tp_rank]` (this rank's gathered buffer, [2][M][K] bf16, double buffered by call parity)
// while the tiles of this rank's own rows are computed straight from `x_shard`.  M = tp * rows of a shard, and
// a shard must hold a multiple of 128 rows.  state: ints [8..11] of the same array the reduce kernels use;
// peer_sig: counters [16..31] of every rank's signal pad.
extern "C" int rb_ag_gemm(const void* x_shard, const void* B, void* C, int M, int N, int K, int ldb, int ldc, int tp,
                          int tp_rank, void* const* peer_ag, unsigned* const* peer_sig, int* state, int bn,
                          unsigned long long wait_ns, int* err_flag, cudaStream_t stream) {
  using namespace rb;
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  if (tp < 1 || tp > 8 || tp_rank < 0 || tp_rank >= tp) return -4;
  if ((M % tp) || ((M / tp) % BM) || (K % 8) || (ldb % 8)) return -2;
  GemmParams p{};
  p.M = M; p.N = N; p.K = K; p.ldc = ldc; p.C = C;
  p.lbo_a = p.lbo_b = BK * 128; p.sbo_a = p.sbo_b = 1024;
  p.err = err_flag; p.k_splits = 1;
  p.tp = tp; p.tp_rank = tp_rank; p.ag_rows = M / tp; p.ag_src = x_shard;
  for (int r = 0; r < tp; ++r) { p.peer_ag[r] = peer_ag[r]; p.peer_sig[r] = peer_sig[r]; }
  p.pr_state = state; p.wait_ns = wait_ns;
  p.tm_rot = tp_rank * (p.ag_rows / BM);  // own rows first
  CUtensorMap ta, tb, tg;
  int rc = make_operand_map(&ta, x_shard, false, p.ag_rows, K, K, BM);
  if (rc) return rc;
  rc = make_operand_map(&tg, peer_ag[tp_rank], false, 2 * M, K, K, BM);
  if (rc) return rc;
  rc = make_operand_map(&tb, B, false, N, K, ldb, bn);
  if (rc) return rc;
  if (bn == 256) return launch<256, true, kEpiAllGather>(ta, tb, p, stream, &tg);
  if (bn == 128) return launch<128, true, kEpiAllGather>(ta, tb, p, stream, &tg);
  if (bn == 64) return launch<64, true, kEpiAllGather>(ta, tb, p, stream, &tg);
  return -3;
}
