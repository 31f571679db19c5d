// CTA-pair GEMM for sm_100a: two CTAs of a cluster work on one 256 x BN tile with `tcgen05.mma.cta_group::2`.
//
//   C[M,N] (+)= A_op[M,K] * B_op[N,K]^T        bf16 in, fp32 accumulate, bf16 or fp32 out
//
// Why a pair: a single-CTA 128 x 256 tile has to pull 16 KB of A and 32 KB of B into shared memory per 64-deep
// k step, which at full tensor rate is close to what the L2 -> shared-memory path of one SM can deliver.  In a
// pair each CTA loads its own 128 rows of A and only HALF of the B tile (the tensor cores of both SMs read both
// halves), so the same math needs two thirds of the fill bandwidth per SM.
//
// Roles per CTA (192 threads): warp 0 = TMA producer (own A rows, own half of B; completion is counted on the
// LEADER CTA's barrier), warp 1 = MMA issuer (leader CTA only; both CTAs allocate TMEM), warps 2..5 = epilogue
// (own 128 accumulator rows: TMEM -> registers -> swizzled shared-memory staging -> TMA store, or TMA
// reduce-add for fp32 accumulation, so gradient accumulation reads nothing back into the SM).
// No load in this file uses cluster multicast; the only multicast is the barrier arrive of `tcgen05.commit`.
// Operand storage is as in gemm_sm100.cu (K-major or MN-major, row-major in global memory).
#include "common.cuh"
#include "host_utils.h"

namespace rb {
namespace g2 {

constexpr int BM = 128;          // rows per CTA (256 per pair)
constexpr int BK = 64;
constexpr int THREADS = 192;

struct Params {
  int M, N, K;
  int tiles_m2, tiles_n;      // pair tiles
  int a_mn, b_mn;
  uint32_t lbo_a, sbo_a, lbo_b, sbo_b;
  int out_fp32, accumulate;
  int* err;
};

template <int BN>
struct Smem {
  static constexpr int kStages = (BN >= 256) ? 5 : 7;
  static constexpr int kABytes = BM * BK * 2;             // 16 KB
  static constexpr int kBBytes = (BN / 2) * BK * 2;       // this CTA's half of the B tile
  static constexpr int kStageBytes = kABytes + kBBytes;
  static constexpr int kEpiOffset = kStages * kStageBytes;   // 4 warps x 2 buffers x 4 KB, 1024-byte aligned
  static constexpr int kEpiBytes = 4 * 2 * 4096;
  static constexpr int kBarOffset = kEpiOffset + kEpiBytes;
  static constexpr int kTotal = kBarOffset + 256 + 1024;     // barriers + alignment slack
};

__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// shared::cluster address of the same shared-memory location in CTA `rank` of this cluster
__device__ __forceinline__ uint32_t map_to_cta(uint32_t smem_addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(smem_addr), "r"(rank));
  return r;
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
// TMA load of this CTA's tile into its own shared memory; the bytes are counted on the barrier at
// `bar_cluster_addr`, which may live in the peer CTA (the leader of the pair).  No multicast.
__device__ __forceinline__ void tma_load_2d_pair(void* smem_dst, const CUtensorMap* m, uint32_t bar_cluster_addr, int x, int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(m)), "r"(bar_cluster_addr), "r"(x), "r"(y)
      : "memory");
}
template <int NCOLS>
__device__ __forceinline__ void tmem_alloc_pair(uint32_t* smem_result) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_result)), "r"(NCOLS)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish_pair() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
template <int NCOLS>
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t taddr) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(NCOLS) : "memory");
}
__device__ __forceinline__ void umma_f16_pair(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// Arrive on the barrier at the same offset in BOTH CTAs of the pair once the MMAs issued so far have completed.
__device__ __forceinline__ void umma_commit_pair(uint64_t* bar) {
  const uint16_t mask = 0x3;
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
               ::"r"(smem_u32(bar)), "h"(mask)
               : "memory");
}
__device__ __forceinline__ void tma_reduce_add_2d(const CUtensorMap* m, const void* smem_src, int x, int y) {
  asm volatile("cp.reduce.async.bulk.tensor.2d.global.shared::cta.add.tile.bulk_group [%0, {%2, %3}], [%1];"
               ::"l"(reinterpret_cast<uint64_t>(m)), "r"(smem_u32(smem_src)), "r"(x), "r"(y)
               : "memory");
}

__device__ __forceinline__ void pair_tile_coords(int t, int tiles_m, int tiles_n, int& tm, int& tn) {
  constexpr int GM = 4;     // 4 pair rows = 1024 rows of A share a sweep over the column tiles (L2 reuse)
  const int per_group = GM * tiles_n;
  const int group = t / per_group;
  const int first_m = group * GM;
  const int gm = min(tiles_m - first_m, GM);
  const int r = t - group * per_group;
  tm = first_m + (r % gm);
  tn = r / gm;
}

template <int BN>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(THREADS, 1)
gemm2_kernel(const __grid_constant__ CUtensorMap tma_a, const __grid_constant__ CUtensorMap tma_b,
             const __grid_constant__ CUtensorMap tma_c, const Params p) {
  using S = Smem<BN>;
  constexpr int kStages = S::kStages;
  constexpr int kTmemCols = 2 * BN;       // two accumulator buffers of BN fp32 columns
  constexpr int HN = BN / 2;              // B rows (N columns) held by one CTA
  extern __shared__ uint8_t smem_raw[];
  // both CTAs of the pair must place their buffers at the same offsets: the dynamic shared-memory window starts at
  // the same address in every CTA of a kernel, so the same round-up gives the same layout
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + S::kBarOffset);
  uint64_t* empty_bar = full_bar + kStages;
  uint64_t* tfull_bar = empty_bar + kStages;   // [2]
  uint64_t* tempty_bar = tfull_bar + 2;        // [2]  (the leader's are the ones waited on)
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tempty_bar + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t cta_rank = cluster_ctarank();
  const bool leader = cta_rank == 0;
  const int k_iters = (p.K + BK - 1) / BK;
  const int n_pairs = gridDim.x / 2, pair_id = blockIdx.x / 2;
  const int total_tiles = p.tiles_m2 * p.tiles_n;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      mbar_init(&full_bar[s], 1);      // the leader's producer arrives once with the bytes of BOTH CTAs' loads
      mbar_init(&empty_bar[s], 1);     // one multicast commit per use
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&tfull_bar[a], 1);
      mbar_init(&tempty_bar[a], 8);    // four epilogue warps in each CTA of the pair
    }
    *abort_flag = 0;
    fence_barrier_init();
  }
  if (warp == 1) {
    tmem_alloc_pair<kTmemCols>(tmem_slot);
    tmem_relinquish_pair();
  }
  tc_fence_before();
  cluster_sync_all();                  // barriers of both CTAs are initialised before anyone signals across
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer (both CTAs)
    if (lane == 0) {
      tma_prefetch_desc(&tma_a);
      tma_prefetch_desc(&tma_b);
      int s = 0;
      uint32_t ph = 0;
      bool ok = true;
      for (int t = pair_id; t < total_tiles && ok; t += n_pairs) {
        int tm, tn;
        pair_tile_coords(t, p.tiles_m2, p.tiles_n, tm, tn);
        const int m0 = tm * 256 + static_cast<int>(cta_rank) * BM;
        const int n0 = tn * BN + static_cast<int>(cta_rank) * HN;
        for (int k = 0; k < k_iters; ++k) {
          if (!mbar_wait(&empty_bar[s], ph ^ 1, abort_flag, p.err)) { ok = false; break; }
          uint8_t* sa = smem + s * S::kStageBytes;
          uint8_t* sb = sa + S::kABytes;
          const uint32_t bar = map_to_cta(smem_u32(&full_bar[s]), 0);
          if (leader) mbar_expect_tx(&full_bar[s], 2 * S::kStageBytes);
          if (!p.a_mn) {
            tma_load_2d_pair(sa, &tma_a, bar, k * BK, m0);
          } else {
#pragma unroll
            for (int c = 0; c < BM / 64; ++c) tma_load_2d_pair(sa + c * (BK * 128), &tma_a, bar, m0 + c * 64, k * BK);
          }
          if (!p.b_mn) {
            tma_load_2d_pair(sb, &tma_b, bar, k * BK, n0);
          } else {
#pragma unroll
            for (int c = 0; c < HN / 64; ++c) tma_load_2d_pair(sb + c * (BK * 128), &tma_b, bar, n0 + c * 64, k * BK);
          }
          if (++s == kStages) { s = 0; ph ^= 1; }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer (leader CTA only)
    if (lane == 0 && leader) {
      const uint32_t idesc = make_idesc_f16(256, BN, true, p.a_mn != 0, p.b_mn != 0);
      int s = 0;
      uint32_t ph = 0;
      int acc = 0;
      uint32_t acc_ph = 0;
      bool ok = true;
      for (int t = pair_id; t < total_tiles && ok; t += n_pairs) {
        if (!mbar_wait(&tempty_bar[acc], acc_ph ^ 1, abort_flag, p.err)) break;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int k = 0; k < k_iters; ++k) {
          if (!mbar_wait(&full_bar[s], ph, abort_flag, p.err)) { ok = false; break; }
          tc_fence_after();
          const uint32_t sa = smem_u32(smem + s * S::kStageBytes);
          const uint32_t sb = sa + S::kABytes;
#pragma unroll
          for (int kk = 0; kk < BK / 16; ++kk) {
            const uint64_t da = p.a_mn ? make_smem_desc(sa + kk * 2048, p.lbo_a, p.sbo_a, kSwizzle128B)
                                       : make_smem_desc(sa + kk * 32, 16, 1024, kSwizzle128B);
            const uint64_t db = p.b_mn ? make_smem_desc(sb + kk * 2048, p.lbo_b, p.sbo_b, kSwizzle128B)
                                       : make_smem_desc(sb + kk * 32, 16, 1024, kSwizzle128B);
            umma_f16_pair(d_tmem, da, db, idesc, (k > 0 || kk > 0) ? 1u : 0u);
          }
          umma_commit_pair(&empty_bar[s]);    // frees the stage in both CTAs once these MMAs have read it
          if (++s == kStages) { s = 0; ph ^= 1; }
        }
        if (!ok) break;
        umma_commit_pair(&tfull_bar[acc]);
        acc ^= 1;
        if (acc == 0) acc_ph ^= 1;
      }
    }
  } else {
    // ------------------------------------------------------------------ epilogue (warps 2..5 of both CTAs)
    const int lane_grp = warp & 3;     // TMEM lanes [32*lane_grp, +32) are visible to this warp
    uint8_t* stage = smem + S::kEpiOffset + lane_grp * 8192;
    const uint32_t tempty_leader[2] = {map_to_cta(smem_u32(&tempty_bar[0]), 0), map_to_cta(smem_u32(&tempty_bar[1]), 0)};
    int acc = 0;
    uint32_t acc_ph = 0;
    int buf = 0;
    for (int t = pair_id; t < total_tiles; t += n_pairs) {
      int tm, tn;
      pair_tile_coords(t, p.tiles_m2, p.tiles_n, tm, tn);
      const int row0 = tm * 256 + static_cast<int>(cta_rank) * BM + lane_grp * 32;
      const int n0 = tn * BN;
      if (!mbar_wait(&tfull_bar[acc], acc_ph, abort_flag, p.err)) break;
      tc_fence_after();
      const uint32_t taddr = tmem_base + acc * BN + (static_cast<uint32_t>(lane_grp * 32) << 16);
      if (!p.out_fp32) {
        // ---- bf16 output: 64 columns (128 bytes per row) per TMA store, two tcgen05.ld in flight per wait
#pragma unroll 1
        for (int c = 0; c < BN / 64; ++c) {
          uint32_t r0[32], r1[32];
          tmem_ld_32x32b_x32(taddr + c * 64, r0);
          tmem_ld_32x32b_x32(taddr + c * 64 + 32, r1);
          tmem_wait_ld();
          if (c == BN / 64 - 1) {          // accumulator fully read: hand the TMEM buffer back before the stores finish
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive_cluster(tempty_leader[acc]);
          }
          if (lane == 0) tma_store_wait_read<1>();     // the store that last read this staging buffer has drained it
          __syncwarp();
          uint8_t* dst = stage + buf * 4096 + lane * 128;
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            uint4 o;
            o.x = pack_bf16(__uint_as_float(r0[8 * j]), __uint_as_float(r0[8 * j + 1]));
            o.y = pack_bf16(__uint_as_float(r0[8 * j + 2]), __uint_as_float(r0[8 * j + 3]));
            o.z = pack_bf16(__uint_as_float(r0[8 * j + 4]), __uint_as_float(r0[8 * j + 5]));
            o.w = pack_bf16(__uint_as_float(r0[8 * j + 6]), __uint_as_float(r0[8 * j + 7]));
            *reinterpret_cast<uint4*>(dst + ((j ^ (lane & 7)) << 4)) = o;
          }
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            uint4 o;
            o.x = pack_bf16(__uint_as_float(r1[8 * j]), __uint_as_float(r1[8 * j + 1]));
            o.y = pack_bf16(__uint_as_float(r1[8 * j + 2]), __uint_as_float(r1[8 * j + 3]));
            o.z = pack_bf16(__uint_as_float(r1[8 * j + 4]), __uint_as_float(r1[8 * j + 5]));
            o.w = pack_bf16(__uint_as_float(r1[8 * j + 6]), __uint_as_float(r1[8 * j + 7]));
            *reinterpret_cast<uint4*>(dst + (((4 + j) ^ (lane & 7)) << 4)) = o;
          }
          fence_proxy_async();
          __syncwarp();
          if (lane == 0 && row0 < p.M && n0 + c * 64 < p.N) {
            tma_store_2d(&tma_c, stage + buf * 4096, n0 + c * 64, row0);
            tma_store_commit();
          } else if (lane == 0) {
            tma_store_commit();     // keep the group count in step with the buffer rotation
          }
          buf ^= 1;
        }
      } else {
        // ---- fp32 output: 32 columns (128 bytes per row) per TMA store / reduce-add
#pragma unroll 1
        for (int c = 0; c < BN / 32; ++c) {
          uint32_t r0[32];
          tmem_ld_32x32b_x32(taddr + c * 32, r0);
          tmem_wait_ld();
          if (c == BN / 32 - 1) {
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive_cluster(tempty_leader[acc]);
          }
          if (lane == 0) tma_store_wait_read<1>();
          __syncwarp();
          uint8_t* dst = stage + buf * 4096 + lane * 128;
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            uint4 o = make_uint4(r0[4 * j], r0[4 * j + 1], r0[4 * j + 2], r0[4 * j + 3]);
            *reinterpret_cast<uint4*>(dst + ((j ^ (lane & 7)) << 4)) = o;
          }
          fence_proxy_async();
          __syncwarp();
          if (lane == 0) {
            if (row0 < p.M && n0 + c * 32 < p.N) {
              if (p.accumulate) tma_reduce_add_2d(&tma_c, stage + buf * 4096, n0 + c * 32, row0);
              else tma_store_2d(&tma_c, stage + buf * 4096, n0 + c * 32, row0);
            }
            tma_store_commit();
          }
          buf ^= 1;
        }
      }
      acc ^= 1;
      if (acc == 0) acc_ph ^= 1;
    }
    if (lane == 0) tma_store_wait<0>();   // every store of this warp has completed before shared memory goes away
    __syncwarp();
  }

  // ------------------------------------------------------------------ teardown
  if (*abort_flag) __nanosleep(50000);   // let any bulk copy still in flight land before shared memory is released
  tc_fence_before();
  cluster_sync_all();                    // the leader's MMAs read the peer's shared memory: leave together
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc_pair<kTmemCols>(tmem_base);
  }
}

static int make_operand_map(CUtensorMap* map, const void* ptr, bool mn_major, int rows_op, int K, int ld, int box_rows) {
  if (!mn_major) return encode_tma_2d_bf16(map, ptr, K, rows_op, ld, BK, box_rows);
  return encode_tma_2d_bf16(map, ptr, rows_op, K, ld, 64, BK);
}

template <int BN>
static int launch(const CUtensorMap& ta, const CUtensorMap& tb, const CUtensorMap& tc, Params p, cudaStream_t stream) {
  using S = Smem<BN>;
  static int max_pairs = -1;
  auto kern = gemm2_kernel<BN>;
  if (max_pairs < 0) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, S::kTotal);
    if (e != cudaSuccess) return static_cast<int>(e);
    // how many CTA pairs the device can hold at once (pairs need two SMs of one GPC)
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(num_sms() / 2 * 2);
    cfg.blockDim = dim3(THREADS);
    cfg.dynamicSmemBytes = S::kTotal;
    int n = 0;
    e = cudaOccupancyMaxActiveClusters(&n, kern, &cfg);
    if (e != cudaSuccess || n <= 0) { (void)cudaGetLastError(); n = num_sms() / 2; }
    if (n > num_sms() / 2) n = num_sms() / 2;
    max_pairs = n;
  }
  p.tiles_m2 = (p.M + 255) / 256;
  p.tiles_n = (p.N + BN - 1) / BN;
  const int tiles = p.tiles_m2 * p.tiles_n;
  const int pairs = tiles < max_pairs ? tiles : max_pairs;
  kern<<<2 * pairs, THREADS, S::kTotal, stream>>>(ta, tb, tc, p);
  rb_note_launch(1);
  return static_cast<int>(cudaGetLastError());
}

}  // namespace g2
}  // namespace rb

// Same contract as rb_gemm (bf16 inputs), without bias.  Returns -20 when the problem does not meet the extra
// requirements of the TMA-store epilogue (C 16-byte aligned with a 16-byte multiple pitch) or is too small
// for pair tiles to pay; callers then use rb_gemm.
extern "C" int rb_gemm_pair(const void* A, const void* B, void* C, int M, int N, int K, int lda, int ldb, int ldc,
                            int a_mn_major, int b_mn_major, int out_fp32, int accumulate, int force_bn, int* err_flag,
                            cudaStream_t stream) {
  using namespace rb;
  using namespace rb::g2;
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  if ((lda % 8) || (ldb % 8) || (reinterpret_cast<uintptr_t>(A) % 16) || (reinterpret_cast<uintptr_t>(B) % 16)) return -2;
  const int esz = out_fp32 ? 4 : 2;
  if ((reinterpret_cast<uintptr_t>(C) % 16) || ((static_cast<long long>(ldc) * esz) % 16)) return -20;
  if (accumulate && !out_fp32) return -20;
  int bn = force_bn;
  if (bn == 0) {
    const int t2 = (M + 255) / 256;
    bn = 256;
    if (t2 * ((N + 255) / 256) < num_sms() / 2 && N > 128) bn = 128;
  }
  if (bn != 256 && bn != 128) return -3;
  Params p{};
  p.M = M; p.N = N; p.K = K;
  p.a_mn = a_mn_major; p.b_mn = b_mn_major;
  p.lbo_a = BK * 128; p.sbo_a = 1024; p.lbo_b = BK * 128; p.sbo_b = 1024;
  p.out_fp32 = out_fp32; p.accumulate = accumulate; p.err = err_flag;
  CUtensorMap ta, tb, tc;
  int rc = make_operand_map(&ta, A, a_mn_major, M, K, lda, BM);
  if (rc) return rc;
  rc = make_operand_map(&tb, B, b_mn_major, N, K, ldb, bn / 2);
  if (rc) return rc;
  if (out_fp32) rc = encode_tma_2d_32bit(&tc, C, N, M, ldc, 32, 32);
  else rc = encode_tma_2d_16bit(&tc, C, N, M, ldc, 64, 32, true, true);
  if (rc) return rc;
  return bn == 256 ? launch<256>(ta, tb, tc, p, stream) : launch<128>(ta, tb, tc, p, stream);
}
