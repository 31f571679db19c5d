// Grouped GEMM for mixture-of-experts layers on sm_100a: ONE launch covers all local experts.
//
// Tokens arrive sorted by expert in a buffer whose per-expert row ranges are padded to multiples of 128 rows
// (padding rows are zero), so a 128-row tile never straddles two experts and the tile -> expert map is a small
// device array.  Nothing about the routing is known on the host: the grid is persistent and every CTA walks the
// tile list it reads from device memory, so no count ever has to be copied back to launch the experts.
//
//   kForward : Y[row, :]  = X[row, :]  * W[e(row)]^T          X [cap, K],   W [E, N, K]   (A, B K-major)
//   kDgrad   : dX[row, :] = dY[row, :] * W[e(row)]            dY [cap, N'], W [E, N', K'] (B MN-major)
//   kWgrad   : dW[e] (+)= dY_e^T * X_e                        reduction over the rows of expert e (A, B MN-major)
//
// Pipeline as in gemm_sm100.cu: warp 0 = TMA producer, warp 1 = MMA issuer + TMEM owner (tcgen05.mma, fp32
// accumulators in TMEM, double buffered), warps 2..5 = epilogue.  Every wait is bounded.
#include "common.cuh"
#include "host_utils.h"

namespace rb {
namespace gg {

constexpr int BM = 128;
constexpr int BK = 64;
constexpr int BN = 128;
constexpr int THREADS = 192;
constexpr int kStages = 6;
constexpr int kABytes = BM * BK * 2;
constexpr int kBBytes = BN * BK * 2;
constexpr int kStageBytes = kABytes + kBBytes;
constexpr int kBarOffset = kStages * kStageBytes;
constexpr int kSmemTotal = kBarOffset + 256 + 1024;
constexpr int kTmemCols = 2 * BN;

enum : int { kForward = 0, kDgrad = 1, kWgrad = 2 };

struct Params {
  int rows_cap;              // rows of the padded token buffer (multiple of 128)
  int N, K;                  // forward / dgrad: output columns and reduction length; wgrad: dW is [N, K]
  int E;                     // local experts
  const int* tile_expert;    // [rows_cap / 128] expert of each 128-row tile, -1 = unused tile
  const int* expert_rows;    // [E + 1] padded row offsets (wgrad)
  void* C;                   // forward / dgrad: bf16 [rows_cap, N]; wgrad: [E, N, K] fp32 or bf16
  int out_fp32, accumulate;
  int* err;
};

// tile t -> (m tile / expert, n tile); n fastest so that consecutive CTAs share the A rows in L2
__device__ __forceinline__ void tile_of(int t, int tiles_n, int& a, int& tn) {
  a = t / tiles_n;
  tn = t - a * tiles_n;
}

template <int MODE>
__global__ void __launch_bounds__(THREADS, 1)
grouped_gemm_kernel(const __grid_constant__ CUtensorMap tma_a, const __grid_constant__ CUtensorMap tma_b, const Params p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + kBarOffset);
  uint64_t* empty_bar = full_bar + kStages;
  uint64_t* tfull_bar = empty_bar + kStages;   // [2]
  uint64_t* tempty_bar = tfull_bar + 2;        // [2]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tempty_bar + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  // work list: forward / dgrad: (128-row tile, n tile); wgrad: (expert, m tile of N, n tile of K)
  const int tiles_n = (MODE == kWgrad) ? (p.K + BN - 1) / BN : (p.N + BN - 1) / BN;
  const int tiles_a = (MODE == kWgrad) ? p.E * ((p.N + BM - 1) / BM) : p.rows_cap / BM;
  const int total = tiles_a * tiles_n;
  const int wg_tiles_m = (p.N + BM - 1) / BM;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) { mbar_init(&full_bar[s], 1); mbar_init(&empty_bar[s], 1); }
    for (int a = 0; a < 2; ++a) { mbar_init(&tfull_bar[a], 1); mbar_init(&tempty_bar[a], 4); }
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

  // k range of a work item: forward / dgrad the whole reduction; wgrad the rows of the expert
  auto k_range = [&](int a, int& k_lo, int& k_hi, int& expert) {
    if constexpr (MODE == kWgrad) {
      expert = a / wg_tiles_m;
      k_lo = p.expert_rows[expert] / BK;
      k_hi = p.expert_rows[expert + 1] / BK;
    } else {
      expert = p.tile_expert[a];
      k_lo = 0;
      k_hi = expert < 0 ? 0 : (((MODE == kForward) ? p.K : p.K) + BK - 1) / BK;
    }
  };
  constexpr bool A_MN = (MODE == kWgrad);
  constexpr bool B_MN = (MODE != kForward);

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      tma_prefetch_desc(&tma_a);
      tma_prefetch_desc(&tma_b);
      int s = 0;
      uint32_t ph = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < total && ok; t += gridDim.x) {
        int a, tn, k_lo, k_hi, e;
        tile_of(t, tiles_n, a, tn);
        k_range(a, k_lo, k_hi, e);
        const int n0 = tn * BN;
        const int m0 = (MODE == kWgrad) ? (a % wg_tiles_m) * BM : a * BM;
        for (int k = k_lo; k < k_hi; ++k) {
          if (!mbar_wait(&empty_bar[s], ph ^ 1, abort_flag, p.err)) { ok = false; break; }
          uint8_t* sa = smem + s * kStageBytes;
          uint8_t* sb = sa + kABytes;
          mbar_expect_tx(&full_bar[s], kStageBytes);
          if constexpr (!A_MN) {
            tma_load_2d(sa, &tma_a, &full_bar[s], k * BK, m0);
          } else {
#pragma unroll
            for (int c = 0; c < BM / 64; ++c) tma_load_2d(sa + c * (BK * 128), &tma_a, &full_bar[s], m0 + c * 64, k * BK);
          }
          if constexpr (MODE == kForward) {
            tma_load_2d(sb, &tma_b, &full_bar[s], k * BK, e * p.N + n0);
          } else if constexpr (MODE == kDgrad) {
#pragma unroll
            for (int c = 0; c < BN / 64; ++c) tma_load_2d(sb + c * (BK * 128), &tma_b, &full_bar[s], n0 + c * 64, e * p.K + k * BK);
          } else {
#pragma unroll
            for (int c = 0; c < BN / 64; ++c) tma_load_2d(sb + c * (BK * 128), &tma_b, &full_bar[s], n0 + c * 64, k * BK);
          }
          if (++s == kStages) { s = 0; ph ^= 1; }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      const uint32_t idesc = make_idesc_f16(BM, BN, true, A_MN, B_MN);
      int s = 0, acc = 0;
      uint32_t ph = 0, acc_ph = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < total && ok; t += gridDim.x) {
        int a, tn, k_lo, k_hi, e;
        tile_of(t, tiles_n, a, tn);
        k_range(a, k_lo, k_hi, e);
        if (k_lo >= k_hi) continue;     // unused tile / expert without tokens: nothing to multiply
        if (!mbar_wait(&tempty_bar[acc], acc_ph ^ 1, abort_flag, p.err)) break;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int k = k_lo; k < k_hi; ++k) {
          if (!mbar_wait(&full_bar[s], ph, abort_flag, p.err)) { ok = false; break; }
          tc_fence_after();
          const uint32_t sa = smem_u32(smem + s * kStageBytes);
          const uint32_t sb = sa + kABytes;
#pragma unroll
          for (int kk = 0; kk < BK / 16; ++kk) {
            const uint64_t da = A_MN ? make_smem_desc(sa + kk * 2048, BK * 128, 1024, kSwizzle128B)
                                     : make_smem_desc(sa + kk * 32, 16, 1024, kSwizzle128B);
            const uint64_t db = B_MN ? make_smem_desc(sb + kk * 2048, BK * 128, 1024, kSwizzle128B)
                                     : make_smem_desc(sb + kk * 32, 16, 1024, kSwizzle128B);
            umma_f16(d_tmem, da, db, idesc, (k > k_lo || kk > 0) ? 1u : 0u);
          }
          umma_commit(&empty_bar[s]);
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
    const int lane_grp = warp & 3;
    int acc = 0;
    uint32_t acc_ph = 0;
    for (int t = blockIdx.x; t < total; t += gridDim.x) {
      int a, tn, k_lo, k_hi, e;
      tile_of(t, tiles_n, a, tn);
      k_range(a, k_lo, k_hi, e);
      const int n0 = tn * BN;
      const bool empty = k_lo >= k_hi;
      // an expert without tokens adds nothing to an accumulated gradient; everywhere else an empty work item (an
      // unused tile of the padded buffer, an expert without tokens) is written as zeros so no row is left undefined
      if (empty && MODE == kWgrad && p.accumulate) continue;
      int out_row, out_rows, out_cols;
      size_t out_base;
      if constexpr (MODE == kWgrad) {
        out_row = (a % wg_tiles_m) * BM + lane_grp * 32 + lane;
        out_rows = p.N;
        out_cols = p.K;
        out_base = static_cast<size_t>(e) * p.N * p.K;
      } else {
        out_row = a * BM + lane_grp * 32 + lane;
        out_rows = p.rows_cap;
        out_cols = p.N;
        out_base = 0;
      }
      if (!empty) {
        if (!mbar_wait(&tfull_bar[acc], acc_ph, abort_flag, p.err)) break;
        tc_fence_after();
      }
      const uint32_t taddr = tmem_base + acc * BN + (static_cast<uint32_t>(lane_grp * 32) << 16);
#pragma unroll 1
      for (int c = 0; c < BN / 32; ++c) {
        uint32_t r[32];
        if (!empty) {
          tmem_ld_32x32b_x32(taddr + c * 32, r);
          tmem_wait_ld();
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) r[i] = 0;
        }
        const int col = n0 + c * 32;
        if (out_row >= out_rows || col >= out_cols) continue;
        const size_t off = out_base + static_cast<size_t>(out_row) * out_cols + col;
        const bool full = (col + 32 <= out_cols);
        if (p.out_fp32) {
          float* out = reinterpret_cast<float*>(p.C) + off;
          if (full && (out_cols % 4 == 0)) {
#pragma unroll
            for (int i = 0; i < 8; ++i) {
              float4 o = make_float4(__uint_as_float(r[4 * i]), __uint_as_float(r[4 * i + 1]), __uint_as_float(r[4 * i + 2]),
                                     __uint_as_float(r[4 * i + 3]));
              if (p.accumulate) {
                const float4 old = reinterpret_cast<float4*>(out)[i];
                o.x += old.x; o.y += old.y; o.z += old.z; o.w += old.w;
              }
              reinterpret_cast<float4*>(out)[i] = o;
            }
          } else {
            for (int i = 0; i < 32 && col + i < out_cols; ++i)
              out[i] = p.accumulate ? out[i] + __uint_as_float(r[i]) : __uint_as_float(r[i]);
          }
        } else {
          __nv_bfloat16* out = reinterpret_cast<__nv_bfloat16*>(p.C) + off;
          if (full && (out_cols % 8 == 0)) {
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              uint4 o;
              o.x = pack_bf16(__uint_as_float(r[8 * i]), __uint_as_float(r[8 * i + 1]));
              o.y = pack_bf16(__uint_as_float(r[8 * i + 2]), __uint_as_float(r[8 * i + 3]));
              o.z = pack_bf16(__uint_as_float(r[8 * i + 4]), __uint_as_float(r[8 * i + 5]));
              o.w = pack_bf16(__uint_as_float(r[8 * i + 6]), __uint_as_float(r[8 * i + 7]));
              reinterpret_cast<uint4*>(out)[i] = o;
            }
          } else {
            for (int i = 0; i < 32 && col + i < out_cols; ++i) out[i] = __float2bfloat16(__uint_as_float(r[i]));
          }
        }
      }
      if (!empty) {
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&tempty_bar[acc]);
        acc ^= 1;
        if (acc == 0) acc_ph ^= 1;
      }
    }
  }

  if (*abort_flag) __nanosleep(50000);
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc<kTmemCols>(tmem_base);
  }
}

template <int MODE>
static int launch(const CUtensorMap& ta, const CUtensorMap& tb, const Params& p, int work_items, cudaStream_t st) {
  static bool attr = false;
  auto kern = grouped_gemm_kernel<MODE>;
  if (!attr) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemTotal);
    if (e != cudaSuccess) return static_cast<int>(e);
    attr = true;
  }
  const int grid = work_items < num_sms() ? work_items : num_sms();
  kern<<<grid, THREADS, kSmemTotal, st>>>(ta, tb, p);
  rb_note_launch(1);
  return static_cast<int>(cudaGetLastError());
}

}  // namespace gg
}  // namespace rb

// X [rows_cap, K] (expert-sorted, 128-row aligned groups), W [E, N, K] -> Y [rows_cap, N] (bf16).
extern "C" int rb_grouped_gemm_fwd(const void* X, const void* W, void* Y, const int* tile_expert, int rows_cap, int N, int K,
                                   int E, int* err, cudaStream_t st) {
  using namespace rb;
  using namespace rb::gg;
  if (rows_cap <= 0 || E <= 0) return 0;
  if (rows_cap % BM || K % 8 || N % 8) return -2;
  CUtensorMap ta, tb;
  int rc = encode_tma_2d_bf16(&ta, X, K, rows_cap, K, BK, BM);
  if (rc) return rc;
  rc = encode_tma_2d_bf16(&tb, W, K, static_cast<uint64_t>(E) * N, K, BK, BN);
  if (rc) return rc;
  Params p{};
  p.rows_cap = rows_cap; p.N = N; p.K = K; p.E = E; p.tile_expert = tile_expert; p.C = Y; p.err = err;
  return launch<kForward>(ta, tb, p, (rows_cap / BM) * ((N + BN - 1) / BN), st);
}

// dY [rows_cap, Nw], W [E, Nw, Kw] -> dX [rows_cap, Kw] (bf16): dX[row] = dY[row] * W[e(row)].
extern "C" int rb_grouped_gemm_dgrad(const void* dY, const void* W, void* dX, const int* tile_expert, int rows_cap, int Nw,
                                     int Kw, int E, int* err, cudaStream_t st) {
  using namespace rb;
  using namespace rb::gg;
  if (rows_cap <= 0 || E <= 0) return 0;
  if (rows_cap % BM || Nw % BK || Kw % 8) return -2;   // the reduction runs over Nw in whole 64-deep steps
  CUtensorMap ta, tb;
  int rc = encode_tma_2d_bf16(&ta, dY, Nw, rows_cap, Nw, BK, BM);
  if (rc) return rc;
  rc = encode_tma_2d_bf16(&tb, W, Kw, static_cast<uint64_t>(E) * Nw, Kw, 64, BK);
  if (rc) return rc;
  Params p{};
  p.rows_cap = rows_cap; p.N = Kw; p.K = Nw; p.E = E; p.tile_expert = tile_expert; p.C = dX; p.err = err;
  return launch<kDgrad>(ta, tb, p, (rows_cap / BM) * ((Kw + BN - 1) / BN), st);
}

// dW[e] (+)= dY_e^T X_e for every local expert; expert_rows [E + 1] are the padded row offsets (multiples of 128).
extern "C" int rb_grouped_gemm_wgrad(const void* dY, const void* X, void* dW, const int* expert_rows, int rows_cap, int Nw,
                                     int Kw, int E, int out_fp32, int accumulate, int* err, cudaStream_t st) {
  using namespace rb;
  using namespace rb::gg;
  if (E <= 0) return 0;
  if (rows_cap % BM || Nw % 8 || Kw % 8) return -2;
  if (accumulate && !out_fp32) return -3;
  CUtensorMap ta, tb;
  int rc = encode_tma_2d_bf16(&ta, dY, Nw, rows_cap, Nw, 64, BK);
  if (rc) return rc;
  rc = encode_tma_2d_bf16(&tb, X, Kw, rows_cap, Kw, 64, BK);
  if (rc) return rc;
  Params p{};
  p.rows_cap = rows_cap; p.N = Nw; p.K = Kw; p.E = E; p.expert_rows = expert_rows; p.C = dW;
  p.out_fp32 = out_fp32; p.accumulate = accumulate; p.err = err;
  return launch<kWgrad>(ta, tb, p, E * ((Nw + BM - 1) / BM) * ((Kw + BN - 1) / BN), st);
}
