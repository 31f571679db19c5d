// Flash attention backward for sm_100a (packed varlen, causal/full, GQA, head_dim 128, bf16).
//
// One CTA owns 128 KV rows of one KV head and walks over every (query head of the
// group, 64-row query block) pair that can see them.  Everything is computed in the
// transposed frame so that each tensor-core tile has M = 128:
//   S^T  = K Q^T            [kv 128][q 64]      (A = K tile, B = Q tile, both K-major)
//   dP^T = V dO^T           [kv 128][q 64]
//   P^T  = exp2(S^T c - lse[q]) ;  dS^T = P^T (dP^T - delta[q]) * scale      (one thread per kv row)
//   dV  += P^T  dO          [kv 128][d 128]     (B = dO tile read MN-major in place)
//   dK  += dS^T Q           [kv 128][d 128]
//   dQ^T = K^T dS^T         [d 128][q 64]       (A = K tile MN-major, B = dS^T tile MN-major)
// dV/dK accumulate in TMEM over the whole walk and are written once (no atomics:
// the CTA visits every query head of its KV head).  dQ^T tiles are added to an
// fp32 accumulation buffer with coalesced red.global (lane = d), converted to
// bf16 by a second small kernel.  The softmax / dS work is split by query columns over two
// warpgroups (columns 0-31 and 32-63 of every tile); the producer warp stages the 64 lse and delta
// values of a query block in shared memory (pre-scaled, +inf / 0 beyond the sequence end) so the
// inner loop has no global loads.  TMEM (512 columns): S^T x2, dP^T x2, dV, dK;
// dQ^T of step i reuses the S^T buffer of step i.
#include "common.cuh"
#include "host_utils.h"

namespace rb {

constexpr int FB_D = 128;
constexpr int FB_BKV = 128;
constexpr int FB_BQ = 64;
constexpr int FB_THREADS = 320;  // 2 softmax warpgroups (warps 0-7), TMA producer (8), MMA issuer (9)
constexpr int FB_KV_BYTES = FB_BKV * FB_D * 2;  // 32 KB
constexpr int FB_Q_BYTES = FB_BQ * FB_D * 2;    // 16 KB
constexpr int FB_PT_BYTES = FB_BKV * FB_BQ * 2; // 16 KB
constexpr int FB_SMEM_K = 0;
constexpr int FB_SMEM_V = FB_SMEM_K + FB_KV_BYTES;
constexpr int FB_SMEM_Q = FB_SMEM_V + FB_KV_BYTES;          // 2 stages
constexpr int FB_SMEM_DO = FB_SMEM_Q + 2 * FB_Q_BYTES;      // 2 stages
constexpr int FB_SMEM_PT = FB_SMEM_DO + 2 * FB_Q_BYTES;
constexpr int FB_SMEM_DS = FB_SMEM_PT + FB_PT_BYTES;
constexpr int FB_SMEM_BAR = FB_SMEM_DS + FB_PT_BYTES;
constexpr int FB_SMEM_LD = FB_SMEM_BAR + 256;      // 2 stages x (64 lse*log2e + 64 delta) floats
constexpr int FB_SMEM_TOTAL = FB_SMEM_LD + 2 * 128 * 4;
constexpr int FB_T_ST = 0;     // two buffers of 64 columns
constexpr int FB_T_DP = 128;   // two buffers of 64 columns
constexpr int FB_T_DV = 256;
constexpr int FB_T_DK = 384;

struct FaBwdParams {
  const int* cu_q;
  const int* cu_k;
  int num_seqs, Hq, Hkv, causal;
  float scale, scale_log2;
  const float* lse;    // [Hq][Tq] natural log
  const float* delta;  // [Hq][Tq] rowsum(O * dO)
  float* dq_acc;       // [Tq][Hq][128] fp32, zero-initialised
  __nv_bfloat16* dK;   // [Tk][Hkv][128]
  __nv_bfloat16* dV;
  int Tq;
  int* err;
};

__global__ void __launch_bounds__(FB_THREADS, 1)
fa_bwd_kernel(const __grid_constant__ CUtensorMap tma_q, const __grid_constant__ CUtensorMap tma_do,
              const __grid_constant__ CUtensorMap tma_k, const __grid_constant__ CUtensorMap tma_v,
              const FaBwdParams p) {
  extern __shared__ __align__(1024) uint8_t smem[];
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + FB_SMEM_BAR);
  uint64_t* kvfull = bars + 0;
  uint64_t* qfull = bars + 1;     // [2]
  uint64_t* qempty = bars + 3;    // [2]
  uint64_t* bar_sdp = bars + 5;   // [2]
  uint64_t* bar_pds = bars + 7;
  uint64_t* bar_mma2 = bars + 8;
  uint64_t* bar_dqfree = bars + 9;  // [2]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 11);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  int* tile_info = reinterpret_cast<int*>(tmem_slot + 2);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int kv_head = blockIdx.y;
  const int G = p.Hq / p.Hkv;

  if (threadIdx.x == 0) {
    int rem = blockIdx.x, seq = -1, kv0 = 0;
    for (int b = 0; b < p.num_seqs; ++b) {
      const int len = p.cu_k[b + 1] - p.cu_k[b];
      const int nb = (len + FB_BKV - 1) / FB_BKV;
      if (rem < nb) { seq = b; kv0 = rem * FB_BKV; break; }
      rem -= nb;
    }
    tile_info[0] = seq;
    tile_info[1] = kv0;
    *abort_flag = 0;
    if ((smem_u32(smem) & 1023u) != 0) {
      tile_info[0] = -1;
      if (p.err) atomicCAS(p.err, kOk, kErrBadArgument);
    }
  }
  __syncthreads();
  const int seq = tile_info[0];
  if (seq < 0) return;
  const int kv0 = tile_info[1];
  const int q_begin = p.cu_q[seq], len_q = p.cu_q[seq + 1] - q_begin;
  const int k_begin = p.cu_k[seq], len_k = p.cu_k[seq + 1] - k_begin;
  const int offset = len_k - len_q;
  // first query row that can see kv0 (causal: q + offset >= kv)
  int q_lo = 0;
  if (p.causal) q_lo = max(0, kv0 - offset);
  const int i_start = q_lo / FB_BQ;
  const int i_end = (len_q + FB_BQ - 1) / FB_BQ;  // exclusive
  const int n_i = max(0, i_end - i_start);
  const int n_it = n_i * G;

  if (threadIdx.x == 0) {
    mbar_init(kvfull, 1);
    for (int s = 0; s < 2; ++s) {
      mbar_init(&qfull[s], 1);
      mbar_init(&qempty[s], 1);
      mbar_init(&bar_sdp[s], 1);
      mbar_init(&bar_dqfree[s], 256);
    }
    mbar_init(bar_pds, 256);
    mbar_init(bar_mma2, 1);
    fence_barrier_init();
  }
  if (warp == 9) {
    tmem_alloc<512>(tmem_slot);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 8) {
    // ================================================================ TMA producer + lse/delta staging (whole warp)
    if (n_it > 0) {
      if (lane == 0) {
        mbar_expect_tx(kvfull, 2 * FB_KV_BYTES);
        tma_load_3d(smem + FB_SMEM_K, &tma_k, kvfull, 0, kv_head, k_begin + kv0);
        tma_load_3d(smem + FB_SMEM_K + FB_KV_BYTES / 2, &tma_k, kvfull, 64, kv_head, k_begin + kv0);
        tma_load_3d(smem + FB_SMEM_V, &tma_v, kvfull, 0, kv_head, k_begin + kv0);
        tma_load_3d(smem + FB_SMEM_V + FB_KV_BYTES / 2, &tma_v, kvfull, 64, kv_head, k_begin + kv0);
      }
      const float log2e = 1.4426950408889634f;
      for (int it = 0; it < n_it; ++it) {
        const int s = it & 1;
        int okw = 1;
        if (lane == 0) okw = mbar_wait(&qempty[s], (static_cast<uint32_t>(it >> 1) & 1) ^ 1, abort_flag, p.err) ? 1 : 0;
        okw = __shfl_sync(0xffffffffu, okw, 0);
        if (!okw) break;
        const int head = kv_head * G + it / n_i;
        const int q0 = (i_start + it % n_i) * FB_BQ;
        const int row = q_begin + q0;
        float* ld = reinterpret_cast<float*>(smem + FB_SMEM_LD) + s * 128;
        const size_t hb = static_cast<size_t>(head) * p.Tq + row;
#pragma unroll
        for (int j = 0; j < 2; ++j) {
          const int qi = lane + 32 * j;
          const bool in = q0 + qi < len_q;
          ld[qi] = in ? __ldg(p.lse + hb + qi) * log2e : INFINITY;
          ld[64 + qi] = in ? __ldg(p.delta + hb + qi) : 0.f;
        }
        __syncwarp();
        if (lane == 0) {
          uint8_t* sq = smem + FB_SMEM_Q + s * FB_Q_BYTES;
          uint8_t* sd = smem + FB_SMEM_DO + s * FB_Q_BYTES;
          mbar_expect_tx(&qfull[s], 2 * FB_Q_BYTES);
          tma_load_3d(sq, &tma_q, &qfull[s], 0, head, row);
          tma_load_3d(sq + FB_Q_BYTES / 2, &tma_q, &qfull[s], 64, head, row);
          tma_load_3d(sd, &tma_do, &qfull[s], 0, head, row);
          tma_load_3d(sd + FB_Q_BYTES / 2, &tma_do, &qfull[s], 64, head, row);
        }
      }
    }
  } else if (warp == 9) {
    // ================================================================ MMA issuer
    if (lane == 0 && n_it > 0) {
      const uint32_t id_sdp = make_idesc_f16(128, FB_BQ, true, false, false);  // K-major x K-major
      const uint32_t id_dvk = make_idesc_f16(128, FB_D, true, false, true);    // P^T K-major, dO/Q MN-major
      const uint32_t id_dq = make_idesc_f16(128, FB_BQ, true, true, true);     // K^T MN-major, dS^T MN-major
      const uint32_t sk = smem_u32(smem + FB_SMEM_K), sv = smem_u32(smem + FB_SMEM_V);
      const uint32_t spt = smem_u32(smem + FB_SMEM_PT), sds = smem_u32(smem + FB_SMEM_DS);
      auto issue_sdp = [&](int it) -> bool {
        const int s = it & 1;
        if (!mbar_wait(&qfull[s], static_cast<uint32_t>(it >> 1) & 1, abort_flag, p.err)) return false;
        tc_fence_after();
        const uint32_t sq = smem_u32(smem + FB_SMEM_Q + s * FB_Q_BYTES);
        const uint32_t sd = smem_u32(smem + FB_SMEM_DO + s * FB_Q_BYTES);
#pragma unroll
        for (int kk = 0; kk < FB_D / 16; ++kk) {
          const uint64_t da = make_smem_desc(sk + (kk >> 2) * (FB_KV_BYTES / 2) + (kk & 3) * 32, 16, 1024, kSwizzle128B);
          const uint64_t db = make_smem_desc(sq + (kk >> 2) * (FB_Q_BYTES / 2) + (kk & 3) * 32, 16, 1024, kSwizzle128B);
          umma_f16(tmem_base + FB_T_ST + s * 64, da, db, id_sdp, kk > 0 ? 1u : 0u);
        }
#pragma unroll
        for (int kk = 0; kk < FB_D / 16; ++kk) {
          const uint64_t da = make_smem_desc(sv + (kk >> 2) * (FB_KV_BYTES / 2) + (kk & 3) * 32, 16, 1024, kSwizzle128B);
          const uint64_t db = make_smem_desc(sd + (kk >> 2) * (FB_Q_BYTES / 2) + (kk & 3) * 32, 16, 1024, kSwizzle128B);
          umma_f16(tmem_base + FB_T_DP + s * 64, da, db, id_sdp, kk > 0 ? 1u : 0u);
        }
        umma_commit(&bar_sdp[s]);
        return true;
      };
      bool ok = mbar_wait(kvfull, 0, abort_flag, p.err);
      if (ok) ok = issue_sdp(0);
      for (int it = 0; it < n_it && ok; ++it) {
        const int s = it & 1;
        if (it + 1 < n_it) {
          if (it >= 1) {  // dQ^T of step it-1 sits in the S^T buffer that step it+1 will overwrite
            if (!mbar_wait(&bar_dqfree[s ^ 1], static_cast<uint32_t>((it - 1) >> 1) & 1, abort_flag, p.err)) break;
            tc_fence_after();
          }
          if (!issue_sdp(it + 1)) break;
        }
        if (!mbar_wait(bar_pds, static_cast<uint32_t>(it) & 1, abort_flag, p.err)) break;
        tc_fence_after();
        const uint32_t sq = smem_u32(smem + FB_SMEM_Q + s * FB_Q_BYTES);
        const uint32_t sd = smem_u32(smem + FB_SMEM_DO + s * FB_Q_BYTES);
#pragma unroll
        for (int kk = 0; kk < FB_BQ / 16; ++kk) {  // dV += P^T dO   (reduction over the 64 query rows)
          const uint64_t da = make_smem_desc(spt + kk * 32, 16, 1024, kSwizzle128B);
          const uint64_t db = make_smem_desc(sd + kk * 2048, FB_Q_BYTES / 2, 1024, kSwizzle128B);
          umma_f16(tmem_base + FB_T_DV, da, db, id_dvk, (it > 0 || kk > 0) ? 1u : 0u);
        }
#pragma unroll
        for (int kk = 0; kk < FB_BQ / 16; ++kk) {  // dK += dS^T Q
          const uint64_t da = make_smem_desc(sds + kk * 32, 16, 1024, kSwizzle128B);
          const uint64_t db = make_smem_desc(sq + kk * 2048, FB_Q_BYTES / 2, 1024, kSwizzle128B);
          umma_f16(tmem_base + FB_T_DK, da, db, id_dvk, (it > 0 || kk > 0) ? 1u : 0u);
        }
#pragma unroll
        for (int kk = 0; kk < FB_BKV / 16; ++kk) {  // dQ^T = K^T dS^T   (reduction over the 128 kv rows)
          const uint64_t da = make_smem_desc(sk + kk * 2048, FB_KV_BYTES / 2, 1024, kSwizzle128B);
          const uint64_t db = make_smem_desc(sds + kk * 2048, FB_PT_BYTES, 1024, kSwizzle128B);
          umma_f16(tmem_base + FB_T_ST + s * 64, da, db, id_dq, kk > 0 ? 1u : 0u);
        }
        umma_commit(&qempty[s]);
        umma_commit(bar_mma2);
      }
    }
  } else {
    // ================================================================ softmax / dS / epilogue (warps 0..7)
    const int wg = warp >> 2;                  // warpgroup: query columns [32*wg, 32*wg+32) of every tile
    const int r = (warp & 3) * 32 + lane;      // kv row of the tile (S^T, dP^T, dV, dK) or d index (dQ^T)
    const int cb = wg * 32;
    const int kv_row = kv0 + r;
    const uint32_t lane_addr = static_cast<uint32_t>((warp & 3) * 32) << 16;
    uint8_t* spt = smem + FB_SMEM_PT + r * 128;
    uint8_t* sds = smem + FB_SMEM_DS + r * 128;
    bool ok = true;

    auto drain_dq = [&](int it) {
      // dQ^T of step `it`: lane = d, this warpgroup's 32 columns = query rows
      const int s = it & 1;
      const int head = kv_head * G + it / n_i;
      const int q0 = (i_start + it % n_i) * FB_BQ + cb;
      tc_fence_after();
      float* base = p.dq_acc + (static_cast<size_t>(q_begin + q0) * p.Hq + head) * FB_D + r;
      const size_t qstride = static_cast<size_t>(p.Hq) * FB_D;
      uint32_t v[32];
      tmem_ld_32x32b_x32(tmem_base + FB_T_ST + s * 64 + lane_addr + cb, v);
      tmem_wait_ld();
      if (q0 + 32 <= len_q) {
#pragma unroll
        for (int i = 0; i < 32; ++i) atomicAdd(base + i * qstride, __uint_as_float(v[i]));
      } else {
#pragma unroll
        for (int i = 0; i < 32; ++i)
          if (q0 + i < len_q) atomicAdd(base + i * qstride, __uint_as_float(v[i]));
      }
      tc_fence_before();
      mbar_arrive(&bar_dqfree[s]);
    };

    for (int it = 0; it < n_it; ++it) {
      const int s = it & 1;
      const int q0 = (i_start + it % n_i) * FB_BQ;
      if (!mbar_wait(&bar_sdp[s], static_cast<uint32_t>(it >> 1) & 1, abort_flag, p.err)) { ok = false; break; }
      // the staged lse/delta were written before this stage's barrier was armed; it has completed long ago
      if (!mbar_wait(&qfull[s], static_cast<uint32_t>(it >> 1) & 1, abort_flag, p.err)) { ok = false; break; }
      tc_fence_after();
      const float4* l4 = reinterpret_cast<const float4*>(smem + FB_SMEM_LD) + s * 32 + wg * 8;
      const float4* d4 = l4 + 16;
      uint32_t pk_p[16], pk_ds[16];
      uint32_t sv[32], dv[32];
      tmem_ld_32x32b_x32(tmem_base + FB_T_ST + s * 64 + lane_addr + cb, sv);
      tmem_ld_32x32b_x32(tmem_base + FB_T_DP + s * 64 + lane_addr + cb, dv);
      tmem_wait_ld();
      const bool full = (kv0 + FB_BKV - 1 < len_k) && (!p.causal || (kv0 + FB_BKV - 1 <= q0 + offset));
      if (full) {
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const float4 l = l4[i], d = d4[i];
          const float p0 = exp2f(fmaf(__uint_as_float(sv[4 * i]), p.scale_log2, -l.x));
          const float p1 = exp2f(fmaf(__uint_as_float(sv[4 * i + 1]), p.scale_log2, -l.y));
          const float p2 = exp2f(fmaf(__uint_as_float(sv[4 * i + 2]), p.scale_log2, -l.z));
          const float p3 = exp2f(fmaf(__uint_as_float(sv[4 * i + 3]), p.scale_log2, -l.w));
          pk_p[2 * i] = pack_bf16(p0, p1);
          pk_p[2 * i + 1] = pack_bf16(p2, p3);
          pk_ds[2 * i] = pack_bf16(p0 * (__uint_as_float(dv[4 * i]) - d.x) * p.scale,
                                   p1 * (__uint_as_float(dv[4 * i + 1]) - d.y) * p.scale);
          pk_ds[2 * i + 1] = pack_bf16(p2 * (__uint_as_float(dv[4 * i + 2]) - d.z) * p.scale,
                                       p3 * (__uint_as_float(dv[4 * i + 3]) - d.w) * p.scale);
        }
      } else {
        const float* lf = reinterpret_cast<const float*>(l4);
        const float* df = reinterpret_cast<const float*>(d4);
        const int qlim = p.causal ? kv_row - offset : -(1 << 30);  // valid iff q >= qlim (and the kv row exists)
        const bool row_ok = kv_row < len_k;
#pragma unroll
        for (int i = 0; i < 32; i += 2) {
          float pv[2], ds[2];
#pragma unroll
          for (int u = 0; u < 2; ++u) {
            const bool valid = row_ok && (q0 + cb + i + u >= qlim);
            const float pr = valid ? exp2f(fmaf(__uint_as_float(sv[i + u]), p.scale_log2, -lf[i + u])) : 0.f;
            pv[u] = pr;
            ds[u] = pr * (__uint_as_float(dv[i + u]) - df[i + u]) * p.scale;
          }
          pk_p[i / 2] = pack_bf16(pv[0], pv[1]);
          pk_ds[i / 2] = pack_bf16(ds[0], ds[1]);
        }
      }
      tc_fence_before();
      if (it > 0) {  // P^T / dS^T buffers are read by the tensor core until step it-1 has completed
        if (!mbar_wait(bar_mma2, static_cast<uint32_t>(it - 1) & 1, abort_flag, p.err)) { ok = false; break; }
      }
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int off = ((wg * 4 + j) ^ (r & 7)) << 4;
        *reinterpret_cast<uint4*>(spt + off) = make_uint4(pk_p[j * 4], pk_p[j * 4 + 1], pk_p[j * 4 + 2], pk_p[j * 4 + 3]);
        *reinterpret_cast<uint4*>(sds + off) = make_uint4(pk_ds[j * 4], pk_ds[j * 4 + 1], pk_ds[j * 4 + 2], pk_ds[j * 4 + 3]);
      }
      fence_proxy_async();
      mbar_arrive(bar_pds);
      if (it > 0) drain_dq(it - 1);
    }
    if (ok && n_it > 0) {
      ok = mbar_wait(bar_mma2, static_cast<uint32_t>(n_it - 1) & 1, abort_flag, p.err);
      if (ok) drain_dq(n_it - 1);
    }
    tc_fence_after();
    // ---- dK / dV: row r of the tile, this warpgroup's half of the head dimension
    const bool live = ok && (kv_row < len_k);
    __nv_bfloat16* outk = p.dK + (static_cast<size_t>(k_begin + kv_row) * p.Hkv + kv_head) * FB_D;
    __nv_bfloat16* outv = p.dV + (static_cast<size_t>(k_begin + kv_row) * p.Hkv + kv_head) * FB_D;
#pragma unroll 1
    for (int which = 0; which < 2; ++which) {
      __nv_bfloat16* out = which ? outk : outv;
      const uint32_t tcol = which ? FB_T_DK : FB_T_DV;
#pragma unroll 1
      for (int c = 2 * wg; c < 2 * wg + 2; ++c) {
        uint32_t o[32];
        if (n_it > 0) {
          tmem_ld_32x32b_x32(tmem_base + tcol + lane_addr + c * 32, o);
          tmem_wait_ld();
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) o[i] = 0;
        }
        if (live) {
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            uint4 pk;
            pk.x = pack_bf16(__uint_as_float(o[8 * i]), __uint_as_float(o[8 * i + 1]));
            pk.y = pack_bf16(__uint_as_float(o[8 * i + 2]), __uint_as_float(o[8 * i + 3]));
            pk.z = pack_bf16(__uint_as_float(o[8 * i + 4]), __uint_as_float(o[8 * i + 5]));
            pk.w = pack_bf16(__uint_as_float(o[8 * i + 6]), __uint_as_float(o[8 * i + 7]));
            reinterpret_cast<uint4*>(out + c * 32)[i] = pk;
          }
        }
      }
    }
  }

  if (*abort_flag) __nanosleep(50000);
  tc_fence_before();
  __syncthreads();
  if (warp == 9) {
    tc_fence_after();
    tmem_dealloc<512>(tmem_base);
  }
}

// delta[h][t] = sum_d O[t][h][d] * dO[t][h][d]; one warp per (t, h)
__global__ void fa_delta_kernel(const __nv_bfloat16* __restrict__ O, const __nv_bfloat16* __restrict__ dO,
                                float* __restrict__ delta, int T, int H) {
  const int warps = (blockDim.x >> 5);
  const int lane = threadIdx.x & 31;
  for (long long w = blockIdx.x * (long long)warps + (threadIdx.x >> 5); w < (long long)T * H; w += (long long)gridDim.x * warps) {
    const uint2 a = reinterpret_cast<const uint2*>(O + w * FB_D)[lane];
    const uint2 b = reinterpret_cast<const uint2*>(dO + w * FB_D)[lane];
    const __nv_bfloat162 a0 = *reinterpret_cast<const __nv_bfloat162*>(&a.x), a1 = *reinterpret_cast<const __nv_bfloat162*>(&a.y);
    const __nv_bfloat162 b0 = *reinterpret_cast<const __nv_bfloat162*>(&b.x), b1 = *reinterpret_cast<const __nv_bfloat162*>(&b.y);
    float s = __low2float(a0) * __low2float(b0) + __high2float(a0) * __high2float(b0) +
              __low2float(a1) * __low2float(b1) + __high2float(a1) * __high2float(b1);
    s = warp_sum(s);
    if (lane == 0) {
      const int t = static_cast<int>(w / H), h = static_cast<int>(w % H);
      delta[static_cast<size_t>(h) * T + t] = s;
    }
  }
}

__global__ void fa_dq_convert_kernel(const float* __restrict__ acc, __nv_bfloat16* __restrict__ dq, long long n) {
  for (long long i = (blockIdx.x * (long long)blockDim.x + threadIdx.x) * 4; i < n; i += (long long)gridDim.x * blockDim.x * 4) {
    const float4 v = *reinterpret_cast<const float4*>(acc + i);
    uint2 o;
    o.x = pack_bf16(v.x, v.y);
    o.y = pack_bf16(v.z, v.w);
    *reinterpret_cast<uint2*>(dq + i) = o;
  }
}

}  // namespace rb

extern "C" int rb_fa_bwd_ex(const void* q, const void* k, const void* v, const void* o, const void* d_o, const float* lse,
                            void* dq, void* dk, void* dv, float* delta, float* dq_acc, const int* cu_q, const int* cu_k,
                            int num_seqs, int Tq, int Tk, int Hq, int Hkv, int causal, float scale, int max_kv_blocks,
                            int flags, int* err, cudaStream_t stream);

// Scratch: delta fp32 [Hq*Tq], dq_acc fp32 [Tq*Hq*128] (zeroed here).  q/k/v/o/do contiguous [T][H][128].
extern "C" int rb_fa_bwd(const void* q, const void* k, const void* v, const void* o, const void* d_o, const float* lse,
                         void* dq, void* dk, void* dv, float* delta, float* dq_acc, const int* cu_q, const int* cu_k,
                         int num_seqs, int Tq, int Tk, int Hq, int Hkv, int causal, float scale, int max_kv_blocks,
                         int* err, cudaStream_t stream) {
  return rb_fa_bwd_ex(q, k, v, o, d_o, lse, dq, dk, dv, delta, dq_acc, cu_q, cu_k, num_seqs, Tq, Tk, Hq, Hkv, causal, scale,
                      max_kv_blocks, 0, err, stream);
}

// flags: 1 = `delta` is given (do not recompute it from o and d_o); 2 = do not zero `dq_acc` first (the caller
// accumulates several calls into it, possibly into another GPU's buffer through a peer mapping: the dQ
// reductions are plain fp32 atomics and work across NVLink); 4 = do not convert `dq_acc` to `dq` at the end.
// q / d_o / lse / delta may alias peer memory (read by TMA without multicast and by read-only loads).
extern "C" int rb_fa_bwd_ex(const void* q, const void* k, const void* v, const void* o, const void* d_o, const float* lse,
                            void* dq, void* dk, void* dv, float* delta, float* dq_acc, const int* cu_q, const int* cu_k,
                            int num_seqs, int Tq, int Tk, int Hq, int Hkv, int causal, float scale, int max_kv_blocks,
                            int flags, int* err, cudaStream_t stream) {
  using namespace rb;
  if (Tq == 0 || Tk == 0 || num_seqs == 0) return 0;
  if (Hq % Hkv) return -2;
  CUtensorMap tq, tdo, tk, tv;
  int rc = encode_tma_3d_16bit(&tq, q, FB_D, Hq, Tq, FB_D, (uint64_t)Hq * FB_D, 64, 1, FB_BQ);
  if (rc) return rc;
  rc = encode_tma_3d_16bit(&tdo, d_o, FB_D, Hq, Tq, FB_D, (uint64_t)Hq * FB_D, 64, 1, FB_BQ);
  if (rc) return rc;
  rc = encode_tma_3d_16bit(&tk, k, FB_D, Hkv, Tk, FB_D, (uint64_t)Hkv * FB_D, 64, 1, FB_BKV);
  if (rc) return rc;
  rc = encode_tma_3d_16bit(&tv, v, FB_D, Hkv, Tk, FB_D, (uint64_t)Hkv * FB_D, 64, 1, FB_BKV);
  if (rc) return rc;
  static bool attr_set = false;
  if (!attr_set) {
    cudaError_t e = cudaFuncSetAttribute(fa_bwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, FB_SMEM_TOTAL);
    if (e != cudaSuccess) return static_cast<int>(e);
    attr_set = true;
  }
  const long long n_dq = (long long)Tq * Hq * FB_D;
  if (!(flags & 2)) cudaMemsetAsync(dq_acc, 0, n_dq * sizeof(float), stream);
  if (!(flags & 1)) {
    const long long rows = (long long)Tq * Hq;
    long long blocks = (rows + 7) / 8;
    if (blocks > num_sms() * 8LL) blocks = num_sms() * 8LL;
    fa_delta_kernel<<<(int)blocks, 256, 0, stream>>>((const __nv_bfloat16*)o, (const __nv_bfloat16*)d_o, delta, Tq, Hq);
  }
  FaBwdParams p{};
  p.cu_q = cu_q; p.cu_k = cu_k; p.num_seqs = num_seqs; p.Hq = Hq; p.Hkv = Hkv; p.causal = causal;
  p.scale = scale; p.scale_log2 = scale * 1.4426950408889634f;
  p.lse = lse; p.delta = delta; p.dq_acc = dq_acc;
  p.dK = (__nv_bfloat16*)dk; p.dV = (__nv_bfloat16*)dv; p.Tq = Tq; p.err = err;
  dim3 grid(max_kv_blocks, Hkv);
  fa_bwd_kernel<<<grid, FB_THREADS, FB_SMEM_TOTAL, stream>>>(tq, tdo, tk, tv, p);
  rb_note_launch(3);
  if (!(flags & 4)) {
    long long blocks = (n_dq / 4 + 255) / 256;
    if (blocks > num_sms() * 8LL) blocks = num_sms() * 8LL;
    fa_dq_convert_kernel<<<(int)blocks, 256, 0, stream>>>(dq_acc, (__nv_bfloat16*)dq, n_dq);
  }
  return static_cast<int>(cudaGetLastError());
}

extern "C" int rb_fa_dq_convert(const float* dq_acc, void* dq, long long n, cudaStream_t stream) {
  using namespace rb;
  if (n == 0) return 0;
  if (n % 4) return -2;
  long long blocks = (n / 4 + 255) / 256;
  if (blocks > num_sms() * 8LL) blocks = num_sms() * 8LL;
  fa_dq_convert_kernel<<<(int)blocks, 256, 0, stream>>>(dq_acc, (__nv_bfloat16*)dq, n);
  rb_note_launch(1);
  return static_cast<int>(cudaGetLastError());
}
