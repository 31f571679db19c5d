// Flash attention forward for sm_100a: packed variable-length sequences, causal
// (bottom-right aligned) or full, grouped-query heads, head_dim 128, bf16.
//
// One CTA owns 128 query rows of one head.  Per 64-row KV block:
//   S = Q K^T      tcgen05.mma, fp32 accumulator in TMEM columns [0, 64)
//   softmax        one thread per query row reads its row of S from TMEM (no
//                  shuffles), keeps a running reference max / sum, writes
//                  P = exp2(S - m) as bf16 into shared memory (128-byte swizzle)
//   O += P V       tcgen05.mma, accumulator in TMEM columns [64, 192); V is the
//                  MN-major B operand, read in place from its [kv][d] tile
// The accumulator is rescaled in TMEM only when the row max grows by more than
// 2^8 (lazy rescaling), which is exact because numerator and denominator share
// the reference.  Warps 0-3: softmax/epilogue, warp 4: TMA, warp 5: MMA issue.
// Two CTAs fit per SM (112 KB shared memory, 256 TMEM columns each) and overlap
// each other's softmax and tensor phases.
#include "common.cuh"
#include "host_utils.h"

namespace rb {

constexpr int FA_D = 128;
constexpr int FA_BQ = 128;
constexpr int FA_BKV = 64;
constexpr int FA_THREADS = 192;
constexpr int FA_Q_BYTES = FA_BQ * FA_D * 2;        // 32 KB (two 64-column halves)
constexpr int FA_KV_BYTES = FA_BKV * FA_D * 2;      // 16 KB
constexpr int FA_P_BYTES = FA_BQ * FA_BKV * 2;      // 16 KB
constexpr int FA_SMEM_Q = 0;
constexpr int FA_SMEM_K = FA_SMEM_Q + FA_Q_BYTES;           // 2 stages
constexpr int FA_SMEM_V = FA_SMEM_K + 2 * FA_KV_BYTES;      // 2 stages
constexpr int FA_SMEM_P = FA_SMEM_V + 2 * FA_KV_BYTES;
constexpr int FA_SMEM_BAR = FA_SMEM_P + FA_P_BYTES;
constexpr int FA_SMEM_TOTAL = FA_SMEM_BAR + 128;
constexpr int FA_TMEM_COLS = 256;
constexpr int FA_TMEM_S = 0;
constexpr int FA_TMEM_O = 64;

struct FaFwdParams {
  const int* cu_q;
  const int* cu_k;
  int num_seqs;
  int Hq, Hkv;
  int causal;
  float scale_log2;  // softmax scale * log2(e)
  __nv_bfloat16* O;  // [Tq][Hq][128] contiguous
  float* lse;        // [Hq][Tq]
  int Tq;
  int* err;
};

__global__ void __launch_bounds__(FA_THREADS, 2)
fa_fwd_kernel(const __grid_constant__ CUtensorMap tma_q, const __grid_constant__ CUtensorMap tma_k,
              const __grid_constant__ CUtensorMap tma_v, const FaFwdParams p) {
  extern __shared__ __align__(1024) uint8_t smem[];
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + FA_SMEM_BAR);
  uint64_t* bar_q = bars + 0;
  uint64_t* bar_s = bars + 1;
  uint64_t* bar_p = bars + 2;
  uint64_t* bar_o = bars + 3;
  uint64_t* kfull = bars + 4;    // [2]
  uint64_t* vfull = bars + 6;    // [2]
  uint64_t* kvempty = bars + 8;  // [2]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 10);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  int* tile_info = reinterpret_cast<int*>(tmem_slot + 2);  // seq, q0

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int head = blockIdx.y;
  const int kv_head = head / (p.Hq / p.Hkv);

  // ---- locate my (sequence, query block): blocks are numbered sequence by sequence
  if (threadIdx.x == 0) {
    int rem = blockIdx.x, seq = -1, q0 = 0;
    for (int b = 0; b < p.num_seqs; ++b) {
      const int len = p.cu_q[b + 1] - p.cu_q[b];
      const int nb = (len + FA_BQ - 1) / FA_BQ;
      if (rem < nb) { seq = b; q0 = rem * FA_BQ; break; }
      rem -= nb;
    }
    tile_info[0] = seq;
    tile_info[1] = q0;
    *abort_flag = 0;
    if ((smem_u32(smem) & 1023u) != 0) {  // swizzled tiles need 1 KB alignment
      tile_info[0] = -1;
      if (p.err) atomicCAS(p.err, kOk, kErrBadArgument);
    }
  }
  __syncthreads();
  const int seq = tile_info[0];
  if (seq < 0) return;  // surplus CTA of the over-provisioned grid
  const int q0 = tile_info[1];
  const int q_begin = p.cu_q[seq], q_end = p.cu_q[seq + 1];
  const int k_begin = p.cu_k[seq], k_end = p.cu_k[seq + 1];
  const int len_q = q_end - q_begin, len_k = k_end - k_begin;
  const int offset = len_k - len_q;  // causal: query i sees keys <= i + offset
  int kv_limit = len_k;
  if (p.causal) kv_limit = min(len_k, q0 + FA_BQ + offset);
  if (kv_limit < 0) kv_limit = 0;
  const int n_blocks = (kv_limit + FA_BKV - 1) / FA_BKV;

  if (threadIdx.x == 0) {
    mbar_init(bar_q, 1);
    mbar_init(bar_s, 1);
    mbar_init(bar_p, 128);
    mbar_init(bar_o, 1);
    for (int s = 0; s < 2; ++s) {
      mbar_init(&kfull[s], 1);
      mbar_init(&vfull[s], 1);
      mbar_init(&kvempty[s], 1);
    }
    fence_barrier_init();
  }
  if (warp == 5) {
    tmem_alloc<FA_TMEM_COLS>(tmem_slot);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 4) {
    // ================================================================ TMA producer
    if (lane == 0 && n_blocks > 0) {
      tma_prefetch_desc(&tma_q);
      tma_prefetch_desc(&tma_k);
      tma_prefetch_desc(&tma_v);
      mbar_expect_tx(bar_q, FA_Q_BYTES);
      tma_load_3d(smem + FA_SMEM_Q, &tma_q, bar_q, 0, head, q_begin + q0);
      tma_load_3d(smem + FA_SMEM_Q + FA_Q_BYTES / 2, &tma_q, bar_q, 64, head, q_begin + q0);
      for (int j = 0; j < n_blocks; ++j) {
        const int s = j & 1;
        const uint32_t use = static_cast<uint32_t>(j >> 1);
        if (!mbar_wait(&kvempty[s], (use & 1) ^ 1, abort_flag, p.err)) break;
        const int row = k_begin + j * FA_BKV;
        uint8_t* sk = smem + FA_SMEM_K + s * FA_KV_BYTES;
        uint8_t* sv = smem + FA_SMEM_V + s * FA_KV_BYTES;
        mbar_expect_tx(&kfull[s], FA_KV_BYTES);
        tma_load_3d(sk, &tma_k, &kfull[s], 0, kv_head, row);
        tma_load_3d(sk + FA_KV_BYTES / 2, &tma_k, &kfull[s], 64, kv_head, row);
        mbar_expect_tx(&vfull[s], FA_KV_BYTES);
        tma_load_3d(sv, &tma_v, &vfull[s], 0, kv_head, row);
        tma_load_3d(sv + FA_KV_BYTES / 2, &tma_v, &vfull[s], 64, kv_head, row);
      }
    }
  } else if (warp == 5) {
    // ================================================================ MMA issuer
    if (lane == 0 && n_blocks > 0) {
      const uint32_t idesc_s = make_idesc_f16(FA_BQ, FA_BKV, true, false, false);
      const uint32_t idesc_o = make_idesc_f16(FA_BQ, FA_D, true, false, true);
      const uint32_t sq = smem_u32(smem + FA_SMEM_Q);
      const uint32_t sp = smem_u32(smem + FA_SMEM_P);
      auto issue_s = [&](int j) -> bool {
        const int s = j & 1;
        if (!mbar_wait(&kfull[s], static_cast<uint32_t>(j >> 1) & 1, abort_flag, p.err)) return false;
        tc_fence_after();
        const uint32_t sk = smem_u32(smem + FA_SMEM_K + s * FA_KV_BYTES);
#pragma unroll
        for (int kk = 0; kk < FA_D / 16; ++kk) {
          const uint64_t da = make_smem_desc(sq + (kk >> 2) * (FA_Q_BYTES / 2) + (kk & 3) * 32, 16, 1024, kSwizzle128B);
          const uint64_t db = make_smem_desc(sk + (kk >> 2) * (FA_KV_BYTES / 2) + (kk & 3) * 32, 16, 1024, kSwizzle128B);
          umma_f16(tmem_base + FA_TMEM_S, da, db, idesc_s, kk > 0 ? 1u : 0u);
        }
        umma_commit(bar_s);
        return true;
      };
      bool ok = mbar_wait(bar_q, 0, abort_flag, p.err);
      if (ok) ok = issue_s(0);
      for (int j = 0; j < n_blocks && ok; ++j) {
        const int s = j & 1;
        if (!mbar_wait(bar_p, static_cast<uint32_t>(j) & 1, abort_flag, p.err)) break;  // P_j written, S consumed
        tc_fence_after();
        if (j + 1 < n_blocks) {
          if (!issue_s(j + 1)) break;
        }
        if (!mbar_wait(&vfull[s], static_cast<uint32_t>(j >> 1) & 1, abort_flag, p.err)) break;
        tc_fence_after();
        const uint32_t sv = smem_u32(smem + FA_SMEM_V + s * FA_KV_BYTES);
#pragma unroll
        for (int kk = 0; kk < FA_BKV / 16; ++kk) {
          const uint64_t da = make_smem_desc(sp + kk * 32, 16, 1024, kSwizzle128B);
          // V tile [kv][d]: 64-column chunks are FA_KV_BYTES/2 apart, 16 kv rows = 2048 bytes
          const uint64_t db = make_smem_desc(sv + kk * 2048, FA_KV_BYTES / 2, 1024, kSwizzle128B);
          umma_f16(tmem_base + FA_TMEM_O, da, db, idesc_o, (j > 0 || kk > 0) ? 1u : 0u);
        }
        umma_commit(&kvempty[s]);
        umma_commit(bar_o);
      }
    }
  } else {
    // ================================================================ softmax + epilogue (warps 0..3)
    const int r = warp * 32 + lane;              // row inside the tile == TMEM lane
    const int q_row = q0 + r;                    // row inside the sequence
    const uint32_t lane_addr = static_cast<uint32_t>(warp * 32) << 16;
    float m_ref = -1e30f, l = 0.f;
    bool ok = true;
    uint8_t* sp = smem + FA_SMEM_P + r * 128;
    for (int j = 0; j < n_blocks; ++j) {
      if (!mbar_wait(bar_s, static_cast<uint32_t>(j) & 1, abort_flag, p.err)) { ok = false; break; }
      tc_fence_after();
      uint32_t raw[64];
      tmem_ld_32x32b_x32(tmem_base + FA_TMEM_S + lane_addr, raw);
      tmem_ld_32x32b_x32(tmem_base + FA_TMEM_S + lane_addr + 32, raw + 32);
      tmem_wait_ld();
      const int col0 = j * FA_BKV;
      int limit = len_k - col0;                                   // columns < limit are inside the sequence
      if (p.causal) limit = min(limit, q_row + offset + 1 - col0);  // and not in the future
      float mx = -1e30f;
#pragma unroll
      for (int c = 0; c < 64; ++c) {
        float s = __uint_as_float(raw[c]) * p.scale_log2;
        s = (c < limit) ? s : -1e30f;
        raw[c] = __float_as_uint(s);
        mx = fmaxf(mx, s);
      }
      // the previous P V must have finished before P is overwritten or O is rescaled
      if (j > 0) {
        if (!mbar_wait(bar_o, static_cast<uint32_t>(j - 1) & 1, abort_flag, p.err)) { ok = false; break; }
        tc_fence_after();
      }
      if (mx > m_ref + 8.f) {
        const float alpha = exp2f(m_ref - mx);
        m_ref = mx;
        l *= alpha;
        if (j > 0) {
#pragma unroll 1
          for (int c = 0; c < FA_D / 32; ++c) {
            uint32_t o[32];
            tmem_ld_32x32b_x32(tmem_base + FA_TMEM_O + lane_addr + c * 32, o);
            tmem_wait_ld();
#pragma unroll
            for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
            tmem_st_32x32b_x32(tmem_base + FA_TMEM_O + lane_addr + c * 32, o);
          }
          tmem_wait_st();
        }
      }
      float sum = 0.f;
#pragma unroll
      for (int c8 = 0; c8 < 8; ++c8) {
        float e[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          e[i] = exp2f(__uint_as_float(raw[c8 * 8 + i]) - m_ref);
          sum += e[i];
        }
        uint4 pk;
        pk.x = pack_bf16(e[0], e[1]);
        pk.y = pack_bf16(e[2], e[3]);
        pk.z = pack_bf16(e[4], e[5]);
        pk.w = pack_bf16(e[6], e[7]);
        *reinterpret_cast<uint4*>(sp + ((c8 ^ (r & 7)) << 4)) = pk;
      }
      l += sum;
      fence_proxy_async();
      tc_fence_before();
      mbar_arrive(bar_p);
    }
    if (ok && n_blocks > 0) ok = mbar_wait(bar_o, static_cast<uint32_t>(n_blocks - 1) & 1, abort_flag, p.err);
    tc_fence_after();
    const bool live = ok && (q_row < len_q);
    const float inv_l = (l > 0.f) ? 1.f / l : 0.f;
    __nv_bfloat16* out = p.O + (static_cast<size_t>(q_begin + q_row) * p.Hq + head) * FA_D;
#pragma unroll 1
    for (int c = 0; c < FA_D / 32; ++c) {
      uint32_t o[32];
      if (n_blocks > 0) {
        tmem_ld_32x32b_x32(tmem_base + FA_TMEM_O + lane_addr + c * 32, o);
        tmem_wait_ld();
      } else {
#pragma unroll
        for (int i = 0; i < 32; ++i) o[i] = 0;
      }
      if (live) {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          uint4 pk;
          pk.x = pack_bf16(__uint_as_float(o[8 * i]) * inv_l, __uint_as_float(o[8 * i + 1]) * inv_l);
          pk.y = pack_bf16(__uint_as_float(o[8 * i + 2]) * inv_l, __uint_as_float(o[8 * i + 3]) * inv_l);
          pk.z = pack_bf16(__uint_as_float(o[8 * i + 4]) * inv_l, __uint_as_float(o[8 * i + 5]) * inv_l);
          pk.w = pack_bf16(__uint_as_float(o[8 * i + 6]) * inv_l, __uint_as_float(o[8 * i + 7]) * inv_l);
          reinterpret_cast<uint4*>(out + c * 32)[i] = pk;
        }
      }
    }
    if (live && p.lse)
      p.lse[static_cast<size_t>(head) * p.Tq + q_begin + q_row] =
          (l > 0.f) ? (m_ref + log2f(l)) * 0.6931471805599453f : -INFINITY;
  }

  if (*abort_flag) __nanosleep(50000);
  tc_fence_before();
  __syncthreads();
  if (warp == 5) {
    tc_fence_after();
    tmem_dealloc<FA_TMEM_COLS>(tmem_base);
  }
}

}  // namespace rb

// q [Tq][Hq][128], k/v [Tk][Hkv][128]; *_tok / *_head are strides in elements (multiples of 8).
extern "C" int rb_fa_fwd(const void* q, const void* k, const void* v, void* o, float* lse, const int* cu_q,
                         const int* cu_k, int num_seqs, int Tq, int Tk, int Hq, int Hkv, long long q_tok,
                         long long q_head, long long k_tok, long long k_head, long long v_tok, long long v_head,
                         int causal, float scale, int max_q_blocks, int* err, cudaStream_t stream) {
  using namespace rb;
  if (Tq == 0 || num_seqs == 0) return 0;
  if (Hq % Hkv) return -2;
  CUtensorMap tq, tk, tv;
  int rc = encode_tma_3d_16bit(&tq, q, FA_D, Hq, Tq, q_head, q_tok, 64, 1, FA_BQ);
  if (rc) return rc;
  rc = encode_tma_3d_16bit(&tk, k, FA_D, Hkv, Tk, k_head, k_tok, 64, 1, FA_BKV);
  if (rc) return rc;
  rc = encode_tma_3d_16bit(&tv, v, FA_D, Hkv, Tk, v_head, v_tok, 64, 1, FA_BKV);
  if (rc) return rc;
  static bool attr_set = false;
  if (!attr_set) {
    cudaError_t e = cudaFuncSetAttribute(fa_fwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, FA_SMEM_TOTAL);
    if (e != cudaSuccess) return static_cast<int>(e);
    attr_set = true;
  }
  FaFwdParams p{};
  p.cu_q = cu_q; p.cu_k = cu_k; p.num_seqs = num_seqs; p.Hq = Hq; p.Hkv = Hkv; p.causal = causal;
  p.scale_log2 = scale * 1.4426950408889634f;
  p.O = reinterpret_cast<__nv_bfloat16*>(o); p.lse = lse; p.Tq = Tq; p.err = err;
  dim3 grid(max_q_blocks, Hq);
  fa_fwd_kernel<<<grid, FA_THREADS, FA_SMEM_TOTAL, stream>>>(tq, tk, tv, p);
  rb_note_launch(1);
  return static_cast<int>(cudaGetLastError());
}
