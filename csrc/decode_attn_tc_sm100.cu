// Paged-KV decode attention on the 5th-generation tensor cores.
//
// One query token per sequence, G = Hq/Hkv query heads share a KV head.  Decode attention is
// bound by reading the KV cache, but on CUDA cores the 2*128*G multiply-adds per cached token
// make it instruction bound well below the HBM rate.  Here the token axis is the M dimension
// of the MMA so every cached token costs a handful of instructions:
//
//   S^T[128 tokens][16]  = K_tile[128][128] * Q^T          (Q padded from G to 16 rows)
//   O^T[128 d][16]      += V_tile^T[128 d][128 tok] * P     (V tile read MN-major in place)
//
// K/V tiles are gathered page by page with TMA (one 16-token box per page and 64-column
// half) into the same swizzled layout a contiguous tile would have.  One thread owns one
// token row of S^T (and one d row of O^T); the per-head running max is shared by the CTA
// (lazy rescaling, threshold 2^8), per-thread partial sums are reduced once at the end.
// CTA = (sequence, kv head, split); partial (m, l, o) go to scratch when splits > 1.
#include "common.cuh"
#include "host_utils.h"

namespace rb {

constexpr int DT_D = 128;
constexpr int DT_TILE = 128;   // tokens per tile
constexpr int DT_PAGE = 16;    // tokens per KV page (block_size)
constexpr int DT_NPAD = 16;    // query heads padded to the MMA N
constexpr int DT_THREADS = 192;
constexpr int DT_KV_BYTES = DT_TILE * DT_D * 2;              // 32 KB: one K tile or one V tile
// K and V tiles share ONE ring of 32 KB buffers (tile j: K in buffer 2j, V in buffer 2j + 1, modulo the ring).  A K
// buffer is free again as soon as the S product has read it, so three buffers keep the loads of a CTA streaming,
// and the CTA is small enough (about 109 KB) for TWO to share an SM: while one CTA is in its prologue or epilogue
// (barrier set-up, TMEM allocation, first-load latency, output stores) the other keeps the memory pipe busy.
constexpr int DT_NBUF = 3;
constexpr int DT_SMEM_KV = 0;
constexpr int DT_SMEM_Q = DT_SMEM_KV + DT_NBUF * DT_KV_BYTES;   // [2 halves][16 rows][128 B]
constexpr int DT_SMEM_P = DT_SMEM_Q + 4096;                  // 2 buffers x [2 halves][16 rows][128 B]
constexpr int DT_SMEM_BAR = DT_SMEM_P + 2 * 4096;
constexpr int DT_SMEM_RED = DT_SMEM_BAR + 256;               // float [4 warps][16] max + [4][16] sums
constexpr int DT_SMEM_TOTAL = DT_SMEM_RED + 1024;
constexpr int DT_TMEM_COLS = 64;
constexpr int DT_T_S = 0;    // two buffers of 16 columns
constexpr int DT_T_O = 32;

struct DecodeTcParams {
  const __nv_bfloat16* q;   // [B][Hq][128]
  const int* block_tables;  // [B][max_blocks]
  const int* ctx_lens;      // [B]
  __nv_bfloat16* out;       // [B][Hq][128]
  float* part_o;            // [B*Hq*splits][128]
  float* part_ml;           // [B*Hq*splits][2]
  int Hq, Hkv, G, max_blocks, num_splits, split_tokens;
  float scale_log2;
  int* err;
};

__global__ void __launch_bounds__(DT_THREADS, 2)
decode_attn_tc_kernel(const __grid_constant__ CUtensorMap tma_k, const __grid_constant__ CUtensorMap tma_v,
                      const DecodeTcParams p) {
  griddep_wait();                    // q and the new K/V rows come from the kernels before this one
  extern __shared__ __align__(1024) uint8_t smem[];
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + DT_SMEM_BAR);
  // S, P and the "PV done" signal are double buffered (index = tile & 1) so that the softmax of tile j+1
  // overlaps the V^T P product of tile j; one barrier per buffer keeps every parity wait unambiguous.
  uint64_t* bar_s = bars + 0;                    // [2]
  uint64_t* bar_p = bars + 2;                    // [2]
  uint64_t* bar_o = bars + 4;                    // [2]
  uint64_t* full = bars + 6;                     // [DT_NBUF]: tile data landed
  uint64_t* empty = full + DT_NBUF;              // [DT_NBUF]: the MMAs that read the buffer have completed
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(empty + DT_NBUF);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  float* red_max = reinterpret_cast<float*>(smem + DT_SMEM_RED);   // [4][16]
  float* red_sum = red_max + 64;                                     // [4][16]

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int b = blockIdx.x, kvh = blockIdx.y, split = blockIdx.z;
  const int G = p.G;
  const int ctx = p.ctx_lens[b];
  const int t_begin = split * p.split_tokens;
  const int t_end = min(ctx, t_begin + p.split_tokens);
  const int n_tiles = t_end > t_begin ? (t_end - t_begin + DT_TILE - 1) / DT_TILE : 0;
  const int* bt = p.block_tables + static_cast<size_t>(b) * p.max_blocks;

  if (threadIdx.x == 0) {
    for (int i = 0; i < 2; ++i) {
      mbar_init(&bar_s[i], 1);
      mbar_init(&bar_p[i], 128);
      mbar_init(&bar_o[i], 1);
    }
    for (int s = 0; s < DT_NBUF; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    *abort_flag = 0;
    if ((smem_u32(smem) & 1023u) != 0) {
      *abort_flag = 1;
      if (p.err) atomicCAS(p.err, kOk, kErrBadArgument);
    }
    fence_barrier_init();
  }
  // stage Q (16 rows x 128 d, rows >= G zero) and clear P, both in the swizzled K-major layout
  for (int i = threadIdx.x; i < 2 * 16 * 8; i += DT_THREADS) {   // 16-byte chunks
    const int half = i / 128, row = (i / 8) % 16, c = i % 8;
    uint4 v = make_uint4(0, 0, 0, 0);
    if (row < G) v = *reinterpret_cast<const uint4*>(p.q + (static_cast<size_t>(b) * p.Hq + kvh * G + row) * DT_D + half * 64 + c * 8);
    const int off = half * 2048 + row * 128 + ((c ^ (row & 7)) << 4);
    *reinterpret_cast<uint4*>(smem + DT_SMEM_Q + off) = v;
    *reinterpret_cast<uint4*>(smem + DT_SMEM_P + off) = make_uint4(0, 0, 0, 0);
    *reinterpret_cast<uint4*>(smem + DT_SMEM_P + 4096 + off) = make_uint4(0, 0, 0, 0);
  }
  fence_proxy_async();
  if (warp == 5) {
    tmem_alloc<DT_TMEM_COLS>(tmem_slot);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const bool dead = (*abort_flag != 0);

  if (warp == 4) {
    // ================================================================ TMA producer (page gather)
    if (lane == 0 && !dead) {
      bool ok = true;
      for (int u = 0; u < 2 * n_tiles && ok; ++u) {      // u even: K of tile u/2, u odd: V of tile u/2
        const int s = u % DT_NBUF;
        if (!mbar_wait(&empty[s], (static_cast<uint32_t>(u / DT_NBUF) & 1) ^ 1, abort_flag, p.err)) { ok = false; break; }
        uint8_t* dst = smem + DT_SMEM_KV + s * DT_KV_BYTES;
        const CUtensorMap* map = (u & 1) ? &tma_v : &tma_k;
        const int page0 = (t_begin + (u >> 1) * DT_TILE) / DT_PAGE;
        mbar_expect_tx(&full[s], DT_KV_BYTES);
        for (int pg = 0; pg < DT_TILE / DT_PAGE; ++pg) {
          const int idx = min(page0 + pg, p.max_blocks - 1);
          const int row = bt[idx] * DT_PAGE;
          tma_load_3d(dst + pg * 2048, map, &full[s], 0, kvh, row);
          tma_load_3d(dst + DT_KV_BYTES / 2 + pg * 2048, map, &full[s], 64, kvh, row);
        }
      }
    }
  } else if (warp == 5) {
    // ================================================================ MMA issuer
    if (lane == 0 && !dead && n_tiles > 0) {
      const uint32_t id_s = make_idesc_f16(128, DT_NPAD, true, false, false);   // K tile x Q^T, both K-major
      const uint32_t id_o = make_idesc_f16(128, DT_NPAD, true, true, false);    // V^T (MN-major) x P (K-major)
      const uint32_t sq = smem_u32(smem + DT_SMEM_Q), sp = smem_u32(smem + DT_SMEM_P);
      auto issue_s = [&](int j) -> bool {
        const int u = 2 * j, s = u % DT_NBUF;
        if (!mbar_wait(&full[s], static_cast<uint32_t>(u / DT_NBUF) & 1, abort_flag, p.err)) return false;
        tc_fence_after();
        const uint32_t sk = smem_u32(smem + DT_SMEM_KV + s * DT_KV_BYTES);
#pragma unroll
        for (int kk = 0; kk < DT_D / 16; ++kk) {
          const uint64_t da = make_smem_desc(sk + (kk >> 2) * (DT_KV_BYTES / 2) + (kk & 3) * 32, 16, 1024, kSwizzle128B);
          const uint64_t db = make_smem_desc(sq + (kk >> 2) * 2048 + (kk & 3) * 32, 16, 1024, kSwizzle128B);
          umma_f16(tmem_base + DT_T_S + (j & 1) * 16, da, db, id_s, kk > 0 ? 1u : 0u);
        }
        umma_commit(&empty[s]);       // the K buffer can be refilled once these MMAs have read it
        umma_commit(&bar_s[j & 1]);
        return true;
      };
      bool ok = issue_s(0);
      if (ok && n_tiles > 1) ok = issue_s(1);
      for (int j = 0; j < n_tiles && ok; ++j) {
        const int u = 2 * j + 1, s = u % DT_NBUF;
        if (!mbar_wait(&bar_p[j & 1], static_cast<uint32_t>(j >> 1) & 1, abort_flag, p.err)) break;
        tc_fence_after();
        if (!mbar_wait(&full[s], static_cast<uint32_t>(u / DT_NBUF) & 1, abort_flag, p.err)) break;
        tc_fence_after();
        const uint32_t sv = smem_u32(smem + DT_SMEM_KV + s * DT_KV_BYTES);
#pragma unroll
        for (int kk = 0; kk < DT_TILE / 16; ++kk) {
          // A = V^T: M = d (two 64-wide chunks DT_KV_BYTES/2 apart), K = tokens (16 rows = 2048 bytes)
          const uint64_t da = make_smem_desc(sv + kk * 2048, DT_KV_BYTES / 2, 1024, kSwizzle128B);
          // B = P[16 heads][128 tokens], K-major, two 64-token halves 2048 bytes apart
          const uint64_t db = make_smem_desc(sp + (j & 1) * 4096 + (kk >> 2) * 2048 + (kk & 3) * 32, 16, 1024, kSwizzle128B);
          umma_f16(tmem_base + DT_T_O, da, db, id_o, (j > 0 || kk > 0) ? 1u : 0u);
        }
        umma_commit(&empty[s]);
        umma_commit(&bar_o[j & 1]);
        // the S buffer of tile j was consumed before bar_p[j & 1] completed: refill it with tile j + 2
        if (j + 2 < n_tiles && !issue_s(j + 2)) break;
      }
    }
  } else {
    // ================================================================ softmax + epilogue (warps 0..3)
    const int r = warp * 32 + lane;   // token row of S^T, d row of O^T
    const uint32_t lane_addr = static_cast<uint32_t>(warp * 32) << 16;
    float m_ref[8], l_part[8];
#pragma unroll
    for (int h = 0; h < 8; ++h) { m_ref[h] = -1e30f; l_part[h] = 0.f; }
    bool ok = !dead;
    // Failure handling: a wait that runs out only clears `ok`; the loop keeps its shape so that all
    // 128 threads still meet at the named barriers (every later wait returns at once after an abort).
    for (int j = 0; j < n_tiles; ++j) {
      if (ok) ok = mbar_wait(&bar_s[j & 1], static_cast<uint32_t>(j >> 1) & 1, abort_flag, p.err);
      tc_fence_after();
      uint32_t raw[16];
      tmem_ld_32x32b_x16(tmem_base + DT_T_S + (j & 1) * 16 + lane_addr, raw);
      tmem_wait_ld();
      const int tok = t_begin + j * DT_TILE + r;
      const bool valid = tok < t_end;
      float s[8];
#pragma unroll
      for (int h = 0; h < 8; ++h) {
        s[h] = (valid && h < G) ? __uint_as_float(raw[h]) * p.scale_log2 : -1e30f;
        const float wm = warp_max(s[h]);
        if (lane == 0) red_max[warp * 16 + h] = wm;
      }
      named_bar_sync(1, 128);
      float alpha[8];
      bool rescale = false;
#pragma unroll
      for (int h = 0; h < 8; ++h) {
        const float tm = fmaxf(fmaxf(red_max[h], red_max[16 + h]), fmaxf(red_max[32 + h], red_max[48 + h]));
        alpha[h] = 1.f;
        if (tm > m_ref[h] + 8.f) {
          alpha[h] = exp2f(m_ref[h] - tm);
          m_ref[h] = tm;
          l_part[h] *= alpha[h];
          rescale = true;
        }
      }
      if (j >= 2) {  // this P buffer was last read by the V^T P product of tile j - 2
        if (ok) ok = mbar_wait(&bar_o[j & 1], static_cast<uint32_t>((j - 2) >> 1) & 1, abort_flag, p.err);
      }
      if (j > 0 && rescale) {   // O^T may only be rescaled once the product of tile j - 1 has landed (rare: lazy threshold)
        if (ok) ok = mbar_wait(&bar_o[(j - 1) & 1], static_cast<uint32_t>((j - 1) >> 1) & 1, abort_flag, p.err);
        tc_fence_after();
        {
          uint32_t o[16];
          tmem_ld_32x32b_x16(tmem_base + DT_T_O + lane_addr, o);
          tmem_wait_ld();
#pragma unroll
          for (int h = 0; h < 8; ++h) o[h] = __float_as_uint(__uint_as_float(o[h]) * alpha[h]);
          tmem_st_32x32b_x16(tmem_base + DT_T_O + lane_addr, o);
          tmem_wait_st();
        }
      }
      // P[h][token r]: K-major [16 rows][128 tokens] as two 64-token halves
      const int half = r >> 6, col = r & 63;
      uint8_t* prow = smem + DT_SMEM_P + (j & 1) * 4096 + half * 2048 + ((col & 7) << 1);
#pragma unroll
      for (int h = 0; h < 8; ++h) {
        if (h < G) {
          const float pv = valid ? exp2f(s[h] - m_ref[h]) : 0.f;
          l_part[h] += pv;
          *reinterpret_cast<__nv_bfloat16*>(prow + h * 128 + (((col >> 3) ^ (h & 7)) << 4)) = __float2bfloat16(pv);
        }
      }
      named_bar_sync(1, 128);   // red_max may be rewritten by the next tile only after everyone has read it
      fence_proxy_async();
      tc_fence_before();
      mbar_arrive(&bar_p[j & 1]);
    }
    if (ok && n_tiles > 1) ok = mbar_wait(&bar_o[(n_tiles - 2) & 1], static_cast<uint32_t>((n_tiles - 2) >> 1) & 1, abort_flag, p.err);
    if (ok && n_tiles > 0) ok = mbar_wait(&bar_o[(n_tiles - 1) & 1], static_cast<uint32_t>((n_tiles - 1) >> 1) & 1, abort_flag, p.err);
    tc_fence_after();
    // ---- total sums per head
#pragma unroll
    for (int h = 0; h < 8; ++h) {
      const float ws = warp_sum(l_part[h]);
      if (lane == 0) red_sum[warp * 16 + h] = ws;
    }
    named_bar_sync(1, 128);
    uint32_t o[16];
    if (n_tiles > 0 && ok) {
      tmem_ld_32x32b_x16(tmem_base + DT_T_O + lane_addr, o);
      tmem_wait_ld();
    } else {
#pragma unroll
      for (int i = 0; i < 16; ++i) o[i] = 0;
    }
#pragma unroll
    for (int h = 0; h < 8; ++h) {
      if (h < G) {
        const float l = red_sum[h] + red_sum[16 + h] + red_sum[32 + h] + red_sum[48 + h];
        const int hq = kvh * G + h;
        const float ov = __uint_as_float(o[h]);
        if (p.num_splits == 1) {
          p.out[(static_cast<size_t>(b) * p.Hq + hq) * DT_D + r] = __float2bfloat16(l > 0.f ? ov / l : 0.f);
        } else {
          const size_t pidx = (static_cast<size_t>(b) * p.Hq + hq) * p.num_splits + split;
          p.part_o[pidx * DT_D + r] = ov;
          if (r == 0) { p.part_ml[pidx * 2] = m_ref[h]; p.part_ml[pidx * 2 + 1] = l; }
        }
      }
    }
  }

  if (*abort_flag) __nanosleep(50000);
  tc_fence_before();
  __syncthreads();
  if (warp == 5) {
    tc_fence_after();
    tmem_dealloc<DT_TMEM_COLS>(tmem_base);
  }
}

__global__ void decode_attn_tc_combine_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml,
                                              __nv_bfloat16* __restrict__ out, int num_splits) {
  const size_t bh = blockIdx.x;
  const int d = threadIdx.x;
  float m = -1e30f;
  for (int s = 0; s < num_splits; ++s) m = fmaxf(m, part_ml[(bh * num_splits + s) * 2]);
  float l = 0.f, o = 0.f;
  for (int s = 0; s < num_splits; ++s) {
    const float w = exp2f(part_ml[(bh * num_splits + s) * 2] - m);
    l += w * part_ml[(bh * num_splits + s) * 2 + 1];
    o += w * part_o[(bh * num_splits + s) * DT_D + d];
  }
  out[bh * DT_D + d] = __float2bfloat16(l > 0.f ? o / l : 0.f);
}

}  // namespace rb

// caches: [num_blocks][16][Hkv][128] bf16 (block_size must be 16).  Scratch as for rb_decode_attn.
extern "C" int rb_decode_attn_tc(const void* q, const void* kc, const void* vc, const int* block_tables,
                                 const int* ctx_lens, void* out, float* part_o, float* part_ml, int B, int Hq, int Hkv,
                                 int num_blocks, int block_size, int max_blocks, int max_ctx, float scale, int splits,
                                 int* err, cudaStream_t st) {
  using namespace rb;
  if (B == 0) return 0;
  const int G = Hq / Hkv;
  if (Hq % Hkv || G > 8 || block_size != DT_PAGE) return -2;
  CUtensorMap tk, tv;
  const uint64_t slots = static_cast<uint64_t>(num_blocks) * block_size;
  int rc = encode_tma_3d_16bit(&tk, kc, DT_D, Hkv, slots, DT_D, static_cast<uint64_t>(Hkv) * DT_D, 64, 1, DT_PAGE);
  if (rc) return rc;
  rc = encode_tma_3d_16bit(&tv, vc, DT_D, Hkv, slots, DT_D, static_cast<uint64_t>(Hkv) * DT_D, 64, 1, DT_PAGE);
  if (rc) return rc;
  static bool attr_set = false;
  if (!attr_set) {
    cudaError_t e = cudaFuncSetAttribute(decode_attn_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, DT_SMEM_TOTAL);
    if (e != cudaSuccess) return static_cast<int>(e);
    attr_set = true;
  }
  DecodeTcParams p{};
  p.q = (const __nv_bfloat16*)q; p.block_tables = block_tables; p.ctx_lens = ctx_lens; p.out = (__nv_bfloat16*)out;
  p.part_o = part_o; p.part_ml = part_ml; p.Hq = Hq; p.Hkv = Hkv; p.G = G; p.max_blocks = max_blocks;
  p.num_splits = splits;
  p.split_tokens = ((max_ctx + splits - 1) / splits + DT_TILE - 1) / DT_TILE * DT_TILE;
  p.scale_log2 = scale * 1.4426950408889634f;
  p.err = err;
  dim3 grid(B, Hkv, splits);
  launch_pdl(decode_attn_tc_kernel, dim3(grid), dim3(DT_THREADS), DT_SMEM_TOTAL, st, tk, tv, p);
  if (splits > 1) decode_attn_tc_combine_kernel<<<B * Hq, DT_D, 0, st>>>(part_o, part_ml, (__nv_bfloat16*)out, splits);
  rb_note_launch(splits > 1 ? 2 : 1);
  return (int)cudaGetLastError();
}
