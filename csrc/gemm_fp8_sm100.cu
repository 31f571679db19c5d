// Block-scaled fp8 (e4m3) GEMM for sm_100a:  C[M,N] (bf16) = (A_q * sa) (B_q * sb)^T
//
//   A_q [M][K] e4m3, sa [M][K/128] fp32      one scale per row and 128-wide K block ("1 x 128", activations)
//   B_q [N][K] e4m3, sb [N/128][K/128] fp32  one scale per 128 x 128 block (weights, `weight_scale_inv`)
//
// which is the blockwise recipe of the reference's fp8 configs (TransformerEngine blockwise fp8,
// scripts/training/text/run-qwen3-30B-A3B-fp8-8xgpu.sh:103-104; weight format of
// relax/backends/megatron/kernels/fp8_kernel.py).  The scales change every 128 elements of K, so the
// tensor core cannot accumulate across K blocks on its own: every K block is multiplied into a fresh TMEM
// accumulator (`tcgen05.mma kind::f8f6f4`, four K=32 steps) and the epilogue warps fold it into fp32
// register accumulators with the product of the two scales.  Two TMEM accumulators alternate, so the
// tensor core works on block kb+1 while block kb is being folded.
//
// One CTA per 128 x 128 output tile; warp 0 = TMA producer, warp 1 = MMA issuer, warps 2..5 = fold + store.
#include "common.cuh"
#include "host_utils.h"

namespace rb {

constexpr int F8_BM = 128, F8_BN = 128, F8_BK = 128;     // BK in elements = bytes
constexpr int F8_STAGES = 4;
constexpr int F8_STAGE_BYTES = (F8_BM + F8_BN) * F8_BK;  // 32 KB
constexpr int F8_THREADS = 192;
constexpr int F8_SMEM_BAR = F8_STAGES * F8_STAGE_BYTES;
constexpr int F8_SMEM_TOTAL = F8_SMEM_BAR + 256 + 1024;

struct Fp8Params {
  int M, N, K, ldc;
  const float* sa;   // [M][kblocks]
  const float* sb;   // [ceil(N/128)][kblocks]
  __nv_bfloat16* C;
  int* err;
};

__device__ __forceinline__ void umma_f8(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}

// Instruction descriptor of kind::f8f6f4: fp32 accumulator, A and B e4m3 (format code 0), both K-major.
__host__ __device__ constexpr uint32_t make_idesc_f8(int m, int n) {
  return (1u << 4) | (static_cast<uint32_t>(n >> 3) << 17) | (static_cast<uint32_t>(m >> 4) << 24);
}

__global__ void __launch_bounds__(F8_THREADS, 1)
gemm_fp8_kernel(const __grid_constant__ CUtensorMap tma_a, const __grid_constant__ CUtensorMap tma_b, const Fp8Params p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + F8_SMEM_BAR);
  uint64_t* empty_bar = full_bar + F8_STAGES;
  uint64_t* tfull_bar = empty_bar + F8_STAGES;   // [2]
  uint64_t* tempty_bar = tfull_bar + 2;          // [2]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tempty_bar + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int tiles_n = (p.N + F8_BN - 1) / F8_BN;
  const int tm = blockIdx.x / tiles_n, tn = blockIdx.x % tiles_n;
  const int m0 = tm * F8_BM, n0 = tn * F8_BN;
  const int kblocks = (p.K + F8_BK - 1) / F8_BK;

  if (threadIdx.x == 0) {
    for (int s = 0; s < F8_STAGES; ++s) {
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
    tmem_alloc<256>(tmem_slot);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    if (lane == 0) {
      tma_prefetch_desc(&tma_a);
      tma_prefetch_desc(&tma_b);
      for (int kb = 0; kb < kblocks; ++kb) {
        const int s = kb % F8_STAGES;
        if (!mbar_wait(&empty_bar[s], (static_cast<uint32_t>(kb / F8_STAGES) & 1) ^ 1, abort_flag, p.err)) break;
        uint8_t* sa = smem + s * F8_STAGE_BYTES;
        uint8_t* sb = sa + F8_BM * F8_BK;
        mbar_expect_tx(&full_bar[s], F8_STAGE_BYTES);
        tma_load_2d(sa, &tma_a, &full_bar[s], kb * F8_BK, m0);
        tma_load_2d(sb, &tma_b, &full_bar[s], kb * F8_BK, n0);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      const uint32_t idesc = make_idesc_f8(F8_BM, F8_BN);
      for (int kb = 0; kb < kblocks; ++kb) {
        const int s = kb % F8_STAGES, acc = kb & 1;
        if (!mbar_wait(&tempty_bar[acc], (static_cast<uint32_t>(kb >> 1) & 1) ^ 1, abort_flag, p.err)) break;
        if (!mbar_wait(&full_bar[s], static_cast<uint32_t>(kb / F8_STAGES) & 1, abort_flag, p.err)) break;
        tc_fence_after();
        const uint32_t sa = smem_u32(smem + s * F8_STAGE_BYTES);
        const uint32_t sb = sa + F8_BM * F8_BK;
#pragma unroll
        for (int kk = 0; kk < F8_BK / 32; ++kk) {   // K = 32 elements = 32 bytes inside the 128-byte swizzle row
          const uint64_t da = make_smem_desc(sa + kk * 32, 16, 1024, kSwizzle128B);
          const uint64_t db = make_smem_desc(sb + kk * 32, 16, 1024, kSwizzle128B);
          umma_f8(tmem_base + acc * F8_BN, da, db, idesc, kk > 0 ? 1u : 0u);
        }
        umma_commit(&empty_bar[s]);
        umma_commit(&tfull_bar[acc]);
      }
    }
  } else {
    const int lane_grp = warp & 3;
    const int row = m0 + lane_grp * 32 + lane;
    const bool live = row < p.M;
    float accv[F8_BN];
#pragma unroll
    for (int i = 0; i < F8_BN; ++i) accv[i] = 0.f;
    const float* sa_row = p.sa + static_cast<size_t>(live ? row : 0) * kblocks;
    const float* sb_row = p.sb + static_cast<size_t>(tn) * kblocks;
    bool ok = true;
    for (int kb = 0; kb < kblocks; ++kb) {
      const int acc = kb & 1;
      const float scale = live ? __ldg(sa_row + kb) * __ldg(sb_row + kb) : 0.f;
      if (!mbar_wait(&tfull_bar[acc], static_cast<uint32_t>(kb >> 1) & 1, abort_flag, p.err)) { ok = false; break; }
      tc_fence_after();
      const uint32_t taddr = tmem_base + acc * F8_BN + (static_cast<uint32_t>(lane_grp * 32) << 16);
#pragma unroll
      for (int c = 0; c < F8_BN / 32; ++c) {
        uint32_t r[32];
        tmem_ld_32x32b_x32(taddr + c * 32, r);
        tmem_wait_ld();
#pragma unroll
        for (int i = 0; i < 32; ++i) accv[c * 32 + i] = fmaf(__uint_as_float(r[i]), scale, accv[c * 32 + i]);
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&tempty_bar[acc]);
    }
    if (ok && live) {
      __nv_bfloat16* out = p.C + static_cast<size_t>(row) * p.ldc + n0;
      if (n0 + F8_BN <= p.N && (p.ldc % 8) == 0) {
#pragma unroll
        for (int i = 0; i < F8_BN; i += 8) {
          uint4 pk;
          pk.x = pack_bf16(accv[i], accv[i + 1]);
          pk.y = pack_bf16(accv[i + 2], accv[i + 3]);
          pk.z = pack_bf16(accv[i + 4], accv[i + 5]);
          pk.w = pack_bf16(accv[i + 6], accv[i + 7]);
          *reinterpret_cast<uint4*>(out + i) = pk;
        }
      } else {
#pragma unroll
        for (int i = 0; i < F8_BN; ++i)   // static indices keep the accumulators in registers
          if (n0 + i < p.N) out[i] = __float2bfloat16(accv[i]);
      }
    }
  }

  if (*abort_flag) __nanosleep(50000);
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc<256>(tmem_base);
  }
}

}  // namespace rb

// A_q [M][K] and B_q [N][K] are e4m3 bytes with row pitches lda / ldb (bytes, multiples of 16).
extern "C" int rb_gemm_fp8_blockscaled(const void* A, const float* sa, const void* B, const float* sb, void* C, int M, int N,
                                       int K, int lda, int ldb, int ldc, int* err, cudaStream_t stream) {
  using namespace rb;
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  if ((lda % 16) || (ldb % 16) || (K % 16) || (reinterpret_cast<uintptr_t>(A) % 16) || (reinterpret_cast<uintptr_t>(B) % 16))
    return -2;
  CUtensorMap ta, tb;
  int rc = encode_tma_2d_8bit(&ta, A, K, M, lda, F8_BK, F8_BM);
  if (rc) return rc;
  rc = encode_tma_2d_8bit(&tb, B, K, N, ldb, F8_BK, F8_BN);
  if (rc) return rc;
  static bool attr_set = false;
  if (!attr_set) {
    cudaError_t e = cudaFuncSetAttribute(gemm_fp8_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, F8_SMEM_TOTAL);
    if (e != cudaSuccess) return static_cast<int>(e);
    attr_set = true;
  }
  Fp8Params p{};
  p.M = M; p.N = N; p.K = K; p.ldc = ldc; p.sa = sa; p.sb = sb; p.C = reinterpret_cast<__nv_bfloat16*>(C); p.err = err;
  const int tiles = ((M + F8_BM - 1) / F8_BM) * ((N + F8_BN - 1) / F8_BN);
  gemm_fp8_kernel<<<tiles, F8_THREADS, F8_SMEM_TOTAL, stream>>>(ta, tb, p);
  rb_note_launch(1);
  return static_cast<int>(cudaGetLastError());
}
