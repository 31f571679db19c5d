// Host helpers shared by the kernel translation units: SM count, tensor-map
// encoding through the driver entry point (no link-time dependency on libcuda).
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdlib.h>

extern "C" void rb_note_launch(int n);
extern "C" long long rb_launch_count();
extern "C" void rb_reset_launch_count();

namespace rb {

// Programmatic dependent launch: a kernel launched through launch_pdl may become resident while its predecessor
// in the stream is still draining and run everything that does not depend on the predecessor's output (barrier
// set-up, TMEM allocation, weight prefetch) before its griddepcontrol.wait.  Every kernel launched this way executes
// that wait in all of its threads before it reads or writes anything an earlier kernel may touch.
// Off unless RELAX_B200_PDL=1 (the waits are no-ops without the attribute): inside the captured decode graph the
// launch gaps are already closed, and the measured step time was the same with and without it (10.69 vs 10.68 ms at
// batch 128); letting dependents start while the primary still runs made the step slower (11.4 ms).
inline bool pdl_enabled() {
  static int v = -1;
  if (v < 0) {
    const char* e = getenv("RELAX_B200_PDL");
    v = (e != nullptr && e[0] == '1') ? 1 : 0;
  }
  return v != 0;
}

template <typename... KArgs, typename... Args>
inline cudaError_t launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st, Args&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute at[1];
  at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  at[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = at;
  cfg.numAttrs = pdl_enabled() ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

inline int num_sms() {
  static int n = 0;
  if (n == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
    if (n <= 0) n = 148;
  }
  return n;
}

// Tensor-map encoding is a driver call and needs a current context on the calling thread.
// Worker threads (e.g. an autograd engine thread) may not have touched the runtime yet.
inline void ensure_context() {
  static thread_local bool done = false;
  if (!done) {
    cudaFree(nullptr);
    done = true;
  }
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

inline EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  if (!fn) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
  }
  return fn;
}

// 2-D row-major tensor of 16-bit elements: `inner` contiguous elements per row, `outer` rows,
// row pitch `ld` elements.  Box = box_inner x box_outer, 128-byte swizzle, zero fill out of bounds.
inline int encode_tma_2d_16bit(CUtensorMap* map, const void* ptr, uint64_t inner, uint64_t outer, uint64_t ld,
                               uint32_t box_inner, uint32_t box_outer, bool is_bf16 = true, bool swizzle128 = true) {
  ensure_context();
  EncodeTiledFn fn = encode_fn();
  if (!fn) return -10;
  cuuint64_t dims[2] = {inner, outer};
  cuuint64_t strides[1] = {ld * 2};
  cuuint32_t box[2] = {box_inner, box_outer};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(map, is_bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2,
                  const_cast<void*>(ptr), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  swizzle128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : -11;
}
inline int encode_tma_2d_bf16(CUtensorMap* map, const void* ptr, uint64_t inner, uint64_t outer, uint64_t ld,
                              uint32_t box_inner, uint32_t box_outer) {
  return encode_tma_2d_16bit(map, ptr, inner, outer, ld, box_inner, box_outer, true, true);
}

// 2-D row-major tensor of 8-bit elements (fp8): `inner` bytes per row, pitch `ld` bytes; 128-byte swizzle.
inline int encode_tma_2d_8bit(CUtensorMap* map, const void* ptr, uint64_t inner, uint64_t outer, uint64_t ld,
                              uint32_t box_inner, uint32_t box_outer) {
  ensure_context();
  EncodeTiledFn fn = encode_fn();
  if (!fn) return -10;
  cuuint64_t dims[2] = {inner, outer};
  cuuint64_t strides[1] = {ld};
  cuuint32_t box[2] = {box_inner, box_outer};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(ptr), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : -11;
}

// 2-D row-major tensor of 32-bit elements (fp32 outputs written or reduce-added by TMA): pitch `ld` elements.
inline int encode_tma_2d_32bit(CUtensorMap* map, const void* ptr, uint64_t inner, uint64_t outer, uint64_t ld,
                               uint32_t box_inner, uint32_t box_outer) {
  ensure_context();
  EncodeTiledFn fn = encode_fn();
  if (!fn) return -10;
  cuuint64_t dims[2] = {inner, outer};
  cuuint64_t strides[1] = {ld * 4};
  cuuint32_t box[2] = {box_inner, box_outer};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, const_cast<void*>(ptr), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : -11;
}

// 3-D variant (e.g. [tokens][heads][head_dim] with a head stride).
inline int encode_tma_3d_16bit(CUtensorMap* map, const void* ptr, uint64_t d0, uint64_t d1, uint64_t d2,
                               uint64_t stride1_elems, uint64_t stride2_elems, uint32_t b0, uint32_t b1, uint32_t b2,
                               bool is_bf16 = true) {
  ensure_context();
  EncodeTiledFn fn = encode_fn();
  if (!fn) return -10;
  cuuint64_t dims[3] = {d0, d1, d2};
  cuuint64_t strides[2] = {stride1_elems * 2, stride2_elems * 2};
  cuuint32_t box[3] = {b0, b1, b2};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = fn(map, is_bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 3,
                  const_cast<void*>(ptr), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : -11;
}

}  // namespace rb
