// Host-side helpers shared by the launchers: TMA tensor-map encoding through the driver
// entry point (no link-time dependency on libcuda), device properties, error strings.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>

namespace ob {

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                  const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// cuTensorMapEncodeTiled is a driver call and needs the device's primary context current in the
// calling thread.  A thread that has made no runtime call yet (an autograd worker entering its
// first backward through a GEMM) has none: bind it once per thread through the runtime.
inline void ensure_thread_context() {
  static thread_local bool ready = false;
  if (!ready) {
    int dev = 0;
    if (cudaGetDevice(&dev) == cudaSuccess) cudaSetDevice(dev);
    ready = true;
  }
}

inline EncodeTiledFn get_encode_fn() {
  ensure_thread_context();
  static EncodeTiledFn fn = nullptr;
  if (!fn) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess ||
        q != cudaDriverEntryPointSuccess)
      return nullptr;
    fn = (EncodeTiledFn)p;
  }
  return fn;
}

// rank-2 bf16 map over a row-major [rows, cols] view with row pitch `ld` elements;
// box = box_rows x box_cols, 128-byte swizzle when box_cols*2 == 128, none otherwise.
inline int make_tmap_2d(CUtensorMap* m, const void* base, uint64_t rows, uint64_t cols, uint64_t ld,
                        uint32_t box_rows, uint32_t box_cols, int elem_bytes = 2,
                        bool swizzle = true) {
  EncodeTiledFn fn = get_encode_fn();
  if (!fn) return -1;
  cuuint64_t dims[2] = {cols, rows};
  cuuint64_t strides[1] = {ld * (uint64_t)elem_bytes};
  cuuint32_t box[2] = {box_cols, box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUtensorMapDataType dt = elem_bytes == 2 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16
                                           : CU_TENSOR_MAP_DATA_TYPE_FLOAT32;
  CUresult r = fn(m, dt, 2, const_cast<void*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE,
                  swizzle ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : (int)r;
}

// rank-3 bf16 map: dims (d0 innermost, d1, d2) with byte strides s1, s2.
inline int make_tmap_3d(CUtensorMap* m, const void* base, uint64_t d0, uint64_t d1, uint64_t d2,
                        uint64_t s1_bytes, uint64_t s2_bytes, uint32_t b0, uint32_t b1,
                        uint32_t b2, bool swizzle = true) {
  EncodeTiledFn fn = get_encode_fn();
  if (!fn) return -1;
  cuuint64_t dims[3] = {d0, d1, d2};
  cuuint64_t strides[2] = {s1_bytes, s2_bytes};
  cuuint32_t box[3] = {b0, b1, b2};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = fn(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(base), dims, strides,
                  box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  swizzle ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : (int)r;
}

inline int num_sms() {
  static int n[64] = {0};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64) dev = 0;
  if (!n[dev]) cudaDeviceGetAttribute(&n[dev], cudaDevAttrMultiProcessorCount, dev);
  return n[dev];
}

// Raise a kernel's dynamic shared-memory limit once per device (the attribute is per device, and
// one process may drive several).
#define OB_ENSURE_DYN_SMEM(kern, bytes)                                                               \
  do {                                                                                                \
    static bool done__[64] = {};                                                                      \
    int dev__ = 0;                                                                                    \
    cudaGetDevice(&dev__);                                                                            \
    if (dev__ < 0 || dev__ >= 64) dev__ = 0;                                                          \
    if (!done__[dev__]) {                                                                             \
      cudaError_t ce__ = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes); \
      if (ce__ != cudaSuccess) return 4000 + (int)ce__;                                               \
      done__[dev__] = true;                                                                           \
    }                                                                                                 \
  } while (0)

#define OB_CHECK_LAUNCH()                                  \
  do {                                                     \
    cudaError_t e__ = cudaGetLastError();                  \
    if (e__ != cudaSuccess) return 1000 + (int)e__;        \
  } while (0)

}  // namespace ob
