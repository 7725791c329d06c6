// Host helpers: build TMA tensor maps through the driver entry point (no link-time
// dependency on libcuda) and report errors as negative codes.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>

// Number of kernel launches issued by this library since load (read by the benchmark).
extern "C" long long ttb_launch_counter;
#define TTB_COUNT_LAUNCH(n) (ttb_launch_counter += (n))

// Index values that come from user data (token ids, labels, positions) are never used out of range: the kernel substitutes a
// safe value and counts the event in a per-file device counter, which the host reads through ttb_index_violations().  With
// TTB_DEBUG_BOUNDS=1 the Python layer turns a non-zero count into an exception at its next device check.
#define TTB_DEFINE_VIOLATION_COUNTER(name)                                          \
  static __device__ unsigned int g_violations_##name;                               \
  extern "C" unsigned int ttb_violations_##name(int reset) {                        \
    unsigned int v = 0;                                                             \
    if (cudaMemcpyFromSymbol(&v, g_violations_##name, sizeof(v)) != cudaSuccess) return 0xffffffffu; \
    if (reset && v != 0) {                                                          \
      const unsigned int z = 0;                                                     \
      cudaMemcpyToSymbol(g_violations_##name, &z, sizeof(z));                       \
    }                                                                               \
    return v;                                                                       \
  }
#define TTB_NOTE_VIOLATION(name) atomicAdd(&g_violations_##name, 1u)

namespace ttb {

enum : int {
  kOk = 0,
  kErrBadShape = -1,      // a size/alignment rule of the kernel was violated
  kErrDriver = -2,        // tensor-map creation or launch failed
  kErrTooLarge = -3,      // exceeds a stated static limit
  kErrDeviceTimeout = -4  // a bounded device-side wait ran out
};

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

inline EncodeTiledFn encode_tiled_fn() {
  static EncodeTiledFn fn = nullptr;
  if (fn) return fn;
  void* p = nullptr;
  cudaDriverEntryPointQueryResult q;
  if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess ||
      q != cudaDriverEntryPointSuccess)
    return nullptr;
  fn = reinterpret_cast<EncodeTiledFn>(p);
  return fn;
}

// 2-D row-major tensor [rows, cols] of `elem_bytes`-wide elements; box = [box_rows, box_cols];
// 128-byte swizzle requires box_cols * elem_bytes == 128.  row_stride_elems >= cols.
inline int make_tmap_2d(CUtensorMap* out, const void* base, CUtensorMapDataType dt, int elem_bytes, uint64_t rows,
                        uint64_t cols, uint64_t row_stride_elems, uint32_t box_rows, uint32_t box_cols,
                        CUtensorMapSwizzle swz) {
  EncodeTiledFn fn = encode_tiled_fn();
  if (!fn) return kErrDriver;
  if ((reinterpret_cast<uintptr_t>(base) & 15) || ((row_stride_elems * elem_bytes) & 15)) return kErrBadShape;
  cuuint64_t dims[2] = {cols, rows};
  cuuint64_t strides[1] = {row_stride_elems * static_cast<uint64_t>(elem_bytes)};
  cuuint32_t box[2] = {box_cols, box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(out, dt, 2, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, swz,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS)
    fprintf(stderr, "[ttb] cuTensorMapEncodeTiled failed: code %d (rows=%llu cols=%llu stride=%llu box=%ux%u)\n",
            static_cast<int>(r), (unsigned long long)rows, (unsigned long long)cols,
            (unsigned long long)row_stride_elems, box_rows, box_cols);
  return r == CUDA_SUCCESS ? kOk : kErrDriver;
}

// 3-D tensor [d2, d1, d0] (d0 innermost, contiguous) with byte strides for d1 and d2.
inline int make_tmap_3d(CUtensorMap* out, const void* base, CUtensorMapDataType dt, uint64_t d0, uint64_t d1,
                        uint64_t d2, uint64_t stride1_bytes, uint64_t stride2_bytes, uint32_t b0, uint32_t b1,
                        uint32_t b2, CUtensorMapSwizzle swz) {
  EncodeTiledFn fn = encode_tiled_fn();
  if (!fn) return kErrDriver;
  if ((reinterpret_cast<uintptr_t>(base) & 15) || (stride1_bytes & 15) || (stride2_bytes & 15)) return kErrBadShape;
  cuuint64_t dims[3] = {d0, d1, d2};
  cuuint64_t strides[2] = {stride1_bytes, stride2_bytes};
  cuuint32_t box[3] = {b0, b1, b2};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = fn(out, dt, 3, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, swz,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? kOk : kErrDriver;
}

inline int sm_count() {
  static int n = 0;
  if (!n) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
  }
  return n;
}

}  // namespace ttb
