// Multi-tensor AdamW and squared-gradient-norm kernels: one launch covers every parameter
// of a group through a device-resident metadata table.  Semantics: torch.optim.AdamW
// (decoupled weight decay, bias-corrected moments), fp32 math, state stored in the
// parameter dtype; an optional fp32 master copy keeps the exact weights for bf16 params.
// The gradient multiplier may live on the device (token-count normalisation and clipping
// coefficient are then applied without a host synchronisation).
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "common/tmap.h"

namespace ttb {

struct TensorMeta {
  void* p;
  const void* g;
  void* m;
  void* v;
  float* master;          // nullptr when absent
  long long numel;
  long long chunk_start;  // prefix sum of chunk counts
};

static constexpr int kChunk = 4096;

template <typename T>
__device__ __forceinline__ float to_f(T v);
template <>
__device__ __forceinline__ float to_f<float>(float v) { return v; }
template <>
__device__ __forceinline__ float to_f<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }
template <typename T>
__device__ __forceinline__ T from_f(float v);
template <>
__device__ __forceinline__ float from_f<float>(float v) { return v; }
template <>
__device__ __forceinline__ __nv_bfloat16 from_f<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

__device__ __forceinline__ int find_tensor(const TensorMeta* metas, int n, long long chunk) {
  int lo = 0, hi = n - 1;
  while (lo < hi) {
    const int mid = (lo + hi + 1) >> 1;
    if (metas[mid].chunk_start <= chunk) lo = mid; else hi = mid - 1;
  }
  return lo;
}

template <typename T>
__global__ void __launch_bounds__(256)
adamw_kernel(const TensorMeta* __restrict__ metas, int n_tensors, long long total_chunks, float lr, float beta1,
             float beta2, float eps, float weight_decay, float inv_bc1, float inv_sqrt_bc2,
             const float* __restrict__ scale_dev, float scale_host) {
  const float gs = scale_host * (scale_dev != nullptr ? *scale_dev : 1.f);
  for (long long chunk = blockIdx.x; chunk < total_chunks; chunk += gridDim.x) {
    const int ti = find_tensor(metas, n_tensors, chunk);
    const TensorMeta tm = metas[ti];
    const long long base = (chunk - tm.chunk_start) * kChunk;
    T* p = static_cast<T*>(tm.p);
    const T* g = static_cast<const T*>(tm.g);
    T* m = static_cast<T*>(tm.m);
    T* v = static_cast<T*>(tm.v);
    if (sizeof(T) == 2 && tm.master == nullptr && base + kChunk <= tm.numel &&
        ((reinterpret_cast<uintptr_t>(p) | reinterpret_cast<uintptr_t>(g) | reinterpret_cast<uintptr_t>(m) | reinterpret_cast<uintptr_t>(v)) & 15) == 0) {
      // full chunk of 16-byte aligned bf16 tensors: 8 elements per thread and access (the chunk offset is a multiple of 8)
      const float decay = 1.f - lr * weight_decay;
#pragma unroll
      for (int it = 0; it < kChunk / (256 * 8); ++it) {
        const long long e = base + (it * 256 + threadIdx.x) * 8;
        const uint4 gq = *reinterpret_cast<const uint4*>(reinterpret_cast<const __nv_bfloat16*>(g) + e);
        uint4 pq = *reinterpret_cast<const uint4*>(reinterpret_cast<const __nv_bfloat16*>(p) + e);
        uint4 mq = *reinterpret_cast<const uint4*>(reinterpret_cast<const __nv_bfloat16*>(m) + e);
        uint4 vq = *reinterpret_cast<const uint4*>(reinterpret_cast<const __nv_bfloat16*>(v) + e);
        const __nv_bfloat162* g2 = reinterpret_cast<const __nv_bfloat162*>(&gq);
        __nv_bfloat162* p2 = reinterpret_cast<__nv_bfloat162*>(&pq);
        __nv_bfloat162* m2 = reinterpret_cast<__nv_bfloat162*>(&mq);
        __nv_bfloat162* v2 = reinterpret_cast<__nv_bfloat162*>(&vq);
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          const float2 gf = __bfloat1622float2(g2[k]), pf = __bfloat1622float2(p2[k]), mf = __bfloat1622float2(m2[k]), vf = __bfloat1622float2(v2[k]);
          float w[2] = {pf.x, pf.y}, m1[2], v1[2];
          const float gr[2] = {gf.x * gs, gf.y * gs}, mo[2] = {mf.x, mf.y}, vo[2] = {vf.x, vf.y};
#pragma unroll
          for (int q = 0; q < 2; ++q) {
            m1[q] = beta1 * mo[q] + (1.f - beta1) * gr[q];
            v1[q] = beta2 * vo[q] + (1.f - beta2) * gr[q] * gr[q];
            w[q] = w[q] * decay - lr * inv_bc1 * m1[q] / (sqrtf(v1[q]) * inv_sqrt_bc2 + eps);
          }
          p2[k] = __floats2bfloat162_rn(w[0], w[1]);
          m2[k] = __floats2bfloat162_rn(m1[0], m1[1]);
          v2[k] = __floats2bfloat162_rn(v1[0], v1[1]);
        }
        *reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(p) + e) = pq;
        *reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(m) + e) = mq;
        *reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(v) + e) = vq;
      }
      continue;
    }
#pragma unroll 4
    for (int i = threadIdx.x; i < kChunk; i += 256) {
      const long long e = base + i;
      if (e < tm.numel) {
        const float grad = to_f<T>(g[e]) * gs;
        float w = tm.master != nullptr ? tm.master[e] : to_f<T>(p[e]);
        const float m1 = beta1 * to_f<T>(m[e]) + (1.f - beta1) * grad;
        const float v1 = beta2 * to_f<T>(v[e]) + (1.f - beta2) * grad * grad;
        w *= (1.f - lr * weight_decay);
        w -= lr * inv_bc1 * m1 / (sqrtf(v1) * inv_sqrt_bc2 + eps);
        m[e] = from_f<T>(m1);
        v[e] = from_f<T>(v1);
        p[e] = from_f<T>(w);
        if (tm.master != nullptr) tm.master[e] = w;
      }
    }
  }
}

template <typename T>
__global__ void __launch_bounds__(256)
sumsq_kernel(const TensorMeta* __restrict__ metas, int n_tensors, long long total_chunks, float* __restrict__ out) {
  __shared__ float red[8];
  float acc = 0.f;
  for (long long chunk = blockIdx.x; chunk < total_chunks; chunk += gridDim.x) {
    const int ti = find_tensor(metas, n_tensors, chunk);
    const TensorMeta tm = metas[ti];
    const long long base = (chunk - tm.chunk_start) * kChunk;
    const T* g = static_cast<const T*>(tm.g);
    if (sizeof(T) == 2 && base + kChunk <= tm.numel && (reinterpret_cast<uintptr_t>(g) & 15) == 0) {
#pragma unroll
      for (int it = 0; it < kChunk / (256 * 8); ++it) {
        const uint4 gq = *reinterpret_cast<const uint4*>(reinterpret_cast<const __nv_bfloat16*>(g) + base + (it * 256 + threadIdx.x) * 8);
        const __nv_bfloat162* g2 = reinterpret_cast<const __nv_bfloat162*>(&gq);
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          const float2 f = __bfloat1622float2(g2[k]);
          acc += f.x * f.x + f.y * f.y;
        }
      }
      continue;
    }
    for (int i = threadIdx.x; i < kChunk; i += 256) {
      const long long e = base + i;
      if (e < tm.numel) {
        const float f = to_f<T>(g[e]);
        acc += f * f;
      }
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = acc;
  __syncthreads();
  if (threadIdx.x == 0) {
    float t = 0.f;
    for (int i = 0; i < 8; ++i) t += red[i];
    out[blockIdx.x] = t;  // caller sums the per-block partials (deterministic)
  }
}

}  // namespace ttb

using namespace ttb;

extern "C" int ttb_meta_stride() { return static_cast<int>(sizeof(TensorMeta)); }
extern "C" int ttb_optim_chunk() { return kChunk; }
extern "C" int ttb_optim_grid() { return sm_count() * 8; }

// metas: device array of n_tensors TensorMeta records (7 x 8 bytes each).
extern "C" int ttb_adamw(const void* metas, int n_tensors, long long total_chunks, int is_bf16, float lr, float beta1,
                         float beta2, float eps, float weight_decay, float inv_bc1, float inv_sqrt_bc2,
                         const float* scale_dev, float scale_host, void* stream) {
  if (n_tensors <= 0 || total_chunks <= 0) return kOk;
  const long long cap = ttb_optim_grid();
  const int grid = static_cast<int>(total_chunks < cap ? total_chunks : cap);
  auto s = static_cast<cudaStream_t>(stream);
  TTB_COUNT_LAUNCH(1);
  if (is_bf16)
    adamw_kernel<__nv_bfloat16><<<grid, 256, 0, s>>>(static_cast<const TensorMeta*>(metas), n_tensors, total_chunks, lr,
                                                     beta1, beta2, eps, weight_decay, inv_bc1, inv_sqrt_bc2, scale_dev,
                                                     scale_host);
  else
    adamw_kernel<float><<<grid, 256, 0, s>>>(static_cast<const TensorMeta*>(metas), n_tensors, total_chunks, lr, beta1,
                                             beta2, eps, weight_decay, inv_bc1, inv_sqrt_bc2, scale_dev, scale_host);
  return cudaGetLastError() == cudaSuccess ? kOk : kErrDriver;
}

// partials: device float array of ttb_optim_grid() entries (unused tail entries are written as 0).
extern "C" int ttb_grad_sumsq(const void* metas, int n_tensors, long long total_chunks, int is_bf16, float* partials,
                              void* stream) {
  auto s = static_cast<cudaStream_t>(stream);
  const int grid = ttb_optim_grid();
  TTB_COUNT_LAUNCH(1);
  if (is_bf16)
    sumsq_kernel<__nv_bfloat16><<<grid, 256, 0, s>>>(static_cast<const TensorMeta*>(metas), n_tensors, total_chunks,
                                                     partials);
  else
    sumsq_kernel<float><<<grid, 256, 0, s>>>(static_cast<const TensorMeta*>(metas), n_tensors, total_chunks, partials);
  return cudaGetLastError() == cudaSuccess ? kOk : kErrDriver;
}
