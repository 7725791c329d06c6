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


// ----------------------------------------------------------------------------- AdamW with 8-bit moments
// Both moments are stored in one byte per element with one fp32 scale per block of 256 elements:
//     exp_avg     = sign(q) · (|q| / 127)² · scale        (int8; square-root companding: fine steps near zero)
//     exp_avg_sq  = (q / 255)⁴ · scale                    (uint8; fourth-root companding: the second moment spans many decades)
// where scale is the block's largest magnitude.  One warp owns one block: each lane expands its 8 elements, applies the AdamW
// update in fp32 (same formulas as adamw_kernel), the warp reduces the new block maxima, and the lane codes its elements again.
// Memory per parameter: 2 bytes + 8 / 256 instead of 4 (bf16 moments) or 8 (fp32 moments).
static constexpr int kQBlock = 256;

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// Square root through the reciprocal-square-root unit (two instructions; exact enough for a code of 8 bits and for an update that
// is rounded to bf16).  The floor keeps 0 · inf out of the product.
__device__ __forceinline__ float fast_sqrt(float x) { return x * rsqrtf(fmaxf(x, 1e-37f)); }

template <typename T>
__global__ void __launch_bounds__(256, 4)
adamw8bit_kernel(T* __restrict__ p, const T* __restrict__ g, int8_t* __restrict__ mq, uint8_t* __restrict__ vq,
                 float* __restrict__ mscale, float* __restrict__ vscale, long long numel, float lr, float beta1, float beta2,
                 float eps, float weight_decay, float inv_bc1, float inv_sqrt_bc2, const float* __restrict__ scale_dev,
                 float scale_host) {
  const float gs = scale_host * (scale_dev != nullptr ? *scale_dev : 1.f);
  const float decay = 1.f - lr * weight_decay;
  const int lane = threadIdx.x & 31;
  const long long n_blocks = (numel + kQBlock - 1) / kQBlock;
  for (long long blk = static_cast<long long>(blockIdx.x) * 8 + (threadIdx.x >> 5); blk < n_blocks;
       blk += static_cast<long long>(gridDim.x) * 8) {
    const long long e0 = blk * kQBlock + lane * 8;
    const float ms = mscale[blk], vs = vscale[blk];
    float w[8], m1[8], v1[8];
    float m_max = 0.f, v_max = 0.f;
    // full block of 16-byte aligned bf16 tensors: one 16-byte access per lane for p and g, one 8-byte access for each code array
    const bool vec = sizeof(T) == 2 && (blk + 1) * kQBlock <= numel &&
                     ((reinterpret_cast<uintptr_t>(p) | reinterpret_cast<uintptr_t>(g)) & 15) == 0 &&
                     ((reinterpret_cast<uintptr_t>(mq) | reinterpret_cast<uintptr_t>(vq)) & 7) == 0;
    float pin[8], gin[8];
    int qm_in[8], qv_in[8];
    if (vec) {
      const uint4 pu = *reinterpret_cast<const uint4*>(reinterpret_cast<const __nv_bfloat16*>(p) + e0);
      const uint4 gu = *reinterpret_cast<const uint4*>(reinterpret_cast<const __nv_bfloat16*>(g) + e0);
      const uint2 mu = *reinterpret_cast<const uint2*>(mq + e0);
      const uint2 vu = *reinterpret_cast<const uint2*>(vq + e0);
      const __nv_bfloat162* p2 = reinterpret_cast<const __nv_bfloat162*>(&pu);
      const __nv_bfloat162* g2 = reinterpret_cast<const __nv_bfloat162*>(&gu);
      const uint32_t mw[2] = {mu.x, mu.y}, vw[2] = {vu.x, vu.y};
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const float2 pf = __bfloat1622float2(p2[k]), gf = __bfloat1622float2(g2[k]);
        pin[2 * k] = pf.x, pin[2 * k + 1] = pf.y, gin[2 * k] = gf.x, gin[2 * k + 1] = gf.y;
      }
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        qm_in[j] = static_cast<int>(static_cast<int8_t>((mw[j >> 2] >> (8 * (j & 3))) & 0xFFu));
        qv_in[j] = static_cast<int>((vw[j >> 2] >> (8 * (j & 3))) & 0xFFu);
      }
    } else {
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const long long e = e0 + j;
        const bool in = e < numel;
        pin[j] = in ? to_f<T>(p[e]) : 0.f;
        gin[j] = in ? to_f<T>(g[e]) : 0.f;
        qm_in[j] = in ? static_cast<int>(mq[e]) : 0;
        qv_in[j] = in ? static_cast<int>(vq[e]) : 0;
      }
    }
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      if (vec || e0 + j < numel) {
        const float grad = gin[j] * gs;
        const int qm = qm_in[j];
        const float um = static_cast<float>(qm < 0 ? -qm : qm) * (1.f / 127.f);
        const float m0 = (qm < 0 ? -ms : ms) * um * um;
        const float uv = static_cast<float>(qv_in[j]) * (1.f / 255.f);
        const float v0 = vs * (uv * uv) * (uv * uv);
        m1[j] = beta1 * m0 + (1.f - beta1) * grad;
        v1[j] = beta2 * v0 + (1.f - beta2) * grad * grad;
        w[j] = pin[j] * decay - __fdividef(lr * inv_bc1 * m1[j], fast_sqrt(v1[j]) * inv_sqrt_bc2 + eps);
        m_max = fmaxf(m_max, fabsf(m1[j]));
        v_max = fmaxf(v_max, v1[j]);
      } else {
        w[j] = m1[j] = v1[j] = 0.f;
      }
    }
    m_max = warp_max(m_max);
    v_max = warp_max(v_max);
    const float inv_m = m_max > 0.f ? 1.f / m_max : 0.f, inv_v = v_max > 0.f ? 1.f / v_max : 0.f;
    int qm_out[8], qv_out[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const int qm = __float2int_rn(127.f * fast_sqrt(fabsf(m1[j]) * inv_m));
      qm_out[j] = m1[j] < 0.f ? -qm : qm;
      qv_out[j] = __float2int_rn(255.f * fast_sqrt(fast_sqrt(v1[j] * inv_v)));
    }
    if (vec) {
      uint32_t mw[2] = {0u, 0u}, vw[2] = {0u, 0u};
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        mw[j >> 2] |= (static_cast<uint32_t>(qm_out[j]) & 0xFFu) << (8 * (j & 3));
        vw[j >> 2] |= (static_cast<uint32_t>(qv_out[j]) & 0xFFu) << (8 * (j & 3));
      }
      uint4 pu;
      __nv_bfloat162* p2 = reinterpret_cast<__nv_bfloat162*>(&pu);
#pragma unroll
      for (int k = 0; k < 4; ++k) p2[k] = __floats2bfloat162_rn(w[2 * k], w[2 * k + 1]);
      *reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(p) + e0) = pu;
      *reinterpret_cast<uint2*>(mq + e0) = make_uint2(mw[0], mw[1]);
      *reinterpret_cast<uint2*>(vq + e0) = make_uint2(vw[0], vw[1]);
    } else {
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const long long e = e0 + j;
        if (e < numel) {
          mq[e] = static_cast<int8_t>(qm_out[j]);
          vq[e] = static_cast<uint8_t>(qv_out[j]);
          p[e] = from_f<T>(w[j]);
        }
      }
    }
    if (lane == 0) mscale[blk] = m_max, vscale[blk] = v_max;
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

// p, g: numel elements (bf16 or fp32); mq int8 / vq uint8: numel codes; mscale, vscale: ceil(numel / 256) fp32 block scales.
extern "C" int ttb_adamw8bit(void* p, const void* g, void* mq, void* vq, float* mscale, float* vscale, long long numel, int is_bf16,
                             float lr, float beta1, float beta2, float eps, float weight_decay, float inv_bc1, float inv_sqrt_bc2,
                             const float* scale_dev, float scale_host, void* stream) {
  if (numel <= 0) return kOk;
  const long long n_blocks = (numel + kQBlock - 1) / kQBlock;
  const long long want = (n_blocks + 7) / 8, cap = ttb_optim_grid();
  const int grid = static_cast<int>(want < cap ? want : cap);
  auto s = static_cast<cudaStream_t>(stream);
  TTB_COUNT_LAUNCH(1);
  if (is_bf16)
    adamw8bit_kernel<__nv_bfloat16><<<grid, 256, 0, s>>>(static_cast<__nv_bfloat16*>(p), static_cast<const __nv_bfloat16*>(g), static_cast<int8_t*>(mq),
                                                        static_cast<uint8_t*>(vq), mscale, vscale, numel, lr, beta1, beta2, eps, weight_decay, inv_bc1,
                                                        inv_sqrt_bc2, scale_dev, scale_host);
  else
    adamw8bit_kernel<float><<<grid, 256, 0, s>>>(static_cast<float*>(p), static_cast<const float*>(g), static_cast<int8_t*>(mq), static_cast<uint8_t*>(vq),
                                                mscale, vscale, numel, lr, beta1, beta2, eps, weight_decay, inv_bc1, inv_sqrt_bc2, scale_dev, scale_host);
  return cudaGetLastError() == cudaSuccess ? kOk : kErrDriver;
}
