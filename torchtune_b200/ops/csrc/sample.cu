// Token sampling for generation: temperature, optional top-k, one draw per row, in one kernel launch.
//
// The reference divides the logits by the temperature, keeps the top_k largest, takes a softmax and draws with the exponential
// race argmax(p / q), q ~ Exp(1) (torchtune/generation/_generation.py:14-66).  Since p_v = exp(t_v − lse) the winner is
// argmax(t_v − log q_v) over the kept columns, so neither the softmax nor the [rows, vocab] probability tensor is needed.
// One CTA per row: a 4 × 8-bit radix select over the order-preserving integer image of t finds the top_k-th largest value
// (four histogram passes over the row, which stays in L2), one more pass takes the arg-max.  Ties go to the lowest index, as
// torch.argmax does.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "common/tmap.h"

namespace ttb {

static constexpr int kSampleThreads = 1024;

__device__ __forceinline__ uint32_t ordered_key(float f) {
  const uint32_t u = __float_as_uint(f);
  return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}

template <typename T>
__device__ __forceinline__ float scaled_logit(const T* row, int v, float temp);
// bf16 logits: the eager statement divides in bf16, so the quotient is rounded to bf16 before it is compared
template <>
__device__ __forceinline__ float scaled_logit<__nv_bfloat16>(const __nv_bfloat16* row, int v, float temp) {
  return __bfloat162float(__float2bfloat16_rn(__fdiv_rn(__bfloat162float(row[v]), temp)));
}
template <>
__device__ __forceinline__ float scaled_logit<float>(const float* row, int v, float temp) {
  return __fdiv_rn(row[v], temp);
}

template <typename T>
__global__ void __launch_bounds__(kSampleThreads)
sample_kernel(const T* __restrict__ logits, long long ld, const float* __restrict__ q, long long ldq, int* __restrict__ out, int rows, int V, float temp, int top_k) {
  __shared__ unsigned int hist[256];
  __shared__ uint32_t sh_prefix;
  __shared__ int sh_k;
  __shared__ float red_v[kSampleThreads / 32];
  __shared__ int red_i[kSampleThreads / 32];
  const int row = blockIdx.x;
  if (row >= rows) return;
  const T* lr = logits + static_cast<long long>(row) * ld;
  const float* qr = q + static_cast<long long>(row) * ldq;
  uint32_t threshold = 0;  // keep every column
  if (top_k > 0 && top_k < V) {
    if (threadIdx.x == 0) sh_prefix = 0, sh_k = top_k;
    for (int pass = 0; pass < 4; ++pass) {
      const int shift = 24 - 8 * pass;
      if (threadIdx.x < 256) hist[threadIdx.x] = 0;
      __syncthreads();
      const uint32_t prefix = sh_prefix;
      const uint32_t mask = pass == 0 ? 0u : (0xffffffffu << (shift + 8));
      for (int v = threadIdx.x; v < V; v += kSampleThreads) {
        const uint32_t key = ordered_key(scaled_logit<T>(lr, v, temp));
        if ((key & mask) == prefix) atomicAdd(&hist[(key >> shift) & 255u], 1u);
      }
      __syncthreads();
      if (threadIdx.x == 0) {
        int k = sh_k;
        int bin = 255;
        for (; bin > 0; --bin) {
          const int c = static_cast<int>(hist[bin]);
          if (c >= k) break;
          k -= c;
        }
        sh_prefix = prefix | (static_cast<uint32_t>(bin) << shift);
        sh_k = k;
      }
      __syncthreads();
    }
    threshold = sh_prefix;  // key of the top_k-th largest value
  }
  float best = -INFINITY;
  int best_i = 0x7fffffff;
  for (int v = threadIdx.x; v < V; v += kSampleThreads) {
    const float t = scaled_logit<T>(lr, v, temp);
    if (ordered_key(t) < threshold) continue;
    const float s = t - __logf(qr[v]);
    if (s > best || (s == best && v < best_i)) best = s, best_i = v;
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, best, o);
    const int oi = __shfl_xor_sync(0xffffffffu, best_i, o);
    if (ov > best || (ov == best && oi < best_i)) best = ov, best_i = oi;
  }
  if ((threadIdx.x & 31) == 0) red_v[threadIdx.x >> 5] = best, red_i[threadIdx.x >> 5] = best_i;
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int w = 1; w < kSampleThreads / 32; ++w)
      if (red_v[w] > best || (red_v[w] == best && red_i[w] < best_i)) best = red_v[w], best_i = red_i[w];
    out[row] = best_i == 0x7fffffff ? 0 : best_i;
  }
}

}  // namespace ttb

// logits: [rows, V] bf16 (is_bf16 != 0) or fp32, row pitch ld elements; q: [rows, V] fp32 draws from Exp(1), pitch ldq; out: [rows] int32.
// top_k <= 0 or >= V keeps every column.
extern "C" int ttb_sample(const void* logits, long long ld, int is_bf16, const float* q, long long ldq, int* out, int rows, int V, float temperature, int top_k,
                          void* stream) {
  using namespace ttb;
  if (rows <= 0 || V <= 0 || q == nullptr || out == nullptr) return kErrBadShape;
  const float temp = fmaxf(temperature, 1e-5f);
  TTB_COUNT_LAUNCH(1);
  auto s = static_cast<cudaStream_t>(stream);
  if (is_bf16)
    sample_kernel<__nv_bfloat16><<<rows, kSampleThreads, 0, s>>>(static_cast<const __nv_bfloat16*>(logits), ld, q, ldq, out, rows, V, temp, top_k);
  else
    sample_kernel<float><<<rows, kSampleThreads, 0, s>>>(static_cast<const float*>(logits), ld, q, ldq, out, rows, V, temp, top_k);
  return cudaGetLastError() == cudaSuccess ? kOk : kErrDriver;
}
