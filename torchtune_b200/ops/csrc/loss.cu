// Row-wise softmax cross-entropy over a chunk of logits, fused with its gradient.
//
// For each row: lse = logsumexp(logits), loss = lse - logits[label]; with `write_grad` the
// logits are overwritten in place by d(loss)/d(logits) = softmax - onehot (bf16), which the
// caller feeds straight into the dgrad/wgrad GEMMs of the output projection, so the fp32
// [tokens, vocab] tensor of the unfused path never exists.  Rows whose label equals
// ignore_index produce loss 0 and a zero gradient row.
// Reference math: torchtune/modules/loss/cross_entropy_loss.py:87-115 (logits upcast to fp32,
// summed CE) and torchtune/rlhf/sequence_processing.py:138-178 (per-token log-probs).
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "common/tmap.h"

namespace ttb {

static constexpr int kCEThreads = 512;

// Merge two (max, sum-of-exp) partials; a partial that saw no element has s == 0 and is skipped
// (its max is -inf and must not enter an inf - inf subtraction).
__device__ __forceinline__ void online_merge(float& m, float& s, float m2, float s2) {
  if (s2 == 0.f) return;
  if (s == 0.f) {
    m = m2, s = s2;
    return;
  }
  const float nm = fmaxf(m, m2);
  s = s * __expf(m - nm) + s2 * __expf(m2 - nm);
  m = nm;
}

// mode 0: loss + in-place gradient;  mode 1: loss only;  mode 2: in-place gradient scaled by
// row_scale[row] of the *negative* loss (i.e. gradient of log p(label)), for DPO backward.
__global__ void __launch_bounds__(kCEThreads)
softmax_ce_kernel(__nv_bfloat16* __restrict__ logits, const long long* __restrict__ labels,
                  float* __restrict__ loss_out, const float* __restrict__ row_scale, int rows, int V, long long ld,
                  long long ignore_index, int mode) {
  __shared__ float sm_m[kCEThreads / 32], sm_s[kCEThreads / 32];
  __shared__ float sh_m, sh_s;
  const int row = blockIdx.x;
  if (row >= rows) return;
  __nv_bfloat16* lr = logits + static_cast<long long>(row) * ld;
  const long long label = labels[row];
  const bool ignored = label == ignore_index;
  const int nvec = V >> 3;

  if (ignored) {
    if (mode != 1) {
      const uint4 z = make_uint4(0, 0, 0, 0);
      for (int i = threadIdx.x; i < nvec; i += kCEThreads) reinterpret_cast<uint4*>(lr)[i] = z;
    }
    if (threadIdx.x == 0 && loss_out != nullptr) loss_out[row] = 0.f;
    return;
  }

  float m = -INFINITY, s = 0.f;
  for (int i = threadIdx.x; i < nvec; i += kCEThreads) {
    const uint4 u = reinterpret_cast<const uint4*>(lr)[i];
    const __nv_bfloat162* b = reinterpret_cast<const __nv_bfloat162*>(&u);
    float f[8];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 t = __bfloat1622float2(b[j]);
      f[2 * j] = t.x, f[2 * j + 1] = t.y;
    }
    float lm = f[0];
#pragma unroll
    for (int j = 1; j < 8; ++j) lm = fmaxf(lm, f[j]);
    float ls = 0.f;
#pragma unroll
    for (int j = 0; j < 8; ++j) ls += __expf(f[j] - lm);
    online_merge(m, s, lm, ls);
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float m2 = __shfl_xor_sync(0xffffffffu, m, o);
    const float s2 = __shfl_xor_sync(0xffffffffu, s, o);
    online_merge(m, s, m2, s2);
  }
  if ((threadIdx.x & 31) == 0) sm_m[threadIdx.x >> 5] = m, sm_s[threadIdx.x >> 5] = s;
  __syncthreads();
  if (threadIdx.x == 0) {
    float tm = sm_m[0], ts = sm_s[0];
    for (int w = 1; w < kCEThreads / 32; ++w) online_merge(tm, ts, sm_m[w], sm_s[w]);
    sh_m = tm, sh_s = ts;
  }
  __syncthreads();
  const float row_max = sh_m;
  const float lse = row_max + __logf(sh_s);
  if (threadIdx.x == 0 && loss_out != nullptr) loss_out[row] = lse - __bfloat162float(lr[label]);
  if (mode == 1) return;
  __syncthreads();  // the label logit was read above, before anything is overwritten

  const float sign_scale = mode == 2 ? -row_scale[row] : 1.f;
  for (int i = threadIdx.x; i < nvec; i += kCEThreads) {
    uint4 u = reinterpret_cast<const uint4*>(lr)[i];
    __nv_bfloat162* b = reinterpret_cast<__nv_bfloat162*>(&u);
    const long long c0 = static_cast<long long>(i) * 8;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 t = __bfloat1622float2(b[j]);
      float g0 = __expf(t.x - lse), g1 = __expf(t.y - lse);
      if (c0 + 2 * j == label) g0 -= 1.f;
      if (c0 + 2 * j + 1 == label) g1 -= 1.f;
      b[j] = __floats2bfloat162_rn(g0 * sign_scale, g1 * sign_scale);
    }
    reinterpret_cast<uint4*>(lr)[i] = u;
  }
}

}  // namespace ttb

using namespace ttb;

extern "C" int ttb_softmax_ce(void* logits, const long long* labels, float* loss_out, const float* row_scale, int rows,
                              int V, long long ld, long long ignore_index, int mode, void* stream) {
  if ((V & 7) || (ld & 7)) return kErrBadShape;
  if (rows <= 0) return kOk;
  TTB_COUNT_LAUNCH(1);
  softmax_ce_kernel<<<rows, kCEThreads, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<__nv_bfloat16*>(logits), labels, loss_out, row_scale, rows, V, ld, ignore_index, mode);
  return cudaGetLastError() == cudaSuccess ? kOk : kErrDriver;
}
