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

TTB_DEFINE_VIOLATION_COUNTER(loss)

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
// CAP: the softmax runs over z = cap · tanh(x / cap) (Gemma-2 logit soft cap) and the gradient written back is the one with
// respect to the raw logit x: (softmax(z) − onehot) · (1 − (z / cap)²).
template <bool CAP>
__global__ void __launch_bounds__(kCEThreads)
softmax_ce_kernel(__nv_bfloat16* __restrict__ logits, const long long* __restrict__ labels,
                  float* __restrict__ loss_out, const float* __restrict__ row_scale, int rows, int V, long long ld,
                  long long ignore_index, int mode, float cap, float inv_cap) {
  __shared__ float sm_m[kCEThreads / 32], sm_s[kCEThreads / 32];
  __shared__ float sh_m, sh_s;
  const int row = blockIdx.x;
  if (row >= rows) return;
  __nv_bfloat16* lr = logits + static_cast<long long>(row) * ld;
  const long long label = labels[row];
  const bool out_of_range = label != ignore_index && (label < 0 || label >= V);  // treated like an ignored row, and counted
  if (out_of_range && threadIdx.x == 0) TTB_NOTE_VIOLATION(loss);
  const bool ignored = label == ignore_index || out_of_range;
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
    if (CAP) {
#pragma unroll
      for (int j = 0; j < 8; ++j) f[j] = cap * tanhf(f[j] * inv_cap);
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
  if (threadIdx.x == 0 && loss_out != nullptr) {
    float at_label = __bfloat162float(lr[label]);
    if (CAP) at_label = cap * tanhf(at_label * inv_cap);
    loss_out[row] = lse - at_label;
  }
  if (mode == 1) return;
  __syncthreads();  // the label logit was read above, before anything is overwritten

  const float sign_scale = mode == 2 ? -row_scale[row] : 1.f;
  for (int i = threadIdx.x; i < nvec; i += kCEThreads) {
    uint4 u = reinterpret_cast<const uint4*>(lr)[i];
    __nv_bfloat162* b = reinterpret_cast<__nv_bfloat162*>(&u);
    const long long c0 = static_cast<long long>(i) * 8;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      float2 t = __bfloat1622float2(b[j]);
      float d0 = 1.f, d1 = 1.f;  // dz/dx
      if (CAP) {
        const float u0 = tanhf(t.x * inv_cap), u1 = tanhf(t.y * inv_cap);
        t.x = cap * u0, t.y = cap * u1;
        d0 = 1.f - u0 * u0, d1 = 1.f - u1 * u1;
      }
      float g0 = __expf(t.x - lse), g1 = __expf(t.y - lse);
      if (c0 + 2 * j == label) g0 -= 1.f;
      if (c0 + 2 * j + 1 == label) g1 -= 1.f;
      b[j] = __floats2bfloat162_rn(g0 * d0 * sign_scale, g1 * d1 * sign_scale);
    }
    reinterpret_cast<uint4*>(lr)[i] = u;
  }
}

// ----------------------------------------------------------------------------- distillation divergences
// Per row, with p_s = softmax(student), p_t = softmax(teacher) over V columns (fp32 math on bf16 logits):
//   forward KL term   F = −Σ p_t · log p_s          d F / d s_j = p_s(j) − p_t(j)
//   reverse KL        R =  Σ p_s · (log p_s − log p_t)   d R / d s_j = p_s(j) · ((log p_s(j) − log p_t(j)) − R)
// loss_out[row] = w_fwd · F + w_rev · R, grad[row, :] = the same combination of the two gradients (bf16; may alias nothing).
// Columns whose student logit is ±inf contribute nothing (the reference masks them, torchtune/modules/loss/kd_losses.py:54-60,
// 129-140); rows whose label equals ignore_index give loss 0 and a zero gradient row.
static constexpr int kKDThreads = 512;

__device__ __forceinline__ float kd_block_sum(float v, float* scratch) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  __syncthreads();
  if ((threadIdx.x & 31) == 0) scratch[threadIdx.x >> 5] = v;
  __syncthreads();
  float t = 0.f;
  for (int w = 0; w < kKDThreads / 32; ++w) t += scratch[w];
  return t;
}
__device__ __forceinline__ float kd_block_max(float v, float* scratch) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  __syncthreads();
  if ((threadIdx.x & 31) == 0) scratch[threadIdx.x >> 5] = v;
  __syncthreads();
  float t = -INFINITY;
  for (int w = 0; w < kKDThreads / 32; ++w) t = fmaxf(t, scratch[w]);
  return t;
}

__global__ void __launch_bounds__(kKDThreads)
kd_divergence_kernel(const __nv_bfloat16* __restrict__ student, const __nv_bfloat16* __restrict__ teacher, const long long* __restrict__ labels,
                     float* __restrict__ loss_out, __nv_bfloat16* __restrict__ grad, int rows, int V, long long ld_s, long long ld_t, long long ld_g,
                     long long ignore_index, float w_fwd, float w_rev) {
  __shared__ float scratch[kKDThreads / 32];
  const int row = blockIdx.x;
  if (row >= rows) return;
  const int nvec = V >> 3;
  const uint4* sr = reinterpret_cast<const uint4*>(student + static_cast<long long>(row) * ld_s);
  const uint4* tr = reinterpret_cast<const uint4*>(teacher + static_cast<long long>(row) * ld_t);
  uint4* gr = grad != nullptr ? reinterpret_cast<uint4*>(grad + static_cast<long long>(row) * ld_g) : nullptr;
  if (labels[row] == ignore_index) {
    if (gr != nullptr) {
      const uint4 z = make_uint4(0, 0, 0, 0);
      for (int i = threadIdx.x; i < nvec; i += kKDThreads) gr[i] = z;
    }
    if (threadIdx.x == 0) loss_out[row] = 0.f;
    return;
  }
  auto unpack = [](const uint4& u, float (&f)[8]) {
    const __nv_bfloat162* b = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 t = __bfloat1622float2(b[j]);
      f[2 * j] = t.x, f[2 * j + 1] = t.y;
    }
  };
  // pass 1: row maxima (finite values only for the student, whose ±inf columns are masked out)
  float ms = -INFINITY, mt = -INFINITY;
  for (int i = threadIdx.x; i < nvec; i += kKDThreads) {
    float a[8], b[8];
    unpack(sr[i], a);
    unpack(tr[i], b);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      if (!isinf(a[j])) ms = fmaxf(ms, a[j]);
      mt = fmaxf(mt, b[j]);
    }
  }
  ms = kd_block_max(ms, scratch);
  mt = kd_block_max(mt, scratch);
  // pass 2: partition sums and the two cross terms
  float zs = 0.f, zt = 0.f, c_fwd = 0.f, c_rev = 0.f;
  for (int i = threadIdx.x; i < nvec; i += kKDThreads) {
    float a[8], b[8];
    unpack(sr[i], a);
    unpack(tr[i], b);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float et = __expf(b[j] - mt);
      zt += et;
      if (isinf(a[j])) {
        if (a[j] > 0.f) zs = INFINITY;  // +inf student logit: the softmax is degenerate, as in the eager statement
        continue;
      }
      const float ds = a[j] - ms;
      const float es = __expf(ds);
      zs += es;
      c_fwd += et * ds;
      if (!isinf(b[j])) c_rev += es * ((b[j] - mt) - ds);
    }
  }
  zs = kd_block_sum(zs, scratch);
  zt = kd_block_sum(zt, scratch);
  c_fwd = kd_block_sum(c_fwd, scratch);
  c_rev = kd_block_sum(c_rev, scratch);
  const float log_zs = __logf(zs), log_zt = __logf(zt);
  // Σ p_t log p_s over unmasked columns needs the teacher mass on those columns; with no masked column it is exactly 1
  float pt_mass = 0.f;
  if (w_fwd != 0.f) {
    for (int i = threadIdx.x; i < nvec; i += kKDThreads) {
      float a[8], b[8];
      unpack(sr[i], a);
      unpack(tr[i], b);
#pragma unroll
      for (int j = 0; j < 8; ++j)
        if (!isinf(a[j])) pt_mass += __expf(b[j] - mt);
    }
    pt_mass = kd_block_sum(pt_mass, scratch) / zt;
  }
  const float fwd = -(c_fwd / zt - log_zs * pt_mass);          // −Σ p_t log p_s
  const float rev = -(c_rev / zs - (log_zt - log_zs));          // Σ p_s (log p_s − log p_t)
  if (threadIdx.x == 0) loss_out[row] = w_fwd * fwd + w_rev * rev;
  if (gr == nullptr) return;
  for (int i = threadIdx.x; i < nvec; i += kKDThreads) {
    float a[8], b[8], g[8];
    unpack(sr[i], a);
    unpack(tr[i], b);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      if (isinf(a[j])) {
        g[j] = 0.f;
        continue;
      }
      const float lps = a[j] - ms - log_zs, lpt = b[j] - mt - log_zt;
      const float ps = __expf(lps), pt = __expf(lpt);
      float v = w_fwd * (ps * pt_mass - pt);
      if (w_rev != 0.f) v += w_rev * ps * ((isinf(b[j]) ? 0.f : (lps - lpt)) - rev);
      g[j] = v;
    }
    uint4 u;
    __nv_bfloat162* ob = reinterpret_cast<__nv_bfloat162*>(&u);
#pragma unroll
    for (int j = 0; j < 4; ++j) ob[j] = __floats2bfloat162_rn(g[2 * j], g[2 * j + 1]);
    gr[i] = u;
  }
}

}  // namespace ttb

using namespace ttb;

extern "C" int ttb_softmax_ce(void* logits, const long long* labels, float* loss_out, const float* row_scale, int rows,
                              int V, long long ld, long long ignore_index, int mode, void* stream) {
  if ((V & 7) || (ld & 7)) return kErrBadShape;
  if (rows <= 0) return kOk;
  TTB_COUNT_LAUNCH(1);
  softmax_ce_kernel<false><<<rows, kCEThreads, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<__nv_bfloat16*>(logits), labels, loss_out, row_scale, rows, V, ld, ignore_index, mode, 0.f, 0.f);
  return cudaGetLastError() == cudaSuccess ? kOk : kErrDriver;
}

// The same with the logits soft-capped at `softcap` (> 0) before the softmax; see the kernel.
extern "C" int ttb_softmax_ce_capped(void* logits, const long long* labels, float* loss_out, const float* row_scale, int rows,
                                     int V, long long ld, long long ignore_index, int mode, float softcap, void* stream) {
  if ((V & 7) || (ld & 7) || !(softcap > 0.f)) return kErrBadShape;
  if (rows <= 0) return kOk;
  TTB_COUNT_LAUNCH(1);
  softmax_ce_kernel<true><<<rows, kCEThreads, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<__nv_bfloat16*>(logits), labels, loss_out, row_scale, rows, V, ld, ignore_index, mode, softcap, 1.f / softcap);
  return cudaGetLastError() == cudaSuccess ? kOk : kErrDriver;
}


// student, teacher: [rows, V] bf16 (row pitches ld_s / ld_t, multiples of 8); labels: [rows] int64; loss_out: [rows] fp32;
// grad: [rows, V] bf16 (pitch ld_g) or null.  loss = w_fwd · forward-KL term + w_rev · reverse KL per row (see the kernel).
extern "C" int ttb_kd_divergence(const void* student, const void* teacher, const long long* labels, float* loss_out, void* grad, int rows, int V, long long ld_s,
                                 long long ld_t, long long ld_g, long long ignore_index, float w_fwd, float w_rev, void* stream) {
  if ((V & 7) || (ld_s & 7) || (ld_t & 7) || (grad != nullptr && (ld_g & 7))) return kErrBadShape;
  if (rows <= 0) return kOk;
  TTB_COUNT_LAUNCH(1);
  kd_divergence_kernel<<<rows, kKDThreads, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(student), static_cast<const __nv_bfloat16*>(teacher), labels, loss_out, static_cast<__nv_bfloat16*>(grad), rows, V, ld_s, ld_t,
      ld_g, ignore_index, w_fwd, w_rev);
  return cudaGetLastError() == cudaSuccess ? kOk : kErrDriver;
}
