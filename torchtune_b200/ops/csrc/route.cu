// Mixture-of-experts routing and row movement on one GPU.
//
// 1. `ttb_moe_route`: gate logits → sigmoid scores → top-k experts per token, one warp per token (reference: the router's
//    sigmoid + topk pair, torchtune/modules/moe/moe.py:55-84).  Scores are rounded to bf16 before the selection, as the eager
//    statement does when the activations are bf16; ties go to the lower expert index.
//    `ttb_moe_route_bwd`: gradient of the selected scores back to the logits (sigmoid derivative on the k selected entries of
//    each row, zero elsewhere).
// 2. `ttb_moe_gather_rows`: out[j, :] = x[idx[j], :] (· scale[j]) — the token permute in front of the experts, fused with the
//    multiplication by the router score (Llama-4 scales the expert *input*).
// 3. `ttb_moe_combine_rows`: out[t, :] = base[t, :] + Σ_s src[inv[t·k + s], :] (· scale[inv[…]]) — the un-permute + sum behind
//    the experts without atomics: `inv` is the inverse of the expert sort (position of pair (t, s) in expert order), so every
//    output row pulls its k source rows.  The same kernel is the gradient of (2) with respect to x.
// 4. `ttb_moe_row_dots`: out[j] = Σ_d a[idx[j], d] · b[j, d] — the gradient of the scores in (2).
// All row kernels move 16 bytes per thread and accumulate in fp32.
#include "common/ptx.cuh"
#include "common/tmap.h"

namespace ttb {

static constexpr int kRouteMaxExperts = 256;
static constexpr int kRouteMaxK = 8;

__device__ __forceinline__ float bf16_round(float x) { return __bfloat162float(__float2bfloat16_rn(x)); }

// logits: [T, E] bf16 or fp32 (row pitch E); scores_out: [T, k] bf16; selected: [T, k] int64.
template <typename LogitT>
__global__ void __launch_bounds__(256)
moe_route_kernel(const LogitT* __restrict__ logits, long long T, int E, int k, __nv_bfloat16* __restrict__ scores_out,
                 long long* __restrict__ selected) {
  const int lane = threadIdx.x & 31;
  const long long warp = (blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x) >> 5;
  const long long nwarps = (gridDim.x * static_cast<long long>(blockDim.x)) >> 5;
  constexpr int kPer = kRouteMaxExperts / 32;
  for (long long t = warp; t < T; t += nwarps) {
    float val[kPer];
#pragma unroll
    for (int i = 0; i < kPer; ++i) {
      const int e = lane + 32 * i;
      val[i] = -1.f;  // sigmoid scores are positive: -1 marks "no expert" / "already taken"
      if (e < E) {
        const float z = static_cast<float>(logits[t * E + e]);
        val[i] = bf16_round(1.f / (1.f + __expf(-z)));
      }
    }
    for (int s = 0; s < k; ++s) {
      float best = -1.f;
      int best_e = kRouteMaxExperts;
#pragma unroll
      for (int i = 0; i < kPer; ++i) {
        if (val[i] > best) best = val[i], best_e = lane + 32 * i;
      }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        const float ob = __shfl_xor_sync(0xffffffffu, best, o);
        const int oe = __shfl_xor_sync(0xffffffffu, best_e, o);
        if (ob > best || (ob == best && oe < best_e)) best = ob, best_e = oe;
      }
      if (lane == 0) {
        scores_out[t * k + s] = __float2bfloat16_rn(best);
        selected[t * k + s] = best_e;
      }
#pragma unroll
      for (int i = 0; i < kPer; ++i)
        if (lane + 32 * i == best_e) val[i] = -1.f;
    }
  }
}

// dlogits[t, e] = dscore[t, s] · σ(z)(1 − σ(z)) for e = selected[t, s], 0 elsewhere (bf16 or fp32 like the logits).
template <typename LogitT>
__global__ void __launch_bounds__(256)
moe_route_bwd_kernel(const LogitT* __restrict__ logits, const long long* __restrict__ selected, const __nv_bfloat16* __restrict__ dscores,
                     long long T, int E, int k, LogitT* __restrict__ dlogits) {
  const long long n = T * E;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n; i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long t = i / E;
    const int e = static_cast<int>(i - t * E);
    float g = 0.f;
    for (int s = 0; s < k; ++s) {
      if (selected[t * k + s] == e) {
        const float sg = 1.f / (1.f + __expf(-static_cast<float>(logits[i])));
        g += __bfloat162float(dscores[t * k + s]) * sg * (1.f - sg);
      }
    }
    dlogits[i] = static_cast<LogitT>(g);
  }
}

__device__ __forceinline__ void unpack8r(const uint4& u, float (&f)[8]) {
  const __nv_bfloat162* b = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 t = __bfloat1622float2(b[i]);
    f[2 * i] = t.x, f[2 * i + 1] = t.y;
  }
}
__device__ __forceinline__ uint4 pack8r(const float (&f)[8]) {
  uint4 u;
  u.x = pack_bf16x2(f[0], f[1]), u.y = pack_bf16x2(f[2], f[3]), u.z = pack_bf16x2(f[4], f[5]), u.w = pack_bf16x2(f[6], f[7]);
  return u;
}

// out[j, :] = x[idx[j], :] (· scale[j]); rows with idx out of [0, rows_x) are written as zero.
__global__ void __launch_bounds__(256)
moe_gather_rows_kernel(const uint4* __restrict__ x, const long long* __restrict__ idx, const __nv_bfloat16* __restrict__ scale, uint4* __restrict__ out,
                       long long P, int vec_per_row, long long rows_x) {
  const long long total = P * vec_per_row;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total; i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long j = i / vec_per_row;
    const int c = static_cast<int>(i - j * vec_per_row);
    const long long r = idx[j];
    uint4 v = make_uint4(0u, 0u, 0u, 0u);
    if (r >= 0 && r < rows_x) {
      v = __ldg(x + r * vec_per_row + c);
      if (scale != nullptr) {
        float f[8];
        unpack8r(v, f);
        const float s = __bfloat162float(scale[j]);
#pragma unroll
        for (int q = 0; q < 8; ++q) f[q] *= s;
        v = pack8r(f);
      }
    }
    out[i] = v;
  }
}

// out[t, :] = base[t, :] + Σ_{s < k} src[inv[t·k + s], :] (· scale[inv[t·k + s]]); entries of inv outside [0, rows_src) are skipped.
__global__ void __launch_bounds__(256)
moe_combine_rows_kernel(const uint4* __restrict__ src, const long long* __restrict__ inv, const __nv_bfloat16* __restrict__ scale, const uint4* __restrict__ base,
                        uint4* __restrict__ out, long long T, int k, int vec_per_row, long long rows_src) {
  const long long total = T * vec_per_row;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total; i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long t = i / vec_per_row;
    const int c = static_cast<int>(i - t * vec_per_row);
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    if (base != nullptr) unpack8r(__ldg(base + i), acc);
    for (int s = 0; s < k; ++s) {
      const long long j = inv[t * k + s];
      if (j < 0 || j >= rows_src) continue;
      float f[8];
      unpack8r(__ldg(src + j * vec_per_row + c), f);
      const float w = scale != nullptr ? __bfloat162float(scale[j]) : 1.f;
#pragma unroll
      for (int q = 0; q < 8; ++q) acc[q] += f[q] * w;
    }
    out[i] = pack8r(acc);
  }
}

// out[j] = Σ_d a[idx[j], d] · b[j, d]; one warp per row.
__global__ void __launch_bounds__(256)
moe_row_dots_kernel(const uint4* __restrict__ a, const long long* __restrict__ idx, const uint4* __restrict__ b, __nv_bfloat16* __restrict__ out, long long P,
                    int vec_per_row, long long rows_a) {
  const int lane = threadIdx.x & 31;
  const long long warp = (blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x) >> 5;
  const long long nwarps = (gridDim.x * static_cast<long long>(blockDim.x)) >> 5;
  for (long long j = warp; j < P; j += nwarps) {
    const long long r = idx[j];
    float acc = 0.f;
    if (r >= 0 && r < rows_a) {
      for (int c = lane; c < vec_per_row; c += 32) {
        float fa[8], fb[8];
        unpack8r(__ldg(a + r * vec_per_row + c), fa);
        unpack8r(__ldg(b + j * vec_per_row + c), fb);
#pragma unroll
        for (int q = 0; q < 8; ++q) acc += fa[q] * fb[q];
      }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
    if (lane == 0) out[j] = __float2bfloat16_rn(acc);
  }
}

static int row_grid(long long work_items) {
  long long blocks = (work_items + 255) / 256;
  const long long cap = static_cast<long long>(sm_count()) * 8;
  return static_cast<int>(blocks < 1 ? 1 : (blocks > cap ? cap : blocks));
}

}  // namespace ttb

using namespace ttb;

// logits [T, E] (fp32 when logits_fp32 != 0, else bf16) → scores [T, k] bf16, selected [T, k] int64.  E ≤ 256, k ≤ 8, k ≤ E.
extern "C" int ttb_moe_route(const void* logits, int logits_fp32, long long T, int E, int k, void* scores, void* selected, void* stream) {
  if (T <= 0 || E <= 0 || E > kRouteMaxExperts || k <= 0 || k > kRouteMaxK || k > E) return kErrBadShape;
  auto s = static_cast<cudaStream_t>(stream);
  const int grid = row_grid(T * 32);
  TTB_COUNT_LAUNCH(1);
  if (logits_fp32)
    moe_route_kernel<float><<<grid, 256, 0, s>>>(static_cast<const float*>(logits), T, E, k, static_cast<__nv_bfloat16*>(scores), static_cast<long long*>(selected));
  else
    moe_route_kernel<__nv_bfloat16><<<grid, 256, 0, s>>>(static_cast<const __nv_bfloat16*>(logits), T, E, k, static_cast<__nv_bfloat16*>(scores), static_cast<long long*>(selected));
  return cudaGetLastError() == cudaSuccess ? kOk : kErrDriver;
}

extern "C" int ttb_moe_route_bwd(const void* logits, int logits_fp32, const void* selected, const void* dscores, long long T, int E, int k, void* dlogits, void* stream) {
  if (T <= 0 || E <= 0 || E > kRouteMaxExperts || k <= 0 || k > kRouteMaxK) return kErrBadShape;
  auto s = static_cast<cudaStream_t>(stream);
  const int grid = row_grid(T * E);
  TTB_COUNT_LAUNCH(1);
  if (logits_fp32)
    moe_route_bwd_kernel<float><<<grid, 256, 0, s>>>(static_cast<const float*>(logits), static_cast<const long long*>(selected), static_cast<const __nv_bfloat16*>(dscores), T, E, k,
                                                     static_cast<float*>(dlogits));
  else
    moe_route_bwd_kernel<__nv_bfloat16><<<grid, 256, 0, s>>>(static_cast<const __nv_bfloat16*>(logits), static_cast<const long long*>(selected),
                                                             static_cast<const __nv_bfloat16*>(dscores), T, E, k, static_cast<__nv_bfloat16*>(dlogits));
  return cudaGetLastError() == cudaSuccess ? kOk : kErrDriver;
}

// x [rows_x, D] bf16, idx [P] int64, scale [P] bf16 or null → out [P, D] bf16.  D a multiple of 8, pointers 16-byte aligned.
extern "C" int ttb_moe_gather_rows(const void* x, const void* idx, const void* scale, void* out, long long P, int D, long long rows_x, void* stream) {
  if (P <= 0 || D <= 0 || (D & 7) || rows_x <= 0) return kErrBadShape;
  if ((reinterpret_cast<uintptr_t>(x) & 15) || (reinterpret_cast<uintptr_t>(out) & 15)) return kErrBadShape;
  TTB_COUNT_LAUNCH(1);
  moe_gather_rows_kernel<<<row_grid(P * (D / 8)), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const uint4*>(x), static_cast<const long long*>(idx), static_cast<const __nv_bfloat16*>(scale), static_cast<uint4*>(out), P, D / 8, rows_x);
  return cudaGetLastError() == cudaSuccess ? kOk : kErrDriver;
}

// src [rows_src, D] bf16, inv [T, k] int64, scale [rows_src] bf16 or null, base [T, D] bf16 or null → out [T, D] bf16 (may alias base).
extern "C" int ttb_moe_combine_rows(const void* src, const void* inv, const void* scale, const void* base, void* out, long long T, int k, int D, long long rows_src,
                                    void* stream) {
  if (T <= 0 || k <= 0 || D <= 0 || (D & 7) || rows_src < 0) return kErrBadShape;
  if ((reinterpret_cast<uintptr_t>(src) & 15) || (reinterpret_cast<uintptr_t>(out) & 15) || (reinterpret_cast<uintptr_t>(base) & 15)) return kErrBadShape;
  TTB_COUNT_LAUNCH(1);
  moe_combine_rows_kernel<<<row_grid(T * (D / 8)), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const uint4*>(src), static_cast<const long long*>(inv), static_cast<const __nv_bfloat16*>(scale), static_cast<const uint4*>(base), static_cast<uint4*>(out), T, k,
      D / 8, rows_src);
  return cudaGetLastError() == cudaSuccess ? kOk : kErrDriver;
}

// a [rows_a, D] bf16, idx [P] int64, b [P, D] bf16 → out [P] bf16.
extern "C" int ttb_moe_row_dots(const void* a, const void* idx, const void* b, void* out, long long P, int D, long long rows_a, void* stream) {
  if (P <= 0 || D <= 0 || (D & 7) || rows_a <= 0) return kErrBadShape;
  if ((reinterpret_cast<uintptr_t>(a) & 15) || (reinterpret_cast<uintptr_t>(b) & 15)) return kErrBadShape;
  TTB_COUNT_LAUNCH(1);
  moe_row_dots_kernel<<<row_grid(P * 32), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const uint4*>(a), static_cast<const long long*>(idx), static_cast<const uint4*>(b), static_cast<__nv_bfloat16*>(out), P, D / 8, rows_a);
  return cudaGetLastError() == cudaSuccess ? kOk : kErrDriver;
}
