// Memory-bound operators: RMSNorm fwd/bwd, RoPE (interleaved and half-split, fwd and
// inverse), SwiGLU fwd/bwd.  All use 16-byte vector accesses and fp32 math.
// Reference math: torchtune/modules/rms_norm.py:28-60,
// torchtune/modules/position_embeddings.py:69-122, torchtune/modules/feed_forward.py:50-53.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "common/tmap.h"

TTB_DEFINE_VIOLATION_COUNTER(rope)

namespace ttb {

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

template <int THREADS>
__device__ __forceinline__ float block_sum(float v, float* scratch) {
  v = warp_sum(v);
  const int w = threadIdx.x >> 5, l = threadIdx.x & 31;
  __syncthreads();
  if (l == 0) scratch[w] = v;
  __syncthreads();
  float t = (threadIdx.x < THREADS / 32) ? scratch[threadIdx.x] : 0.f;
  if (w == 0) {
    t = warp_sum(t);
    if (l == 0) scratch[0] = t;
  }
  __syncthreads();
  return scratch[0];
}

__device__ __forceinline__ void unpack8(const uint4& u, float (&f)[8]) {
  const __nv_bfloat162* b = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 t = __bfloat1622float2(b[i]);
    f[2 * i] = t.x, f[2 * i + 1] = t.y;
  }
}
__device__ __forceinline__ uint4 pack8(const float (&f)[8]) {
  uint4 u;
  __nv_bfloat162* b = reinterpret_cast<__nv_bfloat162*>(&u);
#pragma unroll
  for (int i = 0; i < 4; ++i) b[i] = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
  return u;
}

// ------------------------------------------------------------------------------- RMSNorm
// One warp per row.  y = bf16(x * rstd) * scale  (the cast before the scale multiply follows
// the reference: normalise in fp32, cast back, then multiply by the bf16 scale).
__global__ void rmsnorm_fwd_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ scale,
                                   __nv_bfloat16* __restrict__ y, float* __restrict__ rstd_out, int rows, int D,
                                   float eps) {
  const int row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (row >= rows) return;
  const int lane = threadIdx.x & 31;
  const uint4* xr = reinterpret_cast<const uint4*>(x + static_cast<long long>(row) * D);
  const int nvec = D >> 3;
  float ss = 0.f;
  for (int i = lane; i < nvec; i += 32) {
    float f[8];
    unpack8(__ldg(xr + i), f);
#pragma unroll
    for (int j = 0; j < 8; ++j) ss += f[j] * f[j];
  }
  ss = warp_sum(ss);
  const float rstd = rsqrtf(ss / D + eps);
  if (lane == 0 && rstd_out != nullptr) rstd_out[row] = rstd;
  uint4* yr = reinterpret_cast<uint4*>(y + static_cast<long long>(row) * D);
  const uint4* sr = reinterpret_cast<const uint4*>(scale);
  for (int i = lane; i < nvec; i += 32) {
    float f[8], s[8];
    unpack8(xr[i], f);
#pragma unroll
    for (int j = 0; j < 8; ++j) f[j] = __bfloat162float(__float2bfloat16_rn(f[j] * rstd));
    if (scale != nullptr) {
      unpack8(__ldg(sr + i), s);
#pragma unroll
      for (int j = 0; j < 8; ++j) f[j] *= s[j];
    }
    yr[i] = pack8(f);
  }
}

// One CTA per row for model-width rows (D >= 1024): every thread loads its MAXV 16-byte pieces up front (all loads in
// flight at once) and keeps them in registers between the sum of squares and the scaling, so x is read once.
template <int THREADS, int MAXV>
__global__ void __launch_bounds__(THREADS)
rmsnorm_fwd_row_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ scale,
                       __nv_bfloat16* __restrict__ y, float* __restrict__ rstd_out, int rows, int D, float eps) {
  __shared__ float scratch[32];
  const int row = blockIdx.x;
  const int nvec = D >> 3;
  const uint4* xr = reinterpret_cast<const uint4*>(x + static_cast<long long>(row) * D);
  uint4 v[MAXV];
#pragma unroll
  for (int k = 0; k < MAXV; ++k) {
    const int i = threadIdx.x + k * THREADS;
    v[k] = i < nvec ? __ldg(xr + i) : make_uint4(0u, 0u, 0u, 0u);
  }
  float ss = 0.f;
#pragma unroll
  for (int k = 0; k < MAXV; ++k) {
    float f[8];
    unpack8(v[k], f);
#pragma unroll
    for (int j = 0; j < 8; ++j) ss += f[j] * f[j];
  }
  ss = block_sum<THREADS>(ss, scratch);
  const float rstd = rsqrtf(ss / D + eps);
  if (threadIdx.x == 0 && rstd_out != nullptr) rstd_out[row] = rstd;
  uint4* yr = reinterpret_cast<uint4*>(y + static_cast<long long>(row) * D);
  const uint4* sr = reinterpret_cast<const uint4*>(scale);
#pragma unroll
  for (int k = 0; k < MAXV; ++k) {
    const int i = threadIdx.x + k * THREADS;
    if (i < nvec) {
      float f[8], s[8];
      unpack8(v[k], f);
#pragma unroll
      for (int j = 0; j < 8; ++j) f[j] = __bfloat162float(__float2bfloat16_rn(f[j] * rstd));
      if (scale != nullptr) {
        unpack8(__ldg(sr + i), s);
#pragma unroll
        for (int j = 0; j < 8; ++j) f[j] *= s[j];
      }
      yr[i] = pack8(f);
    }
  }
}

// Backward: dx = rstd * (g - xhat * mean(g * xhat)),  g = dy * scale,  xhat = x * rstd
//           dscale_partial[cta, :] = sum over the CTA's rows of dy * xhat
// One CTA (256 threads) walks rows blockIdx.x, +gridDim.x, ...; thread t owns columns
// {8*(t + 256*j)}; the per-column partial sums stay in registers until the end.
template <int MAXV>
__global__ void __launch_bounds__(256)
rmsnorm_bwd_kernel(const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ x,
                   const __nv_bfloat16* __restrict__ scale, const float* __restrict__ rstd,
                   __nv_bfloat16* __restrict__ dx, float* __restrict__ dscale_partial, int rows, int D) {
  __shared__ float scratch[32];
  const int nvec = D >> 3;
  float acc[MAXV][8];
#pragma unroll
  for (int v = 0; v < MAXV; ++v)
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[v][j] = 0.f;

  // The loads of the next row are issued before the reduction and the stores of the current one (for up to two pieces per
  // thread; wider rows would spill), so a CTA always has a row in flight.
  constexpr bool kPrefetch = MAXV <= 2;
  uint4 ndy[MAXV], nx[MAXV];
  float nrs = 0.f;
  auto fetch = [&](int r) {
    const uint4* dyr = reinterpret_cast<const uint4*>(dy + static_cast<long long>(r) * D);
    const uint4* xr = reinterpret_cast<const uint4*>(x + static_cast<long long>(r) * D);
#pragma unroll
    for (int v = 0; v < MAXV; ++v) {
      const int i = threadIdx.x + v * 256;
      if (i < nvec) {
        ndy[v] = __ldg(dyr + i);
        nx[v] = __ldg(xr + i);
      }
    }
    nrs = rstd[r];
  };
  if (kPrefetch && static_cast<int>(blockIdx.x) < rows) fetch(blockIdx.x);

  for (int row = blockIdx.x; row < rows; row += gridDim.x) {
    if (!kPrefetch) fetch(row);
    uint4 cdy[MAXV], cx[MAXV];
#pragma unroll
    for (int v = 0; v < MAXV; ++v) cdy[v] = ndy[v], cx[v] = nx[v];
    const float rs = nrs;
    if (kPrefetch && row + static_cast<int>(gridDim.x) < rows) fetch(row + gridDim.x);
    float g[MAXV][8], xh[MAXV][8];
    float dot = 0.f;
#pragma unroll
    for (int v = 0; v < MAXV; ++v) {
      const int i = threadIdx.x + v * 256;
      if (i < nvec) {
        float a[8], b[8], s[8];
        unpack8(cdy[v], a);
        unpack8(cx[v], b);
        if (scale != nullptr) unpack8(__ldg(reinterpret_cast<const uint4*>(scale) + i), s);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          xh[v][j] = b[j] * rs;
          acc[v][j] += a[j] * xh[v][j];
          g[v][j] = scale != nullptr ? a[j] * s[j] : a[j];
          dot += g[v][j] * xh[v][j];
        }
      }
    }
    dot = block_sum<256>(dot, scratch) / D;
    uint4* dxr = reinterpret_cast<uint4*>(dx + static_cast<long long>(row) * D);
#pragma unroll
    for (int v = 0; v < MAXV; ++v) {
      const int i = threadIdx.x + v * 256;
      if (i < nvec) {
        float o[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) o[j] = rs * (g[v][j] - xh[v][j] * dot);
        dxr[i] = pack8(o);
      }
    }
  }
  if (dscale_partial != nullptr) {
    float* out = dscale_partial + static_cast<long long>(blockIdx.x) * D;
#pragma unroll
    for (int v = 0; v < MAXV; ++v) {
      const int i = threadIdx.x + v * 256;
      if (i < nvec) {
#pragma unroll
        for (int j = 0; j < 8; ++j) out[i * 8 + j] = acc[v][j];
      }
    }
  }
}

// ------------------------------------------------------------------------------- RoPE
// x, y: [tokens, heads, d] bf16 (tokens = b*s); cache: [max_seq, d/2, 2] fp32 (cos, sin);
// pos: [tokens] int32 or nullptr (then position = token % seq_len).  inverse rotates by -angle.
template <bool INTERLEAVED>
__global__ void rope_kernel(const __nv_bfloat16* __restrict__ x, __nv_bfloat16* __restrict__ y,
                            const float* __restrict__ cache, const int* __restrict__ pos, long long tokens, int heads,
                            int d, int seq_len, int inverse, int cache_len) {
  // one thread handles 8 consecutive elements (interleaved) or 4+4 mirrored elements (half split)
  const int per_head = INTERLEAVED ? d / 8 : d / 16;
  const long long total = tokens * heads * per_head;
  for (long long idx = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; idx < total;
       idx += static_cast<long long>(gridDim.x) * blockDim.x) {
    const int v = static_cast<int>(idx % per_head);
    const long long th = idx / per_head;
    const long long tok = th / heads;
    int p = pos != nullptr ? pos[tok] : static_cast<int>(tok % seq_len);
    if (p < 0 || p >= cache_len) {  // a position the cache does not hold: position 0 stands in and the event is counted
      if (v == 0 && th % heads == 0) TTB_NOTE_VIOLATION(rope);
      p = 0;
    }
    const float* c = cache + static_cast<long long>(p) * d;  // (d/2) * 2 floats per position
    const __nv_bfloat16* xp = x + th * d;
    __nv_bfloat16* yp = y + th * d;
    if (INTERLEAVED) {
      float f[8], o[8];
      unpack8(*reinterpret_cast<const uint4*>(xp + v * 8), f);
      const float4 cs0 = *reinterpret_cast<const float4*>(c + v * 8);
      const float4 cs1 = *reinterpret_cast<const float4*>(c + v * 8 + 4);
      const float cosv[4] = {cs0.x, cs0.z, cs1.x, cs1.z};
      float sinv[4] = {cs0.y, cs0.w, cs1.y, cs1.w};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float sn = inverse ? -sinv[j] : sinv[j];
        o[2 * j] = f[2 * j] * cosv[j] - f[2 * j + 1] * sn;
        o[2 * j + 1] = f[2 * j + 1] * cosv[j] + f[2 * j] * sn;
      }
      *reinterpret_cast<uint4*>(yp + v * 8) = pack8(o);
    } else {
      // elements [8v, 8v+8) of the first half pair with the same offsets in the second half
      float a[8], b[8], oa[8], ob[8];
      unpack8(*reinterpret_cast<const uint4*>(xp + v * 8), a);
      unpack8(*reinterpret_cast<const uint4*>(xp + d / 2 + v * 8), b);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const float cs = c[(v * 8 + j) * 2];
        const float sn = inverse ? -c[(v * 8 + j) * 2 + 1] : c[(v * 8 + j) * 2 + 1];
        oa[j] = a[j] * cs - b[j] * sn;
        ob[j] = b[j] * cs + a[j] * sn;
      }
      *reinterpret_cast<uint4*>(yp + v * 8) = pack8(oa);
      *reinterpret_cast<uint4*>(yp + d / 2 + v * 8) = pack8(ob);
    }
  }
}

// ------------------------------------------------------------------------------- SwiGLU
// gate/up may be two halves of one [rows, 2H] buffer: row strides are explicit.
__global__ void swiglu_fwd_kernel(const __nv_bfloat16* __restrict__ g, const __nv_bfloat16* __restrict__ u,
                                  __nv_bfloat16* __restrict__ y, long long rows, int H, long long ldg, long long ldu,
                                  long long ldy) {
  const int hv = H >> 3;
  const long long total = rows * hv;
  for (long long idx = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; idx < total;
       idx += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long r = idx / hv;
    const int c = static_cast<int>(idx % hv) * 8;
    float a[8], b[8], o[8];
    unpack8(*reinterpret_cast<const uint4*>(g + r * ldg + c), a);
    unpack8(*reinterpret_cast<const uint4*>(u + r * ldu + c), b);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      // silu rounded to bf16 before the product, as the unfused bf16 reference does
      const float s = __bfloat162float(__float2bfloat16_rn(a[j] / (1.f + __expf(-a[j]))));
      o[j] = s * b[j];
    }
    *reinterpret_cast<uint4*>(y + r * ldy + c) = pack8(o);
  }
}

__global__ void swiglu_bwd_kernel(const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ g,
                                  const __nv_bfloat16* __restrict__ u, __nv_bfloat16* __restrict__ dg,
                                  __nv_bfloat16* __restrict__ du, long long rows, int H, long long lddy, long long ldg,
                                  long long ldu, long long lddg, long long lddu) {
  const int hv = H >> 3;
  const long long total = rows * hv;
  for (long long idx = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; idx < total;
       idx += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long r = idx / hv;
    const int c = static_cast<int>(idx % hv) * 8;
    float d[8], a[8], b[8], oa[8], ob[8];
    unpack8(*reinterpret_cast<const uint4*>(dy + r * lddy + c), d);
    unpack8(*reinterpret_cast<const uint4*>(g + r * ldg + c), a);
    unpack8(*reinterpret_cast<const uint4*>(u + r * ldu + c), b);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float sig = 1.f / (1.f + __expf(-a[j]));
      const float silu = a[j] * sig;
      oa[j] = d[j] * b[j] * (sig + silu * (1.f - sig));
      ob[j] = d[j] * silu;
    }
    *reinterpret_cast<uint4*>(dg + r * lddg + c) = pack8(oa);
    *reinterpret_cast<uint4*>(du + r * lddu + c) = pack8(ob);
  }
}

static inline int grid_for(long long work_items, int threads) {
  long long blocks = (work_items + threads - 1) / threads;
  const long long cap = static_cast<long long>(sm_count()) * 16;
  return static_cast<int>(blocks < 1 ? 1 : (blocks > cap ? cap : blocks));
}

}  // namespace ttb

using namespace ttb;

long long ttb_launch_counter = 0;
extern "C" long long ttb_launch_count() { return ttb_launch_counter; }

// The library links its own CUDA runtime, whose notion of "current device" is per thread and
// independent of the caller's; every launch path calls this first with the caller's device.
extern "C" int ttb_ensure_device(int device) {
  static thread_local int bound = -1;
  if (bound != device) {
    if (cudaSetDevice(device) != cudaSuccess) return kErrDriver;
    bound = device;
  }
  return kOk;
}

extern "C" int ttb_rmsnorm_fwd(const void* x, const void* scale, void* y, float* rstd, int rows, int D, float eps,
                               void* stream) {
  if (D & 7) return kErrBadShape;
  const int warps = 4;
  TTB_COUNT_LAUNCH(1);
  const int nvec_fwd = D >> 3;
  if (nvec_fwd >= 128 && nvec_fwd <= 2048) {
    auto st = static_cast<cudaStream_t>(stream);
    auto xp = static_cast<const __nv_bfloat16*>(x);
    auto sp = static_cast<const __nv_bfloat16*>(scale);
    auto yp = static_cast<__nv_bfloat16*>(y);
    if (nvec_fwd <= 256) rmsnorm_fwd_row_kernel<128, 2><<<rows, 128, 0, st>>>(xp, sp, yp, rstd, rows, D, eps);
    else if (nvec_fwd <= 512) rmsnorm_fwd_row_kernel<128, 4><<<rows, 128, 0, st>>>(xp, sp, yp, rstd, rows, D, eps);
    else if (nvec_fwd <= 1024) rmsnorm_fwd_row_kernel<256, 4><<<rows, 256, 0, st>>>(xp, sp, yp, rstd, rows, D, eps);
    else rmsnorm_fwd_row_kernel<256, 8><<<rows, 256, 0, st>>>(xp, sp, yp, rstd, rows, D, eps);
    return cudaGetLastError() == cudaSuccess ? kOk : kErrDriver;
  }
  rmsnorm_fwd_kernel<<<(rows + warps - 1) / warps, warps * 32, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(x), static_cast<const __nv_bfloat16*>(scale), static_cast<__nv_bfloat16*>(y),
      rstd, rows, D, eps);
  return cudaGetLastError() == cudaSuccess ? kOk : kErrDriver;
}

// dscale_partial: [*n_partials_out rows, D] fp32, caller sums over dim 0.  The caller sizes it
// with ttb_rmsnorm_bwd_partials().
extern "C" int ttb_rmsnorm_bwd_partials(int rows) {
  const int cap = sm_count() * 4;
  return rows < cap ? rows : cap;
}
extern "C" int ttb_rmsnorm_bwd(const void* dy, const void* x, const void* scale, const float* rstd, void* dx,
                               float* dscale_partial, int rows, int D, void* stream) {
  if (D & 7) return kErrBadShape;
  const int grid = ttb_rmsnorm_bwd_partials(rows);
  const int nvec = D >> 3;
  auto s = static_cast<cudaStream_t>(stream);
#define TTB_LAUNCH_RMS_BWD(MAXV)                                                                                  \
  rmsnorm_bwd_kernel<MAXV><<<grid, 256, 0, s>>>(static_cast<const __nv_bfloat16*>(dy),                            \
                                                static_cast<const __nv_bfloat16*>(x),                             \
                                                static_cast<const __nv_bfloat16*>(scale), rstd,                   \
                                                static_cast<__nv_bfloat16*>(dx), dscale_partial, rows, D)
  TTB_COUNT_LAUNCH(1);
  if (nvec <= 256) TTB_LAUNCH_RMS_BWD(1);
  else if (nvec <= 512) TTB_LAUNCH_RMS_BWD(2);
  else if (nvec <= 1024) TTB_LAUNCH_RMS_BWD(4);
  else if (nvec <= 2048) TTB_LAUNCH_RMS_BWD(8);
  else return kErrTooLarge;  // D > 16384
#undef TTB_LAUNCH_RMS_BWD
  return cudaGetLastError() == cudaSuccess ? kOk : kErrDriver;
}

extern "C" int ttb_rope(const void* x, void* y, const float* cache, const int* pos, long long tokens, int heads, int d,
                        int seq_len, int interleaved, int inverse, int cache_len, void* stream) {
  if (d % 16 || cache_len <= 0) return kErrBadShape;
  auto s = static_cast<cudaStream_t>(stream);
  if (interleaved) {
    const long long total = tokens * heads * (d / 8);
    TTB_COUNT_LAUNCH(1);
    rope_kernel<true><<<grid_for(total, 256), 256, 0, s>>>(static_cast<const __nv_bfloat16*>(x),
                                                          static_cast<__nv_bfloat16*>(y), cache, pos, tokens, heads, d,
                                                          seq_len, inverse, cache_len);
  } else {
    const long long total = tokens * heads * (d / 16);
    TTB_COUNT_LAUNCH(1);
    rope_kernel<false><<<grid_for(total, 256), 256, 0, s>>>(static_cast<const __nv_bfloat16*>(x),
                                                           static_cast<__nv_bfloat16*>(y), cache, pos, tokens, heads, d,
                                                           seq_len, inverse, cache_len);
  }
  return cudaGetLastError() == cudaSuccess ? kOk : kErrDriver;
}

extern "C" int ttb_swiglu_fwd(const void* g, const void* u, void* y, long long rows, int H, long long ldg, long long ldu,
                              long long ldy, void* stream) {
  if ((H & 7) || (ldg & 7) || (ldu & 7) || (ldy & 7)) return kErrBadShape;
  TTB_COUNT_LAUNCH(1);
  swiglu_fwd_kernel<<<grid_for(rows * (H >> 3), 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(g), static_cast<const __nv_bfloat16*>(u), static_cast<__nv_bfloat16*>(y), rows,
      H, ldg, ldu, ldy);
  return cudaGetLastError() == cudaSuccess ? kOk : kErrDriver;
}

extern "C" int ttb_swiglu_bwd(const void* dy, const void* g, const void* u, void* dg, void* du, long long rows, int H,
                              long long lddy, long long ldg, long long ldu, long long lddg, long long lddu,
                              void* stream) {
  if ((H & 7) || (lddy & 7) || (ldg & 7) || (ldu & 7) || (lddg & 7) || (lddu & 7)) return kErrBadShape;
  TTB_COUNT_LAUNCH(1);
  swiglu_bwd_kernel<<<grid_for(rows * (H >> 3), 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(dy), static_cast<const __nv_bfloat16*>(g), static_cast<const __nv_bfloat16*>(u),
      static_cast<__nv_bfloat16*>(dg), static_cast<__nv_bfloat16*>(du), rows, H, lddy, ldg, ldu, lddg, lddu);
  return cudaGetLastError() == cudaSuccess ? kOk : kErrDriver;
}

// ------------------------------------------------------------------------------------------
// Allocation-free RMSNorm backward (declaration and contract: rmsnorm_bwd_noalloc.h).
// The per-CTA partial sums of dscale live in a fixed array inside the library image.
#include "rmsnorm_bwd_noalloc.h"

static __device__ __align__(256) float g_rmsnorm_noalloc_partials[TTB_RMSNORM_NOALLOC_MAX_CTAS * TTB_RMSNORM_NOALLOC_MAX_D];

namespace ttb {

// dscale[c] = sum over the first `n_partials` rows of partials[:, c]
__global__ void rmsnorm_noalloc_finalize_kernel(const float* __restrict__ partials, float* __restrict__ dscale,
                                                int n_partials, int D) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= D) return;
  float acc = 0.f;
  for (int r = 0; r < n_partials; ++r) acc += partials[static_cast<long long>(r) * D + c];
  dscale[c] = acc;
}

static constexpr int kNoAllocMaxDevices = 64;

// In host code the array's name is only a stand-in for the symbol; the address usable by
// kernels has to be looked up per device, with that device current.
static float* noalloc_scratch_for_current_device() {
  static float* cached[kNoAllocMaxDevices] = {};
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kNoAllocMaxDevices) return nullptr;
  if (cached[dev] == nullptr) {
    void* p = nullptr;
    if (cudaGetSymbolAddress(&p, g_rmsnorm_noalloc_partials) != cudaSuccess) return nullptr;
    cached[dev] = static_cast<float*>(p);
  }
  return cached[dev];
}

}  // namespace ttb

extern "C" int ttb_rmsnorm_bwd_noalloc(const void* dy, const void* x, const void* scale, const float* rstd, void* dx,
                                       float* dscale, int rows, int D, void* stream) {
  if (rows <= 0 || D <= 0 || (D & 7)) return kErrBadShape;
  if (D > TTB_RMSNORM_NOALLOC_MAX_D) return kErrTooLarge;
  if (scale != nullptr && dscale == nullptr) return kErrBadShape;
  float* scratch = noalloc_scratch_for_current_device();
  if (scratch == nullptr) return kErrDriver;
  const int grid = rows < TTB_RMSNORM_NOALLOC_MAX_CTAS ? rows : TTB_RMSNORM_NOALLOC_MAX_CTAS;
  const int nvec = D >> 3;
  auto s = static_cast<cudaStream_t>(stream);
  float* partials = scale != nullptr ? scratch : nullptr;
  const __nv_bfloat16* dyp = static_cast<const __nv_bfloat16*>(dy);
  const __nv_bfloat16* xp = static_cast<const __nv_bfloat16*>(x);
  const __nv_bfloat16* sp = static_cast<const __nv_bfloat16*>(scale);
  __nv_bfloat16* dxp = static_cast<__nv_bfloat16*>(dx);
  TTB_COUNT_LAUNCH(1);
  if (nvec <= 256) rmsnorm_bwd_kernel<1><<<grid, 256, 0, s>>>(dyp, xp, sp, rstd, dxp, partials, rows, D);
  else if (nvec <= 512) rmsnorm_bwd_kernel<2><<<grid, 256, 0, s>>>(dyp, xp, sp, rstd, dxp, partials, rows, D);
  else rmsnorm_bwd_kernel<4><<<grid, 256, 0, s>>>(dyp, xp, sp, rstd, dxp, partials, rows, D);
  if (cudaGetLastError() != cudaSuccess) return kErrDriver;
  if (scale != nullptr) {
    TTB_COUNT_LAUNCH(1);
    rmsnorm_noalloc_finalize_kernel<<<(D + 255) / 256, 256, 0, s>>>(scratch, dscale, grid, D);
    if (cudaGetLastError() != cudaSuccess) return kErrDriver;
  }
  return kOk;
}


extern "C" unsigned int ttb_violations_embedding(int reset);
extern "C" unsigned int ttb_violations_loss(int reset);

// Out-of-range user indices (token ids, labels, positions) that kernels replaced by a safe value since the last reset.
extern "C" unsigned int ttb_index_violations(int reset) {
  return ttb_violations_rope(reset) + ttb_violations_embedding(reset) + ttb_violations_loss(reset);
}
