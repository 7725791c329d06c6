// Weight (de)quantisation kernels.
//
// NF4 (4-bit NormalFloat with double-quantised block scales) → bf16: the frozen base weights of QLoRA are expanded
// right before the tcgen05 GEMM that consumes them (reference call sites: torchtune/modules/peft/lora.py:137-140,
// torchtune/modules/low_precision/nf4_linear.py:56-70).  Layout: two codes per byte (high nibble first), one int8
// scale per `block` codes, one fp32 factor per `scaler_block` scales, one fp32 mean:
//     w[i] = codebook[code[i]] * (scaler_q[i / block] / scaler_factor[i / block / scaler_block] + scaler_mean)
// Each thread expands 16 codes (one 8-byte load, two 16-byte stores); the kernel is pure HBM streaming
// (0.5 B read + 2 B written per weight).
#include <cuda_fp8.h>

#include "common/ptx.cuh"
#include "common/tmap.h"

namespace ttb {

__constant__ float kNF4[16] = {-1.0f, -0.6961928009986877f, -0.5250730514526367f, -0.39491748809814453f,
                               -0.28444138169288635f, -0.18477343022823334f, -0.09105003625154495f, 0.0f,
                               0.07958029955625534f, 0.16093020141124725f, 0.24611230194568634f, 0.33791524171829224f,
                               0.44070982933044434f, 0.5626170039176941f, 0.7229568362236023f, 1.0f};

__global__ void __launch_bounds__(256)
nf4_dequant_kernel(const uint8_t* __restrict__ packed, const int8_t* __restrict__ scaler_q,
                   const float* __restrict__ scaler_factor, const float* __restrict__ scaler_mean,
                   __nv_bfloat16* __restrict__ out, long long n16, int block, int scaler_block) {
  __shared__ float code[16];
  if (threadIdx.x < 16) code[threadIdx.x] = kNF4[threadIdx.x];
  __syncthreads();
  const float mean = *scaler_mean;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n16;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long e0 = i * 16;  // first element of this thread's 16 (block is a multiple of 16, so one scale applies)
    const long long blk = e0 / block;
    const float scale = static_cast<float>(scaler_q[blk]) / scaler_factor[blk / scaler_block] + mean;
    const uint2 raw = *reinterpret_cast<const uint2*>(packed + e0 / 2);
    const uint32_t words[2] = {raw.x, raw.y};
    uint32_t o[8];
#pragma unroll
    for (int w = 0; w < 2; ++w) {
#pragma unroll
      for (int b = 0; b < 4; ++b) {
        const uint32_t byte = (words[w] >> (8 * b)) & 0xFFu;
        o[w * 4 + b] = pack_bf16x2(code[byte >> 4] * scale, code[byte & 0xFu] * scale);
      }
    }
    uint4* dst = reinterpret_cast<uint4*>(out + e0);
    dst[0] = make_uint4(o[0], o[1], o[2], o[3]);
    dst[1] = make_uint4(o[4], o[5], o[6], o[7]);
  }
}

}  // namespace ttb

// n = number of weights (multiple of 16); block a multiple of 16; packed 8-byte aligned, out 16-byte aligned.
extern "C" int ttb_nf4_dequant(const void* packed, const void* scaler_q, const void* scaler_factor, const void* scaler_mean,
                               void* out, long long n, int block, int scaler_block, void* stream) {
  using namespace ttb;
  if (n <= 0 || (n & 15) || block <= 0 || (block & 15) || scaler_block <= 0) return kErrBadShape;
  if ((reinterpret_cast<uintptr_t>(packed) & 7) || (reinterpret_cast<uintptr_t>(out) & 15)) return kErrBadShape;
  const long long n16 = n / 16;
  long long blocks = (n16 + 255) / 256;
  const long long cap = static_cast<long long>(sm_count()) * 16;
  if (blocks > cap) blocks = cap;
  TTB_COUNT_LAUNCH(1);
  nf4_dequant_kernel<<<static_cast<int>(blocks), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const uint8_t*>(packed), static_cast<const int8_t*>(scaler_q), static_cast<const float*>(scaler_factor),
      static_cast<const float*>(scaler_mean), static_cast<__nv_bfloat16*>(out), n16, block, scaler_block);
  return cudaGetLastError() == cudaSuccess ? kOk : kErrDriver;
}

// ----------------------------------------------------------------------------------------------- fp8 cast (+ transpose)
// One pass over a bf16 matrix x[R, C] produces the two fp8 operands an fp8 linear layer needs: `out` = fp8(x · s_row)
// in the same layout and `out_t` = fp8(x · s_col)ᵀ ([C, R]), so that every product of the layer (forward, input gradient,
// weight gradient) reads K-contiguous operands (gemm_fp8.cu).  Scales are device fp32: one value (stride 0, tensorwise)
// or one per row of the respective output (stride 1: per row of x for `out`, per column of x for `out_t`).
namespace ttb {

template <bool E5M2>
__device__ __forceinline__ uint8_t to_fp8(float v) {
  return static_cast<uint8_t>(__nv_cvt_float_to_fp8(v, __NV_SATFINITE, E5M2 ? __NV_E5M2 : __NV_E4M3));
}

template <bool E5M2>
__global__ void __launch_bounds__(256)
fp8_cast_transpose_kernel(const __nv_bfloat16* __restrict__ x, long long ldx, int R, int C, const float* __restrict__ s_row, int s_row_stride,
                          uint8_t* __restrict__ out, const float* __restrict__ s_col, int s_col_stride, uint8_t* __restrict__ out_t) {
  __shared__ __align__(16) uint8_t tile_t[64][64 + 16];  // [column][row] for the transposed output
  const int r0 = blockIdx.y * 64, c0 = blockIdx.x * 64;
  const int lr = threadIdx.x >> 2, lc = (threadIdx.x & 3) * 16;
  const int r = r0 + lr, c = c0 + lc;
  if (r < R && c < C) {  // R and C are multiples of 16: a 16-element group is inside or outside as a whole
    const uint4* src = reinterpret_cast<const uint4*>(x + static_cast<long long>(r) * ldx + c);
    const uint4 raw[2] = {src[0], src[1]};
    const __nv_bfloat16* h = reinterpret_cast<const __nv_bfloat16*>(raw);
    float v[16];
#pragma unroll
    for (int i = 0; i < 16; ++i) v[i] = __bfloat162float(h[i]);
    if (out != nullptr) {
      const float sr = s_row[s_row_stride ? r : 0];
      uint32_t w[4];
#pragma unroll
      for (int i = 0; i < 4; ++i)
        w[i] = to_fp8<E5M2>(v[4 * i] * sr) | (to_fp8<E5M2>(v[4 * i + 1] * sr) << 8) | (to_fp8<E5M2>(v[4 * i + 2] * sr) << 16) |
               (static_cast<uint32_t>(to_fp8<E5M2>(v[4 * i + 3] * sr)) << 24);
      *reinterpret_cast<uint4*>(out + static_cast<long long>(r) * C + c) = make_uint4(w[0], w[1], w[2], w[3]);
    }
    if (out_t != nullptr) {
#pragma unroll
      for (int i = 0; i < 16; ++i) tile_t[lc + i][lr] = to_fp8<E5M2>(v[i] * s_col[s_col_stride ? c + i : 0]);
    }
  }
  if (out_t == nullptr) return;
  __syncthreads();
  const int tc = c0 + lr, tr = r0 + lc;  // this thread writes 16 consecutive rows of column tc
  if (tc < C && tr < R) *reinterpret_cast<uint4*>(out_t + static_cast<long long>(tc) * R + tr) = *reinterpret_cast<const uint4*>(&tile_t[lr][lc]);
}

}  // namespace ttb

// x: [R, C] bf16 (row stride ldx, multiple of 8), R and C multiples of 16.  out: [R, C] fp8 or nullptr; out_t: [C, R] fp8 or nullptr.
extern "C" int ttb_fp8_cast_transpose(const void* x, long long ldx, int R, int C, const void* s_row, int s_row_stride, void* out,
                                      const void* s_col, int s_col_stride, void* out_t, int e5m2, void* stream) {
  using namespace ttb;
  if (R <= 0 || C <= 0 || (R & 15) || (C & 15) || (ldx & 7)) return kErrBadShape;
  if ((out && !s_row) || (out_t && !s_col) || (!out && !out_t)) return kErrBadShape;
  if ((reinterpret_cast<uintptr_t>(x) & 15) || (reinterpret_cast<uintptr_t>(out) & 15) || (reinterpret_cast<uintptr_t>(out_t) & 15)) return kErrBadShape;
  dim3 grid((C + 63) / 64, (R + 63) / 64);
  if (grid.y > 65535) return kErrTooLarge;
  TTB_COUNT_LAUNCH(1);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (e5m2)
    fp8_cast_transpose_kernel<true><<<grid, 256, 0, s>>>(static_cast<const __nv_bfloat16*>(x), ldx, R, C, static_cast<const float*>(s_row), s_row_stride,
                                                         static_cast<uint8_t*>(out), static_cast<const float*>(s_col), s_col_stride, static_cast<uint8_t*>(out_t));
  else
    fp8_cast_transpose_kernel<false><<<grid, 256, 0, s>>>(static_cast<const __nv_bfloat16*>(x), ldx, R, C, static_cast<const float*>(s_row), s_row_stride,
                                                          static_cast<uint8_t*>(out), static_cast<const float*>(s_col), s_col_stride, static_cast<uint8_t*>(out_t));
  return cudaGetLastError() == cudaSuccess ? kOk : kErrDriver;
}

// ----------------------------------------------------------------------------------------------- NF4 quantise
// Two streaming kernels around a few tiny tensor ops on the per-block scales (mean-centring and int8 coding of the scales stay
// in the framework layer): (1) absmax of every `block` weights, (2) nearest NF4 code of w / scale per weight, packed two per byte
// (high nibble first).  Nearest code = number of codebook midpoints below the normalised value (ties go to the lower code, as an
// argmin over |w - code| does).
namespace ttb {

__global__ void __launch_bounds__(256)
nf4_absmax_kernel(const __nv_bfloat16* __restrict__ w, float* __restrict__ absmax, long long n_blocks, int block) {
  // one warp per block of `block` weights (block is a multiple of 32)
  const long long warp = (blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  const long long n_warps = (static_cast<long long>(gridDim.x) * blockDim.x) >> 5;
  for (long long b = warp; b < n_blocks; b += n_warps) {
    float m = 0.f;
    for (int i = lane; i < block; i += 32) m = fmaxf(m, fabsf(__bfloat162float(w[b * block + i])));
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
    if (lane == 0) absmax[b] = m;
  }
}

__global__ void __launch_bounds__(256)
nf4_encode_kernel(const __nv_bfloat16* __restrict__ w, const float* __restrict__ scales, uint8_t* __restrict__ packed, long long n_pairs,
                  int block) {
  __shared__ float mid[15];
  if (threadIdx.x < 15) mid[threadIdx.x] = 0.5f * (kNF4[threadIdx.x] + kNF4[threadIdx.x + 1]);
  __syncthreads();
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n_pairs;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long e = 2 * i;
    const float sc = fmaxf(scales[e / block], 1e-30f);
    uint32_t codes[2];
#pragma unroll
    for (int k = 0; k < 2; ++k) {
      const float v = fminf(fmaxf(__bfloat162float(w[e + k]) / sc, -1.f), 1.f);
      uint32_t c = 0;
#pragma unroll
      for (int j = 0; j < 15; ++j) c += v > mid[j] ? 1u : 0u;
      codes[k] = c;
    }
    packed[i] = static_cast<uint8_t>((codes[0] << 4) | codes[1]);
  }
}

}  // namespace ttb

extern "C" int ttb_nf4_absmax(const void* w, void* absmax, long long n, int block, void* stream) {
  using namespace ttb;
  if (n <= 0 || block <= 0 || (block & 31) || (n % block)) return kErrBadShape;
  const long long n_blocks = n / block;
  long long blocks = (n_blocks * 32 + 255) / 256;
  const long long cap = static_cast<long long>(sm_count()) * 16;
  if (blocks > cap) blocks = cap;
  TTB_COUNT_LAUNCH(1);
  nf4_absmax_kernel<<<static_cast<int>(blocks), 256, 0, static_cast<cudaStream_t>(stream)>>>(static_cast<const __nv_bfloat16*>(w), static_cast<float*>(absmax),
                                                                                           n_blocks, block);
  return cudaGetLastError() == cudaSuccess ? kOk : kErrDriver;
}

// scales: fp32 [n / block] — the *dequantised* per-block scales, so that the round trip is self-consistent.
extern "C" int ttb_nf4_encode(const void* w, const void* scales, void* packed, long long n, int block, void* stream) {
  using namespace ttb;
  if (n <= 0 || (n & 1) || block <= 0 || (block & 1) || (n % block)) return kErrBadShape;
  const long long n_pairs = n / 2;
  long long blocks = (n_pairs + 255) / 256;
  const long long cap = static_cast<long long>(sm_count()) * 16;
  if (blocks > cap) blocks = cap;
  TTB_COUNT_LAUNCH(1);
  nf4_encode_kernel<<<static_cast<int>(blocks), 256, 0, static_cast<cudaStream_t>(stream)>>>(static_cast<const __nv_bfloat16*>(w), static_cast<const float*>(scales),
                                                                                           static_cast<uint8_t*>(packed), n_pairs, block);
  return cudaGetLastError() == cudaSuccess ? kOk : kErrDriver;
}
