// Weight (de)quantisation kernels.
//
// NF4 (4-bit NormalFloat with double-quantised block scales) → bf16: the frozen base weights of QLoRA are expanded
// right before the tcgen05 GEMM that consumes them (reference call sites: torchtune/modules/peft/lora.py:137-140,
// torchtune/modules/low_precision/nf4_linear.py:56-70).  Layout: two codes per byte (high nibble first), one int8
// scale per `block` codes, one fp32 factor per `scaler_block` scales, one fp32 mean:
//     w[i] = codebook[code[i]] * (scaler_q[i / block] / scaler_factor[i / block / scaler_block] + scaler_mean)
// Each thread expands 16 codes (one 8-byte load, two 16-byte stores); the kernel is pure HBM streaming
// (0.5 B read + 2 B written per weight).
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
