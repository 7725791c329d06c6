// fp8 GEMM on tcgen05 (kind::f8f6f4) with dynamic scales applied in the epilogue.
//
//   C[M,N] (+)= (A[M,K] · B[N,K]ᵀ) · sa[m] · sb[n]  (+ bias[N])         A, B: e4m3 or e5m2, K contiguous; C bf16
//
// Serves fp8 training of the decoder linears (the reference delegates to torchao's Float8Linear,
// torchtune/training/quantization.py:247-273: dynamic tensorwise or rowwise scaling).  All three products of a linear
// layer are expressed with K-contiguous operands — forward x·Wᵀ, input gradient dy·(Wᵀ)ᵀ and weight gradient
// dyᵀ·(xᵀ)ᵀ — the transposed fp8 copies come from the fused cast+transpose kernel in quant.cu, which is also where the
// scales are applied on the way in.  `sa` / `sb` are the *inverse* quantisation scales: one value (tensorwise,
// stride 0) or one per row of A / row of B (rowwise, stride 1).
//
// Same pipeline as the bf16 kernel (gemm.cu): persistent CTAs, warp 0 TMA producer, warp 1 single-lane MMA issuer,
// warp 2 TMEM allocator, warps 4-7 epilogue, double-buffered TMEM accumulators.  A k-block is 128 fp8 values
// (128 bytes = one swizzle row) = 4 MMAs of K = 32; per-SM tensor throughput is twice that of bf16.
#include <cstring>

#include "common/ptx.cuh"
#include "common/tmap.h"

namespace ttb {

static constexpr int F8_BM = 128;
static constexpr int F8_BK = 128;  // bytes == elements
static constexpr int F8_THREADS = 256;
static constexpr int F8_GROUP_M = 16;

struct Fp8Params {
  int M, N, K;
  __nv_bfloat16* C;
  long long ldc;
  const float* sa;  // inverse scale(s) of A
  const float* sb;  // inverse scale(s) of B
  int sa_stride, sb_stride;  // 0: scalar, 1: per row
  const __nv_bfloat16* bias;
  int accumulate;
  uint32_t idesc;
  int* err;
};

template <int BN>
struct Fp8Cfg {
  static constexpr int kABytes = F8_BM * F8_BK;
  static constexpr int kBBytes = BN * F8_BK;
  static constexpr int kStageBytes = kABytes + kBBytes;
  static constexpr int kStages = (200 * 1024 / kStageBytes) > 8 ? 8 : (200 * 1024 / kStageBytes);
  static constexpr int kTmemCols = 2 * BN < 32 ? 32 : 2 * BN;
  static constexpr int kSmemBytes = kStages * kStageBytes + 1024 + 256;
};

// kind::f8f6f4 instruction descriptor: [4,6) D fmt (1 = f32), [7,10) A fmt, [10,13) B fmt (0 = e4m3, 1 = e5m2),
// bits 15/16 A/B major (0 = K), [17,23) N >> 3, [24,29) M >> 4.
static uint32_t make_idesc_fp8(int m, int n, int a_e5m2, int b_e5m2) {
  return (1u << 4) | (static_cast<uint32_t>(a_e5m2 ? 1 : 0) << 7) | (static_cast<uint32_t>(b_e5m2 ? 1 : 0) << 10) |
         (static_cast<uint32_t>(n >> 3) << 17) | (static_cast<uint32_t>(m >> 4) << 24);
}

__device__ __forceinline__ void umma_f8(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
      : "memory");
}

__device__ __forceinline__ void f8_tile_coords(int t, int num_m, int num_n, int& m_blk, int& n_blk) {
  const int per_group = F8_GROUP_M * num_n;
  const int group = t / per_group;
  const int first_m = group * F8_GROUP_M;
  const int gsize = min(F8_GROUP_M, num_m - first_m);
  const int r = t - group * per_group;
  m_blk = first_m + r % gsize;
  n_blk = r / gsize;
}

template <int BN>
__global__ void __launch_bounds__(F8_THREADS, 1)
gemm_fp8_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, Fp8Params p) {
  using Cfg = Fp8Cfg<BN>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + Cfg::kStages * Cfg::kStageBytes);
  uint64_t* full = bars;
  uint64_t* empty = bars + Cfg::kStages;
  uint64_t* tfull = bars + 2 * Cfg::kStages;
  uint64_t* tempty = tfull + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tempty + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int num_m = (p.M + F8_BM - 1) / F8_BM;
  const int num_n = (p.N + BN - 1) / BN;
  const int num_tiles = num_m * num_n;
  const int num_kb = (p.K + F8_BK - 1) / F8_BK;

  if (threadIdx.x == 0) {
    for (int i = 0; i < Cfg::kStages; ++i) {
      mbar_init(&full[i], 1);
      mbar_init(&empty[i], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&tfull[i], 1);
      mbar_init(&tempty[i], 4);
    }
    *abort_flag = 0;
    fence_mbar_init();
  }
  if (warp == 0 && lane == 0) {
    prefetch_tmap(&tmA);
    prefetch_tmap(&tmB);
  }
  if (warp == 2) {
    tmem_alloc(tmem_slot, Cfg::kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    int stage = 0;
    uint32_t phase = 0;
    for (int t = blockIdx.x; t < num_tiles && !*abort_flag; t += gridDim.x) {
      int m_blk, n_blk;
      f8_tile_coords(t, num_m, num_n, m_blk, n_blk);
      for (int kb = 0; kb < num_kb; ++kb) {
        if (!mbar_wait(&empty[stage], phase ^ 1)) {
          *abort_flag = 1;
          if (lane == 0) atomicExch(p.err, 111);
          break;
        }
        if (lane == 0) {
          uint8_t* sa = smem + stage * Cfg::kStageBytes;
          uint8_t* sb = sa + Cfg::kABytes;
          mbar_arrive_expect_tx(&full[stage], Cfg::kStageBytes);
          tma_load_2d(sa, &tmA, &full[stage], kb * F8_BK, m_blk * F8_BM);
          tma_load_2d(sb, &tmB, &full[stage], kb * F8_BK, n_blk * BN);
        }
        __syncwarp();
        if (++stage == Cfg::kStages) {
          stage = 0;
          phase ^= 1;
        }
      }
    }
  } else if (warp == 1) {
    int stage = 0;
    uint32_t phase = 0;
    int acc = 0;
    uint32_t acc_phase = 0;
    for (int t = blockIdx.x; t < num_tiles && !*abort_flag; t += gridDim.x) {
      if (!mbar_wait(&tempty[acc], acc_phase ^ 1)) {
        *abort_flag = 1;
        if (lane == 0) atomicExch(p.err, 112);
        break;
      }
      tc_fence_after();
      const uint32_t d_tmem = tmem_base + acc * BN;
      bool ok = true;
      for (int kb = 0; kb < num_kb; ++kb) {
        if (!mbar_wait(&full[stage], phase)) {
          ok = false;
          break;
        }
        tc_fence_after();
        if (lane == 0) {
          const uint32_t sa = smem_u32(smem + stage * Cfg::kStageBytes);
          const uint32_t sb = sa + Cfg::kABytes;
#pragma unroll
          for (int k = 0; k < F8_BK / 32; ++k) {  // K = 32 per MMA: 32 bytes inside the swizzled 128-byte row
            const uint64_t da = make_smem_desc_sw128(sa + k * 32, 16, 1024);
            const uint64_t db = make_smem_desc_sw128(sb + k * 32, 16, 1024);
            umma_f8(d_tmem, da, db, p.idesc, (kb | k) != 0);
          }
          umma_commit(&empty[stage]);
        }
        __syncwarp();
        if (++stage == Cfg::kStages) {
          stage = 0;
          phase ^= 1;
        }
      }
      if (!ok) {
        *abort_flag = 1;
        if (lane == 0) atomicExch(p.err, 113);
        break;
      }
      if (lane == 0) umma_commit(&tfull[acc]);
      __syncwarp();
      if (++acc == 2) {
        acc = 0;
        acc_phase ^= 1;
      }
    }
  } else if (warp >= 4) {
    const int quarter = warp & 3;
    int acc = 0;
    uint32_t acc_phase = 0;
    for (int t = blockIdx.x; t < num_tiles && !*abort_flag; t += gridDim.x) {
      int m_blk, n_blk;
      f8_tile_coords(t, num_m, num_n, m_blk, n_blk);
      if (!mbar_wait(&tfull[acc], acc_phase)) {
        *abort_flag = 1;
        if (lane == 0) atomicExch(p.err, 114);
        break;
      }
      tc_fence_after();
      const int row = m_blk * F8_BM + quarter * 32 + lane;
      const bool row_ok = row < p.M;
      const float sa = row_ok ? __ldg(p.sa + (p.sa_stride ? row : 0)) : 0.f;
      const float sb0 = p.sb_stride ? 0.f : __ldg(p.sb);
      const uint32_t taddr = tmem_base + acc * BN + (static_cast<uint32_t>(quarter * 32) << 16);
#pragma unroll 1
      for (int c = 0; c < BN / 32; ++c) {
        uint32_t r[32];
        tmem_ld_32x32(taddr + c * 32, r);
        tmem_ld_wait();
        const int col0 = n_blk * BN + c * 32;
        if (row_ok && col0 < p.N) {
          float v[32];
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            const float sb = p.sb_stride ? (col0 + i < p.N ? __ldg(p.sb + col0 + i) : 0.f) : sb0;
            v[i] = __uint_as_float(r[i]) * sa * sb;
          }
          if (p.bias != nullptr) {
#pragma unroll
            for (int i = 0; i < 32; ++i)
              if (col0 + i < p.N) v[i] += __bfloat162float(__ldg(p.bias + col0 + i));
          }
          __nv_bfloat16* dst = p.C + static_cast<long long>(row) * p.ldc + col0;
#pragma unroll
          for (int g = 0; g < 4; ++g) {
            if (col0 + g * 8 + 8 <= p.N) {
              if (p.accumulate) {
                const uint4 old = *reinterpret_cast<const uint4*>(dst + g * 8);
                const __nv_bfloat162* ob = reinterpret_cast<const __nv_bfloat162*>(&old);
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                  const float2 f = __bfloat1622float2(ob[i]);
                  v[g * 8 + 2 * i] += f.x;
                  v[g * 8 + 2 * i + 1] += f.y;
                }
              }
              uint4 o;
              o.x = pack_bf16x2(v[g * 8 + 0], v[g * 8 + 1]);
              o.y = pack_bf16x2(v[g * 8 + 2], v[g * 8 + 3]);
              o.z = pack_bf16x2(v[g * 8 + 4], v[g * 8 + 5]);
              o.w = pack_bf16x2(v[g * 8 + 6], v[g * 8 + 7]);
              *reinterpret_cast<uint4*>(dst + g * 8) = o;
            }
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&tempty[acc]);
      if (++acc == 2) {
        acc = 0;
        acc_phase ^= 1;
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  if (warp == 2) tmem_dealloc(tmem_base, Cfg::kTmemCols);
}

template <int BN>
static int launch_fp8(const void* A, const void* B, const Fp8Params& p, long long lda, long long ldb, cudaStream_t stream) {
  using Cfg = Fp8Cfg<BN>;
  CUtensorMap tmA, tmB;
  int rc = make_tmap_2d(&tmA, A, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, p.M, p.K, lda, F8_BM, F8_BK, CU_TENSOR_MAP_SWIZZLE_128B);
  if (rc != kOk) return rc;
  rc = make_tmap_2d(&tmB, B, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, p.N, p.K, ldb, BN, F8_BK, CU_TENSOR_MAP_SWIZZLE_128B);
  if (rc != kOk) return rc;
  auto kern = gemm_fp8_kernel<BN>;
  static bool attr_set = false;
  if (!attr_set) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::kSmemBytes) != cudaSuccess) return kErrDriver;
    attr_set = true;
  }
  Fp8Params q = p;
  const int num_tiles = ((p.M + F8_BM - 1) / F8_BM) * ((p.N + BN - 1) / BN);
  const int grid = num_tiles < sm_count() ? num_tiles : sm_count();
  TTB_COUNT_LAUNCH(1);
  kern<<<grid, F8_THREADS, Cfg::kSmemBytes, stream>>>(tmA, tmB, q);
  return cudaGetLastError() == cudaSuccess ? kOk : kErrDriver;
}

}  // namespace ttb

// A: [M, K] fp8, B: [N, K] fp8 (row strides lda / ldb in bytes, multiples of 16), C: [M, N] bf16 (ldc multiple of 8).
// a_e5m2 / b_e5m2: 0 = e4m3, 1 = e5m2.  sa / sb: device fp32 inverse scales (stride 0 = one value, 1 = per row of A / B).
extern "C" int ttb_gemm_fp8(const void* A, const void* B, void* C, int M, int N, int K, long long lda, long long ldb, long long ldc,
                            int a_e5m2, int b_e5m2, const void* sa, int sa_stride, const void* sb, int sb_stride, const void* bias,
                            int accumulate, int* err, void* stream) {
  using namespace ttb;
  if (M <= 0 || N <= 0 || K <= 0 || sa == nullptr || sb == nullptr) return kErrBadShape;
  if ((lda & 15) || (ldb & 15) || (ldc & 7) || (N & 7) || (K & 15)) return kErrBadShape;
  Fp8Params p;
  p.M = M, p.N = N, p.K = K, p.C = static_cast<__nv_bfloat16*>(C), p.ldc = ldc;
  p.sa = static_cast<const float*>(sa), p.sb = static_cast<const float*>(sb);
  p.sa_stride = sa_stride ? 1 : 0, p.sb_stride = sb_stride ? 1 : 0;
  p.bias = static_cast<const __nv_bfloat16*>(bias), p.accumulate = accumulate, p.err = err;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (N > 128) {
    p.idesc = make_idesc_fp8(F8_BM, 256, a_e5m2, b_e5m2);
    return launch_fp8<256>(A, B, p, lda, ldb, s);
  }
  if (N > 64) {
    p.idesc = make_idesc_fp8(F8_BM, 128, a_e5m2, b_e5m2);
    return launch_fp8<128>(A, B, p, lda, ldb, s);
  }
  p.idesc = make_idesc_fp8(F8_BM, 64, a_e5m2, b_e5m2);
  return launch_fp8<64>(A, B, p, lda, ldb, s);
}
