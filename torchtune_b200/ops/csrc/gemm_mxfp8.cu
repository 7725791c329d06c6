// Block-scaled fp8 (MX format) GEMM on tcgen05: kind::mxf8f6f4.block_scale with the scale factors in tensor memory.
//
//   C[M,N] = sum_k  A[m,k]·2^(ea[m, k/32] − 127)  ·  B[n,k]·2^(eb[n, k/32] − 127)   (+ bias[N])
//
// A [M, K] and B [N, K] hold e4m3 values, K contiguous; every 32 consecutive values along K share one 8-bit power-of-two scale
// (UE8M0, the OCP MX block format).  The tensor core applies both scales to each K = 32 step in hardware, so the epilogue has
// nothing left to rescale and an outlier only costs precision inside its own 32-value block (the tensorwise / rowwise fp8
// kernel in gemm_fp8.cu loses it for a whole tensor / row).  Used by the "blockwise" fp8 training recipe: forward x·Wᵀ, input
// gradient dy·(Wᵀ)ᵀ and weight gradient dyᵀ·(xᵀ)ᵀ all run here with K-contiguous operands produced by the quantisers below
// (the reference delegates fp8 training to torchao, torchtune/training/quantization.py:247-273).
//
// Scale-factor storage (what the quantisers write and the GEMM reads): for a [R, C] operand the buffer is a grid of
// ceil(R/128) × ceil(C/128) chunks of 512 bytes; chunk (i, j) covers rows [128 i, 128 i + 128) and the four 32-value blocks of
// columns [128 j, 128 j + 128); inside a chunk byte (r mod 32)·16 + ((r mod 128) / 32)·4 + b is the scale of row r, block b.
// One chunk is exactly what one `tcgen05.cp.32x128b.warpx4` moves from shared to tensor memory: 32 lanes × 16 bytes, replicated
// to the four lane quarters, giving 4 tensor-memory columns whose column g holds rows 32 g + lane and whose byte b is block b —
// the layout tcgen05.mma reads with the scale-factor id b in its instruction descriptor.
//
// Pipeline per CTA (persistent over 128 × 256 output tiles): warp 0 producer (TMA tiles of A and B plus three 512-byte bulk
// copies of scale chunks per 128-wide k-block), warp 1 issues per k-block three tcgen05.cp and four MMAs of K = 32, warp 2 owns
// tensor memory, warps 4-11 drain the accumulator.  Tensor memory: 256 accumulator columns + 12 scale columns per pipeline
// stage; two 256-column accumulators would leave no room for the scales (and a 192-wide tile with two accumulators measured slower:
// the main loop is bound by the shared-memory fill rate, which a narrower tile makes worse).  Instead the single accumulator is
// handed back early: eight epilogue warps (two per lane quarter, 128 columns each) pull their part into registers with four
// back-to-back tcgen05.ld, signal the MMA warp, and only then convert and store, so the next tile's main loop overlaps the stores.
// Every wait is bounded and reports through the error word.
#include <cuda_fp8.h>

#include <cstring>

#include "common/ptx.cuh"
#include "common/tmap.h"

namespace ttb {
namespace mx {

static constexpr int BM = 128;
static constexpr int BN = 256;
static constexpr int BK = 128;  // fp8 values = bytes per k-block: four MMAs of K = 32, four scale blocks
static constexpr int kThreads = 384;  // warps 0-3: producer, MMA, tensor-memory owner, spare; warps 4-11: epilogue
static constexpr int kGroupM = 16;
static constexpr int kStages = 4;
static constexpr int kABytes = BM * BK;          // 16 KB
static constexpr int kBBytes = BN * BK;          // 32 KB
static constexpr int kSfChunk = 512;             // scales of 128 rows × 4 blocks
static constexpr int kSfBytes = 3 * kSfChunk;    // one chunk for A, two for B
static constexpr int kStageBytes = kABytes + kBBytes + 2048;  // operands + scales, stage bases stay 1024-byte aligned
static constexpr int kSmemBytes = kStages * kStageBytes + 1024 + 1024;
static constexpr int kAccCols = BN;
static constexpr int kSfColsPerStage = 16;  // 4 (A) + 8 (B), padded to 16
static constexpr int kTmemCols = 512;
static_assert(kAccCols + kStages * kSfColsPerStage <= kTmemCols, "tensor memory budget");
static_assert(kSmemBytes <= 232448, "shared memory budget of one CTA");

struct Params {
  int M, N, K;
  __nv_bfloat16* C;
  long long ldc;
  const uint8_t* sfa;  // scale chunks of A: ceil(M/128) × num_kb
  const uint8_t* sfb;  // scale chunks of B: (2 · ceil(N/256)) × num_kb
  const __nv_bfloat16* bias;
  int accumulate;  // add to the bf16 values already in C
  int* err;
};

// kind::mxf8f6f4 instruction descriptor (block-scaled form): [4,6) B scale id, [7,10) A format, [10,13) B format (0 = e4m3),
// bits 15 / 16 A / B major (0 = K), [17,23) N >> 3, bit 23 scale format (1 = UE8M0), [24,29) M >> 4, [29,31) A scale id.
__host__ __device__ constexpr uint32_t make_idesc_mx(int m, int n) {
  return (static_cast<uint32_t>(n >> 3) << 17) | (1u << 23) | (static_cast<uint32_t>(m >> 4) << 24);
}

// Shared-memory matrix descriptor without swizzle, K-major: 8-row groups of 16-byte rows, `sbo_bytes` between groups.
__device__ __forceinline__ uint64_t make_smem_desc_plain(uint32_t smem_addr, uint32_t sbo_bytes) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((smem_addr >> 4) & 0x3fff);
  d |= static_cast<uint64_t>((sbo_bytes >> 4) & 0x3fff) << 32;
  d |= static_cast<uint64_t>(1) << 46;
  return d;
}

// 32 lanes × 128 bits from shared memory to 4 tensor-memory columns, replicated to the four 32-lane quarters.
__device__ __forceinline__ void tmem_cp_32x128b_x4(uint32_t taddr, uint64_t sdesc) {
  asm volatile("tcgen05.cp.cta_group::1.32x128b.warpx4 [%0], %1;" ::"r"(taddr), "l"(sdesc) : "memory");
}

__device__ __forceinline__ void umma_mx(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, uint32_t sfa, uint32_t sfb, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::mxf8f6f4.block_scale [%0], %1, %2, %3, [%5], [%6], p;\n\t}"
      ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate), "r"(sfa), "r"(sfb)
      : "memory");
}

// Untiled bulk copy global → shared; both addresses and the size are multiples of 16 bytes.
__device__ __forceinline__ void bulk_load(void* smem_dst, const void* gsrc, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(smem_u32(smem_dst)), "l"(gsrc), "r"(bytes),
               "r"(smem_u32(bar))
               : "memory");
}

__device__ __forceinline__ void tile_coords(int t, int num_m, int num_n, int& m_blk, int& n_blk) {
  const int per_group = kGroupM * num_n;
  const int group = t / per_group;
  const int first_m = group * kGroupM;
  const int gsize = min(kGroupM, num_m - first_m);
  const int r = t - group * per_group;
  m_blk = first_m + r % gsize;
  n_blk = r / gsize;
}

__global__ void __launch_bounds__(kThreads, 1)
gemm_mxfp8_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, Params p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + kStages * kStageBytes);
  uint64_t* full = bars;
  uint64_t* empty = bars + kStages;
  uint64_t* tfull = bars + 2 * kStages;
  uint64_t* tempty = tfull + 1;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tempty + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int num_m = (p.M + BM - 1) / BM;
  const int num_n = (p.N + BN - 1) / BN;
  const int num_tiles = num_m * num_n;
  const int num_kb = (p.K + BK - 1) / BK;

  if (threadIdx.x == 0) {
    for (int i = 0; i < kStages; ++i) {
      mbar_init(&full[i], 1);
      mbar_init(&empty[i], 1);
    }
    mbar_init(tfull, 1);
    mbar_init(tempty, 8);
    *abort_flag = 0;
    fence_mbar_init();
  }
  if (warp == 0 && lane == 0) {
    prefetch_tmap(&tmA);
    prefetch_tmap(&tmB);
  }
  if (warp == 2) {
    tmem_alloc(tmem_slot, kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ------------------------------------------------------------------ producer
    int stage = 0;
    uint32_t phase = 0;
    for (int t = blockIdx.x; t < num_tiles && !*abort_flag; t += gridDim.x) {
      int m_blk, n_blk;
      tile_coords(t, num_m, num_n, m_blk, n_blk);
      const uint8_t* sfa_row = p.sfa + static_cast<long long>(m_blk) * num_kb * kSfChunk;
      const uint8_t* sfb_row0 = p.sfb + static_cast<long long>(2 * n_blk) * num_kb * kSfChunk;
      const uint8_t* sfb_row1 = sfb_row0 + static_cast<long long>(num_kb) * kSfChunk;
      for (int kb = 0; kb < num_kb; ++kb) {
        if (!mbar_wait(&empty[stage], phase ^ 1)) {
          *abort_flag = 1;
          if (lane == 0) atomicExch(p.err, 111);
          break;
        }
        if (lane == 0) {
          uint8_t* sa = smem + stage * kStageBytes;
          uint8_t* sb = sa + kABytes;
          uint8_t* ssf = sb + kBBytes;
          mbar_arrive_expect_tx(&full[stage], kABytes + kBBytes + kSfBytes);
          tma_load_2d(sa, &tmA, &full[stage], kb * BK, m_blk * BM);
          tma_load_2d(sb, &tmB, &full[stage], kb * BK, n_blk * BN);
          bulk_load(ssf, sfa_row + kb * kSfChunk, kSfChunk, &full[stage]);
          bulk_load(ssf + kSfChunk, sfb_row0 + kb * kSfChunk, kSfChunk, &full[stage]);
          bulk_load(ssf + 2 * kSfChunk, sfb_row1 + kb * kSfChunk, kSfChunk, &full[stage]);
        }
        __syncwarp();
        if (++stage == kStages) {
          stage = 0;
          phase ^= 1;
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ scale copies + MMAs
    constexpr uint32_t idesc0 = make_idesc_mx(BM, BN);
    int stage = 0;
    uint32_t phase = 0;
    uint32_t acc_phase = 0;
    for (int t = blockIdx.x; t < num_tiles && !*abort_flag; t += gridDim.x) {
      if (!mbar_wait(tempty, acc_phase ^ 1)) {
        *abort_flag = 1;
        if (lane == 0) atomicExch(p.err, 112);
        break;
      }
      tc_fence_after();
      const uint32_t d_tmem = tmem_base;
      bool ok = true;
      for (int kb = 0; kb < num_kb; ++kb) {
        if (!mbar_wait(&full[stage], phase)) {
          ok = false;
          break;
        }
        tc_fence_after();
        if (lane == 0) {
          const uint32_t sa = smem_u32(smem + stage * kStageBytes);
          const uint32_t sb = sa + kABytes;
          const uint32_t ssf = sb + kBBytes;
          const uint32_t t_sfa = tmem_base + kAccCols + stage * kSfColsPerStage;
          const uint32_t t_sfb = t_sfa + 4;
          tmem_cp_32x128b_x4(t_sfa, make_smem_desc_plain(ssf, 128));
          tmem_cp_32x128b_x4(t_sfb, make_smem_desc_plain(ssf + kSfChunk, 128));
          tmem_cp_32x128b_x4(t_sfb + 4, make_smem_desc_plain(ssf + 2 * kSfChunk, 128));
#pragma unroll
          for (int k = 0; k < BK / 32; ++k) {
            const uint64_t da = make_smem_desc_sw128(sa + k * 32, 16, 1024);
            const uint64_t db = make_smem_desc_sw128(sb + k * 32, 16, 1024);
            const uint32_t idesc = idesc0 | (static_cast<uint32_t>(k) << 29) | (static_cast<uint32_t>(k) << 4);
            umma_mx(d_tmem, da, db, idesc, t_sfa, t_sfb, (kb | k) != 0);
          }
          umma_commit(&empty[stage]);  // operands and scale chunks of this stage may be overwritten once these retire
        }
        __syncwarp();
        if (++stage == kStages) {
          stage = 0;
          phase ^= 1;
        }
      }
      if (!ok) {
        *abort_flag = 1;
        if (lane == 0) atomicExch(p.err, 113);
        break;
      }
      if (lane == 0) umma_commit(tfull);
      __syncwarp();
      acc_phase ^= 1;
    }
  } else if (warp >= 4) {
    // ------------------------------------------------------------------ epilogue (8 warps: lane quarter x column half)
    const int quarter = warp & 3;
    const int half = (warp - 4) >> 2;
    uint32_t acc_phase = 0;
    for (int t = blockIdx.x; t < num_tiles && !*abort_flag; t += gridDim.x) {
      int m_blk, n_blk;
      tile_coords(t, num_m, num_n, m_blk, n_blk);
      if (!mbar_wait(tfull, acc_phase)) {
        *abort_flag = 1;
        if (lane == 0) atomicExch(p.err, 114);
        break;
      }
      tc_fence_after();
      const int row = m_blk * BM + quarter * 32 + lane;
      const bool row_ok = row < p.M;
      const uint32_t taddr = tmem_base + half * 128 + (static_cast<uint32_t>(quarter * 32) << 16);
      uint32_t r[4][32];
#pragma unroll
      for (int c = 0; c < 4; ++c) tmem_ld_32x32(taddr + c * 32, r[c]);
      tmem_ld_wait();
      // the accumulator is free for the next tile as soon as its values sit in registers
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(tempty);
      acc_phase ^= 1;
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        const int col0 = n_blk * BN + half * 128 + c * 32;
        if (row_ok && col0 < p.N) {
          __nv_bfloat16* dst = p.C + static_cast<long long>(row) * p.ldc + col0;
#pragma unroll
          for (int g = 0; g < 4; ++g) {
            if (col0 + g * 8 + 8 <= p.N) {
              float v[8];
#pragma unroll
              for (int i = 0; i < 8; ++i) v[i] = __uint_as_float(r[c][g * 8 + i]);
              if (p.bias != nullptr) {
                const uint4 bq = __ldg(reinterpret_cast<const uint4*>(p.bias + col0 + g * 8));
                const __nv_bfloat162* bb = reinterpret_cast<const __nv_bfloat162*>(&bq);
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                  const float2 f = __bfloat1622float2(bb[i]);
                  v[2 * i] += f.x, v[2 * i + 1] += f.y;
                }
              }
              if (p.accumulate) {
                const uint4 old = *reinterpret_cast<const uint4*>(dst + g * 8);
                const __nv_bfloat162* ob = reinterpret_cast<const __nv_bfloat162*>(&old);
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                  const float2 f = __bfloat1622float2(ob[i]);
                  v[2 * i] += f.x, v[2 * i + 1] += f.y;
                }
              }
              uint4 o;
              o.x = pack_bf16x2(v[0], v[1]);
              o.y = pack_bf16x2(v[2], v[3]);
              o.z = pack_bf16x2(v[4], v[5]);
              o.w = pack_bf16x2(v[6], v[7]);
              *reinterpret_cast<uint4*>(dst + g * 8) = o;
            }
          }
        }
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  if (warp == 2) tmem_dealloc(tmem_base, kTmemCols);
}

// ----------------------------------------------------------------------------- quantisers
// Power-of-two scale of a 32-value block with largest magnitude `amax`: 2^(floor(log2 amax) − 8), 8 being the exponent of the
// largest e4m3 binade (448 = 1.75 · 2^8), as the MX specification prescribes; the quotient is rounded to nearest even and
// saturates at ±448.  Returns the biased exponent byte (0 for an all-zero block).
__device__ __forceinline__ uint8_t block_scale_byte(float amax, float& inv_scale) {
  if (!(amax > 0.f)) {
    inv_scale = 0.f;
    return 0;
  }
  int e = static_cast<int>((__float_as_uint(amax) >> 23) & 0xff) - 127;  // floor(log2 amax) for normal floats
  e -= 8;
  e = max(e, -127);
  e = min(e, 127);
  inv_scale = __uint_as_float(static_cast<uint32_t>(127 - e) << 23);  // 2^-e  (e ≥ -127 keeps this finite; e = 127 gives 2^-127 → denormal, flushed: amax that large does not occur in bf16 data)
  return static_cast<uint8_t>(e + 127);
}

__device__ __forceinline__ long long sf_offset(long long r, long long blk, long long chunks_per_row) {
  return ((r >> 7) * chunks_per_row + (blk >> 2)) * 512 + (r & 31) * 16 + ((r & 127) >> 5) * 4 + (blk & 3);
}

// q[r, c] = e4m3(src[r, c] / scale(r, c / 32)): blocks along the contiguous dimension.  One thread per block.
__global__ void __launch_bounds__(256)
mx_quantize_rows_kernel(const __nv_bfloat16* __restrict__ src, long long ld, uint8_t* __restrict__ q, long long ldq, uint8_t* __restrict__ sf, long long R,
                        long long C, long long chunks_per_row) {
  const long long nblk = C >> 5;
  const long long total = R * nblk;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total; i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long r = i / nblk, b = i - r * nblk;
    const uint4* s = reinterpret_cast<const uint4*>(src + r * ld + b * 32);
    uint4 raw[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) raw[j] = s[j];
    float v[32];
    float amax = 0.f;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw[j]);
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const float2 f = __bfloat1622float2(h[k]);
        v[j * 8 + 2 * k] = f.x, v[j * 8 + 2 * k + 1] = f.y;
        amax = fmaxf(amax, fmaxf(fabsf(f.x), fabsf(f.y)));
      }
    }
    float inv;
    sf[sf_offset(r, b, chunks_per_row)] = block_scale_byte(amax, inv);
    uint32_t out[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const uint32_t lo = __nv_cvt_float2_to_fp8x2(make_float2(v[4 * j] * inv, v[4 * j + 1] * inv), __NV_SATFINITE, __NV_E4M3);
      const uint32_t hi = __nv_cvt_float2_to_fp8x2(make_float2(v[4 * j + 2] * inv, v[4 * j + 3] * inv), __NV_SATFINITE, __NV_E4M3);
      out[j] = lo | (hi << 16);
    }
    uint4* d = reinterpret_cast<uint4*>(q + r * ldq + b * 32);
    d[0] = make_uint4(out[0], out[1], out[2], out[3]);
    d[1] = make_uint4(out[4], out[5], out[6], out[7]);
  }
}

// qT[c, r] = e4m3(src[r, c] / scale(c, r / 32)): the transposed operand with blocks along the source's row dimension (which is
// the contiguous dimension of the output).  One thread per (32-row group, column); neighbouring threads take neighbouring columns.
__global__ void __launch_bounds__(256)
mx_quantize_cols_kernel(const __nv_bfloat16* __restrict__ src, long long ld, uint8_t* __restrict__ qT, long long ldq, uint8_t* __restrict__ sf, long long R,
                        long long C, long long chunks_per_row) {
  const long long ngrp = R >> 5;
  const long long total = ngrp * C;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total; i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long g = i / C, c = i - g * C;
    const __nv_bfloat16* s = src + (g * 32) * ld + c;
    float v[32];
    float amax = 0.f;
#pragma unroll
    for (int j = 0; j < 32; ++j) {
      v[j] = __bfloat162float(s[j * ld]);
      amax = fmaxf(amax, fabsf(v[j]));
    }
    float inv;
    sf[sf_offset(c, g, chunks_per_row)] = block_scale_byte(amax, inv);
    uint32_t out[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const uint32_t lo = __nv_cvt_float2_to_fp8x2(make_float2(v[4 * j] * inv, v[4 * j + 1] * inv), __NV_SATFINITE, __NV_E4M3);
      const uint32_t hi = __nv_cvt_float2_to_fp8x2(make_float2(v[4 * j + 2] * inv, v[4 * j + 3] * inv), __NV_SATFINITE, __NV_E4M3);
      out[j] = lo | (hi << 16);
    }
    uint4* d = reinterpret_cast<uint4*>(qT + c * ldq + g * 32);
    d[0] = make_uint4(out[0], out[1], out[2], out[3]);
    d[1] = make_uint4(out[4], out[5], out[6], out[7]);
  }
}

// Both orientations in one pass over the source: q[r, c] with blocks along the columns and qT[c, r] with blocks along the rows.
// One warp per 32 × 32 tile: lane l loads row l (64 bytes), quantises it as a block of q, parks the fp32 values in shared memory
// and then quantises column l of the tile as a block of qT.  R and C are multiples of 32.
__global__ void __launch_bounds__(256)
mx_quantize_both_kernel(const __nv_bfloat16* __restrict__ src, long long ld, uint8_t* __restrict__ q, long long ldq, uint8_t* __restrict__ sf,
                        uint8_t* __restrict__ qT, long long ldqT, uint8_t* __restrict__ sfT, long long R, long long C) {
  __shared__ float tile[8][32][33];
  const int w = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const long long tiles_c = C >> 5;
  const long long total = (R >> 5) * tiles_c;
  const long long chunks_q = (C + 127) / 128, chunks_qT = (R + 127) / 128;
  for (long long t = blockIdx.x * 8LL + w; t < total; t += static_cast<long long>(gridDim.x) * 8) {
    const long long tr = t / tiles_c, tc = t - tr * tiles_c;
    const long long r = tr * 32 + lane;
    const uint4* s4 = reinterpret_cast<const uint4*>(src + r * ld + tc * 32);
    uint4 raw[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) raw[j] = s4[j];
    float v[32];
    float amax = 0.f;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw[j]);
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const float2 f = __bfloat1622float2(h[k]);
        v[j * 8 + 2 * k] = f.x, v[j * 8 + 2 * k + 1] = f.y;
        amax = fmaxf(amax, fmaxf(fabsf(f.x), fabsf(f.y)));
      }
    }
#pragma unroll
    for (int j = 0; j < 32; ++j) tile[w][lane][j] = v[j];
    float inv;
    sf[sf_offset(r, tc, chunks_q)] = block_scale_byte(amax, inv);
    uint32_t out[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const uint32_t lo = __nv_cvt_float2_to_fp8x2(make_float2(v[4 * j] * inv, v[4 * j + 1] * inv), __NV_SATFINITE, __NV_E4M3);
      const uint32_t hi = __nv_cvt_float2_to_fp8x2(make_float2(v[4 * j + 2] * inv, v[4 * j + 3] * inv), __NV_SATFINITE, __NV_E4M3);
      out[j] = lo | (hi << 16);
    }
    uint4* d = reinterpret_cast<uint4*>(q + r * ldq + tc * 32);
    d[0] = make_uint4(out[0], out[1], out[2], out[3]);
    d[1] = make_uint4(out[4], out[5], out[6], out[7]);
    __syncwarp();
    // column `lane` of the tile: 32 source rows = one block of the transposed operand
    amax = 0.f;
#pragma unroll
    for (int j = 0; j < 32; ++j) {
      v[j] = tile[w][j][lane];
      amax = fmaxf(amax, fabsf(v[j]));
    }
    const long long c = tc * 32 + lane;
    sfT[sf_offset(c, tr, chunks_qT)] = block_scale_byte(amax, inv);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const uint32_t lo = __nv_cvt_float2_to_fp8x2(make_float2(v[4 * j] * inv, v[4 * j + 1] * inv), __NV_SATFINITE, __NV_E4M3);
      const uint32_t hi = __nv_cvt_float2_to_fp8x2(make_float2(v[4 * j + 2] * inv, v[4 * j + 3] * inv), __NV_SATFINITE, __NV_E4M3);
      out[j] = lo | (hi << 16);
    }
    d = reinterpret_cast<uint4*>(qT + c * ldqT + tr * 32);
    d[0] = make_uint4(out[0], out[1], out[2], out[3]);
    d[1] = make_uint4(out[4], out[5], out[6], out[7]);
    __syncwarp();
  }
}

}  // namespace mx
}  // namespace ttb

// Bytes of the scale buffer of an operand with `rows` rows and `k` contraction columns (rows are padded to a multiple of 256 so
// that a 256-wide B tile always finds both of its chunks).
extern "C" long long ttb_mx_scale_bytes(long long rows, long long k) {
  return ((rows + 255) / 256) * 2 * ((k + 127) / 128) * 512;
}

// src: bf16 [R, C] (row pitch ld elements).  transpose = 0: q [R, C] (pitch ldq bytes), blocks of 32 along C, scale buffer of
// ttb_mx_scale_bytes(R, C) bytes.  transpose = 1: q [C, R], blocks of 32 along R, scale buffer of ttb_mx_scale_bytes(C, R) bytes.
// The scale buffer must be zero-filled by the caller (padding rows and blocks are never written).  The blocked dimension must be a
// multiple of 32, pitches multiples of 16 bytes.
extern "C" int ttb_mx_quantize(const void* src, long long ld, void* q, long long ldq, void* sf, long long R, long long C, int transpose, void* stream) {
  using namespace ttb;
  if (R <= 0 || C <= 0 || (ldq & 15)) return kErrBadShape;
  if ((reinterpret_cast<uintptr_t>(q) & 15)) return kErrBadShape;
  auto s = static_cast<cudaStream_t>(stream);
  const int grid = sm_count() * 8;
  TTB_COUNT_LAUNCH(1);
  if (!transpose) {
    if ((C & 31) || (ld & 7) || (reinterpret_cast<uintptr_t>(src) & 15)) return kErrBadShape;
    mx::mx_quantize_rows_kernel<<<grid, 256, 0, s>>>(static_cast<const __nv_bfloat16*>(src), ld, static_cast<uint8_t*>(q), ldq, static_cast<uint8_t*>(sf), R, C,
                                                    (C + 127) / 128);
  } else {
    if (R & 31) return kErrBadShape;
    mx::mx_quantize_cols_kernel<<<grid, 256, 0, s>>>(static_cast<const __nv_bfloat16*>(src), ld, static_cast<uint8_t*>(q), ldq, static_cast<uint8_t*>(sf), R, C,
                                                    (R + 127) / 128);
  }
  return cudaGetLastError() == cudaSuccess ? kOk : kErrDriver;
}

// Both operands of a tensor in one pass: q [R, C] with blocks along C and qT [C, R] with blocks along R (scale buffers sf / sfT
// zero-filled by the caller, sized by ttb_mx_scale_bytes(R, C) / (C, R)).  R and C are multiples of 32.
extern "C" int ttb_mx_quantize_both(const void* src, long long ld, void* q, long long ldq, void* sf, void* qT, long long ldqT, void* sfT, long long R, long long C,
                                    void* stream) {
  using namespace ttb;
  if (R <= 0 || C <= 0 || (R & 31) || (C & 31) || (ld & 7) || (ldq & 15) || (ldqT & 15)) return kErrBadShape;
  if ((reinterpret_cast<uintptr_t>(src) & 15) || (reinterpret_cast<uintptr_t>(q) & 15) || (reinterpret_cast<uintptr_t>(qT) & 15)) return kErrBadShape;
  const long long tiles = (R >> 5) * (C >> 5);
  long long grid = (tiles + 7) / 8;
  if (grid > sm_count() * 8LL) grid = sm_count() * 8LL;
  TTB_COUNT_LAUNCH(1);
  mx::mx_quantize_both_kernel<<<static_cast<unsigned>(grid), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(src), ld, static_cast<uint8_t*>(q), ldq, static_cast<uint8_t*>(sf), static_cast<uint8_t*>(qT), ldqT, static_cast<uint8_t*>(sfT), R, C);
  return cudaGetLastError() == cudaSuccess ? kOk : kErrDriver;
}

// A: [M, K] e4m3, B: [N, K] e4m3 (row pitches lda / ldb in bytes, multiples of 16), sfa / sfb: scale buffers as written by
// ttb_mx_quantize for these operands, C: [M, N] bf16 (ldc multiple of 8; accumulate != 0 adds to its contents).  K is a multiple of 32.
extern "C" int ttb_gemm_mxfp8(const void* A, const void* B, const void* sfa, const void* sfb, void* C, int M, int N, int K, long long lda, long long ldb,
                              long long ldc, const void* bias, int accumulate, int* err, void* stream) {
  using namespace ttb;
  if (M <= 0 || N <= 0 || K <= 0 || sfa == nullptr || sfb == nullptr) return kErrBadShape;
  if ((lda & 15) || (ldb & 15) || (ldc & 7) || (N & 7) || (K & 31)) return kErrBadShape;
  if ((reinterpret_cast<uintptr_t>(sfa) & 15) || (reinterpret_cast<uintptr_t>(sfb) & 15) || (reinterpret_cast<uintptr_t>(bias) & 15)) return kErrBadShape;
  mx::Params p;
  p.M = M, p.N = N, p.K = K, p.C = static_cast<__nv_bfloat16*>(C), p.ldc = ldc;
  p.sfa = static_cast<const uint8_t*>(sfa), p.sfb = static_cast<const uint8_t*>(sfb);
  p.bias = static_cast<const __nv_bfloat16*>(bias), p.accumulate = accumulate, p.err = err;
  CUtensorMap tmA, tmB;
  int rc = make_tmap_2d(&tmA, A, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, M, K, lda, mx::BM, mx::BK, CU_TENSOR_MAP_SWIZZLE_128B);
  if (rc != kOk) return rc;
  rc = make_tmap_2d(&tmB, B, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, N, K, ldb, mx::BN, mx::BK, CU_TENSOR_MAP_SWIZZLE_128B);
  if (rc != kOk) return rc;
  static bool attr_set = false;
  if (!attr_set) {
    if (cudaFuncSetAttribute(mx::gemm_mxfp8_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, mx::kSmemBytes) != cudaSuccess) return kErrDriver;
    attr_set = true;
  }
  const int num_tiles = ((M + mx::BM - 1) / mx::BM) * ((N + mx::BN - 1) / mx::BN);
  const int grid = num_tiles < sm_count() ? num_tiles : sm_count();
  TTB_COUNT_LAUNCH(1);
  mx::gemm_mxfp8_kernel<<<grid, mx::kThreads, mx::kSmemBytes, static_cast<cudaStream_t>(stream)>>>(tmA, tmB, p);
  return cudaGetLastError() == cudaSuccess ? kOk : kErrDriver;
}
