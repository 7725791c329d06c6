// bf16 GEMM on pairs of SMs: tcgen05.mma.cta_group::2 with a 256 x 256 output tile per CTA pair.
//
//   C[M,N] (+)= alpha * op(A) * op(B)  (+ bias[N])        (bf16 in, fp32 accumulate in TMEM, bf16 out)
//
// Two CTAs of a thread-block cluster (adjacent SMs) work on one tile.  CTA r of the pair loads rows
// [m0 + 128 r, m0 + 128 r + 128) of A and rows [n0 + 128 r, n0 + 128 r + 128) of B into its own shared memory (plain
// tiled TMA loads of this GPU's memory, no multicast); one thread of the even CTA issues the MMAs, which read both
// CTAs' operand tiles and write 128 accumulator rows into each CTA's tensor memory.  Compared with one CTA per
// 128 x 256 tile every B byte is fetched from L2 and written to shared memory once per 256 output rows instead of once
// per 128, and each SM holds half the operand bytes per k-block, which lifts the shared-memory and L2 traffic per
// FLOP that bounds the single-CTA kernel.
//
// Per CTA: warp 0 TMA producer, warp 1 MMA issuer (even CTA only), warp 2 TMEM allocator, warps 4-7 epilogue.
// Barriers: `full` lives in the even CTA and counts the bytes of both CTAs' loads; `empty` and `tfull` exist in both
// CTAs and are signalled by multicast commits; `tempty` lives in the even CTA and collects the eight epilogue warps.
// Every wait is bounded (error word + abort flag), the two CTAs meet at a cluster barrier before TMEM is released.
#include <cstdlib>
#include <cstring>

#include "common/ptx.cuh"
#include "common/tmap.h"

namespace ttb {
namespace g2 {

static constexpr int BM = 128;   // rows per CTA
static constexpr int PM = 256;   // rows per CTA pair
static constexpr int BN = 256;   // columns per pair tile (each CTA loads 128 of them)
static constexpr int BK = 64;
static constexpr int kThreads = 256;
static constexpr int kGroupM = 16;  // default number of pair-tiles in m per scheduling group (L2 reuse of the B panel)
static constexpr int kABytes = BM * BK * 2;
static constexpr int kBBytes = (BN / 2) * BK * 2;
static constexpr int kStageBytes = kABytes + kBBytes;  // 32 KB per CTA and stage
static constexpr int kStages = 6;
static constexpr int kEpiBytes = 4 * 2 * 4096;  // per epilogue warp two 32 x 64 bf16 staging tiles
static constexpr int kSmemBytes = kStages * kStageBytes + 1024 /*barriers*/ + kEpiBytes + 1024 /*align slack*/;
static_assert(kSmemBytes <= 232448, "shared memory budget of one CTA");
// the SwiGLU form gives one pipeline stage to two more staging tiles per epilogue warp
static constexpr int kStagesSwiglu = 5;
static constexpr int kSmemBytesSwiglu = kStagesSwiglu * kStageBytes + 1024 + 2 * kEpiBytes + 1024;
static_assert(kSmemBytesSwiglu <= 232448, "shared memory budget of one CTA");

struct Params {
  int M, N, K;
  int K2;  // > 0: a second operand pair (tmA2, tmB2) with K2 contraction columns extends the main loop (LoRA: one accumulator)
  void* C;
  long long ldc;
  const __nv_bfloat16* bias;
  const __nv_bfloat16* residual;  // [M, N] (row pitch ldr) added to the product in the epilogue (the residual stream of a decoder layer), or null
  long long ldr;
  float alpha;
  int accumulate;
  int tma_store;
  int group_m;  // pair-tiles in m per scheduling group
  int tile_mult;  // 1, or an odd multiplier coprime to the tile count: tile t is replaced by (t · tile_mult) mod tiles (debug aid)
  int save_gate_up;  // SWIGLU form: also store the two pre-activations (the backward pass needs them)
  int* err;
};

__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ void cluster_sync() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// shared::cluster address of `p` (an address in this CTA's shared memory) as seen in CTA `rank` of the cluster
__device__ __forceinline__ uint32_t map_to_cta(const void* p, uint32_t rank) {
  uint32_t out;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(out) : "r"(smem_u32(p)), "r"(rank));
  return out;
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
// Tiled load into this CTA's shared memory whose byte count is credited to a barrier of the pair's even CTA.
__device__ __forceinline__ void tma_load_2d_pair(void* smem_dst, const CUtensorMap* m, uint32_t bar_cluster_addr, int x, int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(m)), "r"(bar_cluster_addr), "r"(x), "r"(y)
      : "memory");
}
__device__ __forceinline__ void tmem_alloc_pair(uint32_t* smem_result, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_result)), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish_pair() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void umma_f16_pair(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
      : "memory");
}
// Arrive on the barrier at this shared-memory offset in both CTAs of the pair once the MMAs issued so far have completed.
__device__ __forceinline__ void umma_commit_pair(uint64_t* bar) {
  const uint16_t mask = 3;
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;" ::"r"(smem_u32(bar)), "h"(mask)
               : "memory");
}

__device__ __forceinline__ void tile_coords(int t, int num_m, int num_n, int group_m, int& m_blk, int& n_blk) {
  const int per_group = group_m * num_n;
  const int group = t / per_group;
  const int first_m = group * group_m;
  const int gsize = min(group_m, num_m - first_m);
  const int r = t - group * per_group;
  m_blk = first_m + r % gsize;
  n_blk = r / gsize;
}

// SWIGLU: the pair's two B halves come from *two* weight matrices — the even CTA loads 128 rows of the gate projection (tmB), the odd
// CTA the same 128 rows of the up projection (tmB2) — so accumulator columns [0, 128) hold the gate and [128, 256) the up pre-activations
// of the same 128 hidden units, in both CTAs' tensor memory.  The epilogue writes h = silu(gate) · up ([M, N], N = hidden width; tmC) and,
// when the backward pass will need them, gate and up as well (tmG, tmU).  The separate SwiGLU kernel and its re-read of both
// pre-activations disappear; in a gradient-free forward pass the pre-activations never reach HBM at all.
template <bool A_MN, bool B_MN, bool SWIGLU>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kThreads, 1)
gemm2sm_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, const __grid_constant__ CUtensorMap tmC,
               const __grid_constant__ CUtensorMap tmB2, const __grid_constant__ CUtensorMap tmG, const __grid_constant__ CUtensorMap tmU,
               const __grid_constant__ CUtensorMap tmA2, Params p) {
  constexpr int kNS = SWIGLU ? kStagesSwiglu : kStages;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + kNS * kStageBytes);
  uint64_t* full = bars;                 // [kNS]  used in the even CTA
  uint64_t* empty = bars + kNS;      // [kNS]  both CTAs
  uint64_t* tfull = bars + 2 * kNS;  // [2]        both CTAs
  uint64_t* tempty = tfull + 2;          // [2]        used in the even CTA
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tempty + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  uint8_t* epi = smem + kNS * kStageBytes + 1024;
  uint8_t* epi_extra = epi + kEpiBytes;  // SWIGLU: per epilogue warp one more pair of staging tiles (gate, up)

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t cta = cluster_ctarank();  // 0: issues the MMAs
  const int pair = blockIdx.x >> 1;
  const int num_pairs = gridDim.x >> 1;
  const int num_m = (p.M + PM - 1) / PM;
  constexpr int kTileN = SWIGLU ? BN / 2 : BN;  // output columns per tile
  const int num_n = (p.N + kTileN - 1) / kTileN;
  const int num_tiles = num_m * num_n;
  // without SWIGLU, tmA2 / tmB2 are the second operand pair: its k-blocks (zero-filled past K2 by the tensor maps) follow the first pair's
  const int num_kb1 = (p.K + BK - 1) / BK;
  const int num_kb = num_kb1 + ((!SWIGLU && p.K2 > 0) ? (p.K2 + BK - 1) / BK : 0);

  if (threadIdx.x == 0) {
    for (int i = 0; i < kNS; ++i) {
      mbar_init(&full[i], 1);
      mbar_init(&empty[i], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&tfull[i], 1);
      mbar_init(&tempty[i], 8);
    }
    *abort_flag = 0;
    fence_mbar_init();
  }
  if (warp == 0 && lane == 0) {
    prefetch_tmap(&tmA);
    prefetch_tmap(&tmB);
    if (SWIGLU || p.K2 > 0) prefetch_tmap(&tmB2);
    if (!SWIGLU && p.K2 > 0) prefetch_tmap(&tmA2);
  }
  __syncthreads();
  if (warp == 2) {
    tmem_alloc_pair(tmem_slot, 512);
    tmem_relinquish_pair();
  }
  tc_fence_before();
  cluster_sync();  // both CTAs' barriers are initialised and both hold their tensor memory before anything crosses over
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer (both CTAs)
    int stage = 0;
    uint32_t phase = 0;
    for (int t = pair; t < num_tiles && !*abort_flag; t += num_pairs) {
      int m_blk, n_blk;
      tile_coords(p.tile_mult == 1 ? t : static_cast<int>((static_cast<long long>(t) * p.tile_mult) % num_tiles), num_m, num_n, p.group_m, m_blk, n_blk);
      const int a_row = m_blk * PM + static_cast<int>(cta) * BM;
      const int b_row = SWIGLU ? n_blk * (BN / 2) : n_blk * BN + static_cast<int>(cta) * (BN / 2);
      const CUtensorMap* mapB = (SWIGLU && cta == 1) ? &tmB2 : &tmB;
      for (int kb = 0; kb < num_kb; ++kb) {
        if (!mbar_wait(&empty[stage], phase ^ 1)) {
          *abort_flag = 1;
          if (lane == 0) atomicExch(p.err, 111);
          break;
        }
        if (lane == 0) {
          uint8_t* sa = smem + stage * kStageBytes;
          uint8_t* sb = sa + kABytes;
          if (cta == 0) mbar_arrive_expect_tx(&full[stage], 2 * kStageBytes);  // the bytes of both CTAs' loads
          const uint32_t bar = map_to_cta(&full[stage], 0);
          const bool second = !SWIGLU && kb >= num_kb1;
          const CUtensorMap* mA = second ? &tmA2 : &tmA;
          const CUtensorMap* mB = second ? &tmB2 : mapB;
          const int k0 = (second ? kb - num_kb1 : kb) * BK;
          if (A_MN) {
#pragma unroll
            for (int j = 0; j < BM / 64; ++j) tma_load_2d_pair(sa + j * 8192, mA, bar, a_row + j * 64, k0);
          } else {
            tma_load_2d_pair(sa, mA, bar, k0, a_row);
          }
          if (B_MN) {
#pragma unroll
            for (int j = 0; j < (BN / 2) / 64; ++j) tma_load_2d_pair(sb + j * 8192, mB, bar, b_row + j * 64, k0);
          } else {
            tma_load_2d_pair(sb, mB, bar, k0, b_row);
          }
        }
        __syncwarp();
        if (++stage == kNS) {
          stage = 0;
          phase ^= 1;
        }
      }
    }
  } else if (warp == 1 && cta == 0) {
    // ------------------------------------------------------------------ MMA issuer (even CTA)
    constexpr uint32_t idesc = make_idesc_bf16(PM, BN, A_MN, B_MN);
    int stage = 0;
    uint32_t phase = 0;
    int acc = 0;
    uint32_t acc_phase = 0;
    for (int t = pair; t < num_tiles && !*abort_flag; t += num_pairs) {
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
          const uint32_t sa = smem_u32(smem + stage * kStageBytes);
          const uint32_t sb = sa + kABytes;
#pragma unroll
          for (int k = 0; k < BK / 16; ++k) {
            const uint64_t da = A_MN ? make_smem_desc_sw128(sa + k * 2048, 8192, 1024) : make_smem_desc_sw128(sa + k * 32, 16, 1024);
            const uint64_t db = B_MN ? make_smem_desc_sw128(sb + k * 2048, 8192, 1024) : make_smem_desc_sw128(sb + k * 32, 16, 1024);
            umma_f16_pair(d_tmem, da, db, idesc, (kb | k) != 0);
          }
          umma_commit_pair(&empty[stage]);  // both CTAs' producers may refill the stage once these MMAs retire
        }
        __syncwarp();
        if (++stage == kNS) {
          stage = 0;
          phase ^= 1;
        }
      }
      if (!ok) {
        *abort_flag = 1;
        if (lane == 0) atomicExch(p.err, 113);
        break;
      }
      if (lane == 0) umma_commit_pair(&tfull[acc]);
      __syncwarp();
      if (++acc == 2) {
        acc = 0;
        acc_phase ^= 1;
      }
    }
  } else if (warp >= 4) {
    // ------------------------------------------------------------------ epilogue (both CTAs, own 128 rows)
    const int quarter = warp & 3;
    int acc = 0;
    uint32_t acc_phase = 0;
    int buf_toggle = 0;
    uint8_t* my_stage = epi + quarter * 8192;
    for (int t = pair; t < num_tiles && !*abort_flag; t += num_pairs) {
      int m_blk, n_blk;
      tile_coords(p.tile_mult == 1 ? t : static_cast<int>((static_cast<long long>(t) * p.tile_mult) % num_tiles), num_m, num_n, p.group_m, m_blk, n_blk);
      if (!mbar_wait(&tfull[acc], acc_phase)) {
        *abort_flag = 1;
        if (lane == 0) atomicExch(p.err, 114);
        break;
      }
      tc_fence_after();
      const int row0 = m_blk * PM + static_cast<int>(cta) * BM + quarter * 32;
      const int row = row0 + lane;
      const uint32_t taddr = tmem_base + acc * BN + (static_cast<uint32_t>(quarter * 32) << 16);
      if (SWIGLU) {
        // gate = columns [0, 128), up = columns [128, 256) of this CTA's rows; 64 output columns per staged sub-tile
#pragma unroll 1
        for (int c = 0; c < 2; ++c) {
          const int col0 = n_blk * (BN / 2) + c * 64;
          if (col0 >= p.N || row0 >= p.M) break;
          uint8_t* buf_h = my_stage + (buf_toggle & 1) * 4096;
          if (lane == 0) tma_store_wait_read<0>();  // the three stores of the previous sub-tile have read their buffers
          __syncwarp();
          uint8_t* buf_g = epi_extra + quarter * 8192;
          uint8_t* buf_u = buf_g + 4096;
#pragma unroll
          for (int h = 0; h < 2; ++h) {
            uint32_t rg[32], ru[32];
            tmem_ld_32x32(taddr + c * 64 + h * 32, rg);
            tmem_ld_32x32(taddr + 128 + c * 64 + h * 32, ru);
            tmem_ld_wait();
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              float g[8], u[8], o[8];
#pragma unroll
              for (int i = 0; i < 8; ++i) {
                // round the pre-activations to bf16 first: the unfused path computes SwiGLU from the stored bf16 values
                g[i] = __bfloat162float(__float2bfloat16_rn(__uint_as_float(rg[j * 8 + i])));
                u[i] = __bfloat162float(__float2bfloat16_rn(__uint_as_float(ru[j * 8 + i])));
                o[i] = g[i] / (1.f + __expf(-g[i])) * u[i];
              }
              const int chunk = (h * 4 + j) ^ (lane & 7);
              uint4 v;
              v.x = pack_bf16x2(o[0], o[1]), v.y = pack_bf16x2(o[2], o[3]), v.z = pack_bf16x2(o[4], o[5]), v.w = pack_bf16x2(o[6], o[7]);
              *reinterpret_cast<uint4*>(buf_h + lane * 128 + chunk * 16) = v;
              if (p.save_gate_up) {
                v.x = pack_bf16x2(g[0], g[1]), v.y = pack_bf16x2(g[2], g[3]), v.z = pack_bf16x2(g[4], g[5]), v.w = pack_bf16x2(g[6], g[7]);
                *reinterpret_cast<uint4*>(buf_g + lane * 128 + chunk * 16) = v;
                v.x = pack_bf16x2(u[0], u[1]), v.y = pack_bf16x2(u[2], u[3]), v.z = pack_bf16x2(u[4], u[5]), v.w = pack_bf16x2(u[6], u[7]);
                *reinterpret_cast<uint4*>(buf_u + lane * 128 + chunk * 16) = v;
              }
            }
          }
          fence_proxy_async_smem();
          __syncwarp();
          if (lane == 0) {
            tma_store_2d(&tmC, buf_h, col0, row0);
            if (p.save_gate_up) {
              tma_store_2d(&tmG, buf_g, col0, row0);
              tma_store_2d(&tmU, buf_u, col0, row0);
            }
            tma_store_commit();
          }
          ++buf_toggle;
        }
      } else if (p.tma_store) {
#pragma unroll 1
        for (int c = 0; c < BN / 64; ++c) {
          const int col0 = n_blk * BN + c * 64;
          if (col0 >= p.N || row0 >= p.M) break;
          uint8_t* buf = my_stage + (buf_toggle & 1) * 4096;
          if (lane == 0) tma_store_wait_read<1>();
          __syncwarp();
#pragma unroll
          for (int h = 0; h < 2; ++h) {
            uint32_t r[32];
            tmem_ld_32x32(taddr + c * 64 + h * 32, r);
            tmem_ld_wait();
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              float f[8];
#pragma unroll
              for (int i = 0; i < 8; ++i) f[i] = __uint_as_float(r[j * 8 + i]) * p.alpha;
              if (p.bias != nullptr) {
                const int cb = col0 + h * 32 + j * 8;
#pragma unroll
                for (int i = 0; i < 8; ++i)
                  if (cb + i < p.N) f[i] += __bfloat162float(__ldg(p.bias + cb + i));
              }
              if (p.residual != nullptr) {
                const int cb = col0 + h * 32 + j * 8;
                if (row < p.M && cb + 8 <= p.N) {
                  const uint4 rq = __ldg(reinterpret_cast<const uint4*>(p.residual + static_cast<long long>(row) * p.ldr + cb));
                  const __nv_bfloat162* rb = reinterpret_cast<const __nv_bfloat162*>(&rq);
#pragma unroll
                  for (int i = 0; i < 4; ++i) {
                    const float2 t = __bfloat1622float2(rb[i]);
                    f[2 * i] += t.x, f[2 * i + 1] += t.y;
                  }
                }
              }
              uint4 o;
              o.x = pack_bf16x2(f[0], f[1]);
              o.y = pack_bf16x2(f[2], f[3]);
              o.z = pack_bf16x2(f[4], f[5]);
              o.w = pack_bf16x2(f[6], f[7]);
              const int chunk = (h * 4 + j) ^ (lane & 7);
              *reinterpret_cast<uint4*>(buf + lane * 128 + chunk * 16) = o;
            }
          }
          fence_proxy_async_smem();
          __syncwarp();
          if (lane == 0) {
            tma_store_2d(&tmC, buf, col0, row0);
            tma_store_commit();
          }
          ++buf_toggle;
        }
      } else {
#pragma unroll 1
        for (int c = 0; c < BN / 32; ++c) {
          uint32_t r[32];
          tmem_ld_32x32(taddr + c * 32, r);
          tmem_ld_wait();
          const int col0 = n_blk * BN + c * 32;
          if (row < p.M && col0 < p.N) {
            float v[32];
#pragma unroll
            for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]) * p.alpha;
            if (p.bias != nullptr) {
#pragma unroll
              for (int i = 0; i < 32; ++i)
                if (col0 + i < p.N) v[i] += __bfloat162float(__ldg(p.bias + col0 + i));
            }
            if (p.residual != nullptr) {
              const __nv_bfloat16* rr = p.residual + static_cast<long long>(row) * p.ldr + col0;
#pragma unroll
              for (int g = 0; g < 4; ++g) {
                if (col0 + g * 8 + 8 <= p.N) {
                  const uint4 rq = __ldg(reinterpret_cast<const uint4*>(rr + g * 8));
                  const __nv_bfloat162* rb = reinterpret_cast<const __nv_bfloat162*>(&rq);
#pragma unroll
                  for (int i = 0; i < 4; ++i) {
                    const float2 t = __bfloat1622float2(rb[i]);
                    v[g * 8 + 2 * i] += t.x, v[g * 8 + 2 * i + 1] += t.y;
                  }
                }
              }
            }
            __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(p.C) + static_cast<long long>(row) * p.ldc + col0;
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
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(map_to_cta(&tempty[acc], 0));  // the accumulator is free again: tell the even CTA
      if (++acc == 2) {
        acc = 0;
        acc_phase ^= 1;
      }
    }
    if (lane == 0) tma_store_wait<0>();
  }

  // Neither CTA may leave (or give its tensor memory back) while the other one's MMAs, commits or loads can still touch it.
  tc_fence_before();
  __syncthreads();
  cluster_sync();
  tc_fence_after();
  if (warp == 2) tmem_dealloc_pair(tmem_base, 512);
}

// TTB_SHUFFLE_TILES=<n> (debug aid, default off): tiles are visited in the order (t · m) mod tiles with m the first odd number ≥ n
// that is coprime to the tile count.  Results must not depend on the order tiles are computed in; a test that passes with and
// without the variable shows that no tile reads what another one has not written yet.
static int shuffle_multiplier(int num_tiles) {
  static int want = -1;
  if (want < 0) {
    const char* e = getenv("TTB_SHUFFLE_TILES");
    want = (e != nullptr && atoi(e) > 1) ? atoi(e) : 0;
  }
  if (want == 0 || num_tiles < 3) return 1;
  auto gcd = [](int a, int b) {
    while (b) {
      const int t = a % b;
      a = b, b = t;
    }
    return a;
  };
  int m = (want % num_tiles) | 1;
  while (gcd(m, num_tiles) != 1) m += 2;
  return m;
}

template <bool A_MN, bool B_MN, bool SWIGLU>
static int launch(const void* A, const void* B, const void* B2, void* G, void* U, const Params& p, long long lda, long long ldb, cudaStream_t stream,
                  const void* A2 = nullptr, long long lda2 = 0, long long ldb2 = 0) {
  CUtensorMap tmA, tmB, tmB2, tmC, tmG, tmU, tmA2;
  memset(&tmA2, 0, sizeof(tmA2));
  memset(&tmB2, 0, sizeof(tmB2));
  memset(&tmG, 0, sizeof(tmG));
  memset(&tmU, 0, sizeof(tmU));
  int rc;
  if (A_MN)
    rc = make_tmap_2d(&tmA, A, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, p.K, p.M, lda, BK, 64, CU_TENSOR_MAP_SWIZZLE_128B);
  else
    rc = make_tmap_2d(&tmA, A, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, p.M, p.K, lda, BM, BK, CU_TENSOR_MAP_SWIZZLE_128B);
  if (rc != kOk) return rc;
  auto map_b = [&](CUtensorMap* m, const void* ptr) {
    return B_MN ? make_tmap_2d(m, ptr, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, p.K, p.N, ldb, BK, 64, CU_TENSOR_MAP_SWIZZLE_128B)
                : make_tmap_2d(m, ptr, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, p.N, p.K, ldb, BN / 2, BK, CU_TENSOR_MAP_SWIZZLE_128B);
  };
  if ((rc = map_b(&tmB, B)) != kOk) return rc;
  if (SWIGLU && (rc = map_b(&tmB2, B2)) != kOk) return rc;
  if (!SWIGLU && p.K2 > 0) {  // second operand pair: same layouts as the first, its own pitches and contraction length
    if (A_MN)
      rc = make_tmap_2d(&tmA2, A2, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, p.K2, p.M, lda2, BK, 64, CU_TENSOR_MAP_SWIZZLE_128B);
    else
      rc = make_tmap_2d(&tmA2, A2, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, p.M, p.K2, lda2, BM, BK, CU_TENSOR_MAP_SWIZZLE_128B);
    if (rc != kOk) return rc;
    rc = B_MN ? make_tmap_2d(&tmB2, B2, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, p.K2, p.N, ldb2, BK, 64, CU_TENSOR_MAP_SWIZZLE_128B)
              : make_tmap_2d(&tmB2, B2, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, p.N, p.K2, ldb2, BN / 2, BK, CU_TENSOR_MAP_SWIZZLE_128B);
    if (rc != kOk) return rc;
  }
  Params q = p;
  memset(&tmC, 0, sizeof(tmC));
  auto map_c = [&](CUtensorMap* m, void* ptr) {
    return make_tmap_2d(m, ptr, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, p.M, p.N, p.ldc, 32, 64, CU_TENSOR_MAP_SWIZZLE_128B);
  };
  if (SWIGLU) {
    if ((reinterpret_cast<uintptr_t>(p.C) & 15) || map_c(&tmC, p.C) != kOk) return kErrBadShape;
    q.save_gate_up = (G != nullptr && U != nullptr) ? 1 : 0;
    if (q.save_gate_up && (map_c(&tmG, G) != kOk || map_c(&tmU, U) != kOk)) return kErrBadShape;
    q.tma_store = 1;
  } else {
    q.tma_store = (!p.accumulate && (reinterpret_cast<uintptr_t>(p.C) & 15) == 0 && map_c(&tmC, p.C) == kOk) ? 1 : 0;
  }
  auto kern = gemm2sm_kernel<A_MN, B_MN, SWIGLU>;
  constexpr int smem = SWIGLU ? kSmemBytesSwiglu : kSmemBytes;
  static bool attr_set = false;
  if (!attr_set) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess) return kErrDriver;
    attr_set = true;
  }
  const int num_tiles = ((p.M + PM - 1) / PM) * ((p.N + (SWIGLU ? BN / 2 : BN) - 1) / (SWIGLU ? BN / 2 : BN));
  q.tile_mult = shuffle_multiplier(num_tiles);
  const int max_pairs = sm_count() / 2;
  const int pairs = num_tiles < max_pairs ? num_tiles : max_pairs;
  TTB_COUNT_LAUNCH(1);
  kern<<<2 * pairs, kThreads, smem, stream>>>(tmA, tmB, tmC, tmB2, tmG, tmU, tmA2, q);
  return cudaGetLastError() == cudaSuccess ? kOk : kErrDriver;
}

static int group_setting() {
  static int group_m = 0;
  if (group_m == 0) {
    const char* e = getenv("TTB_G2_GROUP_M");
    group_m = (e != nullptr && atoi(e) > 0) ? atoi(e) : kGroupM;
  }
  return group_m;
}

}  // namespace g2
}  // namespace ttb

// C[M,N] (+)= alpha * op(A) * op(B) (+ bias) on CTA pairs; bf16 operands and output.  Same operand conventions as ttb_gemm_bf16:
// a_mn = 0: A is [M, K] row-major (lda = row pitch), 1: A is [K, M]; b_mn = 0: B is [N, K], 1: B is [K, N].
extern "C" int ttb_gemm_bf16_2sm(const void* A, const void* B, void* C, int M, int N, int K, int a_mn, int b_mn, long long lda,
                                 long long ldb, long long ldc, int accumulate, const void* bias, float alpha, int* err, void* stream) {
  using namespace ttb;
  if (M <= 0 || N <= 0 || K <= 0) return kErrBadShape;
  if ((lda & 7) || (ldb & 7) || (ldc & 7) || (N & 7)) return kErrBadShape;
  if ((a_mn ? (M & 7) : (K & 7)) || (b_mn ? (N & 7) : (K & 7))) return kErrBadShape;
  g2::Params p;
  p.M = M, p.N = N, p.K = K, p.C = C, p.ldc = ldc, p.bias = static_cast<const __nv_bfloat16*>(bias), p.alpha = alpha;
  p.accumulate = accumulate, p.tma_store = 0, p.save_gate_up = 0, p.tile_mult = 1, p.err = err, p.K2 = 0;
  p.residual = nullptr, p.ldr = 0;
  p.group_m = g2::group_setting();
  auto s = static_cast<cudaStream_t>(stream);
  if (a_mn) return b_mn ? g2::launch<true, true, false>(A, B, nullptr, nullptr, nullptr, p, lda, ldb, s) : g2::launch<true, false, false>(A, B, nullptr, nullptr, nullptr, p, lda, ldb, s);
  return b_mn ? g2::launch<false, true, false>(A, B, nullptr, nullptr, nullptr, p, lda, ldb, s) : g2::launch<false, false, false>(A, B, nullptr, nullptr, nullptr, p, lda, ldb, s);
}

// C[M,N] = alpha · (A·op(B) + A2·op(B2)) (+ bias) on CTA pairs: the second pair's k-blocks (K2 columns, zero-filled up to a multiple of
// 64 by the tensor maps) extend the main loop, so base and adapter products of a LoRA linear share one accumulator
// (torchtune/modules/peft/lora.py:128-147).  A and A2 are [M, K] / [M, K2] row-major; b_mn = 0: B [N, K], B2 [N, K2]; 1: B [K, N], B2 [K2, N].
extern "C" int ttb_gemm_bf16_dual_2sm(const void* A, const void* B, const void* A2, const void* B2, void* C, int M, int N, int K, int K2, int b_mn,
                                      long long lda, long long ldb, long long lda2, long long ldb2, long long ldc, const void* bias, float alpha,
                                      int* err, void* stream) {
  using namespace ttb;
  if (M <= 0 || N <= 0 || K <= 0 || K2 <= 0 || A2 == nullptr || B2 == nullptr) return kErrBadShape;
  if ((lda & 7) || (ldb & 7) || (lda2 & 7) || (ldb2 & 7) || (ldc & 7) || (N & 7) || (K & 7) || (K2 & 7)) return kErrBadShape;
  g2::Params p;
  p.M = M, p.N = N, p.K = K, p.K2 = K2, p.C = C, p.ldc = ldc, p.bias = static_cast<const __nv_bfloat16*>(bias), p.alpha = alpha;
  p.residual = nullptr, p.ldr = 0;
  p.accumulate = 0, p.tma_store = 0, p.save_gate_up = 0, p.tile_mult = 1, p.err = err;
  p.group_m = g2::group_setting();
  auto s = static_cast<cudaStream_t>(stream);
  return b_mn ? g2::launch<false, true, false>(A, B, B2, nullptr, nullptr, p, lda, ldb, s, A2, lda2, ldb2)
              : g2::launch<false, false, false>(A, B, B2, nullptr, nullptr, p, lda, ldb, s, A2, lda2, ldb2);
}

// Gated MLP up-projection with the activation in the epilogue: H[M, N] = silu(X · W1ᵀ) ⊙ (X · W3ᵀ) with X [M, K], W1 and W3 [N, K]
// (row pitches lda, ldb; all bf16).  gate_out / up_out (both or neither; [M, N], row pitch ldc) receive the two pre-activations
// rounded to bf16, which is what the backward pass of the unfused form would have read.
extern "C" int ttb_gemm_swiglu_bf16_2sm(const void* X, const void* W1, const void* W3, void* H, void* gate_out, void* up_out, int M, int N, int K,
                                        long long lda, long long ldb, long long ldc, int* err, void* stream) {
  using namespace ttb;
  if (M <= 0 || N <= 0 || K <= 0) return kErrBadShape;
  if ((lda & 7) || (ldb & 7) || (ldc & 7) || (N & 7) || (K & 7)) return kErrBadShape;
  if ((gate_out == nullptr) != (up_out == nullptr)) return kErrBadShape;
  g2::Params p;
  p.M = M, p.N = N, p.K = K, p.C = H, p.ldc = ldc, p.bias = nullptr, p.alpha = 1.f;
  p.residual = nullptr, p.ldr = 0;
  p.accumulate = 0, p.tma_store = 1, p.save_gate_up = 0, p.tile_mult = 1, p.err = err, p.K2 = 0;
  p.group_m = g2::group_setting();
  return g2::launch<false, false, true>(X, W1, W3, gate_out, up_out, p, lda, ldb, static_cast<cudaStream_t>(stream));
}


// C[M,N] = A[M,K] · B[N,K]ᵀ (+ bias) + R[M,N]: a linear layer whose output is added to the residual stream in the GEMM epilogue (the
// attention output projection and the MLP down projection of a decoder layer, torchtune/modules/transformer.py:119-135), so the separate
// element-wise add and its re-read of both tensors disappear.  R: bf16, row pitch ldr (multiple of 8), 16-byte aligned; R may not alias C.
extern "C" int ttb_gemm_bf16_2sm_residual(const void* A, const void* B, void* C, const void* R, int M, int N, int K, long long lda, long long ldb, long long ldc,
                                          long long ldr, const void* bias, int* err, void* stream) {
  using namespace ttb;
  if (M <= 0 || N <= 0 || K <= 0 || R == nullptr) return kErrBadShape;
  if ((lda & 7) || (ldb & 7) || (ldc & 7) || (ldr & 7) || (N & 7) || (K & 7) || (reinterpret_cast<uintptr_t>(R) & 15)) return kErrBadShape;
  g2::Params p;
  p.M = M, p.N = N, p.K = K, p.K2 = 0, p.C = C, p.ldc = ldc, p.bias = static_cast<const __nv_bfloat16*>(bias), p.alpha = 1.f;
  p.residual = static_cast<const __nv_bfloat16*>(R), p.ldr = ldr;
  p.accumulate = 0, p.tma_store = 0, p.save_gate_up = 0, p.tile_mult = 1, p.err = err;
  p.group_m = g2::group_setting();
  return g2::launch<false, false, false>(A, B, nullptr, nullptr, nullptr, p, lda, ldb, static_cast<cudaStream_t>(stream));
}
