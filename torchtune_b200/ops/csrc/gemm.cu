// bf16 GEMM on the 5th-generation tensor cores (tcgen05) with TMEM accumulators.
//
//   C[M,N] (+)= alpha * op(A) * op(B)  (+ bias[N])
//
// Persistent, warp-specialised kernel, one CTA per SM:
//   warp 0   TMA producer   (cp.async.bulk.tensor -> 128B-swizzled smem ring, mbarrier tx-count)
//   warp 1   MMA issuer     (one lane issues tcgen05.mma, tcgen05.commit releases smem / signals epilogue)
//   warp 2   TMEM allocator (2 x BN fp32 columns: the epilogue of tile i overlaps the main loop of tile i+1)
//   warps 4-7 epilogue      (tcgen05.ld 32 lanes x 32 columns per warp -> registers -> bf16/fp32 global stores)
//
// Operand layouts: an operand is "K-major" when the contraction index is contiguous
// (X[rows, K]) and "MN-major" when the row/column index is contiguous (X[K, rows]); both are
// consumed directly through the shared-memory matrix descriptor, so forward (NT), dgrad (NN)
// and wgrad (TN) need no transposes.  Serves every nn.Linear of the decoder
// (reference call sites: torchtune/modules/attention.py:234,262-263,303,
// torchtune/modules/feed_forward.py:50-53).
#include <cstring>

#include "common/ptx.cuh"
#include "common/tmap.h"

namespace ttb {

static constexpr int BM = 128;
static constexpr int BK = 64;  // 64 bf16 = 128 bytes = one swizzle row
static constexpr int kThreads = 256;
static constexpr int kGroupM = 16;  // m-tiles per scheduling group (L2 reuse of the B panel)

struct GemmParams {
  int M, N, K;
  void* C;
  long long ldc;
  const __nv_bfloat16* bias;  // [N] or nullptr
  float alpha;
  int out_fp32;    // 0: bf16 C, 1: fp32 C
  int accumulate;  // 1: C += result
  int* err;        // device error word (0 = ok)
  int K2 = 0;         // plain kernel: extent of a second operand pair whose product is accumulated into the same tile
                      // (C = A·op(B) + A2·op(B2), e.g. base weight + low-rank adapter); 0 = none
  int splits = 1;     // plain kernel, fp32 output: the contraction is cut into `splits` ranges, one tile per (m, n, range), partial
                      // sums added with vector atomics into a zero-initialised (or accumulated-into) C — for skinny outputs
                      // whose few tiles would otherwise leave most SMs idle (adapter weight gradients)
  int tma_store = 0;  // 1: bf16 output without accumulation leaves through shared memory + TMA stores (plain kernel)
};

// Tensor-parallel variants of the same kernel (TP template parameter of gemm_body):
//   1  all-gather → GEMM: the M dimension is the concatenation over ranks of per-rank activation shards that live
//      in peer-visible buffers.  Peer memory is not cached in this GPU's L2, so a remote tile read by every n-tile
//      that needs it would cross NVLink N/BN times.  Instead four extra "copier" warps per CTA pull the remote shards
//      into a local gathered buffer, 8 rows at a time in the order the tiles are consumed, and count finished
//      pieces per m-tile; the TMA producer starts with the tiles of the own shard (read in place) and waits (bounded)
//      on a remote tile's counter before loading it from the local copy.  Every byte crosses NVLink once and the
//      transfer overlaps the MMAs of earlier tiles; the gathered activation is a by-product that the weight-gradient
//      GEMM of the backward pass reuses.
//   2  GEMM → reduce-scatter: every output m-tile is stored straight into the staging slot [this rank] of the rank
//      that owns those rows; the owner later sums its `world` slots (ttb_rs_reduce).  Stores to peers start with
//      the next rank so the ranks do not all write to the same GPU at the same time.  The epilogue stages 32 × 64
//      sub-tiles in shared memory and hands them to the TMA store unit (per-thread 16-byte stores to a peer become
//      one NVLink write per row fragment and ran at a fraction of the link rate).
//   5  weight all-gather → GEMM (sharded-parameter data parallelism): the rows of B (the weight's output features) are
//      sharded over the ranks; copier warps pull the remote shards into a local [N, K] buffer n-tile by n-tile while the
//      MMA pipeline works on the n-tiles of the own shard (read in place); tiles run n-major so that a gathered n-tile is
//      consumed by all m-tiles right after it lands.  Shards must be whole n-tiles (rows_per_rank % BN == 0).
static constexpr int kMaxTpWorld = 8;
static constexpr int kTpAgThreads = 384;  // 8 GEMM warps + 4 copier warps
static constexpr int kRsStageBytes = 4 * 2 * 4096;  // TP 2: per epilogue warp two 32 × 64 bf16 staging tiles, 1024 bytes after the stage ring
static constexpr int kCopyPieces = 16;    // pieces per 128-row m-tile
struct alignas(64) TpArgs {
  CUtensorMap tmA[kMaxTpWorld];     // TP 1: per-rank A shard [rows_per_rank, K] (only the own one is loaded from)
                                    // TP 2: per-rank staging buffer as [world * rows_per_rank, N], box 64 × 32 (TMA stores)
  const void* A_src[kMaxTpWorld];   // TP 1: the same shards as raw pointers for the copier warps (row pitch K)
  void* gathered;                   // TP 1: local [world * rows_per_rank, K] buffer the copiers fill
  int* sync;                        // TP 1: [0] piece ticket, [1 + m] finished pieces of m-tile m (zeroed per launch)
  CUtensorMap tmC;                  // TP 1 / 5: the local output [M, N], box 64 × 32 (TMA-store epilogue)
  void* C[kMaxTpWorld];             // TP 2: per-rank staging buffer [world, rows_per_rank, ldc]
  int world, rank, rows_per_rank, gather_own;
  // Optional cross-rank readiness flags (written by ttb_dp_signal on the peers): entry [src * flag_stride + flag_slot] of the local
  // array reaches `flag_epoch` once rank src has placed its shard (TP 1).  nullptr: the caller ordered the ranks itself.
  const int* flags;
  int flag_stride, flag_slot, flag_epoch;
};

__device__ __forceinline__ bool wait_flag_sys(const int* f, int epoch) {
  const long long t0 = clock64();
  unsigned spins = 0;
  while (true) {
    int v;
    asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(f) : "memory");
    if (v >= epoch) return true;
    if ((++spins & 0xff) == 0 && clock64() - t0 > kWaitBudgetCycles) return false;
  }
}

__device__ __forceinline__ bool wait_count(const int* ctr, int target) {
  auto load = [&]() {
    int v;
    asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(v) : "l"(ctr) : "memory");
    return v;
  };
  if (load() >= target) return true;
  const long long t0 = clock64();
  uint32_t spins = 0;
  while (load() < target) {
    if ((++spins & 0xff) == 0 && clock64() - t0 > kWaitBudgetCycles) return false;
  }
  return true;
}

// Grouped (mixture-of-experts) variant, TP == 3: A is [rows, K] with the rows of expert e contiguous; B is a stack of E
// weight matrices addressed through a 3-D tensor map.  A device-side table (built by moe_tile_map_kernel from the
// per-expert row counts, so no host synchronisation is needed) gives, for every m-tile, its expert, its first row and how
// many of its 128 rows belong to that expert; rows past that count are computed but not stored.
struct GroupArgs {
  const int* tile_expert;
  const int* tile_row0;
  const int* tile_rows;
  const int* num_m_tiles;  // device scalar
  // TP == 4 (grouped weight gradient): dW[e][M, N] = A_eᵀ · B_e where A is [rows, M] and B is [rows, N] (both MN-major operands)
  // and expert e owns `counts[e]` consecutive rows — the *reduction* dimension is the ragged one.  Tiles are (expert, m, n);
  // every CTA derives the experts' row ranges from `counts` itself (no host read).  The last 64-row block of an expert also
  // brings in rows of the next expert: the MMA warp zeroes those rows in shared memory (whole 128-byte rows, which the swizzle
  // keeps intact) before issuing.  Experts without rows get a zero gradient.
  const long long* counts;
  int num_experts;
  long long c_expert_stride;
};
static constexpr int kMaxGroupedExperts = 1024;

template <int TP>
__device__ __forceinline__ int tp_rotate_m(int m_blk, int num_m, const TpArgs* tp) {
  if (TP == 0 || TP == 3 || TP == 4 || TP == 5) return m_blk;
  const int tiles_per_rank = tp->rows_per_rank / BM;
  const int first = (TP == 1 ? tp->rank : (tp->rank + 1) % tp->world) * tiles_per_rank;
  const int r = m_blk + first;
  return r >= num_m ? r - num_m : r;
}

template <int BN>
struct GemmCfg {
  static constexpr int kABytes = BM * BK * 2;
  static constexpr int kBBytes = BN * BK * 2;
  static constexpr int kStageBytes = kABytes + kBBytes;
  static constexpr int kStages = (200 * 1024 / kStageBytes) > 8 ? 8 : (200 * 1024 / kStageBytes);
  static constexpr int kTmemCols = 2 * BN < 32 ? 32 : 2 * BN;
  static constexpr int kSmemBytes = kStages * kStageBytes + 1024 /*align slack*/ + 256 /*barriers*/;
};

__device__ __forceinline__ void tile_coords(int t, int num_m, int num_n, int& m_blk, int& n_blk) {
  const int per_group = kGroupM * num_n;
  const int group = t / per_group;
  const int first_m = group * kGroupM;
  const int gsize = min(kGroupM, num_m - first_m);
  const int r = t - group * per_group;
  m_blk = first_m + r % gsize;
  n_blk = r / gsize;
}

static constexpr int kWgPieceRows = 8;  // TP 5: weight rows per copier piece

// TP 5 tile order: n-major, the n-tiles of the own weight shard first (rotation by rank · tiles-per-rank).
template <int BN>
__device__ __forceinline__ void wg_coords(int t, int num_m, int num_n, const TpArgs* tp, int& m_blk, int& n_blk) {
  const int n_idx = t / num_m;
  m_blk = t - n_idx * num_m;
  const int first = tp->rank * (tp->rows_per_rank / BN);
  n_blk = n_idx + first;
  if (n_blk >= num_n) n_blk -= num_n;
}

template <int BN, bool A_MN, bool B_MN, int TP>
__device__ __forceinline__ void gemm_body(const CUtensorMap* tmA_ptr, const CUtensorMap* tmB_ptr, const GemmParams& p,
                                          const TpArgs* tp, const GroupArgs* ga = nullptr, const CUtensorMap* tmC_ptr = nullptr,
                                          const CUtensorMap* tmA2 = nullptr, const CUtensorMap* tmB2 = nullptr) {
  using Cfg = GemmCfg<BN>;
  const CUtensorMap& tmA = *tmA_ptr;
  const CUtensorMap& tmB = *tmB_ptr;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + Cfg::kStages * Cfg::kStageBytes);
  uint64_t* full = bars;
  uint64_t* empty = bars + Cfg::kStages;
  uint64_t* tfull = bars + 2 * Cfg::kStages;
  uint64_t* tempty = tfull + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tempty + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  volatile int* piece_slot = reinterpret_cast<volatile int*>(tmem_slot + 2);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int num_m = TP == 3 ? *ga->num_m_tiles : (p.M + BM - 1) / BM;
  const int num_n = (p.N + BN - 1) / BN;
  const int splits = TP == 0 ? p.splits : 1;
  const int num_tiles = TP == 4 ? ga->num_experts * num_m * num_n : num_m * num_n * splits;
  const int num_kb = (p.K + BK - 1) / BK;
  const int num_kb2 = TP == 0 ? (p.K2 + BK - 1) / BK : 0;  // k-blocks of the second operand pair (same accumulator)
  // TP 4: first row and row count of every expert, after the barrier region
  int* g_row0 = reinterpret_cast<int*>(smem + Cfg::kStages * Cfg::kStageBytes + 256);
  int* g_cnt = g_row0 + kMaxGroupedExperts;
  if (TP == 4 && threadIdx.x == 32) {
    int run = 0;
    for (int e = 0; e < ga->num_experts; ++e) {
      const int c = static_cast<int>(ga->counts[e]);
      g_row0[e] = run;
      g_cnt[e] = c;
      run += c;
    }
  }

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
    // ------------------------------------------------------------------ TMA producer
    int stage = 0;
    uint32_t phase = 0;
    for (int t = blockIdx.x; t < num_tiles && !*abort_flag; t += gridDim.x) {
      int m_blk, n_blk;
      const int split = TP == 0 ? t / (num_m * num_n) : 0;
      tile_coords(TP == 0 ? t - split * (num_m * num_n) : t, num_m, num_n, m_blk, n_blk);
      m_blk = tp_rotate_m<TP>(m_blk, num_m, tp);
      const CUtensorMap* mapA = &tmA;
      int a_row = m_blk * BM;
      if (TP == 1) {
        const int src = a_row / tp->rows_per_rank;
        if (src == tp->rank) {  // own shard: read in place
          mapA = &tp->tmA[src];
          a_row -= src * tp->rows_per_rank;
        } else {  // remote rows: wait until the copier warps (of any CTA) have landed this m-tile in the local buffer
          if (!wait_count(tp->sync + 1 + m_blk, kCopyPieces)) {
            *abort_flag = 1;
            if (lane == 0) atomicExch(p.err, 105);
            break;
          }
          asm volatile("fence.proxy.async;" ::: "memory");  // generic-proxy stores → async-proxy (TMA) reads
        }
      }
      int expert = 0;
      if (TP == 3) {
        a_row = ga->tile_row0[m_blk];
        expert = ga->tile_expert[m_blk];
      }
      int kb_count = num_kb, k_row0 = 0;
      if (TP == 4) {
        expert = t / (num_m * num_n);
        const int r = t - expert * (num_m * num_n);
        m_blk = r % num_m;
        n_blk = r / num_m;
        k_row0 = g_row0[expert];
        kb_count = (g_cnt[expert] + BK - 1) / BK;
      }
      if (TP == 0 && splits > 1) {  // this tile covers k-blocks [kb0, kb0 + kb_count) of the contraction
        const int per = (num_kb + splits - 1) / splits;
        const int kb0 = split * per;
        kb_count = max(0, min(per, num_kb - kb0));
        k_row0 = kb0 * BK;
      }
      const CUtensorMap* mapB = &tmB;
      int b_row = 0;
      if (TP == 5) {
        wg_coords<BN>(t, num_m, num_n, tp, m_blk, n_blk);
        a_row = m_blk * BM;
        b_row = n_blk * BN;
        const int src = b_row / tp->rows_per_rank;
        if (src == tp->rank) {  // own weight shard: read in place
          mapB = &tp->tmA[src];
          b_row -= src * tp->rows_per_rank;
        } else {
          if (!wait_count(tp->sync + 1 + n_blk, BN / kWgPieceRows)) {
            *abort_flag = 1;
            if (lane == 0) atomicExch(p.err, 106);
            break;
          }
          asm volatile("fence.proxy.async;" ::: "memory");
        }
      }
      for (int kb = 0; kb < kb_count + num_kb2; ++kb) {
        if (!mbar_wait(&empty[stage], phase ^ 1)) {
          *abort_flag = 1;
          if (lane == 0) atomicExch(p.err, 101);
          break;
        }
        if (lane == 0) {
          uint8_t* sa = smem + stage * Cfg::kStageBytes;
          uint8_t* sb = sa + Cfg::kABytes;
          mbar_arrive_expect_tx(&full[stage], Cfg::kStageBytes);
          if (TP == 0 && kb >= kb_count) {  // second operand pair: same layouts, its own k index (out-of-range columns read as zero)
            const int k2 = (kb - kb_count) * BK;
            if (A_MN) {
#pragma unroll
              for (int j = 0; j < BM / 64; ++j) tma_load_2d(sa + j * 8192, tmA2, &full[stage], m_blk * BM + j * 64, k2);
            } else {
              tma_load_2d(sa, tmA2, &full[stage], k2, a_row);
            }
            if (B_MN) {
#pragma unroll
              for (int j = 0; j < BN / 64; ++j) tma_load_2d(sb + j * 8192, tmB2, &full[stage], n_blk * BN + j * 64, k2);
            } else {
              tma_load_2d(sb, tmB2, &full[stage], k2, n_blk * BN);
            }
          } else if (A_MN) {
#pragma unroll
            for (int j = 0; j < BM / 64; ++j) tma_load_2d(sa + j * 8192, &tmA, &full[stage], m_blk * BM + j * 64, k_row0 + kb * BK);
          } else {
            tma_load_2d(sa, mapA, &full[stage], k_row0 + kb * BK, a_row);
          }
          if (TP == 0 && kb >= kb_count) {
            // B of the second pair was issued above
          } else if (TP == 3) {
            if (B_MN) {
#pragma unroll
              for (int j = 0; j < BN / 64; ++j) tma_load_3d(sb + j * 8192, &tmB, &full[stage], n_blk * BN + j * 64, kb * BK, expert);
            } else {
              tma_load_3d(sb, &tmB, &full[stage], kb * BK, n_blk * BN, expert);
            }
          } else if (B_MN) {
#pragma unroll
            for (int j = 0; j < BN / 64; ++j) tma_load_2d(sb + j * 8192, &tmB, &full[stage], n_blk * BN + j * 64, k_row0 + kb * BK);
          } else if (TP == 5) {
            tma_load_2d(sb, mapB, &full[stage], kb * BK, b_row);
          } else {
            tma_load_2d(sb, &tmB, &full[stage], k_row0 + kb * BK, n_blk * BN);
          }
        }
        __syncwarp();
        if (++stage == Cfg::kStages) {
          stage = 0;
          phase ^= 1;
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    constexpr uint32_t idesc = make_idesc_bf16(BM, BN, A_MN, B_MN);
    int stage = 0;
    uint32_t phase = 0;
    int acc = 0;
    uint32_t acc_phase = 0;
    for (int t = blockIdx.x; t < num_tiles && !*abort_flag; t += gridDim.x) {
      if (!mbar_wait(&tempty[acc], acc_phase ^ 1)) {
        *abort_flag = 1;
        if (lane == 0) atomicExch(p.err, 102);
        break;
      }
      tc_fence_after();
      const uint32_t d_tmem = tmem_base + acc * BN;
      bool ok = true;
      int kb_count = num_kb, tail_rows = 0;
      if (TP == 0 && splits > 1) {
        const int per = (num_kb + splits - 1) / splits;
        kb_count = max(0, min(per, num_kb - (t / (num_m * num_n)) * per));
      }
      if (TP == 4) {
        const int cnt = g_cnt[t / (num_m * num_n)];
        kb_count = (cnt + BK - 1) / BK;
        tail_rows = cnt % BK;  // valid rows of the last block (0: the block is full)
      }
      for (int kb = 0; kb < kb_count + num_kb2; ++kb) {
        if (!mbar_wait(&full[stage], phase)) {
          ok = false;
          break;
        }
        if (TP == 4 && tail_rows != 0 && kb == kb_count - 1) {
          // rows [tail_rows, 64) of every 64-column box belong to the next expert: zero them (16 bytes per lane and step)
          uint8_t* st = smem + stage * Cfg::kStageBytes;
          constexpr int kBoxes = BM / 64 + BN / 64;
          const int chunks = (BK - tail_rows) * 8;  // 16-byte chunks per box
          for (int i = lane; i < chunks * kBoxes; i += 32) {
            const int box = i / chunks, c = i - box * chunks;
            *reinterpret_cast<uint4*>(st + box * 8192 + tail_rows * 128 + c * 16) = make_uint4(0, 0, 0, 0);
          }
          fence_proxy_async_smem();
          __syncwarp();
        }
        tc_fence_after();
        if (lane == 0) {
          const uint32_t sa = smem_u32(smem + stage * Cfg::kStageBytes);
          const uint32_t sb = sa + Cfg::kABytes;
#pragma unroll
          for (int k = 0; k < BK / 16; ++k) {
            // K-major: 32 bytes per K=16 step inside the swizzled row; SBO = 8 rows * 128 B.
            // MN-major: 16 k-rows = 2 swizzle atoms of 1024 B; LBO = one 64-wide box of BK rows.
            const uint64_t da = A_MN ? make_smem_desc_sw128(sa + k * 2048, 8192, 1024)
                                     : make_smem_desc_sw128(sa + k * 32, 16, 1024);
            const uint64_t db = B_MN ? make_smem_desc_sw128(sb + k * 2048, 8192, 1024)
                                     : make_smem_desc_sw128(sb + k * 32, 16, 1024);
            umma_f16(d_tmem, da, db, idesc, (kb | k) != 0);
          }
          umma_commit(&empty[stage]);  // smem slot reusable once these MMAs retire
        }
        __syncwarp();
        if (++stage == Cfg::kStages) {
          stage = 0;
          phase ^= 1;
        }
      }
      if (!ok) {
        *abort_flag = 1;
        if (lane == 0) atomicExch(p.err, 103);
        break;
      }
      if (lane == 0) umma_commit(&tfull[acc]);
      __syncwarp();
      if (++acc == 2) {
        acc = 0;
        acc_phase ^= 1;
      }
    }
  } else if (warp >= 4 && warp < 8) {
    // ------------------------------------------------------------------ epilogue
    const int quarter = warp & 3;  // TMEM lanes [32*quarter, 32*quarter+32) belong to this warp
    int acc = 0;
    uint32_t acc_phase = 0;
    int rs_buf = 0;  // TP 2: staging buffer toggle
    for (int t = blockIdx.x; t < num_tiles && !*abort_flag; t += gridDim.x) {
      int m_blk, n_blk;
      const int split = TP == 0 ? t / (num_m * num_n) : 0;
      tile_coords(TP == 0 ? t - split * (num_m * num_n) : t, num_m, num_n, m_blk, n_blk);
      m_blk = tp_rotate_m<TP>(m_blk, num_m, tp);
      if (!mbar_wait(&tfull[acc], acc_phase)) {
        *abort_flag = 1;
        if (lane == 0) atomicExch(p.err, 104);
        break;
      }
      bool empty_split = false;  // a range past the end of the contraction: no MMA ran, the accumulator holds stale values
      if (TP == 0 && splits > 1) {
        const int per = (num_kb + splits - 1) / splits;
        empty_split = num_kb - split * per <= 0;
      }
      tc_fence_after();
      if (TP == 5) wg_coords<BN>(t, num_m, num_n, tp, m_blk, n_blk);
      int expert = 0;
      bool empty_expert = false;
      if (TP == 4) {
        expert = t / (num_m * num_n);
        const int r = t - expert * (num_m * num_n);
        m_blk = r % num_m;
        n_blk = r / num_m;
        empty_expert = g_cnt[expert] == 0;  // no MMA ran: the accumulator holds stale values
      }
      int row = m_blk * BM + quarter * 32 + lane;
      bool row_ok = row < p.M;
      if (TP == 3) {
        row = ga->tile_row0[m_blk] + quarter * 32 + lane;
        row_ok = (quarter * 32 + lane) < ga->tile_rows[m_blk];
      }
      const uint32_t taddr = tmem_base + acc * BN + (static_cast<uint32_t>(quarter * 32) << 16);
      if (TP == 2 || ((TP == 0 || TP == 1 || TP == 5) && p.tma_store)) {
        // this warp's 32 rows leave through the TMA store unit, 64 columns at a time (TP 2: into the owner's staging slot)
        uint8_t* stage_base = smem + Cfg::kStages * Cfg::kStageBytes + 1024;  // 1024-byte aligned: after the barrier block
        uint8_t* my_stage = stage_base + quarter * 8192;
        const int row0 = m_blk * BM + quarter * 32;
        const CUtensorMap* mapC = (TP == 1 || TP == 5) ? &tp->tmC : tmC_ptr;
        int slot_row0 = row0;
        if (TP == 2) {
          const int owner = row0 / tp->rows_per_rank;
          slot_row0 = tp->rank * tp->rows_per_rank + (row0 - owner * tp->rows_per_rank);
          mapC = &tp->tmA[owner];
        }
#pragma unroll 1
        for (int c = 0; c < BN / 64; ++c) {
          const int col0 = n_blk * BN + c * 64;
          if (col0 >= p.N || row0 >= p.M) break;
          uint8_t* buf = my_stage + (rs_buf & 1) * 4096;
          if (lane == 0) tma_store_wait_read<1>();  // the store that used this buffer two sub-tiles ago has read it
          __syncwarp();
#pragma unroll
          for (int h = 0; h < 2; ++h) {
            uint32_t r[32];
            tmem_ld_32x32(taddr + c * 64 + h * 32, r);
            tmem_ld_wait();
#pragma unroll
            for (int j = 0; j < 4; ++j) {  // four 16-byte chunks of this half, 128-byte swizzle (chunk ^ row mod 8)
              float f[8];
#pragma unroll
              for (int i = 0; i < 8; ++i) f[i] = __uint_as_float(r[j * 8 + i]) * p.alpha;
              if (TP != 2 && p.bias != nullptr) {
                const int cb = col0 + h * 32 + j * 8;
#pragma unroll
                for (int i = 0; i < 8; ++i)
                  if (cb + i < p.N) f[i] += __bfloat162float(__ldg(p.bias + cb + i));
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
            tma_store_2d(mapC, buf, col0, slot_row0);
            tma_store_commit();
          }
          ++rs_buf;
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&tempty[acc]);
        if (++acc == 2) {
          acc = 0;
          acc_phase ^= 1;
        }
        continue;
      }
#pragma unroll 1
      for (int c = 0; c < BN / 32; ++c) {
        uint32_t r[32];
        tmem_ld_32x32(taddr + c * 32, r);
        tmem_ld_wait();
        const int col0 = n_blk * BN + c * 32;
        if (row_ok && col0 < p.N) {
          float v[32];
#pragma unroll
          for (int i = 0; i < 32; ++i) v[i] = ((TP == 4 && empty_expert) || (TP == 0 && empty_split)) ? 0.f : __uint_as_float(r[i]) * p.alpha;
          if (p.bias != nullptr && split == 0) {
#pragma unroll
            for (int i = 0; i < 32; ++i)
              if (col0 + i < p.N) v[i] += __bfloat162float(__ldg(p.bias + col0 + i));
          }
          if (TP == 0 && splits > 1) {
            float* dst = reinterpret_cast<float*>(p.C) + static_cast<long long>(row) * p.ldc + col0;
#pragma unroll
            for (int g = 0; g < 8; ++g)
              if (col0 + g * 4 + 4 <= p.N) atomicAdd(reinterpret_cast<float4*>(dst + g * 4), make_float4(v[g * 4], v[g * 4 + 1], v[g * 4 + 2], v[g * 4 + 3]));
          } else if (p.out_fp32) {
            float* dst = reinterpret_cast<float*>(p.C) + static_cast<long long>(row) * p.ldc + col0;
#pragma unroll
            for (int g = 0; g < 8; ++g) {
              if (col0 + g * 4 + 4 <= p.N) {
                float4 o = make_float4(v[g * 4], v[g * 4 + 1], v[g * 4 + 2], v[g * 4 + 3]);
                if (p.accumulate) {
                  const float4 old = *reinterpret_cast<const float4*>(dst + g * 4);
                  o.x += old.x, o.y += old.y, o.z += old.z, o.w += old.w;
                }
                *reinterpret_cast<float4*>(dst + g * 4) = o;
              }
            }
          } else {
            __nv_bfloat16* dst;
            if (TP == 2) {
              const int owner = row / tp->rows_per_rank;
              const long long slot_row = static_cast<long long>(tp->rank) * tp->rows_per_rank + (row - owner * tp->rows_per_rank);
              dst = reinterpret_cast<__nv_bfloat16*>(tp->C[owner]) + slot_row * p.ldc + col0;
            } else if (TP == 4) {
              dst = reinterpret_cast<__nv_bfloat16*>(p.C) + expert * ga->c_expert_stride + static_cast<long long>(row) * p.ldc + col0;
            } else {
              dst = reinterpret_cast<__nv_bfloat16*>(p.C) + static_cast<long long>(row) * p.ldc + col0;
            }
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
      if (lane == 0) mbar_arrive(&tempty[acc]);
      if (++acc == 2) {
        acc = 0;
        acc_phase ^= 1;
      }
    }
  }

  if ((TP == 2 || TP == 0 || TP == 1 || TP == 5) && warp >= 4 && warp < 8 && lane == 0) tma_store_wait<0>();  // every staged sub-tile has left shared memory and landed

  if (TP == 5 && warp >= 8) {
    // ------------------------------------------------------------------ copier warps (weight all-gather over peer memory)
    const int ctid = threadIdx.x - 256;
    const int tiles_per_rank = tp->rows_per_rank / BN;
    constexpr int kPieces = BN / kWgPieceRows;
    const int total = (num_n - tiles_per_rank) * kPieces;
    const long long row_vecs = p.K / 8;
    const long long piece_vecs = kWgPieceRows * row_vecs;
    while (true) {
      if (ctid == 0) *piece_slot = atomicAdd(tp->sync, 1);
      asm volatile("bar.sync 1, 128;" ::: "memory");
      const int pc = *piece_slot;
      if (pc >= total) break;
      int n_blk = tp->rank * tiles_per_rank + tiles_per_rank + pc / kPieces;  // remote n-tiles in the order they are consumed
      while (n_blk >= num_n) n_blk -= num_n;
      const long long row0 = static_cast<long long>(n_blk) * BN + (pc % kPieces) * kWgPieceRows;
      const int src = static_cast<int>(row0 / tp->rows_per_rank);
      const uint4* s = reinterpret_cast<const uint4*>(tp->A_src[src]) + (row0 - static_cast<long long>(src) * tp->rows_per_rank) * row_vecs;
      uint4* d = reinterpret_cast<uint4*>(tp->gathered) + row0 * row_vecs;
      for (long long v = ctid; v < piece_vecs; v += 128 * 8) {
        uint4 r[8];
#pragma unroll
        for (int j = 0; j < 8; ++j)
          if (v + j * 128 < piece_vecs) r[j] = __ldcg(s + v + j * 128);
#pragma unroll
        for (int j = 0; j < 8; ++j)
          if (v + j * 128 < piece_vecs) d[v + j * 128] = r[j];
      }
      __threadfence();
      asm volatile("bar.sync 1, 128;" ::: "memory");
      if (ctid == 0) {
        __threadfence();
        atomicAdd(tp->sync + 1 + n_blk, 1);
      }
    }
  }

  if (TP == 1 && warp >= 8) {
    // ------------------------------------------------------------------ copier warps (all-gather over peer memory)
    const int ctid = threadIdx.x - 256;
    const int tiles_per_rank = tp->rows_per_rank / BM;
    const int copy_tiles = tp->gather_own ? num_m : num_m - tiles_per_rank;
    const int total = copy_tiles * kCopyPieces;
    const long long row_vecs = p.K / 8;  // 16-byte vectors per row
    const long long piece_vecs = (BM / kCopyPieces) * row_vecs;
    while (true) {
      if (ctid == 0) *piece_slot = atomicAdd(tp->sync, 1);  // pieces are claimed in consumption order by whichever CTA is free
      asm volatile("bar.sync 1, 128;" ::: "memory");
      const int pc = *piece_slot;
      if (pc >= total) break;
      int i = tiles_per_rank + pc / kCopyPieces;  // position in the rotated order; the own tiles (if copied) come last
      if (i >= num_m) i -= num_m;
      const int m_blk = tp_rotate_m<1>(i, num_m, tp);
      const long long row0 = static_cast<long long>(m_blk) * BM + (pc % kCopyPieces) * (BM / kCopyPieces);
      const int src = static_cast<int>(row0 / tp->rows_per_rank);
      if (tp->flags != nullptr && src != tp->rank) {  // the peer's shard must be in place before it is read
        if (ctid == 0) *piece_slot = wait_flag_sys(tp->flags + src * tp->flag_stride + tp->flag_slot, tp->flag_epoch) ? 1 : 0;
        asm volatile("bar.sync 1, 128;" ::: "memory");
        const int ok = *piece_slot;
        asm volatile("bar.sync 1, 128;" ::: "memory");
        if (!ok) {
          if (ctid == 0) atomicExch(p.err, 107);
          break;
        }
      }
      const uint4* s = reinterpret_cast<const uint4*>(tp->A_src[src]) + (row0 - static_cast<long long>(src) * tp->rows_per_rank) * row_vecs;
      uint4* d = reinterpret_cast<uint4*>(tp->gathered) + row0 * row_vecs;
      for (long long v = ctid; v < piece_vecs; v += 128 * 8) {  // 8 × 16 bytes in flight per thread: NVLink latency needs ≈ 2.5 MB per GPU
        uint4 r[8];
#pragma unroll
        for (int j = 0; j < 8; ++j)
          if (v + j * 128 < piece_vecs) r[j] = __ldcg(s + v + j * 128);
#pragma unroll
        for (int j = 0; j < 8; ++j)
          if (v + j * 128 < piece_vecs) d[v + j * 128] = r[j];
      }
      __threadfence();
      asm volatile("bar.sync 1, 128;" ::: "memory");
      if (ctid == 0) {
        __threadfence();
        atomicAdd(tp->sync + 1 + m_blk, 1);
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  if (warp == 2) tmem_dealloc(tmem_base, Cfg::kTmemCols);
}

template <int BN, bool A_MN, bool B_MN>
__global__ void __launch_bounds__(kThreads, 1)
gemm_bf16_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                 const __grid_constant__ CUtensorMap tmC, const __grid_constant__ CUtensorMap tmA2,
                 const __grid_constant__ CUtensorMap tmB2, GemmParams p) {
  gemm_body<BN, A_MN, B_MN, 0>(&tmA, &tmB, p, nullptr, nullptr, &tmC, &tmA2, &tmB2);
}

template <int BN, bool B_MN, int TP>
__global__ void __launch_bounds__((TP == 1 || TP == 5) ? kTpAgThreads : kThreads, 1)
gemm_tp_kernel(const __grid_constant__ TpArgs tp, const __grid_constant__ CUtensorMap tmA,
               const __grid_constant__ CUtensorMap tmB, GemmParams p) {
  gemm_body<BN, false, B_MN, TP>(&tmA, &tmB, p, &tp);
}

template <int BN, bool B_MN>
__global__ void __launch_bounds__(kThreads, 1)
gemm_grouped_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, GemmParams p, GroupArgs ga) {
  gemm_body<BN, false, B_MN, 3>(&tmA, &tmB, p, nullptr, &ga);
}

template <int BN>
__global__ void __launch_bounds__(kThreads, 1)
gemm_grouped_wgrad_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, GemmParams p, GroupArgs ga) {
  gemm_body<BN, true, true, 4>(&tmA, &tmB, p, nullptr, &ga);
}

// One block: exclusive scan of the per-expert row counts, then one m-tile entry per 128 rows of every expert.
__global__ void moe_tile_map_kernel(const long long* __restrict__ counts, int num_experts, int max_tiles, int* tile_expert,
                                    int* tile_row0, int* tile_rows, int* num_m_tiles) {
  __shared__ long long row0[1025];
  __shared__ int tile0[1025];
  if (threadIdx.x == 0) {
    long long r = 0;
    int t = 0;
    for (int e = 0; e < num_experts; ++e) {
      row0[e] = r;
      tile0[e] = t;
      r += counts[e];
      t += static_cast<int>((counts[e] + BM - 1) / BM);
    }
    row0[num_experts] = r;
    tile0[num_experts] = t;
    *num_m_tiles = t < max_tiles ? t : max_tiles;
  }
  __syncthreads();
  for (int e = threadIdx.x; e < num_experts; e += blockDim.x) {
    const long long cnt = row0[e + 1] - row0[e];
    for (int i = 0, t = tile0[e]; t < tile0[e + 1] && t < max_tiles; ++i, ++t) {
      tile_expert[t] = e;
      tile_row0[t] = static_cast<int>(row0[e] + static_cast<long long>(i) * BM);
      const long long left = cnt - static_cast<long long>(i) * BM;
      tile_rows[t] = static_cast<int>(left < BM ? left : BM);
    }
  }
}

template <int BN, bool B_MN>
static int launch_gemm_grouped(const void* A, const void* B, const GemmParams& p, int num_experts, long long lda, long long ldb,
                               long long expert_stride, const GroupArgs& ga, int max_tiles, cudaStream_t stream) {
  using Cfg = GemmCfg<BN>;
  CUtensorMap tmA, tmB;
  int rc = make_tmap_2d(&tmA, A, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, p.M, p.K, lda, BM, BK, CU_TENSOR_MAP_SWIZZLE_128B);
  if (rc != kOk) return rc;
  if (B_MN)  // per expert [K, N] row-major: dims (N, K, E), box (64, BK, 1)
    rc = make_tmap_3d(&tmB, B, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, p.N, p.K, num_experts, ldb * 2, expert_stride * 2, 64, BK, 1, CU_TENSOR_MAP_SWIZZLE_128B);
  else  // per expert [N, K] row-major: dims (K, N, E), box (BK, BN, 1)
    rc = make_tmap_3d(&tmB, B, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, p.K, p.N, num_experts, ldb * 2, expert_stride * 2, BK, BN, 1, CU_TENSOR_MAP_SWIZZLE_128B);
  if (rc != kOk) return rc;
  auto kern = gemm_grouped_kernel<BN, B_MN>;
  static bool attr_set = false;
  if (!attr_set) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::kSmemBytes) != cudaSuccess) return kErrDriver;
    attr_set = true;
  }
  const long long tiles = static_cast<long long>(max_tiles) * ((p.N + BN - 1) / BN);
  const int grid = tiles < sm_count() ? static_cast<int>(tiles) : sm_count();
  TTB_COUNT_LAUNCH(1);
  kern<<<grid, kThreads, Cfg::kSmemBytes, stream>>>(tmA, tmB, p, ga);
  return cudaGetLastError() == cudaSuccess ? kOk : kErrDriver;
}

// Second operand pair of the plain kernel (same layouts as the first; K2 columns / rows): C = A·op(B) + A2·op(B2).
struct SecondPair {
  const void* A2 = nullptr;
  const void* B2 = nullptr;
  long long lda2 = 0, ldb2 = 0;
};

template <int BN, bool A_MN, bool B_MN>
static int launch_gemm(const void* A, const void* B, const GemmParams& p, long long lda, long long ldb,
                       cudaStream_t stream, const SecondPair& sp = SecondPair()) {
  using Cfg = GemmCfg<BN>;
  CUtensorMap tmA, tmB, tmA2, tmB2;
  memset(&tmA2, 0, sizeof(tmA2));
  memset(&tmB2, 0, sizeof(tmB2));
  int rc;
  if (p.K2 > 0) {
    if (A_MN)
      rc = make_tmap_2d(&tmA2, sp.A2, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, p.K2, p.M, sp.lda2, BK, 64, CU_TENSOR_MAP_SWIZZLE_128B);
    else
      rc = make_tmap_2d(&tmA2, sp.A2, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, p.M, p.K2, sp.lda2, BM, BK, CU_TENSOR_MAP_SWIZZLE_128B);
    if (rc != kOk) return rc;
    if (B_MN)
      rc = make_tmap_2d(&tmB2, sp.B2, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, p.K2, p.N, sp.ldb2, BK, 64, CU_TENSOR_MAP_SWIZZLE_128B);
    else
      rc = make_tmap_2d(&tmB2, sp.B2, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, p.N, p.K2, sp.ldb2, BN, BK, CU_TENSOR_MAP_SWIZZLE_128B);
    if (rc != kOk) return rc;
  }
  // K-major: tensor [rows, K], box [BM|BN rows, 64]; MN-major: tensor [K, rows], box [64 k-rows, 64].
  if (A_MN)
    rc = make_tmap_2d(&tmA, A, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, p.K, p.M, lda, BK, 64, CU_TENSOR_MAP_SWIZZLE_128B);
  else
    rc = make_tmap_2d(&tmA, A, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, p.M, p.K, lda, BM, BK, CU_TENSOR_MAP_SWIZZLE_128B);
  if (rc != kOk) {
    fprintf(stderr, "[ttb] gemm: tensor map for A failed (M=%d K=%d lda=%lld a_mn=%d ptr=%p)\n", p.M, p.K, lda, int(A_MN), A);
    return rc;
  }
  if (B_MN)
    rc = make_tmap_2d(&tmB, B, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, p.K, p.N, ldb, BK, 64, CU_TENSOR_MAP_SWIZZLE_128B);
  else
    rc = make_tmap_2d(&tmB, B, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, p.N, p.K, ldb, BN, BK, CU_TENSOR_MAP_SWIZZLE_128B);
  if (rc != kOk) {
    fprintf(stderr, "[ttb] gemm: tensor map for B failed (N=%d K=%d ldb=%lld b_mn=%d ptr=%p)\n", p.N, p.K, ldb, int(B_MN), B);
    return rc;
  }

  // bf16 outputs that are not accumulated leave through shared memory and TMA stores (box: 64 columns × 32 rows)
  GemmParams q = p;
  CUtensorMap tmC;
  memset(&tmC, 0, sizeof(tmC));
  q.tma_store = (!p.out_fp32 && !p.accumulate && (reinterpret_cast<uintptr_t>(p.C) & 15) == 0) ? 1 : 0;
  if (q.tma_store && make_tmap_2d(&tmC, p.C, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, p.M, p.N, p.ldc, 32, 64, CU_TENSOR_MAP_SWIZZLE_128B) != kOk) q.tma_store = 0;
  constexpr int smem_bytes = Cfg::kSmemBytes + 768 + kRsStageBytes;
  static_assert(smem_bytes <= 232448, "shared memory budget of one CTA");
  auto kern = gemm_bf16_kernel<BN, A_MN, B_MN>;
  static bool attr_set = false;
  if (!attr_set) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes);
    if (e != cudaSuccess) {
      fprintf(stderr, "[ttb] gemm: cudaFuncSetAttribute failed: %s\n", cudaGetErrorString(e));
      return kErrDriver;
    }
    attr_set = true;
  }
  if (q.splits < 1 || (q.splits > 1 && (!q.out_fp32 || q.K2 > 0))) return kErrBadShape;
  const int num_tiles = ((p.M + BM - 1) / BM) * ((p.N + BN - 1) / BN) * q.splits;
  const int grid = num_tiles < sm_count() ? num_tiles : sm_count();
  TTB_COUNT_LAUNCH(1);
  kern<<<grid, kThreads, smem_bytes, stream>>>(tmA, tmB, tmC, tmA2, tmB2, q);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) {
    fprintf(stderr, "[ttb] gemm launch failed: %s (M=%d N=%d K=%d grid=%d)\n", cudaGetErrorString(e), p.M, p.N, p.K, grid);
    return kErrDriver;
  }
  return kOk;
}

template <bool A_MN, bool B_MN>
static int dispatch_bn(const void* A, const void* B, const GemmParams& p, long long lda, long long ldb,
                       cudaStream_t stream, const SecondPair& sp = SecondPair()) {
  if (p.N > 128) return launch_gemm<256, A_MN, B_MN>(A, B, p, lda, ldb, stream, sp);
  if (p.N > 64) return launch_gemm<128, A_MN, B_MN>(A, B, p, lda, ldb, stream, sp);
  return launch_gemm<64, A_MN, B_MN>(A, B, p, lda, ldb, stream, sp);
}

template <int BN, bool B_MN, int TP>
static int launch_gemm_tp(const TpArgs& tp, const void* A, const void* B, const GemmParams& p, long long lda, long long ldb,
                          cudaStream_t stream) {
  using Cfg = GemmCfg<BN>;
  CUtensorMap tmA, tmB;
  // TP 1: `A` is the local gathered [M, K] buffer (row pitch K) that the copier warps fill; TP 2: the local [M, K] operand.
  int rc = make_tmap_2d(&tmA, A, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, p.M, p.K, lda, BM, BK, CU_TENSOR_MAP_SWIZZLE_128B);
  if (rc != kOk) return rc;
  if (B_MN)
    rc = make_tmap_2d(&tmB, B, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, p.K, p.N, ldb, BK, 64, CU_TENSOR_MAP_SWIZZLE_128B);
  else
    rc = make_tmap_2d(&tmB, B, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, p.N, p.K, ldb, BN, BK, CU_TENSOR_MAP_SWIZZLE_128B);
  if (rc != kOk) return rc;
  TpArgs tq = tp;
  GemmParams q = p;
  if (TP == 1 || TP == 5) {
    q.tma_store = (!p.out_fp32 && !p.accumulate && (reinterpret_cast<uintptr_t>(p.C) & 15) == 0 &&
                   make_tmap_2d(&tq.tmC, p.C, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, p.M, p.N, p.ldc, 32, 64, CU_TENSOR_MAP_SWIZZLE_128B) == kOk)
                      ? 1
                      : 0;
  }
  auto kern = gemm_tp_kernel<BN, B_MN, TP>;
  constexpr int smem_bytes = Cfg::kSmemBytes + 768 + kRsStageBytes;  // barriers take the first 256 of the 1024 bytes before the staging tiles
  static_assert(smem_bytes <= 232448, "shared memory budget of one CTA");
  static bool attr_set = false;
  if (!attr_set) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes) != cudaSuccess) return kErrDriver;
    attr_set = true;
  }
  const int num_tiles = ((p.M + BM - 1) / BM) * ((p.N + BN - 1) / BN);
  const int grid = num_tiles < sm_count() ? num_tiles : sm_count();
  TTB_COUNT_LAUNCH(1);
  kern<<<grid, (TP == 1 || TP == 5) ? kTpAgThreads : kThreads, smem_bytes, stream>>>(tq, tmA, tmB, q);
  if (cudaGetLastError() != cudaSuccess) return kErrDriver;
  return kOk;
}

template <int TP>
static int dispatch_tp(const TpArgs& tp, const void* A, const void* B, const GemmParams& p, long long lda, long long ldb, int b_mn,
                       cudaStream_t stream) {
  if (p.N > 128) {
    return b_mn ? launch_gemm_tp<256, true, TP>(tp, A, B, p, lda, ldb, stream) : launch_gemm_tp<256, false, TP>(tp, A, B, p, lda, ldb, stream);
  }
  if (p.N > 64) {
    return b_mn ? launch_gemm_tp<128, true, TP>(tp, A, B, p, lda, ldb, stream) : launch_gemm_tp<128, false, TP>(tp, A, B, p, lda, ldb, stream);
  }
  return b_mn ? launch_gemm_tp<64, true, TP>(tp, A, B, p, lda, ldb, stream) : launch_gemm_tp<64, false, TP>(tp, A, B, p, lda, ldb, stream);
}

// out[rows, N] = sum over `world` staging slots (+ residual) (+ bias), fp32 accumulation, 8 bf16 per thread.
__global__ void __launch_bounds__(256)
rs_reduce_kernel(const __nv_bfloat16* __restrict__ staging, const __nv_bfloat16* __restrict__ residual,
                 const __nv_bfloat16* __restrict__ bias, __nv_bfloat16* __restrict__ out, int world, long long rows, int N,
                 long long ld_stage, long long ld_res, long long ld_out, const int* __restrict__ flags, int flag_stride, int flag_slot,
                 int flag_epoch, int rank, int* __restrict__ err) {
  if (flags != nullptr) {  // every peer's partial tiles must have landed in this rank's staging slots
    __shared__ int give_up;
    if (threadIdx.x == 0) give_up = 0;
    __syncthreads();
    if (threadIdx.x < world && threadIdx.x != rank && !wait_flag_sys(flags + threadIdx.x * flag_stride + flag_slot, flag_epoch)) {
      give_up = 1;
      atomicExch(err, 108);
    }
    __syncthreads();
    if (give_up) return;
  }
  const int vec_per_row = N / 8;
  const long long total = rows * vec_per_row;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long r = i / vec_per_row;
    const int c = static_cast<int>(i - r * vec_per_row) * 8;
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    for (int w = 0; w < world; ++w) {
      const uint4 v = *reinterpret_cast<const uint4*>(staging + (static_cast<long long>(w) * rows + r) * ld_stage + c);
      const __nv_bfloat162* b = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const float2 f = __bfloat1622float2(b[k]);
        acc[2 * k] += f.x, acc[2 * k + 1] += f.y;
      }
    }
    if (residual != nullptr) {
      const uint4 v = *reinterpret_cast<const uint4*>(residual + r * ld_res + c);
      const __nv_bfloat162* b = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const float2 f = __bfloat1622float2(b[k]);
        acc[2 * k] += f.x, acc[2 * k + 1] += f.y;
      }
    }
    if (bias != nullptr) {
#pragma unroll
      for (int k = 0; k < 8; ++k) acc[k] += __bfloat162float(__ldg(bias + c + k));
    }
    uint4 o;
    o.x = pack_bf16x2(acc[0], acc[1]), o.y = pack_bf16x2(acc[2], acc[3]);
    o.z = pack_bf16x2(acc[4], acc[5]), o.w = pack_bf16x2(acc[6], acc[7]);
    *reinterpret_cast<uint4*>(out + r * ld_out + c) = o;
  }
}

}  // namespace ttb

// Tensor-parallel entry points -----------------------------------------------------------
// ttb_gemm_ag_bf16: C[world*rows_per_rank, N] = concat_r(A_ranks[r])[., K] * op(B); A_ranks[r] (contiguous [rows_per_rank, K])
//                   may be peer memory, read once by the copier warps' plain loads; `gathered` is a local contiguous
//                   [world*rows_per_rank, K] buffer that receives the remote rows (and the own rows when gather_own != 0);
//                   `sync` is a local int array of 1 + world*rows_per_rank/128 entries (zeroed here); C, B local.
// ttb_gemm_rs_bf16: partial = A[world*rows_per_rank, K] * op(B); rows of owner o are stored to
//                   C_ranks[o][rank][rows_per_rank][ldc] (C_ranks[o] may be peer memory, written by plain stores).
// rows_per_rank must be a multiple of 128 (one m-tile never spans two ranks).
extern "C" int ttb_gemm_ag_bf16(const void* const* A_ranks, const void* B, void* C, void* gathered, int* sync, int gather_own,
                                int world, int rank, int rows_per_rank, int N, int K, int b_mn, long long ldb, long long ldc,
                                const void* bias, const int* flags, int flag_stride, int flag_slot, int flag_epoch, int* err,
                                void* stream) {
  using namespace ttb;
  if (world < 1 || world > kMaxTpWorld || rank < 0 || rank >= world) return kErrBadShape;
  if (rows_per_rank <= 0 || (rows_per_rank % BM) || N <= 0 || K <= 0) return kErrBadShape;
  if ((ldb & 7) || (ldc & 7) || (N & 7) || (K & 7)) return kErrBadShape;
  if (gathered == nullptr || sync == nullptr || (reinterpret_cast<uintptr_t>(gathered) & 15)) return kErrBadShape;
  TpArgs tp;
  memset(&tp, 0, sizeof(tp));
  tp.world = world, tp.rank = rank, tp.rows_per_rank = rows_per_rank, tp.gather_own = gather_own;
  tp.gathered = gathered, tp.sync = sync;
  tp.flags = flags, tp.flag_stride = flag_stride, tp.flag_slot = flag_slot, tp.flag_epoch = flag_epoch;
  for (int r = 0; r < world; ++r) {
    if (reinterpret_cast<uintptr_t>(A_ranks[r]) & 15) return kErrBadShape;
    tp.A_src[r] = A_ranks[r];
    int rc = make_tmap_2d(&tp.tmA[r], A_ranks[r], CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, rows_per_rank, K, K, BM, BK, CU_TENSOR_MAP_SWIZZLE_128B);
    if (rc != kOk) return rc;
  }
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const size_t sync_bytes = sizeof(int) * (1 + static_cast<size_t>(world) * rows_per_rank / BM);
  if (cudaMemsetAsync(sync, 0, sync_bytes, s) != cudaSuccess) return kErrDriver;
  GemmParams p;
  p.M = world * rows_per_rank, p.N = N, p.K = K, p.C = C, p.ldc = ldc;
  p.bias = static_cast<const __nv_bfloat16*>(bias);
  p.alpha = 1.f, p.out_fp32 = 0, p.accumulate = 0, p.err = err;
  return dispatch_tp<1>(tp, gathered, B, p, K, ldb, b_mn, s);
}

// ttb_gemm_wg_bf16: C[M, world*rows_per_rank] = A[M, K] · concat_r(B_ranks[r])ᵀ (+ bias): B_ranks[r] is rank r's contiguous
//                   [rows_per_rank, K] shard of the weight (peer memory allowed, pulled once by the copier warps);
//                   `gathered` is a local contiguous [world*rows_per_rank, K] buffer that receives the remote shards (the own
//                   rows are not copied); `sync` is a local int array of 1 + N/64 entries (zeroed here).
//                   rows_per_rank must be a multiple of the n-tile (256 when N > 128, else 128 / 64).
extern "C" int ttb_gemm_wg_bf16(const void* A, const void* const* B_ranks, void* C, void* gathered, int* sync, int world, int rank,
                                int rows_per_rank, int M, int K, long long lda, long long ldc, const void* bias, int* err, void* stream) {
  using namespace ttb;
  if (world < 1 || world > kMaxTpWorld || rank < 0 || rank >= world) return kErrBadShape;
  if (rows_per_rank <= 0 || M <= 0 || K <= 0) return kErrBadShape;
  const int N = world * rows_per_rank;
  const int bn = N > 128 ? 256 : (N > 64 ? 128 : 64);
  if ((rows_per_rank % bn) || (lda & 7) || (ldc & 7) || (K & 7)) return kErrBadShape;
  if (gathered == nullptr || sync == nullptr || (reinterpret_cast<uintptr_t>(gathered) & 15)) return kErrBadShape;
  TpArgs tp;
  memset(&tp, 0, sizeof(tp));
  tp.world = world, tp.rank = rank, tp.rows_per_rank = rows_per_rank;
  tp.gathered = gathered, tp.sync = sync;
  for (int r = 0; r < world; ++r) {
    if (reinterpret_cast<uintptr_t>(B_ranks[r]) & 15) return kErrBadShape;
    tp.A_src[r] = B_ranks[r];
    int rc = make_tmap_2d(&tp.tmA[r], B_ranks[r], CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, rows_per_rank, K, K, bn, BK, CU_TENSOR_MAP_SWIZZLE_128B);
    if (rc != kOk) return rc;
  }
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (cudaMemsetAsync(sync, 0, sizeof(int) * (1 + static_cast<size_t>(N) / 64), s) != cudaSuccess) return kErrDriver;
  GemmParams p;
  p.M = M, p.N = N, p.K = K, p.C = C, p.ldc = ldc;
  p.bias = static_cast<const __nv_bfloat16*>(bias);
  p.alpha = 1.f, p.out_fp32 = 0, p.accumulate = 0, p.err = err;
  return dispatch_tp<5>(tp, A, gathered, p, lda, K, 0, s);
}

extern "C" int ttb_gemm_rs_bf16(const void* A, const void* B, void* const* C_ranks, int world, int rank, int rows_per_rank,
                                int N, int K, int b_mn, long long lda, long long ldb, long long ldc, int* err, void* stream) {
  using namespace ttb;
  if (world < 1 || world > kMaxTpWorld || rank < 0 || rank >= world) return kErrBadShape;
  if (rows_per_rank <= 0 || (rows_per_rank % BM) || N <= 0 || K <= 0) return kErrBadShape;
  if ((lda & 7) || (ldb & 7) || (ldc & 7) || (N & 7) || (K & 7)) return kErrBadShape;
  TpArgs tp;
  memset(&tp, 0, sizeof(tp));
  tp.world = world, tp.rank = rank, tp.rows_per_rank = rows_per_rank;
  for (int r = 0; r < world; ++r) {
    tp.C[r] = C_ranks[r];
    // rank r's staging buffer [world, rows_per_rank, ldc] as a 2-D tensor for the epilogue's TMA stores (box: 64 columns × 32 rows)
    int rc = make_tmap_2d(&tp.tmA[r], C_ranks[r], CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, static_cast<uint64_t>(world) * rows_per_rank, N, ldc, 32, 64,
                          CU_TENSOR_MAP_SWIZZLE_128B);
    if (rc != kOk) return rc;
  }
  GemmParams p;
  p.M = world * rows_per_rank, p.N = N, p.K = K, p.C = nullptr, p.ldc = ldc;
  p.bias = nullptr, p.alpha = 1.f, p.out_fp32 = 0, p.accumulate = 0, p.err = err;
  return dispatch_tp<2>(tp, A, B, p, lda, ldb, b_mn, static_cast<cudaStream_t>(stream));
}

extern "C" int ttb_rs_reduce(const void* staging, const void* residual, const void* bias, void* out, int world, long long rows,
                             int N, long long ld_stage, long long ld_res, long long ld_out, const int* flags, int flag_stride,
                             int flag_slot, int flag_epoch, int rank, int* err, void* stream) {
  using namespace ttb;
  if (world < 1 || rows <= 0 || N <= 0 || (N & 7) || (ld_stage & 7) || (ld_out & 7) || (residual && (ld_res & 7))) return kErrBadShape;
  const long long total = rows * (N / 8);
  long long blocks = (total + 255) / 256;
  const long long cap = static_cast<long long>(sm_count()) * 8;
  if (blocks > cap) blocks = cap;
  TTB_COUNT_LAUNCH(1);
  rs_reduce_kernel<<<static_cast<int>(blocks), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(staging), static_cast<const __nv_bfloat16*>(residual), static_cast<const __nv_bfloat16*>(bias),
      static_cast<__nv_bfloat16*>(out), world, rows, N, ld_stage, ld_res, ld_out, flags, flag_stride, flag_slot, flag_epoch, rank, err);
  return cudaGetLastError() == cudaSuccess ? kOk : kErrDriver;
}

namespace ttb {
template <int BN>
static int launch_grouped_wgrad(const void* A, const void* B, const GemmParams& p, long long rows, long long lda, long long ldb, const GroupArgs& ga,
                                cudaStream_t stream) {
  using Cfg = GemmCfg<BN>;
  CUtensorMap tmA, tmB;
  // both operands are [rows, width] row-major read as MN-major: tensor [rows(k), width], box [64 k-rows, 64]
  int rc = make_tmap_2d(&tmA, A, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, rows, p.M, lda, BK, 64, CU_TENSOR_MAP_SWIZZLE_128B);
  if (rc != kOk) return rc;
  rc = make_tmap_2d(&tmB, B, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, rows, p.N, ldb, BK, 64, CU_TENSOR_MAP_SWIZZLE_128B);
  if (rc != kOk) return rc;
  auto kern = gemm_grouped_wgrad_kernel<BN>;
  constexpr int smem = Cfg::kSmemBytes + 2 * kMaxGroupedExperts * static_cast<int>(sizeof(int));
  static bool attr_set = false;
  if (!attr_set) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess) return kErrDriver;
    attr_set = true;
  }
  const long long tiles = static_cast<long long>(ga.num_experts) * ((p.M + BM - 1) / BM) * ((p.N + BN - 1) / BN);
  const int grid = tiles < sm_count() ? static_cast<int>(tiles) : sm_count();
  TTB_COUNT_LAUNCH(1);
  kern<<<grid, kThreads, smem, stream>>>(tmA, tmB, p, ga);
  return cudaGetLastError() == cudaSuccess ? kOk : kErrDriver;
}
}  // namespace ttb

// Grouped weight gradient: dW[e][M, N] (+)= A[rows of e, M]ᵀ · B[rows of e, N]; `counts` is a device array of E int64 row counts
// (rows of expert e contiguous, in expert order); dW is [E, M, N] bf16 with row stride ldc and expert stride c_expert_stride.
extern "C" int ttb_gemm_grouped_wgrad_bf16(const void* A, const void* B, void* dW, const void* counts, long long rows, int num_experts, int M,
                                           int N, long long lda, long long ldb, long long ldc, long long c_expert_stride, int accumulate,
                                           int* err, void* stream) {
  using namespace ttb;
  if (rows <= 0 || num_experts <= 0 || num_experts > kMaxGroupedExperts || M <= 0 || N <= 0) return kErrBadShape;
  if ((lda & 7) || (ldb & 7) || (ldc & 7) || (M & 7) || (N & 7) || (c_expert_stride & 7)) return kErrBadShape;
  GroupArgs ga;
  memset(&ga, 0, sizeof(ga));
  ga.counts = static_cast<const long long*>(counts), ga.num_experts = num_experts, ga.c_expert_stride = c_expert_stride;
  GemmParams p;
  p.M = M, p.N = N, p.K = 0, p.C = dW, p.ldc = ldc;
  p.bias = nullptr, p.alpha = 1.f, p.out_fp32 = 0, p.accumulate = accumulate, p.err = err;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (N > 128) return launch_grouped_wgrad<256>(A, B, p, rows, lda, ldb, ga, s);
  if (N > 64) return launch_grouped_wgrad<128>(A, B, p, rows, lda, ldb, ga, s);
  return launch_grouped_wgrad<64>(A, B, p, rows, lda, ldb, ga, s);
}

// Grouped GEMM: C[rows, N] = A[rows, K] · op(B[e]) for the rows of each expert e.  `counts` is a device array of E int64 row
// counts (rows of expert e are contiguous, in expert order).  `tile_scratch` is a device int array of 3·max_tiles + 1 entries
// with max_tiles = ceil(rows / 128) + E.  b_mn = 0: B[e] is [N, K] row-major; 1: B[e] is [K, N] row-major.
extern "C" int ttb_gemm_grouped_bf16(const void* A, const void* B, void* C, const void* counts, void* tile_scratch, long long rows,
                                     int num_experts, int N, int K, int b_mn, long long lda, long long ldb, long long expert_stride,
                                     long long ldc, int* err, void* stream) {
  using namespace ttb;
  if (rows <= 0 || num_experts <= 0 || num_experts > 1024 || N <= 0 || K <= 0) return kErrBadShape;
  if ((lda & 7) || (ldb & 7) || (ldc & 7) || (N & 7) || (K & 7) || (expert_stride & 7)) return kErrBadShape;
  const int max_tiles = static_cast<int>((rows + BM - 1) / BM) + num_experts;
  int* scratch = static_cast<int*>(tile_scratch);
  GroupArgs ga;
  memset(&ga, 0, sizeof(ga));
  ga.tile_expert = scratch;
  ga.tile_row0 = scratch + max_tiles;
  ga.tile_rows = scratch + 2 * max_tiles;
  ga.num_m_tiles = scratch + 3 * max_tiles;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  TTB_COUNT_LAUNCH(1);
  moe_tile_map_kernel<<<1, 256, 0, s>>>(static_cast<const long long*>(counts), num_experts, max_tiles, scratch, scratch + max_tiles,
                                         scratch + 2 * max_tiles, scratch + 3 * max_tiles);
  if (cudaGetLastError() != cudaSuccess) return kErrDriver;
  GemmParams p;
  p.M = static_cast<int>(rows), p.N = N, p.K = K, p.C = C, p.ldc = ldc;
  p.bias = nullptr, p.alpha = 1.f, p.out_fp32 = 0, p.accumulate = 0, p.err = err;
  if (N > 128)
    return b_mn ? launch_gemm_grouped<256, true>(A, B, p, num_experts, lda, ldb, expert_stride, ga, max_tiles, s)
                : launch_gemm_grouped<256, false>(A, B, p, num_experts, lda, ldb, expert_stride, ga, max_tiles, s);
  if (N > 64)
    return b_mn ? launch_gemm_grouped<128, true>(A, B, p, num_experts, lda, ldb, expert_stride, ga, max_tiles, s)
                : launch_gemm_grouped<128, false>(A, B, p, num_experts, lda, ldb, expert_stride, ga, max_tiles, s);
  return b_mn ? launch_gemm_grouped<64, true>(A, B, p, num_experts, lda, ldb, expert_stride, ga, max_tiles, s)
              : launch_gemm_grouped<64, false>(A, B, p, num_experts, lda, ldb, expert_stride, ga, max_tiles, s);
}

// C ABI -------------------------------------------------------------------------------
// a_mn = 0: A is [M, K] row-major (row stride lda); 1: A is [K, M] row-major.
// b_mn = 0: B is [N, K] row-major (row stride ldb); 1: B is [K, N] row-major.
// Requirements: all leading dimensions and the contiguous extents are multiples of 8
// elements, base pointers 16-byte aligned.  `err` is a device int the kernel sets on a
// bounded-wait timeout.
extern "C" int ttb_gemm_bf16(const void* A, const void* B, void* C, int M, int N, int K, int a_mn, int b_mn,
                             long long lda, long long ldb, long long ldc, int out_fp32, int accumulate,
                             const void* bias, float alpha, int* err, void* stream) {
  using namespace ttb;
  if (M <= 0 || N <= 0 || K <= 0) return kErrBadShape;
  if ((lda & 7) || (ldb & 7) || (ldc & (out_fp32 ? 3 : 7)) || (N & 7)) return kErrBadShape;
  if ((a_mn ? (M & 7) : (K & 7)) || (b_mn ? (N & 7) : (K & 7))) return kErrBadShape;
  GemmParams p;
  p.M = M, p.N = N, p.K = K, p.C = C, p.ldc = ldc;
  p.bias = static_cast<const __nv_bfloat16*>(bias);
  p.alpha = alpha, p.out_fp32 = out_fp32, p.accumulate = accumulate, p.err = err;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (!a_mn && !b_mn) return dispatch_bn<false, false>(A, B, p, lda, ldb, s);
  if (!a_mn && b_mn) return dispatch_bn<false, true>(A, B, p, lda, ldb, s);
  if (a_mn && b_mn) return dispatch_bn<true, true>(A, B, p, lda, ldb, s);
  return dispatch_bn<true, false>(A, B, p, lda, ldb, s);
}

// C[M,N] (+)= alpha · (A·op(B) + A2·op(B2)) (+ bias): one kernel, one accumulator — the second pair's k-blocks (K2 columns, padded
// to 64 with zeros by the tensor map) simply extend the main loop.  Used for LoRA: A2 = s·x·Aᵀ ([M, r]), B2 = lora_b ([N, r]) in
// forward; A2 = s·dy·B ([M, r]), B2 = lora_a ([r, N], b_mn) in the input gradient (torchtune/modules/peft/lora.py:128-147).
// Layout flags and alignment rules as for ttb_gemm_bf16; K2 and the second pair's leading dimensions are multiples of 8.
extern "C" int ttb_gemm_bf16_dual(const void* A, const void* B, const void* A2, const void* B2, void* C, int M, int N, int K, int K2,
                                  int a_mn, int b_mn, long long lda, long long ldb, long long lda2, long long ldb2, long long ldc,
                                  int out_fp32, int accumulate, const void* bias, float alpha, int* err, void* stream) {
  using namespace ttb;
  if (M <= 0 || N <= 0 || K <= 0 || K2 <= 0 || A2 == nullptr || B2 == nullptr) return kErrBadShape;
  if ((lda & 7) || (ldb & 7) || (lda2 & 7) || (ldb2 & 7) || (ldc & (out_fp32 ? 3 : 7)) || (N & 7) || (K2 & 7)) return kErrBadShape;
  if ((a_mn ? (M & 7) : (K & 7)) || (b_mn ? (N & 7) : (K & 7))) return kErrBadShape;
  GemmParams p;
  p.M = M, p.N = N, p.K = K, p.K2 = K2, p.C = C, p.ldc = ldc;
  p.bias = static_cast<const __nv_bfloat16*>(bias);
  p.alpha = alpha, p.out_fp32 = out_fp32, p.accumulate = accumulate, p.err = err;
  SecondPair sp;
  sp.A2 = A2, sp.B2 = B2, sp.lda2 = lda2, sp.ldb2 = ldb2;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (!a_mn && !b_mn) return dispatch_bn<false, false>(A, B, p, lda, ldb, s, sp);
  if (!a_mn && b_mn) return dispatch_bn<false, true>(A, B, p, lda, ldb, s, sp);
  if (a_mn && b_mn) return dispatch_bn<true, true>(A, B, p, lda, ldb, s, sp);
  return dispatch_bn<true, false>(A, B, p, lda, ldb, s, sp);
}

// Split-K form of ttb_gemm_bf16 for skinny outputs: fp32 C (zero-initialised by the caller, or holding a value to add to), the
// contraction cut into `splits` ranges whose partial tiles are added with 16-byte float atomics.
extern "C" int ttb_gemm_bf16_splitk(const void* A, const void* B, void* C, int M, int N, int K, int a_mn, int b_mn, long long lda,
                                    long long ldb, long long ldc, int splits, float alpha, int* err, void* stream) {
  using namespace ttb;
  if (M <= 0 || N <= 0 || K <= 0 || splits < 1 || splits > 64) return kErrBadShape;
  if ((lda & 7) || (ldb & 7) || (ldc & 3) || (N & 7)) return kErrBadShape;
  if ((a_mn ? (M & 7) : (K & 7)) || (b_mn ? (N & 7) : (K & 7))) return kErrBadShape;
  GemmParams p;
  p.M = M, p.N = N, p.K = K, p.C = C, p.ldc = ldc;
  p.bias = nullptr, p.alpha = alpha, p.out_fp32 = 1, p.accumulate = 0, p.err = err, p.splits = splits;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (!a_mn && !b_mn) return dispatch_bn<false, false>(A, B, p, lda, ldb, s);
  if (!a_mn && b_mn) return dispatch_bn<false, true>(A, B, p, lda, ldb, s);
  if (a_mn && b_mn) return dispatch_bn<true, true>(A, B, p, lda, ldb, s);
  return dispatch_bn<true, false>(A, B, p, lda, ldb, s);
}
