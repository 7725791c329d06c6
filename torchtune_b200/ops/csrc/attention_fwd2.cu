// Attention forward, second form: two query tiles per CTA with alternating softmax warpgroups, P kept in tensor memory.
//
// One CTA owns 256 query rows of one head (tiles X = 0, 1 of 128 rows).  Tensor memory holds S_0, S_1 (128 fp32 columns each) and
// O_0, O_1 (head dim 128 each) = 512 columns.  The bf16 probabilities of a tile overwrite the first 64 columns of its own score
// buffer (two values per 32-bit column) and are consumed from there as the A operand of the P·V MMA, so they never pass through
// shared memory, which then has room for both query tiles and double-buffered K and V (192 KB).  While warpgroup X turns S_X into
// P_X (one query row per thread: maximum, exponentials, running sum, lazy rescale of O_X), the tensor core works on the other
// tile: the MMA thread issues  P_0·V_j, Q_0·K_{j+1}ᵀ, P_1·V_j, Q_1·K_{j+1}ᵀ, …  in that order, so neither side waits for the other
// for long.  S_X(j+1) may overwrite P_X(j) because MMAs of one thread execute in issue order.
//
// Masks: per-query bounds lo / hi that do not decrease along the sequence (causal, packed documents, sliding windows, chunks), or
// none.  Each tile visits only its own range of key blocks.  Element-wise masks, soft-capping and head dims other than 128 stay on
// the one-tile kernel in attention.cu.  Every wait is bounded and reports through the error word.
#include "common/ptx.cuh"
#include "common/tmap.h"

namespace ttb {
namespace fa2 {

static constexpr int kBlk = 128;
static constexpr int D = 128;
static constexpr int kPanelBytes = 16384;  // 128 rows x 128 B (64 bf16 columns)
static constexpr int kTileBytes = kBlk * D * 2;
static constexpr int kThreads = 384;
static constexpr float kLog2e = 1.4426950408889634f;
static constexpr float kRescaleThreshold = 8.0f;  // log2 units
static constexpr int kSmemBytes = 6 * kTileBytes + 1024 + 256;

struct Params {
  int b, s, sk, hq, hkv;
  float scale;
  int causal;
  const int* lo;  // [b, s] or nullptr
  const int* hi;  // [b, s] or nullptr (causal: q, else sk - 1)
  __nv_bfloat16* o;
  float* lse;
  int* err;
};

__device__ __forceinline__ uint64_t desc_kmajor(uint32_t base, int k) {
  return make_smem_desc_sw128(base + (k >> 2) * kPanelBytes + (k & 3) * 32, 16, 1024);
}
__device__ __forceinline__ uint64_t desc_mnmajor(uint32_t base, int k) {
  return make_smem_desc_sw128(base + k * 2048, kPanelBytes, 1024);
}
__device__ __forceinline__ float max3(float a, float b, float c) {
  float d;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
  return d;
}
__device__ __forceinline__ uint64_t pack_f32x2(float lo, float hi) {
  uint64_t d;
  asm("mov.b64 %0, {%1, %2};" : "=l"(d) : "f"(lo), "f"(hi));
  return d;
}
__device__ __forceinline__ uint64_t pack_u32x2(uint32_t lo, uint32_t hi) {
  uint64_t d;
  asm("mov.b64 %0, {%1, %2};" : "=l"(d) : "r"(lo), "r"(hi));
  return d;
}
__device__ __forceinline__ void unpack_f32x2(uint64_t v, float& lo, float& hi) {
  asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}
__device__ __forceinline__ uint64_t fma_f32x2(uint64_t a, uint64_t b, uint64_t c) {
  uint64_t d;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
  return d;
}
__device__ __forceinline__ uint64_t add_f32x2(uint64_t a, uint64_t b) {
  uint64_t d;
  asm("add.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
  return d;
}
__device__ __forceinline__ void fail(volatile int* abort_flag, int* err, int code) {
  *abort_flag = 1;
  atomicExch(err, code);
}

__global__ void __launch_bounds__(kThreads, 1)
attn_fwd2_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK, const __grid_constant__ CUtensorMap tmV, Params p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sQ[2] = {smem, smem + kTileBytes};
  uint8_t* sK[2] = {smem + 2 * kTileBytes, smem + 3 * kTileBytes};
  uint8_t* sV[2] = {smem + 4 * kTileBytes, smem + 5 * kTileBytes};
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + 6 * kTileBytes);
  uint64_t* q_full = bars;        // both query tiles
  uint64_t* k_full = bars + 1;    // [2]
  uint64_t* k_empty = bars + 3;   // [2]
  uint64_t* v_full = bars + 5;    // [2]
  uint64_t* v_empty = bars + 7;   // [2]
  uint64_t* s_full = bars + 9;    // [2] per tile
  uint64_t* p_full = bars + 11;   // [2] per tile, 4 warps arrive
  uint64_t* o_done = bars + 13;   // [2] per tile
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 15);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int h = blockIdx.y, bi = blockIdx.z;
  const int hk = h / (p.hq / p.hkv);
  const int q0 = blockIdx.x * 2 * kBlk;
  const int row_base = bi * p.s;
  const int krow_base = bi * p.sk;

  // Key-block range of each tile: [begin, begin + count).  The bounds are monotone, so first and last row give them.
  int begin[2], count[2];
#pragma unroll
  for (int x = 0; x < 2; ++x) {
    const int qa = q0 + x * kBlk;
    if (qa >= p.s) {
      begin[x] = 0, count[x] = 0;
      continue;
    }
    const int qz = min(qa + kBlk, p.s) - 1;
    const int lo_first = p.lo != nullptr ? max(p.lo[row_base + qa], 0) : 0;
    const int hi_last = p.hi != nullptr ? p.hi[row_base + qz] : (p.causal ? qz : p.sk - 1);
    const int end_tok = min(p.sk, hi_last + 1);
    begin[x] = lo_first / kBlk;
    count[x] = max((end_tok + kBlk - 1) / kBlk - begin[x], 0);
  }
  int u_begin, u_end;  // union of the two ranges
  if (count[0] > 0 && count[1] > 0) {
    u_begin = min(begin[0], begin[1]);
    u_end = max(begin[0] + count[0], begin[1] + count[1]);
  } else if (count[0] > 0) {
    u_begin = begin[0], u_end = begin[0] + count[0];
  } else {
    u_begin = begin[1], u_end = begin[1] + count[1];
  }
  const int n_union = u_end - u_begin;

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(&k_full[i], 1);
      mbar_init(&k_empty[i], 1);
      mbar_init(&v_full[i], 1);
      mbar_init(&v_empty[i], 1);
      mbar_init(&s_full[i], 1);
      mbar_init(&p_full[i], 4);
      mbar_init(&o_done[i], 1);
    }
    *abort_flag = 0;
    fence_mbar_init();
  }
  if (warp == 2) {
    tmem_alloc(tmem_slot, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tS[2] = {tmem_base, tmem_base + 128};
  const uint32_t tO[2] = {tmem_base + 256, tmem_base + 384};

  if (warp == 0) {
    // ---------------------------------------------------------------- TMA producer
    if (lane == 0 && n_union > 0) {
      mbar_arrive_expect_tx(q_full, 2 * kTileBytes);
      for (int x = 0; x < 2; ++x)
        for (int j = 0; j < 2; ++j) tma_load_2d(sQ[x] + j * kPanelBytes, &tmQ, q_full, h * D + j * 64, row_base + q0 + x * kBlk);
    }
    uint32_t phase = 0;
    for (int i = 0; i < n_union && !*abort_flag; ++i) {
      const int st = i & 1;
      const int kv0 = (u_begin + i) * kBlk;
      if (!mbar_wait(&k_empty[st], phase ^ 1)) {
        fail(abort_flag, p.err, 211);
        break;
      }
      if (lane == 0) {
        mbar_arrive_expect_tx(&k_full[st], kTileBytes);
        for (int j = 0; j < 2; ++j) tma_load_2d(sK[st] + j * kPanelBytes, &tmK, &k_full[st], hk * D + j * 64, krow_base + kv0);
      }
      __syncwarp();
      if (!mbar_wait(&v_empty[st], phase ^ 1)) {
        fail(abort_flag, p.err, 212);
        break;
      }
      if (lane == 0) {
        mbar_arrive_expect_tx(&v_full[st], kTileBytes);
        for (int j = 0; j < 2; ++j) tma_load_2d(sV[st] + j * kPanelBytes, &tmV, &v_full[st], hk * D + j * 64, krow_base + kv0);
      }
      __syncwarp();
      if (st == 1) phase ^= 1;
    }
  } else if (warp == 1) {
    // ---------------------------------------------------------------- MMA issuer
    constexpr uint32_t idesc_s = make_idesc_bf16(128, 128, false, false);
    constexpr uint32_t idesc_o = make_idesc_bf16(128, D, false, true);
    const uint32_t aQ[2] = {smem_u32(sQ[0]), smem_u32(sQ[1])};
    const uint32_t aK[2] = {smem_u32(sK[0]), smem_u32(sK[1])};
    const uint32_t aV[2] = {smem_u32(sV[0]), smem_u32(sV[1])};
    bool ok = n_union == 0 || mbar_wait(q_full, 0);
    int k_ready = u_begin - 1;  // highest block whose K tile has been waited for
    int v_ready = u_begin - 1;
    auto active = [&](int x, int j) { return count[x] > 0 && j >= begin[x] && j < begin[x] + count[x]; };
    // S_x(j) = Q_x · K_jᵀ; the K stage is handed back after the last tile that reads it
    auto issue_s = [&](int x, int j) -> bool {
      const int i = j - u_begin, st = i & 1;
      if (j > k_ready) {
        if (!mbar_wait(&k_full[st], (i >> 1) & 1)) return false;
        k_ready = j;
      }
      tc_fence_after();
      if (lane == 0) {
#pragma unroll
        for (int k = 0; k < D / 16; ++k) umma_f16(tS[x], desc_kmajor(aQ[x], k), desc_kmajor(aK[st], k), idesc_s, k != 0);
        umma_commit(&s_full[x]);
        const bool other_later = (x == 0) && active(1, j);  // tile 1 issues its S(j) after tile 0's
        if (!other_later) umma_commit(&k_empty[st]);
      }
      __syncwarp();
      return true;
    };
    for (int j = u_begin; j < u_end && ok && !*abort_flag; ++j) {
      for (int x = 0; x < 2 && ok; ++x)
        if (active(x, j) && j == begin[x]) ok = issue_s(x, j);  // first block of a tile
      for (int x = 0; x < 2 && ok; ++x) {
        if (!active(x, j)) continue;
        const int n = j - begin[x];  // tile-local block counter
        const int i = j - u_begin, st = i & 1;
        if (!mbar_wait(&p_full[x], n & 1)) {
          ok = false;
          break;
        }
        if (j > v_ready) {
          if (!mbar_wait(&v_full[st], (i >> 1) & 1)) {
            ok = false;
            break;
          }
          v_ready = j;
        }
        tc_fence_after();
        if (lane == 0) {
#pragma unroll
          for (int k = 0; k < kBlk / 16; ++k) umma_f16_ts(tO[x], tS[x] + k * 8, desc_mnmajor(aV[st], k), idesc_o, (n | k) != 0);
          const bool other_later = (x == 0) && active(1, j);
          if (!other_later) umma_commit(&v_empty[st]);
          if (n + 1 == count[x]) umma_commit(&o_done[x]);
        }
        __syncwarp();
        if (n + 1 < count[x]) ok = issue_s(x, j + 1);
      }
    }
    if (!ok) fail(abort_flag, p.err, 213);
  } else if (warp >= 4) {
    // ---------------------------------------------------------------- softmax / correction / epilogue, one warpgroup per tile
    const int x = (warp - 4) >> 2;
    const int quarter = warp & 3;
    const int r = quarter * 32 + lane;
    const int qa = q0 + x * kBlk;
    const int q_idx = qa + r;
    const int q_last = min(qa + kBlk, p.s) - 1;
    const uint32_t lane_sel = static_cast<uint32_t>(quarter * 32) << 16;
    const bool row_valid = q_idx < p.s;
    const bool tile_valid = qa < p.s;
    const int lo_row = (p.lo != nullptr && row_valid) ? p.lo[row_base + q_idx] : 0;
    const int hi_row = (p.hi != nullptr) ? (row_valid ? p.hi[row_base + q_idx] : -1) : (p.causal ? (row_valid ? q_idx : -1) : (row_valid ? p.sk - 1 : -1));
    const int lo_max = (p.lo == nullptr || !tile_valid) ? 0 : p.lo[row_base + q_last];
    const int hi_min = !tile_valid ? -1 : ((p.hi != nullptr) ? p.hi[row_base + qa] : (p.causal ? qa : p.sk - 1));
    const bool ragged_rows = qa + kBlk > p.s;  // rows past the end of the sequence must be masked in every block
    const float c = p.scale * kLog2e;
    float m_used = -INFINITY, l = 0.f;
    bool ok = true;
    for (int n = 0; n < count[x] && !*abort_flag; ++n) {
      const int kv0 = (begin[x] + n) * kBlk;
      if (!mbar_wait(&s_full[x], n & 1)) {
        ok = false;
        break;
      }
      tc_fence_after();
      const bool need_mask = ragged_rows || (kv0 + kBlk - 1 > hi_min) || (kv0 < lo_max) || (kv0 + kBlk > p.sk);
      uint32_t sv[4][32];
#pragma unroll
      for (int ch = 0; ch < 4; ++ch) tmem_ld_32x32(tS[x] + lane_sel + ch * 32, sv[ch]);
      tmem_ld_wait();
      // Raw scores stay in registers; the softmax scale is folded into the exponent (exp2(s·c − m·c)) and, c being positive, the row
      // maximum is taken on the raw values.  Three-input max and two-wide fp32 arithmetic halve the instruction count of the two
      // passes over the row.
      if (need_mask) {
#pragma unroll
        for (int ch = 0; ch < 4; ++ch) {
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            const int j = kv0 + ch * 32 + i;
            if (j < lo_row || j > hi_row || j >= p.sk) sv[ch][i] = 0xff800000u;  // -inf
          }
        }
      }
      float mx2[2] = {-INFINITY, -INFINITY};
#pragma unroll
      for (int ch = 0; ch < 4; ++ch) {
#pragma unroll
        for (int i = 0; i < 32; i += 4) {
          mx2[0] = max3(mx2[0], __uint_as_float(sv[ch][i]), __uint_as_float(sv[ch][i + 1]));
          mx2[1] = max3(mx2[1], __uint_as_float(sv[ch][i + 2]), __uint_as_float(sv[ch][i + 3]));
        }
      }
      const float mx = fmaxf(mx2[0], mx2[1]) * c;  // -inf stays -inf
      float alpha = 1.f;
      const float m_new = fmaxf(m_used, mx);
      bool rescale = false;
      if (m_new > m_used + kRescaleThreshold || m_used == -INFINITY) {
        if (m_new != -INFINITY) {
          alpha = (m_used == -INFINITY) ? 0.f : fast_exp2(m_used - m_new);
          rescale = (m_used != -INFINITY);
          m_used = m_new;
        }
      }
      const float neg_m = (m_used == -INFINITY) ? 0.f : -m_used;
      const uint64_t c2 = pack_f32x2(c, c), nm2 = pack_f32x2(neg_m, neg_m);
      uint64_t sum2[2] = {0ull, 0ull};
      uint32_t pk[2][32];  // 128 probabilities as bf16 pairs: column c of the P operand holds keys 2c and 2c + 1
#pragma unroll
      for (int ch = 0; ch < 4; ++ch) {
#pragma unroll
        for (int i = 0; i < 32; i += 2) {
          const uint64_t t = fma_f32x2(pack_u32x2(sv[ch][i], sv[ch][i + 1]), c2, nm2);
          float t0, t1;
          unpack_f32x2(t, t0, t1);
          const float e0 = fast_exp2(t0), e1 = fast_exp2(t1);
          sum2[(i >> 1) & 1] = add_f32x2(sum2[(i >> 1) & 1], pack_f32x2(e0, e1));
          pk[ch >> 1][(ch & 1) * 16 + (i >> 1)] = pack_bf16x2(e0, e1);
        }
      }
      float s0, s1, s2, s3;
      unpack_f32x2(sum2[0], s0, s1);
      unpack_f32x2(sum2[1], s2, s3);
      const float sum4[4] = {s0, s1, s2, s3};
      l = l * alpha + (sum4[0] + sum4[1]) + (sum4[2] + sum4[3]);
      // O_x is idle here: the S_x MMA that produced these scores was issued after the previous P_x·V
      if (n > 0 && __any_sync(0xffffffffu, rescale)) {
#pragma unroll 1
        for (int ch = 0; ch < D / 32; ++ch) {
          uint32_t v[32];
          tmem_ld_32x32(tO[x] + lane_sel + ch * 32, v);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 32; ++i) v[i] = __float_as_uint(__uint_as_float(v[i]) * alpha);
          tmem_st_32x32(tO[x] + lane_sel + ch * 32, v);
        }
      }
      tmem_st_32x32(tS[x] + lane_sel, pk[0]);
      tmem_st_32x32(tS[x] + lane_sel + 32, pk[1]);
      tmem_st_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&p_full[x]);
    }
    if (ok && count[x] > 0 && !*abort_flag) ok = mbar_wait(&o_done[x], 0);
    if (!ok) {
      fail(abort_flag, p.err, 214);
    } else if (tile_valid) {
      tc_fence_after();
      const float inv_l = l > 0.f ? 1.f / l : 0.f;
      __nv_bfloat16* orow = p.o + (static_cast<long long>(row_base + q_idx) * p.hq + h) * D;
#pragma unroll 1
      for (int ch = 0; ch < D / 32; ++ch) {
        uint32_t v[32];
        if (count[x] > 0) {
          tmem_ld_32x32(tO[x] + lane_sel + ch * 32, v);
          tmem_ld_wait();
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) v[i] = 0;
        }
        if (row_valid) {
#pragma unroll
          for (int g = 0; g < 4; ++g) {
            uint4 u;
            u.x = pack_bf16x2(__uint_as_float(v[g * 8 + 0]) * inv_l, __uint_as_float(v[g * 8 + 1]) * inv_l);
            u.y = pack_bf16x2(__uint_as_float(v[g * 8 + 2]) * inv_l, __uint_as_float(v[g * 8 + 3]) * inv_l);
            u.z = pack_bf16x2(__uint_as_float(v[g * 8 + 4]) * inv_l, __uint_as_float(v[g * 8 + 5]) * inv_l);
            u.w = pack_bf16x2(__uint_as_float(v[g * 8 + 6]) * inv_l, __uint_as_float(v[g * 8 + 7]) * inv_l);
            *reinterpret_cast<uint4*>(orow + ch * 32 + g * 8) = u;
          }
        }
      }
      if (row_valid) p.lse[(static_cast<long long>(bi) * p.hq + h) * p.s + q_idx] = (l > 0.f) ? m_used + log2f(l) : -INFINITY;
    }
  }

  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  if (warp == 2) tmem_dealloc(tmem_base, 512);
}

static int make_head_map(CUtensorMap* m, const void* base, int b, int s, int heads) {
  return make_tmap_2d(m, base, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, static_cast<uint64_t>(b) * s, static_cast<uint64_t>(heads) * D,
                      static_cast<uint64_t>(heads) * D, kBlk, 64, CU_TENSOR_MAP_SWIZZLE_128B);
}

}  // namespace fa2
}  // namespace ttb

// Forward attention for head dim 128 with monotone per-query bounds (or none): q [b, s, hq, 128], k / v [b, sk, hkv, 128], o like q,
// lse [b, hq, s] (log2 domain).  lo / hi as in ttb_attn_fwd; they must not decrease along the sequence.
extern "C" int ttb_attn_fwd2(const void* q, const void* k, const void* v, void* o, float* lse, const int* lo, const int* hi, int b, int s, int sk,
                             int hq, int hkv, float scale, int causal, int* err, void* stream) {
  using namespace ttb;
  if (hq % hkv || s <= 0 || sk <= 0 || b <= 0) return kErrBadShape;
  if (causal && hi == nullptr && s != sk) return kErrBadShape;
  fa2::Params p{};
  p.b = b, p.s = s, p.sk = sk, p.hq = hq, p.hkv = hkv, p.scale = scale, p.causal = causal, p.lo = lo, p.hi = hi;
  p.o = static_cast<__nv_bfloat16*>(o), p.lse = lse, p.err = err;
  CUtensorMap tq, tk, tv;
  int rc;
  if ((rc = fa2::make_head_map(&tq, q, b, s, hq)) != kOk) return rc;
  if ((rc = fa2::make_head_map(&tk, k, b, sk, hkv)) != kOk) return rc;
  if ((rc = fa2::make_head_map(&tv, v, b, sk, hkv)) != kOk) return rc;
  static bool attr = false;
  if (!attr) {
    if (cudaFuncSetAttribute(fa2::attn_fwd2_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, fa2::kSmemBytes) != cudaSuccess) return kErrDriver;
    attr = true;
  }
  dim3 grid((s + 2 * fa2::kBlk - 1) / (2 * fa2::kBlk), hq, b);
  TTB_COUNT_LAUNCH(1);
  fa2::attn_fwd2_kernel<<<grid, fa2::kThreads, fa2::kSmemBytes, static_cast<cudaStream_t>(stream)>>>(tq, tk, tv, p);
  return cudaGetLastError() == cudaSuccess ? kOk : kErrDriver;
}
