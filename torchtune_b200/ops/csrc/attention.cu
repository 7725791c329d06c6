// Grouped-query flash attention forward/backward on tcgen05 tensor cores.
//
// Layout: Q [b, s, hq, d], K/V [b, s, hkv, d] (bf16, contiguous), query head h reads KV head
// h / (hq / hkv) — KV heads are never expanded (the reference materialises the expansion,
// torchtune/modules/attention.py:287-290).  Every structured mask the framework uses
// (causal, packed documents, Llama-4 chunks, sliding window; reference:
// torchtune/modules/attention_utils.py:133-182, torchtune/models/llama4/_chunked_attention.py:39-49)
// reduces to a per-query lower bound lo[q] that is non-decreasing in q, plus the causal upper
// bound hi[q] = q:  key j is visible to query q  iff  lo[q] <= j <= hi[q].
//
// Forward: one CTA per (128-query block, query head, batch).  S = Q·Kᵀ and O += P·V run on
// tcgen05 with S double-buffered in TMEM so the next block's scores are computed while the
// softmax warps work; O stays in TMEM and is rescaled lazily (only when a row maximum grows
// by more than 2^8).  Backward: one CTA per (128-key block, KV head, batch) loops over the
// query heads of its group and the query blocks that can see it, accumulating dK/dV in TMEM
// and adding dQ partial tiles into an fp32 buffer.
#include "common/ptx.cuh"
#include "common/tmap.h"

namespace ttb {

static constexpr int kBlk = 128;          // query rows / key rows per tile
static constexpr int kPanelBytes = 16384;  // 128 rows x 128 B (64 bf16 columns)
static constexpr float kLog2e = 1.4426950408889634f;
static constexpr float kRescaleThreshold = 8.0f;  // log2 units

struct AttnParams {
  int b, s, hq, hkv, d;
  int sk;            // key / value length (s is the query length; cross-attention and cached decoding have sk != s)
  float scale;       // softmax scale (1/sqrt(d) by default)
  int causal;        // hi[q] = q when no `hi` array is given (requires sk == s)
  const int* lo;     // [b, s] lower visible key index per query, or nullptr (= 0)
  const int* hi;     // [b, s] upper visible key index per query, or nullptr (= q if causal, else sk - 1)
  const uint8_t* kmask;  // [b, s, sk] 1 = visible, or nullptr; applied on top of lo / hi (arbitrary boolean masks)
  int monotone;      // lo and hi are non-decreasing along the sequence (structured masks): block ranges can be cut at tile borders
  float softcap;     // > 0: scores pass through softcap * tanh(score / softcap) before the softmax
  __nv_bfloat16* o;  // fwd out [b, s, hq, d]
  float* lse;        // [b, hq, s] log2-domain log-sum-exp of scaled scores
  // backward only
  const float* delta;  // [b, hq, s] rowsum(dO * O)
  float* dq_accum;     // [b, s, hq, d] fp32, zero-initialised
  __nv_bfloat16* dk;   // [b, s, hkv, d]
  __nv_bfloat16* dv;
  int* err;
};

// K-major operand tile [128 rows, d] stored as d/64 panels of [128 rows x 128 B], 128B swizzle.
// Descriptor for the k-th K=16 slice of the contraction (contraction index contiguous).
__device__ __forceinline__ uint64_t desc_kmajor(uint32_t base, int k) {
  return make_smem_desc_sw128(base + (k >> 2) * kPanelBytes + (k & 3) * 32, 16, 1024);
}
// Same storage read with the *row* index as contraction (MN-major operand): slice k covers rows
// [16k, 16k+16); consecutive 64-column panels are kPanelBytes apart (leading byte offset).
__device__ __forceinline__ uint64_t desc_mnmajor(uint32_t base, int k) {
  return make_smem_desc_sw128(base + k * 2048, kPanelBytes, 1024);
}

// Byte offset of element (row, col) inside a swizzled tile of 64-column panels.
__device__ __forceinline__ uint32_t swz_offset(int row, int col) {
  const int panel = col >> 6;
  const int chunk = (col & 63) >> 3;  // 16-byte chunk inside the 128-byte row
  return panel * kPanelBytes + row * 128 + ((chunk ^ (row & 7)) << 4) + (col & 7) * 2;
}

__device__ __forceinline__ float fast_tanh(float x) {
  float y;
  asm("tanh.approx.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// two-wide fp32 arithmetic (one instruction per pair of values held in a 64-bit register)
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
__device__ __forceinline__ uint64_t mul_f32x2(uint64_t a, uint64_t b) {
  uint64_t d;
  asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
  return d;
}

__device__ __forceinline__ void fail(volatile int* abort_flag, int* err, int code) {
  *abort_flag = 1;
  atomicExch(err, code);
}

// ===================================================================================== forward
// EXTRA compiles in soft-capping and the element-wise boolean mask; the plain instantiation keeps the hot loop free of both.
template <int D, bool EXTRA>
__global__ void __launch_bounds__(256, 1)
attn_fwd_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                const __grid_constant__ CUtensorMap tmV, AttnParams p) {
  constexpr int kTileBytes = kBlk * D * 2;  // one [128, D] bf16 tile
  constexpr int kPanels = D / 64;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sQ = smem;
  uint8_t* sK[2] = {sQ + kTileBytes, sQ + 3 * kTileBytes};
  uint8_t* sV[2] = {sQ + 2 * kTileBytes, sQ + 4 * kTileBytes};
  uint8_t* sP = sQ + 5 * kTileBytes;              // [128 q, 128 kv] bf16 = 32 KB
  uint64_t* bars = reinterpret_cast<uint64_t*>(sP + 2 * kPanelBytes);
  uint64_t* q_full = bars;
  uint64_t* kv_full = bars + 1;   // [2]
  uint64_t* kv_empty = bars + 3;  // [2]
  uint64_t* s_full = bars + 5;    // [2]
  uint64_t* s_free = bars + 7;    // [2]
  uint64_t* p_full = bars + 9;
  uint64_t* pv_done = bars + 10;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 11);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  int* range = reinterpret_cast<int*>(tmem_slot + 2);  // [0] smallest lo, [1] largest hi over the tile's rows

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int qblk = blockIdx.x, h = blockIdx.y, bi = blockIdx.z;
  const int hk = h / (p.hq / p.hkv);
  const int q0 = qblk * kBlk;
  const int row_base = bi * p.s;    // row of token 0 of this batch entry in the [b*s, h*d] view of Q / O
  const int krow_base = bi * p.sk;  // the same for K / V
  const int q_last = min(q0 + kBlk, p.s) - 1;

  // Key blocks this tile visits: [min lo, max hi] over its rows.  Structured masks are monotone, so the first and last row
  // give the bounds; arbitrary masks reduce over all rows (threads 128..255 below).
  if (threadIdx.x == 0) {
    range[0] = (p.lo != nullptr && p.monotone) ? p.lo[row_base + q0] : (p.lo != nullptr ? p.sk : 0);
    range[1] = (p.hi != nullptr) ? (p.monotone ? p.hi[row_base + q_last] : -1) : (p.causal ? q_last : p.sk - 1);
  }
  __syncthreads();
  if (!p.monotone && threadIdx.x >= 128 && q0 + static_cast<int>(threadIdx.x) - 128 <= q_last) {
    const int row = row_base + q0 + threadIdx.x - 128;
    if (p.lo != nullptr) atomicMin(&range[0], p.lo[row]);
    if (p.hi != nullptr) atomicMax(&range[1], p.hi[row]);
  }
  __syncthreads();
  const int kv_begin = max(range[0], 0) / kBlk;
  const int kv_end_tok = min(p.sk, range[1] + 1);
  const int n_blocks = max((kv_end_tok + kBlk - 1) / kBlk - kv_begin, 0);

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(&kv_full[i], 1);
      mbar_init(&kv_empty[i], 1);
      mbar_init(&s_full[i], 1);
      mbar_init(&s_free[i], 4);
    }
    mbar_init(p_full, 4);
    mbar_init(pv_done, 1);
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
  const uint32_t tO = tmem_base + 256;

  if (warp == 0) {
    // ---------------------------------------------------------------- TMA producer
    if (lane == 0) {
      mbar_arrive_expect_tx(q_full, kTileBytes);
      for (int j = 0; j < kPanels; ++j) tma_load_2d(sQ + j * kPanelBytes, &tmQ, q_full, h * D + j * 64, row_base + q0);
    }
    uint32_t phase = 0;
    for (int it = 0; it < n_blocks && !*abort_flag; ++it) {
      const int st = it & 1;
      if (!mbar_wait(&kv_empty[st], phase ^ 1)) {
        fail(abort_flag, p.err, 201);
        break;
      }
      if (lane == 0) {
        const int kv0 = (kv_begin + it) * kBlk;
        mbar_arrive_expect_tx(&kv_full[st], 2 * kTileBytes);
        for (int j = 0; j < kPanels; ++j) {
          tma_load_2d(sK[st] + j * kPanelBytes, &tmK, &kv_full[st], hk * D + j * 64, krow_base + kv0);
          tma_load_2d(sV[st] + j * kPanelBytes, &tmV, &kv_full[st], hk * D + j * 64, krow_base + kv0);
        }
      }
      __syncwarp();
      if (st == 1) phase ^= 1;
    }
  } else if (warp == 1) {
    // ---------------------------------------------------------------- MMA issuer
    constexpr uint32_t idesc_s = make_idesc_bf16(128, 128, false, false);
    constexpr uint32_t idesc_o = make_idesc_bf16(128, D, false, true);
    const uint32_t aQ = smem_u32(sQ), aP = smem_u32(sP);
    const uint32_t aK[2] = {smem_u32(sK[0]), smem_u32(sK[1])};
    const uint32_t aV[2] = {smem_u32(sV[0]), smem_u32(sV[1])};
    bool ok = mbar_wait(q_full, 0);
    auto issue_s = [&](int it) -> bool {
      const int st = it & 1;
      const uint32_t ph = (it >> 1) & 1;
      if (!mbar_wait(&kv_full[st], ph)) return false;
      if (!mbar_wait(&s_free[st], ph ^ 1)) return false;  // S buffer consumed by the softmax warps
      tc_fence_after();
      if (lane == 0) {
#pragma unroll
        for (int k = 0; k < D / 16; ++k) umma_f16(tS[st], desc_kmajor(aQ, k), desc_kmajor(aK[st], k), idesc_s, k != 0);
        umma_commit(&s_full[st]);
      }
      __syncwarp();
      return true;
    };
    if (ok && n_blocks > 0) ok = issue_s(0);
    for (int it = 0; it < n_blocks && ok && !*abort_flag; ++it) {
      const int st = it & 1;
      if (it + 1 < n_blocks) ok = issue_s(it + 1);
      if (!ok) break;
      if (!mbar_wait(p_full, it & 1)) {
        ok = false;
        break;
      }
      tc_fence_after();
      if (lane == 0) {
#pragma unroll
        for (int k = 0; k < kBlk / 16; ++k) umma_f16(tO, desc_kmajor(aP, k), desc_mnmajor(aV[st], k), idesc_o, (it | k) != 0);
        umma_commit(&kv_empty[st]);
        umma_commit(pv_done);
      }
      __syncwarp();
    }
    if (!ok) fail(abort_flag, p.err, 202);
  } else if (warp >= 4) {
    // ---------------------------------------------------------------- softmax / correction / epilogue
    const int quarter = warp & 3;
    const int r = quarter * 32 + lane;  // row inside the tile
    const int q_idx = q0 + r;
    const uint32_t lane_sel = static_cast<uint32_t>(quarter * 32) << 16;
    const bool row_valid = q_idx < p.s;
    const int lo_row = (p.lo != nullptr && row_valid) ? p.lo[row_base + q_idx] : 0;
    const int hi_row = (p.hi != nullptr) ? (row_valid ? p.hi[row_base + q_idx] : -1) : (p.causal ? q_idx : p.sk - 1);
    // a block needs element-wise masking unless every key in it is visible to every row of the tile
    const int lo_max = (p.lo == nullptr) ? 0 : (p.monotone ? p.lo[row_base + q_last] : p.sk);
    const int hi_min = (p.hi != nullptr) ? (p.monotone ? p.hi[row_base + q0] : -1) : (p.causal ? q0 : p.sk - 1);
    const uint8_t* mrow = (EXTRA && p.kmask != nullptr && row_valid) ? p.kmask + static_cast<long long>(row_base + q_idx) * p.sk : nullptr;
    const float c = p.scale * kLog2e;
    const float cap_in = p.softcap > 0.f ? p.scale / p.softcap : 0.f;  // score → tanh argument
    const float cap_out = p.softcap * kLog2e;                           // tanh → log2-domain logit
    float m_used = -INFINITY, l = 0.f;
    bool ok = true;
    for (int it = 0; it < n_blocks && !*abort_flag; ++it) {
      const int st = it & 1;
      const int kv0 = (kv_begin + it) * kBlk;
      if (!mbar_wait(&s_full[st], (it >> 1) & 1)) {
        ok = false;
        break;
      }
      tc_fence_after();
      const bool need_mask = (kv0 + kBlk - 1 > hi_min) || (kv0 < lo_max) || (kv0 + kBlk > p.sk) || (EXTRA && p.kmask != nullptr);
      // The whole score row (128 fp32) is read from TMEM once — four loads issued back to back, one wait — and stays in
      // registers for both the maximum and the exponentials.
      uint32_t sv[4][32];
#pragma unroll
      for (int ch = 0; ch < 4; ++ch) tmem_ld_32x32(tS[st] + lane_sel + ch * 32, sv[ch]);
      tmem_ld_wait();
      // S buffer free for the scores of block it+2 (its values now live in registers)
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&s_free[st]);
      float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};  // four independent chains instead of one of length 128
#pragma unroll
      for (int ch = 0; ch < 4; ++ch) {
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          float x = (EXTRA && p.softcap > 0.f) ? fast_tanh(__uint_as_float(sv[ch][i]) * cap_in) * cap_out : __uint_as_float(sv[ch][i]) * c;
          if (need_mask) {
            const int j = kv0 + ch * 32 + i;
            if (j < lo_row || j > hi_row || j >= p.sk || (mrow != nullptr && !mrow[min(j, p.sk - 1)])) x = -INFINITY;
          }
          sv[ch][i] = __float_as_uint(x);
          mx4[i & 3] = fmaxf(mx4[i & 3], x);
        }
      }
      const float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3]));
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
      const float m_safe = (m_used == -INFINITY) ? 0.f : m_used;
      // exponentials and their running sum (four chains) are computed before the wait below, so only the stores into the
      // single P buffer have to follow the previous P·V
      float sum4[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int ch = 0; ch < 4; ++ch) {
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          const float e = fast_exp2(__uint_as_float(sv[ch][i]) - m_safe);
          sum4[i & 3] += e;
          sv[ch][i] = __float_as_uint(e);
        }
      }
      const float sum = (sum4[0] + sum4[1]) + (sum4[2] + sum4[3]);
      // P may only be overwritten (and O rescaled) once the previous P·V has retired
      if (it > 0) {
        if (!mbar_wait(pv_done, (it - 1) & 1)) {
          ok = false;
          break;
        }
        tc_fence_after();
      }
#pragma unroll
      for (int ch = 0; ch < 4; ++ch) {
#pragma unroll
        for (int g = 0; g < 4; ++g) {
          uint4 u;
          u.x = pack_bf16x2(__uint_as_float(sv[ch][g * 8 + 0]), __uint_as_float(sv[ch][g * 8 + 1]));
          u.y = pack_bf16x2(__uint_as_float(sv[ch][g * 8 + 2]), __uint_as_float(sv[ch][g * 8 + 3]));
          u.z = pack_bf16x2(__uint_as_float(sv[ch][g * 8 + 4]), __uint_as_float(sv[ch][g * 8 + 5]));
          u.w = pack_bf16x2(__uint_as_float(sv[ch][g * 8 + 6]), __uint_as_float(sv[ch][g * 8 + 7]));
          *reinterpret_cast<uint4*>(sP + swz_offset(r, ch * 32 + g * 8)) = u;
        }
      }
      l = l * alpha + sum;
      // lazy correction of the running output
      if (it > 0 && __any_sync(0xffffffffu, rescale)) {
#pragma unroll 1
        for (int ch = 0; ch < D / 32; ++ch) {
          uint32_t v[32];
          tmem_ld_32x32(tO + lane_sel + ch * 32, v);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 32; ++i) v[i] = __float_as_uint(__uint_as_float(v[i]) * alpha);
          tmem_st_32x32(tO + lane_sel + ch * 32, v);
        }
        tmem_st_wait();
      }
      fence_proxy_async_smem();  // generic-proxy smem writes -> visible to the tensor-core proxy
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(p_full);
    }
    if (ok && n_blocks > 0 && !*abort_flag) ok = mbar_wait(pv_done, (n_blocks - 1) & 1);
    if (!ok) {
      fail(abort_flag, p.err, 203);
    } else {
      tc_fence_after();
      const float inv_l = l > 0.f ? 1.f / l : 0.f;
      __nv_bfloat16* orow = p.o + (static_cast<long long>(row_base + q_idx) * p.hq + h) * D;
#pragma unroll 1
      for (int ch = 0; ch < D / 32; ++ch) {
        uint32_t v[32];
        if (n_blocks > 0) {
          tmem_ld_32x32(tO + lane_sel + ch * 32, v);
          tmem_ld_wait();
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) v[i] = 0;
        }
        if (q_idx < p.s) {
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
      if (q_idx < p.s) p.lse[(static_cast<long long>(bi) * p.hq + h) * p.s + q_idx] = (l > 0.f) ? m_used + log2f(l) : -INFINITY;
    }
  }

  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  if (warp == 2) tmem_dealloc(tmem_base, 512);
}

// ===================================================================================== backward
// delta[b, h, q] = sum_d dO * O (fp32); one warp per (token, head).
__global__ void attn_delta_kernel(const __nv_bfloat16* __restrict__ o, const __nv_bfloat16* __restrict__ d_o,
                                  float* __restrict__ delta, int b, int s, int hq, int d) {
  const long long w = (blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  const long long total = static_cast<long long>(b) * s * hq;
  if (w >= total) return;
  const __nv_bfloat16* po = o + w * d;
  const __nv_bfloat16* pd = d_o + w * d;
  float acc = 0.f;
  for (int i = lane * 2; i < d; i += 64) {
    const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(po + i));
    const float2 g = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(pd + i));
    acc += a.x * g.x + a.y * g.y;
  }
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, off);
  if (lane == 0) {
    const long long tok = w / hq;
    const int h = static_cast<int>(w % hq);
    const long long bi = tok / s, si = tok % s;
    delta[(bi * hq + h) * s + si] = acc;
  }
}

template <int D, bool EXTRA>
__global__ void __launch_bounds__(256, 1)
attn_bwd_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmdO, AttnParams p) {
  constexpr int kTileBytes = kBlk * D * 2;
  constexpr int kPanels = D / 64;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sK = smem;
  uint8_t* sV = sK + kTileBytes;
  uint8_t* sQ = sV + kTileBytes;
  uint8_t* sdO = sQ + kTileBytes;
  uint8_t* sP = sdO + kTileBytes;          // [128 q, 128 kv] bf16
  uint8_t* sdS = sP + 2 * kPanelBytes;     // [128 q, 128 kv] bf16
  uint64_t* bars = reinterpret_cast<uint64_t*>(sdS + 2 * kPanelBytes);
  uint64_t* kv_full = bars;
  uint64_t* qdo_full = bars + 1;
  uint64_t* qdo_empty = bars + 2;
  uint64_t* sdp_full = bars + 3;
  uint64_t* pds_full = bars + 4;
  uint64_t* dq_full = bars + 5;
  uint64_t* dq_free = bars + 6;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 7);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int kvblk = blockIdx.x, hk = blockIdx.y, bi = blockIdx.z;
  const int group = p.hq / p.hkv;
  const int kv0 = kvblk * kBlk;
  const int row_base = bi * p.s;
  const int krow_base = bi * p.sk;
  const int nq_blocks = (p.s + kBlk - 1) / kBlk;
  // Query blocks that can see this key block.  With monotone bounds: from the first block whose last row reaches the key
  // block (hi) to the last block whose first row has not yet moved past it (lo).  Arbitrary masks visit every block.
  int qb_begin = (p.hi == nullptr && p.causal) ? kvblk : 0;
  int qb_end = nq_blocks;
  if (p.monotone) {
    if (p.hi != nullptr) {
      while (qb_begin < nq_blocks && p.hi[row_base + min((qb_begin + 1) * kBlk, p.s) - 1] < kv0) ++qb_begin;
    }
    if (p.lo != nullptr) {
      for (int qb = qb_begin; qb < nq_blocks; ++qb) {
        if (p.lo[row_base + qb * kBlk] > kv0 + kBlk - 1) {
          qb_end = qb;
          break;
        }
      }
    }
  }
  const int iters_per_head = max(qb_end - qb_begin, 0);
  const int n_iters = iters_per_head * group;

  if (threadIdx.x == 0) {
    mbar_init(kv_full, 1);
    mbar_init(qdo_full, 1);
    mbar_init(qdo_empty, 1);
    mbar_init(sdp_full, 1);
    mbar_init(pds_full, 4);
    mbar_init(dq_full, 1);
    mbar_init(dq_free, 4);
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
  const uint32_t tS = tmem_base;         // scores, later reused for the dQ partial tile
  const uint32_t tdP = tmem_base + 128;
  const uint32_t tdV = tmem_base + 256;
  const uint32_t tdK = tmem_base + 384;

  if (warp == 0) {
    // ---------------------------------------------------------------- TMA producer
    if (lane == 0) {
      mbar_arrive_expect_tx(kv_full, 2 * kTileBytes);
      for (int j = 0; j < kPanels; ++j) {
        tma_load_2d(sK + j * kPanelBytes, &tmK, kv_full, hk * D + j * 64, krow_base + kv0);
        tma_load_2d(sV + j * kPanelBytes, &tmV, kv_full, hk * D + j * 64, krow_base + kv0);
      }
    }
    for (int it = 0; it < n_iters && !*abort_flag; ++it) {
      if (!mbar_wait(qdo_empty, (it & 1) ^ 1)) {
        fail(abort_flag, p.err, 301);
        break;
      }
      if (lane == 0) {
        const int h = hk * group + it / iters_per_head;
        const int q0 = (qb_begin + it % iters_per_head) * kBlk;
        mbar_arrive_expect_tx(qdo_full, 2 * kTileBytes);
        for (int j = 0; j < kPanels; ++j) {
          tma_load_2d(sQ + j * kPanelBytes, &tmQ, qdo_full, h * D + j * 64, row_base + q0);
          tma_load_2d(sdO + j * kPanelBytes, &tmdO, qdo_full, h * D + j * 64, row_base + q0);
        }
      }
      __syncwarp();
    }
  } else if (warp == 1) {
    // ---------------------------------------------------------------- MMA issuer
    constexpr uint32_t idesc_s = make_idesc_bf16(128, 128, false, false);  // Q·Kᵀ and dO·Vᵀ
    constexpr uint32_t idesc_t = make_idesc_bf16(128, D, true, true);      // Pᵀ·dO and dSᵀ·Q
    constexpr uint32_t idesc_q = make_idesc_bf16(128, D, false, true);     // dS·K
    const uint32_t aK = smem_u32(sK), aV = smem_u32(sV), aQ = smem_u32(sQ), adO = smem_u32(sdO);
    const uint32_t aP = smem_u32(sP), adS = smem_u32(sdS);
    bool ok = mbar_wait(kv_full, 0);
    for (int it = 0; it < n_iters && ok && !*abort_flag; ++it) {
      const uint32_t ph = it & 1;
      if (!mbar_wait(qdo_full, ph) || !mbar_wait(dq_free, ph ^ 1)) {
        ok = false;
        break;
      }
      tc_fence_after();
      if (lane == 0) {
#pragma unroll
        for (int k = 0; k < D / 16; ++k) umma_f16(tS, desc_kmajor(aQ, k), desc_kmajor(aK, k), idesc_s, k != 0);
#pragma unroll
        for (int k = 0; k < D / 16; ++k) umma_f16(tdP, desc_kmajor(adO, k), desc_kmajor(aV, k), idesc_s, k != 0);
        umma_commit(sdp_full);
      }
      __syncwarp();
      if (!mbar_wait(pds_full, ph)) {
        ok = false;
        break;
      }
      tc_fence_after();
      if (lane == 0) {
#pragma unroll
        for (int k = 0; k < kBlk / 16; ++k) umma_f16(tdV, desc_mnmajor(aP, k), desc_mnmajor(adO, k), idesc_t, (it | k) != 0);
#pragma unroll
        for (int k = 0; k < kBlk / 16; ++k) umma_f16(tdK, desc_mnmajor(adS, k), desc_mnmajor(aQ, k), idesc_t, (it | k) != 0);
#pragma unroll
        for (int k = 0; k < kBlk / 16; ++k) umma_f16(tS, desc_kmajor(adS, k), desc_mnmajor(aK, k), idesc_q, k != 0);
        umma_commit(qdo_empty);
        umma_commit(dq_full);
      }
      __syncwarp();
    }
    if (!ok) fail(abort_flag, p.err, 302);
  } else if (warp >= 4) {
    // ---------------------------------------------------------------- softmax-backward / dQ / epilogue
    const int quarter = warp & 3;
    const int r = quarter * 32 + lane;
    const uint32_t lane_sel = static_cast<uint32_t>(quarter * 32) << 16;
    const float c = p.scale * kLog2e;
    const float cap_in = p.softcap > 0.f ? p.scale / p.softcap : 0.f;
    const float cap_out = p.softcap * kLog2e;
    bool ok = true;
    for (int it = 0; it < n_iters && !*abort_flag; ++it) {
      const uint32_t ph = it & 1;
      const int h = hk * group + it / iters_per_head;
      const int q0 = (qb_begin + it % iters_per_head) * kBlk;
      const int q_idx = q0 + r;
      const bool row_ok = q_idx < p.s;
      const long long stat = (static_cast<long long>(bi) * p.hq + h) * p.s + q_idx;
      const float lse = row_ok ? p.lse[stat] : 0.f;
      const float dlt = row_ok ? p.delta[stat] : 0.f;
      const int lo_row = (p.lo != nullptr && row_ok) ? p.lo[row_base + q_idx] : 0;
      const int hi_row = (p.hi != nullptr) ? (row_ok ? p.hi[row_base + q_idx] : -1) : (p.causal ? q_idx : p.sk - 1);
      const uint8_t* mrow = (EXTRA && p.kmask != nullptr && row_ok) ? p.kmask + static_cast<long long>(row_base + q_idx) * p.sk : nullptr;
      if (!mbar_wait(sdp_full, ph)) {
        ok = false;
        break;
      }
      tc_fence_after();
      // A block every row of which sees every key (the interior of a causal or packed mask) needs no per-element test: the bounds
      // are monotone, so the tile's largest lo and smallest hi decide.  Such blocks take the two-wide fp32 path below.
      bool interior = !EXTRA && (p.monotone || (p.lo == nullptr && p.hi == nullptr)) && q0 + kBlk <= p.s && kv0 + kBlk <= p.sk;
      if (interior) {
        const int lo_max = p.lo != nullptr ? p.lo[row_base + q0 + kBlk - 1] : 0;
        const int hi_min = p.hi != nullptr ? p.hi[row_base + q0] : (p.causal ? q0 : p.sk - 1);
        interior = lo_max <= kv0 && hi_min >= kv0 + kBlk - 1;
      }
#pragma unroll 1
      for (int ch = 0; ch < 4; ++ch) {
        uint32_t sv[32], dv[32];
        tmem_ld_32x32(tS + lane_sel + ch * 32, sv);
        tmem_ld_32x32(tdP + lane_sel + ch * 32, dv);
        tmem_ld_wait();
        if (interior) {
          // p = exp2(s·c − lse),  dS = p · (dP − delta) · scale, two elements per instruction
          const uint64_t c2 = pack_f32x2(c, c), nl2 = pack_f32x2(-lse, -lse), nd2 = pack_f32x2(-dlt, -dlt), sc2 = pack_f32x2(p.scale, p.scale);
#pragma unroll
          for (int g = 0; g < 4; ++g) {
            uint32_t pu[4], du[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              const int e = g * 8 + 2 * i;
              float t0, t1;
              unpack_f32x2(fma_f32x2(pack_u32x2(sv[e], sv[e + 1]), c2, nl2), t0, t1);
              const float p0 = fast_exp2(t0), p1 = fast_exp2(t1);
              const uint64_t p2 = pack_f32x2(p0, p1);
              float d0, d1;
              unpack_f32x2(mul_f32x2(mul_f32x2(p2, sc2), add_f32x2(pack_u32x2(dv[e], dv[e + 1]), nd2)), d0, d1);
              pu[i] = pack_bf16x2(p0, p1);
              du[i] = pack_bf16x2(d0, d1);
            }
            const uint32_t off = swz_offset(r, ch * 32 + g * 8);
            *reinterpret_cast<uint4*>(sP + off) = make_uint4(pu[0], pu[1], pu[2], pu[3]);
            *reinterpret_cast<uint4*>(sdS + off) = make_uint4(du[0], du[1], du[2], du[3]);
          }
          continue;
        }
        float pr[32], ds[32];
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          const int j = kv0 + ch * 32 + i;
          const bool vis = row_ok && j >= lo_row && j <= hi_row && j < p.sk && lse != -INFINITY && (mrow == nullptr || mrow[min(j, p.sk - 1)]);
          if (EXTRA && p.softcap > 0.f) {  // logit = softcap · tanh(score / softcap): the chain rule adds the factor 1 − tanh²
            const float th = fast_tanh(__uint_as_float(sv[i]) * cap_in);
            pr[i] = vis ? fast_exp2(th * cap_out - lse) : 0.f;
            ds[i] = pr[i] * (__uint_as_float(dv[i]) - dlt) * p.scale * (1.f - th * th);
          } else {
            pr[i] = vis ? fast_exp2(__uint_as_float(sv[i]) * c - lse) : 0.f;
            ds[i] = pr[i] * (__uint_as_float(dv[i]) - dlt) * p.scale;
          }
        }
#pragma unroll
        for (int g = 0; g < 4; ++g) {
          uint4 u, w;
          u.x = pack_bf16x2(pr[g * 8 + 0], pr[g * 8 + 1]);
          u.y = pack_bf16x2(pr[g * 8 + 2], pr[g * 8 + 3]);
          u.z = pack_bf16x2(pr[g * 8 + 4], pr[g * 8 + 5]);
          u.w = pack_bf16x2(pr[g * 8 + 6], pr[g * 8 + 7]);
          w.x = pack_bf16x2(ds[g * 8 + 0], ds[g * 8 + 1]);
          w.y = pack_bf16x2(ds[g * 8 + 2], ds[g * 8 + 3]);
          w.z = pack_bf16x2(ds[g * 8 + 4], ds[g * 8 + 5]);
          w.w = pack_bf16x2(ds[g * 8 + 6], ds[g * 8 + 7]);
          const uint32_t off = swz_offset(r, ch * 32 + g * 8);
          *reinterpret_cast<uint4*>(sP + off) = u;
          *reinterpret_cast<uint4*>(sdS + off) = w;
        }
      }
      fence_proxy_async_smem();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(pds_full);
      // dQ partial tile: dS·K, added into the fp32 accumulator
      if (!mbar_wait(dq_full, ph)) {
        ok = false;
        break;
      }
      tc_fence_after();
      float* dq_row = p.dq_accum + (static_cast<long long>(row_base + q_idx) * p.hq + h) * D;
      // The whole partial tile is pulled into registers first and the buffer handed back, so the next iteration's Q·Kᵀ and dO·Vᵀ
      // run while this one's atomics drain.
      uint32_t dqv[D / 32][32];
#pragma unroll
      for (int ch = 0; ch < D / 32; ++ch) tmem_ld_32x32(tS + lane_sel + ch * 32, dqv[ch]);
      tmem_ld_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(dq_free);
      if (row_ok) {
#pragma unroll
        for (int ch = 0; ch < D / 32; ++ch) {
#pragma unroll
          for (int i = 0; i < 8; ++i)
            atomicAdd(reinterpret_cast<float4*>(dq_row + ch * 32 + i * 4),
                      make_float4(__uint_as_float(dqv[ch][i * 4]), __uint_as_float(dqv[ch][i * 4 + 1]),
                                  __uint_as_float(dqv[ch][i * 4 + 2]), __uint_as_float(dqv[ch][i * 4 + 3])));
        }
      }
    }
    if (!ok) {
      fail(abort_flag, p.err, 303);
    } else {
      // all MMAs of the last iteration retired when dq_full fired; write dK and dV
      const int kv_idx = kv0 + r;
      __nv_bfloat16* dkrow = p.dk + (static_cast<long long>(krow_base + kv_idx) * p.hkv + hk) * D;
      __nv_bfloat16* dvrow = p.dv + (static_cast<long long>(krow_base + kv_idx) * p.hkv + hk) * D;
#pragma unroll 1
      for (int ch = 0; ch < D / 32; ++ch) {
        uint32_t a[32], bb[32];
        if (n_iters > 0) {
          tmem_ld_32x32(tdK + lane_sel + ch * 32, a);
          tmem_ld_32x32(tdV + lane_sel + ch * 32, bb);
          tmem_ld_wait();
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) a[i] = 0, bb[i] = 0;
        }
        if (kv_idx < p.sk) {
#pragma unroll
          for (int g = 0; g < 4; ++g) {
            uint4 u, w;
            u.x = pack_bf16x2(__uint_as_float(a[g * 8 + 0]), __uint_as_float(a[g * 8 + 1]));
            u.y = pack_bf16x2(__uint_as_float(a[g * 8 + 2]), __uint_as_float(a[g * 8 + 3]));
            u.z = pack_bf16x2(__uint_as_float(a[g * 8 + 4]), __uint_as_float(a[g * 8 + 5]));
            u.w = pack_bf16x2(__uint_as_float(a[g * 8 + 6]), __uint_as_float(a[g * 8 + 7]));
            w.x = pack_bf16x2(__uint_as_float(bb[g * 8 + 0]), __uint_as_float(bb[g * 8 + 1]));
            w.y = pack_bf16x2(__uint_as_float(bb[g * 8 + 2]), __uint_as_float(bb[g * 8 + 3]));
            w.z = pack_bf16x2(__uint_as_float(bb[g * 8 + 4]), __uint_as_float(bb[g * 8 + 5]));
            w.w = pack_bf16x2(__uint_as_float(bb[g * 8 + 6]), __uint_as_float(bb[g * 8 + 7]));
            *reinterpret_cast<uint4*>(dkrow + ch * 32 + g * 8) = u;
            *reinterpret_cast<uint4*>(dvrow + ch * 32 + g * 8) = w;
          }
        }
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  if (warp == 2) tmem_dealloc(tmem_base, 512);
}

template <int D>
static int fwd_smem_bytes() { return 5 * kBlk * D * 2 + 2 * kPanelBytes + 1024 + 256; }
template <int D>
static int bwd_smem_bytes() { return 4 * kBlk * D * 2 + 4 * kPanelBytes + 1024 + 256; }

static int make_head_map(CUtensorMap* m, const void* base, int b, int s, int heads, int d) {
  // [b*s, heads*d] row-major, boxes of 128 rows x 64 columns
  return make_tmap_2d(m, base, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, static_cast<uint64_t>(b) * s,
                      static_cast<uint64_t>(heads) * d, static_cast<uint64_t>(heads) * d, kBlk, 64,
                      CU_TENSOR_MAP_SWIZZLE_128B);
}

template <int D>
static int launch_fwd(const void* q, const void* k, const void* v, const AttnParams& p, cudaStream_t st) {
  CUtensorMap tq, tk, tv;
  int rc;
  if ((rc = make_head_map(&tq, q, p.b, p.s, p.hq, D)) != kOk) return rc;
  if ((rc = make_head_map(&tk, k, p.b, p.sk, p.hkv, D)) != kOk) return rc;
  if ((rc = make_head_map(&tv, v, p.b, p.sk, p.hkv, D)) != kOk) return rc;
  const bool extra = p.softcap > 0.f || p.kmask != nullptr;
  auto kern = extra ? attn_fwd_kernel<D, true> : attn_fwd_kernel<D, false>;
  static bool attr[2] = {false, false};
  if (!attr[extra]) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, fwd_smem_bytes<D>()) != cudaSuccess) return kErrDriver;
    attr[extra] = true;
  }
  dim3 grid((p.s + kBlk - 1) / kBlk, p.hq, p.b);
  TTB_COUNT_LAUNCH(1);
  kern<<<grid, 256, fwd_smem_bytes<D>(), st>>>(tq, tk, tv, p);
  return cudaGetLastError() == cudaSuccess ? kOk : kErrDriver;
}

template <int D>
static int launch_bwd(const void* q, const void* k, const void* v, const void* d_o, const AttnParams& p, cudaStream_t st) {
  CUtensorMap tq, tk, tv, tdo;
  int rc;
  if ((rc = make_head_map(&tq, q, p.b, p.s, p.hq, D)) != kOk) return rc;
  if ((rc = make_head_map(&tk, k, p.b, p.sk, p.hkv, D)) != kOk) return rc;
  if ((rc = make_head_map(&tv, v, p.b, p.sk, p.hkv, D)) != kOk) return rc;
  if ((rc = make_head_map(&tdo, d_o, p.b, p.s, p.hq, D)) != kOk) return rc;
  const bool extra = p.softcap > 0.f || p.kmask != nullptr;
  auto kern = extra ? attn_bwd_kernel<D, true> : attn_bwd_kernel<D, false>;
  static bool attr[2] = {false, false};
  if (!attr[extra]) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, bwd_smem_bytes<D>()) != cudaSuccess) return kErrDriver;
    attr[extra] = true;
  }
  dim3 grid((p.sk + kBlk - 1) / kBlk, p.hkv, p.b);
  TTB_COUNT_LAUNCH(1);
  kern<<<grid, 256, bwd_smem_bytes<D>(), st>>>(tq, tk, tv, tdo, p);
  return cudaGetLastError() == cudaSuccess ? kOk : kErrDriver;
}

}  // namespace ttb

using namespace ttb;

// Optional mask description shared by forward and backward (all pointers may be null):
//   lo, hi   int32 [b, s]: key j is visible to query q iff lo[q] <= j <= hi[q]; without `hi` the upper bound is q when `causal`
//            (needs sk == s), else sk - 1; `monotone` != 0 promises both arrays are non-decreasing along the sequence
//   kmask    uint8 [b, s, sk], 1 = visible, applied on top of the bounds (arbitrary boolean masks; pass lo / hi = first / last
//            visible key per row with monotone = 0 so that key blocks outside every row's range are skipped)
//   softcap  > 0: scores pass through softcap * tanh(score * scale / softcap)
extern "C" int ttb_attn_fwd(const void* q, const void* k, const void* v, void* o, float* lse, const int* lo, const int* hi,
                            const void* kmask, int monotone, int b, int s, int sk, int hq, int hkv, int d, float scale, int causal,
                            float softcap, int* err, void* stream) {
  if ((d != 64 && d != 128) || hq % hkv || s <= 0 || sk <= 0) return kErrBadShape;
  if (causal && hi == nullptr && s != sk) return kErrBadShape;
  AttnParams p{};
  p.b = b, p.s = s, p.sk = sk, p.hq = hq, p.hkv = hkv, p.d = d, p.scale = scale, p.causal = causal, p.lo = lo, p.hi = hi;
  p.kmask = static_cast<const uint8_t*>(kmask), p.monotone = monotone, p.softcap = softcap;
  p.o = static_cast<__nv_bfloat16*>(o), p.lse = lse, p.err = err;
  auto st = static_cast<cudaStream_t>(stream);
  return d == 128 ? launch_fwd<128>(q, k, v, p, st) : launch_fwd<64>(q, k, v, p, st);
}

// delta: [b, hq, s] fp32 scratch, dq_accum: [b, s, hq, d] fp32 zero-filled by the caller; dk, dv: [b, sk, hkv, d].
extern "C" int ttb_attn_bwd(const void* q, const void* k, const void* v, const void* o, const void* d_o,
                            const float* lse, float* delta, float* dq_accum, void* dk, void* dv, const int* lo, const int* hi,
                            const void* kmask, int monotone, int b, int s, int sk, int hq, int hkv, int d, float scale, int causal,
                            float softcap, int* err, void* stream) {
  if ((d != 64 && d != 128) || hq % hkv || s <= 0 || sk <= 0) return kErrBadShape;
  if (causal && hi == nullptr && s != sk) return kErrBadShape;
  auto st = static_cast<cudaStream_t>(stream);
  const long long warps = static_cast<long long>(b) * s * hq;
  TTB_COUNT_LAUNCH(1);
  attn_delta_kernel<<<static_cast<unsigned>((warps * 32 + 255) / 256), 256, 0, st>>>(
      static_cast<const __nv_bfloat16*>(o), static_cast<const __nv_bfloat16*>(d_o), delta, b, s, hq, d);
  AttnParams p{};
  p.b = b, p.s = s, p.sk = sk, p.hq = hq, p.hkv = hkv, p.d = d, p.scale = scale, p.causal = causal, p.lo = lo, p.hi = hi;
  p.kmask = static_cast<const uint8_t*>(kmask), p.monotone = monotone, p.softcap = softcap;
  p.lse = const_cast<float*>(lse), p.delta = delta, p.dq_accum = dq_accum;
  p.dk = static_cast<__nv_bfloat16*>(dk), p.dv = static_cast<__nv_bfloat16*>(dv), p.err = err;
  return d == 128 ? launch_bwd<128>(q, k, v, d_o, p, st) : launch_bwd<64>(q, k, v, d_o, p, st);
}
