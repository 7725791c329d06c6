// Peer-memory plumbing and the fused data-parallel optimizer kernel.
//
// One process drives one GPU.  Flat parameter and gradient buffers are allocated with
// cudaMalloc, exported as CUDA IPC handles and mapped by every peer, so a kernel on any rank
// can load/store any rank's buffer over NVLink (plain peer loads/stores; no TMA is involved).
//
// dp_reduce_adamw_bcast: the gradient reduce-scatter, the fp32 scale/cast, the sharded AdamW
// update and the parameter all-gather of a ZeRO-style data-parallel step as ONE kernel.
// The rank owning shard [begin, end) pulls the bf16 gradient slices of all peers (16-byte
// peer loads), sums them in fp32, applies AdamW to its slice of the moments and pushes the
// new bf16 parameters into every peer's parameter buffer (16-byte peer stores).  Reference
// equivalents: FSDP2 reduce-scatter + `scale_grads_` + `torch.optim.AdamW(fused=True)` +
// all-gather (recipes/full_finetune_distributed.py:1030-1050, training/_distributed.py:661-714).
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <string.h>

#include "common/tmap.h"

namespace ttb {

static constexpr int kMaxRanks = 16;

struct PeerTable {
  const __nv_bfloat16* grad[kMaxRanks];  // every rank's flat gradient buffer
  __nv_bfloat16* param[kMaxRanks];       // every rank's flat parameter buffer
};

__device__ __forceinline__ void unpack8f(const uint4& u, float (&f)[8]) {
  const __nv_bfloat162* b = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 t = __bfloat1622float2(b[i]);
    f[2 * i] = t.x, f[2 * i + 1] = t.y;
  }
}
__device__ __forceinline__ uint4 pack8f(const float (&f)[8]) {
  uint4 u;
  __nv_bfloat162* b = reinterpret_cast<__nv_bfloat162*>(&u);
#pragma unroll
  for (int i = 0; i < 4; ++i) b[i] = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
  return u;
}

// Cross-rank "bucket is final" flags (no collective library involved, so nothing has to be scheduled next to the persistent
// GEMM kernels but two small kernels of this file): rank p stores `epoch` into flags_q[p][slot] on every peer q once its
// gradients of bucket `slot` are complete (dp_signal_kernel, stream-ordered after the layer's backward); the reduce kernel of
// rank q waits, with a cycle budget, until all peers' entries for that slot have reached the epoch.
static constexpr int kMaxBuckets = 4096;
static long long g_flag_wait_cycles = 4000000000LL;  // host-side setting, passed to every launch (ttb_dp_set_wait_cycles)

struct FlagTable {
  int* flags[kMaxRanks];
};

__global__ void dp_signal_kernel(FlagTable t, int world, int rank, int slot, int epoch) {
  __threadfence_system();
  if (threadIdx.x < world && threadIdx.x != rank) {
    int* dst = t.flags[threadIdx.x] + rank * kMaxBuckets + slot;
    asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(dst), "r"(epoch) : "memory");
  }
}

// Bounded wait of one rank for its peers' flags (one warp; lane p watches peer p's entry).  Runs as a launch of its own in
// front of the kernel that consumes the peers' data, so that giving up is a decision for the whole grid: on timeout it stores
// 201 in the error word, and every CTA of the consumer returns at once when it finds the error word set.
__global__ void dp_wait_kernel(const int* __restrict__ my_flags, int world, int rank, int slot, int epoch, int* __restrict__ err,
                               long long wait_cycles) {
  if (threadIdx.x < world && threadIdx.x != rank) {
    const int* f = my_flags + threadIdx.x * kMaxBuckets + slot;
    const long long t0 = clock64();
    int v;
    unsigned spins = 0;
    while (true) {
      asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(f) : "memory");
      if (v >= epoch) break;
      if ((++spins & 0xff) == 0 && clock64() - t0 > wait_cycles) {
        atomicExch(err, 201);
        break;
      }
    }
  }
}

// mode 0: reduce + AdamW + broadcast in one pass.
// mode 1: reduce only -> reduced fp32 gradient into `gsum` (shard-local) and per-block partial
//         sums of squares into `sumsq_partials` (for global-norm clipping).
// mode 2: AdamW + broadcast reading the already reduced `gsum`.
// `guard` (optional): the device error word.  When it is set — a preceding dp_wait_kernel gave up, or any earlier kernel
// reported an error — every CTA returns without touching parameters, moments or partial sums, so a failed step leaves the
// optimizer state as it was.
template <int WORLD, int mode>
__global__ void __launch_bounds__(256, 3)
dp_reduce_adamw_bcast_kernel(PeerTable peers, int rank, long long begin, long long count, __nv_bfloat16* __restrict__ m,
                             __nv_bfloat16* __restrict__ v, float* __restrict__ gsum, float* __restrict__ sumsq_partials,
                             const float* __restrict__ scale_dev, float scale_host, float lr, float beta1, float beta2,
                             float eps, float weight_decay, float inv_bc1, float inv_sqrt_bc2,
                             const int* __restrict__ guard, int bcast, int accumulate) {
  __shared__ float red[8];
  if (guard != nullptr && *reinterpret_cast<const volatile int*>(guard) != 0) return;
  const float gs = scale_host * (scale_dev != nullptr ? *scale_dev : 1.f);
  const long long nvec = count >> 3;  // shards are multiples of 8 elements
  float sq = 0.f;
  // U vectors per thread and trip, all loads issued before the first dependent instruction: with one or two ranks the kernel is
  // bound by this GPU's HBM and needs the extra bytes in flight (more ranks are NVLink-bound and short of registers instead).
  constexpr int U = WORLD <= 2 ? 2 : 1;
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  for (long long i0 = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i0 < nvec; i0 += stride * U) {
    uint4 raw[U][WORLD], wq[U], mq[U], vq[U];
    float4 ga[U], gb[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const long long i = i0 + u * stride;
      if (i >= nvec) continue;
      const long long e = begin + i * 8;
      if (mode == 2 || (mode == 1 && accumulate)) {
        ga[u] = *reinterpret_cast<const float4*>(gsum + i * 8);
        gb[u] = *reinterpret_cast<const float4*>(gsum + i * 8 + 4);
      }
      if (mode != 2) {
#pragma unroll
        for (int r = 0; r < WORLD; ++r) {
          // start with the next rank so that the 8 ranks do not all hit the same peer at once
          const int src = (rank + 1 + r) % WORLD;
          raw[u][r] = *reinterpret_cast<const uint4*>(peers.grad[src] + e);
        }
      }
      if (mode != 1) {
        wq[u] = *reinterpret_cast<const uint4*>(peers.param[rank] + e);
        mq[u] = *reinterpret_cast<const uint4*>(m + i * 8);
        vq[u] = *reinterpret_cast<const uint4*>(v + i * 8);
      }
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const long long i = i0 + u * stride;
      if (i >= nvec) continue;
      const long long e = begin + i * 8;
      float g[8];
      if (mode == 2) {
        g[0] = ga[u].x, g[1] = ga[u].y, g[2] = ga[u].z, g[3] = ga[u].w, g[4] = gb[u].x, g[5] = gb[u].y, g[6] = gb[u].z, g[7] = gb[u].w;
      } else {
#pragma unroll
        for (int j = 0; j < 8; ++j) g[j] = 0.f;
#pragma unroll
        for (int r = 0; r < WORLD; ++r) {
          float f[8];
          unpack8f(raw[u][r], f);
#pragma unroll
          for (int j = 0; j < 8; ++j) g[j] += f[j];
        }
      }
      if (mode == 1) {
        if (accumulate) {  // a further micro-batch: add to the reduced gradient of the earlier ones
          g[0] += ga[u].x, g[1] += ga[u].y, g[2] += ga[u].z, g[3] += ga[u].w, g[4] += gb[u].x, g[5] += gb[u].y, g[6] += gb[u].z, g[7] += gb[u].w;
        }
#pragma unroll
        for (int j = 0; j < 8; ++j) sq += g[j] * g[j];
        *reinterpret_cast<float4*>(gsum + i * 8) = make_float4(g[0], g[1], g[2], g[3]);
        *reinterpret_cast<float4*>(gsum + i * 8 + 4) = make_float4(g[4], g[5], g[6], g[7]);
        continue;
      }
      float w[8], m1[8], v1[8];
      unpack8f(wq[u], w);
      unpack8f(mq[u], m1);
      unpack8f(vq[u], v1);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const float grad = g[j] * gs;
        m1[j] = beta1 * m1[j] + (1.f - beta1) * grad;
        v1[j] = beta2 * v1[j] + (1.f - beta2) * grad * grad;
        w[j] *= (1.f - lr * weight_decay);
        w[j] -= lr * inv_bc1 * m1[j] / (sqrtf(v1[j]) * inv_sqrt_bc2 + eps);
      }
      *reinterpret_cast<uint4*>(m + i * 8) = pack8f(m1);
      *reinterpret_cast<uint4*>(v + i * 8) = pack8f(v1);
      const uint4 out = pack8f(w);
      if (!bcast) {  // sharded parameters: the owner keeps the only copy
        *reinterpret_cast<uint4*>(peers.param[rank] + e) = out;
        continue;
      }
#pragma unroll
      for (int r = 0; r < WORLD; ++r) {
        const int dst = (rank + r) % WORLD;
        *reinterpret_cast<uint4*>(peers.param[dst] + e) = out;
      }
    }
  }
  if (mode == 1) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) sq += __shfl_xor_sync(0xffffffffu, sq, o);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = sq;
    __syncthreads();
    if (threadIdx.x == 0) {
      float t = 0.f;
      for (int i = 0; i < 8; ++i) t += red[i];
      sumsq_partials[blockIdx.x] = t;
    }
  }
  __threadfence_system();  // peer stores visible before the host-side barrier that follows
}

// Parameter all-gather of a sharded-parameter (ZeRO-3) bucket as a pull over peer memory: dst[r · piece + i] = shard_r[i] for
// every rank r (16-byte peer loads, local stores).  `guard` as above.
struct ShardTable {
  const __nv_bfloat16* shard[kMaxRanks];
};

template <int WORLD>
__global__ void __launch_bounds__(256, 4)
zero3_gather_kernel(ShardTable t, int rank, long long piece, __nv_bfloat16* __restrict__ dst, const int* __restrict__ guard) {
  if (guard != nullptr && *reinterpret_cast<const volatile int*>(guard) != 0) return;
  const long long nvec = piece >> 3;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < nvec;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    uint4 raw[WORLD];
#pragma unroll
    for (int r = 0; r < WORLD; ++r) {
      const int src = (rank + 1 + r) % WORLD;  // every rank starts with a different peer
      raw[r] = *reinterpret_cast<const uint4*>(t.shard[src] + i * 8);
    }
#pragma unroll
    for (int r = 0; r < WORLD; ++r) {
      const int src = (rank + 1 + r) % WORLD;
      *reinterpret_cast<uint4*>(dst + src * piece + i * 8) = raw[r];
    }
  }
}

// Context-parallel head / sequence exchange as a push over peer memory (the all-to-all around attention).
//   mode 0 (sequence → heads): src is this rank's [b, s_l, W, h_l, dv] view of its sequence block (all heads); rank j receives the
//          h_l heads it owns, placed at sequence block `rank` of its [b, W·s_l, h_l, dv] buffer.
//   mode 1 (heads → sequence): src is this rank's [b, W, s_l, h_l, dv] view of the whole sequence (its h_l heads); rank j receives its
//          sequence block, placed at head group `rank` of its [b, s_l, W·h_l, dv] buffer.
// dv counts 16-byte vectors per (token, head).  One launch writes every peer's buffer, each thread starting with a different peer.
struct CpTable {
  uint4* dst[kMaxRanks];
};

__global__ void __launch_bounds__(256)
cp_exchange_kernel(const uint4* __restrict__ src, CpTable t, int world, int rank, int mode, long long b, long long s_l, long long h_l, long long dv) {
  const long long per_peer = b * s_l * h_l * dv;
  const long long total = per_peer * world;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total; i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const int jj = static_cast<int>(i / per_peer);
    const int j = (rank + 1 + jj) % world;  // the ranks do not all start on the same peer
    long long r = i - jj * per_peer;
    const long long v = r % dv;
    r /= dv;
    const long long hi = r % h_l;
    r /= h_l;
    const long long si = r % s_l;
    const long long bi = r / s_l;
    long long so, dof;
    if (mode == 0) {
      so = (((bi * s_l + si) * world + j) * h_l + hi) * dv + v;
      dof = ((bi * (world * s_l) + rank * s_l + si) * h_l + hi) * dv + v;
    } else {
      so = (((bi * world + j) * s_l + si) * h_l + hi) * dv + v;
      dof = ((bi * s_l + si) * (world * h_l) + rank * h_l + hi) * dv + v;
    }
    t.dst[j][dof] = src[so];
  }
  __threadfence_system();  // peer stores visible before the signal that follows in stream order
}

}  // namespace ttb

using namespace ttb;

// ----------------------------------------------------------------------------- IPC helpers
extern "C" int ttb_ipc_alloc(long long bytes, void** out) {
  return cudaMalloc(out, static_cast<size_t>(bytes)) == cudaSuccess ? kOk : kErrDriver;
}
extern "C" int ttb_ipc_free(void* p) { return cudaFree(p) == cudaSuccess ? kOk : kErrDriver; }
// handle_out: 64 bytes
extern "C" int ttb_ipc_get_handle(void* p, void* handle_out) {
  cudaIpcMemHandle_t h;
  if (cudaIpcGetMemHandle(&h, p) != cudaSuccess) return kErrDriver;
  memcpy(handle_out, &h, sizeof(h));
  return kOk;
}
extern "C" int ttb_ipc_open(const void* handle, void** out) {
  cudaIpcMemHandle_t h;
  memcpy(&h, handle, sizeof(h));
  cudaError_t e = cudaIpcOpenMemHandle(out, h, cudaIpcMemLazyEnablePeerAccess);
  if (e != cudaSuccess) {
    fprintf(stderr, "[ttb] cudaIpcOpenMemHandle failed: %s\n", cudaGetErrorString(e));
    return kErrDriver;
  }
  return kOk;
}
extern "C" int ttb_ipc_close(void* p) { return cudaIpcCloseMemHandle(p) == cudaSuccess ? kOk : kErrDriver; }
extern "C" int ttb_dp_grid() { return sm_count() * 3; }

// grad_ptrs / param_ptrs: host arrays of `world` device pointers (peer-mapped flat buffers).
// [begin, begin+count) is this rank's shard (count % 8 == 0, begin % 8 == 0).
// bcast = 0: the new parameters are stored to param_ptrs[rank] only (sharded parameters; the other entries are not touched).
// accumulate = 1 (mode 1): add the reduced gradient to what `gsum` already holds (gradient accumulation over micro-batches;
// the partial sums of squares then describe the accumulated gradient).
// my_flags != null: first wait (bounded, one warp, its own launch) until every peer's entry [peer][slot] of this rank's flag
// array has reached `epoch`.  grid_ctas > 0 limits the kernel to that many CTAs (a bucket processed *during* backward is bound
// by NVLink, not HBM: a few dozen CTAs keep the links busy and leave the SMs' issue slots and the HBM to the GEMMs they run
// beside; the kernel uses no shared memory, so its CTAs fit next to a resident GEMM CTA).
extern "C" int ttb_dp_reduce_adamw_bcast(void* const* grad_ptrs, void* const* param_ptrs, int world, int rank,
                                         long long begin, long long count, void* m, void* v, float* gsum,
                                         float* sumsq_partials, const float* scale_dev, float scale_host, float lr,
                                         float beta1, float beta2, float eps, float weight_decay, float inv_bc1,
                                         float inv_sqrt_bc2, int mode, const int* my_flags, int slot, int epoch, int* err,
                                         int grid_ctas, int bcast, int accumulate, void* stream) {
  if (world < 1 || world > kMaxRanks || (begin & 7) || (count & 7) || mode < 0 || mode > 2) return kErrBadShape;
  if (my_flags != nullptr && (slot < 0 || slot >= kMaxBuckets || err == nullptr)) return kErrBadShape;
  if (count == 0) return kOk;
  PeerTable t{};
  for (int r = 0; r < world; ++r) {
    t.grad[r] = static_cast<const __nv_bfloat16*>(grad_ptrs[r]);
    t.param[r] = static_cast<__nv_bfloat16*>(param_ptrs[r]);
  }
  const int full = ttb_dp_grid();
  const int grid = (grid_ctas > 0 && grid_ctas < full) ? grid_ctas : full;
  auto s = static_cast<cudaStream_t>(stream);
  auto mm = static_cast<__nv_bfloat16*>(m);
  auto vv = static_cast<__nv_bfloat16*>(v);
  const int* guard = nullptr;
  if (my_flags != nullptr && world > 1) {
    TTB_COUNT_LAUNCH(1);
    dp_wait_kernel<<<1, 32, 0, s>>>(my_flags, world, rank, slot, epoch, err, g_flag_wait_cycles);
    guard = err;
  }
  TTB_COUNT_LAUNCH(1);
#define TTB_DP_LAUNCH(W, MODE)                                                                                         \
  dp_reduce_adamw_bcast_kernel<W, MODE><<<grid, 256, 0, s>>>(t, rank, begin, count, mm, vv, gsum, sumsq_partials, scale_dev,   \
                                                             scale_host, lr, beta1, beta2, eps, weight_decay, inv_bc1,     \
                                                             inv_sqrt_bc2, guard, bcast, accumulate)
#define TTB_DP_CASE(W)                   \
  case W:                                \
    if (mode == 0) TTB_DP_LAUNCH(W, 0);  \
    else if (mode == 1) TTB_DP_LAUNCH(W, 1); \
    else TTB_DP_LAUNCH(W, 2);            \
    break;
  switch (world) {
    TTB_DP_CASE(1)
    TTB_DP_CASE(2)
    TTB_DP_CASE(3)
    TTB_DP_CASE(4)
    TTB_DP_CASE(6)
    TTB_DP_CASE(8)
    TTB_DP_CASE(16)
    default:
      return kErrBadShape;
  }
#undef TTB_DP_CASE
#undef TTB_DP_LAUNCH
  return cudaGetLastError() == cudaSuccess ? kOk : kErrDriver;
}

// shard_ptrs: `world` device pointers to the ranks' shards of one bucket (piece elements each, piece % 8 == 0); dst: local
// buffer of world · piece elements.  my_flags != null: wait first (bounded) until every peer's entry [peer][slot] has reached
// `epoch` (the peers' optimizer updates of this bucket are complete).
extern "C" int ttb_zero3_gather(void* const* shard_ptrs, int world, int rank, long long piece, void* dst, const int* my_flags, int slot,
                                int epoch, int* err, int grid_ctas, void* stream) {
  if (world < 1 || world > kMaxRanks || rank < 0 || rank >= world || piece <= 0 || (piece & 7)) return kErrBadShape;
  if (my_flags != nullptr && (slot < 0 || slot >= kMaxBuckets || err == nullptr)) return kErrBadShape;
  ShardTable t{};
  for (int r = 0; r < world; ++r) t.shard[r] = static_cast<const __nv_bfloat16*>(shard_ptrs[r]);
  const int full = ttb_dp_grid();
  const int grid = (grid_ctas > 0 && grid_ctas < full) ? grid_ctas : full;
  auto s = static_cast<cudaStream_t>(stream);
  const int* guard = nullptr;
  if (my_flags != nullptr && world > 1) {
    TTB_COUNT_LAUNCH(1);
    dp_wait_kernel<<<1, 32, 0, s>>>(my_flags, world, rank, slot, epoch, err, g_flag_wait_cycles);
    guard = err;
  }
  TTB_COUNT_LAUNCH(1);
  auto d = static_cast<__nv_bfloat16*>(dst);
#define TTB_Z3_CASE(W) \
  case W:              \
    zero3_gather_kernel<W><<<grid, 256, 0, s>>>(t, rank, piece, d, guard); \
    break;
  switch (world) {
    TTB_Z3_CASE(1)
    TTB_Z3_CASE(2)
    TTB_Z3_CASE(3)
    TTB_Z3_CASE(4)
    TTB_Z3_CASE(6)
    TTB_Z3_CASE(8)
    TTB_Z3_CASE(16)
    default:
      return kErrBadShape;
  }
#undef TTB_Z3_CASE
  return cudaGetLastError() == cudaSuccess ? kOk : kErrDriver;
}

// Bounded wait on this rank's flag array as a launch of its own: returns (in stream order) once every peer's entry
// [peer][slot] has reached `epoch`, or stores 201 in the error word when the cycle budget runs out.  Together with
// ttb_dp_signal this is a barrier between the ranks that needs no collective library.
extern "C" int ttb_dp_wait(const int* my_flags, int world, int rank, int slot, int epoch, int* err, void* stream) {
  if (world < 1 || world > kMaxRanks || rank < 0 || rank >= world || slot < 0 || slot >= kMaxBuckets || err == nullptr) return kErrBadShape;
  if (world == 1) return kOk;
  TTB_COUNT_LAUNCH(1);
  dp_wait_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(my_flags, world, rank, slot, epoch, err, g_flag_wait_cycles);
  return cudaGetLastError() == cudaSuccess ? kOk : kErrDriver;
}

// flag_ptrs: `world` device pointers, rank q's flag array int[world][4096] (peer-mapped).  Stores `epoch` into entry [rank][slot]
// of every peer's array; stream order makes it follow the work that completes this rank's gradients of that bucket.
extern "C" int ttb_dp_signal(void* const* flag_ptrs, int world, int rank, int slot, int epoch, void* stream) {
  if (world < 1 || world > kMaxRanks || rank < 0 || rank >= world || slot < 0 || slot >= kMaxBuckets) return kErrBadShape;
  FlagTable t{};
  for (int r = 0; r < world; ++r) t.flags[r] = static_cast<int*>(flag_ptrs[r]);
  TTB_COUNT_LAUNCH(1);
  dp_signal_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(t, world, rank, slot, epoch);
  return cudaGetLastError() == cudaSuccess ? kOk : kErrDriver;
}
extern "C" int ttb_dp_max_buckets() { return kMaxBuckets; }

// Cycle budget of the cross-rank flag wait (default 4e9 ≈ 2–3 s).  When it runs out the wait kernel stores 201 in the error word
// and the kernels that follow it return without touching parameters or optimizer state; the host raises on its next check.
extern "C" void ttb_dp_set_wait_cycles(long long cycles) { g_flag_wait_cycles = cycles > 0 ? cycles : 4000000000LL; }


// dst_ptrs: `world` device pointers (rank j's receive buffer, peer-mapped; entry `rank` is the own buffer).  Shapes in the kernel comment;
// every pointer 16-byte aligned.  The caller orders the launch between a "receive buffers are free" wait and a "data has arrived" signal.
extern "C" int ttb_cp_exchange(const void* src, void* const* dst_ptrs, int world, int rank, int mode, long long b, long long s_l, long long h_l, long long dv, void* stream) {
  if (world < 1 || world > kMaxRanks || rank < 0 || rank >= world || (mode != 0 && mode != 1) || b <= 0 || s_l <= 0 || h_l <= 0 || dv <= 0) return kErrBadShape;
  CpTable t{};
  for (int r = 0; r < world; ++r) {
    if (reinterpret_cast<uintptr_t>(dst_ptrs[r]) & 15) return kErrBadShape;
    t.dst[r] = static_cast<uint4*>(dst_ptrs[r]);
  }
  if (reinterpret_cast<uintptr_t>(src) & 15) return kErrBadShape;
  const long long total = b * s_l * h_l * dv * world;
  long long grid = (total + 255) / 256;
  const long long cap = static_cast<long long>(ttb_dp_grid());
  if (grid > cap) grid = cap;
  TTB_COUNT_LAUNCH(1);
  cp_exchange_kernel<<<static_cast<unsigned>(grid), 256, 0, static_cast<cudaStream_t>(stream)>>>(static_cast<const uint4*>(src), t, world, rank, mode, b, s_l, h_l, dv);
  return cudaGetLastError() == cudaSuccess ? kOk : kErrDriver;
}
