// Expert-parallel token exchange over NVLink peer memory.
//
// The reference routes tokens to experts on one device (torchtune/modules/moe/moe.py:111-186) and has no expert
// parallelism; an all-to-all based design would permute rows by expert, exchange them with a collective and permute the
// received rows again into expert-major order (torchtune/modules/moe/indices.py:144-217).  Here the three steps are one
// kernel: every rank knows all ranks' per-expert counts, so it can compute the final expert-major row of each of its
// routed (token, expert) pairs on the destination rank and *stores the row there directly* (`ep_push`).  The way back
// (`ep_pull`) loads each pair's result row from the peer that computed it.  No intermediate send/receive buffers, no
// second permutation, and no host synchronisation: the plan is built on the device from device-resident counts.
//
//   ttb_ep_plan   counts of all ranks → for every local pair its (destination rank, destination row) and the number
//                 of rows this rank receives per local expert
//   ttb_ep_push   x[token[j]] (· scale[j]) → recv_buffer[dest_rank[j]][dest_row[j]]
//   ttb_ep_pull   out[j] = result_buffer[dest_rank[j]][dest_row[j]]
//
// Ordering between ranks (counts visible before the plan, pushed rows visible before the expert GEMMs, results
// complete before the pull) is the caller's job: stream-ordered barriers between the launches.  No kernel here waits.
#include "common/ptx.cuh"
#include "common/tmap.h"

namespace ttb {

static constexpr int kMaxEpWorld = 8;
struct EpPeers {
  void* ptr[kMaxEpWorld];
};

// One CTA.  counts[r] → int64 [num_experts] of rank r (expert e lives on rank e / experts_per_rank).
// pair j of this rank (pairs sorted by expert, stable) goes to rank d = e / experts_per_rank, row
//   row0_d(e) + Σ_{r < rank} counts[r][e] + (j − first pair of e),   row0_d(e) = Σ_{e' < e on d} Σ_r counts[r][e'].
__global__ void __launch_bounds__(1024)
ep_plan_kernel(EpPeers counts, int world, int rank, int num_experts, int experts_per_rank, long long n_pairs,
               int* __restrict__ dest_rank, int* __restrict__ dest_row, long long* __restrict__ recv_counts,
               int* __restrict__ recv_total) {
  extern __shared__ long long sm[];
  long long* base = sm;                      // [E] destination row of this rank's first pair of expert e
  long long* first = sm + num_experts;       // [E + 1] first local pair of expert e
  long long* cnt = first + num_experts + 1;  // [world, E] all ranks' counts (one round of peer loads, in parallel)
  for (int i = threadIdx.x; i < world * num_experts; i += blockDim.x)
    cnt[i] = __ldcg(static_cast<const long long*>(counts.ptr[i / num_experts]) + i % num_experts);
  __syncthreads();
  if (threadIdx.x == 0) {
    long long run = 0;
    for (int e = 0; e < num_experts; ++e) {
      first[e] = run;
      run += cnt[rank * num_experts + e];
    }
    first[num_experts] = run;
    long long row0 = 0;
    for (int e = 0; e < num_experts; ++e) {
      if (e % experts_per_rank == 0) row0 = 0;
      long long before = 0, total = 0;
      for (int r = 0; r < world; ++r) {
        const long long c = cnt[r * num_experts + e];
        if (r < rank) before += c;
        total += c;
      }
      base[e] = row0 + before;
      if (e / experts_per_rank == rank) recv_counts[e - rank * experts_per_rank] = total;
      row0 += total;
      if (e / experts_per_rank == rank && e % experts_per_rank == experts_per_rank - 1) *recv_total = static_cast<int>(row0);
    }
  }
  __syncthreads();
  for (long long j = threadIdx.x; j < n_pairs; j += blockDim.x) {
    int lo = 0, hi = num_experts;  // largest e with first[e] <= j (first[E] = n_pairs > j)
    while (hi - lo > 1) {
      const int mid = (lo + hi) >> 1;
      if (first[mid] <= j) lo = mid; else hi = mid;
    }
    const int e = lo;  // empty experts share their start with the next one; the search lands on the last of them
    dest_rank[j] = e / experts_per_rank;
    dest_row[j] = static_cast<int>(base[e] + (j - first[e]));
  }
}

// One CTA per pair (grid-stride); 16-byte vectors; optional per-pair scale in fp32.
__global__ void __launch_bounds__(256)
ep_push_kernel(const __nv_bfloat16* __restrict__ x, const long long* __restrict__ token, const __nv_bfloat16* __restrict__ scale,
               const int* __restrict__ dest_rank, const int* __restrict__ dest_row, EpPeers recv, long long n_pairs, int dim,
               long long capacity) {
  const int vecs = dim / 8;
  for (long long j = blockIdx.x; j < n_pairs; j += gridDim.x) {
    const long long row = dest_row[j];
    if (row < 0 || row >= capacity) continue;  // cannot happen with a worst-case capacity; never write out of bounds
    const uint4* src = reinterpret_cast<const uint4*>(x + (token ? token[j] : j) * dim);
    uint4* dst = reinterpret_cast<uint4*>(static_cast<__nv_bfloat16*>(recv.ptr[dest_rank[j]]) + row * dim);
    const float sc = scale ? __bfloat162float(scale[j]) : 1.f;
    for (int v = threadIdx.x; v < vecs; v += blockDim.x) {
      uint4 val = src[v];
      if (scale) {
        __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&val);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const float2 f = __bfloat1622float2(h[i]);
          // same rounding as the single-device path: the product of two bf16 values rounded to bf16
          h[i] = __floats2bfloat162_rn(f.x * sc, f.y * sc);
        }
      }
      dst[v] = val;
    }
  }
}

__global__ void __launch_bounds__(256)
ep_pull_kernel(EpPeers result, const int* __restrict__ dest_rank, const int* __restrict__ dest_row, __nv_bfloat16* __restrict__ out,
               long long n_pairs, int dim, long long capacity) {
  const int vecs = dim / 8;
  for (long long j = blockIdx.x; j < n_pairs; j += gridDim.x) {
    const long long row = dest_row[j];
    uint4* dst = reinterpret_cast<uint4*>(out + j * dim);
    if (row < 0 || row >= capacity) {
      for (int v = threadIdx.x; v < vecs; v += blockDim.x) dst[v] = make_uint4(0, 0, 0, 0);
      continue;
    }
    const uint4* src = reinterpret_cast<const uint4*>(static_cast<const __nv_bfloat16*>(result.ptr[dest_rank[j]]) + row * dim);
    for (int v = threadIdx.x; v < vecs; v += blockDim.x) dst[v] = __ldcg(src + v);
  }
}

static int fill_peers(EpPeers& p, const void* const* ptrs, int world) {
  if (world < 1 || world > kMaxEpWorld) return kErrBadShape;
  for (int r = 0; r < kMaxEpWorld; ++r) p.ptr[r] = r < world ? const_cast<void*>(ptrs[r]) : nullptr;
  return kOk;
}

}  // namespace ttb

extern "C" int ttb_ep_plan(const void* const* counts_ranks, int world, int rank, int num_experts, long long n_pairs, void* dest_rank,
                           void* dest_row, void* recv_counts, void* recv_total, void* stream) {
  using namespace ttb;
  EpPeers c;
  if (fill_peers(c, counts_ranks, world) != kOk) return kErrBadShape;
  if (rank < 0 || rank >= world || num_experts <= 0 || num_experts % world || num_experts > 512 || n_pairs < 0) return kErrBadShape;
  const size_t smem = sizeof(long long) * (2 * num_experts + 1 + static_cast<size_t>(world) * num_experts);
  TTB_COUNT_LAUNCH(1);
  ep_plan_kernel<<<1, 1024, smem, static_cast<cudaStream_t>(stream)>>>(c, world, rank, num_experts, num_experts / world, n_pairs,
                                                                       static_cast<int*>(dest_rank), static_cast<int*>(dest_row),
                                                                       static_cast<long long*>(recv_counts), static_cast<int*>(recv_total));
  return cudaGetLastError() == cudaSuccess ? kOk : kErrDriver;
}

// x: [*, dim] bf16 local; token: int64 [n_pairs] row of x per pair (nullptr: pair j reads row j); scale: bf16 [n_pairs] or nullptr;
// recv_ranks[r]: rank r's receive buffer [capacity, dim] bf16 (peer memory, written by plain stores).
extern "C" int ttb_ep_push(const void* x, const void* token, const void* scale, const void* dest_rank, const void* dest_row,
                           const void* const* recv_ranks, int world, long long n_pairs, int dim, long long capacity, void* stream) {
  using namespace ttb;
  EpPeers r;
  if (fill_peers(r, recv_ranks, world) != kOk) return kErrBadShape;
  if (n_pairs < 0 || dim <= 0 || (dim & 7) || capacity <= 0) return kErrBadShape;
  if (n_pairs == 0) return kOk;
  long long blocks = n_pairs;
  const long long cap = static_cast<long long>(sm_count()) * 16;
  if (blocks > cap) blocks = cap;
  TTB_COUNT_LAUNCH(1);
  ep_push_kernel<<<static_cast<int>(blocks), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(x), static_cast<const long long*>(token), static_cast<const __nv_bfloat16*>(scale),
      static_cast<const int*>(dest_rank), static_cast<const int*>(dest_row), r, n_pairs, dim, capacity);
  return cudaGetLastError() == cudaSuccess ? kOk : kErrDriver;
}

// out[j, :] = result_ranks[dest_rank[j]][dest_row[j], :]  (peer memory read by plain loads).
extern "C" int ttb_ep_pull(const void* const* result_ranks, int world, const void* dest_rank, const void* dest_row, void* out,
                           long long n_pairs, int dim, long long capacity, void* stream) {
  using namespace ttb;
  EpPeers r;
  if (fill_peers(r, result_ranks, world) != kOk) return kErrBadShape;
  if (n_pairs < 0 || dim <= 0 || (dim & 7) || capacity <= 0) return kErrBadShape;
  if (n_pairs == 0) return kOk;
  long long blocks = n_pairs;
  const long long cap = static_cast<long long>(sm_count()) * 16;
  if (blocks > cap) blocks = cap;
  TTB_COUNT_LAUNCH(1);
  ep_pull_kernel<<<static_cast<int>(blocks), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      r, static_cast<const int*>(dest_rank), static_cast<const int*>(dest_row), static_cast<__nv_bfloat16*>(out), n_pairs, dim, capacity);
  return cudaGetLastError() == cudaSuccess ? kOk : kErrDriver;
}
