// Mixture-of-experts index kernels.
//
// 1. `ttb_moe_route_sort`: stable counting sort of the routed (token, slot) pairs by expert id.  Replaces the
//    `histc` + stable `argsort` pair of the router (torchtune/modules/moe/moe.py:55-84): one launch, one CTA,
//    output `counts[E]` (tokens per expert) and `order[n]` (the stable permutation that sorts `expert_ids`).
// 2. `ttb_moe_permute_indices`: gather indices that regroup rank-major runs into expert-major blocks padded to an
//    alignment (torchtune/modules/moe/indices.py:22-217, which fills with a Triton kernel after a host-side scan).
//    Here every output slot *pulls* its source index — no pre-fill with -1, no scan on the host, one launch.
#include "common/ptx.cuh"
#include "common/tmap.h"

namespace ttb {

constexpr int kSortThreads = 1024;
constexpr int kSortWarps = kSortThreads / 32;
constexpr int kMaxExperts = 256;

// One CTA walks the ids in rounds of 1024; in each round a warp ranks its 32 consecutive entries with match_any and
// the per-warp counts are prefix-summed through shared memory, which keeps the order of equal ids (stability).
// Pass 0 counts, an exclusive scan turns counts into bases, pass 1 scatters.
__global__ void __launch_bounds__(kSortThreads)
moe_route_sort_kernel(const long long* __restrict__ ids, int n, int num_experts, long long* __restrict__ counts,
                      long long* __restrict__ order, long long* __restrict__ inverse) {
  __shared__ int base[kMaxExperts];                 // running output position per expert
  __shared__ int warp_cnt[kSortWarps][kMaxExperts]; // per-round, per-warp counts
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  for (int e = tid; e < num_experts; e += kSortThreads) base[e] = 0;
  __syncthreads();
  // pass 0: histogram
  for (int i = tid; i < n; i += kSortThreads) {
    const int e = static_cast<int>(ids[i]);
    if (e >= 0 && e < num_experts) atomicAdd(&base[e], 1);
  }
  __syncthreads();
  if (tid == 0) {
    int run = 0;
    for (int e = 0; e < num_experts; ++e) {
      const int c = base[e];
      counts[e] = c;
      base[e] = run;
      run += c;
    }
  }
  __syncthreads();
  // pass 1: stable scatter
  for (int start = 0; start < n; start += kSortThreads) {
    for (int j = tid; j < kSortWarps * num_experts; j += kSortThreads) (&warp_cnt[0][0])[(j / num_experts) * kMaxExperts + j % num_experts] = 0;
    __syncthreads();
    const int i = start + tid;
    int e = -1;
    if (i < n) {
      e = static_cast<int>(ids[i]);
      if (e < 0 || e >= num_experts) e = -1;
    }
    const unsigned same = __match_any_sync(0xffffffffu, e);
    const int rank_in_warp = __popc(same & ((1u << lane) - 1u));
    if (e >= 0 && rank_in_warp == 0) warp_cnt[warp][e] = __popc(same);
    __syncthreads();
    if (e >= 0) {
      int pos = base[e] + rank_in_warp;
      for (int w = 0; w < warp; ++w) pos += warp_cnt[w][e];
      order[pos] = i;
      if (inverse != nullptr) inverse[i] = pos;  // position of entry i in expert order (entries with invalid ids keep their old value)
    }
    __syncthreads();
    for (int x = tid; x < num_experts; x += kSortThreads) {
      int add = 0;
      for (int w = 0; w < kSortWarps; ++w) add += warp_cnt[w][x];
      base[x] += add;
    }
    __syncthreads();
  }
}

// counts: [num_ranks, experts_per_rank] rows received from rank r for local expert e (rank-major runs in the input).
// Output slot p belongs to expert e (blocks padded to `alignment`, at least one alignment unit per expert); inside
// the block the runs of rank 0, 1, … follow each other; slots past the expert's rows are -1.
__global__ void __launch_bounds__(256)
moe_permute_indices_kernel(const long long* __restrict__ counts, int experts_per_rank, int num_ranks, int max_len,
                           int alignment, int* __restrict__ permuted, int* __restrict__ m_sizes, int* __restrict__ m_offsets) {
  extern __shared__ int sm[];
  int* in_start = sm;                                  // [R*E] start of run (r, e) in the rank-major input
  int* within = in_start + num_ranks * experts_per_rank;  // [R*E] start of run (r, e) inside expert e's block
  int* out_start = within + num_ranks * experts_per_rank; // [E]
  int* rows_of = out_start + experts_per_rank;            // [E]
  int* out_end = rows_of + experts_per_rank;              // [E] padded end
  if (threadIdx.x == 0) {
    int run = 0;
    for (int i = 0; i < num_ranks * experts_per_rank; ++i) {
      in_start[i] = run;
      run += static_cast<int>(counts[i]);
    }
    int off = 0;
    for (int e = 0; e < experts_per_rank; ++e) {
      int tot = 0;
      for (int r = 0; r < num_ranks; ++r) {
        within[r * experts_per_rank + e] = tot;
        tot += static_cast<int>(counts[r * experts_per_rank + e]);
      }
      int padded = (tot + alignment - 1) / alignment * alignment;
      if (padded < alignment) padded = alignment;
      out_start[e] = off;
      rows_of[e] = tot;
      off += padded;
      out_end[e] = off;
      if (blockIdx.x == 0) {
        m_sizes[e] = padded;
        m_offsets[e] = off;
      }
    }
  }
  __syncthreads();
  for (int p = blockIdx.x * blockDim.x + threadIdx.x; p < max_len; p += gridDim.x * blockDim.x) {
    int e = 0;
    while (e < experts_per_rank && p >= out_end[e]) ++e;
    int v = -1;
    if (e < experts_per_rank) {
      const int q = p - out_start[e];
      if (q < rows_of[e]) {
        int r = num_ranks - 1;
        while (r > 0 && within[r * experts_per_rank + e] > q) --r;
        v = in_start[r * experts_per_rank + e] + (q - within[r * experts_per_rank + e]);
      }
    }
    permuted[p] = v;
  }
}

}  // namespace ttb

// inverse (optional, [n] int64): inverse[i] = position of entry i in the sorted order.
extern "C" int ttb_moe_route_sort(const void* expert_ids, int n, int num_experts, void* counts, void* order, void* inverse, void* stream) {
  using namespace ttb;
  if (n < 0 || num_experts <= 0 || num_experts > kMaxExperts) return kErrBadShape;
  TTB_COUNT_LAUNCH(1);
  moe_route_sort_kernel<<<1, kSortThreads, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const long long*>(expert_ids), n, num_experts, static_cast<long long*>(counts), static_cast<long long*>(order), static_cast<long long*>(inverse));
  return cudaGetLastError() == cudaSuccess ? kOk : kErrDriver;
}

extern "C" int ttb_moe_permute_indices(const void* counts, int experts_per_rank, int num_ranks, int max_len, int alignment,
                                       void* permuted, void* m_sizes, void* m_offsets, void* stream) {
  using namespace ttb;
  const long long runs = static_cast<long long>(experts_per_rank) * num_ranks;
  if (experts_per_rank <= 0 || num_ranks <= 0 || max_len <= 0 || alignment <= 0 || runs > 4096) return kErrBadShape;
  const size_t smem = (2 * runs + 3 * experts_per_rank) * sizeof(int);
  int blocks = (max_len + 255) / 256;
  if (blocks > sm_count() * 4) blocks = sm_count() * 4;
  TTB_COUNT_LAUNCH(1);
  moe_permute_indices_kernel<<<blocks, 256, smem, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const long long*>(counts), experts_per_rank, num_ranks, max_len, alignment, static_cast<int*>(permuted),
      static_cast<int*>(m_sizes), static_cast<int*>(m_offsets));
  return cudaGetLastError() == cudaSuccess ? kOk : kErrDriver;
}
