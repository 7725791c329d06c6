// Token-embedding lookup and its gradient (reference call site: torchtune/modules/transformer.py:652, nn.Embedding).
//
// Forward is a row gather with 16-byte accesses.  The gradient is a scatter-add of `dy` rows into the rows of the
// table.  Instead of atomics (bf16 atomics lose low bits when a frequent token receives thousands of rows, and their
// order is not reproducible) the token ids are sorted first; every run of equal ids is then summed in fp32 by one
// CTA column-slice and added to the table row exactly once.  The result is deterministic.
#include "common/ptx.cuh"
#include "common/tmap.h"

TTB_DEFINE_VIOLATION_COUNTER(embedding)

namespace ttb {

__global__ void __launch_bounds__(256)
embedding_fwd_kernel(const long long* __restrict__ ids, const uint4* __restrict__ table, uint4* __restrict__ out,
                     long long n_tokens, int vec_per_row, long long vocab) {
  for (long long t = blockIdx.x; t < n_tokens; t += gridDim.x) {
    long long id = ids[t];
    if (id < 0 || id >= vocab) {  // never read out of bounds: row 0 stands in and the event is counted
      if (threadIdx.x == 0) TTB_NOTE_VIOLATION(embedding);
      id = 0;
    }
    const uint4* src = table + id * vec_per_row;
    uint4* dst = out + t * vec_per_row;
    for (int v = threadIdx.x; v < vec_per_row; v += blockDim.x) dst[v] = src[v];
  }
}

// sorted_ids[p] ascending, order[p] = row of dy that carries sorted_ids[p].  blockIdx.y selects a 2048-column slice.
__global__ void __launch_bounds__(256)
embedding_bwd_kernel(const long long* __restrict__ sorted_ids, const long long* __restrict__ order,
                     const __nv_bfloat16* __restrict__ dy, __nv_bfloat16* __restrict__ dtable, long long n_tokens, int dim,
                     long long vocab, long long padding_idx) {
  const int col = (blockIdx.y * 256 + threadIdx.x) * 8;
  for (long long p = blockIdx.x; p < n_tokens; p += gridDim.x) {
    const long long id = sorted_ids[p];
    if (p > 0 && sorted_ids[p - 1] == id) continue;  // not the head of a run (uniform over the CTA)
    if (id < 0 || id >= vocab || id == padding_idx || col >= dim) continue;
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    for (long long q = p; q < n_tokens && sorted_ids[q] == id; ++q) {
      const uint4 v = *reinterpret_cast<const uint4*>(dy + order[q] * dim + col);
      const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float2 f = __bfloat1622float2(h[i]);
        acc[2 * i] += f.x;
        acc[2 * i + 1] += f.y;
      }
    }
    uint4* dst = reinterpret_cast<uint4*>(dtable + id * dim + col);
    const uint4 old = *dst;
    const __nv_bfloat162* ho = reinterpret_cast<const __nv_bfloat162*>(&old);
    uint32_t o[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float2 f = __bfloat1622float2(ho[i]);
      o[i] = pack_bf16x2(acc[2 * i] + f.x, acc[2 * i + 1] + f.y);
    }
    *dst = make_uint4(o[0], o[1], o[2], o[3]);
  }
}

}  // namespace ttb

// out[t, :] = table[ids[t], :]; dim a multiple of 8 bf16 (16 bytes), both pointers 16-byte aligned.
extern "C" int ttb_embedding_fwd(const void* ids, const void* table, void* out, long long n_tokens, int dim, long long vocab,
                                 void* stream) {
  using namespace ttb;
  if (n_tokens <= 0 || dim <= 0 || (dim & 7) || vocab <= 0) return kErrBadShape;
  if ((reinterpret_cast<uintptr_t>(table) & 15) || (reinterpret_cast<uintptr_t>(out) & 15)) return kErrBadShape;
  long long blocks = n_tokens;
  const long long cap = static_cast<long long>(sm_count()) * 16;
  if (blocks > cap) blocks = cap;
  TTB_COUNT_LAUNCH(1);
  embedding_fwd_kernel<<<static_cast<int>(blocks), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const long long*>(ids), static_cast<const uint4*>(table), static_cast<uint4*>(out), n_tokens, dim / 8, vocab);
  return cudaGetLastError() == cudaSuccess ? kOk : kErrDriver;
}

// dtable[id, :] += Σ_{p: sorted_ids[p] == id} dy[order[p], :]   (rows of other ids are left untouched).
extern "C" int ttb_embedding_bwd(const void* sorted_ids, const void* order, const void* dy, void* dtable, long long n_tokens,
                                 int dim, long long vocab, long long padding_idx, void* stream) {
  using namespace ttb;
  if (n_tokens <= 0 || dim <= 0 || (dim & 7) || vocab <= 0) return kErrBadShape;
  if ((reinterpret_cast<uintptr_t>(dy) & 15) || (reinterpret_cast<uintptr_t>(dtable) & 15)) return kErrBadShape;
  long long bx = n_tokens;
  if (bx > 65535LL * 32) bx = 65535LL * 32;
  dim3 grid(static_cast<unsigned>(bx), static_cast<unsigned>((dim + 2047) / 2048));
  TTB_COUNT_LAUNCH(1);
  embedding_bwd_kernel<<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const long long*>(sorted_ids), static_cast<const long long*>(order), static_cast<const __nv_bfloat16*>(dy),
      static_cast<__nv_bfloat16*>(dtable), n_tokens, dim, vocab, padding_idx);
  return cudaGetLastError() == cudaSuccess ? kOk : kErrDriver;
}
