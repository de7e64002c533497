// Rows of a step and short causal convolutions over them, shared by the mixers that keep a short history
// (seq_recurrent.cu, seq_ssd.cu).
//
// Filters inside a step.  Row t of an entry reads the entry's earlier rows straight from the step's projection and what
// lies before the entry from the state ([slots][taps - 1][channels] fp32).  The CTA of an entry's FIRST row also computes
// the entry's next taps - 2 rows -- so every read of the old state happens in that CTA -- and then writes the new state;
// CTAs of later rows never touch the state, and the rows in between have no CTA work of their own.
#pragma once
#include <cuda_runtime.h>

#include <cstdint>

#include "seq_engine.h"

namespace kllm {
namespace seq {
namespace {

// asynchronous copies into shared memory: a chunk of rows is on its way while the one before it is worked on
__device__ __forceinline__ void cp_async4(float* dst, const float* src) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(static_cast<uint32_t>(__cvta_generic_to_shared(dst))), "l"(src));
}
__device__ __forceinline__ void cp_async16(float* dst, const float* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(static_cast<uint32_t>(__cvta_generic_to_shared(dst))), "l"(src));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.wait_group 0;" ::: "memory"); }

// the entry that holds row t: the last e with ent_first[e] <= t
__device__ __forceinline__ int entry_of(const StepRows& r, int t) {
  int lo = 0, hi = r.n_entries - 1;
  while (lo < hi) {
    const int mid = (lo + hi + 1) >> 1;
    if (r.ent_first[mid] <= t) lo = mid;
    else hi = mid - 1;
  }
  return lo;
}

// Where a CTA stands in its entry.
struct RowPlace {
  int first, count, pos0, seq;
  int j0;      // index of the CTA's row inside the entry
  int n_here;  // rows this CTA computes (0: none -- the entry's first CTA has them)
};
__device__ __forceinline__ RowPlace place_row(const StepRows& r, int t, int taps) {
  RowPlace p;
  const int e = entry_of(r, t);
  p.first = r.ent_first[e], p.count = r.ent_count[e], p.pos0 = r.ent_pos0[e], p.seq = r.tok_seq[t];
  p.j0 = t - p.first;
  const int hist = taps - 1;
  if (p.j0 == 0) p.n_here = min(p.count, max(hist, 1));
  else p.n_here = p.j0 < hist ? 0 : 1;
  return p;
}

// One filtered value: channel c of the row at position `pos` (row `first + pos - pos0` of the step).  in: the step's
// inputs, `stride` floats per row; bias (optional) is added to every input; st: the sequence's state (row i = position
// pos0 - hist + i).
__device__ __forceinline__ float conv_at(const float* __restrict__ in, int stride, int c, int C, int taps,
                                         const float* __restrict__ w, const float* __restrict__ bias,
                                         const float* __restrict__ st, const RowPlace& p, int pos) {
  const int hist = taps - 1;
  const float b = bias ? bias[c] : 0.f;
  float acc = 0.f;
  for (int k = 0; k < taps; ++k) {
    const int sp = pos - hist + k;
    if (sp < 0) continue;
    const float u = sp >= p.pos0 ? in[static_cast<size_t>(p.first + sp - p.pos0) * stride + c] + b
                                 : st[static_cast<size_t>(hist - (p.pos0 - sp)) * C + c];
    acc = fmaf(w ? w[c * taps + k] : (k == hist ? 1.0f : 0.f), u, acc);  // no weights: the row itself
  }
  return acc;
}

// The state after the entry: row i = the input at position end - hist + i.  In place: row i only reads old rows >= i.
// Channels c0 .. c0 + n - 1 only (the CTA's own).
__device__ __forceinline__ void conv_state_write(const float* __restrict__ in, int stride, int C, int taps,
                                                 const float* __restrict__ bias, float* __restrict__ st, const RowPlace& p,
                                                 int c0, int n) {
  const int hist = taps - 1, end = p.pos0 + p.count;
  for (int c = c0 + threadIdx.x; c < c0 + n; c += blockDim.x) {
    const float b = bias ? bias[c] : 0.f;
    for (int i = 0; i < hist; ++i) {
      const int sp = end - hist + i;
      float v = 0.f;
      if (sp >= p.pos0) v = in[static_cast<size_t>(p.first + sp - p.pos0) * stride + c] + b;
      else if (sp >= 0) v = st[static_cast<size_t>(hist - (p.pos0 - sp)) * C + c];
      st[static_cast<size_t>(i) * C + c] = v;
    }
  }
}

}  // namespace
}  // namespace seq
}  // namespace kllm
