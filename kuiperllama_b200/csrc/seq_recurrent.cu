// Mixers of the sequence-batch engine whose memory is a short history and a recurrent state instead of (or beside) a
// key/value cache:
//   short convolutions   a causal filter of `taps` taps per channel over the rows of a sequence; the last taps - 1 inputs
//                        are state of the sequence ([slots][taps - 1][channels] fp32)
//   qk_conv_prepare      query / key preparation for an attention whose projections pass such a filter: bias, filter, the
//                        keys as they are into the value pages, rotary positions, queries out and keys into the key pages
//   selective scan       ssm_conv (filter + SiLU) and ssm_scan (input-dependent steps, a diagonal state per channel)
//   gated delta rule     delta_prepare (filter + SiLU, unit vectors, beta, decays, gates), delta_rule (the recurrence over a
//                        matrix state per head) and delta_out (per-head RMS norm and gate)
// Everything here is fp32 except what leaves for a matrix product (compute type AT).
//
// Filters inside a step.  Row t of an entry reads the entry's earlier rows straight from the step's projection and what
// lies before the entry from the state.  The CTA of an entry's FIRST row also computes the entry's next taps - 2 rows --
// so every read of the old state happens in that CTA -- and then writes the new state; CTAs of later rows never touch
// the state, and the rows in between have no CTA work of their own.
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <algorithm>
#include <cstdint>

#include "seq_engine.h"

namespace kllm {
namespace seq {
namespace {

constexpr unsigned kAll = 0xffffffffu;

template <typename AT> __device__ __forceinline__ AT from_f(float v);
template <> __device__ __forceinline__ float from_f<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 from_f<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(kAll, v, o);
  return v;
}
__device__ __forceinline__ float sigmoidf(float z) { return 1.0f / (1.0f + expf(-z)); }
__device__ __forceinline__ float siluf(float z) { return z / (1.0f + expf(-z)); }
__device__ __forceinline__ float softplusf(float z) { return z > 20.0f ? z : log1pf(expf(z)); }

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
__device__ __forceinline__ void conv_state_write(const float* __restrict__ in, int stride, int C, int taps,
                                                 const float* __restrict__ bias, float* __restrict__ st, const RowPlace& p) {
  const int hist = taps - 1, end = p.pos0 + p.count;
  for (int c = threadIdx.x; c < C; c += blockDim.x) {
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

// ---- attention behind a filter ------------------------------------------------------------------------------------------
template <typename AT>
__device__ __forceinline__ AT* page_row(AT* base, const PagedKV& kv, int seq, int pos, int row) {
  const int page = kv.table[static_cast<size_t>(seq) * kv.table_stride + pos / kv.page];
  return base + (static_cast<size_t>(page) * kv.page + pos % kv.page) * row;
}

template <typename AT>
__global__ void qk_conv_prepare_kernel(AttnShape a, AttnPrep pr, const float* __restrict__ qk, StepRows rows,
                                       AT* __restrict__ q, PagedKV kv) {
  extern __shared__ float cs[];  // [C] the filtered row
  const RowPlace p = place_row(rows, blockIdx.x, pr.taps);
  if (p.n_here == 0) return;
  const int qn = a.heads * a.dim, C = qn + a.kv_heads * a.dim, hist = pr.taps - 1;
  float* st = hist > 0 ? pr.conv_state + static_cast<size_t>(p.seq) * hist * C : nullptr;
  const int rd = pr.rope_dims, half = rd / 2;
  for (int jj = 0; jj < p.n_here; ++jj) {
    const int t = blockIdx.x + jj, pos = p.pos0 + p.j0 + jj;
    for (int c = threadIdx.x; c < C; c += blockDim.x) cs[c] = conv_at(qk, C, c, C, pr.taps, pr.conv_w, pr.bias, st, p, pos);
    __syncthreads();
    AT* krow = page_row(static_cast<AT*>(kv.k), kv, p.seq, pos, kv.k_row);
    AT* vrow = page_row(static_cast<AT*>(kv.v), kv, p.seq, pos, kv.v_row);
    for (int c = threadIdx.x; c < C; c += blockDim.x) {
      const bool is_q = c < qn;
      const int d = (is_q ? c : c - qn) % a.dim;
      float v = cs[c];
      if (!is_q) vrow[c - qn] = from_f<AT>(v);  // the values: keys before the rotation
      if (d < rd) {
        int i, partner;
        bool lead;  // the member of the pair that becomes u cos - v sin
        if (pr.rope_pairing == KLLM_SEQ_ROPE_PAIRS) i = d >> 1, partner = d ^ 1, lead = (d & 1) == 0;
        else lead = d < half, i = lead ? d : d - half, partner = lead ? d + half : d - half;
        const float freq = powf(pr.rope_base, -2.0f * static_cast<float>(i) / static_cast<float>(rd));
        const float ang = static_cast<float>(pos) * freq;
        const float co = cosf(ang), si = sinf(ang);
        const float o = cs[c - d + partner];
        v = lead ? v * co - o * si : v * co + o * si;
      }
      if (is_q) q[static_cast<size_t>(t) * qn + c] = from_f<AT>(v);
      else krow[c - qn] = from_f<AT>(v);
    }
    __syncthreads();
  }
  if (p.j0 == 0 && hist > 0) conv_state_write(qk, C, C, pr.taps, pr.bias, st, p);
}

// ---- selective scan ----------------------------------------------------------------------------------------------------
template <typename AT>
__global__ void ssm_conv_kernel(int inner, int taps, const float* __restrict__ conv_w, const float* __restrict__ conv_b,
                                const float* __restrict__ uz, float* __restrict__ conv_state, StepRows rows,
                                float* __restrict__ uc, AT* __restrict__ uc_ct) {
  const RowPlace p = place_row(rows, blockIdx.x, taps);
  if (p.n_here == 0) return;
  const int hist = taps - 1;
  float* st = hist > 0 ? conv_state + static_cast<size_t>(p.seq) * hist * inner : nullptr;
  for (int jj = 0; jj < p.n_here; ++jj) {
    const int t = blockIdx.x + jj, pos = p.pos0 + p.j0 + jj;
    for (int c = threadIdx.x; c < inner; c += blockDim.x) {
      const float v = siluf(conv_at(uz, 2 * inner, c, inner, taps, conv_w, nullptr, st, p, pos) + (conv_b ? conv_b[c] : 0.f));
      uc[static_cast<size_t>(t) * inner + c] = v;
      uc_ct[static_cast<size_t>(t) * inner + c] = from_f<AT>(v);
    }
  }
  if (p.j0 == 0 && hist > 0) {
    __syncthreads();
    conv_state_write(uz, 2 * inner, inner, taps, nullptr, st, p);
  }
}

constexpr int kScanThreads = 128;
constexpr int kScanChunk = 32;   // rows staged in shared memory at a time
constexpr int kScanPerLane = 4;  // states per thread: up to 32 lanes share a channel, so state <= 128

// One CTA: one entry, CH = kScanThreads / L channels; L lanes share a channel and hold its states n = lane, lane + L, ...
// Chunks of kScanChunk rows are staged in shared memory (the low-rank rows, u, z), the step sizes of the chunk are
// computed by all threads, then the recurrence runs over the chunk's rows.
template <typename AT>
__global__ void __launch_bounds__(kScanThreads)
ssm_scan_kernel(kllm_seq_ssm m, int L, const float* __restrict__ uz, const float* __restrict__ uc,
                const float* __restrict__ low, float* __restrict__ state, StepRows rows,
                const int32_t* __restrict__ ent_seq, AT* __restrict__ out) {
  const int e = blockIdx.y;
  const int first = rows.ent_first[e], count = rows.ent_count[e], pos0 = rows.ent_pos0[e], seq = ent_seq[e];
  const int CH = kScanThreads / L;
  const int c0 = blockIdx.x * CH;
  const int lane = threadIdx.x % L, cl = threadIdx.x / L, c = c0 + cl;
  const bool live = c < m.inner;
  const int R = m.dt_rank, N = m.state, LW = R + 2 * N;
  extern __shared__ float sm[];
  float* low_s = sm;                          // [chunk][LW]
  float* u_s = low_s + kScanChunk * LW;       // [chunk][CH]
  float* z_s = u_s + kScanChunk * CH;         // [chunk][CH]
  float* dt_s = z_s + kScanChunk * CH;        // [chunk][CH]
  float* y_s = dt_s + kScanChunk * CH;        // [chunk][CH]

  float S[kScanPerLane], A[kScanPerLane];
  float* st = state + (static_cast<size_t>(seq) * m.inner + (live ? c : 0)) * N;
#pragma unroll
  for (int k = 0; k < kScanPerLane; ++k) {
    const int n = lane + k * L;
    const bool on = live && n < N;
    S[k] = on && pos0 > 0 ? st[n] : 0.f;
    A[k] = on ? m.a[static_cast<size_t>(c) * N + n] : 0.f;
  }
  const float dskip = live ? m.d[c] : 0.f;
  for (int r0 = 0; r0 < count; r0 += kScanChunk) {
    const int nr = min(kScanChunk, count - r0);
    __syncthreads();
    for (int i = threadIdx.x; i < nr * LW; i += kScanThreads)
      low_s[i] = low[static_cast<size_t>(first + r0) * LW + i];
    for (int i = threadIdx.x; i < nr * CH; i += kScanThreads) {
      const int r = i / CH, cc = c0 + i % CH;
      const size_t row = static_cast<size_t>(first + r0 + r);
      u_s[i] = cc < m.inner ? uc[row * m.inner + cc] : 0.f;
      z_s[i] = cc < m.inner ? uz[row * 2 * m.inner + m.inner + cc] : 0.f;
    }
    __syncthreads();
    for (int i = threadIdx.x; i < nr * CH; i += kScanThreads) {
      const int r = i / CH, cc = c0 + i % CH;
      float acc = 0.f;
      if (cc < m.inner) {
        const float* wr = m.w_dt + static_cast<size_t>(cc) * R;
        for (int k = 0; k < R; ++k) acc = fmaf(wr[k], low_s[r * LW + k], acc);
        acc = softplusf(acc + m.dt_b[cc]);
      }
      dt_s[i] = acc;
    }
    __syncthreads();
    for (int r = 0; r < nr; ++r) {
      const float dt = dt_s[r * CH + cl], u = u_s[r * CH + cl];
      const float du = dt * u;
      const float* Bn = low_s + r * LW + R;
      const float* Cn = Bn + N;
      float y = 0.f;
#pragma unroll
      for (int k = 0; k < kScanPerLane; ++k) {
        const int n = lane + k * L;
        if (n < N) {
          S[k] = fmaf(expf(dt * A[k]), S[k], du * Bn[n]);
          y = fmaf(S[k], Cn[n], y);
        }
      }
      for (int o = L >> 1; o > 0; o >>= 1) y += __shfl_xor_sync(kAll, y, o);
      if (lane == 0) y_s[r * CH + cl] = (y + dskip * u) * siluf(z_s[r * CH + cl]);
    }
    __syncthreads();
    for (int i = threadIdx.x; i < nr * CH; i += kScanThreads) {
      const int r = i / CH, cc = c0 + i % CH;
      if (cc < m.inner) out[static_cast<size_t>(first + r0 + r) * m.inner + cc] = from_f<AT>(y_s[i]);
    }
  }
#pragma unroll
  for (int k = 0; k < kScanPerLane; ++k) {
    const int n = lane + k * L;
    if (live && n < N) st[n] = S[k];
  }
}

// ---- gated delta rule ---------------------------------------------------------------------------------------------------
// One CTA per row (see the note on filters at the top).  Shared memory: the filtered q | k | v row, then the two low-rank rows.
__global__ void delta_prepare_kernel(kllm_seq_delta m, const float* __restrict__ proj, float* __restrict__ conv_state,
                                     StepRows rows, float* __restrict__ prep) {
  extern __shared__ float cs[];
  const RowPlace p = place_row(rows, blockIdx.x, m.conv_taps);
  if (p.n_here == 0) return;
  const int qn = m.kv_heads * m.dim, vn = m.heads * m.vdim, C = 2 * qn + vn, hist = m.conv_taps - 1;
  const int stride = C + m.heads + m.decay_rank + m.gate_rank;
  const int prow = delta_prep_row(m);
  float* st = hist > 0 ? conv_state + static_cast<size_t>(p.seq) * hist * C : nullptr;
  float* lowa = cs + C;               // [decay_rank]
  float* lowg = lowa + m.decay_rank;  // [gate_rank]
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
  for (int jj = 0; jj < p.n_here; ++jj) {
    const int t = blockIdx.x + jj, pos = p.pos0 + p.j0 + jj;
    const float* row = proj + static_cast<size_t>(t) * stride;
    float* dst = prep + static_cast<size_t>(t) * prow;
    for (int c = threadIdx.x; c < C; c += blockDim.x)
      cs[c] = siluf(conv_at(proj, stride, c, C, m.conv_taps, m.conv_w, nullptr, st, p, pos));
    for (int i = threadIdx.x; i < m.decay_rank + m.gate_rank; i += blockDim.x) lowa[i] = row[C + m.heads + i];
    __syncthreads();
    // unit vectors: query heads, then key heads
    for (int u = warp; u < 2 * m.kv_heads; u += nw) {
      const float* src = cs + u * m.dim;
      float ss = 0.f;
      for (int d = lane; d < m.dim; d += 32) ss = fmaf(src[d], src[d], ss);
      ss = warp_sum(ss);
      float rinv = 1.0f / sqrtf(ss + 1e-6f);
      if (u < m.kv_heads) rinv *= 1.0f / sqrtf(static_cast<float>(m.dim));
      for (int d = lane; d < m.dim; d += 32) dst[u * m.dim + d] = src[d] * rinv;
    }
    for (int i = threadIdx.x; i < vn; i += blockDim.x) dst[2 * qn + i] = cs[2 * qn + i];
    float* beta = dst + 2 * qn + vn;
    for (int h = threadIdx.x; h < m.heads; h += blockDim.x) beta[h] = sigmoidf(row[C + h]);
    float* decay = beta + m.heads;
    for (int i = threadIdx.x; i < m.heads * m.dim; i += blockDim.x) {
      const float* wr = m.w_a2 + static_cast<size_t>(i) * m.decay_rank;
      float acc = 0.f;
      for (int k = 0; k < m.decay_rank; ++k) acc = fmaf(wr[k], lowa[k], acc);
      decay[i] = expf(-m.rate[i / m.dim] * softplusf(acc + m.dt_bias[i]));
    }
    float* gate = decay + m.heads * m.dim;
    for (int i = threadIdx.x; i < vn; i += blockDim.x) {
      const float* wr = m.w_g2 + static_cast<size_t>(i) * m.gate_rank;
      float acc = 0.f;
      for (int k = 0; k < m.gate_rank; ++k) acc = fmaf(wr[k], lowg[k], acc);
      gate[i] = sigmoidf(acc);
    }
    __syncthreads();
  }
  if (p.j0 == 0 && hist > 0) conv_state_write(proj, stride, C, m.conv_taps, nullptr, st, p);
}

constexpr int kDeltaThreads = 128;
constexpr int kDeltaChunk = 16;  // rows staged in shared memory at a time
constexpr int kDeltaRows = 32;   // key channels per thread: L lanes share a value column, so dim <= 32 * L

// One CTA: one entry, one head, COLS = kDeltaThreads / L value columns.  L lanes share a column j and hold the rows
// i = lane, lane + L, ... of S[:, j].  Per row of the entry: S <- g S; u = beta (v_j - S[:, j] . k); S[:, j] += k u;
// o_j = S[:, j] . q -- every column on its own, the two dot products joined over the column's lanes.
__global__ void __launch_bounds__(kDeltaThreads)
delta_rule_kernel(kllm_seq_delta m, int L, const float* __restrict__ prep, float* __restrict__ state, StepRows rows,
                  const int32_t* __restrict__ ent_seq, float* __restrict__ o) {
  const int e = blockIdx.z, h = blockIdx.y;
  const int first = rows.ent_first[e], count = rows.ent_count[e], pos0 = rows.ent_pos0[e], seq = ent_seq[e];
  const int COLS = kDeltaThreads / L;
  const int lane = threadIdx.x % L, jl = threadIdx.x / L, j = blockIdx.x * COLS + jl;
  const bool live = j < m.vdim;
  const int D = m.dim, qn = m.kv_heads * D, vn = m.heads * m.vdim;
  const int g = h / (m.heads / m.kv_heads);
  const int prow = delta_prep_row(m);
  const int off_q = g * D, off_k = qn + g * D, off_v = 2 * qn + h * m.vdim, off_b = 2 * qn + vn + h,
            off_g = 2 * qn + vn + m.heads + h * D;
  extern __shared__ float sm[];
  float* q_s = sm;                        // [chunk][D]
  float* k_s = q_s + kDeltaChunk * D;     // [chunk][D]
  float* g_s = k_s + kDeltaChunk * D;     // [chunk][D]
  float* v_s = g_s + kDeltaChunk * D;     // [chunk][COLS]
  float* b_s = v_s + kDeltaChunk * COLS;  // [chunk]
  float* o_s = b_s + kDeltaChunk;         // [chunk][COLS]

  float S[kDeltaRows];
  float* st = state + ((static_cast<size_t>(seq) * m.heads + h) * D) * m.vdim + (live ? j : 0);
#pragma unroll
  for (int r = 0; r < kDeltaRows; ++r) {
    const int i = lane + r * L;
    S[r] = live && i < D && pos0 > 0 ? st[static_cast<size_t>(i) * m.vdim] : 0.f;
  }
  for (int r0 = 0; r0 < count; r0 += kDeltaChunk) {
    const int nr = min(kDeltaChunk, count - r0);
    __syncthreads();
    for (int i = threadIdx.x; i < nr * D; i += kDeltaThreads) {
      const float* row = prep + static_cast<size_t>(first + r0 + i / D) * prow;
      const int d = i % D;
      q_s[i] = row[off_q + d], k_s[i] = row[off_k + d], g_s[i] = row[off_g + d];
    }
    for (int i = threadIdx.x; i < nr * COLS; i += kDeltaThreads) {
      const int jj = blockIdx.x * COLS + i % COLS;
      v_s[i] = jj < m.vdim ? prep[static_cast<size_t>(first + r0 + i / COLS) * prow + off_v + jj] : 0.f;
    }
    for (int i = threadIdx.x; i < nr; i += kDeltaThreads) b_s[i] = prep[static_cast<size_t>(first + r0 + i) * prow + off_b];
    __syncthreads();
    for (int r = 0; r < nr; ++r) {
      const float* kq = k_s + r * D;
      const float* qq = q_s + r * D;
      const float* gg = g_s + r * D;
      float pred = 0.f;
#pragma unroll
      for (int x = 0; x < kDeltaRows; ++x) {
        const int i = lane + x * L;
        if (i < D) {
          S[x] *= gg[i];
          pred = fmaf(S[x], kq[i], pred);
        }
      }
      for (int w = L >> 1; w > 0; w >>= 1) pred += __shfl_xor_sync(kAll, pred, w);
      const float u = b_s[r] * (v_s[r * COLS + jl] - pred);
      float out = 0.f;
#pragma unroll
      for (int x = 0; x < kDeltaRows; ++x) {
        const int i = lane + x * L;
        if (i < D) {
          S[x] = fmaf(kq[i], u, S[x]);
          out = fmaf(S[x], qq[i], out);
        }
      }
      for (int w = L >> 1; w > 0; w >>= 1) out += __shfl_xor_sync(kAll, out, w);
      if (lane == 0) o_s[r * COLS + jl] = out;
    }
    __syncthreads();
    for (int i = threadIdx.x; i < nr * COLS; i += kDeltaThreads) {
      const int jj = blockIdx.x * COLS + i % COLS;
      if (jj < m.vdim) o[static_cast<size_t>(first + r0 + i / COLS) * vn + h * m.vdim + jj] = o_s[i];
    }
  }
#pragma unroll
  for (int r = 0; r < kDeltaRows; ++r) {
    const int i = lane + r * L;
    if (live && i < D) st[static_cast<size_t>(i) * m.vdim] = S[r];
  }
}

// a warp per (row, head)
template <typename AT>
__global__ void delta_out_kernel(kllm_seq_delta m, const float* __restrict__ o, const float* __restrict__ prep, float eps,
                                 AT* __restrict__ out, int T) {
  const int lane = threadIdx.x & 31;
  const size_t u = static_cast<size_t>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (u >= static_cast<size_t>(T) * m.heads) return;
  const size_t t = u / m.heads;
  const int h = static_cast<int>(u % m.heads);
  const int vn = m.heads * m.vdim;
  const float* src = o + t * vn + h * m.vdim;
  const float* gate = prep + t * delta_prep_row(m) + 2 * m.kv_heads * m.dim + vn + m.heads + m.heads * m.dim + h * m.vdim;
  float ss = 0.f;
  for (int d = lane; d < m.vdim; d += 32) ss = fmaf(src[d], src[d], ss);
  ss = warp_sum(ss);
  const float rinv = 1.0f / sqrtf(ss / static_cast<float>(m.vdim) + eps);
  for (int d = lane; d < m.vdim; d += 32)
    out[t * vn + h * m.vdim + d] = from_f<AT>(src[d] * rinv * m.out_norm_w[d] * gate[d]);
}

#define KLLM_SEQ_DISPATCH(dtype, CALL)                         \
  do {                                                         \
    if ((dtype) == KLLM_SEQ_F32) {                             \
      using AT = float;                                        \
      CALL;                                                    \
    } else if ((dtype) == KLLM_SEQ_BF16) {                     \
      using AT = __nv_bfloat16;                                \
      CALL;                                                    \
    } else {                                                   \
      return KLLM_E_INVALID;                                   \
    }                                                          \
  } while (0)

inline int done() {
  count_launch();
  return cuda_rc(cudaGetLastError());
}

// lanes that share a unit whose `n` elements are spread `per` to a lane: the smallest power of two that fits
inline int lanes_for(int n, int per) {
  int L = 1;
  while (L < 32 && L * per < n) L *= 2;
  return L;
}

}  // namespace

int launch_qk_conv_prepare(int dtype, const AttnShape& a, const AttnPrep& p, const float* qk, const StepRows& rows, void* q,
                           const PagedKV& kv, int T, cudaStream_t s) {
  const int C = (a.heads + a.kv_heads) * a.dim;
  if (p.taps < 1 || (p.taps > 1 && !p.conv_state) || (p.rope_dims & 1) || p.rope_dims > a.dim) return KLLM_E_INVALID;
  const size_t smem = static_cast<size_t>(C) * sizeof(float);
  if (smem > 48 * 1024) return KLLM_E_UNSUPPORTED;
  const int threads = C >= 2048 ? 512 : 256;
  KLLM_SEQ_DISPATCH(dtype, (qk_conv_prepare_kernel<AT><<<T, threads, smem, s>>>(a, p, qk, rows, static_cast<AT*>(q), kv)));
  return done();
}

int launch_ssm_conv(int dtype, const kllm_seq_ssm& m, const float* uz, float* conv_state, const StepRows& rows, float* uc,
                    void* uc_ct, int T, cudaStream_t s) {
  const int threads = m.inner >= 2048 ? 512 : 256;
  KLLM_SEQ_DISPATCH(dtype, (ssm_conv_kernel<AT><<<T, threads, 0, s>>>(m.inner, m.conv_taps, m.conv_w, m.conv_b, uz, conv_state,
                                                                     rows, uc, static_cast<AT*>(uc_ct))));
  return done();
}

int launch_ssm_scan(int dtype, const kllm_seq_ssm& m, const float* uz, const float* uc, const float* low, float* state,
                    const StepRows& rows, const int32_t* ent_seq, int max_count, void* out, cudaStream_t s) {
  (void)max_count;
  if (m.state > 32 * kScanPerLane) return KLLM_E_UNSUPPORTED;
  // at least 4 lanes per channel: at most 32 channels of a chunk in shared memory
  const int L = std::max(4, lanes_for(m.state, m.state > 32 ? kScanPerLane : 1));
  const int CH = kScanThreads / L;
  const size_t smem = (static_cast<size_t>(kScanChunk) * (m.dt_rank + 2 * m.state) + 4 * static_cast<size_t>(kScanChunk) * CH) *
                      sizeof(float);
  if (smem > 48 * 1024) return KLLM_E_UNSUPPORTED;
  const dim3 grid((m.inner + CH - 1) / CH, rows.n_entries);
  KLLM_SEQ_DISPATCH(dtype, (ssm_scan_kernel<AT><<<grid, kScanThreads, smem, s>>>(m, L, uz, uc, low, state, rows, ent_seq,
                                                                                static_cast<AT*>(out))));
  return done();
}

int launch_delta_prepare(const kllm_seq_delta& m, const float* proj, float* conv_state, const StepRows& rows, float* prep, int T,
                         cudaStream_t s) {
  const int C = 2 * m.kv_heads * m.dim + m.heads * m.vdim;
  const size_t smem = (static_cast<size_t>(C) + m.decay_rank + m.gate_rank) * sizeof(float);
  if (smem > 48 * 1024) return KLLM_E_UNSUPPORTED;
  delta_prepare_kernel<<<T, 256, smem, s>>>(m, proj, conv_state, rows, prep);
  return done();
}

int launch_delta_rule(const kllm_seq_delta& m, const float* prep, float* state, const StepRows& rows, const int32_t* ent_seq,
                      int max_count, float* o, cudaStream_t s) {
  (void)max_count;
  if (m.dim > 32 * kDeltaRows) return KLLM_E_UNSUPPORTED;
  const int L = lanes_for(m.dim, kDeltaRows);
  const int COLS = kDeltaThreads / L;
  const size_t smem = (3 * static_cast<size_t>(kDeltaChunk) * m.dim + 2 * static_cast<size_t>(kDeltaChunk) * COLS + kDeltaChunk) *
                      sizeof(float);
  if (smem > 48 * 1024) return KLLM_E_UNSUPPORTED;
  const dim3 grid((m.vdim + COLS - 1) / COLS, m.heads, rows.n_entries);
  delta_rule_kernel<<<grid, kDeltaThreads, smem, s>>>(m, L, prep, state, rows, ent_seq, o);
  return done();
}

int launch_delta_out(int dtype, const kllm_seq_delta& m, const float* o, const float* prep, float eps, void* out, int T,
                     cudaStream_t s) {
  const size_t units = static_cast<size_t>(T) * m.heads;
  const unsigned blocks = static_cast<unsigned>((units + 3) / 4);
  KLLM_SEQ_DISPATCH(dtype, (delta_out_kernel<AT><<<blocks, 128, 0, s>>>(m, o, prep, eps, static_cast<AT*>(out), T)));
  return done();
}

}  // namespace seq
}  // namespace kllm
