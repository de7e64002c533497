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
constexpr int kScanPerLane = 4;  // states per thread: up to 32 lanes share a channel, so state <= 128

// One CTA: one entry, CH = kScanThreads / L channels; L lanes share a channel, lane l holds its states 4l .. 4l + 3.
// The rows of W_dt of the CTA's channels stay in shared memory.  Chunks of `chunk` rows are staged in shared memory (the
// low-rank rows, u, z), the step sizes of the chunk are computed by all threads, then the recurrence runs over the
// chunk's rows.
template <typename AT>
__global__ void __launch_bounds__(kScanThreads)
ssm_scan_kernel(kllm_seq_ssm m, int L, int chunk, const float* __restrict__ uz, const float* __restrict__ uc,
                const float* __restrict__ low, float* __restrict__ state, StepRows rows,
                const int32_t* __restrict__ ent_seq, AT* __restrict__ out) {
  const int e = blockIdx.y;
  const int first = rows.ent_first[e], count = rows.ent_count[e], pos0 = rows.ent_pos0[e], seq = ent_seq[e];
  const int CH = kScanThreads / L;
  const int c0 = blockIdx.x * CH;
  const int lane = threadIdx.x % L, cl = threadIdx.x / L, c = c0 + cl;
  const bool live = c < m.inner;
  const int R = m.dt_rank, N = m.state, LW = R + 2 * N, RW = R + 1;
  extern __shared__ float sm[];
  float* w_s = sm;                        // [CH][R + 1] rows of W_dt
  float* low_s = w_s + CH * RW;           // [chunk][LW]
  float* u_s = low_s + chunk * LW;        // [chunk][CH]
  float* z_s = u_s + chunk * CH;          // [chunk][CH]
  float* dt_s = z_s + chunk * CH;         // [chunk][CH]
  float* y_s = dt_s + chunk * CH;         // [chunk][CH]

  for (int i = threadIdx.x; i < CH * R; i += kScanThreads) {
    const int cc = c0 + i / R;
    w_s[(i / R) * RW + i % R] = cc < m.inner ? m.w_dt[static_cast<size_t>(cc) * R + i % R] : 0.f;
  }
  float S[kScanPerLane], A[kScanPerLane];
  float* st = state + (static_cast<size_t>(seq) * m.inner + (live ? c : 0)) * N;
#pragma unroll
  for (int k = 0; k < kScanPerLane; ++k) {
    const int n = lane * kScanPerLane + k;
    const bool on = live && n < N;
    S[k] = on && pos0 > 0 ? st[n] : 0.f;
    A[k] = on ? m.a[static_cast<size_t>(c) * N + n] : 0.f;
  }
  const float dskip = live ? m.d[c] : 0.f;
  for (int r0 = 0; r0 < count; r0 += chunk) {
    const int nr = min(chunk, count - r0);
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
      const int r = i / CH, ci = i % CH;
      const float* wr = w_s + ci * RW;
      const float* lr = low_s + r * LW;
      float a0 = 0.f, a1 = 0.f;
      int k = 0;
      for (; k + 1 < R; k += 2) {
        a0 = fmaf(wr[k], lr[k], a0);
        a1 = fmaf(wr[k + 1], lr[k + 1], a1);
      }
      if (k < R) a0 = fmaf(wr[k], lr[k], a0);
      dt_s[i] = c0 + ci < m.inner ? softplusf(a0 + a1 + m.dt_b[c0 + ci]) : 0.f;
    }
    __syncthreads();
    for (int r = 0; r < nr; ++r) {
      const float dt = dt_s[r * CH + cl], u = u_s[r * CH + cl];
      const float du = dt * u;
      const float* Bn = low_s + r * LW + R + lane * kScanPerLane;
      const float* Cn = Bn + N;
      float y = 0.f;
#pragma unroll
      for (int k = 0; k < kScanPerLane; ++k) {
        if (lane * kScanPerLane + k < N) {
          S[k] = fmaf(expf(dt * A[k]), S[k], du * Bn[k]);
          y = fmaf(S[k], Cn[k], y);
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
    const int n = lane * kScanPerLane + k;
    if (live && n < N) st[n] = S[k];
  }
}

// ---- gated delta rule ---------------------------------------------------------------------------------------------------
// where the parts of a prepared row start (see delta_prep_row)
struct DeltaRow {
  int q, k, v, decay, gate, beta;
};
__host__ __device__ inline DeltaRow delta_row(const kllm_seq_delta& m) {
  const int qn = m.kv_heads * m.dim, vn = m.heads * m.vdim, dn = m.heads * m.dim;
  return DeltaRow{0, qn, 2 * qn, 2 * qn + vn, 2 * qn + vn + dn, 2 * qn + 2 * vn + dn};
}

template <typename AT>
__global__ void delta_low_kernel(kllm_seq_delta m, const float* __restrict__ proj, AT* __restrict__ low, size_t total) {
  const size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= total) return;
  const int nl = m.decay_rank + m.gate_rank;
  const int C = 2 * m.kv_heads * m.dim + m.heads * m.vdim;
  low[i] = from_f<AT>(proj[(i / nl) * (C + m.heads + nl) + C + m.heads + i % nl]);
}

// One CTA per row (see the note on filters at the top).  Shared memory: the filtered q | k | v row.
__global__ void delta_prepare_kernel(kllm_seq_delta m, const float* __restrict__ proj, const float* __restrict__ low2,
                                     float* __restrict__ conv_state, StepRows rows, float* __restrict__ prep) {
  extern __shared__ float cs[];
  const RowPlace p = place_row(rows, blockIdx.x, m.conv_taps);
  if (p.n_here == 0) return;
  const int qn = m.kv_heads * m.dim, vn = m.heads * m.vdim, dn = m.heads * m.dim, C = 2 * qn + vn, hist = m.conv_taps - 1;
  const int stride = C + m.heads + m.decay_rank + m.gate_rank;
  const int prow = delta_prep_row(m);
  const DeltaRow at = delta_row(m);
  float* st = hist > 0 ? conv_state + static_cast<size_t>(p.seq) * hist * C : nullptr;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
  for (int jj = 0; jj < p.n_here; ++jj) {
    const int t = blockIdx.x + jj, pos = p.pos0 + p.j0 + jj;
    const float* row = proj + static_cast<size_t>(t) * stride;
    const float* l2 = low2 + static_cast<size_t>(t) * (dn + vn);
    float* dst = prep + static_cast<size_t>(t) * prow;
    for (int c = threadIdx.x; c < C; c += blockDim.x)
      cs[c] = siluf(conv_at(proj, stride, c, C, m.conv_taps, m.conv_w, nullptr, st, p, pos));
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
    for (int i = threadIdx.x; i < vn; i += blockDim.x) dst[at.v + i] = cs[2 * qn + i];
    for (int h = threadIdx.x; h < m.heads; h += blockDim.x) dst[at.beta + h] = sigmoidf(row[C + h]);
    for (int i = threadIdx.x; i < dn; i += blockDim.x)
      dst[at.decay + i] = expf(-m.rate[i / m.dim] * softplusf(l2[i] + m.dt_bias[i]));
    for (int i = threadIdx.x; i < vn; i += blockDim.x) dst[at.gate + i] = sigmoidf(l2[dn + i]);
    __syncthreads();
  }
  if (p.j0 == 0 && hist > 0) conv_state_write(proj, stride, C, m.conv_taps, nullptr, st, p);
}

constexpr int kDeltaThreads = 128;
constexpr int kDeltaPad = 4;  // floats between the row slices of two lanes in shared memory: their 16-byte loads hit different banks

__device__ __forceinline__ void cp_async4(float* dst, const float* src) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(static_cast<uint32_t>(__cvta_generic_to_shared(dst))), "l"(src));
}
__device__ __forceinline__ void cp_async16(float* dst, const float* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(static_cast<uint32_t>(__cvta_generic_to_shared(dst))), "l"(src));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.wait_group 0;" ::: "memory"); }

// One CTA: one entry, one head, COLS = kDeltaThreads / L value columns.  L lanes share a column j; lane l holds the rows
// l * RP .. l * RP + RP - 1 of S[:, j] in registers.  Per row of the entry: S <- g S; u = beta (v_j - S[:, j] . k);
// S[:, j] += k u; o_j = S[:, j] . q -- every column on its own, the two dot products joined over the column's lanes.
// Chunks of `chunk` rows (q, k, g of the head, v of the CTA's columns, beta) come through two shared-memory buffers by
// cp.async: the next chunk is on its way while the current one is worked on.  VEC: every part of a prepared row starts on
// 16 bytes (dim and vdim multiples of 4), so the copies are 16 bytes wide.
template <int RP, bool VEC>
__global__ void __launch_bounds__(kDeltaThreads)
delta_rule_kernel(kllm_seq_delta m, int L, int chunk, const float* __restrict__ prep, float* __restrict__ state,
                  StepRows rows, const int32_t* __restrict__ ent_seq, float* __restrict__ o) {
  const int e = blockIdx.z, h = blockIdx.y;
  const int first = rows.ent_first[e], count = rows.ent_count[e], pos0 = rows.ent_pos0[e], seq = ent_seq[e];
  const int COLS = kDeltaThreads / L;
  const int lane = threadIdx.x % L, jl = threadIdx.x / L, j0 = blockIdx.x * COLS, j = j0 + jl;
  const bool live = j < m.vdim;
  const int D = m.dim, vn = m.heads * m.vdim;
  const int g = h / (m.heads / m.kv_heads);
  const int prow = delta_prep_row(m);
  const DeltaRow at = delta_row(m);
  const int off_q = at.q + g * D, off_k = at.k + g * D, off_v = at.v + h * m.vdim + j0, off_g = at.decay + h * D,
            off_b = at.beta + h;
  const int LS = RP + kDeltaPad, DP = L * LS;      // a lane's slice, a row of q / k / g in shared memory
  const int per = 3 * DP + COLS + 4;               // floats of one row of a chunk: q | k | g | v | beta (+ pad)
  extern __shared__ __align__(16) float sm[];
  float* o_s = sm + 2 * chunk * per;               // [chunk][COLS]
  for (int i = threadIdx.x; i < 2 * chunk * per; i += kDeltaThreads) sm[i] = 0.f;  // the padding stays zero
  __syncthreads();

  auto stage = [&](int r0, int nr, float* buf) {
    if (VEC) {
      const int dv = D / 4, cv = min(COLS, m.vdim - j0) / 4;
      const int tasks = nr * (3 * dv + cv);
      for (int i = threadIdx.x; i < tasks; i += kDeltaThreads) {
        const int r = i / (3 * dv + cv), x = i % (3 * dv + cv);
        const float* src = prep + static_cast<size_t>(first + r0 + r) * prow;
        float* dst = buf + r * per;
        if (x < 3 * dv) {
          const int part = x / dv, d = (x % dv) * 4;
          cp_async16(dst + part * DP + (d / RP) * LS + d % RP, src + (part == 0 ? off_q : part == 1 ? off_k : off_g) + d);
        } else {
          cp_async16(dst + 3 * DP + (x - 3 * dv) * 4, src + off_v + (x - 3 * dv) * 4);
        }
      }
    } else {
      const int cv = min(COLS, m.vdim - j0);
      const int tasks = nr * (3 * D + cv);
      for (int i = threadIdx.x; i < tasks; i += kDeltaThreads) {
        const int r = i / (3 * D + cv), x = i % (3 * D + cv);
        const float* src = prep + static_cast<size_t>(first + r0 + r) * prow;
        float* dst = buf + r * per;
        if (x < 3 * D) {
          const int part = x / D, d = x % D;
          cp_async4(dst + part * DP + (d / RP) * LS + d % RP, src + (part == 0 ? off_q : part == 1 ? off_k : off_g) + d);
        } else {
          cp_async4(dst + 3 * DP + (x - 3 * D), src + off_v + (x - 3 * D));
        }
      }
    }
    for (int r = threadIdx.x; r < nr; r += kDeltaThreads)
      cp_async4(buf + r * per + 3 * DP + COLS, prep + static_cast<size_t>(first + r0 + r) * prow + off_b);
    cp_async_commit();
  };

  float S[RP];
  float* st = state + ((static_cast<size_t>(seq) * m.heads + h) * D) * m.vdim + (live ? j : 0);
#pragma unroll
  for (int x = 0; x < RP; ++x) {
    const int i = lane * RP + x;
    S[x] = live && i < D && pos0 > 0 ? st[static_cast<size_t>(i) * m.vdim] : 0.f;
  }
  stage(0, min(chunk, count), sm);
  int which = 0;
  for (int r0 = 0; r0 < count; r0 += chunk, which ^= 1) {
    const int nr = min(chunk, count - r0);
    float* buf = sm + which * chunk * per;
    cp_async_wait_all();
    __syncthreads();  // the chunk has landed; the other buffer and o_s are free
    if (r0 + chunk < count) stage(r0 + chunk, min(chunk, count - r0 - chunk), sm + (which ^ 1) * chunk * per);
    for (int r = 0; r < nr; ++r) {
      const float* row = buf + r * per;
      const float4* q4 = reinterpret_cast<const float4*>(row + lane * LS);
      const float4* k4 = reinterpret_cast<const float4*>(row + DP + lane * LS);
      const float4* g4 = reinterpret_cast<const float4*>(row + 2 * DP + lane * LS);
      float p0 = 0.f, p1 = 0.f, p2 = 0.f, p3 = 0.f;
#pragma unroll
      for (int x = 0; x < RP / 4; ++x) {
        const float4 gg = g4[x], kk = k4[x];
        S[4 * x] *= gg.x, S[4 * x + 1] *= gg.y, S[4 * x + 2] *= gg.z, S[4 * x + 3] *= gg.w;
        p0 = fmaf(S[4 * x], kk.x, p0), p1 = fmaf(S[4 * x + 1], kk.y, p1);
        p2 = fmaf(S[4 * x + 2], kk.z, p2), p3 = fmaf(S[4 * x + 3], kk.w, p3);
      }
      float pred = (p0 + p1) + (p2 + p3);
      for (int w = L >> 1; w > 0; w >>= 1) pred += __shfl_xor_sync(kAll, pred, w);
      const float u = row[3 * DP + COLS] * (row[3 * DP + jl] - pred);
      p0 = p1 = p2 = p3 = 0.f;
#pragma unroll
      for (int x = 0; x < RP / 4; ++x) {
        const float4 kk = k4[x], qq = q4[x];
        S[4 * x] = fmaf(kk.x, u, S[4 * x]), S[4 * x + 1] = fmaf(kk.y, u, S[4 * x + 1]);
        S[4 * x + 2] = fmaf(kk.z, u, S[4 * x + 2]), S[4 * x + 3] = fmaf(kk.w, u, S[4 * x + 3]);
        p0 = fmaf(S[4 * x], qq.x, p0), p1 = fmaf(S[4 * x + 1], qq.y, p1);
        p2 = fmaf(S[4 * x + 2], qq.z, p2), p3 = fmaf(S[4 * x + 3], qq.w, p3);
      }
      float out = (p0 + p1) + (p2 + p3);
      for (int w = L >> 1; w > 0; w >>= 1) out += __shfl_xor_sync(kAll, out, w);
      if (lane == 0) o_s[r * COLS + jl] = out;
    }
    __syncthreads();
    for (int i = threadIdx.x; i < nr * COLS; i += kDeltaThreads) {
      const int jj = j0 + i % COLS;
      if (jj < m.vdim) o[static_cast<size_t>(first + r0 + i / COLS) * vn + h * m.vdim + jj] = o_s[i];
    }
  }
#pragma unroll
  for (int x = 0; x < RP; ++x) {
    const int i = lane * RP + x;
    if (live && i < D) st[static_cast<size_t>(i) * m.vdim] = S[x];
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
  const float* gate = prep + t * delta_prep_row(m) + delta_row(m).gate + h * m.vdim;
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
  if (m.state > 32 * kScanPerLane) return KLLM_E_UNSUPPORTED;
  // at least 4 lanes per channel: at most 32 channels of a chunk in shared memory
  const int L = std::max(4, lanes_for(m.state, kScanPerLane));
  const int CH = kScanThreads / L;
  auto smem_for = [&](int chunk) {
    return (static_cast<size_t>(CH) * (m.dt_rank + 1) + static_cast<size_t>(chunk) * (m.dt_rank + 2 * m.state) +
            4 * static_cast<size_t>(chunk) * CH) * sizeof(float);
  };
  int chunk = 32;
  while (chunk > 1 && (smem_for(chunk) > 48 * 1024 || chunk / 2 >= max_count)) chunk /= 2;
  if (smem_for(chunk) > 48 * 1024) return KLLM_E_UNSUPPORTED;
  const dim3 grid((m.inner + CH - 1) / CH, rows.n_entries);
  KLLM_SEQ_DISPATCH(dtype, (ssm_scan_kernel<AT><<<grid, kScanThreads, smem_for(chunk), s>>>(m, L, chunk, uz, uc, low, state, rows,
                                                                                          ent_seq, static_cast<AT*>(out))));
  return done();
}

int launch_delta_low(int dtype, const kllm_seq_delta& m, const float* proj, void* low, int T, cudaStream_t s) {
  const size_t total = static_cast<size_t>(T) * (m.decay_rank + m.gate_rank);
  const unsigned blocks = static_cast<unsigned>((total + 255) / 256);
  KLLM_SEQ_DISPATCH(dtype, (delta_low_kernel<AT><<<blocks, 256, 0, s>>>(m, proj, static_cast<AT*>(low), total)));
  return done();
}

int launch_delta_prepare(const kllm_seq_delta& m, const float* proj, const float* low2, float* conv_state, const StepRows& rows,
                         float* prep, int T, cudaStream_t s) {
  const int C = 2 * m.kv_heads * m.dim + m.heads * m.vdim;
  const size_t smem = static_cast<size_t>(C) * sizeof(float);
  if (smem > 48 * 1024) return KLLM_E_UNSUPPORTED;
  delta_prepare_kernel<<<T, 256, smem, s>>>(m, proj, low2, conv_state, rows, prep);
  return done();
}

int launch_delta_rule(const kllm_seq_delta& m, const float* prep, float* state, const StepRows& rows, const int32_t* ent_seq,
                      int max_count, float* o, cudaStream_t s) {
  // 16 rows of a column per thread while that leaves at most 8 lanes to a column, else 32
  const int RP = m.dim <= 128 ? 16 : 32;
  if (m.dim > 32 * RP || m.dim > 256) return KLLM_E_UNSUPPORTED;
  const int L = lanes_for(m.dim, RP);
  const int COLS = kDeltaThreads / L;
  const int per = 3 * L * (RP + kDeltaPad) + COLS + 4;
  auto smem_for = [&](int chunk) { return (2 * static_cast<size_t>(chunk) * per + static_cast<size_t>(chunk) * COLS) * sizeof(float); };
  int chunk = 16;
  while (chunk > 1 && (smem_for(chunk) > 48 * 1024 || chunk / 2 >= max_count)) chunk /= 2;
  if (smem_for(chunk) > 48 * 1024) return KLLM_E_UNSUPPORTED;
  const bool vec = m.dim % 4 == 0 && m.vdim % 4 == 0;
  const dim3 grid((m.vdim + COLS - 1) / COLS, m.heads, rows.n_entries);
#define KLLM_DELTA(R, V) delta_rule_kernel<R, V><<<grid, kDeltaThreads, smem_for(chunk), s>>>(m, L, chunk, prep, state, rows, ent_seq, o)
  if (RP == 16) {
    if (vec) KLLM_DELTA(16, true);
    else KLLM_DELTA(16, false);
  } else {
    if (vec) KLLM_DELTA(32, true);
    else KLLM_DELTA(32, false);
  }
#undef KLLM_DELTA
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
