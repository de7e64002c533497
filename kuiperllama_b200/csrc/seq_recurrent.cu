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
#include "seq_rows.cuh"

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

// ---- attention behind a filter ------------------------------------------------------------------------------------------
template <typename AT>
__device__ __forceinline__ AT* page_row(AT* base, const PagedKV& kv, int seq, int pos, int row) {
  const int page = kv.table[static_cast<size_t>(seq) * kv.table_stride + pos / kv.page];
  return base + (static_cast<size_t>(page) * kv.page + pos % kv.page) * row;
}

// One CTA per (row, query or key head): unit u < heads is query head u, the others are the key heads.
template <typename AT>
__global__ void qk_conv_prepare_kernel(AttnShape a, AttnPrep pr, const float* __restrict__ qk, StepRows rows,
                                       AT* __restrict__ q, PagedKV kv) {
  extern __shared__ float cs[];  // [dim] the head's filtered row
  const RowPlace p = place_row(rows, blockIdx.x, pr.taps);
  if (p.n_here == 0) return;
  const int u = blockIdx.y;
  const bool is_q = u < a.heads;
  const int qn = a.heads * a.dim, C = qn + a.kv_heads * a.dim, hist = pr.taps - 1, c0 = u * a.dim;
  float* st = hist > 0 ? pr.conv_state + static_cast<size_t>(p.seq) * hist * C : nullptr;
  const int rd = pr.rope_dims, half = rd / 2;
  for (int jj = 0; jj < p.n_here; ++jj) {
    const int t = blockIdx.x + jj, pos = p.pos0 + p.j0 + jj;
    for (int d = threadIdx.x; d < a.dim; d += blockDim.x)
      cs[d] = conv_at(qk, C, c0 + d, C, pr.taps, pr.conv_w, pr.bias, st, p, pos);
    __syncthreads();
    AT* krow = is_q ? nullptr : page_row(static_cast<AT*>(kv.k), kv, p.seq, pos, kv.k_row) + (c0 - qn);
    AT* vrow = is_q ? nullptr : page_row(static_cast<AT*>(kv.v), kv, p.seq, pos, kv.v_row) + (c0 - qn);
    for (int d = threadIdx.x; d < a.dim; d += blockDim.x) {
      float v = cs[d];
      if (!is_q) vrow[d] = from_f<AT>(v);  // the values: keys before the rotation
      if (d < rd) {
        int i, partner;
        bool lead;  // the member of the pair that becomes u cos - v sin
        if (pr.rope_pairing == KLLM_SEQ_ROPE_PAIRS) i = d >> 1, partner = d ^ 1, lead = (d & 1) == 0;
        else lead = d < half, i = lead ? d : d - half, partner = lead ? d + half : d - half;
        const float freq = powf(pr.rope_base, -2.0f * static_cast<float>(i) / static_cast<float>(rd));
        const float ang = static_cast<float>(pos) * freq;
        const float co = cosf(ang), si = sinf(ang);
        const float o = cs[partner];
        v = lead ? v * co - o * si : v * co + o * si;
      }
      if (is_q) q[static_cast<size_t>(t) * qn + c0 + d] = from_f<AT>(v);
      else krow[d] = from_f<AT>(v);
    }
    __syncthreads();
  }
  if (p.j0 == 0 && hist > 0) conv_state_write(qk, C, C, pr.taps, pr.bias, st, p, c0, a.dim);
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
  const int c0 = blockIdx.y * blockDim.x, c = c0 + threadIdx.x;
  for (int jj = 0; jj < p.n_here; ++jj) {
    const int t = blockIdx.x + jj, pos = p.pos0 + p.j0 + jj;
    if (c < inner) {
      const float v = siluf(conv_at(uz, 2 * inner, c, inner, taps, conv_w, nullptr, st, p, pos) + (conv_b ? conv_b[c] : 0.f));
      uc[static_cast<size_t>(t) * inner + c] = v;
      uc_ct[static_cast<size_t>(t) * inner + c] = from_f<AT>(v);
    }
  }
  // the thread that read a channel's old state is the one that writes its new one
  if (p.j0 == 0 && hist > 0) conv_state_write(uz, 2 * inner, inner, taps, nullptr, st, p, c0, min(static_cast<int>(blockDim.x), inner - c0));
}

constexpr int kScanThreads = 128;
constexpr int kScanPerLane = 4;  // states per thread: up to 32 lanes share a channel, so state <= 128
constexpr int kScanSeg = 128;          // rows of a segment when long entries are scanned in parallel
constexpr int kScanParallelFrom = 256; // entries longer than this are cut into segments

// Long entries.  The recurrence S_t = exp(d_t a) S_(t-1) + b_t is linear, so an entry is cut into segments of kScanSeg rows
// that are scanned at the same time, each from an empty state (the first from the sequence's): with D_t the sum of the step
// sizes from the segment's start to row t, the true state is S_t = S'_t + exp(a D_t) S_start, S' the segment's own scan.
//   ssm_scan_kernel<SEGMENTS>   the segment's own scan: y' (fp32, ungated), D_t of every row, the segment's last S' and D
//   ssm_carry_kernel            S_start of every segment, one after the other; the sequence's new state
//   ssm_finish_kernel           y = y' + sum_n C_n exp(a_n D_t) S_start[n]; gate with silu(z); compute type
// Scratch (fp32): y' [T][inner] | D [T][inner] | last S' (then S_start) [segments][inner][state] | last D [segments][inner].
struct ScanScratch {
  float* yl;
  float* cum;
  float* send;
  float* cend;
};
__host__ __device__ inline int scan_segment_id(int first, int e, int seg) { return first / kScanSeg + e + seg; }

// One CTA: one entry, CH = kScanThreads / L channels; L lanes share a channel, lane l holds its states 4l .. 4l + 3.
// The rows of W_dt of the CTA's channels stay in shared memory.  Chunks of `chunk` rows are staged in shared memory (the
// low-rank rows, u, z), the step sizes of the chunk are computed by all threads, then the recurrence runs over the
// chunk's rows.
template <typename AT, bool SEGMENTS>
__global__ void __launch_bounds__(kScanThreads)
ssm_scan_kernel(kllm_seq_ssm m, int L, int chunk, const float* __restrict__ uz, const float* __restrict__ uc,
                const float* __restrict__ low, float* __restrict__ state, StepRows rows,
                const int32_t* __restrict__ ent_seq, AT* __restrict__ out, ScanScratch sc) {
  const int e = SEGMENTS ? blockIdx.z : blockIdx.y, seg = SEGMENTS ? blockIdx.y : 0;
  const int e_first = rows.ent_first[e], e_count = rows.ent_count[e], pos0 = rows.ent_pos0[e], seq = ent_seq[e];
  if (SEGMENTS && seg * kScanSeg >= e_count) return;
  // the rows of this CTA: the whole entry, or one segment of it
  const int first = SEGMENTS ? e_first + seg * kScanSeg : e_first;
  const int count = SEGMENTS ? min(kScanSeg, e_count - seg * kScanSeg) : e_count;
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
    S[k] = on && pos0 > 0 && seg == 0 ? st[n] : 0.f;
    A[k] = on ? m.a[static_cast<size_t>(c) * N + n] : 0.f;
  }
  const float dskip = live ? m.d[c] : 0.f;
  float cum = 0.f;  // the sum of the step sizes since the segment's start
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
      if (SEGMENTS) {
        cum += dt;
        if (lane == 0) y_s[r * CH + cl] = y + dskip * u, dt_s[r * CH + cl] = cum;  // this row's dt is no longer needed
      } else if (lane == 0) {
        y_s[r * CH + cl] = (y + dskip * u) * siluf(z_s[r * CH + cl]);
      }
    }
    __syncthreads();
    for (int i = threadIdx.x; i < nr * CH; i += kScanThreads) {
      const int r = i / CH, cc = c0 + i % CH;
      if (cc >= m.inner) continue;
      const size_t at = static_cast<size_t>(first + r0 + r) * m.inner + cc;
      if (SEGMENTS) sc.yl[at] = y_s[i], sc.cum[at] = dt_s[i];
      else out[at] = from_f<AT>(y_s[i]);
    }
  }
  if (SEGMENTS) {
    const size_t sid = scan_segment_id(e_first, e, seg);
    if (live && lane == 0) sc.cend[sid * m.inner + c] = cum;
    st = sc.send + (sid * m.inner + (live ? c : 0)) * N;
  }
#pragma unroll
  for (int k = 0; k < kScanPerLane; ++k) {
    const int n = lane * kScanPerLane + k;
    if (live && n < N) st[n] = S[k];
  }
}

// One thread per (entry, channel, state): the start state of every segment after the first, and the sequence's new state.
__global__ void ssm_carry_kernel(kllm_seq_ssm m, float* __restrict__ state, StepRows rows, const int32_t* __restrict__ ent_seq,
                                 ScanScratch sc) {
  const int e = blockIdx.y;
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= m.inner * m.state) return;
  const int first = rows.ent_first[e], count = rows.ent_count[e];
  const int segs = (count + kScanSeg - 1) / kScanSeg;
  const float a = m.a[i];
  const int c = i / m.state;
  const size_t per = static_cast<size_t>(m.inner) * m.state;
  float carry = sc.send[scan_segment_id(first, e, 0) * per + i];  // the first segment started from the sequence's state
  for (int sgm = 1; sgm < segs; ++sgm) {
    const size_t sid = scan_segment_id(first, e, sgm);
    const float own = sc.send[sid * per + i];
    sc.send[sid * per + i] = carry;
    carry = fmaf(expf(a * sc.cend[sid * m.inner + c]), carry, own);
  }
  state[static_cast<size_t>(ent_seq[e]) * per + i] = carry;
}

// One CTA: CH channels of one segment; L lanes share a channel as in the scan.  Rows are independent here.
template <typename AT>
__global__ void __launch_bounds__(kScanThreads)
ssm_finish_kernel(kllm_seq_ssm m, int L, const float* __restrict__ uz, const float* __restrict__ low, StepRows rows,
                  AT* __restrict__ out, ScanScratch sc) {
  const int e = blockIdx.z, seg = blockIdx.y;
  const int e_first = rows.ent_first[e], e_count = rows.ent_count[e];
  if (seg * kScanSeg >= e_count) return;
  const int first = e_first + seg * kScanSeg, count = min(kScanSeg, e_count - seg * kScanSeg);
  const int CH = kScanThreads / L;
  const int lane = threadIdx.x % L, cl = threadIdx.x / L, c = blockIdx.x * CH + cl;
  const bool live = c < m.inner;
  const int R = m.dt_rank, N = m.state, LW = R + 2 * N;
  float S0[kScanPerLane], A[kScanPerLane];
  const size_t sid = scan_segment_id(e_first, e, seg);
#pragma unroll
  for (int k = 0; k < kScanPerLane; ++k) {
    const int n = lane * kScanPerLane + k;
    const bool on = live && n < N && seg > 0;
    S0[k] = on ? sc.send[(sid * m.inner + c) * N + n] : 0.f;
    A[k] = on ? m.a[static_cast<size_t>(c) * N + n] : 0.f;
  }
  for (int r = 0; r < count; ++r) {
    const size_t row = static_cast<size_t>(first + r);
    float corr = 0.f;
    if (seg > 0 && live) {
      const float cum = sc.cum[row * m.inner + c];
      const float* Cn = low + row * LW + R + N + lane * kScanPerLane;
#pragma unroll
      for (int k = 0; k < kScanPerLane; ++k)
        if (lane * kScanPerLane + k < N) corr = fmaf(Cn[k] * expf(A[k] * cum), S0[k], corr);
    }
    for (int o = L >> 1; o > 0; o >>= 1) corr += __shfl_xor_sync(kAll, corr, o);
    if (lane == 0 && live)
      out[row * m.inner + c] = from_f<AT>((sc.yl[row * m.inner + c] + corr) * siluf(uz[row * 2 * m.inner + m.inner + c]));
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

// One CTA per (row, head h) (see the note on filters at the top): the head's value channels, decays, gates and beta, and --
// for h < kv_heads -- query head h and key head h.  Shared memory: the filtered q | k | v channels of the CTA.
__global__ void delta_prepare_kernel(kllm_seq_delta m, const float* __restrict__ proj, const float* __restrict__ low2,
                                     float* __restrict__ conv_state, StepRows rows, float* __restrict__ prep) {
  extern __shared__ float cs[];  // [dim] q, [dim] k, [vdim] v
  const RowPlace p = place_row(rows, blockIdx.x, m.conv_taps);
  if (p.n_here == 0) return;
  const int h = blockIdx.y;
  const bool has_qk = h < m.kv_heads;
  const int D = m.dim, V = m.vdim;
  const int qn = m.kv_heads * D, vn = m.heads * V, dn = m.heads * D, C = 2 * qn + vn, hist = m.conv_taps - 1;
  const int stride = C + m.heads + m.decay_rank + m.gate_rank;
  const int prow = delta_prep_row(m);
  const DeltaRow at = delta_row(m);
  float* st = hist > 0 ? conv_state + static_cast<size_t>(p.seq) * hist * C : nullptr;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  for (int jj = 0; jj < p.n_here; ++jj) {
    const int t = blockIdx.x + jj, pos = p.pos0 + p.j0 + jj;
    const float* row = proj + static_cast<size_t>(t) * stride;
    const float* l2 = low2 + static_cast<size_t>(t) * (dn + vn);
    float* dst = prep + static_cast<size_t>(t) * prow;
    for (int i = threadIdx.x; i < (has_qk ? 2 * D : 0) + V; i += blockDim.x) {
      const bool is_v = !has_qk || i >= 2 * D;
      const int c = is_v ? 2 * qn + h * V + (i - (has_qk ? 2 * D : 0)) : (i < D ? h * D + i : qn + h * D + (i - D));
      cs[is_v ? 2 * D + (i - (has_qk ? 2 * D : 0)) : i] = siluf(conv_at(proj, stride, c, C, m.conv_taps, m.conv_w, nullptr, st, p, pos));
    }
    __syncthreads();
    if (has_qk && warp < 2) {  // unit vectors: warp 0 the query head, warp 1 the key head
      const float* src = cs + warp * D;
      float ss = 0.f;
      for (int d = lane; d < D; d += 32) ss = fmaf(src[d], src[d], ss);
      ss = warp_sum(ss);
      float rinv = 1.0f / sqrtf(ss + 1e-6f);
      if (warp == 0) rinv *= 1.0f / sqrtf(static_cast<float>(D));
      float* out = dst + (warp == 0 ? at.q : at.k) + h * D;
      for (int d = lane; d < D; d += 32) out[d] = src[d] * rinv;
    }
    for (int i = threadIdx.x; i < V; i += blockDim.x) {
      dst[at.v + h * V + i] = cs[2 * D + i];
      dst[at.gate + h * V + i] = sigmoidf(l2[dn + h * V + i]);
    }
    if (threadIdx.x == 0) dst[at.beta + h] = sigmoidf(row[C + h]);
    for (int i = threadIdx.x; i < D; i += blockDim.x)
      dst[at.decay + h * D + i] = expf(-m.rate[h] * softplusf(l2[h * D + i] + m.dt_bias[h * D + i]));
    __syncthreads();
  }
  if (p.j0 == 0 && hist > 0) {
    if (has_qk) {
      conv_state_write(proj, stride, C, m.conv_taps, nullptr, st, p, h * D, D);
      conv_state_write(proj, stride, C, m.conv_taps, nullptr, st, p, qn + h * D, D);
    }
    conv_state_write(proj, stride, C, m.conv_taps, nullptr, st, p, 2 * qn + h * V, V);
  }
}

constexpr int kDeltaThreads = 128;
constexpr int kDeltaPad = 4;  // floats between the row slices of two lanes in shared memory: their 16-byte loads hit different banks

// One CTA: one entry, one head, COLS = kDeltaThreads / L value columns.  L lanes share a column j; lane l holds the rows
// l * RP .. l * RP + RP - 1 of S[:, j] in registers.  Per row of the entry: S <- g S; u = beta (v_j - S[:, j] . k);
// S[:, j] += k u; o_j = S[:, j] . q -- every column on its own, the two dot products joined over the column's lanes.
// Chunks of `chunk` rows (q, k, g of the head, v of the CTA's columns, beta) come through two shared-memory buffers by
// cp.async: the next chunk is on its way while the current one is worked on.  VEC: every part of a prepared row starts on
// 16 bytes (dim and vdim multiples of 4), so the copies are 16 bytes wide.
// Only the prediction's dot product is joined over the lanes inside the loop over rows (the next row's state waits for
// it); the read-out leaves its per-lane parts in shared memory and they are added when the chunk is written out.
//
// Long entries (MODE 1 and 2; MODE 0 walks a whole entry).  A row maps the state linearly, S_t = M_t S_(t-1) + k_t u'_t with
// M_t = (I - beta k k^T) diag(g), so an entry is cut into segments of kDeltaSeg rows that are walked at the same time:
//   MODE 1   every segment from an empty state (the first from the sequence's), with dim more columns that start as the
//            identity and are fed zero values: they end as the segment's product of the M_t.  No read-out.  The end states
//            go to the scratch E [segment][head][dim][vdim + dim].
//   carry    the start state of every segment, one after the other: S_start(s+1) = S'_end(s) + M(s) S_start(s); it
//            replaces S'_end(s) in E; the last one is the sequence's new state
//   MODE 2   every segment again, from its start state, with the read-out (the first segment starts from the copy of the
//            sequence's old state that MODE 1 left behind the blocks of E: the carry has overwritten the state by then)
constexpr int kDeltaSeg = 128;
constexpr int kDeltaParallelFrom = 256;
__host__ __device__ inline int delta_segment_id(int first, int e, int seg) { return first / kDeltaSeg + e + seg; }

template <int RP, int L, bool VEC, int MODE>
__global__ void __launch_bounds__(kDeltaThreads)
delta_rule_kernel(kllm_seq_delta m, int chunk, const float* __restrict__ prep, float* __restrict__ state,
                  StepRows rows, const int32_t* __restrict__ ent_seq, float* __restrict__ o, float* __restrict__ E,
                  float* __restrict__ S0, int segs_max) {
  const int e = MODE ? blockIdx.z / segs_max : blockIdx.z, seg = MODE ? blockIdx.z % segs_max : 0, h = blockIdx.y;
  const int e_first = rows.ent_first[e], e_count = rows.ent_count[e], pos0 = rows.ent_pos0[e], seq = ent_seq[e];
  if (MODE && seg * kDeltaSeg >= e_count) return;
  // the product of an entry's first segment is never used (that segment starts from the sequence's own state): CTAs that
  // hold identity columns only have nothing to do there.  (The last segment's is: the carry ends with the new state.)
  if (MODE == 1 && seg == 0 && static_cast<int>(blockIdx.x) * (kDeltaThreads / L) >= m.vdim) return;
  const int first = MODE ? e_first + seg * kDeltaSeg : e_first;
  const int count = MODE ? min(kDeltaSeg, e_count - seg * kDeltaSeg) : e_count;
  constexpr int COLS = kDeltaThreads / L;
  const int lane = threadIdx.x % L, jl = threadIdx.x / L, j0 = blockIdx.x * COLS, j = j0 + jl;
  const int ncols = MODE == 1 ? m.vdim + m.dim : m.vdim;  // MODE 1: the identity columns follow the value columns
  const bool live = j < ncols, ident = MODE == 1 && j >= m.vdim;
  const int D = m.dim, vn = m.heads * m.vdim;
  const int g = h / (m.heads / m.kv_heads);
  const int prow = delta_prep_row(m);
  const DeltaRow at = delta_row(m);
  const int off_q = at.q + g * D, off_k = at.k + g * D, off_v = at.v + h * m.vdim + j0, off_g = at.decay + h * D,
            off_b = at.beta + h;
  constexpr int LS = RP + kDeltaPad, DP = L * LS;  // a lane's slice, a row of q / k / g in shared memory
  constexpr int per = 3 * DP + COLS + 4;           // floats of one row of a chunk: q | k | g | v | beta (+ pad)
  extern __shared__ __align__(16) float sm[];
  float* o_s = sm + 2 * chunk * per;               // [chunk][COLS][L] the read-out's parts
  for (int i = threadIdx.x; i < 2 * chunk * per; i += kDeltaThreads) sm[i] = 0.f;  // the padding stays zero
  __syncthreads();

  auto stage = [&](int r0, int nr, float* buf) {
    if (VEC) {
      const int dv = D / 4, cv = max(0, min(COLS, m.vdim - j0)) / 4;
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
      const int cv = max(0, min(COLS, m.vdim - j0));
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
  float* st = state + ((static_cast<size_t>(seq) * m.heads + h) * D) * m.vdim + (live && !ident ? j : 0);
  // this segment's block of E: [dim][vdim + dim]
  float* Es = MODE ? E + ((static_cast<size_t>(delta_segment_id(e_first, e, seg)) * m.heads + h) * D) * (m.vdim + D) + (live ? j : 0)
                   : nullptr;
#pragma unroll
  for (int x = 0; x < RP; ++x) {
    const int i = lane * RP + x;
    const bool on = live && i < D;
    // the copy of the entry's old state: [entry][head][dim][vdim]
    float* keep = MODE ? S0 + ((static_cast<size_t>(e) * m.heads + h) * D + i) * m.vdim + j : nullptr;
    if (ident) S[x] = on && i == j - m.vdim ? 1.0f : 0.f;
    else if (MODE == 2) S[x] = on ? (seg > 0 ? Es[static_cast<size_t>(i) * (m.vdim + D)] : *keep) : 0.f;
    else S[x] = on && pos0 > 0 && seg == 0 ? st[static_cast<size_t>(i) * m.vdim] : 0.f;
    if (MODE == 1 && seg == 0 && on && !ident) *keep = S[x];
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
#pragma unroll
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
      if (MODE != 1) o_s[r * kDeltaThreads + threadIdx.x] = (p0 + p1) + (p2 + p3);
    }
    __syncthreads();
    for (int i = threadIdx.x; MODE != 1 && i < nr * COLS; i += kDeltaThreads) {
      const int jj = j0 + i % COLS;
      float out = 0.f;
#pragma unroll
      for (int l = 0; l < L; ++l) out += o_s[i * L + l];
      if (jj < m.vdim) o[static_cast<size_t>(first + r0 + i / COLS) * vn + h * m.vdim + jj] = out;
    }
  }
  if (MODE == 2) return;  // the carry wrote the sequence's new state
#pragma unroll
  for (int x = 0; x < RP; ++x) {
    const int i = lane * RP + x;
    if (live && i < D) {
      if (MODE == 1) Es[static_cast<size_t>(i) * (m.vdim + D)] = S[x];
      else st[static_cast<size_t>(i) * m.vdim] = S[x];
    }
  }
}

// One CTA: one entry, one head, JB = groups * kCarryCols value columns; thread (i, group) owns S[i][its kCarryCols
// columns].  Per segment the product M(s) S_start(s) goes through shared memory: S_start(s) as the CTA's columns of the
// state at hand, M in tiles of kCarryTile columns.  The tiles of ALL segments are known before the carry starts, so they
// stream through two buffers by cp.async, one (segment, tile) ahead of the arithmetic; only the state is sequential.
constexpr int kCarryCols = 8;
constexpr int kCarryTile = 16;
__global__ void __launch_bounds__(256)
delta_carry_kernel(kllm_seq_delta m, float* __restrict__ state, StepRows rows, const int32_t* __restrict__ ent_seq,
                   float* __restrict__ E, int groups) {
  extern __shared__ float sm[];
  const int e = blockIdx.z, h = blockIdx.y;
  const int first = rows.ent_first[e], count = rows.ent_count[e];
  const int D = m.dim, V = m.vdim, EW = V + D, JB = groups * kCarryCols;
  constexpr int TW = kCarryTile + 1;
  float* Ms = sm;                 // [2][D][kCarryTile + 1]
  float* cur = Ms + 2 * D * TW;   // [D][JB]
  const int i = threadIdx.x % D, grp = threadIdx.x / D;
  const bool mine = static_cast<int>(threadIdx.x) < groups * D;
  const int jc = grp * kCarryCols, j0 = blockIdx.x * JB + jc;  // this thread's columns: j0 .. j0 + kCarryCols - 1
  const int segs = (count + kDeltaSeg - 1) / kDeltaSeg, tiles = (D + kCarryTile - 1) / kCarryTile;
  auto block = [&](int sgm) { return E + ((static_cast<size_t>(delta_segment_id(first, e, sgm)) * m.heads + h) * D) * EW; };
  auto fetch = [&](int step) {  // tile step % tiles of segment 1 + step / tiles
    const float* Es = block(1 + step / tiles);
    const int l0 = (step % tiles) * kCarryTile;
    float* dst = Ms + (step & 1) * D * TW;
    for (int idx = threadIdx.x; idx < D * kCarryTile; idx += blockDim.x) {
      const int r = idx / kCarryTile, l = idx % kCarryTile;
      if (l0 + l < D) cp_async4(dst + r * TW + l, Es + static_cast<size_t>(r) * EW + V + l0 + l);
    }
    cp_async_commit();
  };
  float c[kCarryCols], own[kCarryCols], acc[kCarryCols];
  {
    const float* E0 = block(0) + static_cast<size_t>(i) * EW;  // the first segment started from the sequence's state
#pragma unroll
    for (int x = 0; x < kCarryCols; ++x) c[x] = mine && j0 + x < V ? E0[j0 + x] : 0.f;
  }
  const int total = (segs - 1) * tiles;
  if (total > 0) fetch(0);
  for (int step = 0; step < total; ++step) {
    const int sgm = 1 + step / tiles, tile = step % tiles;
    float* Es = block(sgm);
    if (tile == 0) {  // a segment begins: its start state goes to shared memory, its own end state is on its way
      __syncthreads();  // the previous segment's reads of cur are over
#pragma unroll
      for (int x = 0; x < kCarryCols; ++x) {
        if (mine) cur[i * JB + jc + x] = c[x];
        own[x] = mine && j0 + x < V ? Es[static_cast<size_t>(i) * EW + j0 + x] : 0.f;
        acc[x] = 0.f;
      }
    }
    cp_async_wait_all();
    __syncthreads();  // the tile has landed, cur is written, the other buffer is free
    if (step + 1 < total) fetch(step + 1);
    if (mine) {
      const float* mt = Ms + (step & 1) * D * TW + i * TW;
      const int l0 = tile * kCarryTile, nl = min(kCarryTile, D - l0);
      for (int l = 0; l < nl; ++l) {
        const float mv = mt[l];
        const float* cr = cur + (l0 + l) * JB + jc;
#pragma unroll
        for (int x = 0; x < kCarryCols; ++x) acc[x] = fmaf(mv, cr[x], acc[x]);
      }
    }
    if (tile == tiles - 1 && mine) {
#pragma unroll
      for (int x = 0; x < kCarryCols; ++x) {
        if (j0 + x < V) Es[static_cast<size_t>(i) * EW + j0 + x] = c[x];  // the segment's start state, for the second pass
        c[x] = own[x] + acc[x];
      }
    }
  }
  if (mine) {
    float* out = state + ((static_cast<size_t>(ent_seq[e]) * m.heads + h) * D + i) * V;
#pragma unroll
    for (int x = 0; x < kCarryCols; ++x)
      if (j0 + x < V) out[j0 + x] = c[x];
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
  (void)C;
  const size_t smem = static_cast<size_t>(a.dim) * sizeof(float);
  const int threads = std::min(256, (a.dim + 31) / 32 * 32);
  const dim3 grid(T, a.heads + a.kv_heads);
  KLLM_SEQ_DISPATCH(dtype, (qk_conv_prepare_kernel<AT><<<grid, threads, smem, s>>>(a, p, qk, rows, static_cast<AT*>(q), kv)));
  return done();
}

int launch_ssm_conv(int dtype, const kllm_seq_ssm& m, const float* uz, float* conv_state, const StepRows& rows, float* uc,
                    void* uc_ct, int T, cudaStream_t s) {
  const int threads = 256;
  const dim3 grid(T, (m.inner + threads - 1) / threads);
  KLLM_SEQ_DISPATCH(dtype, (ssm_conv_kernel<AT><<<grid, threads, 0, s>>>(m.inner, m.conv_taps, m.conv_w, m.conv_b, uz, conv_state,
                                                                     rows, uc, static_cast<AT*>(uc_ct))));
  return done();
}

size_t ssm_scan_scratch_bytes(const kllm_seq_ssm& m, int T, int n_entries, int max_count) {
  if (max_count <= kScanParallelFrom) return 0;
  const size_t segs = static_cast<size_t>(T) / kScanSeg + n_entries + 1;
  return (2 * static_cast<size_t>(T) * m.inner + segs * m.inner * (m.state + 1)) * sizeof(float);
}

int launch_ssm_scan(int dtype, const kllm_seq_ssm& m, const float* uz, const float* uc, const float* low, float* state,
                    const StepRows& rows, const int32_t* ent_seq, int max_count, int T, float* scratch, void* out,
                    cudaStream_t s) {
  if (m.state > 32 * kScanPerLane) return KLLM_E_UNSUPPORTED;
  // at least 4 lanes per channel: at most 32 channels of a chunk in shared memory
  const int L = std::max(4, lanes_for(m.state, kScanPerLane));
  const int CH = kScanThreads / L;
  const bool segments = max_count > kScanParallelFrom && scratch != nullptr;
  const int longest = segments ? kScanSeg : max_count;
  auto smem_for = [&](int chunk) {
    return (static_cast<size_t>(CH) * (m.dt_rank + 1) + static_cast<size_t>(chunk) * (m.dt_rank + 2 * m.state) +
            4 * static_cast<size_t>(chunk) * CH) * sizeof(float);
  };
  int chunk = 32;
  while (chunk > 1 && (smem_for(chunk) > 48 * 1024 || chunk / 2 >= longest)) chunk /= 2;
  if (smem_for(chunk) > 48 * 1024) return KLLM_E_UNSUPPORTED;
  const unsigned blocks = (m.inner + CH - 1) / CH;
  if (!segments) {
    const dim3 grid(blocks, rows.n_entries);
    KLLM_SEQ_DISPATCH(dtype, (ssm_scan_kernel<AT, false><<<grid, kScanThreads, smem_for(chunk), s>>>(
                                 m, L, chunk, uz, uc, low, state, rows, ent_seq, static_cast<AT*>(out), ScanScratch{})));
    return done();
  }
  const size_t segs = static_cast<size_t>(T) / kScanSeg + rows.n_entries + 1;
  ScanScratch sc;
  sc.yl = scratch;
  sc.cum = sc.yl + static_cast<size_t>(T) * m.inner;
  sc.send = sc.cum + static_cast<size_t>(T) * m.inner;
  sc.cend = sc.send + segs * m.inner * m.state;
  const dim3 grid(blocks, (max_count + kScanSeg - 1) / kScanSeg, rows.n_entries);
  KLLM_SEQ_DISPATCH(dtype, (ssm_scan_kernel<AT, true><<<grid, kScanThreads, smem_for(chunk), s>>>(
                               m, L, chunk, uz, uc, low, state, rows, ent_seq, static_cast<AT*>(out), sc)));
  count_launch();
  const dim3 cgrid((m.inner * m.state + 127) / 128, rows.n_entries);
  ssm_carry_kernel<<<cgrid, 128, 0, s>>>(m, state, rows, ent_seq, sc);
  count_launch();
  KLLM_SEQ_DISPATCH(dtype, (ssm_finish_kernel<AT><<<grid, kScanThreads, 0, s>>>(m, L, uz, low, rows, static_cast<AT*>(out), sc)));
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
  const size_t smem = (2 * static_cast<size_t>(m.dim) + m.vdim) * sizeof(float);
  if (smem > 48 * 1024) return KLLM_E_UNSUPPORTED;
  const dim3 grid(T, m.heads);
  delta_prepare_kernel<<<grid, 128, smem, s>>>(m, proj, low2, conv_state, rows, prep);
  return done();
}

size_t delta_rule_scratch_bytes(const kllm_seq_delta& m, int T, int n_entries, int max_count) {
  if (max_count <= kDeltaParallelFrom) return 0;
  const size_t segs = static_cast<size_t>(T) / kDeltaSeg + n_entries + 1;
  return (segs * m.heads * m.dim * (m.vdim + m.dim) + static_cast<size_t>(n_entries) * m.heads * m.dim * m.vdim) * sizeof(float);
}

int launch_delta_rule(const kllm_seq_delta& m, const float* prep, float* state, const StepRows& rows, const int32_t* ent_seq,
                      int max_count, int T, float* scratch, float* o, cudaStream_t s) {
  // 16 rows of a column per thread while that leaves at most 8 lanes to a column, else 32
  const int RP = m.dim <= 128 ? 16 : 32;
  if (m.dim > 256) return KLLM_E_UNSUPPORTED;
  const int L = lanes_for(m.dim, RP);
  const int COLS = kDeltaThreads / L;
  const int per = 3 * L * (RP + kDeltaPad) + COLS + 4;
  const bool segments = max_count > kDeltaParallelFrom && scratch != nullptr;
  const int longest = segments ? kDeltaSeg : max_count;
  auto smem_for = [&](int chunk) { return (2 * static_cast<size_t>(chunk) * per + static_cast<size_t>(chunk) * kDeltaThreads) * sizeof(float); };
  int chunk = 16;
  while (chunk > 1 && (smem_for(chunk) > 48 * 1024 || chunk / 2 >= longest)) chunk /= 2;
  if (smem_for(chunk) > 48 * 1024) return KLLM_E_UNSUPPORTED;
  const bool vec = m.dim % 4 == 0 && m.vdim % 4 == 0;
  const int segs_max = segments ? (max_count + kDeltaSeg - 1) / kDeltaSeg : 1;
  float* keep = segments ? scratch + (static_cast<size_t>(T) / kDeltaSeg + rows.n_entries + 1) * m.heads * m.dim * (m.vdim + m.dim)
                         : nullptr;
#define KLLM_DELTA_M(R, LN, MODE, COLSN)                                                                                  \
  do {                                                                                                                    \
    const dim3 grid(((COLSN) + COLS - 1) / COLS, m.heads, rows.n_entries * segs_max);                                      \
    if (vec)                                                                                                              \
      delta_rule_kernel<R, LN, true, MODE><<<grid, kDeltaThreads, smem_for(chunk), s>>>(m, chunk, prep, state, rows, ent_seq, o, \
                                                                                         scratch, keep, segs_max);       \
    else                                                                                                                  \
      delta_rule_kernel<R, LN, false, MODE><<<grid, kDeltaThreads, smem_for(chunk), s>>>(m, chunk, prep, state, rows, ent_seq, o, \
                                                                                          scratch, keep, segs_max);      \
  } while (0)
#define KLLM_DELTA(MODE, COLSN)                      \
  do {                                               \
    if (RP == 32) KLLM_DELTA_M(32, 8, MODE, COLSN);  \
    else if (L == 1) KLLM_DELTA_M(16, 1, MODE, COLSN); \
    else if (L == 2) KLLM_DELTA_M(16, 2, MODE, COLSN); \
    else if (L == 4) KLLM_DELTA_M(16, 4, MODE, COLSN); \
    else KLLM_DELTA_M(16, 8, MODE, COLSN);           \
  } while (0)
  if (!segments) {
    KLLM_DELTA(0, m.vdim);
    return done();
  }
  KLLM_DELTA(1, m.vdim + m.dim);
  count_launch();
  const int groups = std::max(1, std::min(8, 256 / m.dim));
  const int JB = groups * kCarryCols;
  const dim3 cgrid((m.vdim + JB - 1) / JB, m.heads, rows.n_entries);
  const size_t csmem = (2 * static_cast<size_t>(m.dim) * (kCarryTile + 1) + static_cast<size_t>(m.dim) * JB) * sizeof(float);
  delta_carry_kernel<<<cgrid, 256, csmem, s>>>(m, state, rows, ent_seq, scratch, groups);
  count_launch();
  KLLM_DELTA(2, m.vdim);
#undef KLLM_DELTA
#undef KLLM_DELTA_M
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
