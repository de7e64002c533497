// State-space duality mixer of the sequence-batch engine (KLLM_SEQ_MIXER_SSD): a selective scan whose decay is one number
// per head and token, with a matrix state per head.
//
//   ssd_conv   x | B | C channels of the input projection through a short causal convolution (state: the last taps - 1
//              inputs, see seq_rows.cuh) and SiLU
//   ssd_scan   step sizes dt = softplus(. + dt_bias), decays exp(a dt), and per head the recurrence
//              S <- exp(a dt) S + dt B x^T,  y = S^T C + d x   over the rows of every entry, from the sequence's state
//   ssd_out    y * silu(z), RMS norm in equal parts of the inner width, weight, conversion to the compute type
//
// Everything here is fp32; only ssd_out's result (the input of the output projection) is in the compute type.
//
// State layout: [slots][heads][vdim][state] -- the `state` coordinates of one value column lie side by side; the lanes
// that share a column hold contiguous runs of them.
//
// Long entries.  The recurrence is linear in S, so an entry is cut into segments of kSsdSeg rows that are walked at the
// same time, each from an empty state (the first from the sequence's): with c_t the sum of a dt from the segment's start
// to row t, the true output is y_t = y'_t + exp(c_t) S_start^T C_t, y' the segment's own walk.
//   ssd_scan_kernel<1>   the segment's own walk: y', c_t of every row, the segment's last S' and c
//   ssd_carry_kernel     S_start of every segment, one after the other; the sequence's new state
//   ssd_finish_kernel    y += exp(c_t) S_start^T C_t: per segment and head a product [rows x state] [state x vdim]
#include <cuda_runtime.h>

#include <algorithm>
#include <cstdint>

#include "seq_engine.h"
#include "seq_rows.cuh"

namespace kllm {
namespace seq {
namespace {

constexpr unsigned kAll = 0xffffffffu;
constexpr int kSsdThreads = 128;
constexpr int kSsdRows = 8;           // state coordinates of a column per lane (of each of 4 columns) ...
constexpr int kSsdRowsWide = 16;      // ... or, for states beyond 256 coordinates, of each of 2 columns
constexpr int kSsdSeg = 128;          // rows of a segment when long entries are walked in parallel
constexpr int kSsdParallelFrom = 256; // entries longer than this are cut into segments

template <typename AT> __device__ __forceinline__ AT from_f(float v);
template <> __device__ __forceinline__ float from_f<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 from_f<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

__device__ __forceinline__ float siluf(float z) { return z / (1.0f + expf(-z)); }
__device__ __forceinline__ float softplusf(float z) { return z > 20.0f ? z : log1pf(expf(z)); }

__global__ void ssd_conv_kernel(kllm_seq_ssd m, const float* __restrict__ proj, float* __restrict__ conv_state, StepRows rows,
                                float* __restrict__ xbc) {
  const int taps = m.conv_taps;
  const RowPlace p = place_row(rows, blockIdx.x, taps);
  if (p.n_here == 0) return;
  const int hist = taps - 1, C = ssd_conv_channels(m), P = ssd_proj_row(m);
  const float* in = proj + ssd_inner(m);  // the filtered channels follow the z rows
  float* st = hist > 0 ? conv_state + static_cast<size_t>(p.seq) * hist * C : nullptr;
  const int c0 = blockIdx.y * blockDim.x, c = c0 + threadIdx.x;
  for (int jj = 0; jj < p.n_here; ++jj) {
    const int t = blockIdx.x + jj, pos = p.pos0 + p.j0 + jj;
    if (c < C)
      xbc[static_cast<size_t>(t) * C + c] =
          siluf(conv_at(in, P, c, C, taps, m.conv_w, nullptr, st, p, pos) + (m.conv_b ? m.conv_b[c] : 0.f));
  }
  // the thread that read a channel's old state is the one that writes its new one
  if (p.j0 == 0 && hist > 0) conv_state_write(in, P, C, taps, nullptr, st, p, c0, min(static_cast<int>(blockDim.x), C - c0));
}

struct SsdScratch {
  float* cum;   // [T][heads]: c_t
  float* send;  // [segments][heads][vdim][state]: a segment's last S', then its S_start
  float* cend;  // [segments][heads]: a segment's last c
};
__host__ __device__ inline int ssd_segment_id(int first, int e, int seg) { return first / kSsdSeg + e + seg; }

// Sums of CC accumulators over the L lanes that share a block of columns.  With L >= CC the lanes first trade halves
// (a lane keeps the columns of its side and adds the partner's sums for them), so that CC values cost CC - 1 shuffles
// instead of CC log2(CC); the remaining strides are plain butterflies.  Returns true in the lanes that hold a total;
// `col` is then the column (0 .. CC - 1) of acc[0].  With L < CC lane 0 holds all CC totals (col = 0, acc[0 .. CC - 1]).
template <int CC>
__device__ __forceinline__ bool join_columns(float (&acc)[CC], int L, int lane, int* col, bool* all) {
  *all = false, *col = 0;
  if (L < CC) {
    for (int o = 1; o < L; o <<= 1) {
#pragma unroll
      for (int c = 0; c < CC; ++c) acc[c] += __shfl_xor_sync(kAll, acc[c], o);
    }
    *all = true;
    return lane == 0;
  }
  int stride = 1, at = 0;
#pragma unroll
  for (int half = CC / 2; half >= 1; half /= 2) {
    const bool up = (lane & stride) != 0;
#pragma unroll
    for (int c = 0; c < half; ++c) {
      const float keep = up ? acc[c + half] : acc[c];
      const float send = up ? acc[c] : acc[c + half];
      acc[c] = keep + __shfl_xor_sync(kAll, send, stride);
    }
    at += up ? half : 0;
    stride <<= 1;
  }
  for (int o = stride; o < L; o <<= 1) acc[0] += __shfl_xor_sync(kAll, acc[0], o);
  *col = at;
  return lane < CC;
}

// One CTA: one entry (MODE 0) or one segment of an entry (MODE 1), one head, COLS = blockDim.x / L * CC value columns.
// L lanes share a block of CC columns; lane l keeps the state coordinates l RS .. l RS + RS - 1 of each of them in
// registers (RS x CC values), so that a row's B and C are read once for CC columns and as 16-byte vectors.  Chunks of
// rows pass through two buffers in shared memory (B and C padded with zeros to L RS coordinates, the columns' x, dt and
// the decay): cp.async brings the next chunk while the current one is walked one row after the other; only the read-out's
// dot products are joined over the L lanes.
template <int MODE, int RS, int CC>
__global__ void __launch_bounds__(kSsdThreads)
ssd_scan_kernel(kllm_seq_ssd m, int L, int chunk, int segs_max, const float* __restrict__ proj, const float* __restrict__ xbc,
                float* __restrict__ state, StepRows rows, const int32_t* __restrict__ ent_seq, float* __restrict__ y,
                SsdScratch sc) {
  const int e = MODE == 0 ? blockIdx.z : blockIdx.z / segs_max, seg = MODE == 0 ? 0 : blockIdx.z % segs_max;
  const int e_first = rows.ent_first[e], e_count = rows.ent_count[e], pos0 = rows.ent_pos0[e], seq = ent_seq[e];
  if (MODE != 0 && seg * kSsdSeg >= e_count) return;
  const int first = MODE == 0 ? e_first : e_first + seg * kSsdSeg;
  const int count = MODE == 0 ? e_count : min(kSsdSeg, e_count - seg * kSsdSeg);
  const int h = blockIdx.y, N = m.state, V = m.vdim, inner = ssd_inner(m);
  const int nthreads = blockDim.x, Ns = L * RS;  // Ns >= N: the padded row of B and C
  const int COLS = nthreads / L * CC;
  const int lane = threadIdx.x % L, cblock = threadIdx.x / L * CC, pcol0 = blockIdx.x * COLS + cblock;
  const int g = h / (m.heads / m.groups);
  const int C = ssd_conv_channels(m), P = ssd_proj_row(m);
  const int b_off = inner + g * N, c_off = inner + m.groups * N + g * N, dt_off = 2 * inner + 2 * m.groups * N + h;
  const float rate = m.a[h], skip = m.d[h], dt_bias = m.dt_bias[h];

  // two buffers of a chunk of rows each: B | C | x | dt (raw, then the step size) | decay
  extern __shared__ __align__(16) float sm[];
  const int per_buf = chunk * (2 * Ns + COLS + 2);
  float* y_s = sm + 2 * per_buf;      // [chunk][COLS]
  float* cum_s = y_s + chunk * COLS;  // [chunk]: c_t
  // the rows r0 .. of the entry on their way into buffer b (coordinates beyond N and columns beyond V are zeros, written
  // by plain stores: the buffer was last read before the barrier that precedes this call)
  auto fetch = [&](int b, int r0) {
    const int nr = min(chunk, count - r0);
    float* B_s = sm + b * per_buf;
    float* C_s = B_s + chunk * Ns;
    float* x_s = C_s + chunk * Ns;
    float* dt_s = x_s + chunk * COLS;
    for (int i = threadIdx.x; i < nr * Ns; i += nthreads) {
      const int n = i % Ns;
      const float* row = xbc + static_cast<size_t>(first + r0 + i / Ns) * C;
      if (n < N) cp_async4(B_s + i, row + b_off + n), cp_async4(C_s + i, row + c_off + n);
      else B_s[i] = 0.f, C_s[i] = 0.f;
    }
    for (int i = threadIdx.x; i < nr * COLS; i += nthreads) {
      const int pc = blockIdx.x * COLS + i % COLS;
      if (pc < V) cp_async4(x_s + i, xbc + static_cast<size_t>(first + r0 + i / COLS) * C + h * V + pc);
      else x_s[i] = 0.f;
    }
    for (int i = threadIdx.x; i < nr; i += nthreads) cp_async4(dt_s + i, proj + static_cast<size_t>(first + r0 + i) * P + dt_off);
    cp_async_commit();
  };

  float S[CC][RS];
  const size_t sid = MODE == 0 ? 0 : ssd_segment_id(e_first, e, seg);
  {
    const float* src = state + (static_cast<size_t>(seq) * m.heads + h) * V * N;
    const bool from_state = pos0 > 0 && seg == 0;
#pragma unroll
    for (int c = 0; c < CC; ++c)
#pragma unroll
      for (int k = 0; k < RS; ++k) {
        const int n = lane * RS + k;
        S[c][k] = from_state && pcol0 + c < V && n < N ? src[static_cast<size_t>(pcol0 + c) * N + n] : 0.f;
      }
  }
  float cum = 0.f;  // the sum of a dt since the segment's start (the same in every thread)
  fetch(0, 0);
  for (int r0 = 0, b = 0; r0 < count; r0 += chunk, b ^= 1) {
    const int nr = min(chunk, count - r0);
    const float* B_s = sm + b * per_buf;
    const float* C_s = B_s + chunk * Ns;
    const float* x_s = C_s + chunk * Ns;
    float* dt_s = sm + b * per_buf + 2 * chunk * Ns + chunk * COLS;
    float* dec_s = dt_s + chunk;
    cp_async_wait_all();
    __syncthreads();  // the chunk has landed; the chunk before it (the other buffer, y_s) has been used up
    if (r0 + chunk < count) fetch(b ^ 1, r0 + chunk);
    for (int i = threadIdx.x; i < nr; i += nthreads) {
      const float dt = softplusf(dt_s[i] + dt_bias);
      dt_s[i] = dt;
      dec_s[i] = expf(rate * dt);
    }
    __syncthreads();
    if (MODE == 1 && threadIdx.x == 0) {
      float c = cum;
      for (int r = 0; r < nr; ++r) c = fmaf(rate, dt_s[r], c), cum_s[r] = c;
    }
    for (int r = 0; r < nr; ++r) {
      const float dec = dec_s[r];
      float Bn[RS], Cn[RS], dx[CC], acc[CC];
#pragma unroll
      for (int k = 0; k < RS; k += 4) {
        *reinterpret_cast<float4*>(Bn + k) = *reinterpret_cast<const float4*>(B_s + r * Ns + lane * RS + k);
        *reinterpret_cast<float4*>(Cn + k) = *reinterpret_cast<const float4*>(C_s + r * Ns + lane * RS + k);
      }
      const float dt = dt_s[r];
#pragma unroll
      for (int c = 0; c < CC; ++c) dx[c] = dt * x_s[r * COLS + cblock + c];
#pragma unroll
      for (int c = 0; c < CC; ++c) {
        acc[c] = 0.f;
#pragma unroll
        for (int k = 0; k < RS; ++k) {
          S[c][k] = fmaf(dec, S[c][k], dx[c] * Bn[k]);
          acc[c] = fmaf(S[c][k], Cn[k], acc[c]);
        }
      }
      int col;
      bool all;
      if (join_columns<CC>(acc, L, lane, &col, &all)) {
        const int n_out = all ? CC : 1;
        for (int c = 0; c < n_out; ++c) {
          const int at = r * COLS + cblock + col + c;
          y_s[at] = fmaf(skip, x_s[at], acc[c]);
        }
      }
    }
    if (MODE == 1)
      for (int r = 0; r < nr; ++r) cum = fmaf(rate, dt_s[r], cum);
    __syncthreads();
    for (int i = threadIdx.x; i < nr * COLS; i += nthreads) {
      const int pc = blockIdx.x * COLS + i % COLS;
      if (pc >= V) continue;
      const size_t at = static_cast<size_t>(first + r0 + i / COLS) * inner + h * V + pc;
      y[at] = y_s[i];
    }
    if (MODE == 1 && blockIdx.x == 0)
      for (int i = threadIdx.x; i < nr; i += nthreads)
        sc.cum[static_cast<size_t>(first + r0 + i) * m.heads + h] = cum_s[i];
  }
  float* dst = MODE == 1 ? sc.send + (sid * m.heads + h) * V * N : state + (static_cast<size_t>(seq) * m.heads + h) * V * N;
  if (MODE == 1 && blockIdx.x == 0 && threadIdx.x == 0) sc.cend[sid * m.heads + h] = cum;
#pragma unroll
  for (int c = 0; c < CC; ++c)
#pragma unroll
    for (int k = 0; k < RS; ++k) {
      const int n = lane * RS + k;
      if (pcol0 + c < V && n < N) dst[static_cast<size_t>(pcol0 + c) * N + n] = S[c][k];
    }
}

// The start state's share of a segment's outputs: y[r][v] += exp(c_r) sum_n C[r][n] S_start[v][n] for the rows of one
// segment, one head and a block of kFinCols value columns.  A plain tiled fp32 product: both operands pass through shared
// memory state-coordinate-major in steps of kFinK, a thread owns 8 rows x 8 columns.
constexpr int kFinCols = 64, kFinK = 32;
__global__ void __launch_bounds__(kSsdThreads)
ssd_finish_kernel(kllm_seq_ssd m, int segs_max, const float* __restrict__ xbc, StepRows rows, float* __restrict__ y,
                  SsdScratch sc) {
  const int e = blockIdx.z / segs_max, seg = blockIdx.z % segs_max;
  if (seg == 0) return;  // the first segment started from the true state
  const int e_first = rows.ent_first[e], e_count = rows.ent_count[e];
  if (seg * kSsdSeg >= e_count) return;
  const int first = e_first + seg * kSsdSeg, count = min(kSsdSeg, e_count - seg * kSsdSeg);
  const int h = blockIdx.y, N = m.state, V = m.vdim, inner = ssd_inner(m), C = ssd_conv_channels(m);
  const int c_off = inner + m.groups * N + h / (m.heads / m.groups) * N;
  const int v0 = blockIdx.x * kFinCols;
  const float* S = sc.send + (static_cast<size_t>(ssd_segment_id(e_first, e, seg)) * m.heads + h) * V * N;
  __shared__ __align__(16) float Cs[kFinK][kSsdSeg + 4];
  __shared__ __align__(16) float Ss[kFinK][kFinCols + 4];
  const int tr = threadIdx.x / 8 * 8, tc = threadIdx.x % 8 * 8;  // 16 blocks of rows x 8 blocks of columns
  float acc[8][8];
#pragma unroll
  for (int i = 0; i < 8; ++i)
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[i][j] = 0.f;
  for (int k0 = 0; k0 < N; k0 += kFinK) {
    __syncthreads();
    for (int i = threadIdx.x; i < kSsdSeg * kFinK; i += kSsdThreads) {
      const int k = i % kFinK, r = i / kFinK;
      Cs[k][r] = r < count && k0 + k < N ? xbc[static_cast<size_t>(first + r) * C + c_off + k0 + k] : 0.f;
    }
    for (int i = threadIdx.x; i < kFinCols * kFinK; i += kSsdThreads) {
      const int k = i % kFinK, v = i / kFinK;
      Ss[k][v] = v0 + v < V && k0 + k < N ? S[static_cast<size_t>(v0 + v) * N + k0 + k] : 0.f;
    }
    __syncthreads();
#pragma unroll 4
    for (int k = 0; k < kFinK; ++k) {
      float a[8], b[8];
      *reinterpret_cast<float4*>(a) = *reinterpret_cast<const float4*>(&Cs[k][tr]);
      *reinterpret_cast<float4*>(a + 4) = *reinterpret_cast<const float4*>(&Cs[k][tr + 4]);
      *reinterpret_cast<float4*>(b) = *reinterpret_cast<const float4*>(&Ss[k][tc]);
      *reinterpret_cast<float4*>(b + 4) = *reinterpret_cast<const float4*>(&Ss[k][tc + 4]);
#pragma unroll
      for (int i = 0; i < 8; ++i)
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
    }
  }
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const int r = tr + i;
    if (r >= count) continue;
    const float dec = expf(sc.cum[static_cast<size_t>(first + r) * m.heads + h]);
    float* yr = y + static_cast<size_t>(first + r) * inner + h * V + v0 + tc;
#pragma unroll
    for (int j = 0; j < 8; ++j)
      if (v0 + tc + j < V) yr[j] += dec * acc[i][j];
  }
}

// One thread per (entry, head, value column, state coordinate): the start state of every segment after the first, and the
// sequence's new state.
__global__ void ssd_carry_kernel(kllm_seq_ssd m, float* __restrict__ state, StepRows rows, const int32_t* __restrict__ ent_seq,
                                 SsdScratch sc) {
  const int e = blockIdx.y;
  const size_t per = static_cast<size_t>(m.heads) * m.vdim * m.state;
  const size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= per) return;
  const int first = rows.ent_first[e], count = rows.ent_count[e];
  const int segs = (count + kSsdSeg - 1) / kSsdSeg;
  const int h = static_cast<int>(i / (static_cast<size_t>(m.vdim) * m.state));
  float carry = sc.send[ssd_segment_id(first, e, 0) * per + i];  // the first segment started from the sequence's state
  constexpr int kAhead = 8;  // a batch of segments is loaded before the chain that depends on the one before it
  for (int sg0 = 1; sg0 < segs; sg0 += kAhead) {
    float own[kAhead], dec[kAhead];
#pragma unroll
    for (int j = 0; j < kAhead; ++j)
      if (sg0 + j < segs) {
        const size_t sid = ssd_segment_id(first, e, sg0 + j);
        own[j] = sc.send[sid * per + i];
        dec[j] = expf(sc.cend[sid * m.heads + h]);
      }
#pragma unroll
    for (int j = 0; j < kAhead; ++j)
      if (sg0 + j < segs) {
        sc.send[ssd_segment_id(first, e, sg0 + j) * per + i] = carry;
        carry = fmaf(dec[j], carry, own[j]);
      }
  }
  state[static_cast<size_t>(ent_seq[e]) * per + i] = carry;
}

// One CTA per (token, part of the norm): the part's gated values, their root mean square, the weight.
template <typename AT>
__global__ void ssd_out_kernel(kllm_seq_ssd m, const float* __restrict__ y, const float* __restrict__ proj, float eps,
                               AT* __restrict__ out) {
  __shared__ float red[33];
  const int t = blockIdx.x, part = blockIdx.y, inner = ssd_inner(m), n = inner / m.norm_groups, P = ssd_proj_row(m);
  const float* yr = y + static_cast<size_t>(t) * inner + part * n;
  const float* zr = proj + static_cast<size_t>(t) * P + part * n;
  float ss = 0.f;
  for (int i = threadIdx.x; i < n; i += blockDim.x) {
    const float v = yr[i] * siluf(zr[i]);
    ss = fmaf(v, v, ss);
  }
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
  for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(kAll, ss, o);
  if (lane == 0) red[warp] = ss;
  __syncthreads();
  float tot = 0.f;
  for (int i = 0; i < nw; ++i) tot += red[i];
  const float rinv = 1.0f / sqrtf(tot / static_cast<float>(n) + eps);
  const float* w = m.out_norm_w + part * n;
  AT* o = out + static_cast<size_t>(t) * inner + part * n;
  for (int i = threadIdx.x; i < n; i += blockDim.x) o[i] = from_f<AT>(yr[i] * siluf(zr[i]) * rinv * w[i]);
}

inline int done() {
  count_launch();
  return cuda_rc(cudaGetLastError());
}

// lanes that share a block of columns: the smallest power of two that leaves each at most `per_lane` state coordinates
inline int ssd_lanes(int state, int per_lane) {
  int L = 1;
  while (L * per_lane < state) L *= 2;
  return L;
}

struct SsdLaunch {
  dim3 grid;
  int threads, L, chunk, segs_max;
  size_t smem;
};

template <int MODE, int RS, int CC>
void ssd_scan_launch(const SsdLaunch& l, const kllm_seq_ssd& m, const float* proj, const float* xbc, float* state,
                     const StepRows& rows, const int32_t* ent_seq, float* y, const SsdScratch& sc, cudaStream_t s) {
  ssd_scan_kernel<MODE, RS, CC><<<l.grid, l.threads, l.smem, s>>>(m, l.L, l.chunk, l.segs_max, proj, xbc, state, rows, ent_seq,
                                                                 y, sc);
  count_launch();
}

}  // namespace

int launch_ssd_conv(const kllm_seq_ssd& m, const float* proj, float* conv_state, const StepRows& rows, float* xbc, int T,
                    cudaStream_t s) {
  if (m.conv_taps < 1 || (m.conv_taps > 1 && !conv_state)) return KLLM_E_INVALID;
  const int threads = 256;
  const dim3 grid(T, (ssd_conv_channels(m) + threads - 1) / threads);
  ssd_conv_kernel<<<grid, threads, 0, s>>>(m, proj, conv_state, rows, xbc);
  return done();
}

size_t ssd_scan_scratch_bytes(const kllm_seq_ssd& m, int T, int n_entries, int max_count) {
  if (max_count <= kSsdParallelFrom) return 0;
  const size_t segs = static_cast<size_t>(T) / kSsdSeg + n_entries + 1;
  return (static_cast<size_t>(T) * m.heads + segs * m.heads * (static_cast<size_t>(m.vdim) * m.state + 1)) * sizeof(float);
}

int launch_ssd_scan(const kllm_seq_ssd& m, const float* proj, const float* xbc, float* state, const StepRows& rows,
                    const int32_t* ent_seq, int max_count, int T, float* scratch, float* y, cudaStream_t s) {
  if (m.state > 32 * kSsdRowsWide || m.heads % m.groups) return KLLM_E_UNSUPPORTED;
  // a thread keeps 8 coordinates of 4 columns, or (states beyond 256) 16 coordinates of 2 columns
  const bool wide = m.state > 32 * kSsdRows;
  const int RS = wide ? kSsdRowsWide : kSsdRows, CC = wide ? 2 : 4;
  SsdLaunch l;
  l.L = ssd_lanes(m.state, RS);
  // as many threads as the head's columns need, in whole warps
  const int col_blocks = (m.vdim + CC - 1) / CC;
  l.threads = std::min(kSsdThreads, (l.L * col_blocks + 31) / 32 * 32);
  const int COLS = l.threads / l.L * CC;
  const bool segments = max_count > kSsdParallelFrom && scratch != nullptr;
  const int longest = segments ? kSsdSeg : max_count;
  auto smem_for = [&](int chunk) {
    return static_cast<size_t>(chunk) * (2 * (2 * l.L * RS + COLS + 2) + COLS + 1) * sizeof(float);  // two buffers, y, c_t
  };
  int chunk = 32;
  while (chunk > 1 && (smem_for(chunk) > 48 * 1024 || chunk / 2 >= longest)) chunk /= 2;
  if (smem_for(chunk) > 48 * 1024) return KLLM_E_UNSUPPORTED;
  l.chunk = chunk, l.smem = smem_for(chunk);
  const unsigned blocks = (m.vdim + COLS - 1) / COLS;
#define KLLM_SSD_SCAN(MODE, sc)                                                                                    \
  (wide ? ssd_scan_launch<MODE, kSsdRowsWide, 2>(l, m, proj, xbc, state, rows, ent_seq, y, sc, s)                  \
        : ssd_scan_launch<MODE, kSsdRows, 4>(l, m, proj, xbc, state, rows, ent_seq, y, sc, s))
  if (!segments) {
    l.grid = dim3(blocks, m.heads, rows.n_entries), l.segs_max = 1;
    KLLM_SSD_SCAN(0, SsdScratch{});
    return cuda_rc(cudaGetLastError());
  }
  const size_t segs = static_cast<size_t>(T) / kSsdSeg + rows.n_entries + 1;
  SsdScratch sc;
  sc.cum = scratch;
  sc.send = sc.cum + static_cast<size_t>(T) * m.heads;
  sc.cend = sc.send + segs * m.heads * m.vdim * m.state;
  l.segs_max = (max_count + kSsdSeg - 1) / kSsdSeg;
  l.grid = dim3(blocks, m.heads, rows.n_entries * l.segs_max);
  KLLM_SSD_SCAN(1, sc);
  const size_t per = static_cast<size_t>(m.heads) * m.vdim * m.state;
  const dim3 cgrid(static_cast<unsigned>((per + 127) / 128), rows.n_entries);
  ssd_carry_kernel<<<cgrid, 128, 0, s>>>(m, state, rows, ent_seq, sc);
  count_launch();
#undef KLLM_SSD_SCAN
  static_assert(kSsdThreads == 128 && kSsdSeg == 128, "ssd_finish_kernel: 16 x 8 threads own 8 x 8 outputs of a 128 x 64 tile");
  const dim3 fgrid((m.vdim + kFinCols - 1) / kFinCols, m.heads, rows.n_entries * l.segs_max);
  ssd_finish_kernel<<<fgrid, kSsdThreads, 0, s>>>(m, l.segs_max, xbc, rows, y, sc);
  count_launch();
  return cuda_rc(cudaGetLastError());
}

int launch_ssd_out(int dtype, const kllm_seq_ssd& m, const float* y, const float* proj, float eps, void* out, int T,
                   cudaStream_t s) {
  if (m.norm_groups <= 0 || ssd_inner(m) % m.norm_groups) return KLLM_E_INVALID;
  const int n = ssd_inner(m) / m.norm_groups;
  const int threads = n >= 1024 ? 256 : 128;
  const dim3 grid(T, m.norm_groups);
  if (dtype == KLLM_SEQ_F32) ssd_out_kernel<float><<<grid, threads, 0, s>>>(m, y, proj, eps, static_cast<float*>(out));
  else if (dtype == KLLM_SEQ_BF16)
    ssd_out_kernel<__nv_bfloat16><<<grid, threads, 0, s>>>(m, y, proj, eps, static_cast<__nv_bfloat16*>(out));
  else return KLLM_E_INVALID;
  return done();
}

}  // namespace seq
}  // namespace kllm
