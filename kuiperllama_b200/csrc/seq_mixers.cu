// Kernels of the mixers that keep something other than per-head keys and values, and of the dense feed-forward:
//
//   attention through a latent   latent_prepare (RMS norms of the two down-projections, rotation of the shared key part,
//                                scatter of [latent | rotated part] into the pages, gates), latent_absorb (a head's plain
//                                query dimensions carried into the latent space, W_uk^T q, and the rotation of its rotated
//                                dimensions), latent_expand (W_uv on the weighted sum of latents).  Between absorb and expand
//                                the paged attention kernel of seq_kernels.cu runs with one key/value "head" of
//                                kv_rank + rot_dim key and kv_rank value dimensions that every query head shares.
//   linear attention             the decayed-state recurrence, chunk by chunk, and its output norm with the sigmoid gate
//   activations                  xIELU and squared ReLU between the two products of a dense feed-forward
//
// Positions and angles, norms, gates, decays and the recurrent state are fp32 in both compute types.
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <cstdint>

#include "seq_engine.h"

namespace kllm {
namespace seq {
namespace {

constexpr unsigned kAll = 0xffffffffu;

__device__ __forceinline__ float to_f(float v) { return v; }
__device__ __forceinline__ float to_f(__nv_bfloat16 v) { return __bfloat162float(v); }
template <typename AT> __device__ __forceinline__ AT from_f(float v);
template <> __device__ __forceinline__ float from_f<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 from_f<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(kAll, v, o);
  return v;
}
__device__ __forceinline__ float block_sum(float v, float* red) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
  v = warp_sum(v);
  __syncthreads();
  if (lane == 0) red[warp] = v;
  __syncthreads();
  float t = 0.f;
  for (int i = 0; i < nw; ++i) t += red[i];
  return t;
}
__device__ __forceinline__ float sigmoidf(float z) { return 1.0f / (1.0f + expf(-z)); }
__device__ __forceinline__ float siluf(float z) { return z / (1.0f + expf(-z)); }

// Rotary position: coordinate i < dims / 2 pairs with i + dims / 2; angle = pos * base^(-2 i / dims); coordinates past
// `dims` pass unchanged.  v: the vector before rotation.
__device__ __forceinline__ float rotated(const float* v, int i, int dims, float base, int pos) {
  if (i >= dims) return v[i];
  const int half = dims >> 1;
  const int j = i < half ? i : i - half;
  const float freq = exp2f(-2.0f * static_cast<float>(j) / static_cast<float>(dims) * log2f(base));
  float sn, cs;
  sincosf(static_cast<float>(pos) * freq, &sn, &cs);
  return i < half ? v[i] * cs - v[i + half] * sn : v[i] * cs + v[i - half] * sn;
}

// ---- latent attention: down-projections -> normed query latent, cache row, gates -----------------------------------------
template <typename AT>
__global__ void latent_prepare_kernel(LatentShape a, const float* __restrict__ proj, const float* __restrict__ q_norm_w,
                                      const float* __restrict__ kv_norm_w, float eps, const int32_t* __restrict__ tok_seq,
                                      const int32_t* __restrict__ tok_pos, AT* __restrict__ cq, float* __restrict__ gates,
                                      PagedKV kv, AT* __restrict__ c_rows, float* __restrict__ kr_rows) {
  __shared__ float red[33];
  const int t = blockIdx.x;
  const int stride = a.q_rank + a.kv_rank + a.rot_dim + a.heads;
  const float* row = proj + static_cast<size_t>(t) * stride;
  const int seq = tok_seq[t], pos = tok_pos[t];
  float ss = 0.f;
  for (int i = threadIdx.x; i < a.q_rank; i += blockDim.x) ss += row[i] * row[i];
  const float rq = 1.0f / sqrtf(block_sum(ss, red) / static_cast<float>(a.q_rank) + eps);
  for (int i = threadIdx.x; i < a.q_rank; i += blockDim.x)
    cq[static_cast<size_t>(t) * a.q_rank + i] = from_f<AT>(row[i] * rq * q_norm_w[i]);
  const float* c = row + a.q_rank;
  ss = 0.f;
  for (int i = threadIdx.x; i < a.kv_rank; i += blockDim.x) ss += c[i] * c[i];
  const float rc = 1.0f / sqrtf(block_sum(ss, red) / static_cast<float>(a.kv_rank) + eps);
  const int page = kv.table[static_cast<size_t>(seq) * kv.table_stride + pos / kv.page];
  AT* dst = static_cast<AT*>(kv.k) + (static_cast<size_t>(page) * kv.page + pos % kv.page) * kv.k_row;
  for (int i = threadIdx.x; i < a.kv_rank; i += blockDim.x) {
    const AT v = from_f<AT>(c[i] * rc * kv_norm_w[i]);
    dst[i] = v;
    if (c_rows) c_rows[static_cast<size_t>(t) * a.kv_rank + i] = v;
  }
  const float* kr = c + a.kv_rank;
  for (int i = threadIdx.x; i < a.rot_dim; i += blockDim.x) {
    const float v = rotated(kr, i, a.rope_dims, a.rope_base, pos);
    dst[a.kv_rank + i] = from_f<AT>(v);
    if (kr_rows) kr_rows[static_cast<size_t>(t) * a.rot_dim + i] = v;
  }
  const float* g = kr + a.rot_dim;
  for (int h = threadIdx.x; h < a.heads; h += blockDim.x) gates[static_cast<size_t>(t) * a.heads + h] = sigmoidf(g[h]);
}

// ---- latent attention: queries into the latent space --------------------------------------------------------------------
// One CTA: kAbsTokens tokens of one head.  qa[t, h, r] = sum_d q[t, h, d] * W_uk[h * dim + d, r]: thread r walks the
// rows d of the head's block of W_uk (coalesced over r) with the tokens' queries in shared memory.
constexpr int kAbsTokens = 16;
template <typename AT>
__global__ void latent_absorb_kernel(LatentShape a, const float* __restrict__ q, const AT* __restrict__ w_uk,
                                     const int32_t* __restrict__ tok_pos, float* __restrict__ qa, int T) {
  extern __shared__ float qs[];  // [kAbsTokens][dim + rot_dim]
  const int h = blockIdx.y, t0 = blockIdx.x * kAbsTokens;
  const int n = min(kAbsTokens, T - t0);
  const int dq = a.dim + a.rot_dim, dl = a.kv_rank + a.rot_dim;
  for (int i = threadIdx.x; i < n * dq; i += blockDim.x)
    qs[i] = q[(static_cast<size_t>(t0 + i / dq) * a.heads + h) * dq + i % dq];
  __syncthreads();
  const AT* w = w_uk + static_cast<size_t>(h) * a.dim * a.kv_rank;
  // blockIdx.z: a slice of the latent coordinates, so that a step of few tokens still spreads over many SMs
  for (int r = blockIdx.z * blockDim.x + threadIdx.x; r < a.kv_rank; r += gridDim.z * blockDim.x) {
    float acc[kAbsTokens];
#pragma unroll
    for (int j = 0; j < kAbsTokens; ++j) acc[j] = 0.f;
#pragma unroll 8
    for (int d = 0; d < a.dim; ++d) {
      const float wv = to_f(w[static_cast<size_t>(d) * a.kv_rank + r]);
#pragma unroll
      for (int j = 0; j < kAbsTokens; ++j) acc[j] = fmaf(qs[j * dq + d], wv, acc[j]);
    }
#pragma unroll
    for (int j = 0; j < kAbsTokens; ++j)
      if (j < n) qa[(static_cast<size_t>(t0 + j) * a.heads + h) * dl + r] = acc[j];
  }
  if (blockIdx.z != 0) return;
  for (int i = threadIdx.x; i < n * a.rot_dim; i += blockDim.x) {
    const int j = i / a.rot_dim, c = i % a.rot_dim;
    qa[(static_cast<size_t>(t0 + j) * a.heads + h) * dl + a.kv_rank + c] =
        rotated(qs + j * dq + a.dim, c, a.rope_dims, a.rope_base, tok_pos[t0 + j]);
  }
}

// ---- latent attention with per-head keys and values (prompt steps on the tensor cores) ---------------------------------------
// q [T, heads, dim + rot_dim] fp32 -> the same in the compute type with the rotated part rotated
template <typename AT>
__global__ void latent_pack_q_kernel(LatentShape a, const float* __restrict__ q, const int32_t* __restrict__ tok_pos,
                                     AT* __restrict__ out) {
  const int t = blockIdx.x, dq = a.dim + a.rot_dim;
  const int pos = tok_pos[t];
  const float* row = q + static_cast<size_t>(t) * a.heads * dq;
  for (int i = threadIdx.x; i < a.heads * dq; i += blockDim.x) {
    const int h = i / dq, d = i % dq;
    const float v = d < a.dim ? row[i] : rotated(row + h * dq + a.dim, d - a.dim, a.rope_dims, a.rope_base, pos);
    out[static_cast<size_t>(t) * a.heads * dq + i] = from_f<AT>(v);
  }
}
// kp [T, heads * dim] fp32 (W_uk c) and kr [T, rot_dim] (rotated, shared by the heads) -> k [T, heads, dim + rot_dim];
// vp [T, heads * vdim] fp32 (W_uv c) -> v, both in the compute type
template <typename AT>
__global__ void latent_pack_kv_kernel(LatentShape a, const float* __restrict__ kp, const float* __restrict__ kr,
                                      const float* __restrict__ vp, AT* __restrict__ k, AT* __restrict__ v) {
  const int t = blockIdx.x, dq = a.dim + a.rot_dim;
  for (int i = threadIdx.x; i < a.heads * dq; i += blockDim.x) {
    const int h = i / dq, d = i % dq;
    const float x = d < a.dim ? kp[(static_cast<size_t>(t) * a.heads + h) * a.dim + d]
                              : kr[static_cast<size_t>(t) * a.rot_dim + d - a.dim];
    k[static_cast<size_t>(t) * a.heads * dq + i] = from_f<AT>(x);
  }
  for (int i = threadIdx.x; i < a.heads * a.vdim; i += blockDim.x)
    v[static_cast<size_t>(t) * a.heads * a.vdim + i] = from_f<AT>(vp[static_cast<size_t>(t) * a.heads * a.vdim + i]);
}

// ---- latent attention: weighted sums of latents -> per-head values ---------------------------------------------------------
// One CTA: kAbsTokens tokens of one head; a warp per output row of W_uv's head block, dotted with every token's latent sum.
template <typename AT>
__global__ void latent_expand_kernel(LatentShape a, const float* __restrict__ ol, const AT* __restrict__ w_uv,
                                     AT* __restrict__ out, int T) {
  extern __shared__ float ls[];  // [kAbsTokens][kv_rank]
  const int h = blockIdx.y, t0 = blockIdx.x * kAbsTokens;
  const int n = min(kAbsTokens, T - t0);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
  for (int i = threadIdx.x; i < kAbsTokens * a.kv_rank; i += blockDim.x) {
    const int j = i / a.kv_rank;
    ls[i] = j < n ? ol[(static_cast<size_t>(t0 + j) * a.heads + h) * a.kv_rank + i % a.kv_rank] : 0.f;
  }
  __syncthreads();
  for (int f = warp; f < a.vdim; f += nw) {
    const AT* w = w_uv + (static_cast<size_t>(h) * a.vdim + f) * a.kv_rank;
    float acc[kAbsTokens];
#pragma unroll
    for (int j = 0; j < kAbsTokens; ++j) acc[j] = 0.f;
    for (int r = lane; r < a.kv_rank; r += 32) {
      const float wv = to_f(w[r]);
#pragma unroll
      for (int j = 0; j < kAbsTokens; ++j) acc[j] = fmaf(ls[j * a.kv_rank + r], wv, acc[j]);
    }
#pragma unroll
    for (int j = 0; j < kAbsTokens; ++j) {
      const float v = warp_sum(acc[j]);
      if (lane == 0 && j < n) out[(static_cast<size_t>(t0 + j) * a.heads + h) * a.vdim + f] = from_f<AT>(v);
    }
  }
}

// The same for steps of single tokens, fused with the merge of the key splits: a CTA per (token, head) joins the splits'
// (max, sum, unnormalised latent sums), adds the sink to the denominator, applies the gate, and multiplies by the head's
// block of W_uv -- the merged latent sum never leaves shared memory.
template <typename AT>
__global__ void latent_merge_expand_kernel(LatentShape a, int splits, const float* __restrict__ ws,
                                           const float* __restrict__ gates, const float* __restrict__ sink,
                                           const AT* __restrict__ w_uv, AT* __restrict__ out) {
  extern __shared__ float ls[];  // [kv_rank]
  const size_t th = blockIdx.x;  // t * heads + h
  const int h = static_cast<int>(th % a.heads);
  const int pstride = a.kv_rank + 2;
  const float* p = ws + th * splits * pstride;
  float M = sink ? sink[h] : -INFINITY;
  for (int s = 0; s < splits; ++s) M = fmaxf(M, p[s * pstride]);
  float L = sink ? expf(sink[h] - M) : 0.f;
  for (int s = 0; s < splits; ++s) {
    const float m = p[s * pstride];
    if (m > -INFINITY) L += p[s * pstride + 1] * expf(m - M);
  }
  const float g = (gates ? gates[th] : 1.0f) / L;
  for (int d = threadIdx.x; d < a.kv_rank; d += blockDim.x) {
    float o = 0.f;
    for (int s = 0; s < splits; ++s) {
      const float m = p[s * pstride];
      if (m > -INFINITY) o += p[s * pstride + 2 + d] * expf(m - M);
    }
    ls[d] = o * g;
  }
  __syncthreads();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
  for (int f = warp; f < a.vdim; f += nw) {
    const AT* w = w_uv + (static_cast<size_t>(h) * a.vdim + f) * a.kv_rank;
    float acc = 0.f;
    for (int r = lane; r < a.kv_rank; r += 32) acc = fmaf(ls[r], to_f(w[r]), acc);
    acc = warp_sum(acc);
    if (lane == 0) out[th * a.vdim + f] = from_f<AT>(acc);
  }
}

// ---- linear attention ---------------------------------------------------------------------------------------------------------
// Per head, with decay l:  S_t = l S_(t-1) + k_t v_t^T,  o_t = S_t^T q_t.  Columns of S are independent, so one CTA takes
// one entry, one head and kLinCols value columns, and walks the entry's tokens in chunks of kLinChunk.  For a chunk of n
// tokens with the state S before it:
//     o_i = l^(i+1) S^T q_i + sum_(j <= i) l^(i-j) (q_i . k_j) v_j
//     S  <- l^n S + sum_j l^(n-1-j) k_j v_j^T
// Only non-negative powers of l appear.  Everything is fp32; silu is applied to q, k, v as they are loaded.
// Fill shared memory from global memory with U loads of a thread in flight before the first is used: the tiles of these
// kernels are small and each CTA waits for them once, so the loop is bound by load latency, not by bandwidth.
template <int U, typename Load, typename Store>
__device__ __forceinline__ void staged_fill(int total, Load load, Store store) {
  for (int i0 = threadIdx.x; i0 < total; i0 += blockDim.x * U) {
    float v[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int i = i0 + u * blockDim.x;
      v[u] = i < total ? load(i) : 0.f;
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int i = i0 + u * blockDim.x;
      if (i < total) store(i, v[u]);
    }
  }
}

constexpr int kLinChunk = 32;
constexpr int kLinCols = 32;
constexpr int kLinThreads = 128;
constexpr int kLinParallelFrom = 2 * kLinChunk;  // steps whose longest entry has more tokens take the chunk-parallel kernels

__global__ void __launch_bounds__(kLinThreads)
linear_attention_kernel(int heads, int dim, int vdim, const float* __restrict__ decay, const float* __restrict__ proj,
                        float* __restrict__ state, const int32_t* __restrict__ ent_first,
                        const int32_t* __restrict__ ent_count, const int32_t* __restrict__ ent_seq,
                        const int32_t* __restrict__ ent_pos0, float* __restrict__ o) {
  extern __shared__ float sm[];
  const int e = blockIdx.z, h = blockIdx.y, c0 = blockIdx.x * kLinCols;
  const int count = ent_count[e], first = ent_first[e], seq = ent_seq[e];
  const int cols = min(kLinCols, vdim - c0);
  const int dp = dim + 1;
  float* Qs = sm;                         // [chunk][dp]
  float* Ks = Qs + kLinChunk * dp;        // [chunk][dp]
  float* Vs = Ks + kLinChunk * dp;        // [chunk][kLinCols]
  float* As = Vs + kLinChunk * kLinCols;  // [chunk][chunk + 1]
  float* Ss = As + kLinChunk * (kLinChunk + 1);  // [dim][kLinCols]
  float* pw = Ss + dim * kLinCols;        // [chunk + 1] powers of the decay
  const int tid = threadIdx.x;
  const float lam = decay[h];
  const float llog = logf(lam);
  if (tid <= kLinChunk) pw[tid] = tid == 0 ? 1.0f : expf(llog * static_cast<float>(tid));
  float* sg = state + ((static_cast<size_t>(seq) * heads + h) * dim) * vdim;
  const bool fresh = ent_pos0[e] == 0;
  staged_fill<8>(dim * kLinCols,
                 [&](int i) { return (!fresh && i % kLinCols < cols) ? sg[static_cast<size_t>(i / kLinCols) * vdim + c0 + i % kLinCols] : 0.f; },
                 [&](int i, float v) { Ss[i] = v; });
  const int qn = heads * dim, vn = heads * vdim;
  const int stride = 2 * qn + 2 * vn;
  for (int base = 0; base < count; base += kLinChunk) {
    const int n = min(kLinChunk, count - base);
    __syncthreads();  // the previous chunk's tiles are no longer read; Ss / pw are written
    const float* rows = proj + static_cast<size_t>(first + base) * stride;
    staged_fill<8>(n * dim, [&](int i) { return rows[static_cast<size_t>(i / dim) * stride + h * dim + i % dim]; },
                   [&](int i, float v) { Qs[(i / dim) * dp + i % dim] = siluf(v); });
    staged_fill<8>(n * dim, [&](int i) { return rows[static_cast<size_t>(i / dim) * stride + qn + h * dim + i % dim]; },
                   [&](int i, float v) { Ks[(i / dim) * dp + i % dim] = siluf(v); });
    staged_fill<8>(n * kLinCols,
                   [&](int i) { return i % kLinCols < cols ? rows[static_cast<size_t>(i / kLinCols) * stride + 2 * qn + h * vdim + c0 + i % kLinCols] : 0.f; },
                   [&](int i, float v) { Vs[i] = siluf(v); });
    __syncthreads();
    for (int i = tid; i < n * n; i += kLinThreads) {  // decayed scores inside the chunk
      const int r = i / n, j = i % n;
      float acc = 0.f;
      if (j <= r) {
        for (int d = 0; d < dim; ++d) acc = fmaf(Qs[r * dp + d], Ks[j * dp + d], acc);
        acc *= pw[r - j];
      }
      As[r * (kLinChunk + 1) + j] = acc;
    }
    __syncthreads();
    for (int i = tid; i < n * kLinCols; i += kLinThreads) {  // outputs
      const int r = i / kLinCols, c = i % kLinCols;
      float carry = 0.f;
      for (int d = 0; d < dim; ++d) carry = fmaf(Qs[r * dp + d], Ss[d * kLinCols + c], carry);
      float acc = carry * pw[r + 1];
      for (int j = 0; j <= r; ++j) acc = fmaf(As[r * (kLinChunk + 1) + j], Vs[j * kLinCols + c], acc);
      if (c < cols) o[static_cast<size_t>(first + base + r) * vn + h * vdim + c0 + c] = acc;
    }
    __syncthreads();
    for (int i = tid; i < dim * kLinCols; i += kLinThreads) {  // the state after the chunk
      const int d = i / kLinCols, c = i % kLinCols;
      float acc = Ss[i] * pw[n];
      for (int j = 0; j < n; ++j) acc = fmaf(Ks[j * dp + d] * pw[n - 1 - j], Vs[j * kLinCols + c], acc);
      Ss[i] = acc;
    }
  }
  __syncthreads();
  for (int i = tid; i < dim * kLinCols; i += kLinThreads) {
    const int d = i / kLinCols, c = i % kLinCols;
    if (c < cols) sg[static_cast<size_t>(d) * vdim + c0 + c] = Ss[i];
  }
}

// ---- linear attention over long entries: chunks in parallel ---------------------------------------------------------------
// The recurrence above is sequential only in the state.  For entries of many chunks it is cut into three kernels:
//   linear_chunk_sums_kernel   every chunk on its own: U_c = sum_j l^(n-1-j) k_j v_j^T                       (parallel)
//   linear_scan_kernel         S_before(c) in place of U_c, chunk after chunk: S <- l^n S + U_c; the final state  (per element)
//   linear_chunk_out_kernel    every chunk on its own: o_i = l^(i+1) S_before^T q_i + decayed scores inside the chunk
// Chunk j of entry e lives in slot (first_e + j * chunk) / chunk + e of the scratch buffer [slots][heads][dim][vdim].
__device__ __forceinline__ size_t chunk_slot(int first, int base, int e) { return static_cast<size_t>((first + base) / kLinChunk + e); }

__host__ __device__ inline int lin_dp(int dim) { return ((dim + 3) & ~3) + 4; }  // row stride of Qs / Ks: 16-byte rows, odd in 16-byte units for dim % 8 == 0

// A thread keeps 8 consecutive key coordinates of one value column: two 16-byte broadcast loads and one column load
// feed 8 multiply-adds.
__global__ void __launch_bounds__(kLinThreads)
linear_chunk_sums_kernel(int heads, int dim, int vdim, const float* __restrict__ decay, const float* __restrict__ proj,
                         const int32_t* __restrict__ ent_first, const int32_t* __restrict__ ent_count,
                         float* __restrict__ sums) {
  extern __shared__ __align__(16) float sm[];
  const int e = blockIdx.z, h = blockIdx.y;
  const int n_slices = (vdim + kLinCols - 1) / kLinCols;
  const int chunk = blockIdx.x / n_slices, c0 = (blockIdx.x % n_slices) * kLinCols;
  const int count = ent_count[e], first = ent_first[e], base = chunk * kLinChunk;
  if (base >= count) return;
  const int n = min(kLinChunk, count - base);
  const int cols = min(kLinCols, vdim - c0);
  const int d8 = (dim + 7) & ~7, dp = lin_dp(dim);
  float* Ks = sm;                       // [chunk][dp], already times l^(n-1-j); zeros from dim to d8
  float* Vs = Ks + kLinChunk * dp;      // [chunk][kLinCols]
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const float llog = logf(decay[h]);
  const int qn = heads * dim, vn = heads * vdim, stride = 2 * qn + 2 * vn;
  const float* rows = proj + static_cast<size_t>(first + base) * stride;
  staged_fill<8>(n * d8,
                 [&](int i) { return i % d8 < dim ? rows[static_cast<size_t>(i / d8) * stride + qn + h * dim + i % d8] : 0.f; },
                 [&](int i, float v) {
                   const int j = i / d8;
                   const float w = n - 1 - j == 0 ? 1.0f : expf(llog * static_cast<float>(n - 1 - j));
                   Ks[j * dp + i % d8] = siluf(v) * w;
                 });
  staged_fill<8>(n * kLinCols,
                 [&](int i) { return i % kLinCols < cols ? rows[static_cast<size_t>(i / kLinCols) * stride + 2 * qn + h * vdim + c0 + i % kLinCols] : 0.f; },
                 [&](int i, float v) { Vs[i] = siluf(v); });
  __syncthreads();
  float* out = sums + (chunk_slot(first, base, e) * heads + h) * dim * vdim;
  for (int d0 = warp * 8; d0 < d8; d0 += (kLinThreads / 32) * 8) {
    float acc[8];
#pragma unroll
    for (int k = 0; k < 8; ++k) acc[k] = 0.f;
    for (int j = 0; j < n; ++j) {
      const float v = Vs[j * kLinCols + lane];
      const float4 a = *reinterpret_cast<const float4*>(Ks + j * dp + d0);
      const float4 b = *reinterpret_cast<const float4*>(Ks + j * dp + d0 + 4);
      acc[0] = fmaf(a.x, v, acc[0]), acc[1] = fmaf(a.y, v, acc[1]), acc[2] = fmaf(a.z, v, acc[2]), acc[3] = fmaf(a.w, v, acc[3]);
      acc[4] = fmaf(b.x, v, acc[4]), acc[5] = fmaf(b.y, v, acc[5]), acc[6] = fmaf(b.z, v, acc[6]), acc[7] = fmaf(b.w, v, acc[7]);
    }
#pragma unroll
    for (int k = 0; k < 8; ++k)
      if (d0 + k < dim && lane < cols) out[static_cast<size_t>(d0 + k) * vdim + c0 + lane] = acc[k];
  }
}

__global__ void linear_scan_kernel(int heads, int dim, int vdim, const float* __restrict__ decay, float* __restrict__ state,
                                   const int32_t* __restrict__ ent_first, const int32_t* __restrict__ ent_count,
                                   const int32_t* __restrict__ ent_seq, const int32_t* __restrict__ ent_pos0,
                                   float* __restrict__ sums) {
  const int e = blockIdx.z, h = blockIdx.y;
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= dim * vdim) return;
  const int count = ent_count[e], first = ent_first[e];
  const float llog = logf(decay[h]);
  const float full = expf(llog * static_cast<float>(kLinChunk));
  float* sg = state + (static_cast<size_t>(ent_seq[e]) * heads + h) * dim * vdim + i;
  float s = ent_pos0[e] == 0 ? 0.f : *sg;
  // the chunk sums are fetched eight chunks ahead: the loads do not depend on one another, only the sums do
  constexpr int U = 8;
  for (int base = 0; base < count; base += U * kLinChunk) {
    float add[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int b = base + u * kLinChunk;
      add[u] = b < count ? sums[(chunk_slot(first, b, e) * heads + h) * dim * vdim + i] : 0.f;
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int b = base + u * kLinChunk;
      if (b >= count) break;
      const int n = min(kLinChunk, count - b);
      sums[(chunk_slot(first, b, e) * heads + h) * dim * vdim + i] = s;
      s = fmaf(s, n == kLinChunk ? full : expf(llog * static_cast<float>(n)), add[u]);
    }
  }
  *sg = s;
}

// Each thread keeps kLinChunk / warps rows (warp + warps * k) of one column: a 16-byte broadcast load brings four coordinates
// of a row.  Eight warps per CTA: the shared-memory tiles allow few CTAs per SM, so the warps have to come from the CTA.  Rows and coordinates past the chunk are zero-filled.
constexpr int kLinAs = kLinChunk + 4;

constexpr int kLinOutThreads = 256, kLinOutWarps = kLinOutThreads / 32;
__global__ void __launch_bounds__(kLinOutThreads)
linear_chunk_out_kernel(int heads, int dim, int vdim, const float* __restrict__ decay, const float* __restrict__ proj,
                        const int32_t* __restrict__ ent_first, const int32_t* __restrict__ ent_count,
                        const float* __restrict__ sums, float* __restrict__ o) {
  extern __shared__ __align__(16) float sm[];
  const int e = blockIdx.z, h = blockIdx.y;
  const int n_slices = (vdim + kLinCols - 1) / kLinCols;
  const int chunk = blockIdx.x / n_slices, c0 = (blockIdx.x % n_slices) * kLinCols;
  const int count = ent_count[e], first = ent_first[e], base = chunk * kLinChunk;
  if (base >= count) return;
  const int n = min(kLinChunk, count - base);
  const int cols = min(kLinCols, vdim - c0);
  const int d4 = (dim + 3) & ~3, dp = lin_dp(dim);
  float* Qs = sm;                          // [chunk][dp]
  float* Ks = Qs + kLinChunk * dp;         // [chunk][dp]
  float* Vs = Ks + kLinChunk * dp;         // [chunk][kLinCols]
  float* As = Vs + kLinChunk * kLinCols;   // [chunk][kLinAs]
  float* Ss = As + kLinChunk * kLinAs;     // [d4][kLinCols]
  float* pw = Ss + d4 * kLinCols;          // [chunk + 1]
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const float llog = logf(decay[h]);
  if (tid <= kLinChunk) pw[tid] = tid == 0 ? 1.0f : expf(llog * static_cast<float>(tid));
  const float* sb = sums + (chunk_slot(first, base, e) * heads + h) * dim * vdim;
  staged_fill<8>(d4 * kLinCols,
                 [&](int i) { return (i / kLinCols < dim && i % kLinCols < cols) ? sb[static_cast<size_t>(i / kLinCols) * vdim + c0 + i % kLinCols] : 0.f; },
                 [&](int i, float v) { Ss[i] = v; });
  const int qn = heads * dim, vn = heads * vdim, stride = 2 * qn + 2 * vn;
  const float* rows = proj + static_cast<size_t>(first + base) * stride;
  // silu(0) = 0: rows and coordinates past the chunk load as zeros
  staged_fill<8>(kLinChunk * d4,
                 [&](int i) { return (i / d4 < n && i % d4 < dim) ? rows[static_cast<size_t>(i / d4) * stride + h * dim + i % d4] : 0.f; },
                 [&](int i, float v) { Qs[(i / d4) * dp + i % d4] = siluf(v); });
  staged_fill<8>(kLinChunk * d4,
                 [&](int i) { return (i / d4 < n && i % d4 < dim) ? rows[static_cast<size_t>(i / d4) * stride + qn + h * dim + i % d4] : 0.f; },
                 [&](int i, float v) { Ks[(i / d4) * dp + i % d4] = siluf(v); });
  staged_fill<8>(kLinChunk * kLinCols,
                 [&](int i) { return (i / kLinCols < n && i % kLinCols < cols) ? rows[static_cast<size_t>(i / kLinCols) * stride + 2 * qn + h * vdim + c0 + i % kLinCols] : 0.f; },
                 [&](int i, float v) { Vs[i] = siluf(v); });
  __syncthreads();
  constexpr int R = kLinChunk / kLinOutWarps;  // rows per thread
  {  // decayed scores inside the chunk: lane = key j, rows warp + 8 k
    float acc[R];
#pragma unroll
    for (int k = 0; k < R; ++k) acc[k] = 0.f;
    for (int d = 0; d < d4; d += 4) {
      const float4 kv = *reinterpret_cast<const float4*>(Ks + lane * dp + d);
#pragma unroll
      for (int k = 0; k < R; ++k) {
        const float4 qv = *reinterpret_cast<const float4*>(Qs + (warp + kLinOutWarps * k) * dp + d);
        acc[k] = fmaf(qv.x, kv.x, fmaf(qv.y, kv.y, fmaf(qv.z, kv.z, fmaf(qv.w, kv.w, acc[k]))));
      }
    }
#pragma unroll
    for (int k = 0; k < R; ++k) {
      const int r = warp + kLinOutWarps * k;
      As[r * kLinAs + lane] = (lane <= r && r < n) ? acc[k] * pw[r - lane] : 0.f;
    }
  }
  __syncthreads();
  {  // outputs: lane = column, rows warp + 8 k
    float acc[R];
#pragma unroll
    for (int k = 0; k < R; ++k) acc[k] = 0.f;
    for (int d = 0; d < d4; d += 4) {
      const float s0 = Ss[d * kLinCols + lane], s1 = Ss[(d + 1) * kLinCols + lane], s2 = Ss[(d + 2) * kLinCols + lane],
                  s3 = Ss[(d + 3) * kLinCols + lane];
#pragma unroll
      for (int k = 0; k < R; ++k) {
        const float4 qv = *reinterpret_cast<const float4*>(Qs + (warp + kLinOutWarps * k) * dp + d);
        acc[k] = fmaf(qv.x, s0, fmaf(qv.y, s1, fmaf(qv.z, s2, fmaf(qv.w, s3, acc[k]))));
      }
    }
#pragma unroll
    for (int k = 0; k < R; ++k) acc[k] *= pw[min(warp + kLinOutWarps * k + 1, kLinChunk)];
    for (int j = 0; j < kLinChunk; j += 4) {
      const float v0 = Vs[j * kLinCols + lane], v1 = Vs[(j + 1) * kLinCols + lane], v2 = Vs[(j + 2) * kLinCols + lane],
                  v3 = Vs[(j + 3) * kLinCols + lane];
#pragma unroll
      for (int k = 0; k < R; ++k) {
        const float4 av = *reinterpret_cast<const float4*>(As + (warp + kLinOutWarps * k) * kLinAs + j);
        acc[k] = fmaf(av.x, v0, fmaf(av.y, v1, fmaf(av.z, v2, fmaf(av.w, v3, acc[k]))));
      }
    }
#pragma unroll
    for (int k = 0; k < R; ++k) {
      const int r = warp + kLinOutWarps * k;
      if (r < n && lane < cols) o[static_cast<size_t>(first + base + r) * vn + h * vdim + c0 + lane] = acc[k];
    }
  }
}

template <typename AT>
__global__ void linear_out_kernel(int qn, int vn, const float* __restrict__ o, const float* __restrict__ proj,
                                  const float* __restrict__ norm_w, float eps, AT* __restrict__ out) {
  __shared__ float red[33];
  const int t = blockIdx.x;
  const float* row = o + static_cast<size_t>(t) * vn;
  const float* g = proj + static_cast<size_t>(t) * (2 * qn + 2 * vn) + 2 * qn + vn;
  float ss = 0.f;
  for (int i = threadIdx.x; i < vn; i += blockDim.x) ss += row[i] * row[i];
  const float rinv = 1.0f / sqrtf(block_sum(ss, red) / static_cast<float>(vn) + eps);
  for (int i = threadIdx.x; i < vn; i += blockDim.x)
    out[static_cast<size_t>(t) * vn + i] = from_f<AT>(row[i] * rinv * norm_w[i] * sigmoidf(g[i]));
}

// ---- activations ---------------------------------------------------------------------------------------------------------------
template <typename AT>
__global__ void activation_kernel(int act, float a, float b, const float* __restrict__ z, AT* __restrict__ out, size_t n) {
  const size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const float v = z[i];
  float r;
  if (act == KLLM_SEQ_ACT_XIELU) r = v > 0.f ? a * v * v + 0.5f * v : b * (expm1f(v) - v) + 0.5f * v;
  else r = v > 0.f ? v * v : 0.f;
  out[i] = from_f<AT>(r);
}

__global__ void scale_kernel(float* __restrict__ v, float scale, float cap, size_t n) {
  const size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= n) return;
  float z = v[i] * scale;
  if (cap > 0.f) z = cap * tanhf(z / cap);
  v[i] = z;
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
}  // namespace

int launch_latent_prepare(int dtype, const LatentShape& a, const float* proj, const float* q_norm_w, const float* kv_norm_w,
                          float eps, const int32_t* tok_seq, const int32_t* tok_pos, void* cq, float* gates,
                          const PagedKV& kv, void* c_rows, float* kr_rows, int T, cudaStream_t s) {
  KLLM_SEQ_DISPATCH(dtype, (latent_prepare_kernel<AT><<<T, 128, 0, s>>>(a, proj, q_norm_w, kv_norm_w, eps, tok_seq, tok_pos,
                                                                       static_cast<AT*>(cq), gates, kv,
                                                                       static_cast<AT*>(c_rows), kr_rows)));
  return done();
}

int launch_latent_pack_q(int dtype, const LatentShape& a, const float* q, const int32_t* tok_pos, void* out, int T,
                         cudaStream_t s) {
  KLLM_SEQ_DISPATCH(dtype, (latent_pack_q_kernel<AT><<<T, 256, 0, s>>>(a, q, tok_pos, static_cast<AT*>(out))));
  return done();
}

int launch_latent_pack_kv(int dtype, const LatentShape& a, const float* kp, const float* kr, const float* vp, void* k, void* v,
                          int T, cudaStream_t s) {
  KLLM_SEQ_DISPATCH(dtype, (latent_pack_kv_kernel<AT><<<T, 256, 0, s>>>(a, kp, kr, vp, static_cast<AT*>(k),
                                                                       static_cast<AT*>(v))));
  return done();
}

int launch_latent_absorb(int dtype, const LatentShape& a, const float* q, const void* w_uk, const int32_t* tok_pos, float* qa,
                         int T, cudaStream_t s) {
  const size_t smem = static_cast<size_t>(kAbsTokens) * (a.dim + a.rot_dim) * sizeof(float);
  if (smem > 48 * 1024) return KLLM_E_UNSUPPORTED;
  // few tokens: 64 latent coordinates per CTA; many tokens: the whole latent (the queries are staged once per CTA)
  const int threads = T <= kAbsTokens ? 64 : (a.kv_rank <= 64 ? 64 : (a.kv_rank <= 128 ? 128 : 256));
  const dim3 grid((T + kAbsTokens - 1) / kAbsTokens, a.heads, (a.kv_rank + threads - 1) / threads);
  KLLM_SEQ_DISPATCH(dtype, (latent_absorb_kernel<AT><<<grid, threads, smem, s>>>(a, q, static_cast<const AT*>(w_uk), tok_pos,
                                                                                qa, T)));
  return done();
}

int launch_latent_merge_expand(int dtype, const LatentShape& a, int splits, const float* ws, const float* gates,
                               const float* sink, const void* w_uv, void* out, int T, cudaStream_t s) {
  const size_t smem = static_cast<size_t>(a.kv_rank) * sizeof(float);
  KLLM_SEQ_DISPATCH(dtype, (latent_merge_expand_kernel<AT><<<T * a.heads, 256, smem, s>>>(
                               a, splits, ws, gates, sink, static_cast<const AT*>(w_uv), static_cast<AT*>(out))));
  return done();
}

int launch_latent_expand(int dtype, const LatentShape& a, const float* ol, const void* w_uv, void* out, int T, cudaStream_t s) {
  const size_t smem = static_cast<size_t>(kAbsTokens) * a.kv_rank * sizeof(float);
  if (smem > 48 * 1024) return KLLM_E_UNSUPPORTED;
  const dim3 grid((T + kAbsTokens - 1) / kAbsTokens, a.heads);
  KLLM_SEQ_DISPATCH(dtype, (latent_expand_kernel<AT><<<grid, 256, smem, s>>>(a, ol, static_cast<const AT*>(w_uv),
                                                                            static_cast<AT*>(out), T)));
  return done();
}

size_t linear_attention_scratch_bytes(int heads, int dim, int vdim, int T, int n_entries, int max_count) {
  if (max_count <= kLinParallelFrom) return 0;
  return (static_cast<size_t>(T) / kLinChunk + n_entries + 1) * heads * dim * vdim * sizeof(float);
}

int launch_linear_attention(int heads, int dim, int vdim, const float* decay, const float* proj, float* state, int n_entries,
                            const int32_t* ent_first, const int32_t* ent_count, const int32_t* ent_seq,
                            const int32_t* ent_pos0, int max_count, float* scratch, float* o, cudaStream_t s) {
  const size_t smem = (2 * static_cast<size_t>(kLinChunk) * (dim + 1) + kLinChunk * kLinCols + kLinChunk * (kLinChunk + 1) +
                       static_cast<size_t>(dim) * kLinCols + kLinChunk + 1) * sizeof(float);
  if (smem > 200 * 1024) return KLLM_E_UNSUPPORTED;
  static size_t configured = 0;
  if (smem > 48 * 1024 && smem > configured) {
    const cudaError_t e = cudaFuncSetAttribute(linear_attention_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                               static_cast<int>(smem));
    if (e != cudaSuccess) return cuda_rc(e);
    configured = smem;
  }
  if (max_count > kLinParallelFrom && scratch != nullptr) {  // long entries: chunks in parallel
    const size_t smem_out = (2 * static_cast<size_t>(kLinChunk) * lin_dp(dim) + kLinChunk * kLinCols + kLinChunk * kLinAs +
                             static_cast<size_t>((dim + 3) & ~3) * kLinCols + kLinChunk + 4) * sizeof(float);
    static size_t configured_out = 0;
    if (smem_out > 48 * 1024 && smem_out > configured_out) {
      cudaError_t e = cudaFuncSetAttribute(linear_chunk_out_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                           static_cast<int>(smem_out));
      if (e == cudaSuccess)
        e = cudaFuncSetAttribute(linear_chunk_sums_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem_out));
      if (e != cudaSuccess) return cuda_rc(e);
      configured_out = smem_out;
    }
    const int n_slices = (vdim + kLinCols - 1) / kLinCols, chunks = (max_count + kLinChunk - 1) / kLinChunk;
    const dim3 grid(chunks * n_slices, heads, n_entries);
    const size_t smem_sums = (static_cast<size_t>(kLinChunk) * lin_dp(dim) + kLinChunk * kLinCols) * sizeof(float);
    linear_chunk_sums_kernel<<<grid, kLinThreads, smem_sums, s>>>(heads, dim, vdim, decay, proj, ent_first, ent_count, scratch);
    count_launch();
    const dim3 sgrid((dim * vdim + 127) / 128, heads, n_entries);
    linear_scan_kernel<<<sgrid, 128, 0, s>>>(heads, dim, vdim, decay, state, ent_first, ent_count, ent_seq, ent_pos0, scratch);
    count_launch();
    linear_chunk_out_kernel<<<grid, kLinOutThreads, smem_out, s>>>(heads, dim, vdim, decay, proj, ent_first, ent_count, scratch, o);
    return done();
  }
  const dim3 grid((vdim + kLinCols - 1) / kLinCols, heads, n_entries);
  linear_attention_kernel<<<grid, kLinThreads, smem, s>>>(heads, dim, vdim, decay, proj, state, ent_first, ent_count, ent_seq,
                                                         ent_pos0, o);
  return done();
}

int launch_linear_out(int dtype, int heads, int dim, int vdim, const float* o, const float* proj, const float* norm_w, float eps,
                      void* out, int T, cudaStream_t s) {
  KLLM_SEQ_DISPATCH(dtype, (linear_out_kernel<AT><<<T, 128, 0, s>>>(heads * dim, heads * vdim, o, proj, norm_w, eps,
                                                                   static_cast<AT*>(out))));
  return done();
}

int launch_activation(int dtype, int act, float a, float b, const float* z, void* out, size_t n, cudaStream_t s) {
  if (act != KLLM_SEQ_ACT_XIELU && act != KLLM_SEQ_ACT_RELU2) return KLLM_E_UNSUPPORTED;
  const unsigned blocks = static_cast<unsigned>((n + 255) / 256);
  KLLM_SEQ_DISPATCH(dtype, (activation_kernel<AT><<<blocks, 256, 0, s>>>(act, a, b, z, static_cast<AT*>(out), n)));
  return done();
}

int launch_scale(float* v, float scale, float cap, size_t n, cudaStream_t s) {
  scale_kernel<<<static_cast<unsigned>((n + 255) / 256), 256, 0, s>>>(v, scale == 0.f ? 1.0f : scale, cap, n);
  return done();
}

}  // namespace seq
}  // namespace kllm
