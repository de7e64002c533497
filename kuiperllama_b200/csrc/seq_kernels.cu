// Kernels of the sequence-batch engine other than the matrix products: embedding rows (with their norm), the fused
// residual / norm step (layer norm or RMS norm; token shift for single-token steps; router), the token shift over longer
// entries, query-key preparation with the scatter into the paged cache, causal paged attention (prompt tiles and single
// decode rows through the same kernel, keys split over CTAs, optional window, sink and fp32 queries), the softmax and the
// grouped sigmoid router with top-k selection, and the routed experts one (token, expert) pair at a time for steps of a
// few tokens.  The mixers with other kinds of memory (latents, recurrent state) are in seq_mixers.cu.
//
// Every kernel is a template on the compute type AT (float or __nv_bfloat16): what the matrix products read and
// write.  Norms, scores, softmax weights, router and residual are fp32 in both instantiations.
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <algorithm>

#include <cfloat>
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
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(kAll, v, o));
  return v;
}
// sum over the block; `red` holds one float per warp (+1).  Every thread gets the total.
__device__ __forceinline__ float block_sum(float v, float* red) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
  v = warp_sum(v);
  __syncthreads();  // `red` may still be read from the previous reduction
  if (lane == 0) red[warp] = v;
  __syncthreads();
  float t = 0.f;
  for (int i = 0; i < nw; ++i) t += red[i];
  return t;
}

// 16-byte vectors of the compute type, widened to fp32
template <typename AT> struct VecOf;
template <> struct VecOf<float> {
  static constexpr int N = 4;
  __device__ static __forceinline__ void load(const float* p, float* f) {
    const float4 v = *reinterpret_cast<const float4*>(p);
    f[0] = v.x, f[1] = v.y, f[2] = v.z, f[3] = v.w;
  }
};
template <> struct VecOf<__nv_bfloat16> {
  static constexpr int N = 8;
  __device__ static __forceinline__ void load(const __nv_bfloat16* p, float* f) {
    const uint4 v = *reinterpret_cast<const uint4*>(p);
    const uint32_t u[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      f[2 * i] = __uint_as_float(u[i] << 16);
      f[2 * i + 1] = __uint_as_float(u[i] & 0xffff0000u);
    }
  }
};

// dot of a weight row (compute type, global) with an fp32 vector in shared memory, spread over the warp's lanes;
// every lane returns the total.  Four 16-byte loads are in flight per lane before the first multiply.
template <typename AT>
__device__ __forceinline__ float warp_dot(const AT* __restrict__ w, const float* __restrict__ xs, int K, int lane) {
  constexpr int V = VecOf<AT>::N;
  float acc = 0.f;
  if ((K % V) == 0 && (reinterpret_cast<uintptr_t>(w) & 15) == 0) {
    for (int k = lane * V; k < K; k += 4 * 32 * V) {
      float f[4][V];
#pragma unroll
      for (int j = 0; j < 4; ++j)
        if (k + j * 32 * V < K) VecOf<AT>::load(w + k + j * 32 * V, f[j]);
#pragma unroll
      for (int j = 0; j < 4; ++j)
        if (k + j * 32 * V < K) {
#pragma unroll
          for (int i = 0; i < V; ++i) acc = fmaf(f[j][i], xs[k + j * 32 * V + i], acc);
        }
    }
  } else {
    for (int k = lane; k < K; k += 32) acc = fmaf(to_f(w[k]), xs[k], acc);
  }
  return warp_sum(acc);
}
// two rows against the same vector (a gate row and its up row)
template <typename AT>
__device__ __forceinline__ void warp_dot2(const AT* __restrict__ w0, const AT* __restrict__ w1,
                                          const float* __restrict__ xs, int K, int lane, float& r0, float& r1) {
  constexpr int V = VecOf<AT>::N;
  float a0 = 0.f, a1 = 0.f;
  if ((K % V) == 0 && ((reinterpret_cast<uintptr_t>(w0) | reinterpret_cast<uintptr_t>(w1)) & 15) == 0) {
    for (int k = lane * V; k < K; k += 2 * 32 * V) {
      float f[2][2][V];
#pragma unroll
      for (int j = 0; j < 2; ++j)
        if (k + j * 32 * V < K) {
          VecOf<AT>::load(w0 + k + j * 32 * V, f[j][0]);
          VecOf<AT>::load(w1 + k + j * 32 * V, f[j][1]);
        }
#pragma unroll
      for (int j = 0; j < 2; ++j)
        if (k + j * 32 * V < K) {
#pragma unroll
          for (int i = 0; i < V; ++i) {
            const float x = xs[k + j * 32 * V + i];
            a0 = fmaf(f[j][0][i], x, a0);
            a1 = fmaf(f[j][1][i], x, a1);
          }
        }
    }
  } else {
    for (int k = lane; k < K; k += 32) {
      a0 = fmaf(to_f(w0[k]), xs[k], a0);
      a1 = fmaf(to_f(w1[k]), xs[k], a1);
    }
  }
  r0 = warp_sum(a0);
  r1 = warp_sum(a1);
}

// ---- embedding ----------------------------------------------------------------------------------------------------
// mean and 1 / sqrt(var + eps) of a row in shared memory (layer norm), or 0 and 1 / sqrt(mean square + eps) (RMS norm)
__device__ __forceinline__ void row_stats(const float* buf, int W, int kind, float eps, float* red, float& mean, float& rstd) {
  const float inv_w = 1.0f / static_cast<float>(W);
  mean = 0.f;
  if (kind == KLLM_SEQ_NORM_LAYER) {
    float s = 0.f;
    for (int i = threadIdx.x; i < W; i += blockDim.x) s += buf[i];
    mean = block_sum(s, red) * inv_w;
  }
  float q = 0.f;
  for (int i = threadIdx.x; i < W; i += blockDim.x) {
    const float d = buf[i] - mean;
    q += d * d;
  }
  rstd = 1.0f / sqrtf(block_sum(q, red) * inv_w + eps);
}

template <typename AT>
__global__ void embed_kernel(const AT* __restrict__ table, const int32_t* __restrict__ tokens, float* __restrict__ x,
                             float* __restrict__ copy, NormW norm, float eps, float scale, int width) {
  extern __shared__ float buf[];
  __shared__ float red[33];
  const int t = blockIdx.x;
  const AT* row = table + static_cast<size_t>(tokens[t]) * width;
  if (norm.w == nullptr) {
    for (int i = threadIdx.x; i < width; i += blockDim.x) {
      const float v = to_f(row[i]) * scale;
      x[static_cast<size_t>(t) * width + i] = v;
      if (copy) copy[static_cast<size_t>(t) * width + i] = v;
    }
    return;
  }
  for (int i = threadIdx.x; i < width; i += blockDim.x) buf[i] = to_f(row[i]) * scale;
  __syncthreads();
  float mean, rstd;
  row_stats(buf, width, norm.kind, eps, red, mean, rstd);
  for (int i = threadIdx.x; i < width; i += blockDim.x) {
    const float v = (buf[i] - mean) * rstd * norm.w[i] + (norm.b ? norm.b[i] : 0.f);
    x[static_cast<size_t>(t) * width + i] = v;
    if (copy) copy[static_cast<size_t>(t) * width + i] = v;
  }
}

// ---- router ---------------------------------------------------------------------------------------------------------
// The warps of a CTA share the experts' logits of ONE token whose row `xs` is in shared memory in fp32 (a warp per
// expert row, fp32 weights); warp 0 then does the softmax over all experts and picks the top-k.  `z`: [experts] shared.
__device__ void route_token(const RouterArgs& r, const float* xs, float* z, int t, int width) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
  const int experts = r.experts, top = r.top;
  for (int e = warp; e < experts + (r.w_sg ? 1 : 0); e += nw) {
    const float* w = e < experts ? r.w_router + static_cast<size_t>(e) * width : r.w_sg;
    const float acc = warp_dot<float>(w, xs, width, lane);
    if (lane == 0) {
      if (e < experts) z[e] = acc + (r.bias ? r.bias[e] : 0.f);
      else r.sgate[t] = 1.0f / (1.0f + expf(-acc));
    }
  }
  __syncthreads();
  if (warp != 0) return;
  if (r.kind == KLLM_SEQ_ROUTER_SIGMOID) {
    // z: scores s;  c: choice scores (s + correction, -inf outside the kept groups and once chosen);  gs: group scores
    float* c = z + experts;
    float* gs = c + experts;
    for (int e = lane; e < experts; e += 32) {
      const float sc = 1.0f / (1.0f + expf(-z[e]));
      z[e] = sc;
      c[e] = sc + (r.correction ? r.correction[e] : 0.f);
    }
    __syncwarp();
    if (r.groups > 0) {
      const int size = experts / r.groups;
      for (int g = lane; g < r.groups; g += 32) {
        float b0 = -INFINITY, b1 = -INFINITY;
        for (int i = 0; i < size; ++i) {
          const float v = c[g * size + i];
          if (v > b0) b1 = b0, b0 = v;
          else if (v > b1) b1 = v;
        }
        gs[g] = size > 1 ? b0 + b1 : b0;
      }
      __syncwarp();
      // the groups_keep best groups keep their scores (marked by +inf in gs); the others' experts drop out
      for (int k = 0; k < r.groups_keep; ++k) {
        float best = -INFINITY;
        int bi = 0x7fffffff;
        for (int g = lane; g < r.groups; g += 32) {
          const float v = gs[g];
          if (v != INFINITY && (v > best || bi == 0x7fffffff)) best = v, bi = g;
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
          const float ob = __shfl_xor_sync(kAll, best, o);
          const int oi = __shfl_xor_sync(kAll, bi, o);
          if (oi != 0x7fffffff && (bi == 0x7fffffff || ob > best || (ob == best && oi < bi))) best = ob, bi = oi;
        }
        if (lane == 0 && bi != 0x7fffffff) gs[bi] = INFINITY;
        __syncwarp();
      }
      for (int e = lane; e < experts; e += 32)
        if (gs[e / size] != INFINITY) c[e] = -INFINITY;
      __syncwarp();
    }
    for (int k = 0; k < top; ++k) {
      float best = -INFINITY;
      int bi = 0x7fffffff;
      for (int e = lane; e < experts; e += 32) {
        const float v = c[e];
        if (v > best) best = v, bi = e;
      }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        const float ob = __shfl_xor_sync(kAll, best, o);
        const int oi = __shfl_xor_sync(kAll, bi, o);
        if (ob > best || (ob == best && oi < bi)) best = ob, bi = oi;
      }
      if (bi == 0x7fffffff) bi = 0;  // fewer eligible experts than `top`: a configuration error, kept in range
      if (lane == 0) {
        r.top_idx[static_cast<size_t>(t) * top + k] = bi;
        r.top_w[static_cast<size_t>(t) * top + k] = z[bi] * r.scale;
        c[bi] = -INFINITY;
      }
      __syncwarp();
    }
    return;
  }
  if (r.kind == KLLM_SEQ_ROUTER_TOP_SOFTMAX) {
    // the largest logits (lowest index on ties); the first chosen is the maximum, so its exponential is 1
    float first = 0.f, sum = 0.f;
    for (int k = 0; k < top; ++k) {
      float best = -INFINITY;
      int bi = 0x7fffffff;
      for (int e = lane; e < experts; e += 32) {
        const float v = z[e];
        if (v > best) best = v, bi = e;  // ascending e: the lowest index wins a tie inside the lane
      }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        const float ob = __shfl_xor_sync(kAll, best, o);
        const int oi = __shfl_xor_sync(kAll, bi, o);
        if (ob > best || (ob == best && oi < bi)) best = ob, bi = oi;
      }
      if (bi == 0x7fffffff) bi = 0;  // logits that are not numbers: kept in range
      if (k == 0) first = best;
      const float p = expf(best - first);
      sum += p;
      if (lane == 0) {
        r.top_idx[static_cast<size_t>(t) * top + k] = bi;
        r.top_w[static_cast<size_t>(t) * top + k] = p;
        z[bi] = -INFINITY;
      }
      __syncwarp();
    }
    const float inv = r.scale / sum;
    for (int k = lane; k < top; k += 32) r.top_w[static_cast<size_t>(t) * top + k] *= inv;
    return;
  }
  float mx = -INFINITY;
  for (int e = lane; e < experts; e += 32) mx = fmaxf(mx, z[e]);
  mx = warp_max(mx);
  float sum = 0.f;
  for (int e = lane; e < experts; e += 32) {
    const float p = expf(z[e] - mx);
    z[e] = p;
    sum += p;
  }
  sum = warp_sum(sum);
  __syncwarp();
  for (int e = lane; e < experts; e += 32) z[e] = z[e] / sum;
  __syncwarp();
  float chosen_sum = 0.f;
  for (int k = 0; k < top; ++k) {
    float best = -1.0f;
    int bi = 0x7fffffff;
    for (int e = lane; e < experts; e += 32) {
      const float v = z[e];
      if (v > best) best = v, bi = e;  // ascending e: the lowest index wins a tie inside the lane
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ob = __shfl_xor_sync(kAll, best, o);
      const int oi = __shfl_xor_sync(kAll, bi, o);
      if (ob > best || (ob == best && oi < bi)) best = ob, bi = oi;
    }
    chosen_sum += best;
    if (lane == 0) {
      r.top_idx[static_cast<size_t>(t) * top + k] = bi;
      r.top_w[static_cast<size_t>(t) * top + k] = best;
      z[bi] = -2.0f;  // softmax outputs are >= 0: never chosen again
    }
    __syncwarp();
  }
  const float inv = r.scale / (chosen_sum + 1e-20f);
  for (int k = lane; k < top; k += 32) r.top_w[static_cast<size_t>(t) * top + k] *= inv;
}

template <typename AT>
__global__ void router_kernel(const AT* __restrict__ h, RouterArgs r, int width) {
  extern __shared__ float sm[];  // the router's scratch, then [width] the token's row in fp32
  float* z = sm;
  float* xs = sm + router_smem_floats(r);
  const int t = blockIdx.x;
  const AT* x = h + static_cast<size_t>(t) * width;
  for (int k = threadIdx.x; k < width; k += blockDim.x) xs[k] = to_f(x[k]);
  __syncthreads();
  route_token(r, xs, z, t, width);
}

// ---- residual + norms -----------------------------------------------------------------------------------------------
// Layer norm: (v - mean) / sqrt(var + eps) * w + b, var = mean of squared deviations.  RMS norm: v / sqrt(mean(v^2) + eps) * w.
template <typename AT>
__global__ void resid_norm_kernel(ResidNormArgs a) {
  extern __shared__ float buf[];  // [width], then the router's scratch when the kernel also routes
  __shared__ float red[33];
  const int W = a.width;
  const int r = blockIdx.x;
  const size_t src = static_cast<size_t>(a.rows ? a.rows[r] : r) * W;
  const size_t dst = static_cast<size_t>(r) * W;
  const bool changes = a.y1 != nullptr || a.add != nullptr || a.add_rows != nullptr;
  if (a.y1 != nullptr) {
    const float g = a.s2 ? a.s2[r] : 1.0f;
    const float c1 = a.c1, c3 = a.c3, c4 = a.c4;
    // each mixer's output may pass an RMS norm of its own before the sum
    float r1 = 1.0f, r3 = 1.0f;
    if (a.n1.w != nullptr || (a.y3 != nullptr && a.n3.w != nullptr)) {
      float q1 = 0.f, q3 = 0.f;
      for (int i = threadIdx.x; i < W; i += blockDim.x) {
        const float v1 = a.y1[src + i], v3 = a.y3 ? a.y3[src + i] : 0.f;
        q1 = fmaf(v1, v1, q1), q3 = fmaf(v3, v3, q3);
      }
      const float inv_w = 1.0f / static_cast<float>(W);
      if (a.n1.w != nullptr) r1 = 1.0f / sqrtf(block_sum(q1, red) * inv_w + a.eps);
      if (a.y3 != nullptr && a.n3.w != nullptr) r3 = 1.0f / sqrtf(block_sum(q3, red) * inv_w + a.eps);
    }
    for (int i = threadIdx.x; i < W; i += blockDim.x) {
      float u = c1 * (a.n1.w ? a.y1[src + i] * r1 * a.n1.w[i] : a.y1[src + i]);
      if (a.y3) u += c3 * (a.n3.w ? a.y3[src + i] * r3 * a.n3.w[i] : a.y3[src + i]);
      if (a.y2) u += g * a.y2[src + i];
      if (a.y4) u += c4 * a.y4[src + i];
      buf[i] = u;
    }
    float mean = 0.f, rstd = 1.f;
    if (a.post.w != nullptr) {
      __syncthreads();
      row_stats(buf, W, a.post.kind, a.eps, red, mean, rstd);
    }
    for (int i = threadIdx.x; i < W; i += blockDim.x) {
      float v = a.x[src + i];
      if (a.post.w != nullptr) v += (buf[i] - mean) * rstd * a.post.w[i] + (a.post.b ? a.post.b[i] : 0.f);
      else v += buf[i];
      if (a.add_rows) v += a.add_rows[src + i];
      if (a.add) v += a.add[i];
      buf[i] = v;
      if (!a.rows) a.x[dst + i] = v;
    }
  } else {
    for (int i = threadIdx.x; i < W; i += blockDim.x) {
      float v = a.x[src + i];
      if (a.add_rows) v += a.add_rows[src + i];
      if (a.add) v += a.add[i];
      if (changes && !a.rows) a.x[dst + i] = v;
      buf[i] = v;
    }
  }
  const bool plain = a.pre.kind == KLLM_SEQ_NORM_NONE;  // the sublayer reads the row as it is
  if (a.pre.w == nullptr && !(plain && (a.out != nullptr || a.out_f32 != nullptr))) return;
  __syncthreads();
  float mean = 0.f, rstd = 1.0f;
  if (!plain) row_stats(buf, W, a.pre.kind, a.eps, red, mean, rstd);
  const bool route = a.router.w_router != nullptr;
  if (a.out_f32 != nullptr) {  // fp32 rows for a token-shift kernel
    for (int i = threadIdx.x; i < W; i += blockDim.x)
      a.out_f32[dst + i] = plain ? buf[i] : (buf[i] - mean) * rstd * a.pre.w[i] + (a.pre.b ? a.pre.b[i] : 0.f);
    return;
  }
  AT* out = static_cast<AT*>(a.out) + dst;
  float* state = nullptr;
  bool first = true;
  if (a.shift.mu != nullptr) {
    state = a.shift.state + static_cast<size_t>(a.shift.tok_seq[r]) * W;
    first = a.shift.tok_pos[r] == 0;
  }
  for (int i = threadIdx.x; i < W; i += blockDim.x) {
    float h = plain ? buf[i] : (buf[i] - mean) * rstd * a.pre.w[i] + (a.pre.b ? a.pre.b[i] : 0.f);
    if (state != nullptr) {
      const float prev = first ? 0.f : state[i];
      state[i] = h;
      h = h + (prev - h) * a.shift.mu[i];
    }
    const AT o = from_f<AT>(h);
    out[i] = o;
    if (route) buf[i] = to_f(o);  // the router reads what the experts read: the row in the compute type
  }
  if (!route) return;
  __syncthreads();
  route_token(a.router, buf, buf + W, r, W);
}

// One CTA per row; the CTA of an entry's first row also moves the entry's last h into the state (it alone touches it).
template <typename AT>
__global__ void token_shift_kernel(const float* __restrict__ h, const float* __restrict__ mu, float* __restrict__ state,
                                   const int32_t* __restrict__ tok_seq, const int32_t* __restrict__ tok_pos,
                                   const int32_t* __restrict__ ent_first, const int32_t* __restrict__ ent_count,
                                   int n_entries, AT* __restrict__ out, int W) {
  const int t = blockIdx.x;
  // the entry of this row: entries are few, rows of an entry are consecutive
  int e = 0;
  while (e + 1 < n_entries && ent_first[e + 1] <= t) ++e;
  const bool first_row = ent_first[e] == t;
  const float* cur = h + static_cast<size_t>(t) * W;
  float* st = state + static_cast<size_t>(tok_seq[t]) * W;
  const float* last = h + static_cast<size_t>(ent_first[e] + ent_count[e] - 1) * W;
  const bool start = tok_pos[t] == 0;
  for (int i = threadIdx.x; i < W; i += blockDim.x) {
    float prev;
    if (first_row) {
      prev = start ? 0.f : st[i];
      st[i] = last[i];
    } else {
      prev = cur[i - W];
    }
    const float v = cur[i];
    out[static_cast<size_t>(t) * W + i] = from_f<AT>(v + (prev - v) * mu[i]);
  }
}

// ---- query / key preparation ----------------------------------------------------------------------------------------
template <typename AT>
__device__ __forceinline__ AT* page_row(AT* base, const PagedKV& kv, int seq, int pos, int heads, int dim) {
  const int page = kv.table[static_cast<size_t>(seq) * kv.table_stride + pos / kv.page];
  return base + (static_cast<size_t>(page) * kv.page + pos % kv.page) * heads * dim;
}

// One warp per query / key head (per map of a head, when the heads hold several): the head's row goes through shared
// memory -- head norm with weights (before the rotation), rotation of the first rope.dims coordinates, unit norm (after
// it), temperature -- and leaves as a query row or as the key row of the token's page.  Angles, cos and sin are fp32.
template <typename AT>
__global__ void qk_prepare_kernel(AttnShape a, RopeArgs rope, const float* __restrict__ qkvg,
                                  const float* __restrict__ qnorm_w, const float* __restrict__ knorm_w, float eps,
                                  const int32_t* __restrict__ tok_seq, const int32_t* __restrict__ tok_pos,
                                  AT* __restrict__ q, float* __restrict__ gates, PagedKV kv) {
  extern __shared__ float head_rows[];  // [warps][dim]
  const int t = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
  const int maps = v_share_of(a);
  const int qn = a.heads * a.dim, kn = a.kv_heads * a.dim, vn = a.kv_heads / maps * a.vdim, gn = gate_floats(a);
  const int stride = qn + kn + vn + gn;
  const float* row = qkvg + static_cast<size_t>(t) * stride;
  const int seq = tok_seq[t], pos = tok_pos[t];
  float temp = 1.0f;
  if (a.temp_every > 0) temp = 1.0f + a.temp_coef * logf(static_cast<float>((pos + 1) / a.temp_every) + 1.0f);
  AT* krow = page_row(static_cast<AT*>(kv.k), kv, seq, pos, a.kv_heads, a.dim);
  AT* vrow = page_row(static_cast<AT*>(kv.v), kv, seq, pos, a.kv_heads / maps, a.vdim);
  const int rep = a.heads / a.kv_heads;
  const int rd = rope.dims, half = rd / 2;
  const float inv_dim = 1.0f / static_cast<float>(a.dim);
  float* hr = head_rows + warp * a.dim;
  for (int u = warp; u < a.heads + a.kv_heads; u += nw) {
    const bool is_q = u < a.heads;
    const float* src = row + (is_q ? u * a.dim : qn + (u - a.heads) * a.dim);
    AT* dst;
    if (is_q) {
      // projection order: head by head, a head's maps side by side; q order: see launch_qk_prepare
      const int h = u / maps, m = u % maps;
      const int j = ((h / rep) * maps + m) * rep + h % rep;
      dst = q + (static_cast<size_t>(t) * a.heads + j) * a.dim;
    } else {
      dst = krow + (u - a.heads) * a.dim;
    }
    float rinv = 1.0f;
    if (a.qk_norm == KLLM_SEQ_QKNORM_WEIGHTED) {
      float ss = 0.f;
      for (int d = lane; d < a.dim; d += 32) ss = fmaf(src[d], src[d], ss);
      rinv = 1.0f / sqrtf(warp_sum(ss) * inv_dim + eps);
    }
    const float* nw_ = is_q ? qnorm_w : knorm_w;
    for (int d = lane; d < a.dim; d += 32) hr[d] = a.qk_norm == KLLM_SEQ_QKNORM_WEIGHTED ? src[d] * rinv * nw_[d] : src[d];
    __syncwarp();
    for (int i = lane; i < half; i += 32) {
      const int d0 = rope.pairing == KLLM_SEQ_ROPE_PAIRS ? 2 * i : i, d1 = rope.pairing == KLLM_SEQ_ROPE_PAIRS ? 2 * i + 1 : i + half;
      const float freq = rope.freq ? rope.freq[i] : powf(rope.base, -2.0f * static_cast<float>(i) / static_cast<float>(rd));
      const float ang = static_cast<float>(pos) * freq;
      const float co = cosf(ang) * rope.mag, si = sinf(ang) * rope.mag;
      const float x0 = hr[d0], x1 = hr[d1];
      hr[d0] = x0 * co - x1 * si;
      hr[d1] = x1 * co + x0 * si;
    }
    __syncwarp();
    float post = is_q ? temp : 1.0f;
    if (a.qk_norm == KLLM_SEQ_QKNORM_UNIT) {
      float ss = 0.f;
      for (int d = lane; d < a.dim; d += 32) ss = fmaf(hr[d], hr[d], ss);
      post *= 1.0f / sqrtf(warp_sum(ss) * inv_dim + eps);
    }
    for (int d = lane; d < a.dim; d += 32) dst[d] = from_f<AT>(hr[d] * post);
    __syncwarp();
  }
  for (int i = threadIdx.x; i < vn; i += blockDim.x) vrow[i] = from_f<AT>(row[qn + kn + i]);
  for (int i = threadIdx.x; i < gn; i += blockDim.x)
    gates[static_cast<size_t>(t) * gn + i] = 1.0f / (1.0f + expf(-row[qn + kn + vn + i]));
}

// ---- attention ------------------------------------------------------------------------------------------------------
// One CTA: one entry of the step, one key/value head g, kAttnRows consecutive rows (row r of the entry = token r / rep,
// query head g * rep + r % rep, rep = heads / kv_heads), one split of the keys.  Tiles of kAttnKeys keys go through
// shared memory in fp32; scores, the running maximum / sum and the output accumulators are fp32 (online softmax).
// The partial result of a split is (m, l, o[vdim]) per row; attention_merge_kernel combines the splits, applies the
// output gate and converts to the compute type.
// SPARSE: the launch has tiles with few rows (decode steps: heads / kv_heads rows) -- rows that do not exist are skipped
// and the key tiles come in with 16-byte loads; otherwise (prompts) every loop is fully unrolled over the 16 rows of a
// thread.
// RS: rows a thread keeps in registers -- 16 for full tiles; sparse tiles of at most 8 rows are compiled with 4, so that
// the unrolled row loops do not issue twelve predicated-off iterations per step.
template <typename AT, int C, bool SPARSE, int RS>
__global__ void __launch_bounds__(kAttnThreads)
attention_kernel(AttnShape a, const void* __restrict__ q_, PagedKV kv, const int32_t* __restrict__ ent_first,
                 const int32_t* __restrict__ ent_count, const int32_t* __restrict__ ent_seq,
                 const int32_t* __restrict__ ent_pos0, int splits, float* __restrict__ ws) {
  const int e = blockIdx.y / a.kv_heads, g = blockIdx.y % a.kv_heads, split = blockIdx.z;
  const int gv = g / v_share_of(a);  // the value head this key head reads
  const int rep = a.heads / a.kv_heads;
  const int count = ent_count[e], first = ent_first[e], seq = ent_seq[e], pos0 = ent_pos0[e];
  const int n_rows = count * rep;
  const int r0 = blockIdx.x * kAttnRows;
  if (r0 >= n_rows) return;
  const int rows_here = min(kAttnRows, n_rows - r0);
  const int pmax = pos0 + (r0 + rows_here - 1) / rep;  // last position any row of the tile sees
  const int n_tiles = pmax / kAttnKeys + 1;
  // with a window the first row of the tile sees nothing before its position - window + 1
  const int tile_first = a.window > 0 ? max(0, pos0 + r0 / rep - a.window + 1) / kAttnKeys : 0;
  // tiles before the window that hold kept first positions come ahead of the window's tiles: the list of this CTA's
  // tiles is [0, keep_tiles) then [tile_first, n_tiles), cut into `splits` parts
  const int keep_tiles = a.window > 0 ? min(tile_first, (a.keep_first + kAttnKeys - 1) / kAttnKeys) : 0;
  const int list_n = keep_tiles + n_tiles - tile_first;
  const int per = (list_n + splits - 1) / splits;
  const int tile_lo = split * per, tile_hi = min(list_n, tile_lo + per);

  const int dq = (a.dim + 3) & ~3, dk = dq + 1;
  extern __shared__ float sm[];
  float* Qs = sm;                                  // [rows][dq], scaled
  float* Ks = Qs + kAttnRows * dq;                 // [keys][dk]
  float* Vs = Ks + kAttnKeys * dk;                 // [keys][vdim]
  float* Ss = Vs + kAttnKeys * a.vdim;             // [rows][keys]
  float* m_s = Ss + kAttnRows * kAttnKeys;         // [rows]
  float* l_s = m_s + kAttnRows;
  float* al_s = l_s + kAttnRows;

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  // SPARSE: only the rows that exist are filled (and read)
  for (int i = tid; i < (SPARSE ? rows_here : kAttnRows) * dq; i += kAttnThreads) {
    const int r = i / dq, d = i % dq;
    float v = 0.f;
    if (r < rows_here && d < a.dim) {
      const int rr = r0 + r;
      const int t = first + rr / rep, h = g * rep + rr % rep;
      const size_t qi = (static_cast<size_t>(t) * a.heads + h) * a.dim + d;
      v = (a.q_f32 ? static_cast<const float*>(q_)[qi] : to_f(static_cast<const AT*>(q_)[qi])) * a.scale;
    }
    Qs[i] = v;
  }
  if (tid < kAttnRows) {
    m_s[tid] = -INFINITY;
    l_s[tid] = 0.f;
  }
  // this thread's part of the score tile and of the output
  const int key = tid % kAttnKeys, rg = tid / kAttnKeys;  // rows rg*16 .. rg*16+15
  constexpr int RPT = RS;
  static_assert(SPARSE || RS == kAttnRows / (kAttnThreads / kAttnKeys), "a full tile gives each thread group 16 rows");
  float acc[RPT][C];
#pragma unroll
  for (int i = 0; i < RPT; ++i)
#pragma unroll
    for (int c = 0; c < C; ++c) acc[i][c] = 0.f;

  const AT* kbase = static_cast<const AT*>(kv.k);
  const AT* vbase = static_cast<const AT*>(kv.v);
  const int32_t* table = kv.table + static_cast<size_t>(seq) * kv.table_stride;
  const bool vec_tiles = SPARSE && (a.dim % VecOf<AT>::N) == 0 && (a.vdim % VecOf<AT>::N) == 0 &&
                         (kv.k_row % VecOf<AT>::N) == 0 && (kv.v_row % VecOf<AT>::N) == 0;
  // Rows of this thread: thread group rg takes rows rg * rpt .. rg * rpt + my_rows - 1.  A full tile gives each of the
  // two groups 16 rows; a SPARSE tile (a decode step fills only heads / kv_heads rows) splits the rows that exist
  // between the groups, so both halves of the CTA work.
  const int rpt = SPARSE ? (rows_here + 1) / 2 : RPT;
  const int my_rows = max(0, min(rpt, rows_here - rg * rpt));

  for (int li = tile_lo; li < tile_hi; ++li) {
    const int tile = li < keep_tiles ? li : tile_first + (li - keep_tiles);
    const int k0 = tile * kAttnKeys;
    __syncthreads();  // previous tile's K, V, S are no longer read
    if (vec_tiles) {  // 16-byte loads: a key's row is dim / V chunks
      constexpr int V = VecOf<AT>::N;
      const int kc = a.dim / V, vc = a.vdim / V;
      // eight chunks per thread are in flight before the first is stored: a split of a decode step has one or two
      // tiles, so the tile's load latency is paid once, not once per chunk
      constexpr int U = 8;
      const int total = kAttnKeys * (kc + vc);
      for (int base = tid; base < total; base += kAttnThreads * U) {
        float f[U][V];
#pragma unroll
        for (int u = 0; u < U; ++u) {
          const int idx = base + u * kAttnThreads;
#pragma unroll
          for (int i = 0; i < V; ++i) f[u][i] = 0.f;
          if (idx < total) {
            const int j = idx / (kc + vc), c = idx % (kc + vc);
            const int kj = k0 + j;
            if (kj <= pmax) {
              const size_t slot = static_cast<size_t>(table[kj / kv.page]) * kv.page + kj % kv.page;
              if (c < kc) VecOf<AT>::load(kbase + slot * kv.k_row + g * a.dim + c * V, f[u]);
              else VecOf<AT>::load(vbase + slot * kv.v_row + gv * a.vdim + (c - kc) * V, f[u]);
            }
          }
        }
#pragma unroll
        for (int u = 0; u < U; ++u) {
          const int idx = base + u * kAttnThreads;
          if (idx < total) {
            const int j = idx / (kc + vc), c = idx % (kc + vc);
            float* dst = c < kc ? Ks + j * dk + c * V : Vs + j * a.vdim + (c - kc) * V;
#pragma unroll
            for (int i = 0; i < V; ++i) dst[i] = f[u][i];
          }
        }
      }
      if (dk > a.dim)
        for (int idx = tid; idx < kAttnKeys * (dk - a.dim); idx += kAttnThreads)
          Ks[(idx / (dk - a.dim)) * dk + a.dim + idx % (dk - a.dim)] = 0.f;
    } else {
    for (int j = warp; j < kAttnKeys; j += kAttnThreads / 32) {
      const int kj = k0 + j;
      float* kd = Ks + j * dk;
      float* vd = Vs + j * a.vdim;
      if (kj <= pmax) {
        const size_t slot = static_cast<size_t>(table[kj / kv.page]) * kv.page + kj % kv.page;
        const AT* ksrc = kbase + slot * kv.k_row + g * a.dim;
        const AT* vsrc = vbase + slot * kv.v_row + gv * a.vdim;
        for (int d = lane; d < dk; d += 32) kd[d] = d < a.dim ? to_f(ksrc[d]) : 0.f;
        for (int d = lane; d < a.vdim; d += 32) vd[d] = to_f(vsrc[d]);
      } else {
        for (int d = lane; d < dk; d += 32) kd[d] = 0.f;
        for (int d = lane; d < a.vdim; d += 32) vd[d] = 0.f;
      }
    }
    }
    __syncthreads();
    {  // scores
      float sc[RPT];
#pragma unroll
      for (int i = 0; i < RPT; ++i) sc[i] = 0.f;
      const float* kp = Ks + key * dk;
      for (int d = 0; d < dq; d += 4) {
        const float k0v = kp[d], k1v = kp[d + 1], k2v = kp[d + 2], k3v = kp[d + 3];
#pragma unroll
        for (int i = 0; i < RPT; ++i) {
          if (SPARSE && i >= my_rows) break;
          const float4 qv = *reinterpret_cast<const float4*>(Qs + (rg * rpt + i) * dq + d);
          sc[i] = fmaf(qv.x, k0v, sc[i]);
          sc[i] = fmaf(qv.y, k1v, sc[i]);
          sc[i] = fmaf(qv.z, k2v, sc[i]);
          sc[i] = fmaf(qv.w, k3v, sc[i]);
        }
      }
      const int kj = k0 + key;
#pragma unroll
      for (int i = 0; i < RPT; ++i) {
        if (SPARSE && i >= my_rows) break;  // the softmax below reads only rows that exist
        const int r = rg * rpt + i;
        const int pr = pos0 + (r0 + r) / rep;
        const bool visible = r < rows_here && kj <= pr && (a.window == 0 || pr - kj < a.window || kj < a.keep_first);
        float sv = sc[i];
        if (a.softcap > 0.f) sv = a.softcap * tanhf(sv / a.softcap);
        Ss[r * kAttnKeys + key] = visible ? sv : -INFINITY;
      }
    }
    __syncthreads();
    for (int r = warp; r < (SPARSE ? rows_here : kAttnRows); r += kAttnThreads / 32) {  // online softmax, a warp per row
      const float v0 = Ss[r * kAttnKeys + lane], v1 = Ss[r * kAttnKeys + lane + 32];
      const float m_old = m_s[r];
      const float m_new = fmaxf(m_old, warp_max(fmaxf(v0, v1)));
      float p0 = 0.f, p1 = 0.f, alpha = 1.0f;
      if (m_new > -INFINITY) {
        p0 = expf(v0 - m_new);
        p1 = expf(v1 - m_new);
        alpha = expf(m_old - m_new);
      }
      Ss[r * kAttnKeys + lane] = p0;
      Ss[r * kAttnKeys + lane + 32] = p1;
      const float s = warp_sum(p0 + p1);
      if (lane == 0) {
        m_s[r] = m_new;
        l_s[r] = l_s[r] * alpha + s;
        al_s[r] = alpha;
      }
    }
    __syncthreads();
#pragma unroll
    for (int i = 0; i < RPT; ++i) {
      if (SPARSE && i >= my_rows) break;
      const float al = al_s[rg * rpt + i];
#pragma unroll
      for (int c = 0; c < C; ++c) acc[i][c] *= al;
    }
    for (int j = 0; j < kAttnKeys; j += 4) {
      float vv[4][C];
#pragma unroll
      for (int jj = 0; jj < 4; ++jj)
#pragma unroll
        for (int c = 0; c < C; ++c) {
          const int col = key + c * kAttnKeys;
          vv[jj][c] = col < a.vdim ? Vs[(j + jj) * a.vdim + col] : 0.f;
        }
#pragma unroll
      for (int i = 0; i < RPT; ++i) {
        if (SPARSE && i >= my_rows) break;
        const float4 p = *reinterpret_cast<const float4*>(Ss + (rg * rpt + i) * kAttnKeys + j);
#pragma unroll
        for (int c = 0; c < C; ++c) {
          acc[i][c] = fmaf(p.x, vv[0][c], acc[i][c]);
          acc[i][c] = fmaf(p.y, vv[1][c], acc[i][c]);
          acc[i][c] = fmaf(p.z, vv[2][c], acc[i][c]);
          acc[i][c] = fmaf(p.w, vv[3][c], acc[i][c]);
        }
      }
    }
  }
  __syncthreads();
  const int pstride = a.vdim + 2;
#pragma unroll
  for (int i = 0; i < RPT; ++i) {
    const int r = rg * rpt + i;
    if (i >= my_rows || r >= rows_here) continue;
    const int rr = r0 + r;
    const int t = first + rr / rep, h = g * rep + rr % rep;
    float* p = ws + ((static_cast<size_t>(t) * a.heads + h) * splits + split) * pstride;
    if (key == 0) {
      p[0] = m_s[r];
      p[1] = l_s[r];
    }
#pragma unroll
    for (int c = 0; c < C; ++c) {
      const int col = key + c * kAttnKeys;
      if (col < a.vdim) p[2 + col] = acc[i][c];
    }
  }
}

template <typename AT>
__global__ void attention_merge_kernel(int heads, int vdim, int splits, const float* __restrict__ ws,
                                       const float* __restrict__ gates, int gate_kind, const float* __restrict__ sink,
                                       int out_f32, void* __restrict__ out_) {
  const size_t th = blockIdx.x;  // t * heads + h
  const int pstride = vdim + 2;
  const float* p = ws + th * splits * pstride;
  float M = sink ? sink[th % heads] : -INFINITY;
  for (int s = 0; s < splits; ++s) M = fmaxf(M, p[s * pstride]);
  float L = sink ? expf(sink[th % heads] - M) : 0.f;
  for (int s = 0; s < splits; ++s) {
    const float m = p[s * pstride];
    if (m > -INFINITY) L += p[s * pstride + 1] * expf(m - M);
  }
  const bool per_element = gates != nullptr && gate_kind == KLLM_SEQ_GATE_ELEMENT;
  const float head_gate = gates && !per_element ? gates[th] : 1.0f;
  for (int d = threadIdx.x; d < vdim; d += blockDim.x) {
    float o = 0.f;
    for (int s = 0; s < splits; ++s) {
      const float m = p[s * pstride];
      if (m > -INFINITY) o += p[s * pstride + 2 + d] * expf(m - M);
    }
    const float gate = per_element ? gates[th * vdim + d] : head_gate;
    if (out_f32) static_cast<float*>(out_)[th * vdim + d] = o / L * gate;
    else static_cast<AT*>(out_)[th * vdim + d] = from_f<AT>(o / L * gate);
  }
}

// Differential attention, few rows (single-token steps).  One CTA per (token, head), a thread per value: the key splits of the head's two maps are joined (each map has a
// softmax of its own), o = a1 - lambda * a2, then o / sqrt(mean(o^2) + eps) * out_scale over the head's values and the
// output gate.  The maps of head h (key group g = h / rep) lie at attention heads (2 g + m) * rep + h % rep.
template <typename AT>
__global__ void diff_merge_row_kernel(int heads, int rep, int vdim, int splits, const float* __restrict__ ws,
                                  const float* __restrict__ gates, int gate_kind, float lambda, float out_scale, float eps,
                                  AT* __restrict__ out) {
  extern __shared__ float orow[];  // [vdim]
  __shared__ float red[33];
  const int t = blockIdx.x / heads, h = blockIdx.x % heads;
  const int pstride = vdim + 2;
  const float* p[2];
  float M[2], L[2];
  for (int m = 0; m < 2; ++m) {
    const size_t th = static_cast<size_t>(t) * heads * 2 + ((h / rep) * 2 + m) * rep + h % rep;
    p[m] = ws + th * splits * pstride;
    M[m] = -INFINITY, L[m] = 0.f;
    for (int s = 0; s < splits; ++s) M[m] = fmaxf(M[m], p[m][s * pstride]);
    for (int s = 0; s < splits; ++s) {
      const float mm = p[m][s * pstride];
      if (mm > -INFINITY) L[m] += p[m][s * pstride + 1] * expf(mm - M[m]);
    }
  }
  float ss = 0.f;
  for (int d = threadIdx.x; d < vdim; d += blockDim.x) {
    float o[2] = {0.f, 0.f};
    for (int m = 0; m < 2; ++m)
      for (int s = 0; s < splits; ++s) {
        const float mm = p[m][s * pstride];
        if (mm > -INFINITY) o[m] += p[m][s * pstride + 2 + d] * expf(mm - M[m]);
      }
    const float v = o[0] / L[0] - lambda * (o[1] / L[1]);
    orow[d] = v;
    ss = fmaf(v, v, ss);
  }
  const float rinv = out_scale / sqrtf(block_sum(ss, red) / static_cast<float>(vdim) + eps);
  const size_t th = static_cast<size_t>(t) * heads + h;
  const float head_gate = gates && gate_kind == KLLM_SEQ_GATE_HEAD ? gates[th] : 1.0f;
  for (int d = threadIdx.x; d < vdim; d += blockDim.x) {
    const float gate = gates && gate_kind == KLLM_SEQ_GATE_ELEMENT ? gates[th * vdim + d] : head_gate;
    out[th * vdim + d] = from_f<AT>(orow[d] * rinv * gate);
  }
}

// Differential attention, many rows (prompts).  One warp per (token, head): the key splits of the head's two maps are joined (each map has a
// softmax of its own), o = a1 - lambda * a2, then o / sqrt(mean(o^2) + eps) * out_scale over the head's values and the
// output gate.  The maps of head h (key group g = h / rep) lie at attention heads (2 g + m) * rep + h % rep.  A lane keeps
// its values (vdim <= 256: at most kDiffPerLane) in registers between the two sweeps.
constexpr int kDiffWarps = 4, kDiffPerLane = 8;
constexpr int kDiffRowsForWarps = 1024;  // (token, head) rows from which the warp form is used
template <typename AT>
__global__ void diff_merge_kernel(int n_rows, int heads, int rep, int vdim, int splits, const float* __restrict__ ws,
                                  const float* __restrict__ gates, int gate_kind, float lambda, float out_scale, float eps,
                                  AT* __restrict__ out) {
  const int row = blockIdx.x * kDiffWarps + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (row >= n_rows) return;
  const int t = row / heads, h = row % heads;
  const int pstride = vdim + 2;
  const float* p[2];
  float M[2], L[2];
  for (int m = 0; m < 2; ++m) {
    const size_t th = static_cast<size_t>(t) * heads * 2 + ((h / rep) * 2 + m) * rep + h % rep;
    p[m] = ws + th * splits * pstride;
    M[m] = -INFINITY, L[m] = 0.f;
    for (int s = 0; s < splits; ++s) M[m] = fmaxf(M[m], p[m][s * pstride]);
    for (int s = 0; s < splits; ++s) {
      const float mm = p[m][s * pstride];
      if (mm > -INFINITY) L[m] += p[m][s * pstride + 1] * expf(mm - M[m]);
    }
  }
  float vals[kDiffPerLane];
  float ss = 0.f;
#pragma unroll
  for (int i = 0; i < kDiffPerLane; ++i) {
    const int d = lane + 32 * i;
    vals[i] = 0.f;
    if (d >= vdim) continue;
    float o[2] = {0.f, 0.f};
    for (int m = 0; m < 2; ++m)
      for (int s = 0; s < splits; ++s) {
        const float mm = p[m][s * pstride];
        if (mm > -INFINITY) o[m] += p[m][s * pstride + 2 + d] * expf(mm - M[m]);
      }
    vals[i] = o[0] / L[0] - lambda * (o[1] / L[1]);
    ss = fmaf(vals[i], vals[i], ss);
  }
  for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
  const float rinv = out_scale / sqrtf(ss / static_cast<float>(vdim) + eps);
  const size_t th = static_cast<size_t>(row);
  const float head_gate = gates && gate_kind == KLLM_SEQ_GATE_HEAD ? gates[th] : 1.0f;
#pragma unroll
  for (int i = 0; i < kDiffPerLane; ++i) {
    const int d = lane + 32 * i;
    if (d >= vdim) continue;
    const float gate = gates && gate_kind == KLLM_SEQ_GATE_ELEMENT ? gates[th * vdim + d] : head_gate;
    out[th * vdim + d] = from_f<AT>(vals[i] * rinv * gate);
  }
}

// ---- routed experts, pair by pair ----------------------------------------------------------------------------------
// Expert rows per CTA: 16 (four per warp) when a step has many pairs; 4 (one per warp) when it has few, so that a decode
// step spreads over every SM and a warp waits for memory once or twice instead of eight times.
__host__ __device__ inline int pair_rows(int pairs) { return pairs <= 32 ? 4 : 16; }
// With a shared expert riding along (sh.ff > 0) the grid has T more "pairs": pair T * top + t is token t's pass
// through the shared expert, whose inner activations go to sh.inter [T, sh.ff].
template <typename AT>
__global__ void expert_gate_up_kernel(const AT* __restrict__ h, const AT* __restrict__ gate_up,
                                      const int32_t* __restrict__ top_idx, AT* __restrict__ inter, int T, int top, int ff,
                                      int width, SharedExpert sh, GatedAct ga) {
  const int act = ga.kind;
  extern __shared__ float xs[];  // [width]
  const int pair = blockIdx.x;
  const bool is_shared = pair >= T * top;
  const int t = is_shared ? pair - T * top : pair / top;
  const int rows = is_shared ? sh.ff : ff;
  const int kPairRows = pair_rows(T * top);
  if (static_cast<int>(blockIdx.y) * kPairRows >= rows) return;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
  for (int i = threadIdx.x; i < width; i += blockDim.x) xs[i] = to_f(h[static_cast<size_t>(t) * width + i]);
  __syncthreads();
  const AT* wg = is_shared ? static_cast<const AT*>(sh.gate_up)
                           : gate_up + static_cast<size_t>(top_idx[pair]) * (act == KLLM_SEQ_ACT_RELU2 ? 1 : 2) * ff * width;
  const AT* wu = wg + static_cast<size_t>(rows) * width;
  AT* dst = is_shared ? static_cast<AT*>(sh.inter) + static_cast<size_t>(t) * sh.ff
                      : inter + static_cast<size_t>(pair) * ff;
  const int f_end = min(rows, (blockIdx.y + 1) * kPairRows);
  if (act == KLLM_SEQ_ACT_RELU2) {
    for (int f = blockIdx.y * kPairRows + warp; f < f_end; f += nw) {
      const float uv = fmaxf(warp_dot(wg + static_cast<size_t>(f) * width, xs, width, lane), 0.f);
      if (lane == 0) dst[f] = from_f<AT>(uv * uv);
    }
    return;
  }
  if (is_shared) ga.limit = sh.limit;
  for (int f = blockIdx.y * kPairRows + warp; f < f_end; f += nw) {
    float gv, uv;
    warp_dot2(wg + static_cast<size_t>(f) * width, wu + static_cast<size_t>(f) * width, xs, width, lane, gv, uv);
    if (lane == 0) dst[f] = from_f<AT>(gated_act(ga, gv, uv));
  }
}

template <typename AT>
__global__ void expert_down_kernel(const AT* __restrict__ inter, const AT* __restrict__ down,
                                   const int32_t* __restrict__ top_idx, const float* __restrict__ top_w,
                                   float* __restrict__ y, int top, int ff, int width, SharedExpert sh) {
  extern __shared__ float xs[];  // [top][ff], then [sh.ff]
  const int t = blockIdx.x;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
  for (int i = threadIdx.x; i < top * ff; i += blockDim.x) xs[i] = to_f(inter[static_cast<size_t>(t) * top * ff + i]);
  for (int i = threadIdx.x; i < sh.ff; i += blockDim.x)
    xs[top * ff + i] = to_f(static_cast<const AT*>(sh.inter)[static_cast<size_t>(t) * sh.ff + i]);
  const float shared_w = sh.ff > 0 && sh.gate ? sh.gate[t] : 1.0f;
  __syncthreads();
  const int kPairRows = pair_rows(static_cast<int>(gridDim.x) * top);
  const int n_end = min(width, (blockIdx.y + 1) * kPairRows);
  for (int n = blockIdx.y * kPairRows + warp; n < n_end; n += nw) {
    float acc = 0.f;
    for (int k = 0; k < top; ++k) {
      const int e = top_idx[static_cast<size_t>(t) * top + k];
      const AT* w = down + (static_cast<size_t>(e) * width + n) * ff;
      acc += top_w[static_cast<size_t>(t) * top + k] * warp_dot(w, xs + k * ff, ff, lane);
    }
    if (sh.ff > 0)
      acc += shared_w * warp_dot(static_cast<const AT*>(sh.down) + static_cast<size_t>(n) * sh.ff, xs + top * ff, sh.ff, lane);
    if (lane == 0) y[static_cast<size_t>(t) * width + n] = acc;
  }
}

__global__ void combine_pairs_kernel(const float* __restrict__ yp, const float* __restrict__ top_w,
                                     float* __restrict__ y, int top, int width) {
  const int t = blockIdx.x;
  for (int i = threadIdx.x; i < width; i += blockDim.x) {
    float acc = 0.f;
    for (int k = 0; k < top; ++k)
      acc += top_w[static_cast<size_t>(t) * top + k] * yp[(static_cast<size_t>(t) * top + k) * width + i];
    y[static_cast<size_t>(t) * width + i] = acc;
  }
}

template <typename AT>
__global__ void gated_act_kernel(GatedAct act, const float* __restrict__ gu, AT* __restrict__ out, int ff, size_t total) {
  const size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= total) return;
  const size_t t = i / ff;
  const int f = static_cast<int>(i % ff);
  const float g = gu[t * 2 * ff + f], u = gu[t * 2 * ff + ff + f];
  out[i] = from_f<AT>(gated_act(act, g, u));
}

// ---- greedy id of each logits row (lowest index on ties) ------------------------------------------------------------
__global__ void argmax_rows_kernel(const float* __restrict__ logits, int32_t* __restrict__ out, int vocab) {
  __shared__ float bv[32];
  __shared__ int bi[32];
  const float* row = logits + static_cast<size_t>(blockIdx.x) * vocab;
  float best = -INFINITY;
  int idx = 0x7fffffff;
  for (int i = threadIdx.x; i < vocab; i += blockDim.x) {
    const float v = row[i];
    if (v > best || (v == best && i < idx)) best = v, idx = i;
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ob = __shfl_xor_sync(kAll, best, o);
    const int oi = __shfl_xor_sync(kAll, idx, o);
    if (ob > best || (ob == best && oi < idx)) best = ob, idx = oi;
  }
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (lane == 0) bv[warp] = best, bi[warp] = idx;
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int w = 1; w < static_cast<int>(blockDim.x >> 5); ++w)
      if (bv[w] > best || (bv[w] == best && bi[w] < idx)) best = bv[w], idx = bi[w];
    out[blockIdx.x] = idx == 0x7fffffff ? 0 : idx;
  }
}

// ---- pairs grouped by expert (one CTA) --------------------------------------------------------
__global__ void sort_pairs_kernel(const int32_t* __restrict__ top_idx, int n_pairs, int experts, int block,
                                  int32_t* __restrict__ counts, int32_t* __restrict__ sorted_pair,
                                  int32_t* __restrict__ block_expert, int cap) {
  extern __shared__ int32_t sh[];  // [experts] counts, [experts + 1] block offsets
  int32_t* cnt = sh;
  int32_t* off = sh + experts;
  for (int e = threadIdx.x; e < experts; e += blockDim.x) cnt[e] = 0;
  __syncthreads();
  for (int p = threadIdx.x; p < n_pairs; p += blockDim.x) atomicAdd(&cnt[top_idx[p]], 1);
  __syncthreads();
  if (threadIdx.x == 0) {
    int o = 0;
    for (int e = 0; e < experts; ++e) {
      off[e] = o;
      counts[e] = cnt[e];
      o += (cnt[e] + block - 1) / block * block;
    }
    off[experts] = o;
    counts[experts] = o;
  }
  __syncthreads();
  const int used = off[experts];
  for (int i = threadIdx.x; i < cap; i += blockDim.x) sorted_pair[i] = -1;
  for (int b = threadIdx.x; b < cap / block; b += blockDim.x) {
    int ex = -1;
    if (b * block < used)
      for (int e = 0; e < experts; ++e)
        if (b * block >= off[e] && b * block < off[e + 1]) ex = e;
    block_expert[b] = ex;
  }
  __syncthreads();
  // stable fill: each expert's pairs in ascending pair order.  A warp per expert walks the list 32 pairs at a time;
  // a pair's place is the count of matching pairs before it (ballot + population count)
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
  for (int e = warp; e < experts; e += nw) {
    int o = off[e];
    if (cnt[e] == 0) continue;
    for (int base = 0; base < n_pairs; base += 32) {
      const int p = base + lane;
      const bool mine = p < n_pairs && top_idx[p] == e;
      const unsigned m = __ballot_sync(kAll, mine);
      if (mine) sorted_pair[o + __popc(m & ((1u << lane) - 1u))] = p;
      o += __popc(m);
    }
  }
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

int launch_embed(int dtype, const void* table, const int32_t* tokens, float* x, float* copy, const NormW& norm, float eps,
                 float scale, int T, int width, cudaStream_t s) {
  if (scale == 0.f) scale = 1.0f;
  const size_t smem = static_cast<size_t>(width) * sizeof(float);
  if (smem > 48 * 1024) return KLLM_E_UNSUPPORTED;
  KLLM_SEQ_DISPATCH(dtype, (embed_kernel<AT><<<T, 128, smem, s>>>(static_cast<const AT*>(table), tokens, x, copy, norm, eps,
                                                                 scale, width)));
  return done();
}

int launch_token_shift(int dtype, const float* h, const float* mu, float* state, const int32_t* tok_seq,
                       const int32_t* tok_pos, const int32_t* ent_first, const int32_t* ent_count, int n_entries, void* out,
                       int T, int width, cudaStream_t s) {
  KLLM_SEQ_DISPATCH(dtype, (token_shift_kernel<AT><<<T, 128, 0, s>>>(h, mu, state, tok_seq, tok_pos, ent_first, ent_count,
                                                                    n_entries, static_cast<AT*>(out), width)));
  return done();
}

int launch_resid_norm(const ResidNormArgs& a, cudaStream_t s) {
  const size_t smem = (static_cast<size_t>(a.width) + (a.router.w_router ? router_smem_floats(a.router) : 0)) * sizeof(float);
  if (smem > 200 * 1024) return KLLM_E_UNSUPPORTED;
  if (a.router.w_router && (a.router.top > a.router.experts || a.router.experts <= 0 || a.router.top <= 0 || !a.pre.w))
    return KLLM_E_INVALID;
  const int threads = a.width >= 1024 ? 256 : 128;
  if (smem > 48 * 1024) {
    KLLM_SEQ_DISPATCH(a.dtype, (cudaFuncSetAttribute(resid_norm_kernel<AT>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                                     static_cast<int>(smem))));
  }
  KLLM_SEQ_DISPATCH(a.dtype, (resid_norm_kernel<AT><<<a.T, threads, smem, s>>>(a)));
  return done();
}

int launch_qk_prepare(int dtype, const AttnShape& a, const RopeArgs& rope_, const float* qkvg, const float* qnorm_w,
                      const float* knorm_w, float eps, const int32_t* tok_seq, const int32_t* tok_pos, void* q, float* gates,
                      const PagedKV& kv, int T, cudaStream_t s) {
  RopeArgs rope = rope_;
  if (rope.mag == 0.f) rope.mag = 1.0f;
  if (rope.dims < 0 || (rope.dims & 1) || rope.dims > a.dim || a.kv_heads % v_share_of(a) || a.heads % v_share_of(a) ||
      a.dim > 512)
    return KLLM_E_INVALID;
  // a warp per head: few tokens get as many warps as there are query and key heads (at most 16: the kernel's registers
  // do not fit 1024 threads); a head's row lives in shared memory
  int warps = T <= 64 ? std::min(16, std::max(4, a.heads + a.kv_heads)) : 4;
  warps = std::max(1, std::min(warps, 48 * 1024 / (4 * a.dim)));
  const size_t smem = static_cast<size_t>(warps) * a.dim * sizeof(float);
  KLLM_SEQ_DISPATCH(dtype, (qk_prepare_kernel<AT><<<T, 32 * warps, smem, s>>>(a, rope, qkvg, qnorm_w, knorm_w, eps, tok_seq,
                                                                             tok_pos, static_cast<AT*>(q), gates, kv)));
  return done();
}

int launch_diff_merge(int dtype, const AttnShape& a, int splits, const float* ws, const float* gates, float lambda,
                      float out_scale, float eps, void* out, int T, cudaStream_t s) {
  if (v_share_of(a) != 2 || a.heads % 2 || a.kv_heads % 2 || a.sink != nullptr) return KLLM_E_UNSUPPORTED;
  const int heads = a.heads / 2;
  if (a.vdim > 32 * kDiffPerLane) return KLLM_E_UNSUPPORTED;
  const int n_rows = T * heads;
  if (n_rows < kDiffRowsForWarps) {  // latency matters more than the CTA count: a thread per value
    const int threads = a.vdim <= 64 ? 64 : 128;
    KLLM_SEQ_DISPATCH(dtype, (diff_merge_row_kernel<AT><<<n_rows, threads, a.vdim * sizeof(float), s>>>(
                                 heads, a.heads / a.kv_heads, a.vdim, splits, ws, a.gate ? gates : nullptr, a.gate, lambda,
                                 out_scale, eps, static_cast<AT*>(out))));
    return done();
  }
  KLLM_SEQ_DISPATCH(dtype, (diff_merge_kernel<AT><<<(n_rows + kDiffWarps - 1) / kDiffWarps, 32 * kDiffWarps, 0, s>>>(
                               n_rows, heads, a.heads / a.kv_heads, a.vdim, splits, ws, a.gate ? gates : nullptr, a.gate, lambda,
                               out_scale, eps, static_cast<AT*>(out))));
  return done();
}

size_t attention_workspace_bytes(const AttnShape& a, int T, int splits) {
  return static_cast<size_t>(T) * a.heads * splits * (a.vdim + 2) * sizeof(float);
}

template <typename AT, int C, bool SPARSE, int RS>
static int launch_attention_cs(const AttnShape& a, const void* q, const PagedKV& kv, int n_entries,
                              const int32_t* ent_first, const int32_t* ent_count, const int32_t* ent_seq,
                              const int32_t* ent_pos0, int max_count, int splits, float* ws, cudaStream_t s) {
  const int dq = (a.dim + 3) & ~3;
  const size_t smem = (static_cast<size_t>(kAttnRows) * dq + static_cast<size_t>(kAttnKeys) * (dq + 1) +
                       static_cast<size_t>(kAttnKeys) * a.vdim + kAttnRows * kAttnKeys + 3 * kAttnRows) * sizeof(float);
  if (smem > 220 * 1024) return KLLM_E_UNSUPPORTED;
  static size_t configured = 0;
  if (smem > 48 * 1024 && smem > configured) {
    const cudaError_t e = cudaFuncSetAttribute(attention_kernel<AT, C, SPARSE, RS>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                               static_cast<int>(smem));
    if (e != cudaSuccess) return cuda_rc(e);
    configured = smem;
  }
  const int rep = a.heads / a.kv_heads;
  const dim3 grid((max_count * rep + kAttnRows - 1) / kAttnRows, n_entries * a.kv_heads, splits);
  attention_kernel<AT, C, SPARSE, RS><<<grid, kAttnThreads, smem, s>>>(a, q, kv, ent_first, ent_count, ent_seq, ent_pos0, splits,
                                                                       ws);
  return done();
}

template <typename AT, int C>
static int launch_attention_c(const AttnShape& a, const void* q, const PagedKV& kv, int n_entries,
                              const int32_t* ent_first, const int32_t* ent_count, const int32_t* ent_seq,
                              const int32_t* ent_pos0, int max_count, int splits, float* ws, cudaStream_t s) {
  if (max_count * (a.heads / a.kv_heads) < kAttnRows)
    return max_count * (a.heads / a.kv_heads) <= 8
               ? launch_attention_cs<AT, C, true, 4>(a, q, kv, n_entries, ent_first, ent_count, ent_seq, ent_pos0, max_count,
                                                     splits, ws, s)
               : launch_attention_cs<AT, C, true, 16>(a, q, kv, n_entries, ent_first, ent_count, ent_seq, ent_pos0, max_count, splits,
                                            ws, s);
  return launch_attention_cs<AT, C, false, 16>(a, q, kv, n_entries, ent_first, ent_count, ent_seq, ent_pos0, max_count, splits,
                                           ws, s);
}

int launch_attention(int dtype, const AttnShape& a, const void* q, const float* gates, const PagedKV& kv,
                     int n_entries, const int32_t* ent_first, const int32_t* ent_count, const int32_t* ent_seq,
                     const int32_t* ent_pos0, int max_count, int max_ctx, int splits, float* ws, void* out, int T,
                     const int32_t* tok_seq, const int32_t* tok_pos, cudaStream_t s) {
  (void)max_ctx, (void)tok_seq, (void)tok_pos;
  if (a.kv_heads <= 0 || a.heads % a.kv_heads != 0 || a.vdim > 4 * kAttnKeys || a.dim <= 0 || a.vdim <= 0)
    return KLLM_E_UNSUPPORTED;
  const int C = (a.vdim + kAttnKeys - 1) / kAttnKeys;
  int rc = 0;
  if (attention_mma_usable(dtype, a, max_count)) {
    rc = launch_attention_mma(a, q, gates, kv, n_entries, ent_first, ent_count, ent_seq, ent_pos0, max_count, splits, ws,
                              out, s);
    if (rc || (splits == 1 && !a.no_merge)) return rc;
  } else {
#define KLLM_ATTN_C(c)                                                                                              \
  KLLM_SEQ_DISPATCH(dtype, (rc = launch_attention_c<AT, c>(a, q, kv, n_entries, ent_first, ent_count, ent_seq, ent_pos0, \
                                                           max_count, splits, ws, s)))
  switch (C) {
    case 1: KLLM_ATTN_C(1); break;
    case 2: KLLM_ATTN_C(2); break;
    case 3: KLLM_ATTN_C(3); break;
    default: KLLM_ATTN_C(4); break;
  }
#undef KLLM_ATTN_C
  }
  if (rc || a.no_merge) return rc;
  KLLM_SEQ_DISPATCH(dtype, (attention_merge_kernel<AT><<<T * a.heads, 64, 0, s>>>(a.heads, a.vdim, splits, ws,
                                                                                 a.gate ? gates : nullptr, a.gate, a.sink,
                                                                                 a.out_f32, out)));
  return done();
}

int launch_router(int dtype, const void* h, const float* w_router, const float* w_sg, int experts, int top,
                  float scale, int32_t* top_idx, float* top_w, float* sgate, int T, int width, cudaStream_t s) {
  if (top > experts || experts <= 0 || top <= 0) return KLLM_E_INVALID;
  const RouterArgs r{w_router, w_sg, experts, top, scale, top_idx, top_w, sgate, KLLM_SEQ_ROUTER_SOFTMAX, nullptr, 0, 0};
  const size_t smem = (router_smem_floats(r) + width) * sizeof(float);
  if (smem > 48 * 1024) return KLLM_E_UNSUPPORTED;
  KLLM_SEQ_DISPATCH(dtype, (router_kernel<AT><<<T, 256, smem, s>>>(static_cast<const AT*>(h), r, width)));
  return done();
}

bool shared_expert_rides_along(int top, int ff, int shared_ff) {
  return (static_cast<size_t>(top) * ff + shared_ff) * sizeof(float) <= 48 * 1024;
}

int launch_expert_gate_up(int dtype, const void* h, const void* gate_up, const int32_t* top_idx, void* inter, int T,
                          int top, int ff, int width, const SharedExpert& sh, const GatedAct& act, cudaStream_t s) {
  if (act.kind != KLLM_SEQ_ACT_SWIGLU && act.kind != KLLM_SEQ_ACT_CLAMP_SWIGLU && (act.kind != KLLM_SEQ_ACT_RELU2 || sh.ff > 0))
    return KLLM_E_UNSUPPORTED;
  const size_t smem = static_cast<size_t>(width) * sizeof(float);
  if (smem > 48 * 1024) return KLLM_E_UNSUPPORTED;
  const int kPairRows = pair_rows(T * top);
  const dim3 grid(T * top + (sh.ff > 0 ? T : 0), (std::max(ff, sh.ff) + kPairRows - 1) / kPairRows);
  KLLM_SEQ_DISPATCH(dtype, (expert_gate_up_kernel<AT><<<grid, 128, smem, s>>>(static_cast<const AT*>(h),
                                                                             static_cast<const AT*>(gate_up), top_idx,
                                                                             static_cast<AT*>(inter), T, top, ff, width,
                                                                             sh, act)));
  return done();
}

int launch_expert_down(int dtype, const void* inter, const void* down, const int32_t* top_idx, const float* top_w,
                       float* y, int T, int top, int ff, int width, const SharedExpert& sh, cudaStream_t s) {
  const size_t smem = (static_cast<size_t>(top) * ff + sh.ff) * sizeof(float);
  if (smem > 48 * 1024) return KLLM_E_UNSUPPORTED;
  const int kPairRows = pair_rows(T * top);
  const dim3 grid(T, (width + kPairRows - 1) / kPairRows);
  KLLM_SEQ_DISPATCH(dtype, (expert_down_kernel<AT><<<grid, 128, smem, s>>>(static_cast<const AT*>(inter),
                                                                          static_cast<const AT*>(down), top_idx, top_w,
                                                                          y, top, ff, width, sh)));
  return done();
}

int launch_combine_pairs(const float* yp, const float* top_w, float* y, int T, int top, int width, cudaStream_t s) {
  combine_pairs_kernel<<<T, 256, 0, s>>>(yp, top_w, y, top, width);
  return done();
}

int launch_gated_act(int dtype, const GatedAct& act, const float* gu, void* out, int T, int ff, cudaStream_t s) {
  const size_t total = static_cast<size_t>(T) * ff;
  const unsigned blocks = static_cast<unsigned>((total + 255) / 256);
  KLLM_SEQ_DISPATCH(dtype, (gated_act_kernel<AT><<<blocks, 256, 0, s>>>(act, gu, static_cast<AT*>(out), ff, total)));
  return done();
}

int launch_argmax_rows(const float* logits, int32_t* out, int rows, int vocab, cudaStream_t s) {
  argmax_rows_kernel<<<rows, 1024, 0, s>>>(logits, out, vocab);
  return done();
}

int launch_sort_pairs(const int32_t* top_idx, int n_pairs, int experts, int block, int32_t* counts,
                      int32_t* sorted_pair, int32_t* block_expert, int cap, cudaStream_t s) {
  const size_t smem = (2 * static_cast<size_t>(experts) + 1) * sizeof(int32_t);
  if (smem > 48 * 1024) return KLLM_E_UNSUPPORTED;
  sort_pairs_kernel<<<1, 1024, smem, s>>>(top_idx, n_pairs, experts, block, counts, sorted_pair, block_expert, cap);
  return done();
}

}  // namespace seq
}  // namespace kllm
