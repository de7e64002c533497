// Matrix products of the sequence-batch engine:  out[T, N] (fp32) = a[T, K] . w[N, K]^T, a and w in the compute type
// (float: true fp32 multiply-add, no reduced-precision tensor mode; __nv_bfloat16: bf16 operands, fp32 accumulation).
//
//   rows_kernel     T <= 8 (decode steps): the weights are streamed once, a warp per output feature, all rows of `a`
//                   against each 16-byte weight vector -- bound by the weight bytes
//   tiled_kernel    any shape: 64 x 64 x 16 tiles through shared memory, 4 x 4 outputs per thread (fp32 FMA)
//   umma_kernel     bf16, T >= 64, K % 8 == 0: 128 weight rows x BN tokens per CTA on tcgen05.mma (kind::f16, operands
//                   by TMA with 128-byte swizzle, accumulator in TMEM)                      [seq_gemm_umma.cuh]
//   grouped_kernel  the tiled kernel over row blocks that each belong to one expert (rows gathered by index, the
//                   SiLU-gate product as an optional epilogue)
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <cstdint>
#include <cstdlib>

#include "seq_engine.h"
#include "seq_gemm_umma.cuh"

namespace kllm {
namespace seq {
namespace {

__device__ __forceinline__ float ld_f(const float* p) { return *p; }
__device__ __forceinline__ float ld_f(const __nv_bfloat16* p) { return __bfloat162float(*p); }
__device__ __forceinline__ void st_t(float* p, float v) { *p = v; }
__device__ __forceinline__ void st_t(__nv_bfloat16* p, float v) { *p = __float2bfloat16_rn(v); }

template <typename AT> struct Vec16;
template <> struct Vec16<float> {
  static constexpr int N = 4;
  __device__ static __forceinline__ void load(const float* p, float* f) {
    const float4 v = __ldg(reinterpret_cast<const float4*>(p));
    f[0] = v.x, f[1] = v.y, f[2] = v.z, f[3] = v.w;
  }
  __device__ static __forceinline__ void load_stream(const float* p, float* f) {
    float4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.f32 {%0,%1,%2,%3}, [%4];"
                 : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "l"(p));
    f[0] = v.x, f[1] = v.y, f[2] = v.z, f[3] = v.w;
  }
};
template <> struct Vec16<__nv_bfloat16> {
  static constexpr int N = 8;
  __device__ static __forceinline__ void widen(const uint4& v, float* f) {
    const uint32_t u[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      f[2 * i] = __uint_as_float(u[i] << 16);
      f[2 * i + 1] = __uint_as_float(u[i] & 0xffff0000u);
    }
  }
  __device__ static __forceinline__ void load(const __nv_bfloat16* p, float* f) {
    widen(__ldg(reinterpret_cast<const uint4*>(p)), f);
  }
  __device__ static __forceinline__ void load_stream(const __nv_bfloat16* p, float* f) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    widen(v, f);
  }
};

// ---- a few rows against every weight row ----------------------------------------------------------------------------
template <typename AT, int R, bool VEC>
__global__ void __launch_bounds__(256)
rows_kernel(const AT* __restrict__ a, const AT* __restrict__ w, float* __restrict__ out, int T, int K, int N) {
  constexpr int V = Vec16<AT>::N;
  const int lane = threadIdx.x & 31;
  const int n = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (n >= N) return;
  const AT* wr = w + static_cast<size_t>(n) * K;
  float acc[R];
#pragma unroll
  for (int r = 0; r < R; ++r) acc[r] = 0.f;
  if (VEC) {
    for (int k = lane * V; k < K; k += 32 * V) {
      float wf[V];
      Vec16<AT>::load_stream(wr + k, wf);
#pragma unroll
      for (int r = 0; r < R; ++r) {
        if (r < T) {
          float af[V];
          Vec16<AT>::load(a + static_cast<size_t>(r) * K + k, af);
#pragma unroll
          for (int i = 0; i < V; ++i) acc[r] = fmaf(af[i], wf[i], acc[r]);
        }
      }
    }
  } else {
    for (int k = lane; k < K; k += 32) {
      const float wv = ld_f(wr + k);
#pragma unroll
      for (int r = 0; r < R; ++r)
        if (r < T) acc[r] = fmaf(ld_f(a + static_cast<size_t>(r) * K + k), wv, acc[r]);
    }
  }
#pragma unroll
  for (int r = 0; r < R; ++r) {
    float v = acc[r];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    if (lane == 0 && r < T) out[static_cast<size_t>(r) * N + n] = v;
  }
}

// ---- tiled fp32-FMA product (plain and grouped) ---------------------------------------------------------------------
constexpr int TM = 64, TN = 64, TK = 16;

// GROUPED: row i of block b is pair sorted_pair[b * TM + i] (or -1); its `a` row is pair / a_row_div, the weights are
// those of expert block_expert[b].  EPI 1 computes gate and up together (weights: ff gate rows then ff up rows); EPI 2
// squares the positive part of a single product.
template <typename AT, bool GROUPED, int EPI>
__global__ void __launch_bounds__(256)
tiled_kernel(const AT* __restrict__ a, const AT* __restrict__ w, void* __restrict__ out_, int T, int K, int N,
             const int32_t* __restrict__ sorted_pair, const int32_t* __restrict__ block_expert, int a_row_div,
             GatedAct act = GatedAct{KLLM_SEQ_ACT_SWIGLU, 0.f, 0.f}) {
  __shared__ float As[TK][TM + 4];
  __shared__ float Ws[EPI == 1 ? 2 : 1][TK][TN + 4];
  __shared__ int32_t rowsrc[TM], rowdst[TM];
  const int tid = threadIdx.x;
  const int m0 = blockIdx.y * TM, n0 = blockIdx.x * TN;
  if (GROUPED) {
    const int ex = block_expert[blockIdx.y];
    if (ex < 0) return;
    w += static_cast<size_t>(ex) * (EPI == 1 ? 2 : 1) * N * K;
    if (tid < TM) {
      const int p = sorted_pair[m0 + tid];
      rowdst[tid] = p;
      rowsrc[tid] = p < 0 ? -1 : p / a_row_div;
    }
  } else if (tid < TM) {
    const int r = m0 + tid;
    rowsrc[tid] = rowdst[tid] = r < T ? r : -1;
  }
  __syncthreads();
  const int tx = tid % 16, ty = tid / 16;  // outputs rows ty*4.., columns tx*4..
  float acc[EPI == 1 ? 2 : 1][4][4];
#pragma unroll
  for (int z = 0; z < (EPI == 1 ? 2 : 1); ++z)
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
      for (int j = 0; j < 4; ++j) acc[z][i][j] = 0.f;
  // loading: thread -> (row = tid / 4, four consecutive k = (tid % 4) * 4 ..)
  const int lr = tid / 4, lk = (tid % 4) * 4;
  for (int k0 = 0; k0 < K; k0 += TK) {
    {
      const int src = rowsrc[lr];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int k = k0 + lk + i;
        As[lk + i][lr] = (src >= 0 && k < K) ? ld_f(a + static_cast<size_t>(src) * K + k) : 0.f;
      }
#pragma unroll
      for (int z = 0; z < (EPI == 1 ? 2 : 1); ++z) {
        const int n = n0 + lr;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const int k = k0 + lk + i;
          Ws[z][lk + i][lr] = (n < N && k < K) ? ld_f(w + (static_cast<size_t>(z) * N + n) * K + k) : 0.f;
        }
      }
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < TK; ++kk) {
      const float4 av = *reinterpret_cast<const float4*>(&As[kk][ty * 4]);
      const float ar[4] = {av.x, av.y, av.z, av.w};
#pragma unroll
      for (int z = 0; z < (EPI == 1 ? 2 : 1); ++z) {
        const float4 wv = *reinterpret_cast<const float4*>(&Ws[z][kk][tx * 4]);
        const float wr[4] = {wv.x, wv.y, wv.z, wv.w};
#pragma unroll
        for (int i = 0; i < 4; ++i)
#pragma unroll
          for (int j = 0; j < 4; ++j) acc[z][i][j] = fmaf(ar[i], wr[j], acc[z][i][j]);
      }
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int dst = rowdst[ty * 4 + i];
    if (dst < 0) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int n = n0 + tx * 4 + j;
      if (n >= N) continue;
      if (EPI == 1) {
        const float g = acc[0][i][j], u = acc[EPI == 1 ? 1 : 0][i][j];
        st_t(static_cast<AT*>(out_) + static_cast<size_t>(dst) * N + n, gated_act(act, g, u));
      } else if (EPI == 2) {
        const float u = fmaxf(acc[0][i][j], 0.f);
        st_t(static_cast<AT*>(out_) + static_cast<size_t>(dst) * N + n, u * u);
      } else {
        static_cast<float*>(out_)[static_cast<size_t>(dst) * N + n] = acc[0][i][j];
      }
    }
  }
}

template <typename AT>
int gemm_t(const AT* a, const AT* w, float* out, int T, int K, int N, cudaStream_t s, bool* umma_used) {
  constexpr int V = Vec16<AT>::N;
  if (T <= 8) {
    const bool vec = (K % V) == 0 && (reinterpret_cast<uintptr_t>(a) & 15) == 0 && (reinterpret_cast<uintptr_t>(w) & 15) == 0;
    const int warps = 8;
    const dim3 grid((N + warps - 1) / warps);
#define KLLM_ROWS(R)                                                                  \
  do {                                                                                \
    if (vec) rows_kernel<AT, R, true><<<grid, warps * 32, 0, s>>>(a, w, out, T, K, N); \
    else rows_kernel<AT, R, false><<<grid, warps * 32, 0, s>>>(a, w, out, T, K, N);    \
  } while (0)
    if (T <= 1) KLLM_ROWS(1);
    else if (T <= 2) KLLM_ROWS(2);
    else if (T <= 4) KLLM_ROWS(4);
    else KLLM_ROWS(8);
#undef KLLM_ROWS
    count_launch();
    return cuda_rc(cudaGetLastError());
  }
  if (umma::usable<AT>(a, w, T, K, N)) {
    *umma_used = true;
    return umma::launch(a, w, out, T, K, N, s);
  }
  const dim3 grid((N + TN - 1) / TN, (T + TM - 1) / TM);
  tiled_kernel<AT, false, 0><<<grid, 256, 0, s>>>(a, w, out, T, K, N, nullptr, nullptr, 1);
  count_launch();
  return cuda_rc(cudaGetLastError());
}

template <typename AT>
int grouped_t(const GroupedArgs& g, cudaStream_t s) {
  const dim3 grid((g.N + TN - 1) / TN, g.n_blocks);
  if (g.block != TM) return KLLM_E_INVALID;
  if (g.epilogue == 1)
    tiled_kernel<AT, true, 1><<<grid, 256, 0, s>>>(static_cast<const AT*>(g.a), static_cast<const AT*>(g.w), g.out, 0, g.K,
                                                  g.N, g.sorted_pair, g.block_expert, g.a_row_div, g.act);
  else if (g.epilogue == 2)
    tiled_kernel<AT, true, 2><<<grid, 256, 0, s>>>(static_cast<const AT*>(g.a), static_cast<const AT*>(g.w), g.out, 0, g.K,
                                                  g.N, g.sorted_pair, g.block_expert, g.a_row_div);
  else
    tiled_kernel<AT, true, 0><<<grid, 256, 0, s>>>(static_cast<const AT*>(g.a), static_cast<const AT*>(g.w), g.out, 0, g.K,
                                                  g.N, g.sorted_pair, g.block_expert, g.a_row_div);
  count_launch();
  return cuda_rc(cudaGetLastError());
}

}  // namespace

static bool g_umma_used;
int gemm(int dtype, const void* a, const void* w, float* out, int T, int K, int N, cudaStream_t s) {
  if (!a || !w || !out || T <= 0 || K <= 0 || N <= 0) return KLLM_E_INVALID;
  if (dtype == KLLM_SEQ_F32) return gemm_t(static_cast<const float*>(a), static_cast<const float*>(w), out, T, K, N, s, &g_umma_used);
  if (dtype == KLLM_SEQ_BF16)
    return gemm_t(static_cast<const __nv_bfloat16*>(a), static_cast<const __nv_bfloat16*>(w), out, T, K, N, s, &g_umma_used);
  return KLLM_E_INVALID;
}

int gemm_take_error() {
  if (!g_umma_used) return 0;
  g_umma_used = false;
  return umma::take_error();
}

bool grouped_tensor_core_usable(int dtype, int width, int ff) {
  return dtype == KLLM_SEQ_BF16 && umma::grouped_usable(width, ff) && umma::grouped_usable(ff, width);
}

int gather_rows_bf16(const void* a, const int32_t* sorted_pair, int div, void* out, int rows, int K, cudaStream_t s) {
  if ((K % 8) != 0) return KLLM_E_UNSUPPORTED;
  umma::gather_rows_kernel<<<rows, 128, 0, s>>>(static_cast<const __nv_bfloat16*>(a), sorted_pair, div,
                                               static_cast<__nv_bfloat16*>(out), K);
  count_launch();
  return cuda_rc(cudaGetLastError());
}

int gemm_grouped(int dtype, const GroupedArgs& g, cudaStream_t s) {
  if (g.sorted_layout) {
    if (dtype != KLLM_SEQ_BF16 || g.block != umma::GBN) return KLLM_E_INVALID;
    g_umma_used = true;
    if (g.epilogue == 1)
      return umma::launch_grouped<1>(g.a, g.w, g.out, g.sorted_pair, g.block_expert, g.n_blocks, g.experts, g.K, g.N, s, g.act);
    if (g.epilogue == 2)
      return umma::launch_grouped<2>(g.a, g.w, g.out, g.sorted_pair, g.block_expert, g.n_blocks, g.experts, g.K, g.N, s);
    return umma::launch_grouped<0>(g.a, g.w, g.out, g.sorted_pair, g.block_expert, g.n_blocks, g.experts, g.K, g.N, s);
  }
  if (dtype == KLLM_SEQ_F32) return grouped_t<float>(g, s);
  if (dtype == KLLM_SEQ_BF16) return grouped_t<__nv_bfloat16>(g, s);
  return KLLM_E_INVALID;
}

}  // namespace seq
}  // namespace kllm
