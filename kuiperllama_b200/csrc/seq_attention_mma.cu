// Prompt attention of the sequence-batch engine on the tensor cores (bf16 operands, fp32 accumulation).
//
// Same problem as attention_kernel in seq_kernels.cu -- causal softmax attention of a ragged batch over paged keys and
// values, query heads grouped over key/value heads -- for steps that bring many rows: one CTA takes 64 consecutive rows
// of one entry and one key/value head (row r = token r / rep, query head g * rep + r % rep, so the `rep` query heads of
// a token share every key tile), one warp 16 of them.
//
//   scores    S = Q K^T by mma.sync m16n8k16 (bf16 x bf16 -> fp32); scale, causal mask, running maximum and sum, and
//             the exponentials (ex2.approx on scores in units of log2, relative error about 2^-22) are fp32 in
//             registers (online softmax); only tiles that touch the diagonal are masked
//   weights   the fp32 weights p enter the second product as TWO bf16 terms, p = hi + lo (lo = p - hi rounded), so the
//             product sees them to about 2^-17 instead of 2^-9: the values are bf16 already, the weights are not
//   output    O += (hi + lo) V, fp32 accumulators; V fragments come transposed out of shared memory (ldmatrix.trans)
//   tiles     64 keys x (dim | vdim) bf16 through a two-stage cp.async ring, rows padded by 16 bytes (conflict-free
//             fragment loads); keys past the last visible position are zero-filled
//   sizes     the kernel is compiled for head sizes of 64 and 128; a model's dim / vdim (multiples of 8) run in the
//             next size up with the missing columns zero-filled in shared memory and never stored
//
// With one split the kernel divides by the sum, applies the output gate and writes the compute type; with several it
// leaves (max, sum, unnormalised output) per split for attention_merge_kernel, like the fp32 kernel.
// tcgen05 is not used here: at head sizes of 64..128 a 64-row tile is small against TMEM's 128-lane accumulators, and
// the softmax between the two products wants the scores in registers anyway.
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <cmath>
#include <cstdint>

#include "seq_engine.h"

namespace kllm {
namespace seq {
namespace {

constexpr int kRows = 64, kKeys = 64, kThreads = 128;

__device__ __forceinline__ void mma_bf16(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src, bool valid) {
  const int n = valid ? 16 : 0;  // 0 bytes read: the 16 bytes are zero-filled
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(n) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}

__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
               : "r"(addr));
}

// (x, y) -> packed bf16 pairs hi and lo with x ~ hi.x + lo.x; the lower index sits in the low half
__device__ __forceinline__ void split_pack(float x, float y, uint32_t& hi, uint32_t& lo) {
  const __nv_bfloat162 h2 = __floats2bfloat162_rn(x, y);
  hi = *reinterpret_cast<const uint32_t*>(&h2);
  const float xh = __uint_as_float(hi << 16), yh = __uint_as_float(hi & 0xffff0000u);  // a bf16 is the top half of a float
  const __nv_bfloat162 l2 = __floats2bfloat162_rn(x - xh, y - yh);
  lo = *reinterpret_cast<const uint32_t*>(&l2);
}

__device__ __forceinline__ float exp2_approx(float x) {  // 2^x, relative error about 2^-22; 2^-inf = 0
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ void ldmatrix_x4(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
               : "r"(addr));
}

__device__ __forceinline__ float quad_max(float v) {
  v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, 1));
  return fmaxf(v, __shfl_xor_sync(0xffffffffu, v, 2));
}
__device__ __forceinline__ float quad_sum(float v) {
  v += __shfl_xor_sync(0xffffffffu, v, 1);
  return v + __shfl_xor_sync(0xffffffffu, v, 2);
}

template <int DIM, int VDIM>
__global__ void __launch_bounds__(kThreads, (DIM + VDIM <= 128) ? 4 : (DIM > 128 ? 1 : 0))
attention_mma_kernel(AttnShape a, const __nv_bfloat16* __restrict__ q, PagedKV kv, const int32_t* __restrict__ ent_first,
                     const int32_t* __restrict__ ent_count, const int32_t* __restrict__ ent_seq,
                     const int32_t* __restrict__ ent_pos0, int splits, float* __restrict__ ws,
                     const float* __restrict__ gates, __nv_bfloat16* __restrict__ out) {
  constexpr int LDK = DIM + 8, LDV = VDIM + 8;  // bf16 elements per shared-memory row
  constexpr int KS = DIM / 16;                  // k-steps of Q K^T
  constexpr int NB = VDIM / 8;                  // 8-column blocks of the output
  constexpr int KC = DIM / 8, VC = VDIM / 8;    // 16-byte chunks per key / value row
  // grid: x = (entry, key/value head), y = row tile, z = split.  CTAs are handed out in x-fastest order, so the tiles
  // of equal weight (the same rows of every head) start together, heaviest first
  const int e = blockIdx.x / a.kv_heads, g = blockIdx.x % a.kv_heads, split = blockIdx.z;
  const int gv = g / v_share_of(a);  // the value head this key head reads
  const int rep = a.heads / a.kv_heads;
  const int dim = a.dim, vdim = a.vdim;  // <= DIM, VDIM; multiples of 8
  const int count = ent_count[e], first = ent_first[e], seq = ent_seq[e], pos0 = ent_pos0[e];
  const int n_rows = count * rep;
  const int r0 = (gridDim.y - 1 - blockIdx.y) * kRows;  // the tiles with the most keys start first
  if (r0 >= n_rows) return;
  const int rows_here = min(kRows, n_rows - r0);
  const int pmax = pos0 + (r0 + rows_here - 1) / rep;  // last position any row of the tile sees
  const int n_tiles = pmax / kKeys + 1;
  // with a window the first row of the tile sees nothing before its position - window + 1
  const int window = a.window;
  const int tile_first = window > 0 ? max(0, pos0 + r0 / rep - window + 1) / kKeys : 0;
  // tiles before the window that hold kept first positions come ahead of the window's tiles: this CTA's list of tiles
  // is [0, keep_tiles) then [tile_first, n_tiles), cut into `splits` parts
  const int keep_first = window > 0 ? a.keep_first : 0;
  const int keep_tiles = min(tile_first, (keep_first + kKeys - 1) / kKeys);
  const int list_n = keep_tiles + n_tiles - tile_first;
  const int per = (list_n + splits - 1) / splits;
  const int tile_lo = split * per, tile_hi = min(list_n, tile_lo + per);
  auto tile_of = [&](int li) { return li < keep_tiles ? li : tile_first + (li - keep_tiles); };
  const float softcap = a.softcap;

  extern __shared__ __align__(16) unsigned char sm_raw[];
  __nv_bfloat16* Ks = reinterpret_cast<__nv_bfloat16*>(sm_raw);  // [2][keys][LDK]
  __nv_bfloat16* Vs = Ks + 2 * kKeys * LDK;                      // [2][keys][LDV]

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int gq = lane >> 2, t4 = lane & 3;
  // the two rows of this thread's accumulator fragments
  const int rA = r0 + warp * 16 + gq, rB = rA + 8;
  const bool exA = rA < n_rows, exB = rB < n_rows;
  const int posA = exA ? pos0 + rA / rep : -1, posB = exB ? pos0 + rB / rep : -1;  // -1: sees nothing
  const size_t thA = exA ? static_cast<size_t>(first + rA / rep) * a.heads + g * rep + rA % rep : 0;
  const size_t thB = exB ? static_cast<size_t>(first + rB / rep) * a.heads + g * rep + rB % rep : 0;
  const int warp_last = __reduce_max_sync(0xffffffffu, max(posA, posB));  // last position any row of the warp sees
  // first position of the warp's rows (rows that do not exist count as -1: their tiles are always masked)
  const int warp_first = __reduce_min_sync(0xffffffffu, min(posA, posB));
  const float scale2_plain = a.scale * 1.4426950408889634f;  // scores are kept in units of log2: exp(x) = 2^(x log2 e)

  uint32_t qf[KS][4];
  {
    const __nv_bfloat16* qa = q + thA * dim;
    const __nv_bfloat16* qb = q + thB * dim;
#pragma unroll
    for (int ks = 0; ks < KS; ++ks) {
      const int d = ks * 16 + t4 * 2;
      qf[ks][0] = exA && d < dim ? *reinterpret_cast<const uint32_t*>(qa + d) : 0u;
      qf[ks][1] = exB && d < dim ? *reinterpret_cast<const uint32_t*>(qb + d) : 0u;
      qf[ks][2] = exA && d + 8 < dim ? *reinterpret_cast<const uint32_t*>(qa + d + 8) : 0u;
      qf[ks][3] = exB && d + 8 < dim ? *reinterpret_cast<const uint32_t*>(qb + d + 8) : 0u;
    }
  }
  float o[NB][4];
#pragma unroll
  for (int nb = 0; nb < NB; ++nb) o[nb][0] = o[nb][1] = o[nb][2] = o[nb][3] = 0.f;
  float mA = -INFINITY, mB = -INFINITY, lA = 0.f, lB = 0.f;

  const __nv_bfloat16* kbase = static_cast<const __nv_bfloat16*>(kv.k);
  const __nv_bfloat16* vbase = static_cast<const __nv_bfloat16*>(kv.v);
  const int32_t* table = kv.table + static_cast<size_t>(seq) * kv.table_stride;
  const uint32_t ks_addr = static_cast<uint32_t>(__cvta_generic_to_shared(Ks));
  const uint32_t vs_addr = static_cast<uint32_t>(__cvta_generic_to_shared(Vs));

  auto load_tile = [&](int tile, int stage) {
    // two threads per key: the page lookup is done once per key and thread
    const int j = tid >> 1, kj = tile * kKeys + j;
    const bool valid = kj <= pmax;
    size_t slot = 0;
    // no page table: the keys and values are the step's own rows, row of position p = first + p - pos0
    if (valid) slot = kv.table ? static_cast<size_t>(table[kj / kv.page]) * kv.page + kj % kv.page
                               : static_cast<size_t>(first + max(kj - pos0, 0));
#pragma unroll
    for (int c = (tid & 1); c < KC + VC; c += 2) {
      if (c < KC) {
        const bool in = valid && c * 8 < dim;
        cp_async16(ks_addr + ((stage * kKeys + j) * LDK + c * 8) * 2,
                   in ? kbase + slot * kv.k_row + g * dim + c * 8 : kbase, in);
      } else {
        const bool in = valid && (c - KC) * 8 < vdim;
        cp_async16(vs_addr + ((stage * kKeys + j) * LDV + (c - KC) * 8) * 2,
                   in ? vbase + slot * kv.v_row + gv * vdim + (c - KC) * 8 : vbase, in);
      }
    }
    cp_async_commit();
  };

  if (tile_lo < tile_hi) load_tile(tile_of(tile_lo), 0);
  for (int li = tile_lo; li < tile_hi; ++li) {
    const int tile = tile_of(li);
    const int stage = (li - tile_lo) & 1;
    if (li + 1 < tile_hi) {
      load_tile(tile_of(li + 1), stage ^ 1);
      cp_async_wait<1>();
    } else {
      cp_async_wait<0>();
    }
    __syncthreads();
    const int k0 = tile * kKeys;
    // otherwise no row of this warp sees a key of the tile (all later, or all before every row's window)
    if (k0 <= warp_last && (window == 0 || k0 + kKeys - 1 > warp_first - window || k0 < keep_first)) {
      float s[kKeys / 8][4];
#pragma unroll
      for (int j = 0; j < kKeys / 8; ++j) s[j][0] = s[j][1] = s[j][2] = s[j][3] = 0.f;
      {
        // one ldmatrix.x4 = the key fragments (b0, b1) of two k-steps for 8 keys: lane l addresses key row l % 8 of
        // matrix l / 8 (matrices: dims +0, +8, +16, +24 of the same 8 keys)
        const uint32_t kt = ks_addr + (stage * kKeys * LDK + (lane & 7) * LDK + (lane >> 3) * 8) * 2;
#pragma unroll
        for (int ks = 0; ks < KS; ks += 2)
#pragma unroll
          for (int j = 0; j < kKeys / 8; ++j) {
            uint32_t b0, b1, b2, b3;
            ldmatrix_x4(kt + (j * 8 * LDK + ks * 16) * 2, b0, b1, b2, b3);
            mma_bf16(s[j], qf[ks], b0, b1);
            mma_bf16(s[j], qf[ks + 1], b2, b3);
          }
      }
      if (softcap > 0.f) {  // capped scores, then into units of log2 (the scale2 below is replaced by log2 e)
        const float inv = a.scale / softcap;
#pragma unroll
        for (int j = 0; j < kKeys / 8; ++j)
#pragma unroll
          for (int c = 0; c < 4; ++c) s[j][c] = softcap * tanhf(s[j][c] * inv);
      }
      const float scale2 = softcap > 0.f ? 1.4426950408889634f : scale2_plain;
      float mxA = -INFINITY, mxB = -INFINITY;
      if (k0 + kKeys - 1 <= warp_first && (window == 0 || warp_last - k0 < window)) {  // every row of the warp sees the whole tile
#pragma unroll
        for (int j = 0; j < kKeys / 8; ++j) {
          s[j][0] *= scale2, s[j][1] *= scale2, s[j][2] *= scale2, s[j][3] *= scale2;
          mxA = fmaxf(mxA, fmaxf(s[j][0], s[j][1]));
          mxB = fmaxf(mxB, fmaxf(s[j][2], s[j][3]));
        }
      } else {
#pragma unroll
        for (int j = 0; j < kKeys / 8; ++j) {
          const int kj = k0 + j * 8 + t4 * 2;
          const int loA = window > 0 ? posA - window : -1, loB = window > 0 ? posB - window : -1;  // the last key not seen
          s[j][0] = kj <= posA && (kj > loA || kj < keep_first) ? s[j][0] * scale2 : -INFINITY;
          s[j][1] = kj + 1 <= posA && (kj + 1 > loA || kj + 1 < keep_first) ? s[j][1] * scale2 : -INFINITY;
          s[j][2] = kj <= posB && (kj > loB || kj < keep_first) ? s[j][2] * scale2 : -INFINITY;
          s[j][3] = kj + 1 <= posB && (kj + 1 > loB || kj + 1 < keep_first) ? s[j][3] * scale2 : -INFINITY;
          mxA = fmaxf(mxA, fmaxf(s[j][0], s[j][1]));
          mxB = fmaxf(mxB, fmaxf(s[j][2], s[j][3]));
        }
      }
      const float nA = fmaxf(mA, quad_max(mxA)), nB = fmaxf(mB, quad_max(mxB));
      // a row that has seen nothing yet keeps max = -inf; subtracting 0 instead keeps 2^(-inf - 0) = 0 free of NaN
      const float subA = nA > -INFINITY ? nA : 0.f, subB = nB > -INFINITY ? nB : 0.f;
      const float alA = exp2_approx(mA - subA), alB = exp2_approx(mB - subB);
      float sumA = 0.f, sumB = 0.f;
#pragma unroll
      for (int j = 0; j < kKeys / 8; ++j) {
        s[j][0] = exp2_approx(s[j][0] - subA);
        s[j][1] = exp2_approx(s[j][1] - subA);
        s[j][2] = exp2_approx(s[j][2] - subB);
        s[j][3] = exp2_approx(s[j][3] - subB);
        sumA += s[j][0] + s[j][1];
        sumB += s[j][2] + s[j][3];
      }
      mA = nA, mB = nB;
      lA = lA * alA + sumA;  // the quad's partial sums are joined at the end (alpha is the same in a quad)
      lB = lB * alB + sumB;
#pragma unroll
      for (int nb = 0; nb < NB; ++nb) {
        o[nb][0] *= alA, o[nb][1] *= alA;
        o[nb][2] *= alB, o[nb][3] *= alB;
      }
      const uint32_t vt = vs_addr + stage * kKeys * LDV * 2;
      const int mi = lane >> 3;  // which of the four 8x8 matrices this lane addresses
#pragma unroll
      for (int kk = 0; kk < kKeys / 16; ++kk) {
        uint32_t hi[4], lo[4];
        split_pack(s[2 * kk][0], s[2 * kk][1], hi[0], lo[0]);
        split_pack(s[2 * kk][2], s[2 * kk][3], hi[1], lo[1]);
        split_pack(s[2 * kk + 1][0], s[2 * kk + 1][1], hi[2], lo[2]);
        split_pack(s[2 * kk + 1][2], s[2 * kk + 1][3], hi[3], lo[3]);
        const uint32_t row_addr = vt + ((kk * 16 + (mi & 1) * 8 + (lane & 7)) * LDV + (mi >> 1) * 8) * 2;
#pragma unroll
        for (int nb2 = 0; nb2 < NB / 2; ++nb2) {
          uint32_t b0, b1, b2, b3;
          ldmatrix_x4_trans(row_addr + nb2 * 16 * 2, b0, b1, b2, b3);
          mma_bf16(o[2 * nb2], hi, b0, b1);
          mma_bf16(o[2 * nb2], lo, b0, b1);
          mma_bf16(o[2 * nb2 + 1], hi, b2, b3);
          mma_bf16(o[2 * nb2 + 1], lo, b2, b3);
        }
      }
    }
    __syncthreads();  // the stage is loaded again two tiles on
  }
  lA = quad_sum(lA), lB = quad_sum(lB);
  if (splits == 1 && !a.no_merge) {
    if (a.sink != nullptr) {  // exp(sink) joins the denominator; scores are in units of log2
      constexpr float kLog2e = 1.4426950408889634f;
      if (exA) lA = mA > -INFINITY ? lA + exp2_approx(a.sink[thA % a.heads] * kLog2e - mA) : 1.0f;
      if (exB) lB = mB > -INFINITY ? lB + exp2_approx(a.sink[thB % a.heads] * kLog2e - mB) : 1.0f;
    }
    const bool per_element = gates != nullptr && a.gate == KLLM_SEQ_GATE_ELEMENT;
    const float gA = exA && gates && !per_element ? gates[thA] : 1.0f, gB = exB && gates && !per_element ? gates[thB] : 1.0f;
#pragma unroll
    for (int nb = 0; nb < NB; ++nb) {
      const int col = nb * 8 + t4 * 2;
      if (col >= vdim) break;
      float2 eA = make_float2(gA, gA), eB = make_float2(gB, gB);
      if (per_element) {
        if (exA) eA = *reinterpret_cast<const float2*>(gates + thA * vdim + col);
        if (exB) eB = *reinterpret_cast<const float2*>(gates + thB * vdim + col);
      }
      if (exA)
        *reinterpret_cast<__nv_bfloat162*>(out + thA * vdim + col) =
            __floats2bfloat162_rn(o[nb][0] / lA * eA.x, o[nb][1] / lA * eA.y);
      if (exB)
        *reinterpret_cast<__nv_bfloat162*>(out + thB * vdim + col) =
            __floats2bfloat162_rn(o[nb][2] / lB * eB.x, o[nb][3] / lB * eB.y);
    }
    return;
  }
  const int pstride = vdim + 2;
  float* pa = ws + (thA * splits + split) * pstride;
  float* pb = ws + (thB * splits + split) * pstride;
  if (t4 == 0) {
    constexpr float kLn2 = 0.6931471805599453f;  // the merge works with natural logarithms
    if (exA) pa[0] = mA * kLn2, pa[1] = lA;
    if (exB) pb[0] = mB * kLn2, pb[1] = lB;
  }
#pragma unroll
  for (int nb = 0; nb < NB; ++nb) {
    const int col = 2 + nb * 8 + t4 * 2;
    if (col >= pstride) break;
    if (exA) *reinterpret_cast<float2*>(pa + col) = make_float2(o[nb][0], o[nb][1]);
    if (exB) *reinterpret_cast<float2*>(pb + col) = make_float2(o[nb][2], o[nb][3]);
  }
}

template <int DIM, int VDIM>
int launch_mma(const AttnShape& a, const void* q, const float* gates, const PagedKV& kv, int n_entries,
               const int32_t* ent_first, const int32_t* ent_count, const int32_t* ent_seq, const int32_t* ent_pos0,
               int max_count, int splits, float* ws, void* out, cudaStream_t s) {
  constexpr size_t smem = 2 * kKeys * (DIM + 8 + VDIM + 8) * sizeof(__nv_bfloat16);
  static bool configured = false;
  if (smem > 48 * 1024 && !configured) {
    const cudaError_t e = cudaFuncSetAttribute(attention_mma_kernel<DIM, VDIM>,
                                               cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
    if (e != cudaSuccess) return cuda_rc(e);
    configured = true;
  }
  const int rep = a.heads / a.kv_heads;
  const dim3 grid(n_entries * a.kv_heads, (max_count * rep + kRows - 1) / kRows, splits);
  if (grid.y > 65535u) return KLLM_E_UNSUPPORTED;
  attention_mma_kernel<DIM, VDIM><<<grid, kThreads, smem, s>>>(
      a, static_cast<const __nv_bfloat16*>(q), kv, ent_first, ent_count, ent_seq, ent_pos0, splits, ws,
      a.gate ? gates : nullptr, static_cast<__nv_bfloat16*>(out));
  count_launch();
  return cuda_rc(cudaGetLastError());
}

}  // namespace

bool attention_mma_usable(int dtype, const AttnShape& a, int max_count) {
  if (dtype != KLLM_SEQ_BF16 || a.kv_heads <= 0 || a.heads % a.kv_heads) return false;
  // fp32 queries / outputs are the split-key kernel's
  if (a.q_f32 || a.out_f32) return false;
  const bool dims = a.dim % 8 == 0 && a.dim <= 256 && a.vdim % 8 == 0 && a.vdim <= 128;
  // steps of single tokens keep the split-key kernel (and stay capturable: no attribute call on their path)
  return dims && max_count >= 2 && max_count * (a.heads / a.kv_heads) >= 16;
}

int launch_attention_mma(const AttnShape& a, const void* q, const float* gates, const PagedKV& kv, int n_entries,
                         const int32_t* ent_first, const int32_t* ent_count, const int32_t* ent_seq,
                         const int32_t* ent_pos0, int max_count, int splits, float* ws, void* out, cudaStream_t s) {
#define KLLM_MMA(D, V)                                                                                             \
  if (a.dim <= D && a.vdim <= V)                                                                                   \
    return launch_mma<D, V>(a, q, gates, kv, n_entries, ent_first, ent_count, ent_seq, ent_pos0, max_count, splits, ws, \
                            out, s)
  KLLM_MMA(64, 64);
  KLLM_MMA(64, 128);
  KLLM_MMA(128, 64);
  KLLM_MMA(128, 128);
  KLLM_MMA(256, 128);
#undef KLLM_MMA
  return KLLM_E_UNSUPPORTED;
}

}  // namespace seq
}  // namespace kllm
