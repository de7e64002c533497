// bf16 token-block product on the 5th-generation tensor cores (sm_100a):
//     out[T, N] (fp32) = a[T, K] (bf16) . w[N, K]^T (bf16), fp32 accumulation in TMEM
//
// One CTA computes 128 weight rows x BN tokens.  The weight rows are the M side of tcgen05.mma (so an accumulator lane
// is an output feature and a column is a token), the tokens the N side.  Six warps:
//   warp 0      TMA producer: cp.async.bulk.tensor 2-D tiles [128 x 64 bf16] of w and [BN x 64 bf16] of a, 128-byte
//               swizzle, into a ring of shared-memory stages guarded by full / empty mbarriers
//   warp 1      allocates the TMEM columns; one thread issues 4 x tcgen05.mma.cta_group::1.kind::f16 (K = 16 each) per
//               stage on shared-memory descriptors, tcgen05.commit releases the stage and, at the end, the accumulator
//   warps 2-5   epilogue: tcgen05.ld 32 lanes x 32 columns, coalesced stores (a warp's lanes are consecutive features)
// Rows and columns past the matrices are zero-filled by TMA and never stored.  K needs 16-byte rows (K % 8 == 0).
//
// Every mbarrier wait is bounded: a wait that runs out raises a flag in global memory (read by the host after the
// step), tells the other roles to stop, lets copies in flight land, frees the TMEM columns and returns.
#pragma once
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <cstdint>

#include "kllm_host.h"

namespace kllm {
namespace seq {
namespace umma {

constexpr int BM = 128;    // weight rows per CTA = MMA M
constexpr int BK = 64;     // bf16 elements per K block = 128 bytes = one swizzle row
constexpr int UK = 16;     // K of one tcgen05.mma.kind::f16
constexpr int STAGES = 4;
constexpr int A_BYTES = BM * BK * 2;
constexpr int THREADS = 192;
constexpr uint32_t kWaitLimit = 1u << 24;  // try_wait rounds before a wait gives up (each suspends up to ~1 us)

__device__ int g_error;  // != 0: a wait inside umma_kernel ran out

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }
__device__ __forceinline__ void mbar_init(uint32_t bar, int count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
// false: gave up (limit reached, or another role already did)
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* stop) {
  for (uint32_t i = 0; i < kWaitLimit; ++i) {
    uint32_t ok;
    asm volatile(
        "{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}"
        : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    if (ok) return true;
    if ((i & 1023u) == 1023u && *stop) return false;
  }
  *stop = 1;
  g_error = 1;
  return false;
}
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, uint32_t bar, int c0, int c1) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(bar), "r"(c0), "r"(c1) : "memory");
}
// K-major tile, 128-byte swizzle: start address >> 4 in bits [0,14), leading byte offset (unused with swizzle; 1) in
// [16,30), stride byte offset = 8 rows x 128 B = 1024 B >> 4 in [32,46), descriptor version 1 in [46,48), layout type
// SWIZZLE_128B = 2 in [61,64)
__device__ __forceinline__ uint64_t smem_desc(uint32_t saddr) {
  return static_cast<uint64_t>((saddr & 0x3FFFFu) >> 4) | (1ull << 16) | (64ull << 32) | (1ull << 46) | (2ull << 61);
}
// instruction descriptor: D = F32 (1 << 4), A = B = BF16 (1 << 7, 1 << 10), both K-major, N >> 3 in [17,23), M >> 4 in
// [24,29)
__device__ __forceinline__ uint32_t instr_desc(int n) {
  return (1u << 4) | (1u << 7) | (1u << 10) | (static_cast<uint32_t>(n >> 3) << 17) | (static_cast<uint32_t>(BM >> 4) << 24);
}
__device__ __forceinline__ void mma_bf16(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t acc) {
  asm volatile(
      "{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n"
      " tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}" ::"r"(tmem_d),
      "l"(adesc), "l"(bdesc), "r"(idesc), "r"(acc) : "memory");
}
__device__ __forceinline__ void mma_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}

__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
        "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
        "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr) : "memory");
}

template <int BN>
__global__ void __launch_bounds__(THREADS, 1)
umma_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_a,
            float* __restrict__ out, int T, int N, int K) {
  constexpr int B_BYTES = BN * BK * 2;
  constexpr uint32_t TMEM_COLS = BN < 32 ? 32 : BN;
  extern __shared__ uint8_t raw_smem[];
  uint8_t* base = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(raw_smem) + 1023) & ~uintptr_t(1023));
  uint8_t* a_tiles = base;                       // weight tiles (MMA A)
  uint8_t* b_tiles = base + STAGES * A_BYTES;    // token tiles (MMA B)
  uint64_t* bars = reinterpret_cast<uint64_t*>(b_tiles + STAGES * B_BYTES);
  uint64_t* full = bars;
  uint64_t* empty = bars + STAGES;
  uint64_t* tmem_full = bars + 2 * STAGES;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * STAGES + 1);
  volatile int* stop = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n0 = blockIdx.x * BM, t0 = blockIdx.y * BN;
  const int kblocks = (K + BK - 1) / BK;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(smem_u32(&full[s]), 1);
      mbar_init(smem_u32(&empty[s]), 1);
    }
    mbar_init(smem_u32(tmem_full), 1);
    *stop = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)),
                 "r"(TMEM_COLS) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_d = *tmem_slot;

  if (warp == 0) {
    if (lane == 0) {
      for (int kb = 0; kb < kblocks; ++kb) {
        const int s = kb % STAGES;
        if (!mbar_wait(smem_u32(&empty[s]), ((kb / STAGES) & 1) ^ 1u, stop)) break;
        const uint32_t bar = smem_u32(&full[s]);
        mbar_expect_tx(bar, A_BYTES + B_BYTES);
        tma_load_2d(smem_u32(a_tiles + s * A_BYTES), &map_w, bar, kb * BK, n0);
        tma_load_2d(smem_u32(b_tiles + s * B_BYTES), &map_a, bar, kb * BK, t0);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      const uint32_t idesc = instr_desc(BN);
      bool ok = true;
      for (int kb = 0; kb < kblocks && ok; ++kb) {
        const int s = kb % STAGES;
        ok = mbar_wait(smem_u32(&full[s]), (kb / STAGES) & 1, stop);
        if (!ok) break;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint32_t a_addr = smem_u32(a_tiles + s * A_BYTES);
        const uint32_t b_addr = smem_u32(b_tiles + s * B_BYTES);
#pragma unroll
        for (int k = 0; k < BK / UK; ++k)  // 32 bytes of K per instruction, inside the swizzle row
          mma_bf16(tmem_d, smem_desc(a_addr + k * UK * 2), smem_desc(b_addr + k * UK * 2), idesc, (kb > 0 || k > 0) ? 1u : 0u);
        mma_commit(smem_u32(&empty[s]));
      }
      if (ok) mma_commit(smem_u32(tmem_full));
    }
  } else {
    const int quarter = warp & 3;  // a warp may read TMEM lanes 32 * (warp % 4) .. + 31
    if (mbar_wait(smem_u32(tmem_full), 0u, stop)) {
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      const int row = n0 + quarter * 32 + lane;
#pragma unroll 1
      for (int c = 0; c < BN; c += 32) {
        uint32_t r[32];
        const uint32_t taddr = tmem_d + (static_cast<uint32_t>(quarter * 32) << 16) + static_cast<uint32_t>(c);
        asm volatile(
            "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
            "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
            "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
            : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
              "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
              "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
              "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
            : "r"(taddr) : "memory");
        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
        if (row < N) {
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            const int t = t0 + c + j;
            if (t < T) out[static_cast<size_t>(t) * N + row] = __uint_as_float(r[j]);
          }
        }
      }
    }
  }
  if (*stop) {  // a wait ran out: give copies in flight time to land before the shared memory is given up
    for (int i = 0; i < 1000; ++i) __nanosleep(1000);
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == 1) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_d), "r"(TMEM_COLS) : "memory");
  }
}

// ---- grouped form: blocks of 64 rows, each block against the weights of one expert ---------------------------------
// `a` holds the rows in sorted order ([n_blocks * 64, K], padding rows are zero), `w` the experts stacked along the rows.
// EPI 1: the weights of an expert are N gate rows followed by N up rows; both accumulate side by side in TMEM and
//        out[block row, n] = silu(gate) * up in bf16, still in sorted order (the next product reads it as its `a`).
// EPI 0: out[pair, n] = acc in fp32, pair = sorted_pair[block row] (rows of padding are skipped).
// EPI 2: one product; max(acc, 0)^2 in bf16, written in sorted order like EPI 1.
constexpr int GBN = 64;
template <int EPI>
__global__ void __launch_bounds__(THREADS, 1)
umma_grouped_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_a,
                    void* __restrict__ out_, const int32_t* __restrict__ sorted_pair,
                    const int32_t* __restrict__ block_expert, int N, int K, GatedAct act) {
  constexpr int NA = EPI == 1 ? 2 : 1;
  constexpr int B_BYTES = GBN * BK * 2;
  constexpr int STAGE = NA * A_BYTES + B_BYTES;
  constexpr uint32_t TMEM_COLS = NA * GBN;
  const int ex = block_expert[blockIdx.y];
  if (ex < 0) return;  // a block of padding only
  extern __shared__ uint8_t raw_smem[];
  uint8_t* base = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(raw_smem) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(base + STAGES * STAGE);
  uint64_t* full = bars;
  uint64_t* empty = bars + STAGES;
  uint64_t* tmem_full = bars + 2 * STAGES;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * STAGES + 1);
  volatile int* stop = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n0 = blockIdx.x * BM, r0 = blockIdx.y * GBN;
  const int kblocks = (K + BK - 1) / BK;
  const int wrow = ex * NA * N + n0;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(smem_u32(&full[s]), 1);
      mbar_init(smem_u32(&empty[s]), 1);
    }
    mbar_init(smem_u32(tmem_full), 1);
    *stop = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)),
                 "r"(TMEM_COLS) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_d = *tmem_slot;

  if (warp == 0) {
    if (lane == 0) {
      for (int kb = 0; kb < kblocks; ++kb) {
        const int s = kb % STAGES;
        if (!mbar_wait(smem_u32(&empty[s]), ((kb / STAGES) & 1) ^ 1u, stop)) break;
        const uint32_t bar = smem_u32(&full[s]);
        uint8_t* st = base + s * STAGE;
        mbar_expect_tx(bar, STAGE);
        tma_load_2d(smem_u32(st), &map_w, bar, kb * BK, wrow);
        if (NA == 2) tma_load_2d(smem_u32(st + A_BYTES), &map_w, bar, kb * BK, wrow + N);
        tma_load_2d(smem_u32(st + NA * A_BYTES), &map_a, bar, kb * BK, r0);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      const uint32_t idesc = instr_desc(GBN);
      bool ok = true;
      for (int kb = 0; kb < kblocks && ok; ++kb) {
        const int s = kb % STAGES;
        ok = mbar_wait(smem_u32(&full[s]), (kb / STAGES) & 1, stop);
        if (!ok) break;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint32_t st = smem_u32(base + s * STAGE);
        const uint32_t b_addr = st + NA * A_BYTES;
#pragma unroll
        for (int z = 0; z < NA; ++z)
#pragma unroll
          for (int k = 0; k < BK / UK; ++k)
            mma_bf16(tmem_d + z * GBN, smem_desc(st + z * A_BYTES + k * UK * 2), smem_desc(b_addr + k * UK * 2), idesc,
                     (kb > 0 || k > 0) ? 1u : 0u);
        mma_commit(smem_u32(&empty[s]));
      }
      if (ok) mma_commit(smem_u32(tmem_full));
    }
  } else {
    const int quarter = warp & 3;
    if (mbar_wait(smem_u32(tmem_full), 0u, stop)) {
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      const int row = n0 + quarter * 32 + lane;
#pragma unroll 1
      for (int c = 0; c < GBN; c += 32) {
        uint32_t r[32], u[32];
        const uint32_t taddr = tmem_d + (static_cast<uint32_t>(quarter * 32) << 16) + static_cast<uint32_t>(c);
        tmem_ld32(taddr, r);
        if (NA == 2) tmem_ld32(taddr + GBN, u);
        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
        if (row < N) {
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            const int br = r0 + c + j;
            if (EPI == 1) {
              const float g = __uint_as_float(r[j]), up = __uint_as_float(u[j]);
              static_cast<__nv_bfloat16*>(out_)[static_cast<size_t>(br) * N + row] =
                  __float2bfloat16_rn(gated_act(act, g, up));
            } else if (EPI == 2) {
              const float up = fmaxf(__uint_as_float(r[j]), 0.f);
              static_cast<__nv_bfloat16*>(out_)[static_cast<size_t>(br) * N + row] = __float2bfloat16_rn(up * up);
            } else {
              const int pair = sorted_pair[br];
              if (pair >= 0) static_cast<float*>(out_)[static_cast<size_t>(pair) * N + row] = __uint_as_float(r[j]);
            }
          }
        }
      }
    }
  }
  if (*stop) {
    for (int i = 0; i < 1000; ++i) __nanosleep(1000);
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == 1) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_d), "r"(TMEM_COLS) : "memory");
  }
}

// sorted copy of the rows the grouped product reads: row i = a[sorted_pair[i] / div] (zero where sorted_pair[i] < 0)
__global__ void gather_rows_kernel(const __nv_bfloat16* __restrict__ a, const int32_t* __restrict__ sorted_pair, int div,
                                   __nv_bfloat16* __restrict__ out, int K) {
  const int i = blockIdx.x;
  const int p = sorted_pair[i];
  uint4* dst = reinterpret_cast<uint4*>(out + static_cast<size_t>(i) * K);
  if (p < 0) {
    for (int k = threadIdx.x; k < K / 8; k += blockDim.x) dst[k] = make_uint4(0, 0, 0, 0);
  } else {
    const uint4* src = reinterpret_cast<const uint4*>(a + static_cast<size_t>(p / div) * K);
    for (int k = threadIdx.x; k < K / 8; k += blockDim.x) dst[k] = src[k];
  }
}

// ---- host ---------------------------------------------------------------------------------------------------------
using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                   const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                   CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
// cuTensorMapEncodeTiled is looked up at run time, so that the library loads on a machine without a driver
inline EncodeTiledFn encode_tiled() {
  static EncodeTiledFn fn = [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess ||
        q != cudaDriverEntryPointSuccess)
      p = nullptr;
    return reinterpret_cast<EncodeTiledFn>(p);
  }();
  return fn;
}
// [rows, cols] bf16 row-major, box [box_rows x 64 columns], 128-byte swizzle
inline int make_map(CUtensorMap* map, const void* ptr, int rows, int cols, int box_rows) {
  EncodeTiledFn fn = encode_tiled();
  if (fn == nullptr) return KLLM_E_NODEVICE;
  const cuuint64_t dims[2] = {static_cast<cuuint64_t>(cols), static_cast<cuuint64_t>(rows)};
  const cuuint64_t strides[1] = {static_cast<cuuint64_t>(cols) * 2};
  const cuuint32_t box[2] = {static_cast<cuuint32_t>(BK), static_cast<cuuint32_t>(box_rows)};
  const cuuint32_t estr[2] = {1, 1};
  const CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, estr,
                        CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : KLLM_E_INVALID;
}

template <int BN>
inline int launch_bn(const void* a, const void* w, float* out, int T, int K, int N, cudaStream_t stream) {
  CUtensorMap map_w, map_a;
  if (int rc = make_map(&map_w, w, N, K, BM)) return rc;
  if (int rc = make_map(&map_a, a, T, K, BN)) return rc;
  const size_t smem = 1024 + static_cast<size_t>(STAGES) * (A_BYTES + BN * BK * 2) + 256;
  static bool configured = false;
  if (!configured) {
    const cudaError_t e = cudaFuncSetAttribute(umma_kernel<BN>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                               static_cast<int>(smem));
    if (e != cudaSuccess) return static_cast<int>(e);
    configured = true;
  }
  const dim3 grid((N + BM - 1) / BM, (T + BN - 1) / BN);
  umma_kernel<BN><<<grid, THREADS, smem, stream>>>(map_w, map_a, out, T, N, K);
  count_launch();
  return static_cast<int>(cudaGetLastError());
}

template <typename AT>
inline bool usable(const AT*, const AT*, int, int, int) { return false; }
template <>
inline bool usable<__nv_bfloat16>(const __nv_bfloat16* a, const __nv_bfloat16* w, int T, int K, int N) {
  static const bool off = [] { const char* e = getenv("KLLM_SEQ_UMMA"); return e != nullptr && e[0] == '0'; }();
  return !off && T >= 64 && K >= BK && (K % 8) == 0 && N >= 8 && (reinterpret_cast<uintptr_t>(a) & 15) == 0 &&
         (reinterpret_cast<uintptr_t>(w) & 15) == 0;
}

template <typename AT>
inline int launch(const AT*, const AT*, float*, int, int, int, cudaStream_t) { return KLLM_E_UNSUPPORTED; }
template <>
inline int launch<__nv_bfloat16>(const __nv_bfloat16* a, const __nv_bfloat16* w, float* out, int T, int K, int N,
                                 cudaStream_t s) {
  // few feature tiles: narrower token blocks give more CTAs
  const int feature_tiles = (N + BM - 1) / BM;
  if (T <= 64 || feature_tiles * ((T + 127) / 128) < 100) return launch_bn<64>(a, w, out, T, K, N, s);
  if (T <= 128 || feature_tiles * ((T + 255) / 256) < 148) return launch_bn<128>(a, w, out, T, K, N, s);
  return launch_bn<256>(a, w, out, T, K, N, s);
}

inline bool grouped_usable(int K, int N) {
  static const bool off = [] { const char* e = getenv("KLLM_SEQ_UMMA"); return e != nullptr && e[0] == '0'; }();
  return !off && K >= BK && (K % 8) == 0 && N >= 8;
}

// a: [n_blocks * 64, K] bf16 in sorted order; w: [experts * (EPI ? 2 : 1) * N, K]
template <int EPI>
inline int launch_grouped(const void* a, const void* w, void* out, const int32_t* sorted_pair, const int32_t* block_expert,
                          int n_blocks, int experts, int K, int N, cudaStream_t stream,
                          GatedAct act = GatedAct{KLLM_SEQ_ACT_SWIGLU, 0.f, 0.f}) {
  CUtensorMap map_w, map_a;
  if (int rc = make_map(&map_w, w, experts * (EPI == 1 ? 2 : 1) * N, K, BM)) return rc;
  if (int rc = make_map(&map_a, a, n_blocks * GBN, K, GBN)) return rc;
  const size_t smem = 1024 + static_cast<size_t>(STAGES) * ((EPI == 1 ? 2 : 1) * A_BYTES + GBN * BK * 2) + 256;
  static bool configured = false;
  if (!configured) {
    const cudaError_t e = cudaFuncSetAttribute(umma_grouped_kernel<EPI>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                               static_cast<int>(smem));
    if (e != cudaSuccess) return static_cast<int>(e);
    configured = true;
  }
  const dim3 grid((N + BM - 1) / BM, n_blocks);
  umma_grouped_kernel<EPI><<<grid, THREADS, smem, stream>>>(map_w, map_a, out, sorted_pair, block_expert, N, K, act);
  count_launch();
  return static_cast<int>(cudaGetLastError());
}

// 1 when a wait inside the kernel ran out since the last call; clears the flag
inline int take_error() {
  int v = 0;
  if (cudaMemcpyFromSymbol(&v, g_error, sizeof(int)) != cudaSuccess) return 0;
  if (v) {
    const int zero = 0;
    cudaMemcpyToSymbol(g_error, &zero, sizeof(int));
  }
  return v;
}

}  // namespace umma
}  // namespace seq
}  // namespace kllm
