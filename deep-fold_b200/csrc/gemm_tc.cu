// Tensor-core NF4 GEMM for sm_100a: TMA -> dequant warps -> tcgen05.mma -> TMEM.
//
// y[M,N] = bf16( sum_k bf16(LUT[code]*scale)[m,k] * x[k,n] ), N <= 64 per call.
//
// One CTA owns a 128-row tile of W and walks its share of the K tiles (BK = 64 =
// one NF4 group) through a 4-stage ring:
//   warp 0      TMA producer: the packed 128 x 32-byte code tile of each stage
//               (cp.async.bulk.tensor.2d, no multicast) lands in shared memory.
//   warps 2..5  one thread per W row: reads its 32 code bytes, multiplies the
//               codebook value by the row's group scale in FP32, rounds once to
//               bf16 (the reference's A operand, bit for bit) and stores the row
//               into the stage's A tile in the K-major 128-byte-swizzled layout
//               tcgen05 reads; the same threads lay the x tile out K-major as B.
//   warp 1      one elected thread issues four tcgen05.mma (M=128, N=BN, K=16) per
//               stage, accumulating in TMEM, and commits the stage back to the ring.
//   warps 2..5  epilogue: tcgen05.ld of the 128 x BN FP32 accumulator, one row per
//               thread, bf16 store (or FP32 split-K partial).
// Group scales are fetched by the dequant threads with ordinary cached loads: the
// scale matrix's row pitch (K_pad/32 bytes) is not a multiple of 16 bytes for
// most shapes, which a TMA descriptor requires.
//
// Every mbarrier wait is bounded. A wait that runs out records a code in a device
// status word (read with chr_nf4_gemm_status), the role stops issuing work, the
// producer drains its copies in flight and the CTA still frees its TMEM.

#include <cuda.h>

#include <algorithm>

#include "gemm_plan.h"
#include <cstdlib>

#include "nf4_common.cuh"

namespace chr {

namespace {

constexpr int tBM = 128;
constexpr int tBK = 64;
constexpr int tStages = 4;
constexpr int tThreads = 192;
constexpr int tRawBytes = tBM * (tBK / 2);      // 4096
constexpr int tABytes = tBM * tBK * 2;          // 16384
constexpr uint32_t kSpinLimit = 1u << 18;       // bounded mbarrier waits

__device__ int g_gemm_status = 0;

__host__ __device__ constexpr int b_bytes(int bn) { return bn * tBK * 2; }
__host__ __device__ constexpr int stage_bytes(int bn) { return tRawBytes + tABytes + b_bytes(bn); }
__host__ __device__ constexpr int smem_bytes(int bn) { return tStages * stage_bytes(bn) + 1024 /*align*/ + 256 /*barriers*/; }

// ---- PTX wrappers -----------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void *p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}

__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}

__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes)
               : "memory");
}

// Returns false when the phase did not complete within the spin limit.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity) {
  for (uint32_t i = 0; i < kSpinLimit; ++i) {
    uint32_t done;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(done)
        : "r"(bar), "r"(parity)
        : "memory");
    if (done) return true;
  }
  return false;
}

__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap *map, uint32_t bar,
                                            int x, int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(dst), "l"(map), "r"(bar), "r"(x), "r"(y)
      : "memory");
}

__device__ __forceinline__ uint64_t umma_desc(uint32_t saddr) {
  // K-major, 128-byte swizzle: 8-row atoms of 1024 bytes (SBO), version 1.
  uint64_t d = static_cast<uint64_t>((saddr & 0x3FFFFu) >> 4);
  d |= static_cast<uint64_t>(1) << 16;            // leading byte offset (unused here)
  d |= static_cast<uint64_t>(1024 >> 4) << 32;    // stride byte offset
  d |= static_cast<uint64_t>(1) << 46;            // descriptor version (sm_100)
  d |= static_cast<uint64_t>(2) << 61;            // SWIZZLE_128B
  return d;
}

__device__ __forceinline__ void umma_bf16(uint32_t tmem_d, uint64_t da, uint64_t db, uint32_t idesc,
                                          uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, {%5, %5, %5, %5}, p;\n\t}"
      ::"r"(tmem_d), "l"(da), "l"(db), "r"(idesc), "r"(accumulate), "r"(0u)
      : "memory");
}

__device__ __forceinline__ void umma_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar)
               : "memory");
}

__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
        "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
        "=r"(r[14]), "=r"(r[15])
      : "r"(taddr));
}

// Two floats rounded to nearest-even bf16 in one conversion; lo lands in the low half.
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<const uint32_t *>(&v);
}

// ---- kernel -------------------------------------------------------------------
template <int BN>
__global__ void __launch_bounds__(tThreads, 1)
gemm_tc_kernel(const __grid_constant__ CUtensorMap packed_map, const uint16_t *__restrict__ scale,
               const __nv_bfloat16 *__restrict__ x, __nv_bfloat16 *__restrict__ y,
               float *__restrict__ partial, int M, int K, int K_pad, int N, int n_ktiles,
               int tiles_per_split) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  __shared__ float lut[16];
  __shared__ uint32_t tmem_slot;

  const int tid = threadIdx.x;
  const int warp = tid >> 5;
  const int lane = tid & 31;
  const int m0 = blockIdx.x * tBM;
  const int kt0 = blockIdx.y * tiles_per_split;
  const int kt1 = min(n_ktiles, kt0 + tiles_per_split);
  const int n_local = kt1 - kt0;

  // carve shared memory: stages (1024-byte aligned), then barriers
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  auto a_tile = [&](int s) { return base + s * tABytes; };
  auto b_tile = [&](int s) { return base + tStages * tABytes + s * b_bytes(BN); };
  auto raw_tile = [&](int s) { return base + tStages * (tABytes + b_bytes(BN)) + s * tRawBytes; };
  const uint32_t bars = base + tStages * stage_bytes(BN);
  auto raw_full = [&](int s) { return bars + 8 * s; };
  auto ab_full = [&](int s) { return bars + 8 * (tStages + s); };
  auto empty = [&](int s) { return bars + 8 * (2 * tStages + s); };
  const uint32_t acc_full = bars + 8 * (3 * tStages);

  if (tid < 16) lut[tid] = __uint_as_float(kLutBits[tid]);
  if (tid == 0) {
    for (int s = 0; s < tStages; ++s) {
      mbar_init(raw_full(s), 1);
      mbar_init(ab_full(s), 128);
      mbar_init(empty(s), 1);
    }
    mbar_init(acc_full, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    constexpr uint32_t cols = BN < 32 ? 32 : BN;
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                     smem_u32(&tmem_slot)),
                 "r"(cols));
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::);
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_d = tmem_slot;

  if (warp == 0) {
    // ---------------- TMA producer ----------------
    if (lane == 0) {
      bool ok = true;
      int issued = 0;
      for (int i = 0; i < n_local && ok; ++i) {
        const int s = i % tStages;
        if (i >= tStages) ok = mbar_wait(empty(s), ((i / tStages) - 1) & 1);
        if (!ok) break;
        mbar_expect_tx(raw_full(s), tRawBytes);
        tma_load_2d(raw_tile(s), &packed_map, raw_full(s), (kt0 + i) * (tBK / 2), m0);
        issued = i + 1;
      }
      if (!ok) {
        atomicExch(&g_gemm_status, 1);
        // drain: wait (bounded) for the copies this thread put in flight
        for (int i = max(0, issued - tStages); i < issued; ++i) {
          mbar_wait(raw_full(i % tStages), (i / tStages) & 1);
        }
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer ----------------
    if (lane == 0) {
      constexpr uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) |
                                 (static_cast<uint32_t>(BN >> 3) << 17) |
                                 (static_cast<uint32_t>(tBM >> 4) << 24);
      bool ok = true;
      for (int i = 0; i < n_local && ok; ++i) {
        const int s = i % tStages;
        ok = mbar_wait(ab_full(s), (i / tStages) & 1);
        if (!ok) break;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll
        for (int k4 = 0; k4 < tBK / 16; ++k4) {
          umma_bf16(tmem_d, umma_desc(a_tile(s) + k4 * 32), umma_desc(b_tile(s) + k4 * 32), idesc,
                    (i > 0 || k4 > 0) ? 1u : 0u);
        }
        umma_commit(empty(s));
      }
      if (ok) {
        umma_commit(acc_full);
      } else {
        atomicExch(&g_gemm_status, 2);
      }
    }
  } else {
    // ---------------- dequant + B fill (128 threads, one W row each) ----------------
    const int r = tid - 64;                 // 0..127
    const int grow = m0 + r;
    const bool row_live = grow < M;
    const int n_groups = K_pad / kGroup;
    const uint32_t a_row_off = static_cast<uint32_t>((r >> 3) * 1024 + (r & 7) * 128);
    const int sw = r & 7;
    bool ok = true;
    uint16_t s_bits = 0;
    if (row_live && n_local > 0) {
      s_bits = __ldg(scale + static_cast<size_t>(grow) * n_groups + kt0);
    }
    for (int i = 0; i < n_local && ok; ++i) {
      const int s = i % tStages;
      const int kt = kt0 + i;
      const float sc = row_live ? half_bits_to_float(s_bits) : 0.f;
      if (row_live && i + 1 < n_local) {
        s_bits = __ldg(scale + static_cast<size_t>(grow) * n_groups + kt + 1);
      }
      if (i >= tStages) ok = mbar_wait(empty(s), ((i / tStages) - 1) & 1);
      if (!ok) break;
      ok = mbar_wait(raw_full(s), (i / tStages) & 1);
      if (!ok) break;

      // A: this row's 64 codes -> 64 bf16, eight 16-byte chunks, chunk c at c ^ (row & 7)
      const uint32_t raw = raw_tile(s) + r * 32;
      const int k_base = kt * tBK;
#pragma unroll
      for (int hlf = 0; hlf < 2; ++hlf) {
        uint4 pk;
        asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];"
                     : "=r"(pk.x), "=r"(pk.y), "=r"(pk.z), "=r"(pk.w)
                     : "r"(raw + hlf * 16));
        const uint32_t wv[4] = {pk.x, pk.y, pk.z, pk.w};
#pragma unroll
        for (int c4 = 0; c4 < 4; ++c4) {
          const int c = hlf * 4 + c4;       // chunk of 8 codes
          uint32_t o[4];
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const uint32_t byte = (wv[c4] >> (8 * e)) & 0xFFu;
            const int k = k_base + c * 8 + 2 * e;
            float lo = lut[byte & 0xFu] * sc;
            float hi = lut[byte >> 4] * sc;
            if (k >= K) lo = 0.f;
            if (k + 1 >= K) hi = 0.f;
            o[e] = pack_bf16(lo, hi);
          }
          const uint32_t dst = a_tile(s) + a_row_off + static_cast<uint32_t>((c ^ sw) * 16);
          asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(dst), "r"(o[0]), "r"(o[1]),
                       "r"(o[2]), "r"(o[3])
                       : "memory");
        }
      }

      // B: x[k, n] (n contiguous in global) laid out K-major: row n, 64 k's, swizzled.
      // thread r: k = r / 2 of this tile, columns (r & 1) * BN/2 .. + BN/2.
      {
        const int kk = r >> 1;
        const int k = k_base + kk;
        const int n_first = (r & 1) * (BN / 2);
        const __nv_bfloat16 *src = x + static_cast<size_t>(k) * N;
        const uint32_t chunk = static_cast<uint32_t>(kk >> 3);
        const uint32_t within = static_cast<uint32_t>((kk & 7) * 2);
#pragma unroll
        for (int j = 0; j < BN / 2; ++j) {
          const int n = n_first + j;
          unsigned short v = 0;
          if (k < K && n < N) v = __bfloat16_as_ushort(src[n]);
          const uint32_t dst = b_tile(s) + static_cast<uint32_t>((n >> 3) * 1024 + (n & 7) * 128) +
                               ((chunk ^ static_cast<uint32_t>(n & 7)) * 16) + within;
          asm volatile("st.shared.u16 [%0], %1;" ::"r"(dst), "h"(v) : "memory");
        }
      }
      // generic-proxy writes -> visible to the tensor core (async proxy), then signal
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
      mbar_arrive(ab_full(s));
    }
    if (!ok) atomicExch(&g_gemm_status, 3);

    // ---------------- epilogue ----------------
    if (ok && n_local > 0) ok = mbar_wait(acc_full, 0);
    if (!ok) atomicExch(&g_gemm_status, 4);
    ok = __all_sync(0xffffffffu, ok);      // the TMEM loads below are warp-collective
    if (ok) {
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      const int quad = warp & 3;            // TMEM lane quadrant this warp may read
      const int row = m0 + quad * 32 + lane;
#pragma unroll
      for (int c0 = 0; c0 < BN; c0 += 16) {
        uint32_t v[16];
        if (n_local > 0) {
          tmem_ld16(tmem_d + (static_cast<uint32_t>(quad * 32) << 16) + c0, v);
          asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
        } else {
#pragma unroll
          for (int e = 0; e < 16; ++e) v[e] = 0u;
        }
        if (row < M) {
#pragma unroll
          for (int e = 0; e < 16; ++e) {
            const int n = c0 + e;
            if (n < N) {
              const float f = __uint_as_float(v[e]);
              if (partial != nullptr) {
                partial[(static_cast<size_t>(blockIdx.y) * M + row) * N + n] = f;
              } else {
                y[static_cast<size_t>(row) * N + n] = __float2bfloat16(f);
              }
            }
          }
        }
      }
    }
  }

  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == 1) {
    constexpr uint32_t cols = BN < 32 ? 32 : BN;
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_d), "r"(cols));
  }
}

// ---- host side -----------------------------------------------------------------
using EncodeTiled = CUresult (*)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *,
                                 const cuuint64_t *, const cuuint64_t *, const cuuint32_t *,
                                 const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle,
                                 CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiled encode_fn() {
  static EncodeTiled fn = [] {
    void *p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess ||
        q != cudaDriverEntryPointSuccess) {
      return static_cast<EncodeTiled>(nullptr);
    }
    return reinterpret_cast<EncodeTiled>(p);
  }();
  return fn;
}

template <int BN>
int launch(const chr_nf4_dev_t &w, const __nv_bfloat16 *x, __nv_bfloat16 *y, int N, float *partial,
           const chr_nf4_plan_t &p, cudaStream_t st) {
  EncodeTiled enc = encode_fn();
  if (enc == nullptr) return kLaunch;
  CUtensorMap map;
  const cuuint64_t dims[2] = {static_cast<cuuint64_t>(w.K_pad / 2), static_cast<cuuint64_t>(w.M)};
  const cuuint64_t strides[1] = {static_cast<cuuint64_t>(w.K_pad / 2)};
  const cuuint32_t box[2] = {tBK / 2, tBM};
  const cuuint32_t elem[2] = {1, 1};
  if (enc(&map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<uint8_t *>(w.packed), dims, strides,
          box, elem, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE,
          CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS) {
    return kLaunch;
  }
  static int attr_done[64] = {};  // per device
  if (!ensure_smem_attr(gemm_tc_kernel<BN>, smem_bytes(BN), attr_done)) return kLaunch;
  const dim3 grid(static_cast<unsigned>(p.grid_x), static_cast<unsigned>(p.grid_y));
  gemm_tc_kernel<BN><<<grid, tThreads, smem_bytes(BN), st>>>(
      map, w.scale, x, y, partial, w.M, w.K, w.K_pad, N, p.n_ktiles, p.tiles_per_split);
  return cudaGetLastError() == cudaSuccess ? kOk : kLaunch;
}

int bn_for(int N) { return N <= 16 ? 16 : (N <= 32 ? 32 : 64); }

// =============================================================================
// Wide GEMM on activation rows: y_rows[N, M] = x_rows[N, K] . dequant(W)^T
// =============================================================================
// Same pipeline, three differences: the activation tile is already K-major in
// global memory (row n of x_rows holds K contiguous values), so TMA loads it
// straight into the 128-byte-swizzled B tile; eight warps dequantize (two threads
// per W row, 32 codes each), which keeps the codebook work ahead of the tensor core
// at BN up to 256; the epilogue writes the transposed tile (consecutive lanes own
// consecutive m, so every store instruction covers 64 contiguous bytes).
#ifndef CHR_ROWS_DEQ_WARPS
#define CHR_ROWS_DEQ_WARPS 16
#endif
// warp 0 TMA, warp 1 MMA, then the dequant + epilogue warps: 128 rows x rParts threads
// per row. The dequant chain (lookup -> multiply -> round -> store) is latency-bound,
// so more warps per scheduler keep it ahead of the tensor core.
constexpr int rDequant = CHR_ROWS_DEQ_WARPS * 32;
constexpr int rThreads = 64 + rDequant;
static_assert(rDequant == 256 || rDequant == 512, "dequant warps: 8 or 16");
// MT: 128-row weight tiles per CTA. With two, a CTA multiplies 256 rows by the same
// activation tile (two TMEM accumulators), which halves the activation bytes pulled
// from L2 per flop: at MT = 1 and BN = 256 every K tile needs 36 KB per CTA, 6.5 TB/s
// over the chip at the rate measured, which is where the kernel stopped scaling.

__host__ __device__ constexpr int rows_stage_bytes(int bn, int mt = 1) {
  return mt * (tRawBytes + tABytes) + bn * tBK * 2;
}
__host__ __device__ constexpr int rows_stages(int bn, int mt = 1) {
  return mt > 1 ? 3 : (bn > 128 ? 4 : 6);
}
__host__ __device__ constexpr int rows_smem_bytes(int bn, int mt = 1) {
  return rows_stages(bn, mt) * rows_stage_bytes(bn, mt) + 1024 + 256;
}

template <int BN, int MT>
__global__ void __launch_bounds__(rThreads, 1)
gemm_rows_kernel(const __grid_constant__ CUtensorMap packed_map,
                 const __grid_constant__ CUtensorMap x_map, const uint16_t *__restrict__ scale,
                 __nv_bfloat16 *y, float *__restrict__ partial, const __nv_bfloat16 *__restrict__ bias,
                 const __nv_bfloat16 *add, int M, int K, int K_pad, int N, int n_ktiles,
                 int tiles_per_split) {
  constexpr int kStages = rows_stages(BN, MT);
  constexpr int kBBytes = BN * tBK * 2;
  constexpr int kABytes = MT * tABytes;
  constexpr int kRawBytes = MT * tRawBytes;
  constexpr uint32_t kAccCols = BN < 32 ? 32 : (BN <= 64 ? 64 : (BN <= 128 ? 128 : 256));
  constexpr uint32_t kCols = kAccCols * MT;
  static_assert(kCols <= 512, "TMEM columns");
  extern __shared__ __align__(16) unsigned char smem_raw[];
  __shared__ float lut[16];
  __shared__ uint32_t tmem_slot;

  const int tid = threadIdx.x;
  const int warp = tid >> 5;
  const int lane = tid & 31;
  const int m0 = blockIdx.x * tBM * MT;
  const int n0 = blockIdx.y * BN;
  const int kt0 = blockIdx.z * tiles_per_split;
  const int kt1 = min(n_ktiles, kt0 + tiles_per_split);
  const int n_local = kt1 - kt0;

  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  auto a_tile = [&](int s) { return base + s * kABytes; };  // MT tiles of tABytes each
  auto b_tile = [&](int s) { return base + kStages * kABytes + s * kBBytes; };
  auto raw_tile = [&](int s) { return base + kStages * (kABytes + kBBytes) + s * kRawBytes; };
  const uint32_t bars = base + kStages * rows_stage_bytes(BN, MT);
  auto in_full = [&](int s) { return bars + 8 * s; };                   // TMA: codes + x tile
  auto ab_full = [&](int s) { return bars + 8 * (kStages + s); };       // dequant done
  auto empty = [&](int s) { return bars + 8 * (2 * kStages + s); };     // MMA done with stage
  const uint32_t acc_full = bars + 8 * (3 * kStages);

  if (tid < 16) lut[tid] = __uint_as_float(kLutBits[tid]);
  if (tid == 0) {
    for (int s = 0; s < kStages; ++s) {
      mbar_init(in_full(s), 1);
      mbar_init(ab_full(s), tBM * MT);
      mbar_init(empty(s), 1);
    }
    mbar_init(acc_full, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                     smem_u32(&tmem_slot)),
                 "r"(kCols));
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::);
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_d = tmem_slot;

  if (warp == 0) {
    if (lane == 0) {
      bool ok = true;
      int issued = 0;
      for (int i = 0; i < n_local && ok; ++i) {
        const int s = i % kStages;
        if (i >= kStages) ok = mbar_wait(empty(s), ((i / kStages) - 1) & 1);
        if (!ok) break;
        mbar_expect_tx(in_full(s), kRawBytes + kBBytes);
        tma_load_2d(raw_tile(s), &packed_map, in_full(s), (kt0 + i) * (tBK / 2), m0);
        tma_load_2d(b_tile(s), &x_map, in_full(s), (kt0 + i) * tBK, n0);
        issued = i + 1;
      }
      if (!ok) {
        atomicExch(&g_gemm_status, 5);
        for (int i = max(0, issued - kStages); i < issued; ++i) {
          mbar_wait(in_full(i % kStages), (i / kStages) & 1);
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) |
                                 (static_cast<uint32_t>(BN >> 3) << 17) |
                                 (static_cast<uint32_t>(tBM >> 4) << 24);
      bool ok = true;
      for (int i = 0; i < n_local && ok; ++i) {
        const int s = i % kStages;
        ok = mbar_wait(ab_full(s), (i / kStages) & 1);
        if (!ok) break;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll
        for (int ti = 0; ti < MT; ++ti) {
#pragma unroll
          for (int k4 = 0; k4 < tBK / 16; ++k4) {
            umma_bf16(tmem_d + ti * kAccCols, umma_desc(a_tile(s) + ti * tABytes + k4 * 32),
                      umma_desc(b_tile(s) + k4 * 32), idesc, (i > 0 || k4 > 0) ? 1u : 0u);
          }
        }
        umma_commit(empty(s));
      }
      if (ok) {
        umma_commit(acc_full);
      } else {
        atomicExch(&g_gemm_status, 6);
      }
    }
  } else {
    // -------- dequant: one thread per (weight row, K tile) --------
    // A K tile is one NF4 group, so a row has ONE scale per tile: the thread rounds the
    // 16 products LUT[i] * scale to bf16 once (the reference's A operand, bit for bit:
    // gpu/nf4/nf4_gemm.cu:319-323 rounds LUT[code] * scale per weight, which is the same
    // 16 values), keeps them in registers as a low-byte and a high-byte plane, and turns
    // the tile's 64 codes into bf16 with byte permutes: no shared-memory lookup and no
    // multiply per weight. The thread groups take the K tiles in turn.
    constexpr int kRows = tBM * MT;
    constexpr int kTeams = rDequant / kRows;  // thread groups, one K tile each at a time
    static_assert(kTeams >= 1 && rDequant % kRows == 0, "dequant threads per row tile");
    const int t = tid - 64;
    const int r = t % kRows;                // row inside the CTA's MT tiles
    const int team = t / kRows;
    const int grow = m0 + r;
    const bool row_live = grow < M;
    const int n_groups = K_pad / kGroup;
    const int rr = r & (tBM - 1);           // row inside its 128-row tile
    const uint32_t a_row_off = static_cast<uint32_t>((r / tBM) * tABytes + (rr >> 3) * 1024 +
                                                     (rr & 7) * 128);
    const int sw = rr & 7;
    bool ok = true;
    // scales of this thread's next two K tiles are kept in flight
    const uint16_t *srow = scale + static_cast<size_t>(row_live ? grow : 0) * n_groups + kt0;
    uint16_t s_now = 0, s_next = 0;
    if (row_live && team < n_local) s_now = __ldg(srow + team);
    if (row_live && team + kTeams < n_local) s_next = __ldg(srow + team + kTeams);
    for (int i = team; i < n_local && ok; i += kTeams) {
      const int s = i % kStages;
      const int kt = kt0 + i;
      const float sc = row_live ? half_bits_to_float(s_now) : 0.f;
      s_now = s_next;
      if (row_live && i + 2 * kTeams < n_local) s_next = __ldg(srow + i + 2 * kTeams);
      // 16 scales share a 32-byte sector: ask for the row's next sector well ahead
      if (row_live && i + 24 < n_local) {
        asm volatile("prefetch.global.L1 [%0];" ::"l"(srow + i + 24));
      }
      // the 16 values of this (row, group), two bf16 per word, then as byte planes
      uint32_t lo_plane[4], hi_plane[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const uint32_t p0 = pack_bf16(lut[4 * j] * sc, lut[4 * j + 1] * sc);
        const uint32_t p1 = pack_bf16(lut[4 * j + 2] * sc, lut[4 * j + 3] * sc);
        lo_plane[j] = __byte_perm(p0, p1, 0x6420);
        hi_plane[j] = __byte_perm(p0, p1, 0x7531);
      }
      if (i >= kStages) ok = mbar_wait(empty(s), ((i / kStages) - 1) & 1);
      if (!ok) break;
      ok = mbar_wait(in_full(s), (i / kStages) & 1);
      if (!ok) break;
      uint32_t wv[8];
      asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];"
                   : "=r"(wv[0]), "=r"(wv[1]), "=r"(wv[2]), "=r"(wv[3])
                   : "r"(raw_tile(s) + r * 32));
      asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];"
                   : "=r"(wv[4]), "=r"(wv[5]), "=r"(wv[6]), "=r"(wv[7])
                   : "r"(raw_tile(s) + r * 32 + 16));
      const int k_base = kt * tBK;
      const bool whole = k_base + tBK <= K;  // no K tail inside this tile
#pragma unroll
      for (int c = 0; c < 8; ++c) {
        uint32_t o[4];
        // eight codes (nibbles, k order) -> eight bf16: entry = table[code & 7] from the
        // lower or the upper half of the table, chosen per byte by the code's bit 3. A
        // permute reads the low 16 bits of its selector: four codes per permute.
        const uint32_t sel8 = wv[c] & 0x77777777u;
        const uint32_t pick8 = ((wv[c] & 0x88888888u) >> 1) + 0x32103210u;
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          const uint32_t sel = h == 0 ? sel8 : sel8 >> 16;
          const uint32_t pick = h == 0 ? pick8 : pick8 >> 16;
          const uint32_t lo = __byte_perm(__byte_perm(lo_plane[0], lo_plane[1], sel),
                                          __byte_perm(lo_plane[2], lo_plane[3], sel), pick);
          const uint32_t hi = __byte_perm(__byte_perm(hi_plane[0], hi_plane[1], sel),
                                          __byte_perm(hi_plane[2], hi_plane[3], sel), pick);
          o[2 * h] = __byte_perm(lo, hi, 0x5140);
          o[2 * h + 1] = __byte_perm(lo, hi, 0x7362);
        }
        if (!whole) {
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const int k = k_base + c * 8 + 2 * e;
            if (k >= K) o[e] &= 0xFFFF0000u;
            if (k + 1 >= K) o[e] &= 0x0000FFFFu;
          }
        }
        const uint32_t dst = a_tile(s) + a_row_off + static_cast<uint32_t>((c ^ sw) * 16);
        asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(dst), "r"(o[0]), "r"(o[1]),
                     "r"(o[2]), "r"(o[3])
                     : "memory");
      }
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
      mbar_arrive(ab_full(s));
    }
    if (!ok) atomicExch(&g_gemm_status, 7);

    // ---------------- epilogue: two warps per TMEM lane quadrant ----------------
    if (ok && n_local > 0) ok = mbar_wait(acc_full, 0);
    if (!ok) atomicExch(&g_gemm_status, 8);
    ok = __all_sync(0xffffffffu, ok);
    if (ok && n_local > 0) {
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      const int quad = warp & 3;
      // warps of a TMEM lane quadrant share out the MT accumulators' columns, 16 at least
      constexpr int kWarpsPerQuad = rDequant / 128;
      constexpr int kUnits = MT * (BN / 16);                       // 16-column units in all
      constexpr int kGroups = kWarpsPerQuad < kUnits ? kWarpsPerQuad : kUnits;
      constexpr int kPerGroup = kUnits / kGroups * 16;             // columns per warp
      static_assert(kUnits % kGroups == 0 && BN % kPerGroup == 0, "epilogue split");
      const int col_group = (warp - 2) >> 2;
      const int g_begin = col_group * kPerGroup;                   // in the MT * BN column space
      const int ti = g_begin / BN;
      const int c_begin = g_begin - ti * BN;
      const int c_end = col_group < kGroups ? c_begin + kPerGroup : c_begin;
      const int row = m0 + ti * tBM + quad * 32 + lane;
      const float bias_row = (bias != nullptr && row < M) ? __bfloat162float(bias[row]) : 0.f;
      for (int c0 = c_begin; c0 < c_end; c0 += 16) {
        uint32_t v[16];
        tmem_ld16(tmem_d + (static_cast<uint32_t>(quad * 32) << 16) + ti * kAccCols + c0, v);
        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
        if (row < M) {
#pragma unroll
          for (int e = 0; e < 16; ++e) {
            const int n = n0 + c0 + e;
            if (n < N) {
              const float f = __uint_as_float(v[e]);
              if (partial != nullptr) {
                partial[(static_cast<size_t>(blockIdx.z) * N + n) * M + row] = f;
              } else {
                // bias and residual join the FP32 sum before its one rounding
                float out = f + bias_row;
                if (add != nullptr) out += __bfloat162float(add[static_cast<size_t>(n) * M + row]);
                y[static_cast<size_t>(n) * M + row] = __float2bfloat16(out);
              }
            }
          }
        }
      }
    }
  }

  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == 1) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_d), "r"(kCols));
  }
}

// y[n, m] = bf16( sum of the split-K partials (in split order) + bias[m] + add[n, m] )
__global__ void reduce_rows_kernel(const float *__restrict__ partial, __nv_bfloat16 *y,
                                   const __nv_bfloat16 *__restrict__ bias, const __nv_bfloat16 *add,
                                   long long total, int splits, int M) {
  const long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= total) return;
  float v = 0.f;
  for (int s = 0; s < splits; ++s) v += partial[static_cast<size_t>(s) * total + i];
  if (bias != nullptr) v += __bfloat162float(bias[i % M]);
  if (add != nullptr) v += __bfloat162float(add[i]);
  y[i] = __float2bfloat16(v);
}

struct RowsPlan {
  int bn, mt, grid_x, grid_y, split, tiles_per_split, n_ktiles;
  long long ws_floats;
};

int rows_force_mt() {  // CHR_NF4_ROWS_MT = 1 | 2 pins the M tiles per CTA (A/B runs)
  static int cached = -1;
  if (cached < 0) {
    const char *env = std::getenv("CHR_NF4_ROWS_MT");
    cached = (env != nullptr && (env[0] == '1' || env[0] == '2')) ? env[0] - '0' : 0;
  }
  return cached;
}

RowsPlan plan_rows(int M, int K_pad, int N, bool have_ws) {
  RowsPlan p{};
  const int n16 = ((N + 15) / 16) * 16;
  p.bn = n16 <= 32 ? 32 : (n16 <= 64 ? 64 : (n16 <= 128 ? 128 : 256));
  if (n16 <= 16) p.bn = 16;
  p.grid_y = (N + p.bn - 1) / p.bn;
  // two weight tiles per CTA once that still leaves at least two full waves of CTAs
  p.mt = 1;
  if (p.bn == 256) {
    const int ctas2 = ((M + 2 * tBM - 1) / (2 * tBM)) * p.grid_y;
    if (ctas2 >= 2 * sm_count()) p.mt = 2;
    if (rows_force_mt() != 0) p.mt = rows_force_mt();
  }
  p.grid_x = (M + tBM * p.mt - 1) / (tBM * p.mt);
  p.n_ktiles = (K_pad + tBK - 1) / tBK;
  // Split-K: with fewer CTAs than a few waves, cutting K lets a launch fill the SMs. The
  // count is chosen by a small cost model, not by "one full wave": 80 CTAs cut in two are
  // 160 CTAs = two waves on 148 SMs, no faster than one. Cost in microseconds: waves x
  // K tiles per CTA x time per K tile (tensor-bound at wide N, dequant-bound below) + the
  // reduction kernel (a launch and split x M x N floats of traffic).
  int want = 1;
  if (have_ws) {
    const int ctas = p.grid_x * p.grid_y;
    const int sms = sm_count();
    const double t_tile = std::max(0.30, 2.0 * tBM * p.mt * p.bn * tBK / 9.4e6);
    const int cap = p.n_ktiles / 8 > 0 ? p.n_ktiles / 8 : 1;  // at least eight K tiles per split
    double best = 0.0;
    for (int sp = 1; sp <= cap && sp <= 16; ++sp) {
      const int tiles = (p.n_ktiles + sp - 1) / sp;
      const int real = (p.n_ktiles + tiles - 1) / tiles;
      if (real != sp) continue;
      const int waves = (ctas * sp + sms - 1) / sms;
      double cost = static_cast<double>(waves) * tiles * t_tile;
      // partials are written by the GEMM and read back by the reduction: 8 bytes per
      // element and split, at the 2.5 TB/s such scattered FP32 traffic reaches
      if (sp > 1) cost += 4.0 + static_cast<double>(sp) * M * N * 8.0 / 2.5e6;
      if (sp == 1 || cost < best) {
        best = cost;
        want = sp;
      }
    }
  }
  p.tiles_per_split = (p.n_ktiles + want - 1) / want;
  p.split = (p.n_ktiles + p.tiles_per_split - 1) / p.tiles_per_split;
  p.ws_floats = p.split > 1 ? static_cast<long long>(p.split) * M * N : 0;
  return p;
}

template <int BN, int MT = 1>
int launch_rows(const chr_nf4_dev_t &w, const __nv_bfloat16 *x, __nv_bfloat16 *y, int N,
                float *partial, const __nv_bfloat16 *bias, const __nv_bfloat16 *add, const RowsPlan &p,
                cudaStream_t st) {
  EncodeTiled enc = encode_fn();
  if (enc == nullptr) return kLaunch;
  CUtensorMap wmap, xmap;
  {
    const cuuint64_t dims[2] = {static_cast<cuuint64_t>(w.K_pad / 2), static_cast<cuuint64_t>(w.M)};
    const cuuint64_t strides[1] = {static_cast<cuuint64_t>(w.K_pad / 2)};
    const cuuint32_t box[2] = {tBK / 2, static_cast<cuuint32_t>(tBM * MT)};
    const cuuint32_t elem[2] = {1, 1};
    if (enc(&wmap, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<uint8_t *>(w.packed), dims, strides,
            box, elem, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE,
            CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS) {
      return kLaunch;
    }
  }
  {
    const cuuint64_t dims[2] = {static_cast<cuuint64_t>(w.K), static_cast<cuuint64_t>(N)};
    const cuuint64_t strides[1] = {static_cast<cuuint64_t>(w.K) * 2};
    const cuuint32_t box[2] = {tBK, static_cast<cuuint32_t>(BN)};
    const cuuint32_t elem[2] = {1, 1};
    if (enc(&xmap, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<__nv_bfloat16 *>(x), dims,
            strides, box, elem, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
            CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS) {
      return kLaunch;
    }
  }
  static int attr_done[64] = {};  // per device
  if (!ensure_smem_attr(gemm_rows_kernel<BN, MT>, rows_smem_bytes(BN, MT), attr_done)) return kLaunch;
  const dim3 grid(static_cast<unsigned>(p.grid_x), static_cast<unsigned>(p.grid_y),
                  static_cast<unsigned>(p.split));
  gemm_rows_kernel<BN, MT><<<grid, rThreads, rows_smem_bytes(BN, MT), st>>>(
      wmap, xmap, w.scale, y, partial, bias, add, w.M, w.K, w.K_pad, N, p.n_ktiles, p.tiles_per_split);
  if (partial != nullptr) {
    const long long total = static_cast<long long>(w.M) * N;
    reduce_rows_kernel<<<static_cast<unsigned>((total + 255) / 256), 256, 0, st>>>(
        partial, y, bias, add, total, p.split, w.M);
  }
  return cudaGetLastError() == cudaSuccess ? kOk : kLaunch;
}


}  // namespace

TileShape tc_tile_shape(int N) {
  return TileShape{tBM, tBK, tThreads, smem_bytes(bn_for(N))};
}

bool tc_supported(int M, int K_pad, int N) {
  (void)M;
  // the packed row pitch must be a multiple of 16 bytes for the TMA descriptor
  return N >= 1 && N <= 64 && (K_pad / 2) % 16 == 0;
}

int launch_gemm_tc(const chr_nf4_dev_t &w, const __nv_bfloat16 *x, __nv_bfloat16 *y, int N,
                   float *partial, const chr_nf4_plan_t &p, cudaStream_t st) {
  switch (bn_for(N)) {
    case 16: return launch<16>(w, x, y, N, partial, p, st);
    case 32: return launch<32>(w, x, y, N, partial, p, st);
    default: return launch<64>(w, x, y, N, partial, p, st);
  }
}

}  // namespace chr

// Reads and clears the GEMM status word: 0 = every bounded wait completed; 1..4 =
// producer / MMA issuer / dequant / epilogue gave up on a wait. Synchronises the device.
extern "C" int chr_nf4_gemm_status(void) {
  int v = 0;
  if (cudaMemcpyFromSymbol(&v, chr::g_gemm_status, sizeof(int)) != cudaSuccess) return chr::kLaunch;
  if (v != 0) {
    const int zero = 0;
    cudaMemcpyToSymbol(chr::g_gemm_status, &zero, sizeof(int));
  }
  return v;
}

// Workspace (FP32 floats) chr_nf4_gemm_rows wants for this shape; 0 = none needed.
extern "C" int64_t chr_nf4_gemm_rows_ws(const chr_nf4_dev_t *w, int32_t N) {
  if (w == nullptr || N < 1 || w->M < 1 || w->K < 1 || !chr::k_pad_ok(w->K, w->K_pad)) return 0;
  return chr::plan_rows(w->M, w->K_pad, N, true).ws_floats;
}

extern "C" int chr_nf4_gemm_rows_add(const chr_nf4_dev_t *w, const void *x_rows, void *y_rows,
                                     int32_t N, const void *bias, const void *add_rows, float *ws,
                                     int64_t ws_floats, void *stream) {
  using namespace chr;
  if (x_rows == nullptr || y_rows == nullptr) return kNull;
  const int rc = check_matrix(w);
  if (rc != kOk) return rc;
  if (N < 1 || N > (1 << 20)) return kRangeN;
  if ((w->K % 8) != 0) return kDims;  // the activation row pitch must be a multiple of 16 bytes
  if (!aligned(w->packed, 16) || !aligned(x_rows, 16) || !aligned(w->scale, 2)) return kAlign;
  RowsPlan p = plan_rows(w->M, w->K_pad, N, ws != nullptr && ws_floats > 0);
  if (p.ws_floats > 0 && ws_floats < p.ws_floats) {
    p = plan_rows(w->M, w->K_pad, N, false);
    if (ws != nullptr && ws_floats > 0) return kWorkspace;
  }
  float *partial = p.split > 1 ? ws : nullptr;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  auto *xb = static_cast<const __nv_bfloat16 *>(x_rows);
  auto *yb = static_cast<__nv_bfloat16 *>(y_rows);
  auto *bb = static_cast<const __nv_bfloat16 *>(bias);
  auto *ab = static_cast<const __nv_bfloat16 *>(add_rows);
  switch (p.bn) {
    case 16: return launch_rows<16>(*w, xb, yb, N, partial, bb, ab, p, st);
    case 32: return launch_rows<32>(*w, xb, yb, N, partial, bb, ab, p, st);
    case 64: return launch_rows<64>(*w, xb, yb, N, partial, bb, ab, p, st);
    case 128: return launch_rows<128>(*w, xb, yb, N, partial, bb, ab, p, st);
    default:
      if (p.mt == 2) return launch_rows<256, 2>(*w, xb, yb, N, partial, bb, ab, p, st);
      return launch_rows<256>(*w, xb, yb, N, partial, bb, ab, p, st);
  }
}

extern "C" int chr_nf4_gemm_rows(const chr_nf4_dev_t *w, const void *x_rows, void *y_rows,
                                 int32_t N, float *ws, int64_t ws_floats, void *stream) {
  return chr_nf4_gemm_rows_add(w, x_rows, y_rows, N, nullptr, nullptr, ws, ws_floats, stream);
}
