// Decode-side NF4 GEMV family for sm_100a: y = dequant(W) . x on CUDA cores.
//
// The path is HBM-bound by design and at 4.25 bits per weight the dequant ALU
// work is what threatens that bound, so the inner loop is three instructions
// per packed byte (two weights):
//   * one byte-permute builds the shared-memory address (code byte << 8 | lane*8),
//   * one 8-byte shared load fetches the pair (LUT[low nibble], LUT[high nibble])
//     as exact FP32 from a 256-entry table replicated once per lane, which makes
//     every lookup bank-conflict free whatever the codes are,
//   * one packed FP32 FMA (fma.rn.f32x2) multiplies the pair with (x_even, x_odd).
// x stays in registers: a lane always owns the same 32 consecutive k of each
// 1024-wide chunk, for every row, so x is read once per CTA. The group scale is
// applied once per 32 codes, after the unscaled FP32 sum. Packed codes and scales
// are streamed with 128-bit / 16-bit no-allocate loads, double-buffered in
// registers one row tile ahead.
//
// Work split: a CTA of S*G warps owns tiles of G*R rows; warp (g, s) walks rows
// g*R..g*R+R-1 of each tile over K slice s (C chunks of 1024). Slice partials are
// combined in shared memory in slice order, so results do not depend on the grid
// and repeat bit for bit. One persistent CTA per SM strides over the tiles.
//
// Numerics followed (reference: gpu/nf4/nf4_gemv.cu:58-80,232-243,383-389,483-494):
// weights are LUT*scale in FP32 (never rounded to bf16), FP32 accumulation, one
// rounding to bf16 after the optional residual / bias / SwiGLU. The summation
// order differs from the reference's, which stays inside its 1e-2 tolerance.

#include "nf4_common.cuh"

namespace chr {
namespace {

constexpr int kChunk = 1024;        // k per warp-wide 16-byte load
#ifndef CHR_GEMV_MAX_WARPS
#define CHR_GEMV_MAX_WARPS 16
#endif
constexpr int kMaxWarps = CHR_GEMV_MAX_WARPS;
constexpr int kTabBytes = 65536;    // 256 byte values x 32 lanes x float2
constexpr int kHeadBytes = 16384;   // partial sums + RMS scratch in front of the table
constexpr int kSmemBytes = kHeadBytes + 2 * kTabBytes;  // room to place the table on a 64 KiB boundary

struct GemvArgs {
  const uint8_t *packed[3];
  const uint16_t *scale[3];
  __nv_bfloat16 *y[3];
  float *y32;                     // MODE 0 only: when set, the FP32 sum is stored unrounded
  const __nv_bfloat16 *extra[3];  // residual (plain) or bias (fused q/k/v); may be null
  int rows_end[3];                // prefix sums of the matrices' M in the fused row space
  int n_rows;                     // rows in the fused space (SwiGLU: M of gate)
  int K;
  int K_pad;
  const __nv_bfloat16 *x;
  const __nv_bfloat16 *rms_w;
  float rms_eps;
  int S;        // K slices (warps per row)
  int G;        // row groups per CTA
  int n_tiles;  // ceil(n_rows / (G * R))
};

// Sum R per-lane values over the warp with half the shuffles of R butterflies.
// Returns, in every lane, the warp total of value index ((lane >> 4) & 1) for R == 2,
// ((lane >> 3) & 3) for R == 4, and of v[0] for R == 1. Fixed order: deterministic.
template <int R>
__device__ __forceinline__ float warp_reduce_rows(float (&v)[R], int lane) {
  if constexpr (R == 4) {
    const bool hi = (lane & 16) != 0;
    float s0 = hi ? v[0] : v[2];
    float s1 = hi ? v[1] : v[3];
    float k0 = hi ? v[2] : v[0];
    float k1 = hi ? v[3] : v[1];
    k0 += __shfl_xor_sync(0xffffffffu, s0, 16);
    k1 += __shfl_xor_sync(0xffffffffu, s1, 16);
    const bool hi8 = (lane & 8) != 0;
    const float send = hi8 ? k0 : k1;
    float keep = hi8 ? k1 : k0;
    keep += __shfl_xor_sync(0xffffffffu, send, 8);
#pragma unroll
    for (int off = 4; off > 0; off >>= 1) keep += __shfl_xor_sync(0xffffffffu, keep, off);
    return keep;  // row index = (lane>>4)*2 + ((lane>>3)&1)
  } else if constexpr (R == 2) {
    const bool hi = (lane & 16) != 0;
    const float send = hi ? v[0] : v[1];
    float keep = hi ? v[1] : v[0];
    keep += __shfl_xor_sync(0xffffffffu, send, 16);
#pragma unroll
    for (int off = 8; off > 0; off >>= 1) keep += __shfl_xor_sync(0xffffffffu, keep, off);
    return keep;  // row index = lane >> 4
  } else {
    return warp_sum_xor(v[0]);
  }
}

template <int R>
__device__ __forceinline__ int reduced_row_of_lane(int lane) {
  if constexpr (R == 4) return ((lane >> 4) << 1) | ((lane >> 3) & 1);
  if constexpr (R == 2) return lane >> 4;
  return 0;
}

// Four code bytes (8 weights): four byte-permutes build the table addresses
// (byte0 <- tab_lane.byte0, byte1 <- code byte, bytes 2,3 <- tab_lane), four 8-byte
// shared loads fetch the (low, high) codebook pairs, four packed FMAs accumulate.
// One asm statement, so nothing is scheduled in between by the front end.
template <bool FIRST>
__device__ __forceinline__ void dot8(uint32_t w, uint32_t tab_lane, f32x2_t x0, f32x2_t x1,
                                     f32x2_t x2, f32x2_t x3, f32x2_t &acc0, f32x2_t &acc1) {
  if constexpr (FIRST) {
    asm volatile(
        "{\n\t.reg .b32 a0, a1, a2, a3;\n\t.reg .b64 t0, t1, t2, t3;\n\t"
        "prmt.b32 a0, %2, %3, 0x7604;\n\t"
        "prmt.b32 a1, %2, %3, 0x7614;\n\t"
        "prmt.b32 a2, %2, %3, 0x7624;\n\t"
        "prmt.b32 a3, %2, %3, 0x7634;\n\t"
        "ld.shared.b64 t0, [a0];\n\t"
        "ld.shared.b64 t1, [a1];\n\t"
        "ld.shared.b64 t2, [a2];\n\t"
        "ld.shared.b64 t3, [a3];\n\t"
        "mul.rn.f32x2 %0, t0, %4;\n\t"
        "mul.rn.f32x2 %1, t1, %5;\n\t"
        "fma.rn.f32x2 %0, t2, %6, %0;\n\t"
        "fma.rn.f32x2 %1, t3, %7, %1;\n\t}"
        : "=&l"(acc0), "=&l"(acc1)
        : "r"(w), "r"(tab_lane), "l"(x0), "l"(x1), "l"(x2), "l"(x3));
  } else {
    asm volatile(
        "{\n\t.reg .b32 a0, a1, a2, a3;\n\t.reg .b64 t0, t1, t2, t3;\n\t"
        "prmt.b32 a0, %2, %3, 0x7604;\n\t"
        "prmt.b32 a1, %2, %3, 0x7614;\n\t"
        "prmt.b32 a2, %2, %3, 0x7624;\n\t"
        "prmt.b32 a3, %2, %3, 0x7634;\n\t"
        "ld.shared.b64 t0, [a0];\n\t"
        "ld.shared.b64 t1, [a1];\n\t"
        "ld.shared.b64 t2, [a2];\n\t"
        "ld.shared.b64 t3, [a3];\n\t"
        "fma.rn.f32x2 %0, t0, %4, %0;\n\t"
        "fma.rn.f32x2 %1, t1, %5, %1;\n\t"
        "fma.rn.f32x2 %0, t2, %6, %0;\n\t"
        "fma.rn.f32x2 %1, t3, %7, %1;\n\t}"
        : "+l"(acc0), "+l"(acc1)
        : "r"(w), "r"(tab_lane), "l"(x0), "l"(x1), "l"(x2), "l"(x3));
  }
}

// Unscaled dot of 32 codes (one uint4) with the lane's 32 x values (16 packed pairs).
__device__ __forceinline__ float dot32(const uint4 pk, const f32x2_t (&xr)[16], uint32_t tab_lane) {
  f32x2_t acc0, acc1;
  dot8<true>(pk.x, tab_lane, xr[0], xr[1], xr[2], xr[3], acc0, acc1);
  dot8<false>(pk.y, tab_lane, xr[4], xr[5], xr[6], xr[7], acc0, acc1);
  dot8<false>(pk.z, tab_lane, xr[8], xr[9], xr[10], xr[11], acc0, acc1);
  dot8<false>(pk.w, tab_lane, xr[12], xr[13], xr[14], xr[15], acc0, acc1);
  float e0, o0, e1, o1;
  unpack_f32x2(acc0, e0, o0);
  unpack_f32x2(acc1, e1, o1);
  return (e0 + e1) + (o0 + o1);
}

// MODE 0: one matrix (+ residual). MODE 1: SwiGLU (gate, up). MODE 2: fused q, k, v
// rows in one row space (+ bias each).
template <int R, int C, int MODE>
__global__ void __launch_bounds__(kMaxWarps * 32, 1)
nf4_gemv_kernel(const GemvArgs a) {
  extern __shared__ __align__(16) unsigned char smem[];
  constexpr int RW = (MODE == 1) ? 2 * R : R;  // weight rows per warp per tile
  const int tid = threadIdx.x;
  const int lane = tid & 31;
  const int warp = tid >> 5;
  const int s = warp % a.S;
  const int g = warp / a.S;

  float *part = reinterpret_cast<float *>(smem);  // [2][S][G*RW]

  const int rt = a.G * R;                 // unit rows per tile
  const int half_stride = a.K_pad >> 1;   // bytes per packed row
  const int n_groups = a.K_pad / kGroup;
  const int last_row = a.n_rows - 1;
  const int last_tile = a.n_tiles - 1;
  bool chunk_live[C];
#pragma unroll
  for (int j = 0; j < C; ++j) chunk_live[j] = (s * C + j) * kChunk + lane * 32 < a.K_pad;
  // this lane's byte / scale offset inside any row (chunk j adds j*512 bytes, j*16 scales)
  const size_t lane_pk = static_cast<size_t>(s) * C * (kChunk / 2) + static_cast<size_t>(lane) * 16;
  const size_t lane_sc = static_cast<size_t>(s) * C * (kChunk / kGroup) + static_cast<size_t>(lane >> 1);

  uint4 cur[RW][C], nxt[RW][C];
  uint16_t cur_s[RW][C], nxt_s[RW][C];

  // Rows and tiles past the end are clamped to the last one: every load stays in
  // bounds without a branch, the duplicates are dropped at the store.
  auto issue = [&](int tile, uint4 (&pk)[RW][C], uint16_t (&sc)[RW][C]) {
    const int row0 = min(tile, last_tile) * rt + g * R;
#pragma unroll
    for (int i = 0; i < RW; ++i) {
      const int unit = min(row0 + (MODE == 1 ? (i >> 1) : i), last_row);
      const uint8_t *pr;
      const uint16_t *sr;
      if constexpr (MODE == 1) {
        pr = ((i & 1) ? a.packed[1] : a.packed[0]) + static_cast<size_t>(unit) * half_stride;
        sr = ((i & 1) ? a.scale[1] : a.scale[0]) + static_cast<size_t>(unit) * n_groups;
      } else if constexpr (MODE == 0) {
        pr = a.packed[0] + static_cast<size_t>(unit) * half_stride;
        sr = a.scale[0] + static_cast<size_t>(unit) * n_groups;
      } else {
        const int m = (unit >= a.rows_end[0]) + (unit >= a.rows_end[1]);
        const int local = unit - (m == 0 ? 0 : (m == 1 ? a.rows_end[0] : a.rows_end[1]));
        pr = (m == 0 ? a.packed[0] : (m == 1 ? a.packed[1] : a.packed[2])) +
             static_cast<size_t>(local) * half_stride;
        sr = (m == 0 ? a.scale[0] : (m == 1 ? a.scale[1] : a.scale[2])) +
             static_cast<size_t>(local) * n_groups;
      }
      pr += lane_pk;
      sr += lane_sc;
#pragma unroll
      for (int j = 0; j < C; ++j) {
        if (chunk_live[j]) {
          pk[i][j] = ld_stream16(pr + j * (kChunk / 2));
          sc[i][j] = ld_stream_u16(sr + j * (kChunk / kGroup));
        } else {
          pk[i][j] = make_uint4(0x77777777u, 0x77777777u, 0x77777777u, 0x77777777u);
          sc[i][j] = 0;
        }
      }
    }
  };

  // The first tile's weights depend on nothing the previous kernel writes: put them
  // in flight, and let the next kernel of the chain start launching, before the
  // table is built and x is read.
  pdl_trigger();
  int tile = blockIdx.x;
  issue(tile, cur, cur_s);

  // Table on a 64 KiB boundary of the shared window so that a byte-permute can
  // splice the code byte into address bits 8..15. Entry (b, l) at b*256 + l*8.
  const uint32_t smem_base = static_cast<uint32_t>(__cvta_generic_to_shared(smem));
  const uint32_t tab_base = (smem_base + kHeadBytes + 0xFFFFu) & ~0xFFFFu;
  for (int i = tid; i < 256 * 32; i += blockDim.x) {
    const int b = i >> 5;
    const float lo = __uint_as_float(kLutBits[b & 15]);
    const float hi = __uint_as_float(kLutBits[b >> 4]);
    const uint32_t addr = tab_base + static_cast<uint32_t>(i) * 8u;
    asm volatile("st.shared.v2.f32 [%0], {%1,%2};" ::"r"(addr), "f"(lo), "f"(hi));
  }
  const uint32_t tab_lane = tab_base + static_cast<uint32_t>(lane) * 8u;

  // x (and the residual / outputs) belong to the previous kernel until it completes.
  pdl_wait();

  // Optional fused RMSNorm: every warp derives the same scale on its own.
  float inv = 1.f;
  if (a.rms_w != nullptr) {
    inv = rsqrtf(warp_sumsq_bf16(a.x, a.K, lane) / static_cast<float>(a.K) + a.rms_eps);
  }

  // The lane's x values for its K slice as packed (even, odd) pairs, zero at and beyond K.
  f32x2_t xr[C][16];
#pragma unroll
  for (int j = 0; j < C; ++j) {
    const int k0 = (s * C + j) * kChunk + lane * 32;
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      const int k = k0 + q * 8;
      uint4 xv = make_uint4(0u, 0u, 0u, 0u);
      uint4 wv = make_uint4(0u, 0u, 0u, 0u);
      if (k + 8 <= a.K) {
        xv = __ldg(reinterpret_cast<const uint4 *>(a.x + k));
        if (a.rms_w != nullptr) wv = __ldg(reinterpret_cast<const uint4 *>(a.rms_w + k));
      } else if (k < a.K) {
        __nv_bfloat16 tx[8], tw[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          const bool in = k + e < a.K;
          tx[e] = in ? a.x[k + e] : __float2bfloat16(0.f);
          tw[e] = (in && a.rms_w != nullptr) ? a.rms_w[k + e] : __float2bfloat16(0.f);
        }
        xv = *reinterpret_cast<const uint4 *>(tx);
        wv = *reinterpret_cast<const uint4 *>(tw);
      }
      const uint32_t xw[4] = {xv.x, xv.y, xv.z, xv.w};
      const uint32_t ww[4] = {wv.x, wv.y, wv.z, wv.w};
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        float lo = bf16_lo(xw[e]);
        float hi = bf16_hi(xw[e]);
        if (a.rms_w != nullptr) {
          lo = __bfloat162float(__float2bfloat16(bf16_lo(ww[e]) * lo * inv));
          hi = __bfloat162float(__float2bfloat16(bf16_hi(ww[e]) * hi * inv));
        }
        xr[j][q * 4 + e] = pack_f32x2(lo, hi);
      }
    }
  }
  __syncthreads();  // table is ready

  // Output routing of a unit row (MODE 2 only needs the three-way split).
  auto store_plain = [&](int unit, float v) {
    if (unit >= a.n_rows) return;
    if constexpr (MODE == 2) {
      const int m = (unit >= a.rows_end[0]) + (unit >= a.rows_end[1]);
      const int local = unit - (m == 0 ? 0 : (m == 1 ? a.rows_end[0] : a.rows_end[1]));
      const __nv_bfloat16 *ex = m == 0 ? a.extra[0] : (m == 1 ? a.extra[1] : a.extra[2]);
      __nv_bfloat16 *yo = m == 0 ? a.y[0] : (m == 1 ? a.y[1] : a.y[2]);
      if (ex != nullptr) v += __bfloat162float(ex[local]);
      yo[local] = __float2bfloat16(v);
    } else {
      if (a.extra[0] != nullptr) v += __bfloat162float(a.extra[0][unit]);
      if (a.y32 != nullptr) {
        a.y32[unit] = v;
      } else {
        a.y[0][unit] = __float2bfloat16(v);
      }
    }
  };

  int buf = 0;
  auto process = [&](int tile, const uint4 (&pk)[RW][C], const uint16_t (&sc)[RW][C]) {
    float sum[RW];
#pragma unroll
    for (int i = 0; i < RW; ++i) {
      sum[i] = 0.f;
#pragma unroll
      for (int j = 0; j < C; ++j) {
        const float d = dot32(pk[i][j], xr[j], tab_lane);
        sum[i] = fmaf(half_bits_to_float(sc[i][j]), d, sum[i]);
      }
    }
    const float tot = warp_reduce_rows<RW>(sum, lane);
    const int my = reduced_row_of_lane<RW>(lane);  // weight-row index this lane holds
    constexpr int lanes_per = 32 / RW;

    if (a.S > 1) {
      float *pb = part + buf * (kMaxWarps * 8);
      if ((lane & (lanes_per - 1)) == 0) pb[s * (a.G * RW) + g * RW + my] = tot;
      __syncthreads();
      if (tid < rt) {
        const int unit = tile * rt + tid;
        if constexpr (MODE == 1) {
          float gsum = 0.f, usum = 0.f;
          for (int q = 0; q < a.S; ++q) {
            gsum += pb[q * (a.G * RW) + 2 * tid];
            usum += pb[q * (a.G * RW) + 2 * tid + 1];
          }
          if (unit < a.n_rows) {
            a.y[0][unit] = __float2bfloat16((gsum / (1.f + expf(-gsum))) * usum);
          }
        } else {
          float v = 0.f;
          for (int q = 0; q < a.S; ++q) v += pb[q * (a.G * RW) + tid];
          store_plain(unit, v);
        }
      }
      buf ^= 1;
    } else {
      if constexpr (MODE == 1) {
        // lanes of weight-row 2u hold gate, of 2u+1 hold up: fetch the partner.
        const float other = __shfl_xor_sync(0xffffffffu, tot, lanes_per);
        if ((lane & (2 * lanes_per - 1)) == 0) {
          const int unit = tile * rt + g * R + (my >> 1);
          if (unit < a.n_rows) {
            a.y[0][unit] = __float2bfloat16((tot / (1.f + expf(-tot))) * other);
          }
        }
      } else {
        if ((lane & (lanes_per - 1)) == 0) store_plain(tile * rt + g * R + my, tot);
      }
    }
  };

  // Two register buffers alternate: the next tile's loads are in flight while the
  // current tile is reduced.
  const int stride = gridDim.x;
  while (tile < a.n_tiles) {
    issue(tile + stride, nxt, nxt_s);
    process(tile, cur, cur_s);
    tile += stride;
    if (tile >= a.n_tiles) break;
    issue(tile + stride, cur, cur_s);
    process(tile, nxt, nxt_s);
    tile += stride;
  }
}

struct Shape {
  int R, C, S, G, n_tiles, grid;
};

// K slices of C*1024 per warp, up to 16 warps per CTA. Rows per warp (R) and row
// groups per CTA (G) minimise the number of passes the busiest SM makes, with a
// small per-tile charge so that long matrices amortise the reduction.
Shape pick_shape(int n_rows, int K_pad, bool swiglu) {
  Shape best{0, 0, 0, 0, 0, 0};
  const int n_chunks = (K_pad + kChunk - 1) / kChunk;
  const int C = n_chunks >= 2 ? 2 : 1;
  const int S = (n_chunks + C - 1) / C;
  if (S > kMaxWarps) return best;
  const int sms = sm_count();
  const int rmax = (swiglu ? 2 : 4) / C;  // keeps both register buffers at <= 4 loads
  float best_cost = 0.f;
  for (int G = kMaxWarps / S; G >= 1; G >>= 1) {
    for (int R = rmax; R >= 1; R >>= 1) {
      const int tiles = (n_rows + G * R - 1) / (G * R);
      const int passes = (tiles + sms - 1) / sms;
      const float cost = static_cast<float>(passes) * (static_cast<float>(R) + 0.25f);
      if (best.R == 0 || cost < best_cost) {
        best_cost = cost;
        best = Shape{R, C, S, G, tiles, tiles < sms ? tiles : sms};
      }
    }
  }
  return best;
}

template <int MODE>
int launch(const GemvArgs &proto, cudaStream_t st) {
  constexpr bool swiglu = MODE == 1;
  GemvArgs a = proto;
  const Shape sh = pick_shape(a.n_rows, a.K_pad, swiglu);
  if (sh.R == 0) return kDims;  // K beyond 16 slices of 2048 is not supported by this path
  a.S = sh.S;
  a.G = sh.G;
  a.n_tiles = sh.n_tiles;
  const dim3 grid(static_cast<unsigned>(sh.grid));
  const dim3 block(static_cast<unsigned>(sh.S * sh.G * 32));

#define CHR_LAUNCH(RR, CC)                                                                   \
  do {                                                                                       \
    static bool attr_done = false;                                                           \
    if (!attr_done) {                                                                        \
      if (cudaFuncSetAttribute(nf4_gemv_kernel<RR, CC, MODE>,                                \
                               cudaFuncAttributeMaxDynamicSharedMemorySize,                  \
                               kSmemBytes) != cudaSuccess) {                                 \
        return kLaunch;                                                                      \
      }                                                                                      \
      attr_done = true;                                                                      \
    }                                                                                        \
    if (launch_chain(nf4_gemv_kernel<RR, CC, MODE>, grid, block, kSmemBytes, st, a) !=       \
        cudaSuccess) {                                                                       \
      return kLaunch;                                                                        \
    }                                                                                        \
  } while (0)

  if (sh.C == 2) {
    if (sh.R == 2) {
      if constexpr (MODE != 1) CHR_LAUNCH(2, 2); else return kLaunch;
    } else {
      CHR_LAUNCH(1, 2);
    }
  } else {
    if (sh.R == 4) {
      if constexpr (MODE != 1) CHR_LAUNCH(4, 1); else return kLaunch;
    } else if (sh.R == 2) {
      CHR_LAUNCH(2, 1);
    } else {
      CHR_LAUNCH(1, 1);
    }
  }
#undef CHR_LAUNCH
  return cudaGetLastError() == cudaSuccess ? kOk : kLaunch;
}

}  // namespace
}  // namespace chr

using namespace chr;

extern "C" int chr_nf4_gemv(const chr_nf4_dev_t *w, const void *x, void *y, void *stream,
                            const void *add, const void *rms_w, float rms_eps) {
  if (w == nullptr || x == nullptr || y == nullptr) return kNull;
  const int rc = check_matrix(w);
  if (rc != kOk) return rc;
  if (!aligned(w->packed, 16) || !aligned(x, 16) || !aligned(w->scale, 2)) return kAlign;
  GemvArgs a{};
  a.packed[0] = w->packed;
  a.scale[0] = w->scale;
  a.y[0] = static_cast<__nv_bfloat16 *>(y);
  a.extra[0] = static_cast<const __nv_bfloat16 *>(add);
  a.rows_end[0] = a.rows_end[1] = a.rows_end[2] = w->M;
  a.n_rows = w->M;
  a.K = w->K;
  a.K_pad = w->K_pad;
  a.x = static_cast<const __nv_bfloat16 *>(x);
  a.rms_w = static_cast<const __nv_bfloat16 *>(rms_w);
  a.rms_eps = rms_eps;
  return launch<0>(a, static_cast<cudaStream_t>(stream));
}

extern "C" int chr_nf4_gemv_f32(const chr_nf4_dev_t *w, const void *x, float *y, void *stream,
                                const void *add, const void *rms_w, float rms_eps) {
  if (w == nullptr || x == nullptr || y == nullptr) return kNull;
  const int rc = check_matrix(w);
  if (rc != kOk) return rc;
  if (!aligned(w->packed, 16) || !aligned(x, 16) || !aligned(w->scale, 2)) return kAlign;
  GemvArgs a{};
  a.packed[0] = w->packed;
  a.scale[0] = w->scale;
  a.y32 = y;
  a.extra[0] = static_cast<const __nv_bfloat16 *>(add);
  a.rows_end[0] = a.rows_end[1] = a.rows_end[2] = w->M;
  a.n_rows = w->M;
  a.K = w->K;
  a.K_pad = w->K_pad;
  a.x = static_cast<const __nv_bfloat16 *>(x);
  a.rms_w = static_cast<const __nv_bfloat16 *>(rms_w);
  a.rms_eps = rms_eps;
  return launch<0>(a, static_cast<cudaStream_t>(stream));
}

extern "C" int chr_nf4_gemv_qkv(const chr_nf4_dev_t *q, const chr_nf4_dev_t *k,
                                const chr_nf4_dev_t *v, const void *x, void *yq, void *yk,
                                void *yv, const void *bq, const void *bk, const void *bv,
                                void *stream, const void *rms_w, float rms_eps) {
  if (q == nullptr || k == nullptr || v == nullptr || x == nullptr || yq == nullptr ||
      yk == nullptr || yv == nullptr) {
    return kNull;
  }
  if (q->M < 1 || k->M < 1 || v->M < 1 || q->K < 1) return kDims;
  if (k->K != q->K || v->K != q->K || k->K_pad != q->K_pad || v->K_pad != q->K_pad) return kDims;
  if (q->packed == nullptr || k->packed == nullptr || v->packed == nullptr ||
      q->scale == nullptr || k->scale == nullptr || v->scale == nullptr) {
    return kDims;
  }
  if (!k_pad_ok(q->K, q->K_pad)) return kKPad;
  if (!aligned(q->packed, 16) || !aligned(k->packed, 16) || !aligned(v->packed, 16) ||
      !aligned(x, 16)) {
    return kAlign;
  }
  GemvArgs a{};
  const chr_nf4_dev_t *m[3] = {q, k, v};
  void *ys[3] = {yq, yk, yv};
  const void *bs[3] = {bq, bk, bv};
  int end = 0;
  for (int i = 0; i < 3; ++i) {
    a.packed[i] = m[i]->packed;
    a.scale[i] = m[i]->scale;
    a.y[i] = static_cast<__nv_bfloat16 *>(ys[i]);
    a.extra[i] = static_cast<const __nv_bfloat16 *>(bs[i]);
    end += m[i]->M;
    a.rows_end[i] = end;
  }
  a.n_rows = end;
  a.K = q->K;
  a.K_pad = q->K_pad;
  a.x = static_cast<const __nv_bfloat16 *>(x);
  a.rms_w = static_cast<const __nv_bfloat16 *>(rms_w);
  a.rms_eps = rms_eps;
  return launch<2>(a, static_cast<cudaStream_t>(stream));
}

extern "C" int chr_nf4_gemv_swiglu(const chr_nf4_dev_t *gate, const chr_nf4_dev_t *up,
                                   const void *x, void *y, void *stream, const void *rms_w,
                                   float rms_eps) {
  if (gate == nullptr || up == nullptr || x == nullptr || y == nullptr) return kNull;
  if (gate->M < 1 || gate->K < 1 || up->M != gate->M || up->K != gate->K ||
      up->K_pad != gate->K_pad) {
    return kDims;
  }
  if (gate->packed == nullptr || up->packed == nullptr || gate->scale == nullptr ||
      up->scale == nullptr) {
    return kDims;
  }
  if (!k_pad_ok(gate->K, gate->K_pad)) return kKPad;
  if (!aligned(gate->packed, 16) || !aligned(up->packed, 16) || !aligned(x, 16)) return kAlign;
  GemvArgs a{};
  a.packed[0] = gate->packed;
  a.scale[0] = gate->scale;
  a.packed[1] = up->packed;
  a.scale[1] = up->scale;
  a.y[0] = static_cast<__nv_bfloat16 *>(y);
  a.rows_end[0] = a.rows_end[1] = a.rows_end[2] = gate->M;
  a.n_rows = gate->M;
  a.K = gate->K;
  a.K_pad = gate->K_pad;
  a.x = static_cast<const __nv_bfloat16 *>(x);
  a.rms_w = static_cast<const __nv_bfloat16 *>(rms_w);
  a.rms_eps = rms_eps;
  return launch<1>(a, static_cast<cudaStream_t>(stream));
}
