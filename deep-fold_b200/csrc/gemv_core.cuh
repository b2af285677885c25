// Device core of the decode-side NF4 GEMV family (sm_100a), shared by the
// one-matrix-per-launch kernels and by the whole-step persistent kernel.
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
// and repeat bit for bit. CTAs stride over the tiles.
//
// Numerics followed (reference: gpu/nf4/nf4_gemv.cu:58-80,232-243,383-389,483-494):
// weights are LUT*scale in FP32 (never rounded to bf16), FP32 accumulation, one
// rounding to bf16 after the optional residual / bias / SwiGLU. The summation
// order differs from the reference's, which stays inside its 1e-2 tolerance.
#pragma once

#include <cstdlib>

#include "nf4_common.cuh"

namespace chr {

constexpr int kChunk = 1024;        // k per warp-wide 16-byte load
#ifndef CHR_GEMV_MAX_WARPS
#define CHR_GEMV_MAX_WARPS 16
#endif
constexpr int kMaxWarps = CHR_GEMV_MAX_WARPS;
constexpr int kTabBytes = 65536;    // 256 byte values x 32 lanes x float2
// Dynamic shared memory of the kernels that use the pair table:
//   [ slice partials kPartBytes | head: staged x (or attention scratch) | pad | table 64 KiB ]
// The table is the LAST 64 KiB of the allocation and must start on a 64 KiB
// boundary of the shared window. Dynamic shared memory starts a few hundred bytes
// into the window (the driver reserves 1 KiB; these kernels declare no static
// shared memory), so the host asks for exactly as much as puts the end of the
// allocation on a boundary: 127 KiB when partials + head fit in 63 KiB. Keeping the
// footprint there matters: the unified L1 holds the weight loads in flight, and at
// 208 KiB of shared memory the 16 warps' 64 KiB of outstanding loads no longer fit
// in what is left of it (measured: lm_head 49 -> 60 us, gate+up 10.7 -> 12.2 us).
constexpr int kPartBytes = 2048;
constexpr int kWindowBytes = 65536;

// Offset of dynamic shared memory inside the shared window for kernels without
// static shared memory, measured once per device by a probe launch (not capturable:
// the first launch on a device must happen outside stream capture).
int smem_window_offset();

// Bytes to request so that the table (last 64 KiB) is aligned; 0 when partials +
// head_bytes cannot be placed in front of it within the 227 KiB a CTA may have.
inline int table_smem_request(int head_bytes) {
  const int off = smem_window_offset();
  if (off < 0) return 0;
  const int front = off + kPartBytes + head_bytes;
  const int table_at = (front + kWindowBytes - 1) / kWindowBytes * kWindowBytes;
  const int request = table_at - off + kTabBytes;
  return request <= 232448 ? request : 0;
}

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

// Activation loads. Inside the persistent step kernel x, the residual and the
// RMSNorm input were written by other CTAs of the same launch, so they are read
// through L2 (ld.global.cg), never through the non-coherent path.
__device__ __forceinline__ uint4 ld_act16(const void *p) {
  return __ldcg(reinterpret_cast<const uint4 *>(p));
}
__device__ __forceinline__ float ld_act_bf16(const __nv_bfloat16 *p) {
  return bf16_lo(static_cast<uint32_t>(__ldcg(reinterpret_cast<const unsigned short *>(p))));
}

// sum(x^2) with the same order as warp_sumsq_bf16 (identical bits), L2-coherent loads.
__device__ __forceinline__ float warp_sumsq_act(const __nv_bfloat16 *x, int n, int lane) {
  float acc = 0.f;
  const int n8 = n >> 3;
#pragma unroll 4
  for (int g = lane; g < n8; g += 32) {
    const uint4 v = ld_act16(x + 8 * g);
    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const float lo = bf16_lo(w[e]);
      const float hi = bf16_hi(w[e]);
      acc = fmaf(lo, lo, acc);
      acc = fmaf(hi, hi, acc);
    }
  }
  for (int i = (n8 << 3) + lane; i < n; i += 32) {
    const float v = ld_act_bf16(x + i);
    acc = fmaf(v, v, acc);
  }
  return warp_sum_xor(acc);
}

// Fill the 64 KiB lookup table at tab_base (a 64 KiB-aligned shared address):
// entry (b, l) at b*256 + l*8 holds (LUT[b & 15], LUT[b >> 4]) as FP32.
__device__ __forceinline__ void build_pair_table(uint32_t tab_base, int tid, int n_threads) {
  for (int i = tid; i < 256 * 32; i += n_threads) {
    const int b = i >> 5;
    const float lo = __uint_as_float(kLutBits[b & 15]);
    const float hi = __uint_as_float(kLutBits[b >> 4]);
    const uint32_t addr = tab_base + static_cast<uint32_t>(i) * 8u;
    asm volatile("st.shared.v2.f32 [%0], {%1,%2};" ::"r"(addr), "f"(lo), "f"(hi));
  }
}

// Shared address of the table: the last 64 KiB of the dynamic allocation. Returns 0
// (never a valid table address) if the host's sizing did not land it on a boundary.
__device__ __forceinline__ uint32_t pair_table_base(const void *smem) {
  const uint32_t smem_base = static_cast<uint32_t>(__cvta_generic_to_shared(smem));
  uint32_t dyn;
  asm("mov.u32 %0, %%dynamic_smem_size;" : "=r"(dyn));
  const uint32_t tab = smem_base + dyn - kTabBytes;
  return (dyn >= kTabBytes && (tab & 0xFFFFu) == 0u) ? tab : 0u;
}

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
//
// One GEMV over the CTA's tiles first_tile, first_tile + tile_stride, ... . Every
// thread of the CTA must call it (it uses __syncthreads); warps beyond S*G only
// take part in the barriers. `part` is kMaxWarps*16 floats of shared memory, `xs`
// 16-byte aligned shared room for K (rounded up to 8) bf16 values, `tab_lane` the
// lane's slot in the pair table. `wait()` is called by every thread once the first
// tile's weights are in flight and before any activation is read: it is where the
// caller orders itself behind the producer of x (and fills the table; the barrier
// after the staging of x publishes it).
template <int R, int C, int MODE, class Wait>
__device__ __forceinline__ void gemv_run(const GemvArgs &a, float *part, __nv_bfloat16 *xs,
                                         uint32_t tab_lane, int first_tile, int tile_stride,
                                         Wait wait) {
  constexpr int RW = (MODE == 1) ? 2 * R : R;  // weight rows per warp per tile
  const int tid = threadIdx.x;
  const int lane = tid & 31;
  const int warp = tid >> 5;
  const bool live_warp = warp < a.S * a.G;
  const int s = warp % a.S;
  const int g = warp / a.S;

  const int rt = a.G * R;                 // unit rows per tile
  const int half_stride = a.K_pad >> 1;   // bytes per packed row
  const int n_groups = a.K_pad / kGroup;
  const int last_row = a.n_rows - 1;
  const int last_tile = a.n_tiles - 1;
  bool chunk_live[C];
#pragma unroll
  for (int j = 0; j < C; ++j) {
    chunk_live[j] = (s * C + j) * kChunk + lane * 32 < a.K_pad;
  }
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

  // The first tile's weights depend on nothing the producer of x writes: put them
  // in flight before waiting for it.
  int tile = first_tile;
  const bool any = tile < a.n_tiles;
  if (any && live_warp) issue(tile, cur, cur_s);

  // The RMSNorm weights are constants too: fetch the lane's slice before waiting, so
  // that after the wait only x itself is on the critical path.
  uint4 wv[C][4];
#pragma unroll
  for (int j = 0; j < C; ++j) {
    const int k0 = (s * C + j) * kChunk + lane * 32;
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      const int k = k0 + q * 8;
      wv[j][q] = make_uint4(0u, 0u, 0u, 0u);
      if (any && live_warp && a.rms_w != nullptr && k < a.K) {
        if (k + 8 <= a.K) {
          wv[j][q] = __ldg(reinterpret_cast<const uint4 *>(a.rms_w + k));
        } else {
          __nv_bfloat16 tw[8];
#pragma unroll
          for (int e = 0; e < 8; ++e) {
            tw[e] = k + e < a.K ? a.rms_w[k + e] : __float2bfloat16(0.f);
          }
          wv[j][q] = *reinterpret_cast<const uint4 *>(tw);
        }
      }
    }
  }
  wait();
  if (!any) return;

  // x is staged once per CTA in shared memory (L2-coherent loads: inside the
  // persistent step kernel it was written by other CTAs of the same launch), so the
  // S*G warps do not each fetch it from L2.
  uint4 *xs4 = reinterpret_cast<uint4 *>(xs);
  const int n8 = (a.K + 7) >> 3;
  for (int i = tid; i < n8; i += blockDim.x) {
    const int k = i * 8;
    uint4 v;
    if (k + 8 <= a.K) {
      v = ld_act16(a.x + k);
    } else {
      __nv_bfloat16 t[8];
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        t[e] = __float2bfloat16(k + e < a.K ? ld_act_bf16(a.x + k + e) : 0.f);
      }
      v = *reinterpret_cast<const uint4 *>(t);
    }
    xs4[i] = v;
  }
  __syncthreads();

  // Optional fused RMSNorm. sum(x^2) is taken by every live warp over the staged
  // copy in the order of warp_sumsq_bf16 (lane l owns the 8-element groups l, l+32,
  // ...; zero padding adds nothing), so every kernel that needs the scale gets the
  // same bits.
  // Warps beyond S*G have nothing more to do: the barriers below count S*G warps.
  if (!live_warp) return;
  const int live_threads = a.S * a.G * 32;
  float inv = 1.f;
  if (a.rms_w != nullptr) {
    float acc = 0.f;
#pragma unroll 4
    for (int g8 = lane; g8 < n8; g8 += 32) {
      const uint4 v = xs4[g8];
      const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float lo = bf16_lo(w[e]);
        const float hi = bf16_hi(w[e]);
        acc = fmaf(lo, lo, acc);
        acc = fmaf(hi, hi, acc);
      }
    }
    inv = rsqrtf(warp_sum_xor(acc) / static_cast<float>(a.K) + a.rms_eps);
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
      if (k < a.K) xv = xs4[k >> 3];
      const uint32_t xw[4] = {xv.x, xv.y, xv.z, xv.w};
      const uint32_t ww[4] = {wv[j][q].x, wv[j][q].y, wv[j][q].z, wv[j][q].w};
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

  // Output routing of a unit row (MODE 2 only needs the three-way split).
  auto store_plain = [&](int unit, float v) {
    if (unit >= a.n_rows) return;
    if constexpr (MODE == 2) {
      const int m = (unit >= a.rows_end[0]) + (unit >= a.rows_end[1]);
      const int local = unit - (m == 0 ? 0 : (m == 1 ? a.rows_end[0] : a.rows_end[1]));
      const __nv_bfloat16 *ex = m == 0 ? a.extra[0] : (m == 1 ? a.extra[1] : a.extra[2]);
      __nv_bfloat16 *yo = m == 0 ? a.y[0] : (m == 1 ? a.y[1] : a.y[2]);
      if (ex != nullptr) v += ld_act_bf16(ex + local);
      yo[local] = __float2bfloat16(v);
    } else {
      if (a.extra[0] != nullptr) v += ld_act_bf16(a.extra[0] + unit);
      if (a.y32 != nullptr) {
        a.y32[unit] = v;
      } else {
        a.y[0][unit] = __float2bfloat16(v);
      }
    }
  };

  int buf = 0;
  auto process = [&](int tile, const uint4 (&pk)[RW][C], const uint16_t (&sc)[RW][C]) {
    constexpr int lanes_per = 32 / RW;
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

    if (a.S > 1) {
      float *pb = part + buf * (kMaxWarps * 8);
      if ((lane & (lanes_per - 1)) == 0) pb[s * (a.G * RW) + g * RW + my] = tot;
      asm volatile("bar.sync 2, %0;" ::"r"(live_threads) : "memory");
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
  while (tile < a.n_tiles) {
    issue(tile + tile_stride, nxt, nxt_s);
    process(tile, cur, cur_s);
    tile += tile_stride;
    if (tile >= a.n_tiles) break;
    issue(tile + tile_stride, cur, cur_s);
    process(tile, nxt, nxt_s);
    tile += tile_stride;
  }
}

struct GemvShape {
  int R, C, S, G, n_tiles, grid;
};

// K slices of C*1024 per warp, up to kMaxWarps warps per CTA. Rows per warp (R) and
// row groups per CTA (G) minimise the number of passes the busiest CTA makes over
// `ctas` CTAs, with a per-tile charge (one row's worth by default, CHR_GEMV_TILE_COST
// overrides it) so that fewer, fatter passes win when a pass is short. R == 0 in the result: K is beyond kMaxWarps slices of 2048.
inline float gemv_tile_cost() {
  static float cached = -1.f;
  if (cached < 0.f) {
    const char *env = std::getenv("CHR_GEMV_TILE_COST");
    const float v = env != nullptr ? static_cast<float>(std::atof(env)) : 0.f;
    cached = (env != nullptr && v >= 0.f && v <= 16.f) ? v : 1.0f;
  }
  return cached;
}

inline GemvShape pick_gemv_shape(int n_rows, int K_pad, bool swiglu, int ctas,
                                 int max_warps = kMaxWarps) {
  GemvShape best{0, 0, 0, 0, 0, 0};
  const int n_chunks = (K_pad + kChunk - 1) / kChunk;
  const int C = n_chunks >= 2 ? 2 : 1;
  const int S = (n_chunks + C - 1) / C;
  if (S > max_warps) return best;
  const int rmax = (swiglu ? 2 : 4) / C;  // keeps both register buffers at <= 4 loads
  float best_cost = 0.f;
  for (int G = max_warps / S; G >= 1; G >>= 1) {
    for (int R = rmax; R >= 1; R >>= 1) {
      const int tiles = (n_rows + G * R - 1) / (G * R);
      const int passes = (tiles + ctas - 1) / ctas;
      const float cost = static_cast<float>(passes) * (static_cast<float>(R) + gemv_tile_cost());
      if (best.R == 0 || cost < best_cost) {
        best_cost = cost;
        best = GemvShape{R, C, S, G, tiles, tiles < ctas ? tiles : ctas};
      }
    }
  }
  return best;
}

}  // namespace chr
