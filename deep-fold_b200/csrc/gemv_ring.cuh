// Device core of the decode-side NF4 GEMV family (sm_100a).
//
// The op is HBM-bound by design (4.25 bits per weight, one multiply-add each).
//
//   * Weight stream. Packed rows are contiguous in memory ([M, K_pad/2] row-major),
//     so a tile of consecutive rows is ONE linear range. A helper warp streams tiles
//     into a shared-memory ring with 1-D bulk copies (cp.async.bulk, own-GPU memory,
//     no multicast) that complete on an mbarrier; the working warps release a slot
//     through a second mbarrier and never meet at a CTA-wide barrier. The copies of
//     several tiles are outstanding while one is consumed and none of that occupies
//     registers; the first tiles are requested before the kernel orders itself
//     behind its predecessor (the weights are constants). The same helper warp
//     combines the K-slice partials of a finished tile, off the workers' path.
//
//   * Lookup. A code byte (two weights) becomes its two codebook values by one
//     shared-memory load from a 256-entry table replicated per lane (bank-conflict
//     free for any codes). The table sits at a fixed address of the shared window
//     with entries 256 bytes apart per byte value, so one byte-permute forms the
//     address (the code byte becomes byte 1 of it). Variant 3 (default) reads the
//     pair as exact FP32 (8 bytes, then one packed FMA: 3 instructions per byte,
//     bound by the shared-memory pipe); variant 0 reads a binary16 pair (4 bytes,
//     two conversions, two FMAs: 6 instructions per byte, bound by instruction
//     issue). Measured on B200 both land within a few percent of each other, so the
//     exact one is the default.
//
// x is kept in registers, a lane owning the same 32 consecutive k of each 1024-wide
// chunk for every row. Accumulation is FP32; the FP16 group scale multiplies the
// unscaled 32-code sum once; slice partials are combined in a fixed order, so
// results do not depend on the grid and repeat bit for bit.
//
// Numerics followed (reference: gpu/nf4/nf4_gemv.cu:58-80,232-243,383-389,483-494):
// weights are LUT*scale in FP32 (never rounded to bf16), FP32 accumulation, one
// rounding to bf16 after the optional residual / bias / SwiGLU. The summation order
// differs from the reference's, which stays inside its 1e-2 tolerance. (Variant 0
// additionally holds the codebook as binary16: relative error <= 2^-12 per level.)
#pragma once

#include <cstdlib>

#include "nf4_common.cuh"

namespace chr {

constexpr int kChunk = 1024;  // k per warp-wide 16-byte read
// Working warps per CTA; one more warp (the helper) requests tiles and combines
// slices. 15 + 1 = 16 warps leaves 128 registers per thread (registers are granted
// per four warps, so a 17th warp would cost as much as a 20th).
#ifndef CHR_GEMV_WORKERS
#define CHR_GEMV_WORKERS 15
#endif
constexpr int kMaxWarps = CHR_GEMV_WORKERS;

// Shared window of a CTA (absolute shared addresses):
//   [dyn base .. 0x10000)   header (barriers, flags), slice partials, staged x,
//                           then as many extra ring slots as fit
//   [0x10000 .. 0x20000)    lookup table (entry of byte value b for lane l at
//                           0x10000 + b*256 + l*4; the upper 128 bytes of each 256
//                           are unused)
//   [0x20000 .. end)        ring slots
// The kernels declare no static shared memory, so the dynamic allocation starts
// right after the 1 KiB the system reserves; whatever the start is, the kernel
// checks it and refuses to run (status word) if the window does not cover what it
// needs. Nothing here needs to know the start on the host.
constexpr uint32_t kTabAbs = 0x10000u;
template <int V>
__host__ __device__ constexpr uint32_t ring_abs() {
  return 0x20000u;
}
constexpr uint32_t kWindowEnd = 0x39000u;  // 1 KiB reserved + 227 KiB
constexpr uint32_t kReserved = 1024u;
constexpr int kMaxSlots = 8;
constexpr uint32_t kHeadBytes = 256u;                    // barriers + flags
constexpr uint32_t kPartBytes = kMaxSlots * 128u * 4u;  // slice partials, one buffer of 128 floats per slot
constexpr uint32_t kWaitPolls = 1u << 20;                // bounded mbarrier waits

// Status codes a kernel leaves in the library's status word.
constexpr int kStGemvWindow = 3001;   // shared window does not cover the layout
constexpr int kStGemvTimeout = 3002;  // a bulk copy did not complete in time

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
  int n_slots;  // ring depth
  int scale_bulk;       // scales travel through the ring (all pieces 16-byte aligned)
  int tail_scale_bulk;  // ... also those of the last, partial tile
  int *status;          // sticky status word (0 = fine)
};

// ---------------------------------------------------------------------------
// mbarrier / bulk-copy primitives (CTA-local, no multicast)
// ---------------------------------------------------------------------------
__device__ __forceinline__ void ring_bar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void ring_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ bool ring_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t done;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(done)
      : "r"(bar), "r"(parity)
      : "memory");
  return done != 0;
}
// Bounded wait: false when the phase did not complete within kWaitPolls polls. The
// blocking form of the probe is used on purpose: it parks the warp instead of
// spending issue slots (spinning on the non-blocking form was measured 1.5x slower
// for the whole kernel).
__device__ __forceinline__ bool ring_wait(uint32_t bar, uint32_t parity) {
  for (uint32_t polls = 0; polls < kWaitPolls; ++polls) {
    if (ring_try_wait(bar, parity)) return true;
  }
  return false;
}
__device__ __forceinline__ void bulk_g2s(uint32_t dst, const void *src, uint32_t bytes,
                                         uint32_t bar) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::
          "r"(dst),
      "l"(src), "r"(bytes), "r"(bar)
      : "memory");
}

__device__ __forceinline__ uint4 lds128(uint32_t a) {
  uint4 v;
  asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "r"(a)
               : "memory");
  return v;
}
__device__ __forceinline__ uint16_t lds_u16(uint32_t a) {
  uint16_t v;
  asm volatile("ld.shared.u16 %0, [%1];" : "=h"(v) : "r"(a) : "memory");
  return v;
}

// ---------------------------------------------------------------------------
// Lookup table and inner product
// ---------------------------------------------------------------------------
// Measured on B200 (148 SMs, 1.965 GHz), inner loop alone on shared-memory data:
//   variant 3: byte-permute, 8-byte lookup of the exact FP32 pair, packed FP32 FMA
//              (3 instructions per byte): 28 weights/clk/SM, the 8-byte lookups fill
//              the shared-memory pipe (two wavefronts each);
//   variant 0: byte-permute, 4-byte lookup of a binary16 pair, two conversions (FMA
//              pipe), two FP32 FMAs (6 instructions per byte): 38 weights/clk/SM, bound
//              by instruction issue (packed FMAs would need 64-bit register pairs,
//              which cost moves when the halves are produced separately).
// HBM at the measured copy rate needs 42 weights/clk/SM.
#ifndef CHR_GEMV_VARIANT
#define CHR_GEMV_VARIANT 3
#endif

__device__ __forceinline__ uint32_t f32_to_f16_bits(float v) {
  return static_cast<uint32_t>(__half_as_ushort(__float2half_rn(v)));
}

// Bytes per lane of a table entry.
template <int V>
__host__ __device__ constexpr uint32_t entry_bytes() {
  return V == 3 ? 8u : 4u;
}

// Fill the table: entry (b, l) at kTabAbs + b*256 + l*entry_bytes.
template <int V>
__device__ __forceinline__ void build_table(int tid, int n_threads) {
  for (int i = tid; i < 256 * 32; i += n_threads) {
    const int b = i >> 5;
    const float lo = __uint_as_float(kLutBits[b & 15]);
    const float hi = __uint_as_float(kLutBits[b >> 4]);
    const uint32_t addr = kTabAbs + static_cast<uint32_t>(b) * 256u +
                          static_cast<uint32_t>(i & 31) * entry_bytes<V>();
    if constexpr (V == 3) {
      asm volatile("st.shared.v2.f32 [%0], {%1,%2};" ::"r"(addr), "f"(lo), "f"(hi) : "memory");
    } else {
      const uint32_t e = f32_to_f16_bits(lo) | (f32_to_f16_bits(hi) << 16);
      asm volatile("st.shared.b32 [%0], %1;" ::"r"(addr), "r"(e) : "memory");
    }
  }
}

// The lane's x values of one chunk (32 consecutive k): FP32 (even, odd) pairs in
// 64-bit registers for the packed FMAs of variant 3, plain FP32 otherwise.
template <int V>
struct XRegs {
  float v[32];
  __device__ __forceinline__ void set(int pair, float even, float odd) {
    v[2 * pair] = even;
    v[2 * pair + 1] = odd;
  }
};
template <>
struct XRegs<3> {
  f32x2_t p[16];
  __device__ __forceinline__ void set(int pair, float even, float odd) {
    p[pair] = pack_f32x2(even, odd);
  }
};

// Four code bytes (8 weights) of word w: variant 0.
__device__ __forceinline__ void dot8_f16(uint32_t w, uint32_t tab_lane, const float *x, float &a0,
                                         float &a1, float &a2, float &a3) {
  asm("{\n\t.reg .b32 d0,d1,d2,d3,t0,t1,t2,t3;\n\t.reg .b16 l0,h0,l1,h1,l2,h2,l3,h3;\n\t"
      ".reg .f32 fl0,fh0,fl1,fh1,fl2,fh2,fl3,fh3;\n\t"
      "prmt.b32 d0,%4,%5,0x7604;\n\tprmt.b32 d1,%4,%5,0x7614;\n\t"
      "prmt.b32 d2,%4,%5,0x7624;\n\tprmt.b32 d3,%4,%5,0x7634;\n\t"
      "ld.shared.b32 t0,[d0];\n\tld.shared.b32 t1,[d1];\n\t"
      "ld.shared.b32 t2,[d2];\n\tld.shared.b32 t3,[d3];\n\t"
      "mov.b32 {l0,h0},t0;\n\tmov.b32 {l1,h1},t1;\n\tmov.b32 {l2,h2},t2;\n\tmov.b32 {l3,h3},t3;\n\t"
      "cvt.f32.f16 fl0,l0;\n\tcvt.f32.f16 fh0,h0;\n\tcvt.f32.f16 fl1,l1;\n\tcvt.f32.f16 fh1,h1;\n\t"
      "cvt.f32.f16 fl2,l2;\n\tcvt.f32.f16 fh2,h2;\n\tcvt.f32.f16 fl3,l3;\n\tcvt.f32.f16 fh3,h3;\n\t"
      "fma.rn.f32 %0,fl0,%6,%0;\n\tfma.rn.f32 %1,fh0,%7,%1;\n\t"
      "fma.rn.f32 %2,fl1,%8,%2;\n\tfma.rn.f32 %3,fh1,%9,%3;\n\t"
      "fma.rn.f32 %0,fl2,%10,%0;\n\tfma.rn.f32 %1,fh2,%11,%1;\n\t"
      "fma.rn.f32 %2,fl3,%12,%2;\n\tfma.rn.f32 %3,fh3,%13,%3;\n\t}"
      : "+f"(a0), "+f"(a1), "+f"(a2), "+f"(a3)
      : "r"(w), "r"(tab_lane), "f"(x[0]), "f"(x[1]), "f"(x[2]), "f"(x[3]), "f"(x[4]), "f"(x[5]),
        "f"(x[6]), "f"(x[7]));
}

// Four code bytes (8 weights) of word w: variant 3. The byte-permute splices the code
// byte into the table address (byte0 <- tab_lane.byte0, byte1 <- code byte, bytes 2,3
// <- tab_lane).
__device__ __forceinline__ void dot8_pair(uint32_t w, uint32_t tab_lane, const f32x2_t *x,
                                          f32x2_t &a0, f32x2_t &a1) {
  asm("{\n\t.reg .b32 d0,d1,d2,d3;\n\t.reg .b64 p0,p1,p2,p3;\n\t"
      "prmt.b32 d0,%2,%3,0x7604;\n\tprmt.b32 d1,%2,%3,0x7614;\n\t"
      "prmt.b32 d2,%2,%3,0x7624;\n\tprmt.b32 d3,%2,%3,0x7634;\n\t"
      "ld.shared.b64 p0,[d0];\n\tld.shared.b64 p1,[d1];\n\t"
      "ld.shared.b64 p2,[d2];\n\tld.shared.b64 p3,[d3];\n\t"
      "fma.rn.f32x2 %0,p0,%4,%0;\n\tfma.rn.f32x2 %1,p1,%5,%1;\n\t"
      "fma.rn.f32x2 %0,p2,%6,%0;\n\tfma.rn.f32x2 %1,p3,%7,%1;\n\t}"
      : "+l"(a0), "+l"(a1)
      : "r"(w), "r"(tab_lane), "l"(x[0]), "l"(x[1]), "l"(x[2]), "l"(x[3]));
}

// Unscaled dot of 32 codes (one uint4) with the lane's 32 x values.
template <int V>
__device__ __forceinline__ float dot32(const uint4 pk, const XRegs<V> &xr, uint32_t tab_lane) {
  if constexpr (V == 3) {
    f32x2_t a0 = 0ull, a1 = 0ull;
    dot8_pair(pk.x, tab_lane, xr.p, a0, a1);
    dot8_pair(pk.y, tab_lane, xr.p + 4, a0, a1);
    dot8_pair(pk.z, tab_lane, xr.p + 8, a0, a1);
    dot8_pair(pk.w, tab_lane, xr.p + 12, a0, a1);
    float e0, o0, e1, o1;
    unpack_f32x2(a0, e0, o0);
    unpack_f32x2(a1, e1, o1);
    return (e0 + e1) + (o0 + o1);
  } else {
    float a0 = 0.f, a1 = 0.f, a2 = 0.f, a3 = 0.f;
    dot8_f16(pk.x, tab_lane, xr.v, a0, a1, a2, a3);
    dot8_f16(pk.y, tab_lane, xr.v + 8, a0, a1, a2, a3);
    dot8_f16(pk.z, tab_lane, xr.v + 16, a0, a1, a2, a3);
    dot8_f16(pk.w, tab_lane, xr.v + 24, a0, a1, a2, a3);
    return (a0 + a2) + (a1 + a3);
  }
}

// Sum R per-lane values over the warp with half the shuffles of R butterflies.
// Returns, in every lane, the warp total of value index ((lane >> 4) & 1) for R == 2,
// ((lane >> 3) & 3) for R == 4, and of v[0] for R == 1. Fixed order: deterministic.
template <int R>
__device__ __forceinline__ float warp_reduce_rows(float (&v)[R], int lane) {
  if constexpr (R == 8) {
    // halve the row set three times (lane bits 4, 3, 2 pick the half kept), then two
    // butterfly steps: row index = (lane >> 2) & 7 read as bits (b4 b3 b2)
    float w[4];
    const bool h4 = (lane & 16) != 0;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float send = h4 ? v[i] : v[i + 4];
      const float keep = h4 ? v[i + 4] : v[i];
      w[i] = keep + __shfl_xor_sync(0xffffffffu, send, 16);
    }
    float u[2];
    const bool h3 = (lane & 8) != 0;
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      const float send = h3 ? w[i] : w[i + 2];
      const float keep = h3 ? w[i + 2] : w[i];
      u[i] = keep + __shfl_xor_sync(0xffffffffu, send, 8);
    }
    const bool h2 = (lane & 4) != 0;
    const float send = h2 ? u[0] : u[1];
    float keep = h2 ? u[1] : u[0];
    keep += __shfl_xor_sync(0xffffffffu, send, 4);
    keep += __shfl_xor_sync(0xffffffffu, keep, 2);
    keep += __shfl_xor_sync(0xffffffffu, keep, 1);
    return keep;  // row index = ((lane>>4)&1)*4 + ((lane>>3)&1)*2 + ((lane>>2)&1)
  } else if constexpr (R == 4) {
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
  if constexpr (R == 8) return (((lane >> 4) & 1) << 2) | (((lane >> 3) & 1) << 1) | ((lane >> 2) & 1);
  if constexpr (R == 4) return ((lane >> 4) << 1) | ((lane >> 3) & 1);
  if constexpr (R == 2) return lane >> 4;
  return 0;
}

// Bytes of one ring slot: the tile's code rows, then (when they travel with them)
// its scale rows.
__host__ __device__ inline uint32_t slot_bytes_of(int rows_in_slot, int K_pad, bool scale_bulk) {
  const uint32_t codes = static_cast<uint32_t>(rows_in_slot) * static_cast<uint32_t>(K_pad >> 1);
  const uint32_t scales =
      scale_bulk ? static_cast<uint32_t>(rows_in_slot) * static_cast<uint32_t>(K_pad / kGroup) * 2u : 0u;
  return (codes + scales + 127u) & ~127u;
}

template <int V>
__host__ __device__ inline uint32_t front_bytes_of(int K) {
  return kHeadBytes + kPartBytes + ((static_cast<uint32_t>(K) + 7u) / 8u) * 16u;
}

// MODE 0: one matrix (+ residual). MODE 1: SwiGLU (gate, up). MODE 2: fused q, k, v
// rows in one row space (+ bias each).
//
// One GEMV over the CTA's tiles first_tile, first_tile + tile_stride, ... . Every
// thread of the CTA must call it. `wait()` is called by every thread once the first
// tiles are requested and the table is filled, before any activation is read: it
// is where the caller orders itself behind the producer of x.
template <int V, int R, int C, int MODE, class Wait>
__device__ __forceinline__ void gemv_run(const GemvArgs &a, unsigned char *smem, int first_tile,
                                         int tile_stride, Wait wait) {
  constexpr int RW = (MODE == 1) ? 2 * R : R;  // weight rows per warp per tile
  const int tid = threadIdx.x;
  const int lane = tid & 31;
  const int warp = tid >> 5;
  const int n_warps = a.S * a.G;
  const int s = warp % a.S;
  const int g = warp / a.S;

  const int rt = a.G * R;                                  // unit rows per tile
  const int slot_rows = (MODE == 1) ? 2 * rt : rt;         // weight rows per slot
  const uint32_t row_bytes = static_cast<uint32_t>(a.K_pad >> 1);
  const uint32_t n_groups = static_cast<uint32_t>(a.K_pad / kGroup);
  const uint32_t codes_bytes = static_cast<uint32_t>(slot_rows) * row_bytes;
  const uint32_t slot_bytes = slot_bytes_of(slot_rows, a.K_pad, a.scale_bulk != 0);
  const int last_row = a.n_rows - 1;
  const int last_tile = a.n_tiles - 1;

  // ---- shared window ----
  const uint32_t base = static_cast<uint32_t>(__cvta_generic_to_shared(smem));
  uint32_t dyn;
  asm("mov.u32 %0, %%dynamic_smem_size;" : "=r"(dyn));
  const uint32_t full_bars = base;             // kMaxSlots x 8 bytes: a tile's bytes have landed
  const uint32_t done_bars = base + 64u;       // kMaxSlots x 8 bytes: every warp is done with the slot
  const uint32_t abort_flag = base + 128u;     // u32
  const uint32_t part_addr = base + kHeadBytes;  // kMaxSlots buffers of slice partials
  const uint32_t xs_addr = part_addr + kPartBytes;
  // shared address of the 16 bytes holding x[8*i8 .. 8*i8+7]
  auto xs_at = [&](uint32_t i8) -> uint32_t { return xs_addr + i8 * 16u; };
  const uint32_t front_end = (base + front_bytes_of<V>(a.K) + 127u) & ~127u;
  const uint32_t window_end = base + dyn;
  const int back_slots =
      window_end > ring_abs<V>() ? static_cast<int>((window_end - ring_abs<V>()) / slot_bytes) : 0;
  const int front_slots = front_end < kTabAbs ? static_cast<int>((kTabAbs - front_end) / slot_bytes) : 0;
  const bool window_ok = (base & 15u) == 0u && front_end <= kTabAbs && window_end >= ring_abs<V>() &&
                         back_slots + front_slots >= a.n_slots && a.n_slots >= 1 &&
                         a.n_slots <= kMaxSlots && static_cast<int>(blockDim.x) == (n_warps + 1) * 32;
  if (!window_ok) {
    if (tid == 0 && a.status != nullptr) atomicCAS(a.status, 0, kStGemvWindow);
    wait();
    return;
  }
  auto slot_addr = [&](int d) -> uint32_t {
    return d < back_slots ? ring_abs<V>() + static_cast<uint32_t>(d) * slot_bytes
                          : front_end + static_cast<uint32_t>(d - back_slots) * slot_bytes;
  };
  const int D = a.n_slots;
  const int n_my = first_tile < a.n_tiles ? (a.n_tiles - first_tile + tile_stride - 1) / tile_stride : 0;
  const bool helper = warp == n_warps;  // the warp after the S*G working warps

  // ---- helper warp, lane 0: request a tile into a slot ----
  auto request = [&](int i) {
    const int tile = first_tile + i * tile_stride;
    const int d = i % D;
    const uint32_t bar = full_bars + static_cast<uint32_t>(d) * 8u;
    const uint32_t dst = slot_addr(d);
    const int row0 = tile * rt;
    const int n = min(rt, a.n_rows - row0);  // unit rows in this tile
    const bool sc = a.scale_bulk != 0 && (tile != last_tile || a.tail_scale_bulk != 0);
    if constexpr (MODE == 1) {
      const uint32_t cb = static_cast<uint32_t>(n) * row_bytes;
      const uint32_t sb = sc ? static_cast<uint32_t>(n) * n_groups * 2u : 0u;
      ring_expect_tx(bar, 2u * (cb + sb));
      bulk_g2s(dst, a.packed[0] + static_cast<size_t>(row0) * row_bytes, cb, bar);
      bulk_g2s(dst + static_cast<uint32_t>(rt) * row_bytes,
               a.packed[1] + static_cast<size_t>(row0) * row_bytes, cb, bar);
      if (sc) {
        const uint32_t sdst = dst + codes_bytes;
        bulk_g2s(sdst, a.scale[0] + static_cast<size_t>(row0) * n_groups, sb, bar);
        bulk_g2s(sdst + static_cast<uint32_t>(rt) * n_groups * 2u,
                 a.scale[1] + static_cast<size_t>(row0) * n_groups, sb, bar);
      }
    } else if constexpr (MODE == 0) {
      const uint32_t cb = static_cast<uint32_t>(n) * row_bytes;
      const uint32_t sb = sc ? static_cast<uint32_t>(n) * n_groups * 2u : 0u;
      ring_expect_tx(bar, cb + sb);
      bulk_g2s(dst, a.packed[0] + static_cast<size_t>(row0) * row_bytes, cb, bar);
      if (sc) bulk_g2s(dst + codes_bytes, a.scale[0] + static_cast<size_t>(row0) * n_groups, sb, bar);
    } else {
      // pieces of the tile, one per matrix it touches
      uint32_t total = 0;
      const int hi = row0 + n;
#pragma unroll
      for (int m = 0; m < 3; ++m) {
        const int m_lo = m == 0 ? 0 : a.rows_end[m - 1];
        const int p_lo = max(row0, m_lo);
        const int p_hi = min(hi, a.rows_end[m]);
        if (p_hi > p_lo) {
          const uint32_t cnt = static_cast<uint32_t>(p_hi - p_lo);
          total += cnt * row_bytes + (sc ? cnt * n_groups * 2u : 0u);
        }
      }
      ring_expect_tx(bar, total);
#pragma unroll
      for (int m = 0; m < 3; ++m) {
        const int m_lo = m == 0 ? 0 : a.rows_end[m - 1];
        const int p_lo = max(row0, m_lo);
        const int p_hi = min(hi, a.rows_end[m]);
        if (p_hi > p_lo) {
          const uint32_t cnt = static_cast<uint32_t>(p_hi - p_lo);
          const size_t local = static_cast<size_t>(p_lo - m_lo);
          const uint32_t in_tile = static_cast<uint32_t>(p_lo - row0);
          const uint8_t *pk = m == 0 ? a.packed[0] : (m == 1 ? a.packed[1] : a.packed[2]);
          const uint16_t *sp = m == 0 ? a.scale[0] : (m == 1 ? a.scale[1] : a.scale[2]);
          bulk_g2s(dst + in_tile * row_bytes, pk + local * row_bytes, cnt * row_bytes, bar);
          if (sc) {
            bulk_g2s(dst + codes_bytes + in_tile * n_groups * 2u, sp + local * n_groups,
                     cnt * n_groups * 2u, bar);
          }
        }
      }
    }
  };

  if (helper && lane == 0) {
    for (int d = 0; d < D; ++d) {
      ring_bar_init(full_bars + static_cast<uint32_t>(d) * 8u, 1u);
      ring_bar_init(done_bars + static_cast<uint32_t>(d) * 8u, static_cast<uint32_t>(n_warps));
    }
    asm volatile("st.shared.u32 [%0], %1;" ::"r"(abort_flag), "r"(0u) : "memory");
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    // The weights depend on nothing the producer of x writes: request the first
    // tiles before waiting for it.
    for (int i = 0; i < D && i < n_my; ++i) request(i);
  }

  // RMSNorm weights are constants too: fetch the lane's slice before waiting.
  const bool worker = warp < n_warps;
  uint4 wv[C][4];
#pragma unroll
  for (int j = 0; j < C; ++j) {
    const int k0 = (s * C + j) * kChunk + lane * 32;
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      const int k = k0 + q * 8;
      wv[j][q] = make_uint4(0u, 0u, 0u, 0u);
      if (n_my > 0 && worker && a.rms_w != nullptr && k < a.K) {
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
  build_table<V>(tid, blockDim.x);
  wait();
  __syncthreads();  // barriers initialised and table complete for everybody
  if (n_my == 0) return;

  // x is staged once per CTA in shared memory, so the warps do not each fetch it
  // from L2.
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
    asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(xs_at(static_cast<uint32_t>(i))),
                 "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w)
                 : "memory");
  }
  __syncthreads();
  // From here on the warps run on their own: workers wait for a slot's bytes, the
  // helper waits for the workers to be done with a slot. No CTA-wide barrier.

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
  auto aborted = [&]() -> bool {
    uint32_t ab;
    asm volatile("ld.shared.u32 %0, [%1];" : "=r"(ab) : "r"(abort_flag) : "memory");
    return ab != 0u;
  };
  auto give_up = [&]() {
    asm volatile("st.shared.u32 [%0], %1;" ::"r"(abort_flag), "r"(1u) : "memory");
    if (lane == 0 && a.status != nullptr) atomicCAS(a.status, 0, kStGemvTimeout);
  };
  constexpr uint32_t part_stride = kPartBytes / kMaxSlots;  // bytes of one slot's partials

  if (helper) {
    // ---- helper warp: combine the slices of a finished tile, then refill its slot ----
    int waited = 0;                 // tiles whose completion (by the workers) was seen
    int requested = min(D, n_my);   // tiles requested so far
    for (int i = 0; i < n_my; ++i) {
      const int tile = first_tile + i * tile_stride;
      const int d = i % D;
      // (every lane waits: one polling lane per warp was measured to resume much later)
      const bool arrived =
          ring_wait(done_bars + static_cast<uint32_t>(d) * 8u, static_cast<uint32_t>(i / D) & 1u);
      if (__any_sync(0xffffffffu, !arrived) || aborted()) {
        give_up();
        break;
      }
      waited = i + 1;
      if (a.S > 1) {
        const uint32_t pbuf = part_addr + static_cast<uint32_t>(d) * part_stride;
        auto part = [&](int idx) -> float {
          float v;
          asm volatile("ld.shared.f32 %0, [%1];"
                       : "=f"(v)
                       : "r"(pbuf + static_cast<uint32_t>(idx) * 4u)
                       : "memory");
          return v;
        };
        for (int u = lane; u < rt; u += 32) {
          const int unit = tile * rt + u;
          if constexpr (MODE == 1) {
            float gsum = 0.f, usum = 0.f;
            for (int q = 0; q < a.S; ++q) {
              gsum += part(q * (a.G * RW) + 2 * u);
              usum += part(q * (a.G * RW) + 2 * u + 1);
            }
            if (unit < a.n_rows) {
              a.y[0][unit] = __float2bfloat16((gsum / (1.f + expf(-gsum))) * usum);
            }
          } else {
            float v = 0.f;
            for (int q = 0; q < a.S; ++q) v += part(q * (a.G * RW) + u);
            store_plain(unit, v);
          }
        }
        __syncwarp();  // the partials are read before the slot is handed out again
      }
      if (lane == 0 && i + D < n_my) request(i + D);
      if (i + D < n_my) requested = i + D + 1;
    }
    if (lane == 0) {
      // After a give-up, copies already requested may still land in this CTA's shared
      // memory: one more bounded wait per outstanding tile before the CTA can exit.
      // (Tiles the workers consumed have completed; waiting on them returns at once.)
      for (int j = waited; j < requested; ++j) {
        ring_wait(full_bars + static_cast<uint32_t>(j % D) * 8u, static_cast<uint32_t>(j / D) & 1u);
      }
    }
    return;
  }
  if (!worker) return;

  // ---- working warps ----
  // Optional fused RMSNorm. sum(x^2) is taken by every working warp over the staged
  // copy in the order of warp_sumsq_bf16 (lane l owns the 8-element groups l, l+32,
  // ...; zero padding adds nothing), so every kernel that needs the scale gets the
  // same bits.
  float inv = 1.f;
  if (a.rms_w != nullptr) {
    float acc = 0.f;
#pragma unroll 4
    for (int g8 = lane; g8 < n8; g8 += 32) {
      const uint4 v = lds128(xs_at(static_cast<uint32_t>(g8)));
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

  // The lane's x values for its K slice, zero at and beyond K. `xval8` returns the
  // eight values k..k+7 (after the optional RMSNorm, rounded to bf16 as the separate
  // RMSNorm kernel would leave them).
  auto xval8 = [&](int k, const uint4 wq, float (&out)[8]) {
    uint4 xv = make_uint4(0u, 0u, 0u, 0u);
    if (k < a.K) xv = lds128(xs_at(static_cast<uint32_t>(k >> 3)));
    const uint32_t xw[4] = {xv.x, xv.y, xv.z, xv.w};
    const uint32_t ww[4] = {wq.x, wq.y, wq.z, wq.w};
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      float lo = bf16_lo(xw[e]);
      float hi = bf16_hi(xw[e]);
      if (a.rms_w != nullptr) {
        lo = __bfloat162float(__float2bfloat16(bf16_lo(ww[e]) * lo * inv));
        hi = __bfloat162float(__float2bfloat16(bf16_hi(ww[e]) * hi * inv));
      }
      out[2 * e] = lo;
      out[2 * e + 1] = hi;
    }
  };
  XRegs<V> xr[C];
#pragma unroll
  for (int j = 0; j < C; ++j) {
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      float t[8];
      xval8((s * C + j) * kChunk + lane * 32 + q * 8, wv[j][q], t);
#pragma unroll
      for (int e = 0; e < 4; ++e) xr[j].set(q * 4 + e, t[2 * e], t[2 * e + 1]);
    }
  }

  const uint32_t tab_lane = kTabAbs + static_cast<uint32_t>(lane) * entry_bytes<V>();
  // This lane's byte / scale offset inside any row, per chunk. A lane whose 32 k lie
  // at or beyond K_pad (last, partial chunk) reads the row's first bytes and first
  // scale instead: in bounds, the row's own data, and multiplied by x = 0.
  uint32_t off_pk[C], off_sc[C];
#pragma unroll
  for (int j = 0; j < C; ++j) {
    const bool live = (s * C + j) * kChunk + lane * 32 < a.K_pad;
    off_pk[j] = live ? static_cast<uint32_t>(s * C + j) * (kChunk / 2) + static_cast<uint32_t>(lane) * 16u : 0u;
    off_sc[j] = live ? static_cast<uint32_t>(s * C + j) * (kChunk / kGroup) + static_cast<uint32_t>(lane >> 1) : 0u;
  }

  // Scale of weight row i of this warp for chunk j when the tile's scales did not
  // travel through the ring: straight from global memory (slow path; alignment-exotic
  // matrices and partial last tiles only).
  auto scale_from_global = [&](int tile, int i, int j) -> uint16_t {
    const int unit = min(tile * rt + g * R + (MODE == 1 ? (i >> 1) : i), last_row);
    const uint16_t *sr;
    if constexpr (MODE == 1) {
      sr = ((i & 1) ? a.scale[1] : a.scale[0]) + static_cast<size_t>(unit) * n_groups;
    } else if constexpr (MODE == 0) {
      sr = a.scale[0] + static_cast<size_t>(unit) * n_groups;
    } else {
      const int m = (unit >= a.rows_end[0]) + (unit >= a.rows_end[1]);
      const int local = unit - (m == 0 ? 0 : (m == 1 ? a.rows_end[0] : a.rows_end[1]));
      sr = (m == 0 ? a.scale[0] : (m == 1 ? a.scale[1] : a.scale[2])) +
           static_cast<size_t>(local) * n_groups;
    }
    return ld_stream_u16(sr + (off_sc[j] >> 1));
  };

  constexpr int lanes_per = 32 / RW;
  const int my = reduced_row_of_lane<RW>(lane);  // weight-row index this lane holds
  // Offsets that do not change from tile to tile (the loop below is bound by
  // instruction issue: everything that can be is computed here, and the slot index
  // and barrier phase are carried along instead of divided out).
  uint32_t row_pk[RW], row_sc[RW];
#pragma unroll
  for (int r = 0; r < RW; ++r) {
    const uint32_t lr = MODE == 1 ? static_cast<uint32_t>((r & 1) * rt + g * R + (r >> 1))
                                  : static_cast<uint32_t>(g * R + r);
    row_pk[r] = lr * row_bytes;
    row_sc[r] = codes_bytes + lr * n_groups * 2u;
  }
#pragma unroll
  for (int j = 0; j < C; ++j) off_sc[j] *= 2u;  // bytes from here on
  const uint32_t part_lane = static_cast<uint32_t>(s * (a.G * RW) + g * RW + my) * 4u;
  const bool part_writer = (lane & (lanes_per - 1)) == 0;
  const bool multi = a.S > 1;
  int d = 0;
  uint32_t phase = 0;
  int tile = first_tile;
  for (int i = 0; i < n_my; ++i) {
    const uint32_t slot = slot_addr(d);
    // One lane per warp polls the barrier (hundreds of threads polling one barrier
    // word delay the copy engine's own updates of it); the warp barrier that follows
    // orders the other lanes' reads of the tile behind lane 0's observation.
    const bool arrived = ring_wait(full_bars + static_cast<uint32_t>(d) * 8u, phase);
    if (__any_sync(0xffffffffu, !arrived)) {
      give_up();
      break;
    }
    const bool sc_ring = a.scale_bulk != 0 && (tile != last_tile || a.tail_scale_bulk != 0);
    uint4 pk[RW][C];
    uint16_t sc[RW][C];
    if (sc_ring) {
#pragma unroll
      for (int r = 0; r < RW; ++r) {
#pragma unroll
        for (int j = 0; j < C; ++j) {
          pk[r][j] = lds128(slot + row_pk[r] + off_pk[j]);
          sc[r][j] = lds_u16(slot + row_sc[r] + off_sc[j]);
        }
      }
    } else {
#pragma unroll
      for (int r = 0; r < RW; ++r) {
#pragma unroll
        for (int j = 0; j < C; ++j) {
          pk[r][j] = lds128(slot + row_pk[r] + off_pk[j]);
          sc[r][j] = scale_from_global(tile, r, j);
        }
      }
    }
    float sum[RW];
#pragma unroll
    for (int r = 0; r < RW; ++r) {
      sum[r] = 0.f;
#pragma unroll
      for (int j = 0; j < C; ++j) {
        const float dsum = dot32<V>(pk[r][j], xr[j], tab_lane);
        sum[r] = fmaf(half_bits_to_float(sc[r][j]), dsum, sum[r]);
      }
    }
    const float tot = warp_reduce_rows<RW>(sum, lane);
    if (multi) {
      if (part_writer) {
        asm volatile("st.shared.f32 [%0], %1;" ::"r"(part_addr + static_cast<uint32_t>(d) * part_stride +
                                                       part_lane),
                     "f"(tot)
                     : "memory");
      }
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
        if (part_writer) store_plain(tile * rt + g * R + my, tot);
      }
    }
    // This warp is done with the slot (codes are in registers, partials written).
    __syncwarp();
    if (lane == 0) {
      asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(done_bars + static_cast<uint32_t>(d) * 8u)
                   : "memory");
    }
    tile += tile_stride;
    if (++d == D) {
      d = 0;
      phase ^= 1u;
    }
  }
}

struct GemvShape {
  int R, C, S, G, n_tiles, grid, n_slots, scale_bulk, tail_scale_bulk;
  uint32_t smem_bytes;
};

// Largest C (chunks of 1024 k held in a lane's registers): x costs 32 registers per chunk.
template <int V>
constexpr int max_chunks_per_warp() {
  return 2;
}

inline float gemv_tile_cost() {
  static float cached = -1.f;
  if (cached < 0.f) {
    const char *env = std::getenv("CHR_GEMV_TILE_COST");
    const float v = env != nullptr ? static_cast<float>(std::atof(env)) : 0.f;
    cached = (env != nullptr && v >= 0.f && v <= 16.f) ? v : 4.0f;
  }
  return cached;
}

// Work split of one launch. A warp owns C chunks of every row it touches (S = slices
// per row), G row groups share a CTA, a warp walks R rows of each tile; the tile
// (G*R rows, contiguous in memory) is what one ring slot holds. Chosen to minimise
// passes x (work per pass + a per-tile charge), under the ring's capacity.
// R == 0 in the result: K is beyond what a CTA can hold (x staging or 16 slices).
// `force_c`, `force_r` > 0 pin the choice (tuning runs).
template <int V>
inline GemvShape pick_gemv_shape(int n_rows, int K, int K_pad, int mode, int ctas, int max_c,
                                 bool scales_aligned, const int *rows_end, int force_c = 0,
                                 int force_r = 0) {
  GemvShape best{};
  const int n_chunks = (K_pad + kChunk - 1) / kChunk;
  const uint32_t n_groups = static_cast<uint32_t>(K_pad / kGroup);
  const uint32_t front = (kReserved + front_bytes_of<V>(K) + 127u) & ~127u;
  if (front > kTabAbs) return best;
  float best_cost = 0.f;
  for (int C = 1; C <= max_c; ++C) {
    if (force_c > 0 && C != force_c) continue;
    const int S = (n_chunks + C - 1) / C;
    if (S > kMaxWarps) continue;
    if (C > 1 && (C - 1) * S >= n_chunks) continue;  // a smaller C covers K with the same S
    const int G = kMaxWarps / S;
    for (int R = (mode == 1 ? 4 : 8); R >= 1; R >>= 1) {
      if (force_r > 0 && R != force_r) continue;
      const int RW = mode == 1 ? 2 * R : R;
      if (RW * C > 8) continue;
      const int rt = G * R;
      const int slot_rows = mode == 1 ? 2 * rt : rt;
      bool sb = scales_aligned && (static_cast<uint32_t>(rt) * n_groups * 2u) % 16u == 0u;
      if (mode == 2 && sb) {
        sb = (static_cast<uint32_t>(rows_end[0]) * n_groups * 2u) % 16u == 0u &&
             (static_cast<uint32_t>(rows_end[1]) * n_groups * 2u) % 16u == 0u;
      }
      const bool tail_sb = sb && (static_cast<uint32_t>(n_rows) * n_groups * 2u) % 16u == 0u;
      const uint32_t slot = slot_bytes_of(slot_rows, K_pad, sb);
      const int cap = static_cast<int>((kWindowEnd - ring_abs<V>()) / slot) +
                      static_cast<int>((kTabAbs - front) / slot);
      const int D = cap < kMaxSlots ? cap : kMaxSlots;
      if (D < 2) continue;
      const int tiles = (n_rows + rt - 1) / rt;
      const int passes = (tiles + ctas - 1) / ctas;
      float cost = static_cast<float>(passes) * (static_cast<float>(RW * C) + gemv_tile_cost());
      if (D < 3) cost *= 1.05f;
      if (best.R == 0 || cost < best_cost) {
        best_cost = cost;
        best = GemvShape{R, C, S, G, tiles, tiles < ctas ? tiles : ctas, D, sb ? 1 : 0,
                         tail_sb ? 1 : 0, 0u};
        // ring slots beyond the back region live in the front region; ask for the
        // whole window whenever any slot does
        const int back = static_cast<int>((kWindowEnd - ring_abs<V>()) / slot);
        const uint32_t end = D <= back ? ring_abs<V>() + static_cast<uint32_t>(D) * slot : kWindowEnd;
        best.smem_bytes = (D <= back ? end : kWindowEnd) - kReserved;
      }
    }
  }
  return best;
}

template <int V, int R, int C, int MODE>
__global__ void __launch_bounds__((kMaxWarps + 1) * 32, 1) nf4_gemv_kernel(const GemvArgs a) {
  extern __shared__ __align__(128) unsigned char smem[];
  // The next kernel of the chain may start launching; it requests its first tiles
  // and fills its table while this one runs.
  pdl_trigger();
  gemv_run<V, R, C, MODE>(a, smem, blockIdx.x, gridDim.x, [] {
    // x (and the residual / outputs) belong to the previous kernel until it completes
    pdl_wait();
  });
}

template <int V, int MODE>
inline int launch_gemv(const GemvArgs &proto, const GemvShape &sh, cudaStream_t st) {
  GemvArgs a = proto;
  a.S = sh.S;
  a.G = sh.G;
  a.n_tiles = sh.n_tiles;
  a.n_slots = sh.n_slots;
  a.scale_bulk = sh.scale_bulk;
  a.tail_scale_bulk = sh.tail_scale_bulk;
  const dim3 grid(static_cast<unsigned>(sh.grid));
  const dim3 block(static_cast<unsigned>((sh.S * sh.G + 1) * 32));  // + the helper warp
  const int smem_bytes = static_cast<int>(kWindowEnd - kReserved);  // one limit for every shape

#define CHR_LAUNCH(RR, CC)                                                                     \
  do {                                                                                         \
    if constexpr ((MODE == 1 ? 2 * (RR) : (RR)) * (CC) <= 8 && (CC) <= max_chunks_per_warp<V>() && \
                  !(MODE == 1 && (RR) == 8)) {                                                 \
      static int attr_done[64] = {};                                                           \
      if (!ensure_smem_attr(nf4_gemv_kernel<V, RR, CC, MODE>, smem_bytes, attr_done)) {        \
        return kLaunch;                                                                        \
      }                                                                                        \
      if (launch_chain(nf4_gemv_kernel<V, RR, CC, MODE>, grid, block, sh.smem_bytes, st, a) != \
          cudaSuccess) {                                                                       \
        return kLaunch;                                                                        \
      }                                                                                        \
      return kOk;                                                                              \
    }                                                                                          \
  } while (0)

  switch (sh.C * 8 + sh.R) {
    case 1 * 8 + 1: CHR_LAUNCH(1, 1); break;
    case 1 * 8 + 2: CHR_LAUNCH(2, 1); break;
    case 1 * 8 + 4: CHR_LAUNCH(4, 1); break;
    case 1 * 8 + 8: CHR_LAUNCH(8, 1); break;
    case 2 * 8 + 1: CHR_LAUNCH(1, 2); break;
    case 2 * 8 + 2: CHR_LAUNCH(2, 2); break;
    case 2 * 8 + 4: CHR_LAUNCH(4, 2); break;
    case 3 * 8 + 1: CHR_LAUNCH(1, 3); break;
    case 3 * 8 + 2: CHR_LAUNCH(2, 3); break;
    case 4 * 8 + 1: CHR_LAUNCH(1, 4); break;
    case 4 * 8 + 2: CHR_LAUNCH(2, 4); break;
    default: break;
  }
#undef CHR_LAUNCH
  return kDims;
}

}  // namespace chr
