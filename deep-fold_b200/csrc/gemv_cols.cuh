// NF4 GEMV for up to four activation rows on the bulk-copy ring (sm_100a): every
// packed weight is read from HBM once, looked up once (the exact FP32 pair table of
// the one-row kernel) and multiplied into all the rows, whose x values sit in
// registers. No counterpart in the reference, whose GEMV takes one row
// (gpu/nf4/nf4_gemv.cu:291-324); numerics are those of the one-row kernel (weights
// LUT*scale in FP32, never rounded to bf16; FP32 accumulation; one rounding).
//
// Why the rows are nearly free. The one-row kernel is bound by its 8-byte table
// lookups (two shared-memory wavefronts per 64 weights). Here a lookup feeds four
// packed FMAs instead of one, and the x pairs are unpacked from bf16 once per code
// word for both weight rows a warp carries: about 6 instructions per weight for four
// rows against 2.7 for one (measured).
//
// Work split (as in gemv_ring.cuh, simplified to one matrix): a CTA of S*G working
// warps and one helper warp; a warp owns one 1024-wide chunk of K (S chunks per CTA,
// at most 11: longer K is cut into slices over grid.y, whose FP32 partials a second
// kernel adds up in slice order) and two weight rows of each tile; a tile is G*2 rows.
// The helper warp requests a tile's row segments with one bulk copy per row (and one
// per row of scales when those are 16-byte aligned), combines the chunks' partial sums
// of a finished tile, adds bias and residual, stores, and hands the slot out again.
// A lane keeps the 32 x values of its chunk for all four rows as packed bf16 pairs
// (64 registers). Every wait is bounded (status 3002).

#pragma once

#include "gemv_ring.cuh"

namespace chr {
namespace {

constexpr int kColsN = 4;         // activation rows per launch (fewer are padded with zeros)
constexpr int kColsRW = 2;        // weight rows a warp carries through a tile
constexpr int kColsWarps = 11;     // working warps per CTA: 12 warps leave 170 registers per thread
constexpr int kColsMaxChunks = kColsWarps;  // chunks of K per CTA (one per working warp row)

struct GemvColsArgs {
  const uint8_t *packed;
  const uint16_t *scale;
  const __nv_bfloat16 *x;     // [N, K] rows
  __nv_bfloat16 *y;           // [N, M] rows (one K slice)
  const __nv_bfloat16 *add;   // [N, M] or null (may alias y)
  const __nv_bfloat16 *bias;  // [M] or null
  float *ws;                  // [n_kslices, N, M] partials (more than one K slice)
  int M, K, K_pad, N;
  int S, G;                   // chunks per K slice (of the first slices), row groups per CTA
  int n_kslices;
  int n_tiles;                // ceil(M / (2 G))
  int n_slots;
  int scale_ring;             // the scale segments travel through the ring
  int *status;
};

template <int DUMMY = 0>
__global__ void __launch_bounds__((kColsWarps + 1) * 32, 1) nf4_gemv_cols_kernel(const GemvColsArgs a) {
  extern __shared__ __align__(128) unsigned char smem[];
  const int tid = threadIdx.x;
  const int lane = tid & 31;
  const int warp = tid >> 5;
  pdl_trigger();

  const int kslice = blockIdx.y;
  const int chunk0 = kslice * a.S;                                // first chunk of this K slice
  const int k_begin = chunk0 * kChunk;
  const int k_len = min(a.S * kChunk, a.K_pad - k_begin);         // multiple of 64
  const int n_chunks = (k_len + kChunk - 1) / kChunk;             // chunks this CTA really has
  const int n_warps = a.S * a.G;
  const int s = warp % a.S;
  const int g = warp / a.S;
  const int rt = a.G * kColsRW;
  const uint32_t row_bytes = static_cast<uint32_t>(a.K_pad >> 1);
  const uint32_t n_groups = static_cast<uint32_t>(a.K_pad / kGroup);
  const uint32_t seg_bytes = static_cast<uint32_t>(k_len >> 1);   // codes of one row in this slice
  const uint32_t seg_groups = static_cast<uint32_t>(k_len / kGroup);
  const uint32_t sc_bytes = seg_groups * 2u;
  const uint32_t codes_bytes = static_cast<uint32_t>(rt) * seg_bytes;
  const uint32_t slot_bytes =
      (codes_bytes + (a.scale_ring != 0 ? static_cast<uint32_t>(rt) * sc_bytes : 0u) + 127u) & ~127u;

  // ---- shared window: [barriers | partials | ring slots ...) [table] [ring slots ...) ----
  const uint32_t base = static_cast<uint32_t>(__cvta_generic_to_shared(smem));
  uint32_t dyn;
  asm("mov.u32 %0, %%dynamic_smem_size;" : "=r"(dyn));
  const uint32_t full_bars = base;
  const uint32_t done_bars = base + 64u;
  const uint32_t abort_flag = base + 128u;
  const uint32_t part_addr = base + kHeadBytes;
  const uint32_t front_end = (part_addr + kPartBytes + 127u) & ~127u;
  const uint32_t window_end = base + dyn;
  const int back_slots =
      window_end > ring_abs<3>() ? static_cast<int>((window_end - ring_abs<3>()) / slot_bytes) : 0;
  const int front_slots = front_end < kTabAbs ? static_cast<int>((kTabAbs - front_end) / slot_bytes) : 0;
  const bool window_ok = (base & 15u) == 0u && front_end <= kTabAbs && window_end >= ring_abs<3>() &&
                         back_slots + front_slots >= a.n_slots && a.n_slots >= 1 &&
                         a.n_slots <= kMaxSlots && static_cast<int>(blockDim.x) == (n_warps + 1) * 32 &&
                         a.S * a.G * kColsRW * kColsN <= 128;
  if (!window_ok) {
    if (tid == 0 && a.status != nullptr) atomicCAS(a.status, 0, kStGemvWindow);
    pdl_wait();
    return;
  }
  auto slot_addr = [&](int d) -> uint32_t {
    return d < back_slots ? ring_abs<3>() + static_cast<uint32_t>(d) * slot_bytes
                          : front_end + static_cast<uint32_t>(d - back_slots) * slot_bytes;
  };
  const int D = a.n_slots;
  const int first_tile = blockIdx.x;
  const int tile_stride = gridDim.x;
  const int n_my = first_tile < a.n_tiles ? (a.n_tiles - first_tile + tile_stride - 1) / tile_stride : 0;
  const bool helper = warp == n_warps;
  const bool worker = warp < n_warps;

  // helper warp: one bulk copy per row of the tile (lane l takes row l), after lane 0
  // has announced the byte count
  auto request = [&](int i) {
    const int tile = first_tile + i * tile_stride;
    const int d = i % D;
    const uint32_t bar = full_bars + static_cast<uint32_t>(d) * 8u;
    const uint32_t dst = slot_addr(d);
    const int row0 = tile * rt;
    const int n = min(rt, a.M - row0);
    if (lane == 0) {
      ring_expect_tx(bar, static_cast<uint32_t>(n) * (seg_bytes + (a.scale_ring != 0 ? sc_bytes : 0u)));
    }
    __syncwarp();
    if (lane < n) {
      const size_t row = static_cast<size_t>(row0 + lane);
      bulk_g2s(dst + static_cast<uint32_t>(lane) * seg_bytes,
               a.packed + row * row_bytes + static_cast<size_t>(k_begin >> 1), seg_bytes, bar);
      if (a.scale_ring != 0) {
        bulk_g2s(dst + codes_bytes + static_cast<uint32_t>(lane) * sc_bytes,
                 a.scale + row * n_groups + static_cast<size_t>(k_begin / kGroup), sc_bytes, bar);
      }
    }
  };

  if (helper) {
    if (lane == 0) {
      for (int d = 0; d < D; ++d) {
        ring_bar_init(full_bars + static_cast<uint32_t>(d) * 8u, 1u);
        ring_bar_init(done_bars + static_cast<uint32_t>(d) * 8u, static_cast<uint32_t>(n_warps));
      }
      asm volatile("st.shared.u32 [%0], %1;" ::"r"(abort_flag), "r"(0u) : "memory");
      asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    __syncwarp();
    // the weights depend on nothing the producer of x writes
    for (int i = 0; i < D && i < n_my; ++i) request(i);
  }
  build_table<3>(tid, blockDim.x);
  pdl_wait();  // x and the residual belong to the previous kernel until it completes
  __syncthreads();
  if (n_my == 0) return;

  auto aborted = [&]() -> bool {
    uint32_t ab;
    asm volatile("ld.shared.u32 %0, [%1];" : "=r"(ab) : "r"(abort_flag) : "memory");
    return ab != 0u;
  };
  auto give_up = [&]() {
    asm volatile("st.shared.u32 [%0], %1;" ::"r"(abort_flag), "r"(1u) : "memory");
    if (lane == 0 && a.status != nullptr) atomicCAS(a.status, 0, kStGemvTimeout);
  };
  constexpr uint32_t part_stride = kPartBytes / kMaxSlots;
  constexpr int kVals = kColsRW * kColsN;  // sums a warp produces per tile: value v = r*4 + n

  if (helper) {
    int waited = 0;
    int requested = min(D, n_my);
    for (int i = 0; i < n_my; ++i) {
      const int tile = first_tile + i * tile_stride;
      const int d = i % D;
      const bool arrived =
          ring_wait(done_bars + static_cast<uint32_t>(d) * 8u, static_cast<uint32_t>(i / D) & 1u);
      if (__any_sync(0xffffffffu, !arrived) || aborted()) {
        give_up();
        break;
      }
      waited = i + 1;
      // partials of the tile: [chunk][row group][value]; sum the chunks in order
      const uint32_t pbuf = part_addr + static_cast<uint32_t>(d) * part_stride;
      for (int idx = lane; idx < a.G * kVals; idx += 32) {
        float v = 0.f;
        for (int q = 0; q < n_chunks; ++q) {
          float p;
          asm volatile("ld.shared.f32 %0, [%1];"
                       : "=f"(p)
                       : "r"(pbuf + static_cast<uint32_t>(q * a.G * kVals + idx) * 4u)
                       : "memory");
          v += p;
        }
        const int gg = idx / kVals;
        const int val = idx - gg * kVals;
        const int n = val & (kColsN - 1);
        const int row = tile * rt + gg * kColsRW + (val >> 2);
        if (n < a.N && row < a.M) {
          const size_t at = static_cast<size_t>(n) * a.M + row;
          if (a.n_kslices > 1) {
            a.ws[static_cast<size_t>(kslice) * a.N * a.M + at] = v;
          } else {
            if (a.bias != nullptr) v += ld_act_bf16(a.bias + row);
            if (a.add != nullptr) v += ld_act_bf16(a.add + at);
            a.y[at] = __float2bfloat16(v);
          }
        }
      }
      __syncwarp();  // the partials are read before the slot is handed out again
      if (i + D < n_my) {
        request(i + D);
        requested = i + D + 1;
      }
    }
    if (lane == 0) {
      // copies already requested may still land after a give-up: one bounded wait each
      for (int j = waited; j < requested; ++j) {
        ring_wait(full_bars + static_cast<uint32_t>(j % D) * 8u, static_cast<uint32_t>(j / D) & 1u);
      }
    }
    return;
  }
  if (!worker) return;

  // ---- working warps ----
  // The lane's 32 k of its chunk, for every activation row, as packed bf16 pairs; zero
  // at and beyond K, for rows the call does not have, and for chunks past the slice.
  const bool chunk_live = s < n_chunks;
  const int k0 = k_begin + s * kChunk + lane * 32;
  const bool lane_live = chunk_live && k0 < a.K_pad;
  uint32_t xb[kColsN][16];
#pragma unroll
  for (int n = 0; n < kColsN; ++n) {
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      uint4 v = make_uint4(0u, 0u, 0u, 0u);
      const int k = k0 + q * 8;
      if (n < a.N && lane_live && k < a.K) {
        const __nv_bfloat16 *src = a.x + static_cast<size_t>(n) * a.K + k;
        if (k + 8 <= a.K && (reinterpret_cast<uintptr_t>(src) & 15u) == 0u) {
          v = ld_act16(src);
        } else {
          __nv_bfloat16 t[8];
#pragma unroll
          for (int e = 0; e < 8; ++e) t[e] = __float2bfloat16(k + e < a.K ? ld_act_bf16(src + e) : 0.f);
          v = *reinterpret_cast<const uint4 *>(t);
        }
      }
      xb[n][4 * q + 0] = v.x;
      xb[n][4 * q + 1] = v.y;
      xb[n][4 * q + 2] = v.z;
      xb[n][4 * q + 3] = v.w;
    }
  }

  const uint32_t tab_lane = kTabAbs + static_cast<uint32_t>(lane) * 8u;
  // A lane without live k reads the row's first bytes and first scale instead: in
  // bounds, and multiplied by x = 0.
  const uint32_t off_pk = lane_live ? static_cast<uint32_t>(s) * (kChunk / 2) + static_cast<uint32_t>(lane) * 16u : 0u;
  const uint32_t off_sc = lane_live ? (static_cast<uint32_t>(s) * (kChunk / kGroup) + static_cast<uint32_t>(lane >> 1)) * 2u : 0u;
  uint32_t row_pk[kColsRW], row_sc[kColsRW];
#pragma unroll
  for (int r = 0; r < kColsRW; ++r) {
    const uint32_t lr = static_cast<uint32_t>(g * kColsRW + r);
    row_pk[r] = lr * seg_bytes + off_pk;
    row_sc[r] = codes_bytes + lr * sc_bytes + off_sc;
  }
  const int my = reduced_row_of_lane<kVals>(lane);  // which of the 8 sums this lane ends up with
  const uint32_t part_lane = static_cast<uint32_t>(s * (a.G * kVals) + g * kVals + my) * 4u;
  const bool part_writer = (lane & (32 / kVals - 1)) == 0;
  const int last_row = a.M - 1;
  int d = 0;
  uint32_t phase = 0;
  int tile = first_tile;
  for (int i = 0; i < n_my; ++i) {
    const uint32_t slot = slot_addr(d);
    const bool arrived = ring_wait(full_bars + static_cast<uint32_t>(d) * 8u, phase);
    if (__any_sync(0xffffffffu, !arrived)) {
      give_up();
      break;
    }
    uint4 pk[kColsRW];
    float sc[kColsRW];
#pragma unroll
    for (int r = 0; r < kColsRW; ++r) {
      pk[r] = lds128(slot + row_pk[r]);
      if (a.scale_ring != 0) {
        sc[r] = half_bits_to_float(lds_u16(slot + row_sc[r]));
      } else {
        const int row = min(tile * rt + g * kColsRW + r, last_row);
        sc[r] = half_bits_to_float(ld_stream_u16(
            a.scale + static_cast<size_t>(row) * n_groups + static_cast<size_t>(k_begin / kGroup) + (off_sc >> 1)));
      }
    }
    f32x2_t acc[kColsRW][kColsN];
#pragma unroll
    for (int r = 0; r < kColsRW; ++r) {
#pragma unroll
      for (int n = 0; n < kColsN; ++n) acc[r][n] = 0ull;
    }
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      // the lookups of this code word for both weight rows, then one activation row
      // after the other: its four x pairs are unpacked once for both weight rows
      f32x2_t p[kColsRW][4];
#pragma unroll
      for (int r = 0; r < kColsRW; ++r) {
        const uint32_t w = q == 0 ? pk[r].x : (q == 1 ? pk[r].y : (q == 2 ? pk[r].z : pk[r].w));
#pragma unroll
        for (int bidx = 0; bidx < 4; ++bidx) {
          uint32_t addr;
          const uint32_t sel = 0x7604u | (static_cast<uint32_t>(bidx) << 4);
          asm("prmt.b32 %0, %1, %2, %3;" : "=r"(addr) : "r"(w), "r"(tab_lane), "r"(sel));
          p[r][bidx] = lds_f32x2(addr);
        }
      }
#pragma unroll
      for (int n = 0; n < kColsN; ++n) {
#pragma unroll
        for (int bidx = 0; bidx < 4; ++bidx) {
          const f32x2_t xp = pack_f32x2(bf16_lo(xb[n][4 * q + bidx]), bf16_hi(xb[n][4 * q + bidx]));
#pragma unroll
          for (int r = 0; r < kColsRW; ++r) acc[r][n] = ffma2(p[r][bidx], xp, acc[r][n]);
        }
      }
    }
    float sum[kVals];
#pragma unroll
    for (int r = 0; r < kColsRW; ++r) {
#pragma unroll
      for (int n = 0; n < kColsN; ++n) {
        float e0, o0;
        unpack_f32x2(acc[r][n], e0, o0);
        sum[r * kColsN + n] = sc[r] * (e0 + o0);
      }
    }
    const float tot = warp_reduce_rows<kVals>(sum, lane);
    if (part_writer) {
      asm volatile("st.shared.f32 [%0], %1;" ::"r"(part_addr + static_cast<uint32_t>(d) * part_stride + part_lane),
                   "f"(tot)
                   : "memory");
    }
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

// Work split of one launch: K slices of at most 11 chunks, S chunks per slice,
// G = 11 / S row groups, as many ring slots as fit (at most 8).
struct GemvColsShape {
  int S, G, n_kslices, n_tiles, n_slots, scale_ring, grid_x;
  uint32_t smem_bytes;
};

inline GemvColsShape pick_cols_shape(int M, int K_pad, bool scales_aligned) {
  GemvColsShape sh{};
  const int n_chunks = (K_pad + kChunk - 1) / kChunk;
  sh.n_kslices = (n_chunks + kColsMaxChunks - 1) / kColsMaxChunks;
  sh.S = (n_chunks + sh.n_kslices - 1) / sh.n_kslices;   // even slices
  sh.n_kslices = (n_chunks + sh.S - 1) / sh.S;
  sh.G = kColsWarps / sh.S;
  if (sh.G * kColsRW * kColsN * sh.S > 128) sh.G = 128 / (kColsRW * kColsN * sh.S);
  if (sh.G < 1) sh.G = 1;
  const int rt = sh.G * kColsRW;
  sh.n_tiles = (M + rt - 1) / rt;
  // every slice's scale segment must start and end on 16 bytes: groups per slice % 8
  const int groups = K_pad / kGroup;
  const int slice_groups = sh.S * (kChunk / kGroup);
  const int last_groups = groups - (sh.n_kslices - 1) * slice_groups;
  sh.scale_ring = scales_aligned && groups % 8 == 0 && slice_groups % 8 == 0 && last_groups % 8 == 0 ? 1 : 0;
  const uint32_t seg = static_cast<uint32_t>(sh.S) * (kChunk / 2);
  const uint32_t slot = (static_cast<uint32_t>(rt) * (seg + (sh.scale_ring ? static_cast<uint32_t>(slice_groups) * 2u : 0u)) + 127u) & ~127u;
  const uint32_t front = (kReserved + kHeadBytes + kPartBytes + 127u) & ~127u;
  const int cap = static_cast<int>((kWindowEnd - ring_abs<3>()) / slot) + static_cast<int>((kTabAbs - front) / slot);
  sh.n_slots = cap < kMaxSlots ? cap : kMaxSlots;
  int gx = sm_count() / sh.n_kslices;
  gx = gx < 1 ? 1 : gx;
  sh.grid_x = sh.n_tiles < gx ? sh.n_tiles : gx;
  sh.smem_bytes = kWindowEnd - kReserved;
  return sh;
}

}  // namespace
}  // namespace chr
