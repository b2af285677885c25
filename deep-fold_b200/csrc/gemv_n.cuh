// NF4 GEMV for N = 1..8 activation columns on CUDA cores (sm_100a): every packed
// weight is read from HBM once and dequantized once for all columns, with the
// numerics of the one-column GEMV (weights LUT*scale in FP32, never rounded to
// bf16; FP32 accumulation; one rounding at the end). No counterpart in the
// reference, whose GEMV is N = 1 (gpu/nf4/nf4_gemv.cu:291-324); batched decode and
// other few-column callers use it where the tensor-core GEMM's bf16 weights are
// not wanted.
//
// Work split. A CTA of 8 warps owns one K slice (at most kSliceK columns of W, so
// that the slice of all N activation rows fits in shared memory as bf16 beside the
// lookup table) and strides over row tiles of 8 warps x 4 rows. A lane owns 32
// consecutive k of each 1024-wide step, as in the one-column kernel; for a step
// it dequantizes its 32 codes of four rows into registers (the exact FP32 pair
// table of the one-column kernel, one 8-byte lookup per code byte) and then walks
// the columns: the lane's 32 x values of column n are read from shared memory once
// and multiplied into all four rows. Per-lane partial sums are reduced by shuffles.
// With more than one K slice the FP32 partials go to a caller workspace and a second
// kernel adds them up in slice order; results do not depend on the grid.
//
// Bound: instruction issue and shared-memory traffic, not HBM, from N = 2 on (each
// weight costs N multiply-adds and each x value is re-read for every four rows).

#pragma once

#include "gemv_ring.cuh"

namespace chr {
namespace {

constexpr int kNWarps = 8;
constexpr int kNRows = 4;                       // rows a warp carries through a step
constexpr int kNTile = kNWarps * kNRows;        // rows per tile
constexpr int kNMaxCols = 8;
constexpr uint32_t kXsAbs = 0x20000u;           // x slices behind the table
constexpr uint32_t kXsBytes = kWindowEnd - kXsAbs;  // 100 KiB

struct GemvNArgs {
  const uint8_t *packed;
  const uint16_t *scale;
  const __nv_bfloat16 *x;    // [N, K] rows
  __nv_bfloat16 *y;          // [N, M] rows (used when n_slices == 1)
  const __nv_bfloat16 *add;  // [N, M] or null (may alias y)
  const __nv_bfloat16 *bias; // [M] or null
  float *ws;                 // [n_slices, N, M] partials (n_slices > 1)
  int M, K, K_pad, N;
  int slice_k;               // columns of W per slice (multiple of 1024)
  int n_slices;
  int *status;
};

// Columns of W per K slice for N activation columns: the bf16 slices of all N rows of
// x must fit in kXsBytes.
inline int slice_k_for(int n_cols) {
  int k = static_cast<int>(kXsBytes / (2u * static_cast<uint32_t>(n_cols)));
  k = k / kChunk * kChunk;
  return k;
}

__global__ void __launch_bounds__(kNWarps * 32, 1) nf4_gemv_n_kernel(const GemvNArgs a) {
  extern __shared__ __align__(128) unsigned char smem[];
  const int tid = threadIdx.x;
  const int lane = tid & 31;
  const int warp = tid >> 5;
  pdl_trigger();
  const uint32_t base = static_cast<uint32_t>(__cvta_generic_to_shared(smem));
  uint32_t dyn;
  asm("mov.u32 %0, %%dynamic_smem_size;" : "=r"(dyn));
  if (base > kTabAbs || base + dyn < kWindowEnd) {
    if (tid == 0 && a.status != nullptr) atomicCAS(a.status, 0, kStGemvWindow);
    return;
  }
  build_table<3>(tid, blockDim.x);
  pdl_wait();  // x, add belong to the previous kernel until it completes

  const int slice = blockIdx.y;
  const int k_lo = slice * a.slice_k;
  const int k_len = min(a.slice_k, a.K_pad - k_lo);           // multiple of 64
  const int n_steps = (k_len + kChunk - 1) / kChunk;
  // stage the slice of every activation row: xs[n][k - k_lo], zero at and beyond K
  const int row8 = a.slice_k / 8;                              // 16-byte pieces per staged row
  for (int i = tid; i < a.N * row8; i += blockDim.x) {
    const int n = i / row8;
    const int k = k_lo + (i - n * row8) * 8;
    uint4 v = make_uint4(0u, 0u, 0u, 0u);
    const __nv_bfloat16 *src = a.x + static_cast<size_t>(n) * a.K + k;
    if (k + 8 <= a.K && (reinterpret_cast<uintptr_t>(src) & 15u) == 0u) {
      v = ld_act16(src);
    } else if (k < a.K) {
      __nv_bfloat16 t[8];
#pragma unroll
      for (int e = 0; e < 8; ++e) t[e] = __float2bfloat16(k + e < a.K ? ld_act_bf16(src + e) : 0.f);
      v = *reinterpret_cast<const uint4 *>(t);
    }
    asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(kXsAbs + static_cast<uint32_t>(i) * 16u),
                 "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w)
                 : "memory");
  }
  __syncthreads();

  const uint32_t tab_lane = kTabAbs + static_cast<uint32_t>(lane) * 8u;
  const size_t row_bytes = static_cast<size_t>(a.K_pad >> 1);
  const int n_groups = a.K_pad / kGroup;
  const int n_tiles = (a.M + kNTile - 1) / kNTile;
  const int last_row = a.M - 1;

  for (int tile = blockIdx.x; tile < n_tiles; tile += gridDim.x) {
    const int row0 = tile * kNTile + warp * kNRows;
    float acc[kNRows][kNMaxCols];
#pragma unroll
    for (int r = 0; r < kNRows; ++r) {
#pragma unroll
      for (int n = 0; n < kNMaxCols; ++n) acc[r][n] = 0.f;
    }
    // codes and scales of the next step, one step ahead
    uint4 nxt[kNRows];
    uint16_t nxt_s[kNRows];
    auto fetch = [&](int step) {
      const int k = k_lo + step * kChunk + lane * 32;
      const bool live = step < n_steps && k < k_lo + k_len;
#pragma unroll
      for (int r = 0; r < kNRows; ++r) {
        const int row = min(row0 + r, last_row);
        nxt[r] = make_uint4(0x77777777u, 0x77777777u, 0x77777777u, 0x77777777u);
        nxt_s[r] = 0;
        if (live) {
          nxt[r] = ld_stream16(a.packed + static_cast<size_t>(row) * row_bytes + (k >> 1));
          nxt_s[r] = ld_stream_u16(a.scale + static_cast<size_t>(row) * n_groups + (k >> 6));
        }
      }
    };
    fetch(0);
    for (int step = 0; step < n_steps; ++step) {
      // dequantize this step's 32 codes of four rows into FP32 (even, odd) codebook
      // pairs; the group scale multiplies each 32-code sum afterwards
      f32x2_t w[kNRows][16];
      float sc[kNRows];
#pragma unroll
      for (int r = 0; r < kNRows; ++r) {
        sc[r] = half_bits_to_float(nxt_s[r]);
        const uint32_t words[4] = {nxt[r].x, nxt[r].y, nxt[r].z, nxt[r].w};
#pragma unroll
        for (int q = 0; q < 4; ++q) {
#pragma unroll
          for (int bidx = 0; bidx < 4; ++bidx) {
            uint32_t addr;
            const uint32_t sel = 0x7604u | (static_cast<uint32_t>(bidx) << 4);
            asm("prmt.b32 %0, %1, %2, %3;" : "=r"(addr) : "r"(words[q]), "r"(tab_lane), "r"(sel));
            w[r][q * 4 + bidx] = lds_f32x2(addr);
          }
        }
      }
      fetch(step + 1);
      const uint32_t xs_lane = kXsAbs + static_cast<uint32_t>(step * kChunk + lane * 32) * 2u;
#pragma unroll
      for (int n = 0; n < kNMaxCols; ++n) {
        if (n < a.N) {
          const uint32_t xa = xs_lane + static_cast<uint32_t>(n) * static_cast<uint32_t>(a.slice_k) * 2u;
          f32x2_t d[kNRows];
#pragma unroll
          for (int r = 0; r < kNRows; ++r) d[r] = 0ull;
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            const uint4 xv = lds128(xa + static_cast<uint32_t>(q) * 16u);
            const uint32_t xw[4] = {xv.x, xv.y, xv.z, xv.w};
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              const f32x2_t xp = pack_f32x2(bf16_lo(xw[e]), bf16_hi(xw[e]));
#pragma unroll
              for (int r = 0; r < kNRows; ++r) d[r] = ffma2(w[r][q * 4 + e], xp, d[r]);
            }
          }
#pragma unroll
          for (int r = 0; r < kNRows; ++r) {
            float e0, o0;
            unpack_f32x2(d[r], e0, o0);
            acc[r][n] = fmaf(sc[r], e0 + o0, acc[r][n]);
          }
        }
      }
    }
    // reduce over the warp and store
#pragma unroll
    for (int n = 0; n < kNMaxCols; ++n) {
      if (n < a.N) {
#pragma unroll
        for (int r = 0; r < kNRows; ++r) {
          const float v = warp_sum_xor(acc[r][n]);
          const int row = row0 + r;
          if (lane == 0 && row < a.M) {
            const size_t at = static_cast<size_t>(n) * a.M + row;
            if (a.n_slices > 1) {
              a.ws[static_cast<size_t>(slice) * a.N * a.M + at] = v;
            } else {
              float out = v;
              if (a.bias != nullptr) out += ld_act_bf16(a.bias + row);
              if (a.add != nullptr) out += ld_act_bf16(a.add + at);
              a.y[at] = __float2bfloat16(out);
            }
          }
        }
      }
    }
  }
}

// y[n, m] = bf16( sum over slices (in slice order) + bias[m] + add[n, m] )
__global__ void gemv_n_reduce_kernel(const float *ws, __nv_bfloat16 *y, const __nv_bfloat16 *add,
                                     const __nv_bfloat16 *bias, int n_slices, int N, int M) {
  pdl_trigger();
  pdl_wait();
  const size_t total = static_cast<size_t>(N) * M;
  for (size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<size_t>(gridDim.x) * blockDim.x) {
    float v = 0.f;
    for (int s = 0; s < n_slices; ++s) v += __ldcg(ws + static_cast<size_t>(s) * total + i);
    if (bias != nullptr) v += ld_act_bf16(bias + (i % M));
    if (add != nullptr) v += ld_act_bf16(add + i);
    y[i] = __float2bfloat16(v);
  }
}

}  // namespace
}  // namespace chr

extern "C" int64_t chr_nf4_gemv_n_ws(const chr_nf4_dev_t *w, int32_t N) {
  using namespace chr;
  if (w == nullptr || N < 1 || N > kNMaxCols || w->M < 1 || w->K_pad < kGroup) return 0;
  const int sk = slice_k_for(N);
  const int n_slices = (w->K_pad + sk - 1) / sk;
  return n_slices > 1 ? static_cast<int64_t>(n_slices) * N * w->M : 0;
}

extern "C" int chr_nf4_gemv_n(const chr_nf4_dev_t *w, const void *x_rows, void *y_rows, int32_t N,
                              const void *add_rows, const void *bias, float *ws, int64_t ws_floats,
                              void *stream) {
  using namespace chr;
  if (w == nullptr || x_rows == nullptr || y_rows == nullptr) return kNull;
  const int rc = check_matrix(w);
  if (rc != kOk) return rc;
  if (N < 1 || N > kNMaxCols) return kRangeN;
  if (!aligned(w->packed, 16) || !aligned(w->scale, 2) || !aligned(x_rows, 2)) return kAlign;
  GemvNArgs a{};
  a.packed = w->packed;
  a.scale = w->scale;
  a.x = static_cast<const __nv_bfloat16 *>(x_rows);
  a.y = static_cast<__nv_bfloat16 *>(y_rows);
  a.add = static_cast<const __nv_bfloat16 *>(add_rows);
  a.bias = static_cast<const __nv_bfloat16 *>(bias);
  a.M = w->M;
  a.K = w->K;
  a.K_pad = w->K_pad;
  a.N = N;
  a.slice_k = slice_k_for(N);
  a.n_slices = (w->K_pad + a.slice_k - 1) / a.slice_k;
  if (a.n_slices == 1) a.slice_k = (w->K_pad + kChunk - 1) / kChunk * kChunk;  // stage no more than K
  a.status = gemv_status_ptr();
  if (a.n_slices > 1) {
    const int64_t need = static_cast<int64_t>(a.n_slices) * N * w->M;
    if (ws == nullptr || ws_floats < need) return kWorkspace;
    a.ws = ws;
  }
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int smem_bytes = static_cast<int>(kWindowEnd - kReserved);
  static int attr_done[64] = {};
  if (!ensure_smem_attr(nf4_gemv_n_kernel, smem_bytes, attr_done)) return kLaunch;
  const int n_tiles = (w->M + kNTile - 1) / kNTile;
  int gx = sm_count() / a.n_slices;
  gx = gx < 1 ? 1 : gx;
  gx = n_tiles < gx ? n_tiles : gx;
  const dim3 grid(static_cast<unsigned>(gx), static_cast<unsigned>(a.n_slices));
  if (launch_chain(nf4_gemv_n_kernel, grid, dim3(kNWarps * 32), smem_bytes, st, a) != cudaSuccess) {
    return kLaunch;
  }
  if (a.n_slices > 1) {
    const size_t total = static_cast<size_t>(N) * w->M;
    const int blocks = static_cast<int>((total + 255) / 256 < 592 ? (total + 255) / 256 : 592);
    if (launch_chain(gemv_n_reduce_kernel, dim3(static_cast<unsigned>(blocks)), dim3(256), 0, st,
                     static_cast<const float *>(a.ws), a.y, a.add, a.bias, a.n_slices, N,
                     w->M) != cudaSuccess) {
      return kLaunch;
    }
  }
  return kOk;
}
