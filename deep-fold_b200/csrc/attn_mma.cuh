// GQA decode attention on the warp-level tensor-core instruction (sm_100a), for head
// dims 16 / 32 / 64 / 128 (reference: gpu/nf4/nf4_gemv.cu:558-727; same entry points and
// semantics as the CUDA-core form in attn_core.cuh, which keeps the other head dims).
//
// Why. The CUDA-core form spends about 120 instructions per cache row and warp (dot
// products of all query heads of the group, shuffles, running softmax per row): at one
// sequence the launch is a latency chain either way, but with many sequences or long
// contexts it runs at 1.5 TB/s of cache traffic. Here the query heads of a kv group
// are the rows of one m16 tile: scores = Q (16 x hd) K^T and out += P V are
// mma.sync.m16n8k16 (bf16 operands, FP32 accumulate), about 2 instructions per cache
// row and warp.
//
// One CTA of 8 warps per (sequence, kv head, split, head chunk of <= 8 heads). Cache
// rows go through a two-stage cp.async ring of 128-row tiles (K and V, rows padded by
// 16 bytes: conflict-free 8x8 matrix loads); a split takes the tiles split,
// split + n_split, ... . Warp w owns rows 16w .. 16w+15 of every tile: its own running
// softmax (exp2, scale folded) and its own 16 x hd output accumulator, folded over the
// warps at the end through shared memory, then over the splits by the last CTA of the
// group to arrive (the workspace layout and the arrival counters of the other form).
// Precision: the rotated query and the probabilities enter the tensor core as two bf16
// terms each (value = hi + lo, 16 mantissa bits), so both products see them at close to
// FP32 precision for twice the (cheap) matrix instructions; K and V are bf16 in the
// cache anyway. The current token's rotated k and its v are rounded to bf16 - what the
// cache row holds - and patched into the staged tile, so every CTA attends the row it or
// a sibling CTA is writing without reading it back.

#pragma once

#include "attn_core.cuh"

namespace chr {

constexpr int kMmaWarps = 8;
constexpr int kMmaThreads = kMmaWarps * 32;
constexpr int kMmaTile = kMmaWarps * 16;  // cache rows per tile
constexpr int kMmaHeads = 8;              // query heads per item (rows 0..7 of the m16 tile)
constexpr int kMmaStages = 2;             // ring depth (three measured no faster: the loop is not latency-bound)

// Per-sequence strides of the batched form (batch == 1: all unused).
struct AttnBatch {
  int batch;
  long long q_stride, kv_act_stride, cache_stride, out_stride, ws_stride;
};

template <int HD>
struct AttnMmaLayout {
  static constexpr int kRowB = HD * 2 + 16;                       // padded row pitch
  static constexpr int kStageBytes = 2 * kMmaTile * kRowB;        // K tile then V tile
  static constexpr int kQBytes = 2 * kMmaHeads * HD * 2;          // rotated q as bf16 hi + lo parts, [2][8][HD]
  static constexpr int kCurBytes = 2 * HD * 2;                    // current k, v (bf16)
  static constexpr int kFoldBytes = kMmaWarps * kMmaHeads * (HD + 2) * 4;  // per-warp (o, m, l)
  static constexpr int kRing = kMmaStages * kStageBytes;
  static constexpr int kBytes = (kRing > kFoldBytes ? kRing : kFoldBytes) + kQBytes + kCurBytes + 256;
};

__device__ __forceinline__ void mma_cp16(uint32_t dst, const void *src, int src_bytes) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(src_bytes)
               : "memory");
}
__device__ __forceinline__ void mma_ldm_x2(uint32_t addr, uint32_t &r0, uint32_t &r1) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x2.shared.b16 {%0, %1}, [%2];" : "=r"(r0), "=r"(r1) : "r"(addr));
}
__device__ __forceinline__ void mma_ldm_x2_trans(uint32_t addr, uint32_t &r0, uint32_t &r1) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x2.trans.shared.b16 {%0, %1}, [%2];"
               : "=r"(r0), "=r"(r1)
               : "r"(addr));
}
__device__ __forceinline__ void mma_bf16(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                         uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, "
      "{%8, %9}, {%0, %1, %2, %3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t mma_pack(float lo, float hi) {
  const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<const uint32_t *>(&v);
}

// `a` is the item's own argument block (batched callers have applied their strides);
// `ctr` its arrival counter. Called by all kMmaThreads threads of the CTA.
template <int HD>
__device__ __forceinline__ void attn_mma_item(const AttnArgs &a, unsigned char *smem_raw, int split,
                                              int kvh, int z, unsigned int *ctr) {
  using L = AttnMmaLayout<HD>;
  constexpr int KS = HD / 16;
  constexpr int NT = HD / 8;
  constexpr int PIECES = HD / 8;
  constexpr float kNeg = -1.0e30f;
  const int tid = threadIdx.x;
  const int lane = tid & 31;
  const int warp = tid >> 5;
  const int g = lane >> 2;
  const int t = lane & 3;
  const int n_kv = a.n_kv, max_seq = a.max_seq;
  const int n_rep = a.n_q / n_kv;
  const int h_first = kvh * n_rep + z * kMmaHeads;
  const int nh = min(kMmaHeads, n_rep - z * kMmaHeads);
  const int half = HD >> 1;

  const uint32_t base = smem_u32(smem_raw);
  const uint32_t q_base = base + (L::kRing > L::kFoldBytes ? L::kRing : L::kFoldBytes);
  const uint32_t cur_base = q_base + L::kQBytes;
  __nv_bfloat16 *q_s = reinterpret_cast<__nv_bfloat16 *>(smem_raw + (q_base - base));
  __nv_bfloat16 *cur_s = reinterpret_cast<__nv_bfloat16 *>(smem_raw + (cur_base - base));
  int *is_last = reinterpret_cast<int *>(smem_raw + (cur_base - base) + L::kCurBytes);

  int vl = __ldcg(a.valid_len);
  const bool have_rope = a.cos != nullptr && a.sin != nullptr && a.position != nullptr;
  long long pos = have_rope ? __ldcg(reinterpret_cast<const long long *>(a.position)) : -1;
  vl = vl < 0 ? 0 : (vl > max_seq ? max_seq : vl);
  if (pos < 0 || pos >= max_seq) pos = -1;
  // Splits beyond the number of tiles have nothing to do: they leave at once, and the
  // others count, stride and merge with the number of splits that have work (every CTA
  // of the group derives the same number from the same valid length).
  const int n_tiles = (vl + kMmaTile - 1) / kMmaTile;
  const int n_split = min(a.n_split, max(n_tiles, 1));
  if (split >= n_split) return;
  const int n_my = split < n_tiles ? (n_tiles - split + n_split - 1) / n_split : 0;

  // A thread copies the same 16-byte piece of every (256 / PIECES)-th row of a tile, K
  // and V: its offsets are fixed, a copy costs an add and a compare.
  constexpr int kRowsPerPass = kMmaThreads / PIECES;
  constexpr int kPasses = kMmaTile / kRowsPerPass;
  static_assert(kMmaThreads % PIECES == 0 && kMmaTile % kRowsPerPass == 0, "tile copy split");
  const int r0 = tid / PIECES;
  const int piece = tid - r0 * PIECES;
  const size_t row_stride = static_cast<size_t>(n_kv) * HD;
  const size_t thread_off = static_cast<size_t>(kvh) * HD + piece * 8;
  const uint32_t thread_dst = static_cast<uint32_t>(r0 * L::kRowB + piece * 16);
  auto load_tile = [&](int i, int stage) {
    const int key0 = (split + i * n_split) * kMmaTile + r0;
    const uint32_t dst = base + stage * L::kStageBytes + thread_dst;
    const __nv_bfloat16 *ks = a.k_cache + static_cast<size_t>(key0) * row_stride + thread_off;
    const __nv_bfloat16 *vs = a.v_cache + static_cast<size_t>(key0) * row_stride + thread_off;
#pragma unroll
    for (int j = 0; j < kPasses; ++j) {
      const bool live = key0 + j * kRowsPerPass < vl;
      const size_t step = static_cast<size_t>(j * kRowsPerPass) * row_stride;
      mma_cp16(dst + j * kRowsPerPass * L::kRowB, live ? ks + step : a.k_cache, live ? 16 : 0);
      mma_cp16(dst + kMmaTile * L::kRowB + j * kRowsPerPass * L::kRowB, live ? vs + step : a.v_cache,
               live ? 16 : 0);
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
  };
#pragma unroll
  for (int i = 0; i < kMmaStages - 1; ++i) {
    if (i < n_my) load_tile(i, i);
  }

  // ---- prologue: rotated q (bf16) for the item's heads, current k / v (bf16) ----
  const __nv_bfloat16 *qg = a.q + static_cast<size_t>(kvh) * a.q_group_stride;
  __nv_bfloat16 *q_lo = q_s + kMmaHeads * HD;
  auto put_q = [&](int idx, float v) {
    const __nv_bfloat16 hi = __float2bfloat16(v);
    q_s[idx] = hi;
    q_lo[idx] = __float2bfloat16(v - __bfloat162float(hi));
  };
  for (int i = tid; i < kMmaHeads * HD; i += kMmaThreads) {
    if (i / HD >= nh) put_q(i, 0.f);
  }
  bool fuse_kv = false;
  if (pos >= 0) {
    const __nv_bfloat16 *c = a.cos + static_cast<size_t>(pos) * HD;
    const __nv_bfloat16 *s = a.sin + static_cast<size_t>(pos) * HD;
    fuse_kv = a.k_act != nullptr && a.v_act != nullptr;
    constexpr int kIters = (kMmaHeads * (HD / 2) + kMmaThreads - 1) / kMmaThreads;
    float qlo[kIters], qhi[kIters];
#pragma unroll
    for (int it = 0; it < kIters; ++it) {
      const int i = tid + it * kMmaThreads;
      const int h = i / half;
      const int d = i - h * half;
      const bool live = i < nh * half;
      const __nv_bfloat16 *qh = qg + static_cast<size_t>(z * kMmaHeads + h) * HD;
      qlo[it] = live ? ld_act_bf16(qh + d) : 0.f;
      qhi[it] = live ? ld_act_bf16(qh + d + half) : 0.f;
    }
    float klo = 0.f, khi = 0.f, vlo = 0.f, vhi = 0.f;
    if (fuse_kv && tid < half) {
      const __nv_bfloat16 *ka = a.k_act + static_cast<size_t>(kvh) * a.kv_act_stride;
      const __nv_bfloat16 *va = a.v_act + static_cast<size_t>(kvh) * a.kv_act_stride;
      klo = ld_act_bf16(ka + tid);
      khi = ld_act_bf16(ka + tid + half);
      vlo = ld_act_bf16(va + tid);
      vhi = ld_act_bf16(va + tid + half);
    }
#pragma unroll
    for (int it = 0; it < kIters; ++it) {
      const int i = tid + it * kMmaThreads;
      const int h = i / half;
      const int d = i - h * half;
      if (i < nh * half) {
        const float cl = __bfloat162float(c[d]), ch = __bfloat162float(c[d + half]);
        const float sl = __bfloat162float(s[d]), sh = __bfloat162float(s[d + half]);
        put_q(h * HD + d, qlo[it] * cl + (-qhi[it]) * sl);
        put_q(h * HD + d + half, qhi[it] * ch + qlo[it] * sh);
      }
    }
    if (fuse_kv && tid < half) {
      const float cl = __bfloat162float(c[tid]), ch = __bfloat162float(c[tid + half]);
      const float sl = __bfloat162float(s[tid]), sh = __bfloat162float(s[tid + half]);
      cur_s[tid] = __float2bfloat16(klo * cl + (-khi) * sl);
      cur_s[tid + half] = __float2bfloat16(khi * ch + klo * sh);
      cur_s[HD + tid] = __float2bfloat16(vlo);
      cur_s[HD + tid + half] = __float2bfloat16(vhi);
    }
  } else {
    for (int i = tid; i < nh * HD; i += kMmaThreads) {
      const int h = i / HD;
      put_q(i, ld_act_bf16(qg + static_cast<size_t>(z * kMmaHeads + h) * HD + (i - h * HD)));
    }
  }
  __syncthreads();

  // The CTA whose tiles hold row `pos` stores the new cache row (one per kv head).
  const int pos_i = fuse_kv ? static_cast<int>(pos) : -1;
  if (fuse_kv && z == 0 && (pos_i / kMmaTile) % n_split == split) {
    const size_t off = (static_cast<size_t>(pos_i) * n_kv + kvh) * HD;
    __nv_bfloat16 *kc = const_cast<__nv_bfloat16 *>(a.k_cache) + off;
    __nv_bfloat16 *vc = const_cast<__nv_bfloat16 *>(a.v_cache) + off;
    for (int d = tid; d < HD; d += kMmaThreads) {
      kc[d] = cur_s[d];
      vc[d] = cur_s[HD + d];
    }
  }

  // query fragments: rows 0..7 of the m16 tile are the item's heads, rows 8..15 are zero
  uint32_t qa0[KS], qa2[KS], ql0[KS], ql2[KS];
#pragma unroll
  for (int ks = 0; ks < KS; ++ks) {
    qa0[ks] = *reinterpret_cast<const uint32_t *>(q_s + g * HD + ks * 16 + 2 * t);
    qa2[ks] = *reinterpret_cast<const uint32_t *>(q_s + g * HD + ks * 16 + 8 + 2 * t);
    ql0[ks] = *reinterpret_cast<const uint32_t *>(q_lo + g * HD + ks * 16 + 2 * t);
    ql2[ks] = *reinterpret_cast<const uint32_t *>(q_lo + g * HD + ks * 16 + 8 + 2 * t);
  }
  const float c2 = a.scale * 1.4426950408889634f;  // scores in units of log2
  float o[NT][4];
#pragma unroll
  for (int i = 0; i < NT; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
  float m_run = kNeg, l_run = 0.f;
  const int lm_row = lane & 7;
  const int lm_mat = (lane >> 3) & 1;

  for (int i = 0; i < n_my; ++i) {
    const int stage = i % kMmaStages;
    // the stage of tile i + 2 held tile i - 1, which every warp left at the end of the
    // last round
    if (i + kMmaStages - 1 < n_my) load_tile(i + kMmaStages - 1, (i + kMmaStages - 1) % kMmaStages);
    const int later = min(n_my - 1 - i, kMmaStages - 1);  // groups requested after tile i's
    if (later >= 2) {
      asm volatile("cp.async.wait_group 2;" ::: "memory");
    } else if (later == 1) {
      asm volatile("cp.async.wait_group 1;" ::: "memory");
    } else {
      asm volatile("cp.async.wait_group 0;" ::: "memory");
    }
    __syncthreads();
    const int kv0 = (split + i * n_split) * kMmaTile;
    const uint32_t k_base = base + stage * L::kStageBytes;
    const uint32_t v_base = k_base + kMmaTile * L::kRowB;
    if (pos_i >= kv0 && pos_i < kv0 + kMmaTile) {
      // the current token's row: from the activation, not from the cache being written
      const int r = pos_i - kv0;
      for (int d = tid; d < HD; d += kMmaThreads) {
        asm volatile("st.shared.b16 [%0], %1;" ::"r"(k_base + r * L::kRowB + d * 2),
                     "h"(*reinterpret_cast<const unsigned short *>(cur_s + d))
                     : "memory");
        asm volatile("st.shared.b16 [%0], %1;" ::"r"(v_base + r * L::kRowB + d * 2),
                     "h"(*reinterpret_cast<const unsigned short *>(cur_s + HD + d))
                     : "memory");
      }
      __syncthreads();
    }
    const int key0 = kv0 + warp * 16;  // this warp's 16 rows of the tile
    if (key0 < vl) {
      float s[2][4];
#pragma unroll
      for (int nt = 0; nt < 2; ++nt) {
        s[nt][0] = s[nt][1] = s[nt][2] = s[nt][3] = 0.f;
#pragma unroll
        for (int ks = 0; ks < KS; ++ks) {
          uint32_t b0, b1;
          mma_ldm_x2(k_base + (warp * 16 + nt * 8 + lm_row) * L::kRowB + (ks * 16 + lm_mat * 8) * 2, b0, b1);
          mma_bf16(s[nt], qa0[ks], 0u, qa2[ks], 0u, b0, b1);
          mma_bf16(s[nt], ql0[ks], 0u, ql2[ks], 0u, b0, b1);
        }
      }
      // this thread's row g (a query head), four keys: key0 + nt*8 + 2t (+1)
      float sv[4];
      float mx = kNeg;
#pragma unroll
      for (int nt = 0; nt < 2; ++nt) {
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          const int key = key0 + nt * 8 + 2 * t + e;
          sv[nt * 2 + e] = key < vl ? s[nt][e] * c2 : kNeg;
          mx = fmaxf(mx, sv[nt * 2 + e]);
        }
      }
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
      const float m_new = fmaxf(m_run, mx);  // finite: the warp's first key is below vl
      const float alpha = exp2f(m_run - m_new);
      float p[4], psum = 0.f;
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        p[e] = exp2f(sv[e] - m_new);  // a masked key gives exp2(-1e30) = 0
        psum += p[e];
      }
      l_run = fmaf(l_run, alpha, psum);
      m_run = m_new;
      if (__any_sync(0xffffffffu, alpha != 1.f)) {
#pragma unroll
        for (int n = 0; n < NT; ++n) {
          o[n][0] *= alpha;
          o[n][1] *= alpha;
        }
      }
      // probabilities of rows 0..7 as the A fragment of one 16-key step (rows 8..15
      // zero), as a bf16 head and a bf16 remainder
      float plo[4];
#pragma unroll
      for (int e = 0; e < 4; ++e) plo[e] = p[e] - __bfloat162float(__float2bfloat16(p[e]));
      const uint32_t pa0 = mma_pack(p[0], p[1]);
      const uint32_t pa2 = mma_pack(p[2], p[3]);
      const uint32_t pl0 = mma_pack(plo[0], plo[1]);
      const uint32_t pl2 = mma_pack(plo[2], plo[3]);
#pragma unroll
      for (int n = 0; n < NT; ++n) {
        uint32_t b0, b1;
        mma_ldm_x2_trans(v_base + (warp * 16 + lm_mat * 8 + lm_row) * L::kRowB + n * 16, b0, b1);
        mma_bf16(o[n], pa0, 0u, pa2, 0u, b0, b1);
        mma_bf16(o[n], pl0, 0u, pl2, 0u, b0, b1);
      }
    }
    __syncthreads();  // this stage is requested again two rounds on
  }

  // ---- fold the warps: (m, l, o) of every warp and head through shared memory ----
  l_run += __shfl_xor_sync(0xffffffffu, l_run, 1);
  l_run += __shfl_xor_sync(0xffffffffu, l_run, 2);
  float *fold = reinterpret_cast<float *>(smem_raw);  // [warp][head][HD + 2]
  {
    float *mine = fold + (warp * kMmaHeads + g) * (HD + 2);
#pragma unroll
    for (int n = 0; n < NT; ++n) {
      mine[n * 8 + 2 * t] = o[n][0];
      mine[n * 8 + 2 * t + 1] = o[n][1];
    }
    if (t == 0) {
      mine[HD] = m_run;
      mine[HD + 1] = l_run;
    }
  }
  __syncthreads();
  for (int i = tid; i < nh * HD; i += kMmaThreads) {
    const int h = i / HD;
    const int d = i - h * HD;
    float mm = kNeg;
#pragma unroll
    for (int w = 0; w < kMmaWarps; ++w) mm = fmaxf(mm, fold[(w * kMmaHeads + h) * (HD + 2) + HD]);
    float ll = 0.f, oo = 0.f;
#pragma unroll
    for (int w = 0; w < kMmaWarps; ++w) {
      const float *src = fold + (w * kMmaHeads + h) * (HD + 2);
      const float wexp = exp2f(src[HD] - mm);
      ll = fmaf(wexp, src[HD + 1], ll);
      oo = fmaf(wexp, src[d], oo);
    }
    const size_t slot = static_cast<size_t>(h_first + h) * a.n_split + split;
    a.o_s[slot * HD + d] = oo;
    if (d == 0) {
      a.m_s[slot] = mm;
      a.l_s[slot] = ll;
    }
  }

  // ---- the last CTA of this (kv head, head chunk) to arrive merges the splits ----
  __threadfence();
  __syncthreads();
  if (tid == 0) {
    const unsigned int seen = atomicAdd(ctr, 1u);
    *is_last = seen == static_cast<unsigned int>(n_split) - 1u;
    if (*is_last) *ctr = 0u;
  }
  __syncthreads();
  if (!*is_last) return;
  __threadfence();
  float *wts = fold;  // [head][kAttnMaxSplit] softmax weights of the splits
  for (int h = warp; h < nh; h += kMmaWarps) {
    const size_t b0 = static_cast<size_t>(h_first + h) * a.n_split;
    const float ms = lane < n_split ? __ldcg(a.m_s + b0 + lane) : kNeg;
    const float ls = lane < n_split ? __ldcg(a.l_s + b0 + lane) : 0.f;
    const float mm = warp_max_xor(ms);
    const float wexp = exp2f(ms - mm);
    const float ll = warp_sum_xor(wexp * ls);
    wts[h * kAttnMaxSplit + lane] = ll > 0.f ? wexp / ll : 0.f;
  }
  __syncthreads();
  for (int i = tid; i < nh * HD; i += kMmaThreads) {
    const int h = i / HD;
    const int d = i - h * HD;
    const float *oh = a.o_s + static_cast<size_t>(h_first + h) * a.n_split * HD + d;
    float oo = 0.f;
    for (int s0 = 0; s0 < n_split; s0 += 8) {
      float pv[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) pv[j] = s0 + j < n_split ? __ldcg(oh + static_cast<size_t>(s0 + j) * HD) : 0.f;
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        if (s0 + j < n_split) oo = fmaf(wts[h * kAttnMaxSplit + s0 + j], pv[j], oo);
      }
    }
    a.out[static_cast<size_t>(h_first + h) * HD + d] = __float2bfloat16(oo);
  }
}

}  // namespace chr
