// Device core of the GQA decode attention (sm_100a)
// (reference: gpu/nf4/nf4_gemv.cu:558-727).
//
// One work item is a (kv head, sequence split, head chunk) triple handled by
// kAttnWarps warps; it serves every query head of the chunk, so a cache row is
// read once per group instead of once per query head. Inside a warp every lane owns
// one 16-byte piece (8 elements) of a cache row, so a warp scores 4, 2 or 1 rows at
// a time (head dim up to 64, 128, 256) and a dot product needs 3, 4 or 5 shuffle
// steps. The token loop is kept free of branches and small: with two to four warps
// per scheduler the kernel is bound by instruction fetch and dependent-issue
// latency, not by memory. The last item of a (kv head, head chunk) to arrive merges
// the splits.
#pragma once

#include "nf4_common.cuh"

namespace chr {

constexpr int kAttnWarps = 16;
constexpr int kAttnStages = 4;      // ring stages per warp
constexpr int kAttnMaxSplit = 32;   // splits actually used: min(n_split, 32)
constexpr int kAttnMergeBatch = 16;  // partial sums a merging thread keeps in flight per pass
constexpr int kAttnThreads = kAttnWarps * 32;
constexpr float kNegInit = -1.0e30f;

// Arrival counters for the merge-by-last-CTA step: one per (kv head, head chunk).
// Zero at load, and the last CTA of a group puts its counter back to zero, so a
// launch leaves them as it found them. Launches of the attention kernel that
// overlap on the device (different streams) would share them and must not.
constexpr int kMaxAttnGroups = 1024;

struct AttnArgs {
  const __nv_bfloat16 *q;        // query heads; kv group g starts at q + g * q_group_stride
  int q_group_stride;
  const __nv_bfloat16 *k_act;    // this token's k / v per kv head (stride kv_act_stride), or null
  const __nv_bfloat16 *v_act;
  int kv_act_stride;
  const __nv_bfloat16 *k_cache;  // [max_seq, n_kv, hd]
  const __nv_bfloat16 *v_cache;
  __nv_bfloat16 *out;            // [n_q, hd]
  float *m_s, *l_s, *o_s;        // split partials
  const int32_t *valid_len;
  const __nv_bfloat16 *cos, *sin;
  const int64_t *position;
  int n_q, n_kv, hd, n_split, max_seq;
  float scale;
};

// Per-warp ring of cache rows, filled with cp.async. A row slot holds 64*P bf16 of K
// and as many of V; a stage holds the rows a warp scores together, one per group of
// 8*P lanes, which makes a stage 1 KB whatever P is.
template <int P>
struct AttnRing {
  static constexpr int kPieces = 8 * P;          // 16-byte pieces of a row slot = lanes per row
  static constexpr int kRows = 32 / kPieces;     // rows per stage
  static constexpr int kRowBytes = 128 * P;      // one K (or V) row slot
  static constexpr int kStageBytes = kRows * 2 * kRowBytes;
  static constexpr int kWarpBytes = kAttnStages * kStageBytes;
};

// P: head dim <= 64*P. H: query heads served by one item. Lives in dynamic shared
// memory (above 48 KB). The ring shares its memory with the warp-combine buffer,
// which is only used after the token loop.
template <int P, int H>
struct AttnSmem {
  float qrot[H][64 * P];  // piece-major: see q_index()
  float krot[64 * P];
  float vcur[64 * P];
  float sm_m[kAttnWarps][H];
  float sm_l[kAttnWarps][H];
  float sm_w[kAttnWarps][H];
  union alignas(16) {
    float sm_o[kAttnWarps][H][64 * P];
    unsigned char ring[kAttnWarps][AttnRing<P>::kWarpBytes];
  };
  int is_last;
};

// Where element d of a rotated query head sits in shared memory: the first four
// elements of every 8-element piece form one plane, the last four a second plane, so
// that the lanes of a row (one piece each) read 16-byte words that lie side by side.
template <int P>
__device__ __forceinline__ int q_index(int d) {
  return ((d & 7) >> 2) * (32 * P) + (d >> 3) * 4 + (d & 3);
}

__device__ __forceinline__ uint32_t smem_u32(const void *p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}
__device__ __forceinline__ void cp_async16(uint32_t dst, const void *src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}
__device__ __forceinline__ uint4 lds128(uint32_t addr) {
  uint4 v;
  asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "r"(addr));
  return v;
}

// Called by the kAttnThreads threads (tid 0..kAttnThreads-1) of one item; `sync`
// is a barrier over exactly those threads. `ctr` is the arrival counter of the
// item's (kv head, head chunk): zero before the first arrival, zero again after
// the last.
template <int P, int H, class Sync>
__device__ __forceinline__ void attn_item(const AttnArgs &a, AttnSmem<P, H> &sm, int split,
                                          int kvh, int z, unsigned int *ctr, int tid, Sync sync) {
  using Ring = AttnRing<P>;
  auto &qrot = sm.qrot;
  auto &krot = sm.krot;
  auto &vcur = sm.vcur;
  auto &sm_m = sm.sm_m;
  auto &sm_l = sm.sm_l;
  auto &sm_w = sm.sm_w;
  auto &sm_o = sm.sm_o;
  int &is_last = sm.is_last;
  const int n_q = a.n_q, n_kv = a.n_kv, hd = a.hd, n_split = a.n_split, max_seq = a.max_seq;
  const float scale = a.scale;
  const __nv_bfloat16 *qg = a.q + static_cast<size_t>(kvh) * a.q_group_stride;
  const int n_rep = n_q / n_kv;
  const int h_first = kvh * n_rep + z * H;  // first query head of this item
  const int nh = min(H, n_rep - z * H);
  const int lane = tid & 31;
  const int warp = tid >> 5;
  const int half = hd >> 1;
  const int grp = lane / Ring::kPieces;    // which of the stage's rows this lane works on
  const int piece = lane % Ring::kPieces;  // the 8 elements of the row this lane owns

  int vl = __ldcg(a.valid_len);
  const bool have_rope = a.cos != nullptr && a.sin != nullptr && a.position != nullptr;
  long long pos = have_rope ? __ldcg(reinterpret_cast<const long long *>(a.position)) : -1;
  vl = vl < 0 ? 0 : (vl > max_seq ? max_seq : vl);
  if (pos < 0 || pos >= max_seq) pos = -1;

  // Row j of this warp: split + (warp + j*kAttnWarps) * n_split; stage s of the ring
  // carries rows j = kRows*s .. kRows*s + kRows-1. The slots start out as zeros (a row
  // that is never requested must not read as NaN), then the requests of the whole ring
  // go out and are in flight while the prologue below runs.
  const int t_step = kAttnWarps * n_split;
  const uint32_t ring_base = smem_u32(&sm.ring[warp][0]);
  const int chunks = (hd + 7) >> 3;  // 8-element pieces of one row (the last may be partial)
  const bool by16 = (hd & 7) == 0 && ((reinterpret_cast<uintptr_t>(a.k_cache) |
                                       reinterpret_cast<uintptr_t>(a.v_cache)) & 15) == 0;
#pragma unroll
  for (int i = 0; i < Ring::kWarpBytes / 512; ++i) {
    asm volatile("st.shared.v4.b32 [%0], {%1, %1, %1, %1};" ::"r"(ring_base + (i * 32 + lane) * 16),
                 "r"(0u)
                 : "memory");
  }
  __syncwarp();
  auto request = [&](int t0, int stage) {
    const uint32_t dst0 = ring_base + stage * Ring::kStageBytes;
    if (by16) {
      // 2 * kPieces pieces per row (K then V), kRows rows: 64 pieces, two per lane
#pragma unroll
      for (int j = 0; j < 2; ++j) {
        const int idx = lane + 32 * j;
        const int r = idx / (2 * Ring::kPieces);
        const int c = idx % (2 * Ring::kPieces);
        const bool is_v = c >= Ring::kPieces;
        const int cc = is_v ? c - Ring::kPieces : c;
        const int t = t0 + r * t_step;
        if (t < vl && cc < chunks) {
          const size_t row = (static_cast<size_t>(t) * n_kv + kvh) * hd;
          cp_async16(dst0 + idx * 16, (is_v ? a.v_cache : a.k_cache) + row + cc * 8);
        }
      }
    } else {
      for (int r = 0; r < Ring::kRows; ++r) {
        const int t = t0 + r * t_step;
        if (t < vl) {
          const size_t row = (static_cast<size_t>(t) * n_kv + kvh) * hd;
          const uint32_t dst = dst0 + r * 2 * Ring::kRowBytes;
          for (int c = lane; c < half; c += 32) {
            const uint32_t kw = __ldg(reinterpret_cast<const uint32_t *>(a.k_cache + row + 2 * c));
            const uint32_t vw = __ldg(reinterpret_cast<const uint32_t *>(a.v_cache + row + 2 * c));
            asm volatile("st.shared.b32 [%0], %1;" ::"r"(dst + c * 4), "r"(kw) : "memory");
            asm volatile("st.shared.b32 [%0], %1;" ::"r"(dst + Ring::kRowBytes + c * 4), "r"(vw)
                         : "memory");
          }
        }
      }
    }
    cp_async_commit();
  };
  const int t_first = split + warp * n_split;
#pragma unroll
  for (int s = 0; s < kAttnStages; ++s) request(t_first + s * Ring::kRows * t_step, s);

  // Query rows the item does not have and elements past hd read as zero in the dot
  // products (the lanes read whole 8-element pieces).
  for (int i = tid; i < H * 64 * P; i += kAttnThreads) {
    const int h = i / (64 * P);
    const int d = i - h * (64 * P);
    if (h >= nh || d >= hd) qrot[h][q_index<P>(d)] = 0.f;
  }
  for (int d = hd + tid; d < 64 * P; d += kAttnThreads) {
    krot[d] = 0.f;
    vcur[d] = 0.f;
  }

  // Prologue: every global load that does not need the position is issued before
  // the first use of the position; the rotary table loads follow in one batch.
  bool fuse_kv = false;
  if (pos >= 0) {
    const __nv_bfloat16 *c = a.cos + static_cast<size_t>(pos) * hd;
    const __nv_bfloat16 *s = a.sin + static_cast<size_t>(pos) * hd;
    constexpr int kQIters = (H * 32 * P + kAttnThreads - 1) / kAttnThreads;
    float qlo[kQIters], qhi[kQIters];
#pragma unroll
    for (int it = 0; it < kQIters; ++it) {
      const int i = tid + it * kAttnThreads;
      const int h = i / half;
      const int d = i - h * half;
      const bool live = i < nh * half;
      const __nv_bfloat16 *qh = qg + static_cast<size_t>(z * H + h) * hd;
      qlo[it] = live ? ld_act_bf16(qh + d) : 0.f;
      qhi[it] = live ? ld_act_bf16(qh + d + half) : 0.f;
    }
    fuse_kv = a.k_act != nullptr && a.v_act != nullptr;
    float klo = 0.f, khi = 0.f, vlo = 0.f, vhi = 0.f;
    if (fuse_kv && tid < half) {
      const __nv_bfloat16 *ka = a.k_act + static_cast<size_t>(kvh) * a.kv_act_stride;
      const __nv_bfloat16 *va = a.v_act + static_cast<size_t>(kvh) * a.kv_act_stride;
      klo = ld_act_bf16(ka + tid);
      khi = ld_act_bf16(ka + tid + half);
      vlo = ld_act_bf16(va + tid);
      vhi = ld_act_bf16(va + tid + half);
    }
    float clo[kQIters], chi[kQIters], slo[kQIters], shi[kQIters];
#pragma unroll
    for (int it = 0; it < kQIters; ++it) {
      const int d = (tid + it * kAttnThreads) % half;
      clo[it] = __bfloat162float(c[d]);
      chi[it] = __bfloat162float(c[d + half]);
      slo[it] = __bfloat162float(s[d]);
      shi[it] = __bfloat162float(s[d + half]);
    }
#pragma unroll
    for (int it = 0; it < kQIters; ++it) {
      const int i = tid + it * kAttnThreads;
      const int h = i / half;
      const int d = i - h * half;
      if (i < nh * half) {
        qrot[h][q_index<P>(d)] = qlo[it] * clo[it] + (-qhi[it]) * slo[it];
        qrot[h][q_index<P>(d + half)] = qhi[it] * chi[it] + qlo[it] * shi[it];
      }
    }
    if (fuse_kv && tid < half) {
      // tid < half <= 128: iteration 0 of the table loads covers d = tid
      krot[tid] = klo * clo[0] + (-khi) * slo[0];
      krot[tid + half] = khi * chi[0] + klo * shi[0];
      vcur[tid] = vlo;
      vcur[tid + half] = vhi;
    }
  } else {
    for (int i = tid; i < nh * hd; i += kAttnThreads) {
      const int h = i / hd;
      const int d = i - h * hd;
      qrot[h][q_index<P>(d)] = ld_act_bf16(qg + static_cast<size_t>(z * H + h) * hd + d);
    }
  }
  sync();

  // One CTA per kv head stores the new cache row; every CTA attends the current
  // token from the FP32 values above, never from the row being written.
  if (fuse_kv && z == 0 && split == static_cast<int>(pos % n_split)) {
    const size_t off = (static_cast<size_t>(pos) * n_kv + kvh) * hd;
    __nv_bfloat16 *kc = const_cast<__nv_bfloat16 *>(a.k_cache) + off;
    __nv_bfloat16 *vc = const_cast<__nv_bfloat16 *>(a.v_cache) + off;
    for (int d = tid; d < hd; d += kAttnThreads) {
      kc[d] = __float2bfloat16(krot[d]);
      vc[d] = __float2bfloat16(vcur[d]);
    }
  }

  // Running softmax of this lane group's rows over the lane's 8 elements.
  float m[H], l[H], acc[H][8];
#pragma unroll
  for (int h = 0; h < H; ++h) {
    m[h] = kNegInit;
    l[h] = 0.f;
#pragma unroll
    for (int e = 0; e < 8; ++e) acc[h][e] = 0.f;
  }
  const uint32_t q_lane = smem_u32(&qrot[0][0]) + piece * 16;

  // One row per lane group: dot products of all H heads (heads the item does not have
  // carry zero queries), 3-5 shuffle steps, one running-softmax update. No branches.
  auto attend = [&](const float (&kf)[8], const float (&vf)[8], bool on) {
    float dots[H];
#pragma unroll
    for (int h = 0; h < H; ++h) {
      const uint4 q0 = lds128(q_lane + h * 256 * P);
      const uint4 q1 = lds128(q_lane + h * 256 * P + 128 * P);
      float d0 = __uint_as_float(q0.x) * kf[0];
      float d1 = __uint_as_float(q0.y) * kf[1];
      d0 = fmaf(__uint_as_float(q0.z), kf[2], d0);
      d1 = fmaf(__uint_as_float(q0.w), kf[3], d1);
      d0 = fmaf(__uint_as_float(q1.x), kf[4], d0);
      d1 = fmaf(__uint_as_float(q1.y), kf[5], d1);
      d0 = fmaf(__uint_as_float(q1.z), kf[6], d0);
      d1 = fmaf(__uint_as_float(q1.w), kf[7], d1);
      dots[h] = d0 + d1;
    }
#pragma unroll
    for (int off = Ring::kPieces / 2; off > 0; off >>= 1) {
#pragma unroll
      for (int h = 0; h < H; ++h) dots[h] += __shfl_xor_sync(0xffffffffu, dots[h], off);
    }
#pragma unroll
    for (int h = 0; h < H; ++h) {
      const float sc = on ? dots[h] * scale : kNegInit;
      const float m2 = fmaxf(m[h], sc);
      const float alpha = __expf(m[h] - m2);
      const float ex = on ? __expf(sc - m2) : 0.f;
      l[h] = fmaf(l[h], alpha, ex);
#pragma unroll
      for (int e = 0; e < 8; ++e) acc[h][e] = fmaf(ex, vf[e], acc[h][e] * alpha);
      m[h] = m2;
    }
  };
  const int skip = fuse_kv ? static_cast<int>(pos) : -1;  // the current row is attended from FP32
  {
    int stage = 0;
    for (int t0 = t_first; t0 < vl; t0 += Ring::kRows * t_step) {
      cp_async_wait<kAttnStages - 1>();
      __syncwarp();
      const int t = t0 + grp * t_step;
      const uint32_t src = ring_base + stage * Ring::kStageBytes + grp * 2 * Ring::kRowBytes + piece * 16;
      const uint4 kb = lds128(src);
      const uint4 vb = lds128(src + Ring::kRowBytes);
      const float kf[8] = {bf16_lo(kb.x), bf16_hi(kb.x), bf16_lo(kb.y), bf16_hi(kb.y),
                           bf16_lo(kb.z), bf16_hi(kb.z), bf16_lo(kb.w), bf16_hi(kb.w)};
      const float vf[8] = {bf16_lo(vb.x), bf16_hi(vb.x), bf16_lo(vb.y), bf16_hi(vb.y),
                           bf16_lo(vb.z), bf16_hi(vb.z), bf16_lo(vb.w), bf16_hi(vb.w)};
      attend(kf, vf, t < vl && t != skip);
      __syncwarp();
      request(t0 + kAttnStages * Ring::kRows * t_step, stage);
      stage = stage + 1 == kAttnStages ? 0 : stage + 1;
    }
    cp_async_wait<0>();
  }
  // The current token, from the FP32 values of the prologue, in the lane group its
  // cache row belongs to.
  if (skip >= 0 && skip < vl && skip % n_split == split) {
    const int j = skip / n_split;  // row index within the split: warp + kAttnWarps * i
    if (j % kAttnWarps == warp) {
      const int own = (j / kAttnWarps) % Ring::kRows;
      const uint32_t kb = smem_u32(&krot[0]) + piece * 32;
      const uint32_t vb = smem_u32(&vcur[0]) + piece * 32;
      const uint4 k0 = lds128(kb), k1 = lds128(kb + 16), v0 = lds128(vb), v1 = lds128(vb + 16);
      const float kf[8] = {__uint_as_float(k0.x), __uint_as_float(k0.y), __uint_as_float(k0.z),
                           __uint_as_float(k0.w), __uint_as_float(k1.x), __uint_as_float(k1.y),
                           __uint_as_float(k1.z), __uint_as_float(k1.w)};
      const float vf[8] = {__uint_as_float(v0.x), __uint_as_float(v0.y), __uint_as_float(v0.z),
                           __uint_as_float(v0.w), __uint_as_float(v1.x), __uint_as_float(v1.y),
                           __uint_as_float(v1.z), __uint_as_float(v1.w)};
      attend(kf, vf, grp == own);
    }
  }

  // The lane groups of the warp fold their running softmax into one.
#pragma unroll
  for (int off = Ring::kPieces; off < 32; off <<= 1) {
#pragma unroll
    for (int h = 0; h < H; ++h) {
      const float mm = fmaxf(m[h], __shfl_xor_sync(0xffffffffu, m[h], off));
      const float w = __expf(m[h] - mm);
      const float ll = l[h] * w;
      l[h] = ll + __shfl_xor_sync(0xffffffffu, ll, off);
      m[h] = mm;
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        const float v = acc[h][e] * w;
        acc[h][e] = v + __shfl_xor_sync(0xffffffffu, v, off);
      }
    }
  }
  sync();  // every warp is done with its ring: the memory becomes the combine buffer

  // Combine the warps into this split's (m, l, o): weights first, then the sums.
  if (grp == 0) {
#pragma unroll
    for (int h = 0; h < H; ++h) {
      if (lane == 0) {
        sm_m[warp][h] = m[h];
        sm_l[warp][h] = l[h];
      }
      float4 *dst = reinterpret_cast<float4 *>(&sm_o[warp][h][piece * 8]);
      dst[0] = make_float4(acc[h][0], acc[h][1], acc[h][2], acc[h][3]);
      dst[1] = make_float4(acc[h][4], acc[h][5], acc[h][6], acc[h][7]);
    }
  }
  sync();
  {
    // thread (h, w): 16 neighbouring lanes hold the 16 warps' values of head h
    static_assert(kAttnWarps == 16, "the weight step maps one head to 16 lanes");
    const int h = tid >> 4;
    const int w = tid & 15;
    const bool valid = h < nh;
    const float ms = valid ? sm_m[w][h] : kNegInit;
    float mm = ms;
#pragma unroll
    for (int off = 8; off > 0; off >>= 1) mm = fmaxf(mm, __shfl_xor_sync(0xffffffffu, mm, off));
    const float wexp = __expf(ms - mm);
    float ll = valid ? wexp * sm_l[w][h] : 0.f;
#pragma unroll
    for (int off = 8; off > 0; off >>= 1) ll += __shfl_xor_sync(0xffffffffu, ll, off);
    if (valid) {
      sm_w[w][h] = wexp;
      if (w == 0) {
        const size_t slot = static_cast<size_t>(h_first + h) * n_split + split;
        a.m_s[slot] = mm;
        a.l_s[slot] = ll;
      }
    }
  }
  sync();
  for (int i = tid; i < nh * hd; i += kAttnThreads) {
    const int h = i / hd;
    const int d = i - h * hd;
    float oo = 0.f;
#pragma unroll
    for (int w = 0; w < kAttnWarps; ++w) oo = fmaf(sm_w[w][h], sm_o[w][h][d], oo);
    const size_t slot = static_cast<size_t>(h_first + h) * n_split + split;
    a.o_s[slot * hd + d] = oo;
  }

  // The last CTA of this (kv head, head chunk) to arrive merges the splits.
  __threadfence();
  sync();
  if (tid == 0) {
    const unsigned int seen = atomicAdd(ctr, 1u);
    is_last = seen == static_cast<unsigned int>(n_split) - 1u;
    if (is_last) *ctr = 0u;
  }
  sync();
  if (!is_last) return;
  __threadfence();
  // The merge runs in passes of kAttnMergeBatch splits: every thread puts the loads of
  // its partial sums of a pass in flight first; during the first pass the splits' (m, l)
  // are fetched and turned into softmax weights meanwhile; the weighted sum runs on
  // registers.
  constexpr int kIters = (H * 64 * P + kAttnThreads - 1) / kAttnThreads;
  float pv[kIters][kAttnMergeBatch];
  auto load_pass = [&](int s0) {
#pragma unroll
    for (int it = 0; it < kIters; ++it) {
      const int i = tid + it * kAttnThreads;
      const int h = i / hd;
      const int d = i - h * hd;
      const float *oh = a.o_s + static_cast<size_t>(h_first + h) * n_split * hd + d;
#pragma unroll
      for (int j = 0; j < kAttnMergeBatch; ++j) {
        const int sidx = s0 + j;
        pv[it][j] = (i < nh * hd && sidx < n_split) ? __ldcg(oh + static_cast<size_t>(sidx) * hd) : 0.f;
      }
    }
  };
  load_pass(0);
  // softmax weights of the splits, once per head: w[h][s] = exp(m_s - max) / sum
  float *wts = &sm_o[0][0][0];  // the combine buffer is free again
  for (int h = warp; h < nh; h += kAttnWarps) {
    const size_t base = static_cast<size_t>(h_first + h) * n_split;
    const float ms = lane < n_split ? __ldcg(a.m_s + base + lane) : kNegInit;
    const float ls = lane < n_split ? __ldcg(a.l_s + base + lane) : 0.f;
    const float mm = warp_max_xor(ms);
    const float wexp = __expf(ms - mm);
    const float ll = warp_sum_xor(wexp * ls);
    wts[h * kAttnMaxSplit + lane] = ll > 0.f ? wexp / ll : 0.f;
  }
  sync();
  float oo[kIters];
#pragma unroll
  for (int it = 0; it < kIters; ++it) oo[it] = 0.f;
  for (int s0 = 0; s0 < n_split; s0 += kAttnMergeBatch) {
    if (s0 > 0) load_pass(s0);
#pragma unroll
    for (int it = 0; it < kIters; ++it) {
      const int i = tid + it * kAttnThreads;
      if (i < nh * hd) {
        const int h = i / hd;
#pragma unroll
        for (int j = 0; j < kAttnMergeBatch; ++j) {
          if (s0 + j < n_split) oo[it] += wts[h * kAttnMaxSplit + s0 + j] * pv[it][j];
        }
      }
    }
  }
#pragma unroll
  for (int it = 0; it < kIters; ++it) {
    const int i = tid + it * kAttnThreads;
    if (i < nh * hd) {
      const int h = i / hd;
      const int d = i - h * hd;
      a.out[static_cast<size_t>(h_first + h) * hd + d] = __float2bfloat16(oo[it]);
    }
  }
}

}  // namespace chr
