// Device core of the GQA decode attention (sm_100a), shared by the per-launch
// kernel and by the whole-step persistent kernel
// (reference: gpu/nf4/nf4_gemv.cu:558-727).
//
// One work item is a (kv head, sequence split, head chunk) triple handled by
// kAttnWarps warps; it serves every query head of the chunk, so a cache row is
// read once per group instead of once per query head. The last item of a
// (kv head, head chunk) to arrive merges the splits.
#pragma once

#include "nf4_common.cuh"

namespace chr {

constexpr int kAttnWarps = 8;
constexpr int kAttnAhead = 4;       // cache rows in flight per warp
constexpr int kAttnMaxSplit = 16;  // splits actually used: min(n_split, 16)
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

// P: bf16 pairs per lane (hd <= 64*P). H: query heads served by one item.
template <int P, int H>
struct AttnSmem {
  float qrot[H][64 * P];
  float krot[64 * P];
  float vcur[64 * P];
  float sm_m[kAttnWarps][H];
  float sm_l[kAttnWarps][H];
  float sm_o[kAttnWarps][H][64 * P];
  int is_last;
};

// Called by the kAttnThreads threads (tid 0..kAttnThreads-1) of one item; `sync`
// is a barrier over exactly those threads. `ctr` is the arrival counter of the
// item's (kv head, head chunk): zero before the first arrival, zero again after
// the last.
template <int P, int H, class Sync>
__device__ __forceinline__ void attn_item(const AttnArgs &a, AttnSmem<P, H> &sm, int split,
                                          int kvh, int z, unsigned int *ctr, int tid, Sync sync) {
  auto &qrot = sm.qrot;
  auto &krot = sm.krot;
  auto &vcur = sm.vcur;
  auto &sm_m = sm.sm_m;
  auto &sm_l = sm.sm_l;
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

  int vl = __ldcg(a.valid_len);
  vl = vl < 0 ? 0 : (vl > max_seq ? max_seq : vl);

  long long pos = -1;
  bool fuse_kv = false;
  const bool have_rope = a.cos != nullptr && a.sin != nullptr && a.position != nullptr;
  if (have_rope) {
    pos = __ldcg(reinterpret_cast<const long long *>(a.position));
    if (pos < 0 || pos >= max_seq) pos = -1;
  }
  if (pos >= 0) {
    const __nv_bfloat16 *c = a.cos + static_cast<size_t>(pos) * hd;
    const __nv_bfloat16 *s = a.sin + static_cast<size_t>(pos) * hd;
    for (int i = tid; i < nh * half; i += kAttnThreads) {
      const int h = i / half;
      const int d = i - h * half;
      const __nv_bfloat16 *qh = qg + static_cast<size_t>(z * H + h) * hd;
      const float lo = ld_act_bf16(qh + d);
      const float hi = ld_act_bf16(qh + d + half);
      qrot[h][d] = lo * __bfloat162float(c[d]) + (-hi) * __bfloat162float(s[d]);
      qrot[h][d + half] = hi * __bfloat162float(c[d + half]) + lo * __bfloat162float(s[d + half]);
    }
    if (a.k_act != nullptr && a.v_act != nullptr) {
      fuse_kv = true;
      const __nv_bfloat16 *ka = a.k_act + static_cast<size_t>(kvh) * a.kv_act_stride;
      const __nv_bfloat16 *va = a.v_act + static_cast<size_t>(kvh) * a.kv_act_stride;
      for (int d = tid; d < half; d += kAttnThreads) {
        const float lo = ld_act_bf16(ka + d);
        const float hi = ld_act_bf16(ka + d + half);
        krot[d] = lo * __bfloat162float(c[d]) + (-hi) * __bfloat162float(s[d]);
        krot[d + half] = hi * __bfloat162float(c[d + half]) + lo * __bfloat162float(s[d + half]);
      }
      for (int d = tid; d < hd; d += kAttnThreads) vcur[d] = ld_act_bf16(va + d);
    }
  } else {
    for (int i = tid; i < nh * hd; i += kAttnThreads) {
      const int h = i / hd;
      const int d = i - h * hd;
      qrot[h][d] = ld_act_bf16(qg + static_cast<size_t>(z * H + h) * hd + d);
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

  // Lane owns elements d = 2*lane + 64*p (+0, +1).
  float qreg[H][2 * P];
#pragma unroll
  for (int h = 0; h < H; ++h) {
#pragma unroll
    for (int p = 0; p < P; ++p) {
      const int d = 2 * lane + 64 * p;
      const bool live = h < nh && d < hd;
      qreg[h][2 * p] = live ? qrot[h][d] : 0.f;
      qreg[h][2 * p + 1] = live ? qrot[h][d + 1] : 0.f;
    }
  }

  float m[H], l[H], acc[H][2 * P];
#pragma unroll
  for (int h = 0; h < H; ++h) {
    m[h] = kNegInit;
    l[h] = 0.f;
#pragma unroll
    for (int e = 0; e < 2 * P; ++e) acc[h][e] = 0.f;
  }

  // Token loop with kAttnAhead rows in flight per warp: a row's K/V are requested
  // that many rows before they are scored. Row i of this warp: split + warp*n_split
  // + i*kAttnWarps*n_split.
  const int t_step = kAttnWarps * n_split;
  auto fetch = [&](int t, uint32_t (&kk)[P], uint32_t (&vv)[P]) {
    const size_t row = (static_cast<size_t>(t) * n_kv + kvh) * hd;
#pragma unroll
    for (int p = 0; p < P; ++p) {
      const int d = 2 * lane + 64 * p;
      const bool live = t < vl && d < hd;
      kk[p] = live ? __ldg(reinterpret_cast<const uint32_t *>(a.k_cache + row + d)) : 0u;
      vv[p] = live ? __ldg(reinterpret_cast<const uint32_t *>(a.v_cache + row + d)) : 0u;
    }
  };
  auto score = [&](int t, const uint32_t (&kb)[P], const uint32_t (&vb)[P]) {
    float kk[2 * P], vv[2 * P];
    const bool cur = fuse_kv && t == pos;
#pragma unroll
    for (int p = 0; p < P; ++p) {
      const int d = 2 * lane + 64 * p;
      if (cur && d < hd) {
        kk[2 * p] = krot[d];
        kk[2 * p + 1] = krot[d + 1];
        vv[2 * p] = vcur[d];
        vv[2 * p + 1] = vcur[d + 1];
      } else {
        kk[2 * p] = bf16_lo(kb[p]);
        kk[2 * p + 1] = bf16_hi(kb[p]);
        vv[2 * p] = bf16_lo(vb[p]);
        vv[2 * p + 1] = bf16_hi(vb[p]);
      }
    }
    float dots[H];
#pragma unroll
    for (int h = 0; h < H; ++h) {
      float dot = 0.f;
#pragma unroll
      for (int e = 0; e < 2 * P; ++e) dot = fmaf(qreg[h][e], kk[e], dot);
      dots[h] = dot;
    }
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) {
#pragma unroll
      for (int h = 0; h < H; ++h) dots[h] += __shfl_xor_sync(0xffffffffu, dots[h], off);
    }
#pragma unroll
    for (int h = 0; h < H; ++h) {
      const float dot = dots[h] * scale;
      const float m2 = fmaxf(m[h], dot);
      const float alpha = __expf(m[h] - m2);
      const float ex = __expf(dot - m2);
      l[h] = l[h] * alpha + ex;
#pragma unroll
      for (int e = 0; e < 2 * P; ++e) acc[h][e] = acc[h][e] * alpha + ex * vv[e];
      m[h] = m2;
    }
  };
  uint32_t kq[kAttnAhead][P], vq[kAttnAhead][P];
  int t = split + warp * n_split;
#pragma unroll
  for (int d = 0; d < kAttnAhead; ++d) fetch(t + d * t_step, kq[d], vq[d]);
  for (; t < vl; t += kAttnAhead * t_step) {
#pragma unroll
    for (int d = 0; d < kAttnAhead; ++d) {
      const int tt = t + d * t_step;
      if (tt < vl) score(tt, kq[d], vq[d]);
      fetch(tt + kAttnAhead * t_step, kq[d], vq[d]);
    }
  }

  // Combine the warps, in warp order, into this split's (m, l, o).
#pragma unroll
  for (int h = 0; h < H; ++h) {
    if (lane == 0) {
      sm_m[warp][h] = m[h];
      sm_l[warp][h] = l[h];
    }
#pragma unroll
    for (int p = 0; p < P; ++p) {
      const int d = 2 * lane + 64 * p;
      sm_o[warp][h][d] = acc[h][2 * p];
      sm_o[warp][h][d + 1] = acc[h][2 * p + 1];
    }
  }
  sync();
  for (int i = tid; i < nh * hd; i += kAttnThreads) {
    const int h = i / hd;
    const int d = i - h * hd;
    float mm = kNegInit;
#pragma unroll
    for (int w = 0; w < kAttnWarps; ++w) mm = fmaxf(mm, sm_m[w][h]);
    float ll = 0.f, oo = 0.f;
#pragma unroll
    for (int w = 0; w < kAttnWarps; ++w) {
      const float wexp = __expf(sm_m[w][h] - mm);
      ll += wexp * sm_l[w][h];
      oo += wexp * sm_o[w][h][d];
    }
    const size_t slot = static_cast<size_t>(h_first + h) * n_split + split;
    a.o_s[slot * hd + d] = oo;
    if (d == 0) {
      a.m_s[slot] = mm;
      a.l_s[slot] = ll;
    }
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
  // One round trip for the merge: every thread puts the loads of its partial sums in
  // flight first, the splits' (m, l) are fetched and turned into softmax weights
  // meanwhile, and the weighted sum runs on registers.
  constexpr int kIters = H * 64 * P / kAttnThreads;
  float pv[kIters][kAttnMaxSplit];
#pragma unroll
  for (int it = 0; it < kIters; ++it) {
    const int i = tid + it * kAttnThreads;
    const int h = i / hd;
    const int d = i - h * hd;
    const float *oh = a.o_s + static_cast<size_t>(h_first + h) * n_split * hd + d;
#pragma unroll
    for (int sidx = 0; sidx < kAttnMaxSplit; ++sidx) {
      pv[it][sidx] = (i < nh * hd && sidx < n_split) ? __ldcg(oh + static_cast<size_t>(sidx) * hd)
                                                     : 0.f;
    }
  }
  // softmax weights of the splits, once per head: w[h][s] = exp(m_s - max) / sum
  float *wts = &sm_o[0][0][0];  // the combine buffer is free again
  for (int h = warp; h < nh; h += kAttnWarps) {
    const size_t base = static_cast<size_t>(h_first + h) * n_split;
    const float ms = lane < n_split ? __ldcg(a.m_s + base + lane) : kNegInit;
    const float ls = lane < n_split ? __ldcg(a.l_s + base + lane) : 0.f;
    const float mm = warp_max_xor(ms);
    const float wexp = __expf(ms - mm);
    const float ll = warp_sum_xor(wexp * ls);
    if (lane < kAttnMaxSplit) wts[h * kAttnMaxSplit + lane] = ll > 0.f ? wexp / ll : 0.f;
  }
  sync();
#pragma unroll
  for (int it = 0; it < kIters; ++it) {
    const int i = tid + it * kAttnThreads;
    if (i < nh * hd) {
      const int h = i / hd;
      const int d = i - h * hd;
      float oo = 0.f;
#pragma unroll
      for (int sidx = 0; sidx < kAttnMaxSplit; ++sidx) {
        oo += wts[h * kAttnMaxSplit + sidx] * pv[it][sidx];
      }
      a.out[static_cast<size_t>(h_first + h) * hd + d] = __float2bfloat16(oo);
    }
  }
}

}  // namespace chr
