// Causal GQA attention of one prefill chunk over the bf16 KV prefix (sm_100a).
//
// The reference runs torch's scaled_dot_product_attention per chunk with a boolean
// mask "key position <= query position" over cache rows 0 .. start+n-1
// (gpu/decodev2/prefill.py:50-92). This kernel computes the same thing straight from
// the cache layout [max_seq, n_kv, hd], without a mask tensor and without the
// transposed cache view: a flash-style pass with the running softmax in registers.
//
// Work split: one CTA of 4 warps per (64 query rows, query head); a warp owns 16
// query rows. Key/value tiles of 64 cache rows travel through a two-stage cp.async
// ring in shared memory (rows padded by 16 bytes, so the 8x8 matrix loads below hit 32
// different banks). Scores and the probability-value product run on the warp-level
// tensor-core instruction (m16n8k16, bf16 operands, FP32 accumulate); probabilities
// are rounded to bf16 before the second product, as every flash kernel does. Prefill
// attention is about 2 % of a chunk's arithmetic (the NF4 GEMMs are the rest), so the
// kernel is built for fidelity and for not needing the mask / transposes, not for the
// tensor-core roofline.

#include "nf4_common.cuh"

namespace chr {
namespace {

constexpr int kPfTile = 64;      // query rows per CTA and cache rows per tile
constexpr int kPfThreads = 128;  // 4 warps x 16 query rows
constexpr float kPfNeg = -1.0e30f;

struct PrefillAttnArgs {
  const __nv_bfloat16 *q;  // [n, n_q, hd], rows q_stride elements apart
  long long q_stride;
  const __nv_bfloat16 *k_cache;  // [max_seq, n_kv, hd]
  const __nv_bfloat16 *v_cache;
  __nv_bfloat16 *out;  // [n, n_q * hd]
  int n, start, n_q, n_kv;
  float scale_log2;  // scale * log2(e)
};

__device__ __forceinline__ uint32_t pf_smem(const void *p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}
// 16 bytes global -> shared; src_bytes = 0 writes zeros instead (rows past the prefix)
__device__ __forceinline__ void pf_cp16(uint32_t dst, const void *src, int src_bytes) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(src_bytes)
               : "memory");
}
__device__ __forceinline__ void pf_ldm_x2(uint32_t addr, uint32_t &r0, uint32_t &r1) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x2.shared.b16 {%0, %1}, [%2];" : "=r"(r0), "=r"(r1) : "r"(addr));
}
__device__ __forceinline__ void pf_ldm_x2_trans(uint32_t addr, uint32_t &r0, uint32_t &r1) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x2.trans.shared.b16 {%0, %1}, [%2];"
               : "=r"(r0), "=r"(r1)
               : "r"(addr));
}
__device__ __forceinline__ void pf_mma(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, "
      "{%8, %9}, {%0, %1, %2, %3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pf_pack(float lo, float hi) {
  const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<const uint32_t *>(&v);
}

template <int HD>
__global__ void __launch_bounds__(kPfThreads) attn_prefill_kernel(const PrefillAttnArgs a) {
  constexpr int KS = HD / 16;          // k-steps of the score product
  constexpr int NT = HD / 8;           // 8-column tiles of the output
  constexpr int PIECES = HD / 8;       // 16-byte pieces of a cache row
  constexpr int ROWB = HD * 2 + 16;    // padded row pitch in shared memory
  constexpr int STAGE = 2 * kPfTile * ROWB;  // K tile then V tile
  extern __shared__ __align__(16) unsigned char pf_smem_raw[];
  const uint32_t base = pf_smem(pf_smem_raw);

  const int tid = threadIdx.x;
  const int lane = tid & 31;
  const int warp = tid >> 5;
  const int g = lane >> 2;  // fragment row
  const int t = lane & 3;   // fragment column pair
  const int head = blockIdx.y;
  const int kvh = head / (a.n_q / a.n_kv);
  const int q0 = blockIdx.x * kPfTile;
  const int seq = a.start + a.n;
  pdl_trigger();
  pdl_wait();  // q and the chunk's cache rows come from the kernels before

  // cache rows this CTA needs: 0 .. start + (its last query row)
  const int q_last = min(q0 + kPfTile, a.n) - 1;
  const int n_tiles = (a.start + q_last) / kPfTile + 1;

  auto load_tile = [&](int kt, int stage) {
    const int kv0 = kt * kPfTile;
    for (int c = tid; c < 2 * kPfTile * PIECES; c += kPfThreads) {
      const bool is_v = c >= kPfTile * PIECES;
      const int cc = is_v ? c - kPfTile * PIECES : c;
      const int row = cc / PIECES;
      const int piece = cc - row * PIECES;
      const int key = kv0 + row;
      const bool live = key < seq;
      const size_t off = (static_cast<size_t>(live ? key : seq - 1) * a.n_kv + kvh) * HD + piece * 8;
      pf_cp16(base + stage * STAGE + (is_v ? kPfTile * ROWB : 0) + row * ROWB + piece * 16,
              (is_v ? a.v_cache : a.k_cache) + off, live ? 16 : 0);
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
  };
  load_tile(0, 0);

  // this warp's 16 query rows as A fragments (rows past the chunk repeat the last row
  // and are never stored)
  const int row0 = q0 + warp * 16 + g;
  const int row1 = row0 + 8;
  uint32_t qf[KS][4];
  {
    const __nv_bfloat16 *qp0 = a.q + static_cast<size_t>(min(row0, a.n - 1)) * a.q_stride + head * HD;
    const __nv_bfloat16 *qp1 = a.q + static_cast<size_t>(min(row1, a.n - 1)) * a.q_stride + head * HD;
#pragma unroll
    for (int ks = 0; ks < KS; ++ks) {
      qf[ks][0] = __ldg(reinterpret_cast<const uint32_t *>(qp0 + ks * 16 + 2 * t));
      qf[ks][1] = __ldg(reinterpret_cast<const uint32_t *>(qp1 + ks * 16 + 2 * t));
      qf[ks][2] = __ldg(reinterpret_cast<const uint32_t *>(qp0 + ks * 16 + 8 + 2 * t));
      qf[ks][3] = __ldg(reinterpret_cast<const uint32_t *>(qp1 + ks * 16 + 8 + 2 * t));
    }
  }
  const int qpos0 = a.start + row0;
  const int qpos1 = a.start + row1;
  const int qpos_min = a.start + q0 + warp * 16;

  float o[NT][4];
#pragma unroll
  for (int i = 0; i < NT; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
  float m0 = kPfNeg, m1 = kPfNeg, l0 = 0.f, l1 = 0.f;
  const float c = a.scale_log2;
  // ldmatrix row addresses: lanes 0-15 name the rows of the two 8x8 matrices
  const int lm_row = lane & 7;
  const int lm_mat = (lane >> 3) & 1;

  for (int kt = 0; kt < n_tiles; ++kt) {
    const int stage = kt & 1;
    if (kt + 1 < n_tiles) {
      load_tile(kt + 1, stage ^ 1);
      asm volatile("cp.async.wait_group 1;" ::: "memory");
    } else {
      asm volatile("cp.async.wait_group 0;" ::: "memory");
    }
    __syncthreads();
    const uint32_t k_base = base + stage * STAGE;
    const uint32_t v_base = k_base + kPfTile * ROWB;
    const int kv0 = kt * kPfTile;

    // scores of 16 query rows x 64 cache rows
    float s[8][4];
#pragma unroll
    for (int nt = 0; nt < 8; ++nt) {
      s[nt][0] = s[nt][1] = s[nt][2] = s[nt][3] = 0.f;
#pragma unroll
      for (int ks = 0; ks < KS; ++ks) {
        uint32_t b0, b1;
        pf_ldm_x2(k_base + (nt * 8 + lm_row) * ROWB + (ks * 16 + lm_mat * 8) * 2, b0, b1);
        pf_mma(s[nt], qf[ks], b0, b1);
      }
    }
    if (kv0 + kPfTile - 1 > qpos_min) {  // the tile reaches past this warp's first row
#pragma unroll
      for (int nt = 0; nt < 8; ++nt) {
        const int key = kv0 + nt * 8 + 2 * t;
        if (key > qpos0) s[nt][0] = kPfNeg;
        if (key + 1 > qpos0) s[nt][1] = kPfNeg;
        if (key > qpos1) s[nt][2] = kPfNeg;
        if (key + 1 > qpos1) s[nt][3] = kPfNeg;
      }
    }
    float mx0 = kPfNeg, mx1 = kPfNeg;
#pragma unroll
    for (int nt = 0; nt < 8; ++nt) {
      mx0 = fmaxf(mx0, fmaxf(s[nt][0], s[nt][1]));
      mx1 = fmaxf(mx1, fmaxf(s[nt][2], s[nt][3]));
    }
    mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1));
    mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
    mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1));
    mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
    const float m0n = fmaxf(m0, mx0), m1n = fmaxf(m1, mx1);
    const float alpha0 = exp2f((m0 - m0n) * c), alpha1 = exp2f((m1 - m1n) * c);
    m0 = m0n;
    m1 = m1n;
    const float off0 = -m0 * c, off1 = -m1 * c;
    float sum0 = 0.f, sum1 = 0.f;
#pragma unroll
    for (int nt = 0; nt < 8; ++nt) {
      // a masked score stays at kPfNeg: exp2 of about -1e30 is exactly zero
      s[nt][0] = exp2f(fmaf(s[nt][0], c, off0));
      s[nt][1] = exp2f(fmaf(s[nt][1], c, off0));
      s[nt][2] = exp2f(fmaf(s[nt][2], c, off1));
      s[nt][3] = exp2f(fmaf(s[nt][3], c, off1));
      sum0 += s[nt][0] + s[nt][1];
      sum1 += s[nt][2] + s[nt][3];
    }
    l0 = fmaf(l0, alpha0, sum0);
    l1 = fmaf(l1, alpha1, sum1);
#pragma unroll
    for (int i = 0; i < NT; ++i) {
      o[i][0] *= alpha0;
      o[i][1] *= alpha0;
      o[i][2] *= alpha1;
      o[i][3] *= alpha1;
    }
    // probabilities (bf16) x values
#pragma unroll
    for (int kk = 0; kk < 4; ++kk) {
      const uint32_t pa[4] = {pf_pack(s[2 * kk][0], s[2 * kk][1]), pf_pack(s[2 * kk][2], s[2 * kk][3]),
                              pf_pack(s[2 * kk + 1][0], s[2 * kk + 1][1]),
                              pf_pack(s[2 * kk + 1][2], s[2 * kk + 1][3])};
#pragma unroll
      for (int i = 0; i < NT; ++i) {
        uint32_t b0, b1;
        pf_ldm_x2_trans(v_base + (kk * 16 + lm_mat * 8 + lm_row) * ROWB + i * 16, b0, b1);
        pf_mma(o[i], pa, b0, b1);
      }
    }
    __syncthreads();  // the other stage is requested again at the top of the next round
  }

  l0 += __shfl_xor_sync(0xffffffffu, l0, 1);
  l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
  l1 += __shfl_xor_sync(0xffffffffu, l1, 1);
  l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
  const float inv0 = l0 > 0.f ? 1.f / l0 : 0.f;
  const float inv1 = l1 > 0.f ? 1.f / l1 : 0.f;
  const size_t out_stride = static_cast<size_t>(a.n_q) * HD;
#pragma unroll
  for (int i = 0; i < NT; ++i) {
    if (row0 < a.n) {
      *reinterpret_cast<uint32_t *>(a.out + row0 * out_stride + head * HD + i * 8 + 2 * t) =
          pf_pack(o[i][0] * inv0, o[i][1] * inv0);
    }
    if (row1 < a.n) {
      *reinterpret_cast<uint32_t *>(a.out + row1 * out_stride + head * HD + i * 8 + 2 * t) =
          pf_pack(o[i][2] * inv1, o[i][3] * inv1);
    }
  }
}

template <int HD>
int launch_prefill_attn(const PrefillAttnArgs &a, cudaStream_t st) {
  constexpr int smem = 2 * 2 * kPfTile * (HD * 2 + 16);
  static int done[64] = {};
  if (!ensure_smem_attr(attn_prefill_kernel<HD>, smem, done)) return kLaunch;
  const dim3 grid(static_cast<unsigned>((a.n + kPfTile - 1) / kPfTile), static_cast<unsigned>(a.n_q));
  const cudaError_t e = launch_chain(attn_prefill_kernel<HD>, grid, dim3(kPfThreads), smem, st, a);
  return e == cudaSuccess ? kOk : kLaunch;
}

}  // namespace
}  // namespace chr

using namespace chr;

extern "C" int chr_nf4_attn_prefill(const void *q, int64_t q_stride, const void *k_cache,
                                    const void *v_cache, void *out, int32_t n, int32_t start,
                                    int32_t n_q, int32_t n_kv, int32_t hd, int32_t max_seq,
                                    float scale, void *stream) {
  if (q == nullptr || k_cache == nullptr || v_cache == nullptr || out == nullptr) return kNull;
  if (n < 1 || start < 0 || n_q < 1 || n_kv < 1 || (n_q % n_kv) != 0 || max_seq < 1 ||
      static_cast<long long>(start) + n > max_seq || n_q > 65535) {
    return kDims;
  }
  if (hd != 16 && hd != 32 && hd != 64 && hd != 128) return kDims;
  if (q_stride < static_cast<long long>(n_q) * hd || (q_stride & 1) != 0) return kDims;
  if (!aligned(q, 4) || !aligned(out, 4) || !aligned(k_cache, 16) || !aligned(v_cache, 16)) return kAlign;
  PrefillAttnArgs a{};
  a.q = static_cast<const __nv_bfloat16 *>(q);
  a.q_stride = q_stride;
  a.k_cache = static_cast<const __nv_bfloat16 *>(k_cache);
  a.v_cache = static_cast<const __nv_bfloat16 *>(v_cache);
  a.out = static_cast<__nv_bfloat16 *>(out);
  a.n = n;
  a.start = start;
  a.n_q = n_q;
  a.n_kv = n_kv;
  a.scale_log2 = scale * 1.4426950408889634f;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  switch (hd) {
    case 16: return launch_prefill_attn<16>(a, st);
    case 32: return launch_prefill_attn<32>(a, st);
    case 64: return launch_prefill_attn<64>(a, st);
    default: return launch_prefill_attn<128>(a, st);
  }
}
