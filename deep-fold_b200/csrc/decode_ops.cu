// Small decode-step kernels for sm_100a: RMSNorm, RoPE + KV write, GQA decode
// attention over the valid KV prefix, packed-embedding row decode and the
// greedy pick + commit.
//
// Attention differs from the reference's launch shape on purpose: one CTA owns a
// (kv head, sequence split) pair and serves every query head of that kv head, so
// a cache row is read once per group instead of once per query head.

#include "attn_mma.cuh"

namespace chr {
namespace {

// ----------------------------------------------------------------------------
// RMSNorm  (reference: gpu/nf4/nf4_gemv.cu:729-751)
// ----------------------------------------------------------------------------
constexpr int kRmsThreads = 256;

__global__ void __launch_bounds__(kRmsThreads) rms_kernel(const __nv_bfloat16 *__restrict__ x,
                                                         const __nv_bfloat16 *__restrict__ w,
                                                         __nv_bfloat16 *__restrict__ y, int n,
                                                         float eps) {
  const int tid = threadIdx.x;
  pdl_trigger();
  pdl_wait();
  // same warp-level sum as the GEMV kernels' fused RMSNorm: identical scale bits
  const float s = rsqrtf(warp_sumsq_bf16(x, n, tid & 31) / static_cast<float>(n) + eps);
  for (int i = tid; i < n; i += kRmsThreads) {
    y[i] = __float2bfloat16(__bfloat162float(w[i]) * __bfloat162float(x[i]) * s);
  }
}

// ----------------------------------------------------------------------------
// Standalone RoPE + cache write  (reference: gpu/nf4/nf4_gemv.cu:497-537)
// ----------------------------------------------------------------------------
__global__ void rope_kv_kernel(__nv_bfloat16 *__restrict__ q, __nv_bfloat16 *__restrict__ k,
                               const __nv_bfloat16 *__restrict__ v,
                               __nv_bfloat16 *__restrict__ k_cache,
                               __nv_bfloat16 *__restrict__ v_cache,
                               const __nv_bfloat16 *__restrict__ cos,
                               const __nv_bfloat16 *__restrict__ sin,
                               const int64_t *__restrict__ position, int n_q, int n_kv, int hd,
                               int max_seq) {
  pdl_trigger();
  pdl_wait();
  const long long pos = *position;
  if (pos < 0 || pos >= max_seq) return;
  const int head = blockIdx.x;
  const bool is_q = head < n_q;
  __nv_bfloat16 *vec = is_q ? q + static_cast<size_t>(head) * hd
                            : k + static_cast<size_t>(head - n_q) * hd;
  const __nv_bfloat16 *c = cos + static_cast<size_t>(pos) * hd;
  const __nv_bfloat16 *s = sin + static_cast<size_t>(pos) * hd;
  const int half = hd >> 1;
  for (int d = threadIdx.x; d < half; d += blockDim.x) {
    const float lo = __bfloat162float(vec[d]);
    const float hi = __bfloat162float(vec[d + half]);
    vec[d] = __float2bfloat16(lo * __bfloat162float(c[d]) + (-hi) * __bfloat162float(s[d]));
    vec[d + half] =
        __float2bfloat16(hi * __bfloat162float(c[d + half]) + lo * __bfloat162float(s[d + half]));
  }
  if (!is_q) {
    __syncthreads();
    const size_t off = (static_cast<size_t>(pos) * n_kv + (head - n_q)) * hd;
    for (int d = threadIdx.x; d < hd; d += blockDim.x) {
      k_cache[off + d] = vec[d];
      v_cache[off + d] = v[static_cast<size_t>(head - n_q) * hd + d];
    }
  }
}

// ----------------------------------------------------------------------------
// GQA decode attention  (reference: gpu/nf4/nf4_gemv.cu:558-727)
// ----------------------------------------------------------------------------
// Arrival counters for the merge-by-last-CTA step: one per (kv head, head chunk).
// Zero at load, and the last CTA of a group puts its counter back to zero, so a
// launch leaves them as it found them. Launches of the attention kernel that
// overlap on the device (different streams) would share them and must not.
__device__ unsigned int g_attn_arrivals[kMaxAttnGroups];

// The item's shared memory is dynamic (above 48 KB for head dims over 64): the limit
// of each kernel is raised once per device, before its first launch.
template <int P, int H, typename Kernel>
static bool attn_smem_ready(Kernel kernel) {
  static int done[64] = {};
  return ensure_smem_attr(kernel, static_cast<int>(sizeof(AttnSmem<P, H>)), done);
}

// Query heads one item serves: the group size when a kernel is built for it, else
// the next size up (the spare heads carry zero queries); groups above 8 heads (4 for
// head dims over 128) are cut into chunks.
static int attn_heads_per_item(int n_rep, int hd) {
  const int cap = hd <= 128 ? 8 : 4;
  if (n_rep >= cap) return cap;
  if (n_rep <= 2) return n_rep;
  if (n_rep <= 4) return 4;
  return n_rep == 5 ? 5 : 8;
}
static int attn_head_chunks(int n_rep, int hd) {
  const int heads = attn_heads_per_item(n_rep, hd);
  return (n_rep + heads - 1) / heads;
}
// Splits of the sequence actually used: the caller's count, at most kAttnMaxSplit,
// halved while the grid (splits x groups, one 512-thread CTA per SM) would not fit
// the device in one wave. A second wave costs more than longer rows per warp save.
static int attn_splits_used(int n_split, long long groups) {
  int s = n_split > kAttnMaxSplit ? kAttnMaxSplit : n_split;
  const long long sms = sm_count();
  while (s > 1 && s * groups > sms) s = (s + 1) / 2;
  return s;
}
#define CHR_ATTN_SHAPES(X)                                                                     \
  X(1, 1) X(1, 2) X(1, 4) X(1, 5) X(1, 8) X(2, 1) X(2, 2) X(2, 4) X(2, 5) X(2, 8) X(4, 1)      \
  X(4, 2) X(4, 4)

// Grid: (splits, kv heads, head chunks); the core is in attn_core.cuh.
template <int P, int H>
__global__ void __launch_bounds__(kAttnThreads, 1) attn_split_kernel(const AttnArgs a) {
  extern __shared__ __align__(16) unsigned char attn_smem[];
  AttnSmem<P, H> &sm = *reinterpret_cast<AttnSmem<P, H> *>(attn_smem);
  pdl_trigger();
  pdl_wait();  // q, k_act, v_act, position and valid_len come from earlier kernels
  unsigned int *ctr = &g_attn_arrivals[(blockIdx.y * gridDim.z + blockIdx.z) % kMaxAttnGroups];
  attn_item<P, H>(a, sm, blockIdx.x, blockIdx.y, blockIdx.z, ctr, threadIdx.x,
                  [] { __syncthreads(); });
}

// The same items for B sequences in one launch: grid.y = B * n_kv; every sequence has
// its own q, current k/v, cache, output, split partials, valid length and position
// (consecutive blocks of the per-sequence sizes).
template <int P, int H>
__global__ void __launch_bounds__(kAttnThreads, 1) attn_batch_kernel(const AttnArgs proto,
                                                                 const AttnBatch bt) {
  extern __shared__ __align__(16) unsigned char attn_smem[];
  AttnSmem<P, H> &sm = *reinterpret_cast<AttnSmem<P, H> *>(attn_smem);
  pdl_trigger();
  pdl_wait();
  const int b = blockIdx.y / proto.n_kv;
  const int kvh = blockIdx.y - b * proto.n_kv;
  AttnArgs a = proto;
  a.q += b * bt.q_stride;
  if (a.k_act != nullptr) a.k_act += b * bt.kv_act_stride;
  if (a.v_act != nullptr) a.v_act += b * bt.kv_act_stride;
  a.k_cache += b * bt.cache_stride;
  a.v_cache += b * bt.cache_stride;
  a.out += b * bt.out_stride;
  a.m_s += b * bt.ws_stride;
  a.l_s += b * bt.ws_stride;
  a.o_s += b * bt.ws_stride;
  a.valid_len += b;
  if (a.position != nullptr) a.position += b;
  unsigned int *ctr = &g_attn_arrivals[(blockIdx.y * gridDim.z + blockIdx.z) % kMaxAttnGroups];
  attn_item<P, H>(a, sm, blockIdx.x, kvh, blockIdx.z, ctr, threadIdx.x, [] { __syncthreads(); });
}

// Tensor-core form (attn_mma.cuh) for head dims 16 / 32 / 64 / 128, one sequence or B.
// Grid: (splits, B * kv heads, head chunks of 8).
template <int HD>
__global__ void __launch_bounds__(kMmaThreads, 1) attn_mma_kernel(const AttnArgs proto,
                                                                const AttnBatch bt) {
  extern __shared__ __align__(16) unsigned char attn_smem[];
  pdl_trigger();
  pdl_wait();  // q, k_act, v_act, position and valid_len come from earlier kernels
  const int b = blockIdx.y / proto.n_kv;
  const int kvh = blockIdx.y - b * proto.n_kv;
  AttnArgs a = proto;
  a.q += b * bt.q_stride;
  if (a.k_act != nullptr) a.k_act += b * bt.kv_act_stride;
  if (a.v_act != nullptr) a.v_act += b * bt.kv_act_stride;
  a.k_cache += b * bt.cache_stride;
  a.v_cache += b * bt.cache_stride;
  a.out += b * bt.out_stride;
  a.m_s += b * bt.ws_stride;
  a.l_s += b * bt.ws_stride;
  a.o_s += b * bt.ws_stride;
  a.valid_len += b;
  if (a.position != nullptr) a.position += b;
  unsigned int *ctr = &g_attn_arrivals[(blockIdx.y * gridDim.z + blockIdx.z) % kMaxAttnGroups];
  attn_mma_item<HD>(a, attn_smem, blockIdx.x, kvh, blockIdx.z, ctr);
}

// CHR_NF4_ATTN=simt keeps every head dim on the CUDA-core form (A/B runs).
static bool attn_mma_wanted(int hd) {
  static int simt = -1;
  if (simt < 0) {
    const char *env = std::getenv("CHR_NF4_ATTN");
    simt = (env != nullptr && env[0] == 's') ? 1 : 0;
  }
  return simt == 0 && (hd == 16 || hd == 32 || hd == 64 || hd == 128);
}

template <int HD>
static cudaError_t launch_attn_mma_hd(const AttnArgs &a, const AttnBatch &bt, dim3 grid, cudaStream_t st) {
  static int done[64] = {};
  if (!ensure_smem_attr(attn_mma_kernel<HD>, AttnMmaLayout<HD>::kBytes, done)) return cudaErrorInvalidValue;
  return launch_chain(attn_mma_kernel<HD>, grid, dim3(kMmaThreads), AttnMmaLayout<HD>::kBytes, st, a, bt);
}

// `a.n_split` is the caller's count on entry; the count used is written back into it
// (and the workspace pointers follow it).
static int launch_attn_mma(AttnArgs a, AttnBatch bt, float *ws, int n_split, cudaStream_t st) {
  const int n_rep = a.n_q / a.n_kv;
  const int chunks = (n_rep + kMmaHeads - 1) / kMmaHeads;
  const long long groups = static_cast<long long>(bt.batch) * a.n_kv * chunks;
  if (groups > kMaxAttnGroups) return kDims;
  n_split = attn_splits_used(n_split, groups);
  const int slots = a.n_q * n_split;
  a.n_split = n_split;
  a.m_s = ws;
  a.l_s = ws + slots;
  a.o_s = ws + 2 * slots;
  bt.ws_stride = static_cast<long long>(slots) * (a.hd + 2);
  const dim3 grid(static_cast<unsigned>(n_split), static_cast<unsigned>(bt.batch * a.n_kv),
                  static_cast<unsigned>(chunks));
  cudaError_t e;
  switch (a.hd) {
    case 16: e = launch_attn_mma_hd<16>(a, bt, grid, st); break;
    case 32: e = launch_attn_mma_hd<32>(a, bt, grid, st); break;
    case 64: e = launch_attn_mma_hd<64>(a, bt, grid, st); break;
    default: e = launch_attn_mma_hd<128>(a, bt, grid, st); break;
  }
  return e == cudaSuccess ? kOk : kLaunch;
}

// ----------------------------------------------------------------------------
// Packed embedding rows  (reference: gpu/host/embedding.py:74-107)
// ----------------------------------------------------------------------------
__global__ void embed_rows_kernel(const uint8_t *__restrict__ packed,
                                  const uint16_t *__restrict__ scale,
                                  const int64_t *__restrict__ ids, __nv_bfloat16 *__restrict__ out,
                                  int32_t *status, const int64_t *position, int32_t *valid_len,
                                  int M, int K, int K_pad) {
  pdl_trigger();
  pdl_wait();
  const int r = blockIdx.y;
  if (r == 0 && blockIdx.x == 0 && threadIdx.x == 0 && position != nullptr &&
      valid_len != nullptr) {
    *valid_len = static_cast<int32_t>(*position + 1);
  }
  const long long id = ids[r];
  const bool bad = id < 0 || id >= M;
  if (bad && blockIdx.x == 0 && threadIdx.x == 0 && status != nullptr) *status = 1;
  // one thread per 8 codes (4 packed bytes -> 16 bytes of bf16)
  const int c8 = blockIdx.x * blockDim.x + threadIdx.x;
  const int k = c8 * 8;
  if (k >= K) return;
  __nv_bfloat16 vals[8];
  if (bad) {
#pragma unroll
    for (int e = 0; e < 8; ++e) vals[e] = __float2bfloat16(0.f);
  } else {
    const uint32_t pk = *reinterpret_cast<const uint32_t *>(
        packed + static_cast<size_t>(id) * (K_pad >> 1) + (k >> 1));
    const float s =
        half_bits_to_float(scale[static_cast<size_t>(id) * (K_pad / kGroup) + (k >> 6)]);
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      const uint32_t code = (pk >> (4 * e)) & 0xFu;
      vals[e] = __float2bfloat16(__uint_as_float(kLutBits[code]) * s);
    }
  }
  __nv_bfloat16 *dst = out + static_cast<size_t>(r) * K + k;
  if (k + 8 <= K && (K & 7) == 0) {
    *reinterpret_cast<uint4 *>(dst) = *reinterpret_cast<const uint4 *>(vals);
  } else {
    for (int e = 0; e < 8 && k + e < K; ++e) dst[e] = vals[e];
  }
}

// ----------------------------------------------------------------------------
// Greedy pick + commit  (reference: gpu/decodev2/step.py:182, state.py:98-103)
// ----------------------------------------------------------------------------
constexpr int kPickThreads = 256;

__device__ __forceinline__ void pick_commit_body(const __nv_bfloat16 *__restrict__ logits, int n,
                                                 int64_t *next_token, int64_t *token,
                                                 int64_t *position, uint8_t *finished, int64_t eos,
                                                 unsigned long long *best, unsigned int *ticket) {
  __shared__ unsigned long long red[kPickThreads / 32];
  __shared__ bool last;
  unsigned long long key = 0ull;
  const int stride = gridDim.x * kPickThreads;
  for (int i = blockIdx.x * kPickThreads + threadIdx.x; i < n; i += stride) {
    const unsigned long long cand = pick_key(__bfloat16_as_ushort(logits[i]), i);
    key = cand > key ? cand : key;
  }
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) {
    const unsigned long long o = __shfl_xor_sync(0xffffffffu, key, off);
    key = o > key ? o : key;
  }
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = key;
  __syncthreads();
  if (threadIdx.x == 0) {
#pragma unroll
    for (int i = 1; i < kPickThreads / 32; ++i) key = red[i] > key ? red[i] : key;
    atomicMax(best, key);
    __threadfence();
    last = atomicAdd(ticket, 1u) == gridDim.x - 1;
    if (last) {
      __threadfence();
      const unsigned long long win = atomicMax(best, 0ull);
      const int64_t idx = static_cast<int64_t>(0xFFFFFFFFu - static_cast<uint32_t>(win));
      *next_token = idx;
      if (token != nullptr) *token = idx;
      if (position != nullptr) *position += 1;
      if (finished != nullptr && idx == eos) *finished |= 1;
      *best = 0ull;
      *ticket = 0u;
    }
  }
}

__global__ void __launch_bounds__(kPickThreads)
pick_commit_kernel(const __nv_bfloat16 *__restrict__ logits, int n, int64_t *next_token,
                   int64_t *token, int64_t *position, uint8_t *finished, int64_t eos,
                   unsigned long long *best, unsigned int *ticket) {
  pdl_trigger();
  pdl_wait();
  pick_commit_body(logits, n, next_token, token, position, finished, eos, best, ticket);
}

// One pick per sequence in one launch: blockIdx.y is the sequence; its logits row,
// registers and 16 bytes of scratch are the b-th of each array.
__global__ void __launch_bounds__(kPickThreads)
pick_commit_batch_kernel(const __nv_bfloat16 *__restrict__ logits, long long row_stride, int n,
                         int64_t *next_token, int64_t *token, int64_t *position, uint8_t *finished,
                         int64_t eos, unsigned long long *scratch) {
  pdl_trigger();
  pdl_wait();
  const int b = blockIdx.y;
  unsigned long long *best = scratch + 2 * b;
  pick_commit_body(logits + b * row_stride, n, next_token + b, token != nullptr ? token + b : nullptr,
                   position != nullptr ? position + b : nullptr,
                   finished != nullptr ? finished + b : nullptr, eos, best,
                   reinterpret_cast<unsigned int *>(best + 1));
}

// The same pick when the logits are split over the ranks of a tensor-parallel group
// (each rank holds a slice of the vocabulary): every rank finds its local best, the
// last CTA pushes that one (key, index) pair into every peer's receive slots with plain
// peer stores, raises a flag on each peer, waits (bounded) for the peers' flags, and
// commits the best of all ranks. Two scalars per rank cross NVLink instead of the
// logits. Epoch and status words as in the fused GEMV exchange.
struct PickPeers {
  int rank, world;
  unsigned long long *keys[CHR_NF4_AR_MAX_RANKS];  // rank p's slots: [2 halves][world]
  unsigned int *flags[CHR_NF4_AR_MAX_RANKS];       // rank p's flags: [world * CHR_NF4_AR_MAX_CTAS]
  unsigned int *epoch;
  int *status;
  unsigned int polls;
};

__global__ void __launch_bounds__(kPickThreads)
pick_commit_tp_kernel(const __nv_bfloat16 *__restrict__ logits, int n, int index_offset,
                      const PickPeers pp, int64_t *next_token, int64_t *token, int64_t *position,
                      uint8_t *finished, int64_t eos, unsigned long long *best,
                      unsigned int *ticket) {
  __shared__ unsigned long long red[kPickThreads / 32];
  pdl_trigger();
  pdl_wait();
  unsigned long long key = 0ull;
  const int stride = gridDim.x * kPickThreads;
  for (int i = blockIdx.x * kPickThreads + threadIdx.x; i < n; i += stride) {
    const unsigned long long cand = pick_key(__bfloat16_as_ushort(logits[i]), i + index_offset);
    key = cand > key ? cand : key;
  }
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) {
    const unsigned long long o = __shfl_xor_sync(0xffffffffu, key, off);
    key = o > key ? o : key;
  }
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = key;
  __syncthreads();
  if (threadIdx.x != 0) return;
#pragma unroll
  for (int i = 1; i < kPickThreads / 32; ++i) key = red[i] > key ? red[i] : key;
  atomicMax(best, key);
  __threadfence();
  if (atomicAdd(ticket, 1u) != gridDim.x - 1) return;
  __threadfence();
  unsigned long long win = atomicMax(best, 0ull);
  *best = 0ull;
  *ticket = 0u;
  // exchange
  const unsigned int e = *reinterpret_cast<volatile unsigned int *>(pp.epoch) + 1u;
  const unsigned int half = (e & 1u) * static_cast<unsigned int>(pp.world);
  for (int p = 0; p < pp.world; ++p) {
    asm volatile("st.relaxed.sys.global.u64 [%0], %1;" ::"l"(pp.keys[p] + half + pp.rank), "l"(win)
                 : "memory");
  }
  __threadfence_system();
  for (int p = 0; p < pp.world; ++p) {
    if (p != pp.rank) {
      asm volatile("st.relaxed.sys.global.u32 [%0], %1;" ::"l"(pp.flags[p] + pp.rank * CHR_NF4_AR_MAX_CTAS),
                   "r"(e)
                   : "memory");
    }
  }
  const bool give_up = *reinterpret_cast<volatile int *>(pp.status) != 0;
  for (int r = 0; r < pp.world && !give_up; ++r) {
    if (r == pp.rank) continue;
    const unsigned int *f = pp.flags[pp.rank] + r * CHR_NF4_AR_MAX_CTAS;
    unsigned int seen = 0, polls = 0;
    for (;;) {
      asm volatile("ld.relaxed.sys.global.u32 %0, [%1];" : "=r"(seen) : "l"(f) : "memory");
      if (static_cast<int>(seen - e) >= 0) break;
      if (++polls >= pp.polls) {
        atomicExch(pp.status, 1);
        break;
      }
    }
  }
  __threadfence_system();
  for (int r = 0; r < pp.world; ++r) {
    unsigned long long other;
    asm volatile("ld.relaxed.sys.global.u64 %0, [%1];" : "=l"(other) : "l"(pp.keys[pp.rank] + half + r)
                 : "memory");
    win = other > win ? other : win;
  }
  const int64_t idx = static_cast<int64_t>(0xFFFFFFFFu - static_cast<uint32_t>(win));
  *next_token = idx;
  if (token != nullptr) *token = idx;
  if (position != nullptr) *position += 1;
  if (finished != nullptr && idx == eos) *finished |= 1;
  __threadfence();
  *reinterpret_cast<volatile unsigned int *>(pp.epoch) = e;
}

}  // namespace
}  // namespace chr

using namespace chr;

extern "C" int chr_nf4_rms(const void *x, const void *w, void *y, int32_t n, float eps,
                           void *stream) {
  if (x == nullptr || w == nullptr || y == nullptr) return kNull;
  if (n < 1) return kDims;
  const cudaError_t e = launch_chain(
      rms_kernel, dim3(1), dim3(kRmsThreads), 0, static_cast<cudaStream_t>(stream),
      static_cast<const __nv_bfloat16 *>(x), static_cast<const __nv_bfloat16 *>(w),
      static_cast<__nv_bfloat16 *>(y), n, eps);
  return e == cudaSuccess ? kOk : kLaunch;
}

extern "C" int chr_nf4_rope_kv(void *q, void *k, const void *v, void *k_cache, void *v_cache,
                               const void *cos, const void *sin, const void *position,
                               int32_t n_q, int32_t n_kv, int32_t hd, int32_t max_seq,
                               void *stream) {
  if (q == nullptr || k == nullptr || v == nullptr || k_cache == nullptr || v_cache == nullptr ||
      cos == nullptr || sin == nullptr || position == nullptr) {
    return kNull;
  }
  if (n_q < 1 || n_kv < 1 || hd < 2 || (hd & 1) != 0 || max_seq < 1) return kDims;
  const cudaError_t e = launch_chain(
      rope_kv_kernel, dim3(static_cast<unsigned>(n_q + n_kv)), dim3(64), 0,
      static_cast<cudaStream_t>(stream), static_cast<__nv_bfloat16 *>(q),
      static_cast<__nv_bfloat16 *>(k), static_cast<const __nv_bfloat16 *>(v),
      static_cast<__nv_bfloat16 *>(k_cache), static_cast<__nv_bfloat16 *>(v_cache),
      static_cast<const __nv_bfloat16 *>(cos), static_cast<const __nv_bfloat16 *>(sin),
      static_cast<const int64_t *>(position), n_q, n_kv, hd, max_seq);
  return e == cudaSuccess ? kOk : kLaunch;
}

extern "C" int chr_nf4_attn(const void *q, const void *k, const void *v, void *out,
                            const void *valid_len, float *ws, int32_t n_q, int32_t n_kv,
                            int32_t hd, int32_t n_split, float scale, void *stream,
                            const void *k_act, const void *v_act, const void *cos,
                            const void *sin, const void *position, int32_t max_seq) {
  if (q == nullptr || k == nullptr || v == nullptr || out == nullptr || valid_len == nullptr ||
      ws == nullptr) {
    return kNull;
  }
  if (n_q < 1 || n_kv < 1 || hd < 2 || hd > 256 || (hd & 1) != 0 || (n_q % n_kv) != 0 ||
      n_split < 1 || n_split > 64 || max_seq < 1) {
    return kDims;
  }
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  // The workspace is sized for the caller's n_split; fewer splits may be used.
  const int n_rep = n_q / n_kv;
  const int n_split_asked = n_split;
  n_split = attn_splits_used(n_split, n_kv * attn_head_chunks(n_rep, hd));
  const int slots = n_q * n_split;
  AttnArgs a{};
  a.q = static_cast<const __nv_bfloat16 *>(q);
  a.q_group_stride = n_rep * hd;
  a.k_act = static_cast<const __nv_bfloat16 *>(k_act);
  a.v_act = static_cast<const __nv_bfloat16 *>(v_act);
  a.kv_act_stride = hd;
  a.k_cache = static_cast<const __nv_bfloat16 *>(k);
  a.v_cache = static_cast<const __nv_bfloat16 *>(v);
  a.out = static_cast<__nv_bfloat16 *>(out);
  a.m_s = ws;
  a.l_s = ws + slots;
  a.o_s = ws + 2 * slots;
  a.valid_len = static_cast<const int32_t *>(valid_len);
  a.cos = static_cast<const __nv_bfloat16 *>(cos);
  a.sin = static_cast<const __nv_bfloat16 *>(sin);
  a.position = static_cast<const int64_t *>(position);
  a.n_q = n_q;
  a.n_kv = n_kv;
  a.hd = hd;
  a.n_split = n_split;
  a.max_seq = max_seq;
  a.scale = scale;

  if (attn_mma_wanted(hd) && aligned(k, 16) && aligned(v, 16)) {
    AttnBatch one{};
    one.batch = 1;
    return launch_attn_mma(a, one, ws, n_split_asked, st);
  }
  const int heads = attn_heads_per_item(n_rep, hd);
  const int head_chunks = (n_rep + heads - 1) / heads;
  if (n_kv * head_chunks > kMaxAttnGroups) return kDims;
  const dim3 grid(static_cast<unsigned>(n_split), static_cast<unsigned>(n_kv),
                  static_cast<unsigned>(head_chunks));
  cudaError_t e = cudaErrorInvalidValue;
#define CHR_ATTN(PP, HH)                                                                       \
  if (pieces == PP && heads == HH) {                                                           \
    if (attn_smem_ready<PP, HH>(attn_split_kernel<PP, HH>)) {                                  \
      e = launch_chain(attn_split_kernel<PP, HH>, grid, dim3(kAttnThreads),                    \
                       sizeof(AttnSmem<PP, HH>), st, a);                                       \
    }                                                                                          \
  }
  const int pieces = hd <= 64 ? 1 : (hd <= 128 ? 2 : 4);
  CHR_ATTN_SHAPES(CHR_ATTN)
#undef CHR_ATTN
  return e == cudaSuccess ? kOk : kLaunch;
}

extern "C" int chr_nf4_attn_batch(const void *q, const void *k, const void *v, void *out,
                                  const void *valid_len, float *ws, int32_t batch, int32_t n_q,
                                  int32_t n_kv, int32_t hd, int32_t n_split, float scale,
                                  void *stream, const void *k_act, const void *v_act,
                                  const void *cos, const void *sin, const void *position,
                                  int32_t max_seq) {
  if (q == nullptr || k == nullptr || v == nullptr || out == nullptr || valid_len == nullptr ||
      ws == nullptr) {
    return kNull;
  }
  if (batch < 1 || n_q < 1 || n_kv < 1 || hd < 2 || hd > 256 || (hd & 1) != 0 ||
      (n_q % n_kv) != 0 || n_split < 1 || n_split > 64 || max_seq < 1) {
    return kDims;
  }
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int n_rep = n_q / n_kv;
  const int n_split_asked = n_split;
  n_split = attn_splits_used(n_split, batch * n_kv * attn_head_chunks(n_rep, hd));
  const int slots = n_q * n_split;
  AttnArgs a{};
  a.q = static_cast<const __nv_bfloat16 *>(q);
  a.q_group_stride = n_rep * hd;
  a.k_act = static_cast<const __nv_bfloat16 *>(k_act);
  a.v_act = static_cast<const __nv_bfloat16 *>(v_act);
  a.kv_act_stride = hd;
  a.k_cache = static_cast<const __nv_bfloat16 *>(k);
  a.v_cache = static_cast<const __nv_bfloat16 *>(v);
  a.out = static_cast<__nv_bfloat16 *>(out);
  a.m_s = ws;
  a.l_s = ws + slots;
  a.o_s = ws + 2 * slots;
  a.valid_len = static_cast<const int32_t *>(valid_len);
  a.cos = static_cast<const __nv_bfloat16 *>(cos);
  a.sin = static_cast<const __nv_bfloat16 *>(sin);
  a.position = static_cast<const int64_t *>(position);
  a.n_q = n_q;
  a.n_kv = n_kv;
  a.hd = hd;
  a.n_split = n_split;
  a.max_seq = max_seq;
  a.scale = scale;
  AttnBatch bt{};
  bt.batch = batch;
  bt.q_stride = static_cast<long long>(n_q) * hd;
  bt.kv_act_stride = static_cast<long long>(n_kv) * hd;
  bt.cache_stride = static_cast<long long>(max_seq) * n_kv * hd;
  bt.out_stride = static_cast<long long>(n_q) * hd;
  bt.ws_stride = static_cast<long long>(slots) * (hd + 2);
  if (attn_mma_wanted(hd) && aligned(k, 16) && aligned(v, 16) &&
      (bt.cache_stride * 2) % 16 == 0) {
    return launch_attn_mma(a, bt, ws, n_split_asked, st);
  }
  const int heads = attn_heads_per_item(n_rep, hd);
  const int chunks = (n_rep + heads - 1) / heads;
  if (static_cast<long long>(batch) * n_kv * chunks > kMaxAttnGroups) return kDims;
  const dim3 grid(static_cast<unsigned>(n_split), static_cast<unsigned>(batch * n_kv),
                  static_cast<unsigned>(chunks));
  cudaError_t e = cudaErrorInvalidValue;
#define CHR_ATTN_B(PP, HH)                                                                     \
  if (pieces == PP && heads == HH) {                                                           \
    if (attn_smem_ready<PP, HH>(attn_batch_kernel<PP, HH>)) {                                  \
      e = launch_chain(attn_batch_kernel<PP, HH>, grid, dim3(kAttnThreads),                    \
                       sizeof(AttnSmem<PP, HH>), st, a, bt);                                   \
    }                                                                                          \
  }
  const int pieces = hd <= 64 ? 1 : (hd <= 128 ? 2 : 4);
  CHR_ATTN_SHAPES(CHR_ATTN_B)
#undef CHR_ATTN_B
  return e == cudaSuccess ? kOk : kLaunch;
}

extern "C" int chr_nf4_embed_rows(const chr_nf4_dev_t *w, const void *ids, int32_t n, void *out,
                                  void *status, const void *position, void *valid_len,
                                  void *stream) {
  if (w == nullptr || ids == nullptr || out == nullptr) return kNull;
  const int rc = check_matrix(w);
  if (rc != kOk) return rc;
  if (n < 1 || n > 65535) return kRangeN;
  if (!aligned(w->packed, 16) || !aligned(out, 16)) return kAlign;
  const int c8 = (w->K + 7) / 8;
  const int threads = 128;
  const dim3 grid(static_cast<unsigned>((c8 + threads - 1) / threads), static_cast<unsigned>(n));
  const cudaError_t e = launch_chain(
      embed_rows_kernel, grid, dim3(threads), 0, static_cast<cudaStream_t>(stream), w->packed,
      w->scale, static_cast<const int64_t *>(ids), static_cast<__nv_bfloat16 *>(out),
      static_cast<int32_t *>(status), static_cast<const int64_t *>(position),
      static_cast<int32_t *>(valid_len), w->M, w->K, w->K_pad);
  return e == cudaSuccess ? kOk : kLaunch;
}

extern "C" int chr_nf4_pick_commit(const void *logits, int32_t n, void *next_token, void *token,
                                   void *position, void *finished, int64_t eos, void *scratch,
                                   void *stream) {
  if (logits == nullptr || next_token == nullptr || scratch == nullptr) return kNull;
  if (n < 1) return kDims;
  if (!aligned(scratch, 8)) return kAlign;
  int blocks = (n + kPickThreads * 8 - 1) / (kPickThreads * 8);
  const int sms = sm_count();
  blocks = blocks < 1 ? 1 : (blocks > sms ? sms : blocks);
  auto *best = static_cast<unsigned long long *>(scratch);
  auto *ticket = reinterpret_cast<unsigned int *>(best + 1);
  const cudaError_t e = launch_chain(
      pick_commit_kernel, dim3(static_cast<unsigned>(blocks)), dim3(kPickThreads), 0,
      static_cast<cudaStream_t>(stream), static_cast<const __nv_bfloat16 *>(logits), n,
      static_cast<int64_t *>(next_token), static_cast<int64_t *>(token),
      static_cast<int64_t *>(position), static_cast<uint8_t *>(finished), eos, best, ticket);
  return e == cudaSuccess ? kOk : kLaunch;
}

extern "C" int chr_nf4_pick_commit_batch(const void *logits, int64_t row_stride, int32_t n,
                                         int32_t batch, void *next_token, void *token,
                                         void *position, void *finished, int64_t eos,
                                         void *scratch, void *stream) {
  if (logits == nullptr || next_token == nullptr || scratch == nullptr) return kNull;
  if (n < 1 || batch < 1 || batch > 65535 || row_stride < n) return kDims;
  if (!aligned(scratch, 8)) return kAlign;
  // a few blocks per sequence: the launch as a whole should cover the SMs once
  int blocks = (n + kPickThreads * 8 - 1) / (kPickThreads * 8);
  const int share = (2 * sm_count() + batch - 1) / batch;
  blocks = blocks < 1 ? 1 : (blocks > share ? share : blocks);
  const cudaError_t e = launch_chain(
      pick_commit_batch_kernel, dim3(static_cast<unsigned>(blocks), static_cast<unsigned>(batch)),
      dim3(kPickThreads), 0, static_cast<cudaStream_t>(stream),
      static_cast<const __nv_bfloat16 *>(logits), static_cast<long long>(row_stride), n,
      static_cast<int64_t *>(next_token), static_cast<int64_t *>(token),
      static_cast<int64_t *>(position), static_cast<uint8_t *>(finished), eos,
      static_cast<unsigned long long *>(scratch));
  return e == cudaSuccess ? kOk : kLaunch;
}

extern "C" int chr_nf4_pick_commit_tp(const void *logits_local, int32_t n_local,
                                      int32_t index_offset, const chr_nf4_peers_t *peers,
                                      void *next_token, void *token, void *position,
                                      void *finished, int64_t eos, void *scratch, void *stream) {
  if (logits_local == nullptr || next_token == nullptr || scratch == nullptr || peers == nullptr) {
    return kNull;
  }
  if (n_local < 1 || index_offset < 0) return kDims;
  if (!aligned(scratch, 8)) return kAlign;
  if (peers->world < 2 || peers->world > CHR_NF4_AR_MAX_RANKS || peers->rank < 0 ||
      peers->rank >= peers->world) {
    return kDims;
  }
  if (peers->epoch == nullptr || peers->status == nullptr) return kNull;
  // the receive buffer holds 2 * world * capacity floats; the keys need 2 * world * 2
  if (peers->capacity < 2) return kWorkspace;
  PickPeers pp{};
  pp.rank = peers->rank;
  pp.world = peers->world;
  pp.polls = peer_polls();
  for (int p = 0; p < peers->world; ++p) {
    if (peers->recv[p] == nullptr || peers->flags[p] == nullptr) return kNull;
    if (!aligned(peers->recv[p], 8)) return kAlign;
    pp.keys[p] = static_cast<unsigned long long *>(peers->recv[p]);
    pp.flags[p] = static_cast<unsigned int *>(peers->flags[p]);
  }
  pp.epoch = static_cast<unsigned int *>(peers->epoch);
  pp.status = static_cast<int *>(peers->status);
  int blocks = (n_local + kPickThreads * 8 - 1) / (kPickThreads * 8);
  const int sms = sm_count();
  blocks = blocks < 1 ? 1 : (blocks > sms ? sms : blocks);
  auto *best = static_cast<unsigned long long *>(scratch);
  auto *ticket = reinterpret_cast<unsigned int *>(best + 1);
  const cudaError_t e = launch_chain(
      pick_commit_tp_kernel, dim3(static_cast<unsigned>(blocks)), dim3(kPickThreads), 0,
      static_cast<cudaStream_t>(stream), static_cast<const __nv_bfloat16 *>(logits_local), n_local,
      index_offset, pp, static_cast<int64_t *>(next_token), static_cast<int64_t *>(token),
      static_cast<int64_t *>(position), static_cast<uint8_t *>(finished), eos, best, ticket);
  return e == cudaSuccess ? kOk : kLaunch;
}

// ----------------------------------------------------------------------------
// Attention for callers that cannot allocate device memory
// ----------------------------------------------------------------------------
// Some hosts of this library have no allocator to ask for the split workspace:
// a binding layer that only forwards pointers it was handed, a plugin loaded
// into a process whose memory pool is owned by someone else and closed to it, or
// code running where cudaMalloc is forbidden (inside a stream capture, or under
// a "no allocation after start-up" rule). For them the split partials live in
// the fixed array below instead of a caller buffer. Every GPU that loads the
// library carries these bytes until the process exits, so the size is kept modest.
constexpr int kStaticAttnFloats = 262144;  // 1 MiB
static __device__ __align__(256) float g_attn_static_ws[kStaticAttnFloats];

namespace {
constexpr int kMaxDevices = 64;
float *g_static_ws_ptr[kMaxDevices] = {};

// The array's name is only a stand-in on the host; the kernel needs the address
// the current device gives it. Looked up once per device, with that device current
// (the caller's `stream` must belong to the current device: the address handed to
// the kernel is the current device's copy of the array). The cache below is written
// without a lock: two host threads that race on a device's first call both store
// the same address.
int static_ws_for_current_device(float **out) {
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return chr::kLaunch;
  if (g_static_ws_ptr[dev] == nullptr) {
    void *p = nullptr;
    if (cudaGetSymbolAddress(&p, g_attn_static_ws) != cudaSuccess || p == nullptr) {
      return chr::kLaunch;
    }
    g_static_ws_ptr[dev] = static_cast<float *>(p);
  }
  *out = g_static_ws_ptr[dev];
  return chr::kOk;
}
}  // namespace

extern "C" int chr_nf4_attn_noalloc(const void *q, const void *k, const void *v, void *out,
                                    const void *valid_len, int32_t n_q, int32_t n_kv, int32_t hd,
                                    int32_t n_split, float scale, void *stream, const void *k_act,
                                    const void *v_act, const void *cos, const void *sin,
                                    const void *position, int32_t max_seq) {
  if (n_q < 1 || hd < 2 || n_split < 1 || n_split > 64) return chr::kDims;
  const long long used_splits = n_split > chr::kAttnMaxSplit ? chr::kAttnMaxSplit : n_split;
  if (static_cast<long long>(n_q) * used_splits * (hd + 2) > kStaticAttnFloats) {
    return chr::kWorkspace;  // beyond the built-in scratch: use chr_nf4_attn with a caller buffer
  }
  float *ws = nullptr;
  const int rc = static_ws_for_current_device(&ws);
  if (rc != chr::kOk) return rc;
  return chr_nf4_attn(q, k, v, out, valid_len, ws, n_q, n_kv, hd, n_split, scale, stream, k_act,
                      v_act, cos, sin, position, max_seq);
}
