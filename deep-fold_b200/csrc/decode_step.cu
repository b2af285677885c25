// One greedy decode step as a single persistent cooperative kernel (sm_100a).
//
// One CTA per SM walks the step's operations in order; a grid-wide
// barrier (one arrival counter in global memory) separates an operation from its
// consumers. What a launch-per-operation chain pays per kernel - launch latency,
// the 64 KiB lookup table rebuilt by every CTA, the first weight loads issued
// only after the previous kernel has drained - is paid once per step or hidden:
// the table is built once, and a CTA puts the first weight tile of the next
// operation in flight before it waits at the barrier.
//
// The GEMV and attention device code is the code the per-operation kernels run
// (gemv_core.cuh, attn_core.cuh) with the same work split, so results are
// bit-identical to the chain.
//
// Waiting: only thread 0 of a CTA polls, with an acquire load, at most
// kBarrierPolls times. When a wait runs out the CTA records the operation's index
// in the status word; every later wait of every CTA returns at once, so the
// kernel always ends. The launch is cooperative, which makes the driver refuse
// it (instead of letting it wait) when the CTAs cannot all be resident.

#include <cstddef>

#include "attn_core.cuh"

namespace chr {
namespace {

#ifndef CHR_STEP_WARPS
#define CHR_STEP_WARPS 8
#endif
// 8 warps leave each thread 255 registers. The GEMV bodies were written for 128
// with their arguments as immediate constant-bank operands; here the arguments of
// most operations are indexed by layer and have to sit in registers, and with 12
// or 16 warps per CTA the bodies spilled inside the tile loop (measured: lm_head
// 115 us at 16 warps, 91 us at 12, 66 us at 8, on the 3B shapes).
constexpr int kStepWarps = CHR_STEP_WARPS;
constexpr int kStepThreads = kStepWarps * 32;
static_assert(kStepWarps <= kMaxWarps && kStepThreads >= kAttnThreads, "step CTA");
constexpr int kStepHeadBytes = kPartBytes;  // wait flag + slice partials
constexpr int kStepAttnBytes = 40960;       // attention scratch; the GEMVs' staged x shares it
constexpr unsigned int kBarrierPolls = 1u << 21;

static_assert(sizeof(AttnSmem<4, 4>) <= kStepAttnBytes, "attention scratch");
static_assert(sizeof(AttnSmem<2, 8>) <= kStepAttnBytes, "attention scratch");
static_assert(64 + 2 * kMaxWarps * 8 * sizeof(float) <= kStepHeadBytes, "head region");

// Shared memory of the step kernel for a model whose longest GEMV input is max_k.
int step_smem_bytes(int max_k) {
  const int xs = ((max_k + 7) / 8) * 16;
  return table_smem_request(xs > kStepAttnBytes ? xs : kStepAttnBytes);
}

// Layout of the caller's sync block (32-bit words).
constexpr int kSyncBar = 0;      // arrivals of the running launch
constexpr int kSyncStatus = 2;   // sticky: index of the operation whose wait gave up
constexpr int kSyncTicket = 3;   // pick: CTAs that have contributed their maximum
constexpr int kSyncBest = 4;     // pick: 64-bit running maximum (words 4, 5)
constexpr int kSyncBadId = 6;    // sticky: 1 after a token id outside the embedding table
constexpr int kSyncAttn = 16;    // attention arrival counters, kMaxAttnGroups words
// 64-bit nanosecond stamps of the last launch, written by CTA 0: [0] kernel start,
// [n] the moment the wait before operation n completed (n < kSyncStamps).
constexpr int kSyncStampWord = kSyncAttn + kMaxAttnGroups;
constexpr int kSyncStamps = (CHR_NF4_STEP_SYNC_BYTES - kSyncStampWord * 4) / 8;
static_assert(kSyncStampWord % 2 == 0 && kSyncStamps >= 256, "sync block");

__device__ __forceinline__ unsigned long long global_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}

// The arguments of every GEMV of the step (four per layer and the lm_head) and the
// layers' cache pointers live in constant memory: the GEMV bodies then take weight
// pointers and sizes as constant operands, as the per-operation kernels do from
// their parameter block, instead of holding them in registers or re-reading them
// from memory that a result store might alias. The table is per device and holds
// one model at a time; it is re-uploaded when a call describes a different one,
// and a launch whose table has been replaced since (a replayed graph of another
// model) notices the epoch mismatch and gives up with status 2000.
constexpr int kMaxStepLayers = 80;
constexpr int kOpsPerLayer = 4;  // q/k/v, o, gate+up, down
constexpr int kMaxOps = kOpsPerLayer * kMaxStepLayers + 1;

struct KvPtrs {
  __nv_bfloat16 *k, *v;
};

struct StepTable {
  unsigned long long epoch;
  GemvArgs ops[kMaxOps];
  KvPtrs kv[kMaxStepLayers];
};
static_assert(sizeof(StepTable) <= 60000, "constant bank");

__constant__ StepTable c_tab;

struct StepParams {
  chr_nf4_step_t s;
  GemvShape qkv, o, gu, down, head;
  unsigned long long epoch;
};

struct GridBarrier {
  unsigned int *bar;
  int *status;
  int *flag;            // shared: 1 while no wait has given up
  unsigned long long *stamps;
  unsigned int epoch;   // barriers this CTA has arrived at

  // Everything this CTA wrote before arrive() is visible to a CTA after its wait().
  __device__ __forceinline__ void arrive() {
    __syncthreads();
    ++epoch;
    if (threadIdx.x == 0) {
      __threadfence();
      atomicAdd(bar, 1u);
    }
  }

  __device__ __forceinline__ void wait(int op) {
    if (threadIdx.x == 0) {
      const unsigned int target = epoch * gridDim.x;
      bool ok = *reinterpret_cast<volatile int *>(status) == 0;
      if (ok) {
        unsigned int seen = 0, polls = 0;
        for (;;) {
          asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(seen) : "l"(bar) : "memory");
          if (seen >= target) break;
          if (++polls >= kBarrierPolls ||
              ((polls & 255u) == 0u && *reinterpret_cast<volatile int *>(status) != 0)) {
            ok = false;
            break;
          }
        }
        if (!ok) atomicCAS(status, 0, op);
      }
      if (blockIdx.x == 0 && op < kSyncStamps) stamps[op] = global_ns();
      __threadfence();
      *flag = ok ? 1 : 0;
    }
    __syncthreads();
  }
};

__device__ __forceinline__ void named_sync_attn() {
  asm volatile("bar.sync 1, %0;" ::"n"(kAttnThreads) : "memory");
}

#ifndef CHR_STEP_INLINE
#define CHR_STEP_INLINE 0
#endif
#if CHR_STEP_INLINE
#define CHR_STEP_BODY __forceinline__
#else
// Each instantiated body is a function of its own, so that its register
// allocation is not squeezed by the others.
#define CHR_STEP_BODY __noinline__
#endif

// FIXED >= 0: the operation's table slot is known at compile time, so its fields
// are immediate constant-bank operands (no registers hold them).
template <int R, int C, int MODE, int FIXED>
__device__ CHR_STEP_BODY void gemv_call(int slot, float *part, __nv_bfloat16 *xs,
                                        uint32_t tab_lane, GridBarrier *gb, int op) {
  const GemvArgs &a = FIXED >= 0 ? c_tab.ops[FIXED] : c_tab.ops[slot];
  gemv_run<R, C, MODE>(a, part, xs, tab_lane, blockIdx.x, gridDim.x, [&] { gb->wait(op); });
}

template <int MODE, int FIXED = -1>
__device__ __forceinline__ void gemv_phase(int slot, const GemvShape &sh, float *part,
                                           __nv_bfloat16 *xs, uint32_t tab_lane, GridBarrier &gb,
                                           int op) {
  if (sh.C == 2) {
    if constexpr (MODE != 1) {
      if (sh.R == 2) {
        gemv_call<2, 2, MODE, FIXED>(slot, part, xs, tab_lane, &gb, op);
        return;
      }
    }
    gemv_call<1, 2, MODE, FIXED>(slot, part, xs, tab_lane, &gb, op);
  } else {
    gemv_call<1, 1, MODE, FIXED>(slot, part, xs, tab_lane, &gb, op);
  }
}

// Embedding row of *token into x (zero row and status 1 for an id outside the table),
// valid_len = position + 1. One CTA.
__device__ __forceinline__ void embed_phase(const chr_nf4_step_t &s, unsigned int *bad_id) {
  const int tid = threadIdx.x;
  const long long id = __ldcg(reinterpret_cast<const long long *>(s.token));
  const int M = s.embed.packed != nullptr ? s.embed.M : s.vocab;
  const bool bad = id < 0 || id >= M;
  if (tid == 0) {
    const long long pos = __ldcg(reinterpret_cast<const long long *>(s.position));
    *reinterpret_cast<int32_t *>(s.valid_len) = static_cast<int32_t>(pos + 1);
    if (bad) *bad_id = 1u;
  }
  __nv_bfloat16 *x = static_cast<__nv_bfloat16 *>(s.x);
  const int K = s.hidden;
  for (int k = tid * 8; k < K; k += kStepThreads * 8) {
    uint4 out = make_uint4(0u, 0u, 0u, 0u);
    if (!bad) {
      if (s.embed.packed != nullptr) {
        const int K_pad = s.embed.K_pad;
        const uint32_t pk = __ldg(reinterpret_cast<const uint32_t *>(
            s.embed.packed + static_cast<size_t>(id) * (K_pad >> 1) + (k >> 1)));
        const float sc = half_bits_to_float(
            __ldg(s.embed.scale + static_cast<size_t>(id) * (K_pad / kGroup) + (k >> 6)));
        __nv_bfloat16 vals[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          vals[e] = __float2bfloat16(__uint_as_float(kLutBits[(pk >> (4 * e)) & 0xFu]) * sc);
        }
        out = *reinterpret_cast<const uint4 *>(vals);
      } else {
        out = __ldg(reinterpret_cast<const uint4 *>(
            static_cast<const __nv_bfloat16 *>(s.embed_dense) + static_cast<size_t>(id) * K + k));
      }
    }
    *reinterpret_cast<uint4 *>(x + k) = out;
  }
}

template <int P, int H>
__device__ CHR_STEP_BODY void attn_phase(const AttnArgs &a, void *scratch, unsigned int *ctrs) {
  const int tid = threadIdx.x;
  if (tid >= kAttnThreads) return;
  auto &sm = *reinterpret_cast<AttnSmem<P, H> *>(scratch);
  const int n_rep = a.n_q / a.n_kv;
  const int nz = (n_rep + H - 1) / H;
  const int items = a.n_split * a.n_kv * nz;
  for (int it = blockIdx.x; it < items; it += gridDim.x) {
    const int split = it % a.n_split;
    const int kvh = (it / a.n_split) % a.n_kv;
    const int z = it / (a.n_split * a.n_kv);
    named_sync_attn();  // the scratch of the previous item is free
    attn_item<P, H>(a, sm, split, kvh, z, ctrs + (kvh * nz + z) % kMaxAttnGroups, tid,
                    [] { named_sync_attn(); });
  }
}

// Maximum of this CTA's slice of the logits; the CTA that takes the last ticket commits.
__device__ __forceinline__ void pick_phase(const chr_nf4_step_t &s, unsigned int *sync_words,
                                           unsigned long long *red) {
  const int tid = threadIdx.x;
  const __nv_bfloat16 *logits = static_cast<const __nv_bfloat16 *>(s.logits);
  unsigned long long key = 0ull;
  for (int i = blockIdx.x * kStepThreads + tid; i < s.vocab; i += gridDim.x * kStepThreads) {
    const unsigned short bits = __ldcg(reinterpret_cast<const unsigned short *>(logits + i));
    const unsigned long long cand = pick_key(bits, i);
    key = cand > key ? cand : key;
  }
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) {
    const unsigned long long o = __shfl_xor_sync(0xffffffffu, key, off);
    key = o > key ? o : key;
  }
  if ((tid & 31) == 0) red[tid >> 5] = key;
  __syncthreads();
  if (tid == 0) {
    for (int i = 1; i < kStepThreads / 32; ++i) key = red[i] > key ? red[i] : key;
    auto *best = reinterpret_cast<unsigned long long *>(sync_words + kSyncBest);
    atomicMax(best, key);
    __threadfence();
    if (atomicAdd(sync_words + kSyncTicket, 1u) == gridDim.x - 1) {
      __threadfence();
      const unsigned long long win = atomicMax(best, 0ull);
      const int64_t idx = static_cast<int64_t>(0xFFFFFFFFu - static_cast<uint32_t>(win));
      *static_cast<int64_t *>(s.next_token) = idx;
      *static_cast<int64_t *>(s.position) += 1;
      if (s.commit) {
        *static_cast<int64_t *>(s.token) = idx;
        if (s.finished != nullptr && idx == s.eos) *static_cast<uint8_t *>(s.finished) |= 1;
      }
      // every CTA is past its last barrier: leave the block as the next launch expects it
      *best = 0ull;
      sync_words[kSyncTicket] = 0u;
      sync_words[kSyncBar] = 0u;
    }
  }
}

__global__ void __launch_bounds__(kStepThreads, 1) decode_step_kernel(const StepParams p) {
  extern __shared__ __align__(16) unsigned char smem[];
  const chr_nf4_step_t &s = p.s;
  const int tid = threadIdx.x;
  unsigned int *sync_words = static_cast<unsigned int *>(s.sync);
  if (c_tab.epoch != p.epoch) {  // the table describes another model by now: touch nothing
    if (blockIdx.x == 0 && tid == 0) {
      atomicCAS(reinterpret_cast<int *>(sync_words + kSyncStatus), 0, 2000);
    }
    return;
  }

  int *flag = reinterpret_cast<int *>(smem);
  float *part = reinterpret_cast<float *>(smem + 64);
  void *attn_scratch = smem + kStepHeadBytes;
  __nv_bfloat16 *xs = reinterpret_cast<__nv_bfloat16 *>(smem + kStepHeadBytes);
  const uint32_t tab_base = pair_table_base(smem);
  if (tab_base == 0u) {  // mis-sized launch (the entry point never produces one)
    if (blockIdx.x == 0 && tid == 0) {
      atomicCAS(reinterpret_cast<int *>(sync_words + kSyncStatus), 0, 3000);
    }
    return;
  }
  const uint32_t tab_lane = tab_base + static_cast<uint32_t>(tid & 31) * 8u;

  GridBarrier gb{sync_words + kSyncBar, reinterpret_cast<int *>(sync_words + kSyncStatus), flag,
                 reinterpret_cast<unsigned long long *>(sync_words + kSyncStampWord), 0u};
  if (blockIdx.x == 0 && tid == 0) gb.stamps[0] = global_ns();

  build_pair_table(tab_base, tid, kStepThreads);
  if (blockIdx.x == 0) embed_phase(s, sync_words + kSyncBadId);
  gb.arrive();

  const int n_rep = s.n_q / s.n_kv;
  int op = 1;
  for (int li = 0; li < s.n_layers; ++li) {
    const int slot = 1 + li * kOpsPerLayer;  // slot 0 is the lm_head

    // ---- RMSNorm + q/k/v ----
    gemv_phase<2>(slot, p.qkv, part, xs, tab_lane, gb, op++);
    gb.arrive();

    // ---- attention (RoPE, KV write, split softmax, merge) ----
    gb.wait(op++);
    {
      AttnArgs a;
      if (s.fused_qkv) {
        const __nv_bfloat16 *base = static_cast<const __nv_bfloat16 *>(s.qkv);
        a.q = base;
        a.q_group_stride = (n_rep + 2) * s.head_dim;
        a.k_act = base + n_rep * s.head_dim;
        a.v_act = base + (n_rep + 1) * s.head_dim;
        a.kv_act_stride = (n_rep + 2) * s.head_dim;
      } else {
        a.q = static_cast<const __nv_bfloat16 *>(s.q);
        a.q_group_stride = n_rep * s.head_dim;
        a.k_act = static_cast<const __nv_bfloat16 *>(s.k);
        a.v_act = static_cast<const __nv_bfloat16 *>(s.v);
        a.kv_act_stride = s.head_dim;
      }
      a.k_cache = c_tab.kv[li].k;
      a.v_cache = c_tab.kv[li].v;
      a.out = static_cast<__nv_bfloat16 *>(s.attn);
      a.n_split = s.n_split > kAttnMaxSplit ? kAttnMaxSplit : s.n_split;
      const int slots = s.n_q * a.n_split;
      a.m_s = s.attn_ws;
      a.l_s = s.attn_ws + slots;
      a.o_s = s.attn_ws + 2 * slots;
      a.valid_len = static_cast<const int32_t *>(s.valid_len);
      a.cos = static_cast<const __nv_bfloat16 *>(s.cos);
      a.sin = static_cast<const __nv_bfloat16 *>(s.sin);
      a.position = static_cast<const int64_t *>(s.position);
      a.n_q = s.n_q;
      a.n_kv = s.n_kv;
      a.hd = s.head_dim;
      a.max_seq = s.max_seq;
      a.scale = s.attn_scale;
      unsigned int *ctrs = sync_words + kSyncAttn;
      if (s.head_dim <= 64) {
        attn_phase<1, 8>(a, attn_scratch, ctrs);
      } else if (s.head_dim <= 128) {
        attn_phase<2, 8>(a, attn_scratch, ctrs);
      } else {
        attn_phase<4, 4>(a, attn_scratch, ctrs);
      }
    }
    gb.arrive();

    // ---- o-proj + residual ----
    gemv_phase<0>(slot + 1, p.o, part, xs, tab_lane, gb, op++);
    gb.arrive();

    // ---- RMSNorm + SwiGLU(gate, up) ----
    gemv_phase<1>(slot + 2, p.gu, part, xs, tab_lane, gb, op++);
    gb.arrive();

    // ---- down-proj + residual ----
    gemv_phase<0>(slot + 3, p.down, part, xs, tab_lane, gb, op++);
    gb.arrive();
  }

  // ---- final RMSNorm + lm_head ----
  gemv_phase<0, 0>(0, p.head, part, xs, tab_lane, gb, op++);
  gb.arrive();

  // ---- greedy pick + commit ----
  gb.wait(op++);
  pick_phase(s, sync_words, reinterpret_cast<unsigned long long *>(part));
}

constexpr int kMaxStepDevices = 64;
int g_step_grid[kMaxStepDevices] = {};
unsigned long long g_tab_epoch[kMaxStepDevices] = {};
uint64_t g_tab_digest[kMaxStepDevices] = {};
unsigned long long g_epoch_counter = 0;

// 64-bit digest of a table of 8-byte words (sizes here are multiples of 8).
uint64_t mix_words(const void *data, size_t bytes) {
  const uint64_t *w = static_cast<const uint64_t *>(data);
  uint64_t h = 0x9E3779B97F4A7C15ull ^ bytes;
  for (size_t i = 0; i < bytes / 8; ++i) {
    h ^= w[i] + 0x9E3779B97F4A7C15ull + (h << 6) + (h >> 2);
    h *= 0xFF51AFD7ED558CCDull;
  }
  return h;
}

GemvArgs gemv_args(const GemvShape &sh, int n_rows, int K, int K_pad, const void *x,
                   const void *rms_w, float eps) {
  GemvArgs a{};
  a.n_rows = n_rows;
  a.K = K;
  a.K_pad = K_pad;
  a.x = static_cast<const __nv_bfloat16 *>(x);
  a.rms_w = static_cast<const __nv_bfloat16 *>(rms_w);
  a.rms_eps = eps;
  a.S = sh.S;
  a.G = sh.G;
  a.n_tiles = sh.n_tiles;
  a.rows_end[0] = a.rows_end[1] = a.rows_end[2] = n_rows;
  return a;
}

// CTAs of the step kernel that fit the current device at once (one per SM when it fits).
int step_grid(int smem_bytes) {
  static int attr_bytes[kMaxStepDevices] = {};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxStepDevices) return 0;
  if (attr_bytes[dev] >= smem_bytes && g_step_grid[dev] > 0) return g_step_grid[dev];
  if (cudaFuncSetAttribute(decode_step_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                           smem_bytes) != cudaSuccess) {
    return 0;
  }
  int per_sm = 0;
  if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, decode_step_kernel, kStepThreads,
                                                    smem_bytes) != cudaSuccess ||
      per_sm < 1) {
    return 0;
  }
  attr_bytes[dev] = smem_bytes;
  g_step_grid[dev] = sm_count();
  return g_step_grid[dev];
}

bool shape_ok(const GemvShape &sh) {
  if (sh.R == 0) return false;
  return (sh.C == 2 && (sh.R == 1 || sh.R == 2)) || (sh.C == 1 && sh.R == 1);
}

// Shapes the persistent kernel instantiates: (R, C) in {(1,1), (1,2), (2,2)}.
GemvShape step_shape(int n_rows, int K_pad, bool swiglu, int ctas) {
  GemvShape sh = pick_gemv_shape(n_rows, K_pad, swiglu, ctas, kStepWarps);
  if (sh.R != 0 && !shape_ok(sh)) {  // K_pad <= 1024 with R > 1: fall back to one row per warp
    const int G = kStepWarps / sh.S;
    const int tiles = (n_rows + G - 1) / G;
    sh = GemvShape{1, sh.C, sh.S, G, tiles, tiles < ctas ? tiles : ctas};
  }
  return sh;
}

}  // namespace
}  // namespace chr

using namespace chr;

extern "C" int chr_nf4_decode_step(const chr_nf4_step_t *step, void *stream) {
  if (step == nullptr) return kNull;
  const chr_nf4_step_t &s = *step;
  if (s.layers == nullptr || s.sync == nullptr || s.token == nullptr || s.position == nullptr ||
      s.next_token == nullptr || s.valid_len == nullptr || s.x == nullptr || s.k == nullptr ||
      s.v == nullptr || s.attn == nullptr || s.down_in == nullptr || s.logits == nullptr ||
      s.attn_ws == nullptr || s.cos == nullptr || s.sin == nullptr || s.final_norm == nullptr ||
      (s.fused_qkv ? s.qkv == nullptr : s.q == nullptr) ||
      (s.embed.packed == nullptr && s.embed_dense == nullptr)) {
    return kNull;
  }
  if (s.n_layers < 1 || s.hidden < 8 || (s.hidden & 7) != 0 || s.intermediate < 1 || s.n_q < 1 ||
      s.n_kv < 1 || (s.n_q % s.n_kv) != 0 || s.head_dim < 2 || s.head_dim > 256 ||
      (s.head_dim & 1) != 0 || s.max_seq < 1 || s.vocab < 1 || s.n_split < 1 || s.n_split > 64) {
    return kDims;
  }
  const int n_rep = s.n_q / s.n_kv;
  const int heads_per_item = s.head_dim <= 128 ? 8 : 4;
  if (s.n_kv * ((n_rep + heads_per_item - 1) / heads_per_item) > kMaxAttnGroups) return kDims;
  int rc = check_matrix(&s.lm_head);
  if (rc != kOk) return rc;
  if (s.lm_head.K != s.hidden || s.lm_head.M != s.vocab) return kDims;
  if (s.embed.packed != nullptr) {
    rc = check_matrix(&s.embed);
    if (rc != kOk) return rc;
    if (s.embed.K != s.hidden) return kDims;
  }
  if (!aligned(s.x, 16) || !aligned(s.attn, 16) || !aligned(s.down_in, 16) ||
      !aligned(s.sync, 8) || !aligned(s.lm_head.packed, 16)) {
    return kAlign;
  }
  const int q_dim_all = s.n_q * s.head_dim;
  const int max_k = s.intermediate > s.hidden ? (s.intermediate > q_dim_all ? s.intermediate : q_dim_all)
                                              : (s.hidden > q_dim_all ? s.hidden : q_dim_all);
  const int smem_bytes = step_smem_bytes(max_k);
  if (smem_bytes == 0) return kDims;
  const int grid = step_grid(smem_bytes);
  if (grid < 1) return kLaunch;

  if (s.n_layers > kMaxStepLayers) return kDims;
  const int q_dim = s.n_q * s.head_dim;
  const int kv_dim = s.n_kv * s.head_dim;
  const int k_pad_h = kGroup * ((s.hidden + kGroup - 1) / kGroup);
  const int k_pad_q = kGroup * ((q_dim + kGroup - 1) / kGroup);
  const int k_pad_i = kGroup * ((s.intermediate + kGroup - 1) / kGroup);
  StepParams p{};
  p.s = s;
  p.s.layers = nullptr;  // the kernel reads the constant table, never the host array
  p.qkv = step_shape(q_dim + 2 * kv_dim, k_pad_h, false, grid);
  p.o = step_shape(s.hidden, k_pad_q, false, grid);
  p.gu = step_shape(s.intermediate, k_pad_h, true, grid);
  p.down = step_shape(s.hidden, k_pad_i, false, grid);
  p.head = step_shape(s.vocab, k_pad_h, false, grid);
  if (!shape_ok(p.qkv) || !shape_ok(p.o) || !shape_ok(p.gu) || !shape_ok(p.down) ||
      !shape_ok(p.head)) {
    return kDims;
  }

  // Assemble the operation table (static staging: the entry point is not re-entrant).
  static StepTable tab;
  const int m_q = s.fused_qkv ? q_dim + 2 * kv_dim : q_dim;
  const int m_kv = s.fused_qkv ? 0 : kv_dim;
  auto *x = static_cast<__nv_bfloat16 *>(s.x);
  for (int li = 0; li < s.n_layers; ++li) {
    const chr_nf4_step_layer_t &src = s.layers[li];
    const chr_nf4_dev_t *m[7] = {&src.q, &src.k, &src.v, &src.o, &src.gate, &src.up, &src.down};
    const int want_m[7] = {m_q, m_kv, m_kv, s.hidden, s.intermediate, s.intermediate, s.hidden};
    const int want_k[7] = {s.hidden, s.hidden, s.hidden, q_dim, s.hidden, s.hidden,
                           s.intermediate};
    for (int i = 0; i < 7; ++i) {
      if (want_m[i] == 0) continue;  // k / v of a fused wqkv
      const int rc_m = check_matrix(m[i]);
      if (rc_m != kOk) return rc_m;
      if (m[i]->M != want_m[i] || m[i]->K != want_k[i]) return kDims;
      if (!aligned(m[i]->packed, 16) || !aligned(m[i]->scale, 2)) return kAlign;
    }
    if (src.norm1 == nullptr || src.norm2 == nullptr || src.k_cache == nullptr ||
        src.v_cache == nullptr) {
      return kNull;
    }
    GemvArgs *ops = tab.ops + 1 + li * kOpsPerLayer;
    // q/k/v (a fused wqkv is the first matrix alone; the unused slots repeat it)
    ops[0] = gemv_args(p.qkv, q_dim + 2 * kv_dim, s.hidden, k_pad_h, s.x, src.norm1, s.rms_eps);
    const chr_nf4_dev_t *qkv[3] = {&src.q, s.fused_qkv ? &src.q : &src.k,
                                   s.fused_qkv ? &src.q : &src.v};
    void *ys[3] = {s.fused_qkv ? s.qkv : s.q, s.k, s.v};
    const void *bs[3] = {src.bq, src.bk, src.bv};
    for (int i = 0; i < 3; ++i) {
      ops[0].packed[i] = qkv[i]->packed;
      ops[0].scale[i] = qkv[i]->scale;
      ops[0].y[i] = static_cast<__nv_bfloat16 *>(ys[i]);
      ops[0].extra[i] = static_cast<const __nv_bfloat16 *>(bs[i]);
    }
    ops[0].rows_end[0] = m_q;
    ops[0].rows_end[1] = m_q + m_kv;
    ops[0].rows_end[2] = m_q + 2 * m_kv;
    // o-proj + residual
    ops[1] = gemv_args(p.o, s.hidden, q_dim, k_pad_q, s.attn, nullptr, s.rms_eps);
    ops[1].packed[0] = src.o.packed;
    ops[1].scale[0] = src.o.scale;
    ops[1].y[0] = x;
    ops[1].extra[0] = x;
    // SwiGLU(gate, up)
    ops[2] = gemv_args(p.gu, s.intermediate, s.hidden, k_pad_h, s.x, src.norm2, s.rms_eps);
    ops[2].packed[0] = src.gate.packed;
    ops[2].scale[0] = src.gate.scale;
    ops[2].packed[1] = src.up.packed;
    ops[2].scale[1] = src.up.scale;
    ops[2].y[0] = static_cast<__nv_bfloat16 *>(s.down_in);
    // down-proj + residual
    ops[3] = gemv_args(p.down, s.hidden, s.intermediate, k_pad_i, s.down_in, nullptr, s.rms_eps);
    ops[3].packed[0] = src.down.packed;
    ops[3].scale[0] = src.down.scale;
    ops[3].y[0] = x;
    ops[3].extra[0] = x;
    tab.kv[li].k = static_cast<__nv_bfloat16 *>(src.k_cache);
    tab.kv[li].v = static_cast<__nv_bfloat16 *>(src.v_cache);
  }
  GemvArgs &head = tab.ops[0];
  head = gemv_args(p.head, s.vocab, s.hidden, k_pad_h, s.x, s.final_norm, s.rms_eps);
  head.packed[0] = s.lm_head.packed;
  head.scale[0] = s.lm_head.scale;
  head.y[0] = static_cast<__nv_bfloat16 *>(s.logits);

  // Upload when this device's copy describes something else.
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxStepDevices) return kLaunch;
  const size_t used_ops = static_cast<size_t>(s.n_layers) * kOpsPerLayer + 1;
  const uint64_t digest = mix_words(tab.ops, used_ops * sizeof(GemvArgs)) ^
                          (mix_words(tab.kv, static_cast<size_t>(s.n_layers) * sizeof(KvPtrs)) << 1);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (g_tab_epoch[dev] == 0 || g_tab_digest[dev] != digest) {
    cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
    if (cudaStreamIsCapturing(st, &cap) != cudaSuccess) return kLaunch;
    // a captured copy would re-read the staging area at every replay: run one step
    // of this model outside the capture first
    if (cap != cudaStreamCaptureStatusNone) return kLaunch;
    tab.epoch = ++g_epoch_counter;
    const size_t bytes = offsetof(StepTable, ops) + used_ops * sizeof(GemvArgs);
    if (cudaMemcpyToSymbolAsync(c_tab, &tab, bytes, 0, cudaMemcpyHostToDevice, st) != cudaSuccess ||
        cudaMemcpyToSymbolAsync(c_tab, tab.kv, static_cast<size_t>(s.n_layers) * sizeof(KvPtrs),
                                offsetof(StepTable, kv), cudaMemcpyHostToDevice,
                                st) != cudaSuccess) {
      return kLaunch;
    }
    g_tab_epoch[dev] = tab.epoch;
    g_tab_digest[dev] = digest;
  }
  p.epoch = g_tab_epoch[dev];

  cudaLaunchConfig_t cfg{};
  cfg.gridDim = dim3(static_cast<unsigned>(grid));
  cfg.blockDim = dim3(kStepThreads);
  cfg.dynamicSmemBytes = static_cast<size_t>(smem_bytes);
  cfg.stream = static_cast<cudaStream_t>(stream);
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeCooperative;
  attr[0].val.cooperative = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  const cudaError_t e = cudaLaunchKernelEx(&cfg, decode_step_kernel, p);
  return e == cudaSuccess ? kOk : kLaunch;
}

extern "C" int chr_nf4_decode_step_status(void *sync) {
  if (sync == nullptr) return kNull;
  if (cudaDeviceSynchronize() != cudaSuccess) return kLaunch;
  int *words = static_cast<int *>(sync);
  int v[8] = {};
  if (cudaMemcpy(v, words, sizeof(v), cudaMemcpyDeviceToHost) != cudaSuccess) return kLaunch;
  if (v[kSyncStatus] != 0 && cudaMemset(words + kSyncStatus, 0, 4) != cudaSuccess) return kLaunch;
  if (v[kSyncBadId] != 0 && cudaMemset(words + kSyncBadId, 0, 4) != cudaSuccess) return kLaunch;
  return v[kSyncStatus] != 0 ? v[kSyncStatus] : (v[kSyncBadId] != 0 ? 1000 : 0);
}
