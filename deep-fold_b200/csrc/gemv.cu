// Decode-side NF4 GEMV family for sm_100a: y = dequant(W) . x on CUDA cores, one
// persistent CTA per SM striding over row tiles that an elected thread streams into
// a shared-memory ring with bulk copies. The device core (ring, inner loop, work
// split, numerics) is in gemv_ring.cuh; this file holds the kernels' C entry points.

#include "gemv_ring.cuh"

namespace chr {

// Sticky status word of the GEMV family on this device: 0, or kStGemvWindow /
// kStGemvTimeout from the kernel that met the problem. Lives in the library, read
// and cleared through chr_nf4_gemv_status().
__device__ int g_gemv_status;

namespace {

// Device address of g_gemv_status, looked up once per device (a host-side runtime
// query, no launch and no allocation). Two host threads racing on the first call
// both store the same value.
int *gemv_status_ptr() {
  static int *ptr[64] = {};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
  if (ptr[dev] == nullptr) {
    void *p = nullptr;
    if (cudaGetSymbolAddress(&p, g_gemv_status) != cudaSuccess) return nullptr;
    ptr[dev] = static_cast<int *>(p);
  }
  return ptr[dev];
}

constexpr int kV = CHR_GEMV_VARIANT;  // the lookup variant this library is built with

bool scales_aligned16(const GemvArgs &a, int n_mats) {
  for (int i = 0; i < n_mats; ++i) {
    if (!aligned(a.scale[i], 16)) return false;
  }
  return true;
}

template <int V, int MODE>
GemvShape shape_for(const GemvArgs &a, int shape_k_pad = 0) {
  const int n_mats = MODE == 0 ? 1 : (MODE == 1 ? 2 : 3);
  GemvShape sh = pick_gemv_shape<V>(a.n_rows, a.K, shape_k_pad > 0 ? shape_k_pad : a.K_pad, MODE,
                                    sm_count(), max_chunks_per_warp<V>(), scales_aligned16(a, n_mats),
                                    a.rows_end);
  return sh;
}

template <int MODE>
int launch(const GemvArgs &proto, cudaStream_t st) {
  GemvArgs a = proto;
  a.status = gemv_status_ptr();
  if (a.status == nullptr) return kLaunch;
  const GemvShape sh = shape_for<kV, MODE>(a);
  if (sh.R == 0) return kDims;  // K beyond what a CTA can stage
  return launch_gemv<kV, MODE>(a, sh, st);
}

// ---------------------------------------------------------------------------
// Row-split GEMV with the cross-GPU sum fused in (see chr_nf4_gemv_allreduce).
// ---------------------------------------------------------------------------

struct PeerArgs {
  int rank, world;
  int capacity;  // rows a source rank's slot holds
  float *recv[CHR_NF4_AR_MAX_RANKS];
  unsigned int *flags[CHR_NF4_AR_MAX_RANKS];
  unsigned int *epoch;  // [0] calls completed, [1] exit ticket
  int *status;
  unsigned int polls;
};

// Exchange protocol: every 8-byte store to a peer carries one FP32 partial and the
// call's epoch, so a row needs neither a fence nor a separate flag: the receiver polls
// the word itself until the epoch matches (one NVLink trip instead of store + system
// fence + flag + poll). Each rank's receive buffer holds, per half (calls alternate
// between two halves) and per source rank, `capacity` such words; a rank keeps its own
// partial as plain floats in its own slot of its own buffer.
template <int V, int R, int C>
__global__ void __launch_bounds__((kMaxWarps + 1) * 32, 1)
nf4_gemv_ar_kernel(const GemvArgs a, const PeerArgs pa) {
  extern __shared__ __align__(128) unsigned char smem[];
  const int tid = threadIdx.x;
  const int M = a.n_rows;
  pdl_trigger();  // the next kernel of the chain may request its tiles meanwhile

  // The epoch is read once the previous kernel of the stream has completed (and with
  // it every earlier one): nobody writes the word before every CTA of the previous
  // call has taken its exit ticket, so all CTAs (and, call for call, all ranks) agree.
  // (kept in the ring header of the dynamic allocation: the kernels of this family
  // declare no static shared memory, their layout counts on it)
  const uint32_t epoch_slot = static_cast<uint32_t>(__cvta_generic_to_shared(smem)) + 144u;
  auto slot_of = [&](int owner, unsigned int e, int source) -> uint2 * {
    return reinterpret_cast<uint2 *>(pa.recv[owner]) +
           (static_cast<size_t>(e & 1u) * pa.world + source) * pa.capacity;
  };
  GemvArgs b = a;
  // Every thread passes the same y32: this rank's own slot of the current half. It
  // depends on the epoch, which is only known after the dependency wait; gemv_run reads
  // b.y32 after wait() returns.
  gemv_run<V, R, C, 0>(b, smem, blockIdx.x, gridDim.x, [&] {
    pdl_wait();  // x and the residual belong to the previous kernel until it ends
    const unsigned int e = *reinterpret_cast<volatile unsigned int *>(pa.epoch) + 1u;
    b.y32 = reinterpret_cast<float *>(slot_of(pa.rank, e, pa.rank));
    if (tid == 0) asm volatile("st.shared.u32 [%0], %1;" ::"r"(epoch_slot), "r"(e) : "memory");
  });
  __syncthreads();  // this CTA's rows are stored (by its helper warp or its workers)
  unsigned int e;
  asm volatile("ld.shared.u32 %0, [%1];" : "=r"(e) : "r"(epoch_slot) : "memory");
  const float *mine = reinterpret_cast<const float *>(slot_of(pa.rank, e, pa.rank));
  // a wait that ran out earlier (status is sticky until the host clears it) means a
  // peer is gone: do not spend the full poll budget again on every call
  const bool give_up = *reinterpret_cast<volatile int *>(pa.status) != 0;

  // Rows of this CTA: tiles blockIdx.x, blockIdx.x + gridDim.x, ... of G*R rows. They
  // are exchanged with one thread per (row, peer), so that neither the peer stores nor
  // the polls of a row queue up behind each other (a thread per row polling its peers
  // one after the other cost about 0.6 us per peer at 8 GPUs); the peers' values meet
  // in shared memory, where a thread per row sums them in rank order.
  const int rt = a.G * R;
  const int my_tiles = blockIdx.x < a.n_tiles ? (a.n_tiles - 1 - blockIdx.x) / gridDim.x + 1 : 0;
  const int n_rows_cta = my_tiles * rt;
  const int others = pa.world - 1;
  constexpr int kArChunk = 1024;  // rows per pass through the gather buffer
  float *gather = reinterpret_cast<float *>(smem + kHeadBytes);  // [rows][others]; the ring is idle now
  auto row_of = [&](int i) { return (blockIdx.x + (i / rt) * gridDim.x) * rt + i % rt; };
  __nv_bfloat16 *y = a.y[0];
  for (int c0 = 0; c0 < n_rows_cta; c0 += kArChunk) {
    const int cn = min(kArChunk, n_rows_cta - c0);
    // 1. push (value, epoch) into every peer's slot for this rank
    for (int idx = tid; idx < cn * others; idx += blockDim.x) {
      const int i = idx / others;
      const int j = idx - i * others;
      const int p = j < pa.rank ? j : j + 1;
      const int row = row_of(c0 + i);
      if (row < M) {
        const float own = __ldcg(mine + row);
        asm volatile("st.relaxed.sys.global.v2.u32 [%0], {%1, %2};" ::"l"(slot_of(p, e, pa.rank) + row),
                     "r"(__float_as_uint(own)), "r"(e)
                     : "memory");
      }
    }
    // 2. collect the peers' words (bounded polls; a word that never comes counts as 0)
    for (int idx = tid; idx < cn * others; idx += blockDim.x) {
      const int i = idx / others;
      const int j = idx - i * others;
      const int p = j < pa.rank ? j : j + 1;
      const int row = row_of(c0 + i);
      float got = 0.f;
      if (row < M) {
        const uint2 *src = slot_of(pa.rank, e, p) + row;
        uint32_t bits = 0u, seen = 0u;
        unsigned int polls = 0;
        for (;;) {
          asm volatile("ld.relaxed.sys.global.v2.u32 {%0, %1}, [%2];" : "=r"(bits), "=r"(seen) : "l"(src)
                       : "memory");
          if (seen == e || give_up) break;
          if (++polls >= pa.polls) {
            atomicExch(pa.status, 1);
            break;
          }
        }
        got = seen == e ? __uint_as_float(bits) : 0.f;
      }
      gather[idx] = got;
    }
    __syncthreads();
    // 3. rank-ordered sum, residual, one rounding
    for (int i = tid; i < cn; i += blockDim.x) {
      const int row = row_of(c0 + i);
      if (row >= M) continue;
      float v = 0.f;
      for (int r = 0; r < pa.world; ++r) {
        v += r == pa.rank ? __ldcg(mine + row) : gather[i * others + (r < pa.rank ? r : r - 1)];
      }
      v += __bfloat162float(y[row]);
      y[row] = __float2bfloat16(v);
    }
    __syncthreads();
  }
  // 4. the last CTA out publishes the new epoch
  __syncthreads();
  if (tid == 0) {
    if (atomicAdd(pa.epoch + 1, 1u) == gridDim.x - 1) {
      pa.epoch[1] = 0u;
      __threadfence();
      *reinterpret_cast<volatile unsigned int *>(pa.epoch) = e;
    }
  }
}

template <int V>
int launch_ar(const GemvArgs &proto, const GemvShape &sh, const PeerArgs &pa, cudaStream_t st) {
  GemvArgs a = proto;
  a.S = sh.S;
  a.G = sh.G;
  a.n_tiles = sh.n_tiles;
  a.n_slots = sh.n_slots;
  a.scale_bulk = sh.scale_bulk;
  a.tail_scale_bulk = sh.tail_scale_bulk;
  const dim3 grid(static_cast<unsigned>(sh.grid));
  const dim3 block(static_cast<unsigned>((sh.S * sh.G + 1) * 32));
  const int smem_limit = static_cast<int>(kWindowEnd - kReserved);
#define CHR_LAUNCH_AR(RR, CC)                                                                  \
  do {                                                                                         \
    static int attr_done[64] = {};                                                             \
    if (!ensure_smem_attr(nf4_gemv_ar_kernel<V, RR, CC>, smem_limit, attr_done)) return kLaunch; \
    if (launch_chain(nf4_gemv_ar_kernel<V, RR, CC>, grid, block, sh.smem_bytes, st, a, pa) !=   \
        cudaSuccess) {                                                                         \
      return kLaunch;                                                                          \
    }                                                                                          \
    return kOk;                                                                                \
  } while (0)
  switch (sh.C * 8 + sh.R) {
    case 1 * 8 + 1: CHR_LAUNCH_AR(1, 1);
    case 1 * 8 + 2: CHR_LAUNCH_AR(2, 1);
    case 1 * 8 + 4: CHR_LAUNCH_AR(4, 1);
    case 1 * 8 + 8: CHR_LAUNCH_AR(8, 1);
    case 2 * 8 + 1: CHR_LAUNCH_AR(1, 2);
    case 2 * 8 + 2: CHR_LAUNCH_AR(2, 2);
    case 2 * 8 + 4: CHR_LAUNCH_AR(4, 2);
    default: break;
  }
#undef CHR_LAUNCH_AR
  return kDims;
}

GemvArgs one_matrix(const chr_nf4_dev_t *w, const void *x, const void *add, const void *rms_w,
                    float rms_eps) {
  GemvArgs a{};
  a.packed[0] = w->packed;
  a.scale[0] = w->scale;
  a.extra[0] = static_cast<const __nv_bfloat16 *>(add);
  a.rows_end[0] = a.rows_end[1] = a.rows_end[2] = w->M;
  a.n_rows = w->M;
  a.K = w->K;
  a.K_pad = w->K_pad;
  a.x = static_cast<const __nv_bfloat16 *>(x);
  a.rms_w = static_cast<const __nv_bfloat16 *>(rms_w);
  a.rms_eps = rms_eps;
  return a;
}

}  // namespace
}  // namespace chr

#include "gemv_n.cuh"  // N-column GEMV: same translation unit, it shares the status word

using namespace chr;

extern "C" int chr_nf4_gemv(const chr_nf4_dev_t *w, const void *x, void *y, void *stream,
                            const void *add, const void *rms_w, float rms_eps) {
  if (w == nullptr || x == nullptr || y == nullptr) return kNull;
  const int rc = check_matrix(w);
  if (rc != kOk) return rc;
  if (!aligned(w->packed, 16) || !aligned(x, 16) || !aligned(w->scale, 2)) return kAlign;
  GemvArgs a = one_matrix(w, x, add, rms_w, rms_eps);
  a.y[0] = static_cast<__nv_bfloat16 *>(y);
  return launch<0>(a, static_cast<cudaStream_t>(stream));
}

extern "C" int chr_nf4_gemv_f32(const chr_nf4_dev_t *w, const void *x, float *y, void *stream,
                                const void *add, const void *rms_w, float rms_eps) {
  if (w == nullptr || x == nullptr || y == nullptr) return kNull;
  const int rc = check_matrix(w);
  if (rc != kOk) return rc;
  if (!aligned(w->packed, 16) || !aligned(x, 16) || !aligned(w->scale, 2)) return kAlign;
  GemvArgs a = one_matrix(w, x, add, rms_w, rms_eps);
  a.y32 = y;
  return launch<0>(a, static_cast<cudaStream_t>(stream));
}

extern "C" int chr_nf4_gemv_shape(int32_t n_rows, int32_t K_pad, int32_t swiglu, int32_t out[6]) {
  if (out == nullptr) return kNull;
  if (n_rows < 1 || K_pad < kGroup || (K_pad % kGroup) != 0) return kDims;
  GemvArgs a{};
  a.n_rows = n_rows;
  a.K = K_pad;
  a.K_pad = K_pad;
  a.rows_end[0] = a.rows_end[1] = a.rows_end[2] = n_rows;
  // alignment of the scale blobs does not change R, C, S, G: report the aligned case
  const GemvShape sh = pick_gemv_shape<kV>(n_rows, K_pad, K_pad, swiglu != 0 ? 1 : 0, sm_count(),
                                          max_chunks_per_warp<kV>(), true, a.rows_end);
  if (sh.R == 0) return kDims;
  out[0] = sh.R;
  out[1] = sh.C;
  out[2] = sh.S;
  out[3] = sh.G;
  out[4] = sh.n_tiles;
  out[5] = sh.grid;
  return kOk;
}

extern "C" int chr_nf4_gemv_status(void) {
  int v = 0;
  if (cudaDeviceSynchronize() != cudaSuccess) return kLaunch;
  if (cudaMemcpyFromSymbol(&v, g_gemv_status, sizeof(int)) != cudaSuccess) return kLaunch;
  if (v != 0) {
    const int zero = 0;
    cudaMemcpyToSymbol(g_gemv_status, &zero, sizeof(int));
  }
  return v;
}

extern "C" int chr_nf4_gemv_allreduce(const chr_nf4_dev_t *w, const void *x, void *y,
                                      const chr_nf4_peers_t *peers, const void *add,
                                      void *stream) {
  if (w == nullptr || x == nullptr || y == nullptr || peers == nullptr) return kNull;
  const int rc = check_matrix(w);
  if (rc != kOk) return rc;
  if (!aligned(w->packed, 16) || !aligned(x, 16) || !aligned(w->scale, 2)) return kAlign;
  if (peers->world < 2 || peers->world > CHR_NF4_AR_MAX_RANKS || peers->rank < 0 ||
      peers->rank >= peers->world) {
    return kDims;
  }
  if (peers->epoch == nullptr || peers->status == nullptr) return kNull;
  // The receive buffers hold `capacity` rows per source rank and half; more rows would
  // run the peer stores into the flag words behind them.
  if (peers->capacity < 1) return kDims;
  if (w->M > peers->capacity) return kWorkspace;
  PeerArgs pa{};
  pa.rank = peers->rank;
  pa.world = peers->world;
  pa.capacity = peers->capacity;
  pa.polls = peer_polls();
  for (int p = 0; p < peers->world; ++p) {
    if (peers->recv[p] == nullptr || peers->flags[p] == nullptr) return kNull;
    pa.recv[p] = static_cast<float *>(peers->recv[p]);
    pa.flags[p] = static_cast<unsigned int *>(peers->flags[p]);
  }
  pa.epoch = static_cast<unsigned int *>(peers->epoch);
  pa.status = static_cast<int *>(peers->status);

  GemvArgs a = one_matrix(w, x, add, nullptr, 0.f);
  a.y[0] = static_cast<__nv_bfloat16 *>(y);
  a.status = gemv_status_ptr();
  if (a.status == nullptr) return kLaunch;
  // Every rank must tile the rows the same way; with uneven K shares the ranks agree
  // on the shape of the longest share.
  int shape_k_pad = a.K_pad;
  if (peers->shape_k_pad > 0) {
    if (peers->shape_k_pad < a.K_pad || (peers->shape_k_pad % kGroup) != 0) return kDims;
    shape_k_pad = peers->shape_k_pad;
  }
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const GemvShape sh = shape_for<kV, 0>(a, shape_k_pad);
  if (sh.R == 0 || sh.grid > CHR_NF4_AR_MAX_CTAS) return kDims;
  return launch_ar<kV>(a, sh, pa, st);
}

extern "C" int chr_nf4_gemv_qkv(const chr_nf4_dev_t *q, const chr_nf4_dev_t *k,
                                const chr_nf4_dev_t *v, const void *x, void *yq, void *yk,
                                void *yv, const void *bq, const void *bk, const void *bv,
                                void *stream, const void *rms_w, float rms_eps) {
  if (q == nullptr || k == nullptr || v == nullptr || x == nullptr || yq == nullptr ||
      yk == nullptr || yv == nullptr) {
    return kNull;
  }
  if (q->M < 1 || k->M < 1 || v->M < 1 || q->K < 1) return kDims;
  if (k->K != q->K || v->K != q->K || k->K_pad != q->K_pad || v->K_pad != q->K_pad) return kDims;
  if (q->packed == nullptr || k->packed == nullptr || v->packed == nullptr ||
      q->scale == nullptr || k->scale == nullptr || v->scale == nullptr) {
    return kDims;
  }
  if (!k_pad_ok(q->K, q->K_pad)) return kKPad;
  if (!aligned(q->packed, 16) || !aligned(k->packed, 16) || !aligned(v->packed, 16) ||
      !aligned(x, 16)) {
    return kAlign;
  }
  GemvArgs a{};
  const chr_nf4_dev_t *m[3] = {q, k, v};
  void *ys[3] = {yq, yk, yv};
  const void *bs[3] = {bq, bk, bv};
  int end = 0;
  for (int i = 0; i < 3; ++i) {
    a.packed[i] = m[i]->packed;
    a.scale[i] = m[i]->scale;
    a.y[i] = static_cast<__nv_bfloat16 *>(ys[i]);
    a.extra[i] = static_cast<const __nv_bfloat16 *>(bs[i]);
    end += m[i]->M;
    a.rows_end[i] = end;
  }
  a.n_rows = end;
  a.K = q->K;
  a.K_pad = q->K_pad;
  a.x = static_cast<const __nv_bfloat16 *>(x);
  a.rms_w = static_cast<const __nv_bfloat16 *>(rms_w);
  a.rms_eps = rms_eps;
  return launch<2>(a, static_cast<cudaStream_t>(stream));
}

extern "C" int chr_nf4_gemv_swiglu(const chr_nf4_dev_t *gate, const chr_nf4_dev_t *up,
                                   const void *x, void *y, void *stream, const void *rms_w,
                                   float rms_eps) {
  if (gate == nullptr || up == nullptr || x == nullptr || y == nullptr) return kNull;
  if (gate->M < 1 || gate->K < 1 || up->M != gate->M || up->K != gate->K ||
      up->K_pad != gate->K_pad) {
    return kDims;
  }
  if (gate->packed == nullptr || up->packed == nullptr || gate->scale == nullptr ||
      up->scale == nullptr) {
    return kDims;
  }
  if (!k_pad_ok(gate->K, gate->K_pad)) return kKPad;
  if (!aligned(gate->packed, 16) || !aligned(up->packed, 16) || !aligned(x, 16)) return kAlign;
  GemvArgs a{};
  a.packed[0] = gate->packed;
  a.scale[0] = gate->scale;
  a.packed[1] = up->packed;
  a.scale[1] = up->scale;
  a.y[0] = static_cast<__nv_bfloat16 *>(y);
  a.rows_end[0] = a.rows_end[1] = a.rows_end[2] = gate->M;
  a.n_rows = gate->M;
  a.K = gate->K;
  a.K_pad = gate->K_pad;
  a.x = static_cast<const __nv_bfloat16 *>(x);
  a.rms_w = static_cast<const __nv_bfloat16 *>(rms_w);
  a.rms_eps = rms_eps;
  return launch<1>(a, static_cast<cudaStream_t>(stream));
}
