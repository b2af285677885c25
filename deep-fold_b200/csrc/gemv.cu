// Decode-side NF4 GEMV family for sm_100a: y = dequant(W) . x on CUDA cores, one
// persistent CTA per SM striding over row tiles. The device core (inner loop, work
// split, numerics) is in gemv_core.cuh; this file holds the kernels launched per
// matrix and their C entry points.

#include "gemv_core.cuh"

namespace chr {
namespace {

template <int R, int C, int MODE>
__global__ void __launch_bounds__(kMaxWarps * 32, 1)
nf4_gemv_kernel(const GemvArgs a) {
  extern __shared__ __align__(16) unsigned char smem[];
  // The next kernel of the chain may start launching; the first tile's weights go
  // in flight inside gemv_run before the table is built and x is read.
  pdl_trigger();
  const uint32_t tab_base = pair_table_base(smem);
  if (tab_base == 0u) return;  // mis-sized launch: the host entry points never produce one
  const uint32_t tab_lane = tab_base + static_cast<uint32_t>(threadIdx.x & 31) * 8u;
  gemv_run<R, C, MODE>(a, reinterpret_cast<float *>(smem),
                       reinterpret_cast<__nv_bfloat16 *>(smem + kPartBytes), tab_lane, blockIdx.x,
                       gridDim.x, [&] {
                         build_pair_table(tab_base, threadIdx.x, blockDim.x);
                         // x (and the residual / outputs) belong to the previous kernel
                         // until it completes
                         pdl_wait();
                       });
}

// ---------------------------------------------------------------------------
// Row-split GEMV with the cross-GPU sum fused in (see chr_nf4_gemv_allreduce).
// ---------------------------------------------------------------------------
constexpr unsigned int kPeerPolls = 1u << 22;

struct PeerArgs {
  int rank, world;
  float *recv[CHR_NF4_AR_MAX_RANKS];
  unsigned int *flags[CHR_NF4_AR_MAX_RANKS];
  unsigned int *epoch;  // [0] calls completed, [1] exit ticket
  int *status;
};

template <int R, int C>
__global__ void __launch_bounds__(kMaxWarps * 32, 1)
nf4_gemv_ar_kernel(const GemvArgs a, const PeerArgs pa) {
  extern __shared__ __align__(16) unsigned char smem[];
  const uint32_t tab_base = pair_table_base(smem);
  if (tab_base == 0u) return;
  const int tid = threadIdx.x;
  const uint32_t tab_lane = tab_base + static_cast<uint32_t>(tid & 31) * 8u;
  const int M = a.n_rows;
  pdl_trigger();  // the next kernel of the chain may build its table meanwhile

  // The epoch is read once the previous kernel of the stream has completed (and with
  // it every earlier one): nobody writes the word before every CTA of the previous
  // call has taken its exit ticket, so all CTAs (and, call for call, all ranks) agree.
  unsigned int e = 0;
  size_t half = 0;
  float *mine = nullptr;
  GemvArgs b = a;
  gemv_run<R, C, 0>(b, reinterpret_cast<float *>(smem),
                    reinterpret_cast<__nv_bfloat16 *>(smem + kPartBytes), tab_lane, blockIdx.x,
                    gridDim.x, [&] {
                      build_pair_table(tab_base, tid, blockDim.x);
                      pdl_wait();  // x and the residual belong to the previous kernel until it ends
                      e = *reinterpret_cast<volatile unsigned int *>(pa.epoch) + 1u;
                      half = static_cast<size_t>(e & 1u) * pa.world * M;
                      mine = pa.recv[pa.rank] + half + static_cast<size_t>(pa.rank) * M;
                      b.y32 = mine;  // the partial lands in this rank's own slot first
                    });
  __syncthreads();  // this CTA's rows are stored

  // Rows of this CTA: tiles blockIdx.x, blockIdx.x + gridDim.x, ... of G*R rows.
  const int rt = a.G * R;
  // 1. push them into every peer's slot for this rank
  for (int tile = blockIdx.x; tile < a.n_tiles; tile += gridDim.x) {
    const int row = tile * rt + tid;
    if (tid < rt && row < M) {
      const float v = __ldcg(mine + row);
      for (int p = 0; p < pa.world; ++p) {
        if (p != pa.rank) pa.recv[p][half + static_cast<size_t>(pa.rank) * M + row] = v;
      }
    }
  }
  __syncthreads();
  // 2. tell the peers' namesake CTAs, then wait for theirs
  const unsigned int slot = static_cast<unsigned int>(pa.rank) * CHR_NF4_AR_MAX_CTAS + blockIdx.x;
  if (tid == 0) {
    __threadfence_system();
    for (int p = 0; p < pa.world; ++p) {
      if (p != pa.rank) {
        // the fence above is the release; the flag itself is a relaxed store
        asm volatile("st.relaxed.sys.global.u32 [%0], %1;" ::"l"(pa.flags[p] + slot), "r"(e)
                     : "memory");
      }
    }
  }
  if (tid < pa.world && tid != pa.rank) {
    const unsigned int *f = pa.flags[pa.rank] + static_cast<unsigned int>(tid) * CHR_NF4_AR_MAX_CTAS +
                            blockIdx.x;
    unsigned int seen = 0, polls = 0;
    // a wait that ran out earlier (status is sticky until the host clears it) means a
    // peer is gone: do not spend the full poll budget again on every call
    const bool give_up = *reinterpret_cast<volatile int *>(pa.status) != 0;
    for (; !give_up;) {
      asm volatile("ld.relaxed.sys.global.u32 %0, [%1];" : "=r"(seen) : "l"(f) : "memory");
      // epochs only grow; the difference form survives the 32-bit wrap
      if (static_cast<int>(seen - e) >= 0) break;
      if (++polls >= kPeerPolls) {
        atomicExch(pa.status, 1);
        break;
      }
    }
    __threadfence_system();
  }
  __syncthreads();
  // 3. sum in rank order, add the residual, round once
  __nv_bfloat16 *y = a.y[0];
  for (int tile = blockIdx.x; tile < a.n_tiles; tile += gridDim.x) {
    const int row = tile * rt + tid;
    if (tid < rt && row < M) {
      float v = 0.f;
      for (int r = 0; r < pa.world; ++r) {
        v += __ldcg(pa.recv[pa.rank] + half + static_cast<size_t>(r) * M + row);
      }
      v += __bfloat162float(y[row]);
      y[row] = __float2bfloat16(v);
    }
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

__global__ void smem_offset_probe(int *out) {
  extern __shared__ __align__(16) unsigned char probe_smem[];
  if (threadIdx.x == 0) *out = static_cast<int>(__cvta_generic_to_shared(probe_smem));
}

template <int MODE>
int launch(const GemvArgs &proto, cudaStream_t st) {
  constexpr bool swiglu = MODE == 1;
  GemvArgs a = proto;
  const GemvShape sh = pick_gemv_shape(a.n_rows, a.K_pad, swiglu, sm_count());
  if (sh.R == 0) return kDims;  // K beyond 16 slices of 2048 is not supported by this path
  const int smem_bytes = table_smem_request(((a.K + 7) / 8) * 16);
  if (smem_bytes == 0) return kDims;  // x does not fit in front of the table
  a.S = sh.S;
  a.G = sh.G;
  a.n_tiles = sh.n_tiles;
  const dim3 grid(static_cast<unsigned>(sh.grid));
  const dim3 block(static_cast<unsigned>(sh.S * sh.G * 32));

#define CHR_LAUNCH(RR, CC)                                                                   \
  do {                                                                                       \
    static int attr_bytes = 0;                                                               \
    if (attr_bytes < smem_bytes) {                                                           \
      if (cudaFuncSetAttribute(nf4_gemv_kernel<RR, CC, MODE>,                                \
                               cudaFuncAttributeMaxDynamicSharedMemorySize,                  \
                               smem_bytes) != cudaSuccess) {                                 \
        return kLaunch;                                                                      \
      }                                                                                      \
      attr_bytes = smem_bytes;                                                               \
    }                                                                                        \
    if (launch_chain(nf4_gemv_kernel<RR, CC, MODE>, grid, block, smem_bytes, st, a) !=       \
        cudaSuccess) {                                                                       \
      return kLaunch;                                                                        \
    }                                                                                        \
  } while (0)

  if (sh.C == 2) {
    if (sh.R == 2) {
      if constexpr (MODE != 1) CHR_LAUNCH(2, 2); else return kLaunch;
    } else {
      CHR_LAUNCH(1, 2);
    }
  } else {
    if (sh.R == 4) {
      if constexpr (MODE != 1) CHR_LAUNCH(4, 1); else return kLaunch;
    } else if (sh.R == 2) {
      CHR_LAUNCH(2, 1);
    } else {
      CHR_LAUNCH(1, 1);
    }
  }
#undef CHR_LAUNCH
  return cudaGetLastError() == cudaSuccess ? kOk : kLaunch;
}

}  // namespace

int smem_window_offset() {
  static int cached[64];
  static bool have[64] = {};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return -1;
  if (have[dev]) return cached[dev];
  int *d = nullptr;
  int v = -1;
  if (cudaMalloc(&d, sizeof(int)) != cudaSuccess) return -1;
  smem_offset_probe<<<1, 32, 1024>>>(d);
  const bool ok = cudaMemcpy(&v, d, sizeof(int), cudaMemcpyDeviceToHost) == cudaSuccess;
  cudaFree(d);
  if (!ok || v < 0 || v > 16384) return -1;
  cached[dev] = v;
  have[dev] = true;
  return v;
}

}  // namespace chr

using namespace chr;

extern "C" int chr_nf4_gemv(const chr_nf4_dev_t *w, const void *x, void *y, void *stream,
                            const void *add, const void *rms_w, float rms_eps) {
  if (w == nullptr || x == nullptr || y == nullptr) return kNull;
  const int rc = check_matrix(w);
  if (rc != kOk) return rc;
  if (!aligned(w->packed, 16) || !aligned(x, 16) || !aligned(w->scale, 2)) return kAlign;
  GemvArgs a{};
  a.packed[0] = w->packed;
  a.scale[0] = w->scale;
  a.y[0] = static_cast<__nv_bfloat16 *>(y);
  a.extra[0] = static_cast<const __nv_bfloat16 *>(add);
  a.rows_end[0] = a.rows_end[1] = a.rows_end[2] = w->M;
  a.n_rows = w->M;
  a.K = w->K;
  a.K_pad = w->K_pad;
  a.x = static_cast<const __nv_bfloat16 *>(x);
  a.rms_w = static_cast<const __nv_bfloat16 *>(rms_w);
  a.rms_eps = rms_eps;
  return launch<0>(a, static_cast<cudaStream_t>(stream));
}

extern "C" int chr_nf4_gemv_f32(const chr_nf4_dev_t *w, const void *x, float *y, void *stream,
                                const void *add, const void *rms_w, float rms_eps) {
  if (w == nullptr || x == nullptr || y == nullptr) return kNull;
  const int rc = check_matrix(w);
  if (rc != kOk) return rc;
  if (!aligned(w->packed, 16) || !aligned(x, 16) || !aligned(w->scale, 2)) return kAlign;
  GemvArgs a{};
  a.packed[0] = w->packed;
  a.scale[0] = w->scale;
  a.y32 = y;
  a.extra[0] = static_cast<const __nv_bfloat16 *>(add);
  a.rows_end[0] = a.rows_end[1] = a.rows_end[2] = w->M;
  a.n_rows = w->M;
  a.K = w->K;
  a.K_pad = w->K_pad;
  a.x = static_cast<const __nv_bfloat16 *>(x);
  a.rms_w = static_cast<const __nv_bfloat16 *>(rms_w);
  a.rms_eps = rms_eps;
  return launch<0>(a, static_cast<cudaStream_t>(stream));
}

extern "C" int chr_nf4_gemv_shape(int32_t n_rows, int32_t K_pad, int32_t swiglu, int32_t out[6]) {
  if (out == nullptr) return kNull;
  if (n_rows < 1 || K_pad < kGroup || (K_pad % kGroup) != 0) return kDims;
  const GemvShape sh = pick_gemv_shape(n_rows, K_pad, swiglu != 0, sm_count());
  if (sh.R == 0) return kDims;
  out[0] = sh.R;
  out[1] = sh.C;
  out[2] = sh.S;
  out[3] = sh.G;
  out[4] = sh.n_tiles;
  out[5] = sh.grid;
  return kOk;
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
  PeerArgs pa{};
  pa.rank = peers->rank;
  pa.world = peers->world;
  for (int p = 0; p < peers->world; ++p) {
    if (peers->recv[p] == nullptr || peers->flags[p] == nullptr) return kNull;
    pa.recv[p] = static_cast<float *>(peers->recv[p]);
    pa.flags[p] = static_cast<unsigned int *>(peers->flags[p]);
  }
  pa.epoch = static_cast<unsigned int *>(peers->epoch);
  pa.status = static_cast<int *>(peers->status);

  GemvArgs a{};
  a.packed[0] = w->packed;
  a.scale[0] = w->scale;
  a.y[0] = static_cast<__nv_bfloat16 *>(y);
  a.extra[0] = static_cast<const __nv_bfloat16 *>(add);
  a.rows_end[0] = a.rows_end[1] = a.rows_end[2] = w->M;
  a.n_rows = w->M;
  a.K = w->K;
  a.K_pad = w->K_pad;
  a.x = static_cast<const __nv_bfloat16 *>(x);
  // Every rank must tile the rows the same way; with uneven K shares the ranks agree
  // on the shape of the longest share.
  int shape_k_pad = a.K_pad;
  if (peers->shape_k_pad > 0) {
    if (peers->shape_k_pad < a.K_pad || (peers->shape_k_pad % kGroup) != 0) return kDims;
    shape_k_pad = peers->shape_k_pad;
  }
  const GemvShape sh = pick_gemv_shape(a.n_rows, shape_k_pad, false, sm_count());
  if (sh.R == 0 || sh.grid > CHR_NF4_AR_MAX_CTAS) return kDims;
  a.S = sh.S;
  a.G = sh.G;
  a.n_tiles = sh.n_tiles;
  const int smem_bytes = table_smem_request(((a.K + 7) / 8) * 16);
  if (smem_bytes == 0) return kDims;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const dim3 grid(static_cast<unsigned>(sh.grid));
  const dim3 block(static_cast<unsigned>(sh.S * sh.G * 32));

#define CHR_LAUNCH_AR(RR, CC)                                                                \
  do {                                                                                       \
    static int attr_bytes = 0;                                                               \
    if (attr_bytes < smem_bytes) {                                                           \
      if (cudaFuncSetAttribute(nf4_gemv_ar_kernel<RR, CC>,                                   \
                               cudaFuncAttributeMaxDynamicSharedMemorySize,                  \
                               smem_bytes) != cudaSuccess) {                                 \
        return kLaunch;                                                                      \
      }                                                                                      \
      attr_bytes = smem_bytes;                                                               \
    }                                                                                        \
    if (launch_chain(nf4_gemv_ar_kernel<RR, CC>, grid, block, smem_bytes, st, a, pa) !=      \
        cudaSuccess) {                                                                       \
      return kLaunch;                                                                        \
    }                                                                                        \
  } while (0)

  if (sh.C == 2) {
    if (sh.R == 2) CHR_LAUNCH_AR(2, 2); else CHR_LAUNCH_AR(1, 2);
  } else {
    if (sh.R == 4) CHR_LAUNCH_AR(4, 1); else if (sh.R == 2) CHR_LAUNCH_AR(2, 1); else CHR_LAUNCH_AR(1, 1);
  }
#undef CHR_LAUNCH_AR
  return cudaGetLastError() == cudaSuccess ? kOk : kLaunch;
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
