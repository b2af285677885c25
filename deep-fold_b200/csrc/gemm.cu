// Prefill-side NF4 GEMM entry points, launch planner and the CUDA-core tile kernel.
//
// y[M,N] = bf16( sum_k bf16(LUT[code]*scale)[m,k] * x[k,n] ), FP32 accumulation,
// x bf16 [K,N] row-major, N <= 64 per call. The tensor-core kernel lives in
// gemm_tc.cu; this file owns argument checking, planning, split-K reduction and
// the SIMT kernel used as the cross-check of the tensor-core path.
//
// Numerics followed (reference: gpu/nf4/nf4_gemm.cu:168-172,319-323,665-678):
// the weight operand is rounded to bf16 once, products are exact in FP32,
// split-K partials are FP32 and are summed in split order, one bf16 rounding.

#include <cstdlib>

#include "gemm_plan.h"
#include "nf4_common.cuh"

namespace chr {

int launch_gemm_tc(const chr_nf4_dev_t &w, const __nv_bfloat16 *x, __nv_bfloat16 *y, int N,
                   float *partial, const chr_nf4_plan_t &p, cudaStream_t st);
TileShape tc_tile_shape(int N);
bool tc_supported(int M, int K_pad, int N);

namespace {

int env_int(const char *name, int fallback) {
  const char *v = std::getenv(name);
  if (v == nullptr || *v == '\0') return fallback;
  char *end = nullptr;
  const long parsed = std::strtol(v, &end, 10);
  return end == v ? fallback : static_cast<int>(parsed);
}

int ceil_div(int a, int b) { return (a + b - 1) / b; }

// ---------------------------------------------------------------------------
// SIMT tile kernel: 64 rows x up to 64 columns per CTA, one NF4 group (64 k) per
// step. 256 threads: thread (ty, tx) owns rows ty*4..ty*4+3 and columns tx+16*c.
// ---------------------------------------------------------------------------
constexpr int sBM = 64;
constexpr int sBK = 64;
constexpr int sBlock = 256;
constexpr int sBN = 64;

__global__ void __launch_bounds__(sBlock)
gemm_simt_kernel(const uint8_t *__restrict__ packed, const uint16_t *__restrict__ scale,
                 const __nv_bfloat16 *__restrict__ x, __nv_bfloat16 *__restrict__ y,
                 float *__restrict__ partial, int M, int K, int K_pad, int N, int n_ktiles,
                 int tiles_per_split) {
  __shared__ float ws[sBM][sBK + 1];
  __shared__ float xs[sBK][sBN];
  __shared__ float lut[16];
  const int tid = threadIdx.x;
  if (tid < 16) lut[tid] = __uint_as_float(kLutBits[tid]);
  const int row0 = blockIdx.x * sBM;
  const int kt0 = blockIdx.y * tiles_per_split;
  const int kt1 = min(n_ktiles, kt0 + tiles_per_split);
  const int ty = tid >> 4;
  const int tx = tid & 15;
  float acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int c = 0; c < 4; ++c) acc[i][c] = 0.f;
  const int half_stride = K_pad >> 1;
  const int n_groups = K_pad / kGroup;
  __syncthreads();

  for (int kt = kt0; kt < kt1; ++kt) {
    const int kbase = kt * sBK;
    // dequantize 64 x 64 weights: thread handles row tid/4, 16 codes (8 bytes)
    {
      const int r = tid >> 2;
      const int seg = tid & 3;
      const int grow = row0 + r;
      float vals[16];
      if (grow < M) {
        const uint2 pk = *reinterpret_cast<const uint2 *>(
            packed + static_cast<size_t>(grow) * half_stride + ((kbase + seg * 16) >> 1));
        const float s = half_bits_to_float(scale[static_cast<size_t>(grow) * n_groups + kt]);
        const uint32_t wv[2] = {pk.x, pk.y};
#pragma unroll
        for (int e = 0; e < 16; ++e) {
          const uint32_t code = (wv[e >> 3] >> (4 * (e & 7))) & 0xFu;
          const int k = kbase + seg * 16 + e;
          const float wq = __bfloat162float(__float2bfloat16(lut[code] * s));
          vals[e] = k < K ? wq : 0.f;
        }
      } else {
#pragma unroll
        for (int e = 0; e < 16; ++e) vals[e] = 0.f;
      }
#pragma unroll
      for (int e = 0; e < 16; ++e) ws[r][seg * 16 + e] = vals[e];
    }
    for (int i = tid; i < sBK * sBN; i += sBlock) {
      const int kk = i / sBN;
      const int n = i - kk * sBN;
      const int k = kbase + kk;
      xs[kk][n] = (k < K && n < N) ? __bfloat162float(x[static_cast<size_t>(k) * N + n]) : 0.f;
    }
    __syncthreads();
#pragma unroll 8
    for (int kk = 0; kk < sBK; ++kk) {
      float a[4], b[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) a[i] = ws[ty * 4 + i][kk];
#pragma unroll
      for (int c = 0; c < 4; ++c) b[c] = xs[kk][tx + 16 * c];
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int c = 0; c < 4; ++c) acc[i][c] = fmaf(a[i], b[c], acc[i][c]);
    }
    __syncthreads();
  }

#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int grow = row0 + ty * 4 + i;
    if (grow >= M) continue;
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      const int n = tx + 16 * c;
      if (n >= N) continue;
      if (partial != nullptr) {
        partial[(static_cast<size_t>(blockIdx.y) * M + grow) * N + n] = acc[i][c];
      } else {
        y[static_cast<size_t>(grow) * N + n] = __float2bfloat16(acc[i][c]);
      }
    }
  }
}

__global__ void reduce_splitk_kernel(const float *__restrict__ partial,
                                     __nv_bfloat16 *__restrict__ y, int total, int splits) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= total) return;
  float v = 0.f;
  for (int s = 0; s < splits; ++s) v += partial[static_cast<size_t>(s) * total + i];
  y[i] = __float2bfloat16(v);
}

int check_args(const chr_nf4_dev_t *w, int N, bool need_ptrs, int max_n) {
  if (w == nullptr) return kNull;
  if (N < 1 || N > max_n) return kRangeN;
  if (w->M < 1 || w->K < 1) return kDims;
  if (need_ptrs && (w->packed == nullptr || w->scale == nullptr)) return kDims;
  if (!k_pad_ok(w->K, w->K_pad)) return kKPad;
  return kOk;
}

}  // namespace

Tuning &tuning() {
  static Tuning t = [] {
    Tuning init{};
    init.path = env_int("CHR_NF4_PATH", 0);
    init.split_k = env_int("CHR_NF4_SPLIT_K", 0);
    init.one_wave = env_int("CHR_NF4_ONE_WAVE", 0);
    if (init.path < 0 || init.path > 2) init.path = 0;
    if (init.split_k < 0) init.split_k = 0;
    if (init.one_wave < 0) init.one_wave = 0;
    return init;
  }();
  return t;
}

int resolved_one_wave() {
  const int w = tuning().one_wave;
  return w > 0 ? w : sm_count();
}

TileShape tile_shape(int path, int N) {
  if (path == kPathTcgen05) return tc_tile_shape(N);
  return TileShape{sBM, sBK, sBlock,
                   static_cast<int>(sizeof(float)) * (sBM * (sBK + 1) + sBK * sBN + 16)};
}

int auto_path(int M, int K_pad, int N) {
  const int forced = tuning().path;
  if (forced == 2) return kPathSimt;
  if (tc_supported(M, K_pad, N)) return kPathTcgen05;
  return kPathSimt;
}

int plan_gemm(int M, int K, int K_pad, int N, int have_ws, chr_nf4_plan_t *out) {
  (void)K;
  chr_nf4_plan_t p{};
  p.path = auto_path(M, K_pad, N);
  const TileShape ts = tile_shape(p.path, N);
  p.bm = ts.bm;
  p.bk = ts.bk;
  p.block = ts.block;
  p.smem_bytes = ts.smem_bytes;
  p.grid_x = ceil_div(M, p.bm);
  p.n_ktiles = ceil_div(K_pad, p.bk);
  int want = 1;
  if (have_ws) {
    const int target = resolved_one_wave() * 2;
    want = tuning().split_k > 0 ? tuning().split_k : ceil_div(target, p.grid_x);
  }
  if (want < 1) want = 1;
  if (want > p.n_ktiles) want = p.n_ktiles;
  p.tiles_per_split = ceil_div(p.n_ktiles, want);
  p.grid_y = ceil_div(p.n_ktiles, p.tiles_per_split);
  p.ws_floats = p.grid_y > 1 ? static_cast<int64_t>(p.grid_y) * M * N : 0;
  p.ctas = p.grid_x * p.grid_y;
  *out = p;
  return kOk;
}

}  // namespace chr

using namespace chr;

extern "C" void chr_nf4_set_tuning(int32_t path, int32_t split_k, int32_t one_wave) {
  Tuning &t = tuning();
  t.path = (path >= 0 && path <= 2) ? path : 0;
  t.split_k = split_k > 0 ? split_k : 0;
  t.one_wave = one_wave > 0 ? one_wave : 0;
}

extern "C" int chr_nf4_gemm_plan(const chr_nf4_dev_t *w, int32_t N, int32_t have_ws,
                                 chr_nf4_plan_t *out) {
  if (out == nullptr) return kNull;
  const int rc = check_args(w, N, false, kPlanMaxN);
  if (rc != kOk) return rc;
  return plan_gemm(w->M, w->K, w->K_pad, N, have_ws, out);
}

extern "C" int chr_nf4_gemm_ws_max(const chr_nf4_dev_t *w, const void *x, void *y, int32_t N,
                                   float *ws, int64_t ws_floats, void *stream, int32_t max_n) {
  if (x == nullptr || y == nullptr) return kNull;
  if (max_n < 1 || max_n > kPlanMaxN) return kRangeN;
  const int rc = check_args(w, N, true, max_n);
  if (rc != kOk) return rc;
  if (!aligned(w->packed, 16) || !aligned(x, 16) || !aligned(w->scale, 2)) return kAlign;
  const int have_ws = (ws != nullptr && ws_floats > 0) ? 1 : 0;
  chr_nf4_plan_t p{};
  plan_gemm(w->M, w->K, w->K_pad, N, have_ws, &p);
  if (p.ws_floats > 0 && (!have_ws || ws_floats < p.ws_floats)) return kWorkspace;
  float *partial = p.grid_y > 1 ? ws : nullptr;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  auto *xb = static_cast<const __nv_bfloat16 *>(x);
  auto *yb = static_cast<__nv_bfloat16 *>(y);
  if (p.path == kPathTcgen05) {
    const int trc = launch_gemm_tc(*w, xb, yb, N, partial, p, st);
    if (trc != kOk) return trc;
  } else {
    const dim3 grid(static_cast<unsigned>(p.grid_x), static_cast<unsigned>(p.grid_y));
    gemm_simt_kernel<<<grid, sBlock, 0, st>>>(w->packed, w->scale, xb, yb, partial, w->M, w->K,
                                              w->K_pad, N, p.n_ktiles, p.tiles_per_split);
  }
  if (partial != nullptr) {
    const int total = w->M * N;
    reduce_splitk_kernel<<<static_cast<unsigned>(ceil_div(total, 256)), 256, 0, st>>>(
        partial, yb, total, p.grid_y);
  }
  return cudaGetLastError() == cudaSuccess ? kOk : kLaunch;
}

extern "C" int chr_nf4_gemm_ws(const chr_nf4_dev_t *w, const void *x, void *y, int32_t N,
                               float *ws, int64_t ws_floats, void *stream) {
  return chr_nf4_gemm_ws_max(w, x, y, N, ws, ws_floats, stream, kLiveMaxN);
}

extern "C" int chr_nf4_gemm(const chr_nf4_dev_t *w, const void *x, void *y, int32_t N,
                            void *stream) {
  return chr_nf4_gemm_ws(w, x, y, N, nullptr, 0, stream);
}
