// NF4 GEMV for N = 1..8 activation rows on CUDA cores (sm_100a): entry points.
//
// The kernel is in gemv_cols.cuh (four activation rows per launch on the bulk-copy
// ring: every packed weight is read from HBM once and looked up once for all rows,
// FP32 weights as in the one-row GEMV). Five to eight rows take two launches. With K
// beyond 11 chunks of 1024 the launch is cut into K slices whose FP32 partials go to a
// caller workspace and are added up, in slice order, by the kernel below; results do
// not depend on the grid. No counterpart in the reference, whose GEMV is N = 1
// (gpu/nf4/nf4_gemv.cu:291-324).

#pragma once

#include "gemv_cols.cuh"

namespace chr {
namespace {

constexpr int kNMaxCols = 8;

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
  const GemvColsShape sh = pick_cols_shape(w->M, w->K_pad, true);
  const int per_launch = N < kColsN ? N : kColsN;
  return sh.n_kslices > 1 ? static_cast<int64_t>(sh.n_kslices) * per_launch * w->M : 0;
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
  const GemvColsShape sh = pick_cols_shape(w->M, w->K_pad, aligned(w->scale, 16));
  if (sh.n_slots < 2) return kDims;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  static int attr_done[64] = {};
  if (!ensure_smem_attr(nf4_gemv_cols_kernel<0>, static_cast<int>(sh.smem_bytes), attr_done)) return kLaunch;
  int *status = gemv_status_ptr();
  if (status == nullptr) return kLaunch;
  for (int n0 = 0; n0 < N; n0 += kColsN) {
    const int n = N - n0 < kColsN ? N - n0 : kColsN;
    GemvColsArgs a{};
    a.packed = w->packed;
    a.scale = w->scale;
    a.x = static_cast<const __nv_bfloat16 *>(x_rows) + static_cast<size_t>(n0) * w->K;
    a.y = static_cast<__nv_bfloat16 *>(y_rows) + static_cast<size_t>(n0) * w->M;
    a.add = add_rows == nullptr ? nullptr
                                : static_cast<const __nv_bfloat16 *>(add_rows) + static_cast<size_t>(n0) * w->M;
    a.bias = static_cast<const __nv_bfloat16 *>(bias);
    a.M = w->M;
    a.K = w->K;
    a.K_pad = w->K_pad;
    a.N = n;
    a.S = sh.S;
    a.G = sh.G;
    a.n_kslices = sh.n_kslices;
    a.n_tiles = sh.n_tiles;
    a.n_slots = sh.n_slots;
    a.scale_ring = sh.scale_ring;
    a.status = status;
    if (sh.n_kslices > 1) {
      const int64_t need = static_cast<int64_t>(sh.n_kslices) * n * w->M;
      if (ws == nullptr || ws_floats < need) return kWorkspace;
      a.ws = ws;
    }
    const dim3 grid(static_cast<unsigned>(sh.grid_x), static_cast<unsigned>(sh.n_kslices));
    const dim3 block(static_cast<unsigned>((sh.S * sh.G + 1) * 32));
    if (launch_chain(nf4_gemv_cols_kernel<0>, grid, block, sh.smem_bytes, st, a) != cudaSuccess) {
      return kLaunch;
    }
    if (sh.n_kslices > 1) {
      const size_t total = static_cast<size_t>(n) * w->M;
      const int blocks = static_cast<int>((total + 255) / 256 < 592 ? (total + 255) / 256 : 592);
      if (launch_chain(gemv_n_reduce_kernel, dim3(static_cast<unsigned>(blocks)), dim3(256), 0, st,
                       static_cast<const float *>(a.ws), a.y, a.add, a.bias, sh.n_kslices, n,
                       w->M) != cudaSuccess) {
        return kLaunch;
      }
    }
  }
  return kOk;
}
