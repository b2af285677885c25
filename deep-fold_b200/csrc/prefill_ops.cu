// Row-wise helpers of the chunked prefill (sm_100a): the elementwise work between
// the GEMMs of a chunk, which the reference leaves to torch ops in the cache dtype
// (gpu/decodev2/prefill.py:58-141). One launch each instead of five to twelve:
//   * RMSNorm of N rows,
//   * RoPE of q and k for N positions + the write of k / v into the cache rows,
//   * silu(gate) * up on the stacked gate/up GEMM output.
// Arithmetic follows what the torch ops do in bf16 (one rounding per op), so a
// chunk gives the same bits whether these kernels or the torch ops run; RMSNorm
// follows the decode kernels' formula bf16(w * x * rsqrt(mean(x^2) + eps)).

#include "nf4_common.cuh"

namespace chr {
namespace {

__device__ __forceinline__ float bf16r(float v) { return __bfloat162float(__float2bfloat16(v)); }

// One warp per row; the same summation order as the decode path's RMSNorm.
__global__ void __launch_bounds__(256) rms_rows_kernel(const __nv_bfloat16 *__restrict__ x,
                                                      const __nv_bfloat16 *__restrict__ w,
                                                      __nv_bfloat16 *__restrict__ y, int N, int K,
                                                      long long x_stride, float eps) {
  const int row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (row >= N) return;
  const __nv_bfloat16 *xr = x + static_cast<size_t>(row) * x_stride;
  const float s = rsqrtf(warp_sumsq_bf16(xr, K, lane) / static_cast<float>(K) + eps);
  __nv_bfloat16 *yr = y + static_cast<size_t>(row) * K;
  // 8 elements per lane and step where the row, the weight and the output allow
  // 16-byte accesses; the same products, rounded the same way, as the scalar tail
  const bool wide = ((reinterpret_cast<uintptr_t>(xr) | reinterpret_cast<uintptr_t>(w) |
                      reinterpret_cast<uintptr_t>(yr)) & 15) == 0;
  const int k8 = wide ? (K & ~7) : 0;
  for (int i = lane * 8; i < k8; i += 256) {
    const uint4 xv = *reinterpret_cast<const uint4 *>(xr + i);
    const uint4 wv = __ldg(reinterpret_cast<const uint4 *>(w + i));
    const uint32_t xs[4] = {xv.x, xv.y, xv.z, xv.w};
    const uint32_t ws[4] = {wv.x, wv.y, wv.z, wv.w};
    uint32_t o[4];
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const __nv_bfloat162 r = __floats2bfloat162_rn(bf16_lo(ws[e]) * bf16_lo(xs[e]) * s,
                                                     bf16_hi(ws[e]) * bf16_hi(xs[e]) * s);
      o[e] = *reinterpret_cast<const uint32_t *>(&r);
    }
    *reinterpret_cast<uint4 *>(yr + i) = make_uint4(o[0], o[1], o[2], o[3]);
  }
  for (int i = k8 + lane; i < K; i += 32) {
    yr[i] = __float2bfloat16(__bfloat162float(w[i]) * __bfloat162float(xr[i]) * s);
  }
}

// One CTA per position. q: [N, n_q, hd] read with row stride q_stride, written
// contiguous to q_out; k, v: [N, n_kv, hd] with their strides, written to the cache
// rows start + n (k rotated). bf16 arithmetic as torch does it: t*cos and
// swapped*sin are rounded, then their sum is.
__global__ void __launch_bounds__(256)
rope_kv_rows_kernel(const __nv_bfloat16 *__restrict__ q, long long q_stride,
                    const __nv_bfloat16 *__restrict__ k, long long k_stride,
                    const __nv_bfloat16 *__restrict__ v, long long v_stride,
                    __nv_bfloat16 *__restrict__ q_out, __nv_bfloat16 *__restrict__ k_cache,
                    __nv_bfloat16 *__restrict__ v_cache, const __nv_bfloat16 *__restrict__ cos,
                    const __nv_bfloat16 *__restrict__ sin, int start, int n_q, int n_kv, int hd) {
  const int n = blockIdx.x;
  const int pos = start + n;
  const int half = hd >> 1;
  const __nv_bfloat16 *c = cos + static_cast<size_t>(pos) * hd;
  const __nv_bfloat16 *s = sin + static_cast<size_t>(pos) * hd;
  const int q_pairs = n_q * half;
  const int k_pairs = n_kv * half;
  for (int i = threadIdx.x; i < q_pairs + k_pairs; i += blockDim.x) {
    const bool is_q = i < q_pairs;
    const int j = is_q ? i : i - q_pairs;
    const int h = j / half;
    const int d = j - h * half;
    const __nv_bfloat16 *src = is_q ? q + static_cast<size_t>(n) * q_stride + h * hd
                                    : k + static_cast<size_t>(n) * k_stride + h * hd;
    __nv_bfloat16 *dst = is_q ? q_out + (static_cast<size_t>(n) * n_q + h) * hd
                              : k_cache + (static_cast<size_t>(pos) * n_kv + h) * hd;
    const float lo = __bfloat162float(src[d]);
    const float hi = __bfloat162float(src[d + half]);
    const float o_lo = bf16r(bf16r(lo * __bfloat162float(c[d])) + bf16r(-hi * __bfloat162float(s[d])));
    const float o_hi = bf16r(bf16r(hi * __bfloat162float(c[d + half])) +
                             bf16r(lo * __bfloat162float(s[d + half])));
    dst[d] = __float2bfloat16(o_lo);
    dst[d + half] = __float2bfloat16(o_hi);
  }
  const int v_elems = n_kv * hd;
  for (int i = threadIdx.x; i < v_elems; i += blockDim.x) {
    v_cache[static_cast<size_t>(pos) * v_elems + i] = v[static_cast<size_t>(n) * v_stride + i];
  }
}

// out[n, i] = bf16( bf16(silu(g)) * u ),  g = gu[n, i], u = gu[n, I + i].
__global__ void __launch_bounds__(256) silu_mul_kernel(const __nv_bfloat16 *__restrict__ gu,
                                                      __nv_bfloat16 *__restrict__ out, int N, int I) {
  const long long total = static_cast<long long>(N) * I;
  const long long idx = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (idx >= total) return;
  const int n = static_cast<int>(idx / I);
  const int i = static_cast<int>(idx - static_cast<long long>(n) * I);
  const float g = __bfloat162float(gu[static_cast<size_t>(n) * 2 * I + i]);
  const float u = __bfloat162float(gu[static_cast<size_t>(n) * 2 * I + I + i]);
  const float sl = bf16r(g / (1.f + expf(-g)));
  out[idx] = __float2bfloat16(sl * u);
}

}  // namespace
}  // namespace chr

using namespace chr;

extern "C" int chr_nf4_rms_rows(const void *x, int64_t x_stride, const void *w, void *y, int32_t N,
                                int32_t K, float eps, void *stream) {
  if (x == nullptr || w == nullptr || y == nullptr) return kNull;
  if (N < 1 || K < 1 || x_stride < K) return kDims;
  if (!aligned(x, 16) || (x_stride % 8) != 0) return kAlign;
  const int rows_per_cta = 8;
  rms_rows_kernel<<<static_cast<unsigned>((N + rows_per_cta - 1) / rows_per_cta), 256, 0,
                    static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16 *>(x), static_cast<const __nv_bfloat16 *>(w),
      static_cast<__nv_bfloat16 *>(y), N, K, x_stride, eps);
  return cudaGetLastError() == cudaSuccess ? kOk : kLaunch;
}

extern "C" int chr_nf4_rope_kv_rows(const void *q, int64_t q_stride, const void *k, int64_t k_stride,
                                    const void *v, int64_t v_stride, void *q_out, void *k_cache,
                                    void *v_cache, const void *cos, const void *sin, int32_t start,
                                    int32_t N, int32_t n_q, int32_t n_kv, int32_t hd,
                                    int32_t max_seq, void *stream) {
  if (q == nullptr || k == nullptr || v == nullptr || q_out == nullptr || k_cache == nullptr ||
      v_cache == nullptr || cos == nullptr || sin == nullptr) {
    return kNull;
  }
  if (N < 1 || n_q < 1 || n_kv < 1 || hd < 2 || (hd & 1) != 0 || start < 0 ||
      static_cast<long long>(start) + N > max_seq || q_stride < static_cast<long long>(n_q) * hd ||
      k_stride < static_cast<long long>(n_kv) * hd || v_stride < static_cast<long long>(n_kv) * hd) {
    return kDims;
  }
  rope_kv_rows_kernel<<<static_cast<unsigned>(N), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16 *>(q), q_stride, static_cast<const __nv_bfloat16 *>(k),
      k_stride, static_cast<const __nv_bfloat16 *>(v), v_stride, static_cast<__nv_bfloat16 *>(q_out),
      static_cast<__nv_bfloat16 *>(k_cache), static_cast<__nv_bfloat16 *>(v_cache),
      static_cast<const __nv_bfloat16 *>(cos), static_cast<const __nv_bfloat16 *>(sin), start, n_q,
      n_kv, hd);
  return cudaGetLastError() == cudaSuccess ? kOk : kLaunch;
}

extern "C" int chr_nf4_silu_mul(const void *gate_up, void *out, int32_t N, int32_t I,
                                void *stream) {
  if (gate_up == nullptr || out == nullptr) return kNull;
  if (N < 1 || I < 1) return kDims;
  const long long total = static_cast<long long>(N) * I;
  silu_mul_kernel<<<static_cast<unsigned>((total + 255) / 256), 256, 0,
                    static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16 *>(gate_up), static_cast<__nv_bfloat16 *>(out), N, I);
  return cudaGetLastError() == cudaSuccess ? kOk : kLaunch;
}
