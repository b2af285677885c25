// Device-side NF4 group-64 encoder: the same arithmetic as the host codec
// (codec.cpp; reference internal/nf4/nf4.go:129-185), one warp per group, so
// that random-init models of tens of billions of weights are quantized where
// they are generated. Results are bit-identical to the host encoder.

#include "nf4_common.cuh"

namespace chr {
namespace {

__global__ void __launch_bounds__(256)
encode_kernel(const float *__restrict__ w, uint8_t *__restrict__ packed,
              uint16_t *__restrict__ scale, int32_t *status, int M, int K, int K_pad) {
  const int n_groups = K_pad / kGroup;
  const long long total = static_cast<long long>(M) * n_groups;
  const int lane = threadIdx.x & 31;
  const long long warp0 = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  const long long n_warps = (static_cast<long long>(gridDim.x) * blockDim.x) >> 5;
  for (long long gidx = warp0; gidx < total; gidx += n_warps) {
    const int r = static_cast<int>(gidx / n_groups);
    const int g = static_cast<int>(gidx - static_cast<long long>(r) * n_groups);
    const int k = g * kGroup + 2 * lane;
    const float *row = w + static_cast<size_t>(r) * K;
    const float v0 = k < K ? row[k] : 0.f;
    const float v1 = k + 1 < K ? row[k + 1] : 0.f;
    if (!isfinite(v0) || !isfinite(v1)) {
      if (status != nullptr) *status = 1;
    }
    float top = warp_max_xor(fmaxf(fabsf(v0), fabsf(v1)));
    if (top == 0.f) top = 1.f;
    __half h = __float2half_rn(top);
    float s = __half2float(h);
    if (!isfinite(s) || s <= 0.f) {
      top = top > 65504.f ? 65504.f : 1.f;
      h = __float2half_rn(top);
      s = __half2float(h);
    }
    uint32_t byte = 0;
#pragma unroll
    for (int e = 0; e < 2; ++e) {
      float u = __fdiv_rn(e == 0 ? v0 : v1, s);
      u = u > 1.f ? 1.f : (u < -1.f ? -1.f : u);
      int best = 0;
      float d = __fsub_rn(u, __uint_as_float(kLutBits[0]));
      float best_d2 = __fmul_rn(d, d);
#pragma unroll
      for (int j = 1; j < 16; ++j) {
        d = __fsub_rn(u, __uint_as_float(kLutBits[j]));
        const float d2 = __fmul_rn(d, d);
        if (d2 < best_d2) {
          best_d2 = d2;
          best = j;
        }
      }
      byte |= static_cast<uint32_t>(best) << (4 * e);
    }
    packed[static_cast<size_t>(r) * (K_pad >> 1) + (k >> 1)] = static_cast<uint8_t>(byte);
    if (lane == 0) scale[static_cast<size_t>(r) * n_groups + g] = __half_as_ushort(h);
  }
}

}  // namespace
}  // namespace chr

using namespace chr;

extern "C" int chr_nf4_encode_dev(const float *w, int32_t M, int32_t K, uint8_t *packed,
                                  uint16_t *scale, int32_t *status, void *stream) {
  if (w == nullptr || packed == nullptr || scale == nullptr) return kNull;
  if (M < 1 || K < 1) return kDims;
  const int k_pad = kGroup * ((K + kGroup - 1) / kGroup);
  const long long groups = static_cast<long long>(M) * (k_pad / kGroup);
  long long blocks = (groups + 7) / 8;
  const long long cap = static_cast<long long>(sm_count()) * 16;
  if (blocks > cap) blocks = cap;
  encode_kernel<<<static_cast<unsigned>(blocks), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      w, packed, scale, status, M, K, k_pad);
  return cudaGetLastError() == cudaSuccess ? kOk : kLaunch;
}
