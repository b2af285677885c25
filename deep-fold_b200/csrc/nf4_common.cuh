// Shared device/host helpers for the sm_100a NF4 kernels.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cstdint>

#include "chr_gpu.h"

namespace chr {

constexpr int kGroup = 64;

// Return codes of the C ABI (reference: gpu/include/chr_gpu.h:30-33).
enum Rc : int {
  kOk = 0,
  kNull = -1,
  kRangeN = -2,
  kDims = -3,
  kKPad = -4,
  kAlign = -5,
  kLaunch = -6,
  kWorkspace = -7,
  kNonFinite = -8,
};

// binary32 bit patterns of the sixteen NF4 levels (docs/spec/nf4.md:37-54).
__device__ __constant__ uint32_t kLutBits[16] = {
    0xBF800000u, 0xBF3239B1u, 0xBF066B30u, 0xBECA32A0u, 0xBE91A24Du, 0xBE3D353Fu,
    0xBDBA7871u, 0x00000000u, 0x3DA2FAFFu, 0x3E24CAE3u, 0x3E7C04DDu, 0x3EAD033Au,
    0x3EE1A4B8u, 0x3F1007ABu, 0x3F3913B3u, 0x3F800000u,
};

inline bool k_pad_ok(int K, int K_pad) {
  return K >= 1 && K_pad >= K && K_pad == kGroup * ((K + kGroup - 1) / kGroup);
}

inline bool aligned(const void *p, uintptr_t a) {
  return (reinterpret_cast<uintptr_t>(p) & (a - 1)) == 0;
}

inline int check_matrix(const chr_nf4_dev_t *w) {
  if (w == nullptr) return kNull;
  if (w->M < 1 || w->K < 1 || w->packed == nullptr || w->scale == nullptr) return kDims;
  if (!k_pad_ok(w->K, w->K_pad)) return kKPad;
  return kOk;
}

// Programmatic dependent launch: kernels of the decode chain are launched with the
// programmatic-stream-serialization attribute, so a kernel's CTAs may start (and
// prefetch weights, build tables) while the previous kernel drains; pdl_wait()
// orders everything after it behind the previous kernel's completion. Both
// instructions are no-ops in a kernel launched without the attribute.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;"); }

bool pdl_enabled();
void set_pdl_enabled(bool on);

constexpr unsigned int kPeerPollsDefault = 1u << 22;
unsigned int &peer_polls();  // process-wide poll budget of the waits for a peer GPU

// Launch with or without the programmatic attribute (process-wide switch).
template <typename... KArgs, typename... Args>
inline cudaError_t launch_chain(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem,
                                cudaStream_t st, Args... args) {
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = pdl_enabled() ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

// Set the dynamic shared-memory limit of a kernel once per device.
template <typename Kernel>
inline bool ensure_smem_attr(Kernel kernel, int bytes, int (&done)[64]) {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return false;
  if (done[dev] >= bytes) return true;
  if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes) != cudaSuccess) {
    return false;
  }
  done[dev] = bytes;
  return true;
}

inline int sm_count() {
  // per device: a process may drive GPUs of different sizes
  static int cached[64] = {};
  int dev = 0, n = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
  if (cached[dev] > 0) return cached[dev];
  if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n < 1) {
    return 148;
  }
  cached[dev] = n;
  return n;
}

__device__ __forceinline__ float bf16_lo(uint32_t v) { return __uint_as_float(v << 16); }
__device__ __forceinline__ float bf16_hi(uint32_t v) { return __uint_as_float(v & 0xFFFF0000u); }

__device__ __forceinline__ float half_bits_to_float(uint16_t h) {
  return __half2float(__ushort_as_half(h));
}

// 16-byte streaming load that does not allocate in L1 (weights are read once).
__device__ __forceinline__ uint4 ld_stream16(const void *p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p));
  return v;
}

__device__ __forceinline__ uint16_t ld_stream_u16(const void *p) {
  uint16_t v;
  asm volatile("ld.global.nc.u16 %0, [%1];" : "=h"(v) : "l"(p));
  return v;
}

// Activation loads go through L2 (ld.global.cg): x, the residual and the RMSNorm
// input were written by the previous kernel of the chain.
__device__ __forceinline__ uint4 ld_act16(const void *p) {
  return __ldcg(reinterpret_cast<const uint4 *>(p));
}
__device__ __forceinline__ float ld_act_bf16(const __nv_bfloat16 *p) {
  return bf16_lo(static_cast<uint32_t>(__ldcg(reinterpret_cast<const unsigned short *>(p))));
}

// Packed FP32 pairs live in 64-bit registers end to end, so that no pack/unpack
// moves surround the packed FMA (fma.rn.f32x2, sm_100).
typedef unsigned long long f32x2_t;

__device__ __forceinline__ f32x2_t pack_f32x2(float lo, float hi) {
  f32x2_t v;
  asm("mov.b64 %0, {%1, %2};" : "=l"(v) : "f"(lo), "f"(hi));
  return v;
}

__device__ __forceinline__ void unpack_f32x2(f32x2_t v, float &lo, float &hi) {
  asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}

__device__ __forceinline__ f32x2_t ffma2(f32x2_t a, f32x2_t b, f32x2_t c) {
  f32x2_t d;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
  return d;
}

__device__ __forceinline__ f32x2_t fmul2(f32x2_t a, f32x2_t b) {
  f32x2_t d;
  asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
  return d;
}

__device__ __forceinline__ f32x2_t lds_f32x2(uint32_t saddr) {
  f32x2_t v;
  asm volatile("ld.shared.b64 %0, [%1];" : "=l"(v) : "r"(saddr));
  return v;
}

__device__ __forceinline__ float warp_sum_xor(float v) {
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) v += __shfl_xor_sync(0xffffffffu, v, off);
  return v;
}

__device__ __forceinline__ float warp_max_xor(float v) {
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, off));
  return v;
}

// sum(x^2) over n bf16 values computed by ONE warp in a fixed order (lane l owns
// the 8-element groups l, l+32, ...; xor butterfly), so every warp of every
// kernel that needs the RMSNorm scale gets the same bits.
__device__ __forceinline__ float warp_sumsq_bf16(const __nv_bfloat16 *__restrict__ x, int n,
                                                int lane) {
  float acc = 0.f;
  const int n8 = n >> 3;
  const uint4 *xv = reinterpret_cast<const uint4 *>(x);
#pragma unroll 4
  for (int g = lane; g < n8; g += 32) {
    const uint4 v = __ldg(xv + g);
    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const float lo = bf16_lo(w[e]);
      const float hi = bf16_hi(w[e]);
      acc = fmaf(lo, lo, acc);
      acc = fmaf(hi, hi, acc);
    }
  }
  for (int i = (n8 << 3) + lane; i < n; i += 32) {
    const float v = __bfloat162float(x[i]);
    acc = fmaf(v, v, acc);
  }
  return warp_sum_xor(acc);
}

// Greedy pick: a key that orders (logit, index) pairs so that the maximum key is the
// argmax with the lowest index on ties; NaN ranks above everything, -0 equals +0.
__device__ __forceinline__ unsigned long long pick_key(uint32_t bf16_bits, int idx) {
  uint32_t b = bf16_bits & 0xFFFFu;
  uint32_t ord;
  if ((b & 0x7FFFu) > 0x7F80u) {
    ord = 0xFFFFu;  // NaN ranks above everything, as torch.argmax does
  } else {
    if (b == 0x8000u) b = 0u;  // -0 equals +0
    ord = (b & 0x8000u) ? (~b & 0xFFFFu) : (b | 0x8000u);
  }
  return (static_cast<unsigned long long>(ord) << 32) |
         static_cast<unsigned long long>(0xFFFFFFFFu - static_cast<uint32_t>(idx));
}

}  // namespace chr
