// Tensor-core (tcgen05) NF4 GEMM for sm_100a -- placeholder until the kernel lands.
#include "gemm_plan.h"
#include "nf4_common.cuh"

namespace chr {

TileShape tc_tile_shape(int N) {
  (void)N;
  return TileShape{128, 64, 192, 0};
}

bool tc_supported(int M, int K_pad, int N) {
  (void)M;
  (void)K_pad;
  (void)N;
  return false;
}

int launch_gemm_tc(const chr_nf4_dev_t &w, const __nv_bfloat16 *x, __nv_bfloat16 *y, int N,
                   float *partial, const chr_nf4_plan_t &p, cudaStream_t st) {
  (void)w; (void)x; (void)y; (void)N; (void)partial; (void)p; (void)st;
  return kLaunch;
}

}  // namespace chr
