// Launch planner shared by the GEMM entry points (host only).
//
// Same contract as the reference's planner (gpu/nf4/nf4_gemm.cu:1545-1619,
// mirrored in gpu/nf4/plan.py:161-236): pure arithmetic on M/K/K_pad/N, split-K
// aimed at two CTAs per SM and capped at the number of K tiles, ws_floats =
// split*M*N FP32 partials when split > 1. The tiles are this library's.
#pragma once

#include "chr_gpu.h"

namespace chr {

constexpr int kLiveMaxN = 32;
constexpr int kPlanMaxN = 64;

enum GemmPath : int {
  kPathTcgen05 = 0,  // TMA + dequant warps + tcgen05.mma, accumulators in TMEM
  kPathSimt = 1,     // CUDA-core tile kernel (debug / cross-check)
};

struct Tuning {
  int path;      // 0 auto, 1 force tcgen05, 2 force SIMT
  int split_k;   // 0 auto, >0 forced
  int one_wave;  // 0 = SM count of the current device
};

Tuning &tuning();
int resolved_one_wave();

// Tile geometry per path.
struct TileShape {
  int bm, bk, block, smem_bytes;
};
TileShape tile_shape(int path, int N);
int auto_path(int M, int K_pad, int N);

int plan_gemm(int M, int K, int K_pad, int N, int have_ws, chr_nf4_plan_t *out);

}  // namespace chr
