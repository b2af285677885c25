// Host-side NF4 group-64 codec (C++, multi-threaded), bit-exact with the
// reference writer: internal/nf4/nf4.go:46-82 (Encode), :85-121 (Decode),
// :129-170 (encodeGroup64), :172-185 (nearest); internal/f16/f16.go:8-85.
//
// Used to quantize synthetic (random-init) models of 3B..32B parameters in
// seconds; the numpy form of the same algorithm needs minutes to hours.

#include <algorithm>
#include <atomic>
#include <cmath>
#include <cstdint>
#include <cstring>
#include <thread>
#include <vector>

#include "chr_gpu.h"

namespace {

constexpr int kGroup = 64;

const uint32_t kLutBits[16] = {
    0xBF800000u, 0xBF3239B1u, 0xBF066B30u, 0xBECA32A0u, 0xBE91A24Du, 0xBE3D353Fu,
    0xBDBA7871u, 0x00000000u, 0x3DA2FAFFu, 0x3E24CAE3u, 0x3E7C04DDu, 0x3EAD033Au,
    0x3EE1A4B8u, 0x3F1007ABu, 0x3F3913B3u, 0x3F800000u,
};

inline float bits_to_f32(uint32_t b) {
  float f;
  std::memcpy(&f, &b, 4);
  return f;
}

inline uint32_t f32_to_bits(float f) {
  uint32_t b;
  std::memcpy(&b, &f, 4);
  return b;
}

// float32 -> binary16, round to nearest even; overflow -> Inf, subnormals kept.
uint16_t f32_to_f16(float f) {
  const uint32_t b = f32_to_bits(f);
  const uint16_t sign = static_cast<uint16_t>((b >> 16) & 0x8000u);
  const int exp = static_cast<int>((b >> 23) & 0xFFu);
  uint32_t mant = b & 0x7FFFFFu;
  if (exp == 0xFF) {
    if (mant != 0) {
      uint16_t n = static_cast<uint16_t>(mant >> 13);
      return static_cast<uint16_t>(sign | 0x7C00u | (n == 0 ? 1 : n));
    }
    return static_cast<uint16_t>(sign | 0x7C00u);
  }
  const int e = exp - 127 + 15;
  if (e >= 0x1F) return static_cast<uint16_t>(sign | 0x7C00u);
  if (e <= 0) {
    if (e < -10) return sign;
    mant |= 1u << 23;
    const uint32_t shift = static_cast<uint32_t>(14 - e);
    const uint32_t round = (mant >> (shift - 1)) & 1u;
    const uint32_t tail = mant & ((1u << (shift - 1)) - 1u);
    uint32_t m = mant >> shift;
    if (round != 0 && (tail != 0 || (m & 1u) != 0)) ++m;
    return static_cast<uint16_t>(sign | m);
  }
  uint16_t half = static_cast<uint16_t>(sign | (e << 10) | (mant >> 13));
  const uint32_t rem = mant & 0x1FFFu;
  if (rem > 0x1000u || (rem == 0x1000u && (half & 1u) != 0)) ++half;
  return half;
}

float f16_to_f32(uint16_t h) {
  const uint32_t sign = static_cast<uint32_t>(h & 0x8000u) << 16;
  const uint32_t exp = (h >> 10) & 0x1Fu;
  uint32_t mant = h & 0x3FFu;
  if (exp == 0) {
    if (mant == 0) return bits_to_f32(sign);
    int e = -1;
    do {
      mant <<= 1;
      ++e;
    } while ((mant & 0x400u) == 0);
    mant &= 0x3FFu;
    return bits_to_f32(sign | static_cast<uint32_t>(127 - 15 - e) << 23 | (mant << 13));
  }
  if (exp == 0x1F) return bits_to_f32(sign | 0x7F800000u | (mant << 13));
  return bits_to_f32(sign | ((exp + 127 - 15) << 23) | (mant << 13));
}

struct Tables {
  float lut[16];
  float mid[15];
  Tables() {
    for (int i = 0; i < 16; ++i) lut[i] = bits_to_f32(kLutBits[i]);
    for (int i = 0; i < 15; ++i) mid[i] = (lut[i] + lut[i + 1]) * 0.5f;
  }
};
const Tables kT;

// First minimum of float32 (u - L[j])^2 over j. The count of midpoints strictly
// below u is the nearest level or its neighbour; the squared distances of the
// three candidates (lowest index wins a tie) settle it exactly.
inline int nearest_code(float u) {
  int c = 0;
  for (int j = 0; j < 15; ++j) c += (u > kT.mid[j]) ? 1 : 0;
  int best = c > 0 ? c - 1 : 0;
  const float d = u - kT.lut[best];
  float best_d2 = d * d;
  const int cands[2] = {c, c < 15 ? c + 1 : 15};
  for (int cand : cands) {
    const float dd = u - kT.lut[cand];
    const float d2 = dd * dd;
    if (d2 < best_d2 || (d2 == best_d2 && cand < best)) {
      best = cand;
      best_d2 = d2;
    }
  }
  return best;
}

int resolve_threads(int threads, int rows) {
  int n = threads > 0 ? threads : static_cast<int>(std::thread::hardware_concurrency());
  if (n < 1) n = 1;
  return std::min(n, std::max(rows, 1));
}

template <typename F>
void parallel_rows(int rows, int threads, F &&fn) {
  const int n = resolve_threads(threads, rows);
  if (n == 1) {
    fn(0, rows);
    return;
  }
  std::vector<std::thread> pool;
  const int per = (rows + n - 1) / n;
  for (int t = 0; t < n; ++t) {
    const int lo = t * per;
    const int hi = std::min(rows, lo + per);
    if (lo >= hi) break;
    pool.emplace_back([=, &fn] { fn(lo, hi); });
  }
  for (auto &th : pool) th.join();
}

}  // namespace

extern "C" int chr_nf4_encode_f32(const float *w, int32_t M, int32_t K, uint8_t *packed,
                                  uint16_t *scale, int32_t threads) {
  if (w == nullptr || packed == nullptr || scale == nullptr) return -1;
  if (M < 1 || K < 1) return -3;
  const int k_pad = kGroup * ((K + kGroup - 1) / kGroup);
  const int n_groups = k_pad / kGroup;
  std::atomic<int> bad{0};
  parallel_rows(M, threads, [&](int lo, int hi) {
    float g[kGroup];
    for (int r = lo; r < hi; ++r) {
      const float *row = w + static_cast<size_t>(r) * K;
      uint8_t *prow = packed + static_cast<size_t>(r) * (k_pad / 2);
      for (int gi = 0; gi < n_groups; ++gi) {
        float top = 0.f;
        for (int i = 0; i < kGroup; ++i) {
          const int k = gi * kGroup + i;
          const float v = k < K ? row[k] : 0.f;
          if (!std::isfinite(v)) bad.store(1, std::memory_order_relaxed);
          g[i] = v;
          const float a = std::fabs(v);
          if (a > top) top = a;
        }
        if (top == 0.f) top = 1.f;
        uint16_t s16 = f32_to_f16(top);
        float s = f16_to_f32(s16);
        if (!std::isfinite(s) || s <= 0.f) {
          top = top > 65504.f ? 65504.f : 1.f;
          s16 = f32_to_f16(top);
          s = f16_to_f32(s16);
        }
        scale[static_cast<size_t>(r) * n_groups + gi] = s16;
        for (int i = 0; i < kGroup; i += 2) {
          float u0 = g[i] / s;
          float u1 = g[i + 1] / s;
          u0 = u0 > 1.f ? 1.f : (u0 < -1.f ? -1.f : u0);
          u1 = u1 > 1.f ? 1.f : (u1 < -1.f ? -1.f : u1);
          prow[(gi * kGroup + i) >> 1] =
              static_cast<uint8_t>(nearest_code(u0) | (nearest_code(u1) << 4));
        }
      }
    }
  });
  return bad.load() ? -8 : 0;
}

extern "C" int chr_nf4_decode_f32(const uint8_t *packed, const uint16_t *scale, int32_t M,
                                  int32_t K, float *w, int32_t threads) {
  if (w == nullptr || packed == nullptr || scale == nullptr) return -1;
  if (M < 1 || K < 1) return -3;
  const int k_pad = kGroup * ((K + kGroup - 1) / kGroup);
  const int n_groups = k_pad / kGroup;
  parallel_rows(M, threads, [&](int lo, int hi) {
    for (int r = lo; r < hi; ++r) {
      const uint8_t *prow = packed + static_cast<size_t>(r) * (k_pad / 2);
      float *out = w + static_cast<size_t>(r) * K;
      for (int k = 0; k < K; ++k) {
        const uint8_t byte = prow[k >> 1];
        const int code = (k & 1) ? (byte >> 4) : (byte & 0xF);
        const float s = f16_to_f32(scale[static_cast<size_t>(r) * n_groups + k / kGroup]);
        out[k] = kT.lut[code] * s;
      }
    }
  });
  return 0;
}
