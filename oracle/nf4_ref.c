/* Plain-C restatement of deep-fold's NF4 group-64 codec and float32 GEMV.
 *
 * TEST INFRASTRUCTURE ONLY: an independent scalar cross-check of the numpy
 * oracle (nf4_ref.py) and a CPU baseline at sizes numpy would need minutes for.
 * Nothing in the shipped package links or loads it. Parity is pinned through
 * the same golden vectors as nf4_ref.py (tests compare the two bit for bit).
 *
 * Reference followed: internal/nf4/nf4.go:85-121 (Decode), :129-170
 * (encodeGroup64), :172-185 (nearest: first minimum of float32 squared
 * distance); internal/f16/f16.go:8-85; gpu/tests/nf4_oracle.py:119-142.
 */
#include <math.h>
#include <stdint.h>
#include <string.h>

#define GROUP 64

static const uint32_t LUT_BITS[16] = {
    0xBF800000u, 0xBF3239B1u, 0xBF066B30u, 0xBECA32A0u, 0xBE91A24Du, 0xBE3D353Fu,
    0xBDBA7871u, 0x00000000u, 0x3DA2FAFFu, 0x3E24CAE3u, 0x3E7C04DDu, 0x3EAD033Au,
    0x3EE1A4B8u, 0x3F1007ABu, 0x3F3913B3u, 0x3F800000u,
};

static float from_bits(uint32_t b) {
  float f;
  memcpy(&f, &b, 4);
  return f;
}

static uint32_t to_bits(float f) {
  uint32_t b;
  memcpy(&b, &f, 4);
  return b;
}

static float half_to_float(uint16_t h) {
  uint32_t sign = (uint32_t)(h & 0x8000u) << 16;
  uint32_t exp = (h >> 10) & 0x1Fu;
  uint32_t mant = h & 0x3FFu;
  if (exp == 0) {
    if (mant == 0) return from_bits(sign);
    /* subnormal: value = mant * 2^-24 */
    return (sign ? -1.0f : 1.0f) * (float)mant * 5.9604644775390625e-08f;
  }
  if (exp == 0x1F) return from_bits(sign | 0x7F800000u | (mant << 13));
  return from_bits(sign | ((exp + 112u) << 23) | (mant << 13));
}

static uint16_t float_to_half(float f) {
  uint32_t b = to_bits(f);
  uint16_t sign = (uint16_t)((b >> 16) & 0x8000u);
  int exp = (int)((b >> 23) & 0xFFu);
  uint32_t mant = b & 0x7FFFFFu;
  if (exp == 0xFF) return (uint16_t)(sign | 0x7C00u | (mant ? (mant >> 13 ? mant >> 13 : 1) : 0));
  int e = exp - 127 + 15;
  if (e >= 0x1F) return (uint16_t)(sign | 0x7C00u);
  if (e <= 0) {
    if (e < -10) return sign;
    mant |= 1u << 23;
    uint32_t shift = (uint32_t)(14 - e);
    uint32_t round = (mant >> (shift - 1)) & 1u;
    uint32_t tail = mant & ((1u << (shift - 1)) - 1u);
    uint32_t m = mant >> shift;
    if (round && (tail || (m & 1u))) ++m;
    return (uint16_t)(sign | m);
  }
  uint16_t h = (uint16_t)(sign | (e << 10) | (mant >> 13));
  uint32_t rem = mant & 0x1FFFu;
  if (rem > 0x1000u || (rem == 0x1000u && (h & 1u))) ++h;
  return h;
}

static int k_padded(int k) { return GROUP * ((k + GROUP - 1) / GROUP); }

/* W_hat[m,k] = LUT[code] * scale, float32. */
void nf4c_decode(const uint8_t *packed, const uint16_t *scale, int m, int k, float *w) {
  int kp = k_padded(k), ng = kp / GROUP;
  for (int r = 0; r < m; ++r) {
    for (int c = 0; c < k; ++c) {
      uint8_t byte = packed[(size_t)r * (kp / 2) + (c >> 1)];
      int code = (c & 1) ? (byte >> 4) : (byte & 0xF);
      w[(size_t)r * k + c] = from_bits(LUT_BITS[code]) * half_to_float(scale[(size_t)r * ng + c / GROUP]);
    }
  }
}

/* Returns 0, or -8 on a non-finite weight. */
int nf4c_encode(const float *w, int m, int k, uint8_t *packed, uint16_t *scale) {
  int kp = k_padded(k), ng = kp / GROUP;
  for (int r = 0; r < m; ++r) {
    for (int g = 0; g < ng; ++g) {
      float v[GROUP], top = 0.f;
      for (int i = 0; i < GROUP; ++i) {
        int c = g * GROUP + i;
        v[i] = c < k ? w[(size_t)r * k + c] : 0.f;
        if (!isfinite(v[i])) return -8;
        if (fabsf(v[i]) > top) top = fabsf(v[i]);
      }
      if (top == 0.f) top = 1.f;
      uint16_t h = float_to_half(top);
      float s = half_to_float(h);
      if (!isfinite(s) || s <= 0.f) {
        top = top > 65504.f ? 65504.f : 1.f;
        h = float_to_half(top);
        s = half_to_float(h);
      }
      scale[(size_t)r * ng + g] = h;
      for (int i = 0; i < GROUP; i += 2) {
        int code[2];
        for (int e = 0; e < 2; ++e) {
          float u = v[i + e] / s;
          if (u > 1.f) u = 1.f;
          if (u < -1.f) u = -1.f;
          int best = 0;
          float d = u - from_bits(LUT_BITS[0]);
          float bd = d * d;
          for (int j = 1; j < 16; ++j) {
            d = u - from_bits(LUT_BITS[j]);
            float d2 = d * d;
            if (d2 < bd) {
              bd = d2;
              best = j;
            }
          }
          code[e] = best;
        }
        packed[(size_t)r * (kp / 2) + ((g * GROUP + i) >> 1)] = (uint8_t)(code[0] | (code[1] << 4));
      }
    }
  }
  return 0;
}

/* y[m] = sum_k W_hat[m,k] * x[k], float32 weights and products, double accumulator. */
void nf4c_gemv(const uint8_t *packed, const uint16_t *scale, int m, int k, const float *x, float *y) {
  int kp = k_padded(k), ng = kp / GROUP;
  float lut[16];
  for (int i = 0; i < 16; ++i) lut[i] = from_bits(LUT_BITS[i]);
  for (int r = 0; r < m; ++r) {
    const uint8_t *row = packed + (size_t)r * (kp / 2);
    double acc = 0.0;
    for (int c = 0; c < k; ++c) {
      uint8_t byte = row[c >> 1];
      int code = (c & 1) ? (byte >> 4) : (byte & 0xF);
      float wv = lut[code] * half_to_float(scale[(size_t)r * ng + c / GROUP]);
      acc += (double)(wv * x[c]);
    }
    y[r] = (float)acc;
  }
}
