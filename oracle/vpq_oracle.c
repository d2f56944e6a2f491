/* vpq_oracle.c -- CPU restatement of vpipe's 4-bit affine quantized linear.
 *
 * TEST INFRASTRUCTURE ONLY (checker and timed CPU baseline); see vpq_oracle.h.
 * Build: oracle/Makefile. This translation unit is compiled with
 * -ffp-contract=off and no ISA extensions so every expression below is one
 * IEEE binary32 operation per C operator, as in the reference shaders built
 * with -fno-fast-math (apple-silicon/metal-compute/cmake/vpipe-metal-kernel.cmake:205-212).
 */
#include "vpq_oracle.h"

#include <math.h>
#include <string.h>

/* ---------------------------------------------------------------- scalars */

/* generative-models/quantize/model-quantizer.cc:56-60 and
 * generative-models/flux2/metal-flux2-transformer.cc:55-58: the integer
 * round-to-nearest-even narrowing, used verbatim for finite inputs. */
uint16_t vpq_o_f32_to_bf16(float f) {
  uint32_t u;
  memcpy(&u, &f, 4);
  return (uint16_t)((u + 0x7fffu + ((u >> 16) & 1u)) >> 16);
}

float vpq_o_bf16_to_f32(uint16_t b) {
  uint32_t u = (uint32_t)b << 16;
  float f;
  memcpy(&f, &u, 4);
  return f;
}

/* The MSL (half) cast: IEEE binary16 round-to-nearest-even, written out on
 * the bit pattern so the result does not depend on compiler _Float16 support. */
uint16_t vpq_o_f32_to_f16(float f) {
  uint32_t u;
  memcpy(&u, &f, 4);
  const uint32_t sign = (u >> 16) & 0x8000u;
  const uint32_t a = u & 0x7fffffffu;
  if (a >= 0x7f800000u) { /* inf / nan */
    return (uint16_t)(sign | 0x7c00u | ((a > 0x7f800000u) ? 0x200u : 0u));
  }
  if (a >= 0x477ff000u) { /* rounds to >= 65520 -> inf */
    return (uint16_t)(sign | 0x7c00u);
  }
  if (a < 0x33000001u) { /* <= 2^-25: rounds to zero (ties-to-even at 2^-25) */
    return (uint16_t)sign;
  }
  int e = (int)(a >> 23) - 127;
  uint32_t m = (a & 0x7fffffu) | 0x800000u; /* 24-bit significand */
  int shift;                                /* bits dropped from m */
  uint32_t base;
  if (e >= -14) { /* normal half */
    shift = 13;
    base = (uint32_t)(e + 15) << 10;
    m &= 0x7fffffu;
  } else { /* subnormal half: value = m * 2^(e-23), unit 2^-24 */
    shift = 13 + (-14 - e);
    base = 0;
  }
  uint32_t q = m >> shift;
  const uint32_t rem = m & ((1u << shift) - 1u);
  const uint32_t half = 1u << (shift - 1);
  if (rem > half || (rem == half && (q & 1u))) { q += 1u; }
  return (uint16_t)(sign | (base + q)); /* carry into the exponent is correct */
}

float vpq_o_f16_to_f32(uint16_t h) {
  const uint32_t sign = ((uint32_t)h & 0x8000u) << 16;
  const uint32_t e = (h >> 10) & 0x1fu;
  const uint32_t m = h & 0x3ffu;
  uint32_t u;
  if (e == 0) {
    if (m == 0) {
      u = sign;
    } else { /* subnormal: m * 2^-24 */
      float f = (float)m * 5.9604644775390625e-8f;
      memcpy(&u, &f, 4);
      u |= sign;
    }
  } else if (e == 31) {
    u = sign | 0x7f800000u | (m << 13);
  } else {
    u = sign | ((e + 112u) << 23) | (m << 13);
  }
  float f;
  memcpy(&f, &u, 4);
  return f;
}

void vpq_o_narrow_f32_bf16(const float* src, uint16_t* dst, size_t n) {
  for (size_t i = 0; i < n; ++i) { dst[i] = vpq_o_f32_to_bf16(src[i]); }
}

void vpq_o_f16_to_bf16(const uint16_t* src, uint16_t* dst, size_t n) {
  for (size_t i = 0; i < n; ++i) {
    dst[i] = vpq_o_f32_to_bf16(vpq_o_f16_to_f32(src[i]));
  }
}

size_t vpq_o_weight_bytes(int N, int K, int bits) {
  return (size_t)N * (size_t)(K * bits / 32) * 4u;
}
size_t vpq_o_scale_bytes(int N, int K, int group) {
  return (size_t)N * (size_t)(K / group) * 2u;
}

/* --------------------------------------------------------------- quantize */

/* MSL min/max on floats: min(x,y) = (y < x) ? y : x, max(x,y) = (x < y) ? y : x.
 * With that definition the running minimum keeps the FIRST element equal to
 * the final minimum, which decides the sign of a zero bias. */
static inline float msl_min(float x, float y) { return (y < x) ? y : x; }
static inline float msl_max(float x, float y) { return (x < y) ? y : x; }

int vpq_o_quant_w4_g64(const uint16_t* w_elt, int src_is_bf16, uint32_t* codes,
                       uint16_t* scales_f16, uint16_t* biases_f16,
                       int K, int N, float clip) {
  if (N <= 0 || K <= 0 || (K % 64) != 0) { return -1; }
  const int KG = K / 64;
  const int WPR = K / 8;
  for (int n = 0; n < N; ++n) {
    for (int grp = 0; grp < KG; ++grp) {
      /* affine_dequant.metal:258-263 */
      const uint16_t* xp = w_elt + (size_t)n * K + (size_t)grp * 64;
      float v[64];
      float mn = INFINITY, mx = -INFINITY;
      for (int i = 0; i < 64; ++i) {
        v[i] = src_is_bf16 ? vpq_o_bf16_to_f32(xp[i]) : vpq_o_f16_to_f32(xp[i]);
        mn = msl_min(mn, v[i]);
        mx = msl_max(mx, v[i]);
      }
      /* :264-268 */
      if (clip < 1.0f) {
        const float mid = 0.5f * (mn + mx);
        mn = mid + (mn - mid) * clip;
        mx = mid + (mx - mid) * clip;
      }
      /* :269-272 */
      const float scale = (mx - mn) / 15.0f;
      const float inv = (scale > 0.0f) ? 1.0f / scale : 0.0f;
      scales_f16[(size_t)n * KG + grp] = vpq_o_f32_to_f16(scale);
      biases_f16[(size_t)n * KG + grp] = vpq_o_f32_to_f16(mn);
      /* :274-284 ; MSL round() is half away from zero == roundf */
      uint32_t* wp = codes + (size_t)n * WPR + (size_t)grp * 8;
      for (int wi = 0; wi < 8; ++wi) {
        uint32_t packed = 0;
        for (int i = 0; i < 8; ++i) {
          int q = (int)roundf((v[wi * 8 + i] - mn) * inv);
          q = q < 0 ? 0 : (q > 15 ? 15 : q);
          packed |= ((uint32_t)q) << (4 * i);
        }
        wp[wi] = packed;
      }
    }
  }
  return 0;
}

/* The template the reference instantiates for w8_g64, w4_g64, w8_g32 and w4_g32
 * (affine_quant_impl<BITS, GROUP>, affine_dequant.metal:243-301). */
int vpq_o_quant(const uint16_t* w_elt, int src_is_bf16, uint32_t* codes, uint16_t* scales_f16,
                uint16_t* biases_f16, int K, int N, int bits, int group, float clip) {
  if (N <= 0 || K <= 0 || (bits != 4 && bits != 8) || (group != 32 && group != 64) || (K % group) != 0) {
    return -1;
  }
  const int KG = K / group;
  const int VPW = 32 / bits;          /* values per word, :255 */
  const int WPG = group / VPW;        /* words per group, :256 */
  const int QMAX = (1 << bits) - 1;
  const int WPR = K * bits / 32;      /* words per row, :258 */
  for (int n = 0; n < N; ++n) {
    for (int grp = 0; grp < KG; ++grp) {
      const uint16_t* xp = w_elt + (size_t)n * K + (size_t)grp * group;
      float v[64];
      float mn = INFINITY, mx = -INFINITY;
      for (int i = 0; i < group; ++i) {
        v[i] = src_is_bf16 ? vpq_o_bf16_to_f32(xp[i]) : vpq_o_f16_to_f32(xp[i]);
        mn = msl_min(mn, v[i]);
        mx = msl_max(mx, v[i]);
      }
      if (clip < 1.0f) {
        const float mid = 0.5f * (mn + mx);
        mn = mid + (mn - mid) * clip;
        mx = mid + (mx - mid) * clip;
      }
      const float scale = (mx - mn) / (float)QMAX;
      const float inv = (scale > 0.0f) ? 1.0f / scale : 0.0f;
      scales_f16[(size_t)n * KG + grp] = vpq_o_f32_to_f16(scale);
      biases_f16[(size_t)n * KG + grp] = vpq_o_f32_to_f16(mn);
      uint32_t* wp = codes + (size_t)n * WPR + (size_t)grp * WPG;
      for (int wi = 0; wi < WPG; ++wi) {
        uint32_t packed = 0;
        for (int i = 0; i < VPW; ++i) {
          int q = (int)roundf((v[wi * VPW + i] - mn) * inv);
          q = q < 0 ? 0 : (q > QMAX ? QMAX : q);
          packed |= ((uint32_t)q) << (bits * i);
        }
        wp[wi] = packed;
      }
    }
  }
  return 0;
}

/* ------------------------------------------------------------- dequantize */

/* affine_dequant_w4g64 / w8g64 / w8g32 (affine_dequant.metal:25-58, 69-98, 107-135) and the
 * group-32 form of the 4-bit one: y = (ELT)(s * q + b), one rounding in f32, one to bf16. */
int vpq_o_dequant_bf16(const uint32_t* codes, const uint16_t* s_bf16, const uint16_t* b_bf16,
                       uint16_t* out_bf16, int K, int N, int bits, int group) {
  if (N <= 0 || K <= 0 || (bits != 4 && bits != 8) || (group != 32 && group != 64) || (K % group) != 0) {
    return -1;
  }
  const int VPW = 32 / bits, Kw = K / VPW, Kg = K / group;
  const uint32_t mask = (1u << bits) - 1u;
  for (int n = 0; n < N; ++n) {
    for (int word = 0; word < Kw; ++word) {
      const int k0 = word * VPW;
      const size_t g = (size_t)n * Kg + (size_t)(k0 / group);
      const float s = vpq_o_bf16_to_f32(s_bf16[g]);
      const float b = vpq_o_bf16_to_f32(b_bf16[g]);
      const uint32_t packed = codes[(size_t)n * Kw + word];
      for (int i = 0; i < VPW; ++i) {
        const uint32_t q = (packed >> (bits * i)) & mask;
        out_bf16[(size_t)n * K + k0 + i] = vpq_o_f32_to_bf16(s * (float)q + b);  /* s*q exact in f32 */
      }
    }
  }
  return 0;
}


void vpq_o_dequant_w4g64_bf16(const uint32_t* codes, const uint16_t* s_bf16,
                              const uint16_t* b_bf16, uint16_t* out_bf16,
                              int K, int N) {
  const int Kw = K >> 3, Kg = K / 64;
  for (int n = 0; n < N; ++n) {
    for (int word = 0; word < Kw; ++word) {
      const int k0 = word << 3;
      const size_t g = (size_t)n * Kg + (size_t)(k0 / 64);
      const float s = vpq_o_bf16_to_f32(s_bf16[g]);
      const float b = vpq_o_bf16_to_f32(b_bf16[g]);
      const uint32_t packed = codes[(size_t)n * Kw + word];
      for (int i = 0; i < 8; ++i) {
        const uint32_t q = (packed >> (4 * i)) & 0xfu;
        /* affine_dequant.metal:49-52: s*q is exact in f32, so mul+add and a
         * fused multiply-add give the same bits. */
        out_bf16[(size_t)n * K + k0 + i] = vpq_o_f32_to_bf16(s * (float)q + b);
      }
    }
  }
}

void vpq_o_dequant_w4g64_f32(const uint32_t* codes, const uint16_t* s_bf16,
                             const uint16_t* b_bf16, float* out_f32,
                             int K, int N) {
  const int Kw = K >> 3, Kg = K / 64;
  for (int n = 0; n < N; ++n) {
    for (int word = 0; word < Kw; ++word) {
      const int k0 = word << 3;
      const size_t g = (size_t)n * Kg + (size_t)(k0 / 64);
      const float s = vpq_o_bf16_to_f32(s_bf16[g]);
      const float b = vpq_o_bf16_to_f32(b_bf16[g]);
      const uint32_t packed = codes[(size_t)n * Kw + word];
      for (int i = 0; i < 8; ++i) {
        const uint32_t q = (packed >> (4 * i)) & 0xfu;
        out_f32[(size_t)n * K + k0 + i] = s * (float)q + b;
      }
    }
  }
}

/* ---------------------------------------------------------------- matmuls */

void vpq_o_matmul_f32_seq(const uint16_t* x_bf16, const float* deq,
                          float* y_f32, int M, int N, int K) {
  for (int m = 0; m < M; ++m) {
    for (int n = 0; n < N; ++n) {
      float acc = 0.0f;
      for (int k = 0; k < K; ++k) {
        acc += vpq_o_bf16_to_f32(x_bf16[(size_t)m * K + k]) * deq[(size_t)n * K + k];
      }
      y_f32[(size_t)m * N + n] = acc;
    }
  }
}

void vpq_o_matmul_f64(const uint16_t* x_bf16, const float* deq,
                      double* y_f64, int M, int N, int K) {
  for (int m = 0; m < M; ++m) {
    for (int n = 0; n < N; ++n) {
      double acc = 0.0;
      for (int k = 0; k < K; ++k) {
        acc += (double)vpq_o_bf16_to_f32(x_bf16[(size_t)m * K + k]) *
               (double)deq[(size_t)n * K + k];
      }
      y_f64[(size_t)m * N + n] = acc;
    }
  }
}

/* ------------------------------------------- QMV in the kernel's own order */

static inline float bf16_round(float f) {
  return vpq_o_bf16_to_f32(vpq_o_f32_to_bf16(f));
}

void vpq_o_qmv_kernel_order(const uint32_t* codes, const uint16_t* s_bf16,
                            const uint16_t* b_bf16, const uint16_t* x_bf16,
                            uint16_t* y_bf16, int K, int N, int M) {
  enum { VPT = 16, BLOCK = 512, LANES = 32 };
  const int Kg = K / 64;
  for (int m = 0; m < M; ++m) {
    const uint16_t* xr = x_bf16 + (size_t)m * K;
    for (int n = 0; n < N; ++n) {
      float result[LANES];
      for (int l = 0; l < LANES; ++l) { result[l] = 0.0f; }
      for (int k = 0; k < K; k += BLOCK) {
        const int krem = K - k;
        for (int l = 0; l < LANES; ++l) {
          const int kk = k + l * VPT;
          float xt[VPT];
          float sum = 0.0f;
          if (krem >= BLOCK) {
            /* load_vector, affine_qmv.metal:57-66: the 4-term partial is
             * formed in the storage type (bf16), then widened. */
            for (int i = 0; i < VPT; i += 4) {
              const float x0 = vpq_o_bf16_to_f32(xr[kk + i]);
              const float x1 = vpq_o_bf16_to_f32(xr[kk + i + 1]);
              const float x2 = vpq_o_bf16_to_f32(xr[kk + i + 2]);
              const float x3 = vpq_o_bf16_to_f32(xr[kk + i + 3]);
              const float t = bf16_round(bf16_round(bf16_round(x0 + x1) + x2) + x3);
              sum += t;
              xt[i] = x0;
              xt[i + 1] = x1 / 16.0f;
              xt[i + 2] = x2 / 256.0f;
              xt[i + 3] = x3 / 4096.0f;
            }
          } else {
            /* load_vector_safe, :89-103: masked tail, partials in float. */
            int valid = K - kk;
            if (valid < 0) { valid = 0; }
            for (int i = 0; i < VPT; i += 4) {
              const float v0 = (i + 0 < valid) ? vpq_o_bf16_to_f32(xr[kk + i]) : 0.0f;
              const float v1 = (i + 1 < valid) ? vpq_o_bf16_to_f32(xr[kk + i + 1]) : 0.0f;
              const float v2 = (i + 2 < valid) ? vpq_o_bf16_to_f32(xr[kk + i + 2]) : 0.0f;
              const float v3 = (i + 3 < valid) ? vpq_o_bf16_to_f32(xr[kk + i + 3]) : 0.0f;
              sum += v0 + v1 + v2 + v3;
              xt[i] = v0;
              xt[i + 1] = v1 / 16.0f;
              xt[i + 2] = v2 / 256.0f;
              xt[i + 3] = v3 / 4096.0f;
            }
          }
          if (kk >= K) { continue; } /* fully masked lane adds 0 */
          /* qdot, :151-174: unshifted 16-bit masks against pre-divided x. */
          const size_t g = (size_t)n * Kg + (size_t)(kk / 64);
          const float s = vpq_o_bf16_to_f32(s_bf16[g]);
          const float b = vpq_o_bf16_to_f32(b_bf16[g]);
          const uint32_t w0 = codes[(size_t)n * (K / 8) + kk / 8];
          const uint32_t w1 = (kk + 8 < K) ? codes[(size_t)n * (K / 8) + kk / 8 + 1] : 0u;
          const uint16_t ws[4] = {(uint16_t)(w0 & 0xffffu), (uint16_t)(w0 >> 16),
                                  (uint16_t)(w1 & 0xffffu), (uint16_t)(w1 >> 16)};
          float accum = 0.0f;
          for (int i = 0; i < 4; ++i) {
            accum += (xt[4 * i] * (float)(ws[i] & 0x000f) +
                      xt[4 * i + 1] * (float)(ws[i] & 0x00f0) +
                      xt[4 * i + 2] * (float)(ws[i] & 0x0f00) +
                      xt[4 * i + 3] * (float)(ws[i] & 0xf000));
          }
          result[l] += s * accum + sum * b;
        }
      }
      /* simd_sum as a butterfly, :268-269 */
      for (int off = 16; off >= 1; off >>= 1) {
        float t[LANES];
        for (int l = 0; l < LANES; ++l) { t[l] = result[l] + result[l ^ off]; }
        for (int l = 0; l < LANES; ++l) { result[l] = t[l]; }
      }
      y_bf16[(size_t)m * N + n] = vpq_o_f32_to_bf16(result[0]);
    }
  }
}

/* -------------------------------------------------------- output byte sizes
 * and the remaining (multithreaded, contraction-tolerant) routines live in
 * vpq_oracle_fast.c */
