/* vpq_oracle_fast.c -- multithreaded parts of the CPU oracle / CPU baseline.
 *
 * TEST INFRASTRUCTURE ONLY; see vpq_oracle.h. Compiled with OpenMP and AVX2+FMA
 * (oracle/Makefile): the contraction is f32 but the summation order (8
 * interleaved partial sums, fused multiply-adds) is not the sequential order
 * of vpq_o_matmul_f32_seq; the two agree to f32 rounding noise.
 *
 * The reference has no CPU matmul. Its CPU-side arithmetic for this path is
 * the f32 dequantise `dq = q*scale + bias` (generative-models/quantize/
 * model-quantizer.cc:252-258) and the fp32 triple-loop test oracle
 * (tests/unit-tests/metal-compute-gemm-mma.cc:441-451); this file is those
 * two, blocked and threaded, nothing more (no BLAS).
 */
#include "vpq_oracle.h"

#include <stdlib.h>
#include <string.h>
#include <time.h>
#ifdef _OPENMP
#include <omp.h>
#endif

int vpq_o_max_threads(void) {
#ifdef _OPENMP
  return omp_get_max_threads();
#else
  return 1;
#endif
}

static double now_s(void) {
  struct timespec ts;
  clock_gettime(CLOCK_MONOTONIC, &ts);
  return (double)ts.tv_sec + 1e-9 * (double)ts.tv_nsec;
}

static inline float bf16f(uint16_t b) {
  uint32_t u = (uint32_t)b << 16;
  float f;
  memcpy(&f, &u, 4);
  return f;
}

/* 4 x-rows against 4 w-rows per inner loop: 16 dot products share 8 loads. */
static void block_4x4(const float* x, const float* w, float* y, int K, int N,
                      int mrows, int nrows) {
  float acc[4][4][8];
  memset(acc, 0, sizeof(acc));
  for (int k = 0; k < K; k += 8) {
    for (int i = 0; i < 4; ++i) {
      const float* xr = x + (size_t)(i < mrows ? i : 0) * K + k;
      for (int j = 0; j < 4; ++j) {
        const float* wr = w + (size_t)(j < nrows ? j : 0) * K + k;
#pragma omp simd
        for (int l = 0; l < 8; ++l) { acc[i][j][l] += xr[l] * wr[l]; }
      }
    }
  }
  for (int i = 0; i < mrows; ++i) {
    for (int j = 0; j < nrows; ++j) {
      const float* a = acc[i][j];
      y[(size_t)i * N + j] =
          ((a[0] + a[4]) + (a[2] + a[6])) + ((a[1] + a[5]) + (a[3] + a[7]));
    }
  }
}

static void matmul_xf32(const float* xf, const float* deq, float* y_f32, int M,
                        int N, int K, int threads) {
  (void)threads;
  const int mb = (M + 3) / 4, nb = (N + 3) / 4;
#pragma omp parallel for schedule(static) num_threads(threads) collapse(2)
  for (int bm = 0; bm < mb; ++bm) {
    for (int bn = 0; bn < nb; ++bn) {
      const int m0 = bm * 4, n0 = bn * 4;
      const int mr = (M - m0 < 4) ? M - m0 : 4;
      const int nr = (N - n0 < 4) ? N - n0 : 4;
      block_4x4(xf + (size_t)m0 * K, deq + (size_t)n0 * K,
                y_f32 + (size_t)m0 * N + n0, K, N, mr, nr);
    }
  }
}

static int pick_threads(int threads) {
  return threads > 0 ? threads : vpq_o_max_threads();
}

void vpq_o_matmul_f32_fast(const uint16_t* x_bf16, const float* deq,
                           float* y_f32, int M, int N, int K, int threads) {
  threads = pick_threads(threads);
  float* xf = (float*)malloc((size_t)M * K * sizeof(float));
  if (!xf) { return; }
#pragma omp parallel for schedule(static) num_threads(threads)
  for (long i = 0; i < (long)M * K; ++i) { xf[i] = bf16f(x_bf16[i]); }
  matmul_xf32(xf, deq, y_f32, M, N, K, threads);
  free(xf);
}

/* W rounded to bf16 first (the steel loader writes the dequantised tile to
 * threadgroup memory as the storage type, affine_qmm_steel.metal:86-95,
 * 231-242), f32 accumulate, one rounding at store (:447-455). */
void vpq_o_qmm_kernel_numerics(const uint32_t* codes, const uint16_t* s_bf16,
                               const uint16_t* b_bf16, const uint16_t* x_bf16,
                               uint16_t* y_bf16, int K, int N, int M, int threads) {
  threads = pick_threads(threads);
  uint16_t* wb = (uint16_t*)malloc((size_t)N * K * 2);
  float* wf = (float*)malloc((size_t)N * K * sizeof(float));
  float* yf = (float*)malloc((size_t)M * N * sizeof(float));
  if (wb && wf && yf) {
    vpq_o_dequant_w4g64_bf16(codes, s_bf16, b_bf16, wb, K, N);
    for (size_t i = 0; i < (size_t)N * K; ++i) { wf[i] = bf16f(wb[i]); }
    vpq_o_matmul_f32_fast(x_bf16, wf, yf, M, N, K, threads);
    for (size_t i = 0; i < (size_t)M * N; ++i) { y_bf16[i] = vpq_o_f32_to_bf16(yf[i]); }
  }
  free(wb);
  free(wf);
  free(yf);
}

double vpq_o_cpu_linear(const uint32_t* codes, const uint16_t* s_bf16,
                        const uint16_t* b_bf16, const uint16_t* x_bf16,
                        uint16_t* y_bf16, float* deq_scratch,
                        int K, int N, int M, int threads) {
  threads = pick_threads(threads);
  const double t0 = now_s();
  const int Kw = K / 8, Kg = K / 64;
  /* dequantise, rows in parallel (dq = q*scale + bias in f32) */
#pragma omp parallel for schedule(static) num_threads(threads)
  for (int n = 0; n < N; ++n) {
    for (int word = 0; word < Kw; ++word) {
      const size_t g = (size_t)n * Kg + (size_t)(word / 8);
      const float s = bf16f(s_bf16[g]);
      const float b = bf16f(b_bf16[g]);
      const uint32_t packed = codes[(size_t)n * Kw + word];
      float* o = deq_scratch + (size_t)n * K + (size_t)word * 8;
      for (int i = 0; i < 8; ++i) {
        o[i] = s * (float)((packed >> (4 * i)) & 0xfu) + b;
      }
    }
  }
  float* xf = (float*)malloc((size_t)M * K * sizeof(float));
  float* yf = (float*)malloc((size_t)M * N * sizeof(float));
  if (xf && yf) {
    for (size_t i = 0; i < (size_t)M * K; ++i) { xf[i] = bf16f(x_bf16[i]); }
    matmul_xf32(xf, deq_scratch, yf, M, N, K, threads);
    for (size_t i = 0; i < (size_t)M * N; ++i) { y_bf16[i] = vpq_o_f32_to_bf16(yf[i]); }
  }
  free(xf);
  free(yf);
  return now_s() - t0;
}
