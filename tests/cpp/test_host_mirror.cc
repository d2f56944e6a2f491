// Parity tests written the way the reference writes its own (tests/unit-tests/
// metal-compute-gemm-mma.cc:253-288,407-498 and model-quantize-roundtrip.cc:84-164): build a
// random 4-bit weight with bf16 scales / biases, run the kernel through load_library /
// function / set_buffer / dispatch / commit().wait(), compare with an fp32 triple loop.
// Uses the C++ host layer include/vpq_host.hpp over the C ABI. Exit code 0 = all passed.
#include <cmath>
#include <cstdio>
#include <cstring>
#include <random>
#include <vector>

#include "vpq_host.hpp"

using namespace vpq::host;

static int g_fail = 0;
#define EXPECT_TRUE(c) do { if (!(c)) { std::printf("EXPECT_TRUE failed: %s (line %d)\n", #c, __LINE__); ++g_fail; } } while (0)

static uint16_t f32_to_bf16(float f) {
  uint32_t u; std::memcpy(&u, &f, 4);
  return (uint16_t)((u + 0x7fffu + ((u >> 16) & 1u)) >> 16);
}
static float bf16_to_f32(uint16_t b) {
  uint32_t u = (uint32_t)b << 16; float f; std::memcpy(&f, &u, 4); return f;
}

struct QWeight {
  std::vector<uint8_t> packed;   // N * K/2, even k = low nibble
  std::vector<uint16_t> scales, biases;
  std::vector<float> deq;
};
static QWeight make_qweight(int N, int K, uint32_t seed) {
  const int G = K / 64;
  QWeight q;
  q.packed.assign((size_t)N * (K / 2), 0);
  q.scales.resize((size_t)N * G); q.biases.resize((size_t)N * G); q.deq.resize((size_t)N * K);
  std::mt19937 rng(seed);
  std::uniform_int_distribution<int> nib(0, 15);
  std::uniform_real_distribution<float> sd(0.005f, 0.02f), bd(-0.1f, 0.1f);
  for (int n = 0; n < N; ++n) {
    for (int g = 0; g < G; ++g) {
      q.scales[(size_t)n * G + g] = f32_to_bf16(sd(rng));
      q.biases[(size_t)n * G + g] = f32_to_bf16(bd(rng));
    }
    for (int k = 0; k < K; ++k) {
      const int v = nib(rng);
      q.packed[(size_t)n * (K / 2) + (k >> 1)] |= (uint8_t)((k & 1) ? (v << 4) : v);
      const float s = bf16_to_f32(q.scales[(size_t)n * G + k / 64]), b = bf16_to_f32(q.biases[(size_t)n * G + k / 64]);
      q.deq[(size_t)n * K + k] = s * (float)v + b;
    }
  }
  return q;
}

static double run_linear(Compute& mc, const char* lib, const char* entry, int M, int N, int K) {
  ComputeFunction fn = mc.load_library(lib).function(entry);
  EXPECT_TRUE(fn.valid());
  std::vector<uint16_t> x((size_t)M * K);
  std::mt19937 rng(555 + M + N + K);
  std::normal_distribution<float> nd(0.0f, 1.0f);
  for (auto& v : x) { v = f32_to_bf16(nd(rng)); }
  QWeight q = make_qweight(N, K, 999 + N + K);
  std::vector<float> ref((size_t)M * N);
  for (int m = 0; m < M; ++m) for (int n = 0; n < N; ++n) {
    float acc = 0.0f;
    for (int k = 0; k < K; ++k) { acc += bf16_to_f32(x[(size_t)m * K + k]) * q.deq[(size_t)n * K + k]; }
    ref[(size_t)m * N + n] = acc;
  }
  SharedBuffer wb = mc.make_shared_buffer(q.packed.size()), sb = mc.make_shared_buffer(q.scales.size() * 2),
               bb = mc.make_shared_buffer(q.biases.size() * 2), xb = mc.make_shared_buffer(x.size() * 2),
               yb = mc.make_shared_buffer((size_t)M * N * 2);
  EXPECT_TRUE(!wb.empty() && !sb.empty() && !bb.empty() && !xb.empty() && !yb.empty());
  std::memcpy(wb.contents(), q.packed.data(), q.packed.size());
  std::memcpy(sb.contents(), q.scales.data(), q.scales.size() * 2);
  std::memcpy(bb.contents(), q.biases.data(), q.biases.size() * 2);
  std::memcpy(xb.contents(), x.data(), x.size() * 2);
  std::memset(yb.contents(), 0, (size_t)M * N * 2);
  CommandStream st;
  {
    ComputeEncoder enc = st.begin_compute();
    enc.set_function(fn);
    enc.set_buffer(0, wb); enc.set_buffer(1, sb); enc.set_buffer(2, bb);
    enc.set_buffer(3, xb); enc.set_buffer(4, yb);
    enc.set_k(K); enc.set_n(N); enc.set_m(M);
    enc.dispatch();
  }
  std::string why;
  EXPECT_TRUE(st.commit().wait_ok(&why));
  const uint16_t* yp = static_cast<const uint16_t*>(yb.contents());
  double num = 0.0, den = 0.0;
  for (size_t i = 0; i < (size_t)M * N; ++i) {
    const double d = (double)bf16_to_f32(yp[i]) - (double)ref[i];
    num += d * d; den += (double)ref[i] * (double)ref[i];
  }
  return den > 0 ? std::sqrt(num / den) : std::sqrt(num);
}

// The fused decode stores through the encoder, against the plain GEMV of the same weights:
// affine_qmv_qkv_w4g64 (outputs in slots 4..6, row counts as constants), affine_qmv_w4g64_add
// (slot 7 = residual) and affine_qmv_swiglu_w4g64 (rows interleaved gate | up, halved output).
static void test_fused_decode_stores(Compute& mc) {
  const int K = 512, Q = 64, KR = 32, V = 32, N = Q + KR + V;
  QWeight q = make_qweight(N, K, 4242);
  std::vector<uint16_t> x(K), res(N);
  std::mt19937 rng(77);
  std::normal_distribution<float> nd(0.0f, 1.0f);
  for (auto& v : x) { v = f32_to_bf16(nd(rng)); }
  for (auto& v : res) { v = f32_to_bf16(nd(rng)); }
  SharedBuffer wb = mc.make_shared_buffer(q.packed.size()), sb = mc.make_shared_buffer(q.scales.size() * 2),
               bb = mc.make_shared_buffer(q.biases.size() * 2), xb = mc.make_shared_buffer(K * 2),
               rb = mc.make_shared_buffer(N * 2), plain = mc.make_shared_buffer(N * 2),
               fused = mc.make_shared_buffer(N * 2), added = mc.make_shared_buffer(N * 2),
               act = mc.make_shared_buffer(N);
  std::memcpy(wb.contents(), q.packed.data(), q.packed.size());
  std::memcpy(sb.contents(), q.scales.data(), q.scales.size() * 2);
  std::memcpy(bb.contents(), q.biases.data(), q.biases.size() * 2);
  std::memcpy(xb.contents(), x.data(), K * 2);
  std::memcpy(rb.contents(), res.data(), N * 2);
  ComputeLibrary lib = mc.load_library("affine_qmv_bf16");
  CommandStream st;
  auto bind = [&](ComputeEncoder& enc, const char* entry) {
    ComputeFunction fn = lib.function(entry);
    EXPECT_TRUE(fn.valid());
    enc.set_function(fn);
    enc.set_buffer(0, wb); enc.set_buffer(1, sb); enc.set_buffer(2, bb); enc.set_buffer(3, xb);
    enc.set_k(K); enc.set_n(N);
  };
  {
    ComputeEncoder enc = st.begin_compute();
    bind(enc, "affine_qmv_w4g64");
    enc.set_buffer(4, plain);
    enc.dispatch();
    bind(enc, "affine_qmv_qkv_w4g64");
    enc.set_buffer(4, fused); enc.set_buffer(5, fused, Q * 2); enc.set_buffer(6, fused, (Q + KR) * 2);
    enc.set_qkv_rows(Q, KR, V);
    enc.dispatch();
    bind(enc, "affine_qmv_w4g64_add");
    enc.set_buffer(4, added); enc.set_buffer(7, rb);
    enc.dispatch();
    bind(enc, "affine_qmv_swiglu_w4g64");
    enc.set_buffer(4, act);
    enc.dispatch();
  }
  std::string why;
  EXPECT_TRUE(st.commit().wait_ok(&why));
  const uint16_t* p = static_cast<const uint16_t*>(plain.contents());
  const uint16_t* f = static_cast<const uint16_t*>(fused.contents());
  const uint16_t* a = static_cast<const uint16_t*>(added.contents());
  const uint16_t* g = static_cast<const uint16_t*>(act.contents());
  int bad = 0;
  for (int n = 0; n < N; ++n) {
    if (f[n] != p[n]) { ++bad; }                                             // q | k | v land where the rows say
    if (a[n] != f32_to_bf16(bf16_to_f32(p[n]) + bf16_to_f32(res[n]))) { ++bad; }  // bf16(bf16(sum) + residual)
  }
  for (int j = 0; j < N / 2; ++j) {  // silu(gate) * up, from unrounded sums: equal to the bf16 route within 2 %
    const float gt = bf16_to_f32(p[2 * j]), up = bf16_to_f32(p[2 * j + 1]);
    const float want = gt / (1.0f + std::exp(-gt)) * up;
    if (std::fabs(bf16_to_f32(g[j]) - want) > 0.02f * std::fabs(want) + 0.02f) { ++bad; }
  }
  std::printf("[fused] qkv / add / swiglu through the encoder: %d mismatches\n", bad);
  EXPECT_TRUE(bad == 0);
}

int main() {
  Compute mc;
  if (!mc.valid()) { std::printf("no CUDA device: nothing to test\n"); return 2; }
  // qmm_mma.correctness shapes, through every name the reference dispatches by
  struct Shape { int M, N, K; const char* tag; };
  const Shape shapes[] = {{64, 64, 64, "tiny"}, {96, 128, 128, "small"}, {130, 320, 256, "edge"},
                          {512, 256, 2560, "deepK"}, {33, 33, 128, "n33"}, {64, 95, 192, "n95"}};
  for (const auto& sh : shapes) {
    const double e1 = run_linear(mc, "affine_qmm_steel_bf16", "affine_qmm_steel_w4g64", sh.M, sh.N, sh.K);
    const double e2 = run_linear(mc, "affine_qmm_mma_bf16", "affine_qmm_mma_w4g64", sh.M, sh.N, sh.K);
    std::printf("[qmm] %-6s M=%d N=%d K=%d  steel rel-L2=%.3e  mma rel-L2=%.3e\n", sh.tag, sh.M, sh.N, sh.K, e1, e2);
    EXPECT_TRUE(e1 < 3e-2 && e2 < 3e-2);
  }
  {
    const double e = run_linear(mc, "affine_qmv_bf16", "affine_qmv_w4g64", 1, 512, 3840);
    std::printf("[qmv] N=512 K=3840 rel-L2=%.3e\n", e);
    EXPECT_TRUE(e < 1e-2);
  }
  test_fused_decode_stores(mc);
  // unknown entry -> invalid function, as ComputeLibrary::function does
  EXPECT_TRUE(!mc.load_library("affine_qmv_bf16").function("nope").valid());
  // quantize -> dequant round trip (model-quantize-roundtrip.cc:84-164): rel-L2 < 0.20 for w4
  {
    const int N = 64, K = 1024;
    SharedBuffer w = mc.make_shared_buffer((size_t)N * K * 2);
    std::mt19937 rng(11);
    std::normal_distribution<float> nd(0.0f, 0.02f);
    uint16_t* wp = static_cast<uint16_t*>(w.contents());
    for (size_t i = 0; i < (size_t)N * K; ++i) { wp[i] = f32_to_bf16(nd(rng)); }
    AffineQuantizer qz(&mc);
    EXPECT_TRUE(qz.valid());
    SharedBuffer codes, s16, b16;
    EXPECT_TRUE(qz.quantize_linear(w, true, N, K, 4, 64, 1.0f, codes, s16, b16));
    EXPECT_TRUE(!qz.quantize_linear(w, true, N, 1000, 4, 64, 1.0f, codes, s16, b16) || true);
    SharedBuffer s = mc.make_shared_buffer((size_t)N * (K / 64) * 2), b = mc.make_shared_buffer((size_t)N * (K / 64) * 2);
    SharedBuffer deq = mc.make_shared_buffer((size_t)N * K * 2);
    CommandStream st;
    EXPECT_TRUE(vpq_scales_f16_to_bf16(s16.contents(), s.contents(), N * (K / 64), st.native()) == VPQ_OK);
    EXPECT_TRUE(vpq_scales_f16_to_bf16(b16.contents(), b.contents(), N * (K / 64), st.native()) == VPQ_OK);
    {
      ComputeEncoder enc = st.begin_compute();
      enc.set_function(mc.load_library("affine_dequant_bf16").function("affine_dequant_w4g64"));
      enc.set_buffer(0, codes); enc.set_buffer(1, s); enc.set_buffer(2, b); enc.set_buffer(3, deq);
      enc.set_k(K); enc.set_n(N);
      enc.dispatch();
    }
    EXPECT_TRUE(st.commit().wait_ok(nullptr));
    const uint16_t* dp = static_cast<const uint16_t*>(deq.contents());
    double num = 0, den = 0;
    for (size_t i = 0; i < (size_t)N * K; ++i) {
      const double d = bf16_to_f32(dp[i]) - bf16_to_f32(wp[i]);
      num += d * d; den += (double)bf16_to_f32(wp[i]) * bf16_to_f32(wp[i]);
    }
    std::printf("[roundtrip] w4 rel-L2=%.4f\n", std::sqrt(num / den));
    EXPECT_TRUE(std::sqrt(num / den) < 0.20);
    // bad arguments: K not a multiple of the group -> false, nothing launched
    SharedBuffer c2, s2, b2;
    EXPECT_TRUE(!qz.quantize_linear(w, true, N, 1000, 4, 64, 1.0f, c2, s2, b2));
  }
  std::printf(g_fail ? "FAILED (%d)\n" : "ALL PASSED\n", g_fail);
  return g_fail ? 1 : 0;
}
