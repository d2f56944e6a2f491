// ref_driver.cc -- runs the reference's own quantize / dequantize shader source on the CPU.
//
// TEST INFRASTRUCTURE ONLY. The reference file
//   gpu-kernels/metal/quant/affine_dequant.metal   (tgo-app-dev/vpipe)
// is #included UNMODIFIED from the read-only reference checkout at build time
// (path given by -DREF_SRC=...; nothing from it is stored in this repository)
// and compiled as C++ against oracle/ref_shim/metal_stdlib. Each exported
// function walks the dispatch grid the reference host code launches and calls
// the kernel once per grid point:
//   quantize  : grid {K/64, N, 1}  generative-models/quantize/affine-quantizer.cc:79-80
//   dequantize: grid {K/8,  N, 1}  gpu-kernels/metal/quant/affine_dequant.metal:15
// Built twice (VPIPE_ELT = half / bfloat), as the reference builds its
// affine_dequant / affine_dequant_bf16 libraries.
#include <metal_stdlib>

#ifndef REF_SRC
#error "REF_SRC must name the reference's affine_dequant.metal"
#endif
#ifndef REF_SFX
#error "REF_SFX must be f16 or bf16"
#endif

namespace {
#include REF_SRC
}  // namespace

#define REF_CAT2(a, b) a##b
#define REF_CAT(a, b) REF_CAT2(a, b)
#define REF_FN(name) REF_CAT(REF_CAT(name, _), REF_SFX)

extern "C" {

// x: [N,K] VPIPE_ELT bit patterns; s,b: F16 bit patterns.
int REF_FN(ref_affine_quant_w4_g64)(const void* x, uint32_t* w, void* s, void* b,
                                    int K, int N, float clip) {
  if (N <= 0 || K <= 0 || (K % 64) != 0) { return -1; }
  for (unsigned n = 0; n < (unsigned)N; ++n) {
    for (unsigned g = 0; g < (unsigned)(K / 64); ++g) {
      affine_quant_w4_g64(static_cast<const VPIPE_ELT*>(x), w,
                          static_cast<half*>(s), static_cast<half*>(b), K, N,
                          clip, metal::uint2(g, n));
    }
  }
  return 0;
}

// s,b,out: VPIPE_ELT bit patterns.
int REF_FN(ref_affine_dequant_w4g64)(const uint32_t* w, const void* s, const void* b,
                                     void* out, int K, int N) {
  if (N <= 0 || K <= 0 || (K % 64) != 0) { return -1; }
  for (unsigned n = 0; n < (unsigned)N; ++n) {
    for (unsigned word = 0; word < (unsigned)(K / 8); ++word) {
      affine_dequant_w4g64(w, static_cast<const VPIPE_ELT*>(s),
                           static_cast<const VPIPE_ELT*>(b),
                           static_cast<VPIPE_ELT*>(out), K, N,
                           metal::uint2(word, n));
    }
  }
  return 0;
}

// The other instantiations of the same template (w8_g64, w8_g32, w4_g32) and the 8-bit
// dequantizers: selected by (bits, group).
int REF_FN(ref_affine_quant)(const void* x, uint32_t* w, void* s, void* b, int K, int N, int bits, int group,
                             float clip) {
  if (N <= 0 || K <= 0 || (K % group) != 0) { return -1; }
  for (unsigned n = 0; n < (unsigned)N; ++n) {
    for (unsigned g = 0; g < (unsigned)(K / group); ++g) {
      const VPIPE_ELT* xp = static_cast<const VPIPE_ELT*>(x);
      half* sp = static_cast<half*>(s);
      half* bp = static_cast<half*>(b);
      const metal::uint2 gid(g, n);
      if (bits == 8 && group == 64) {
        affine_quant_w8_g64(xp, w, sp, bp, K, N, clip, gid);
      } else if (bits == 4 && group == 64) {
        affine_quant_w4_g64(xp, w, sp, bp, K, N, clip, gid);
      } else if (bits == 8 && group == 32) {
        affine_quant_w8_g32(xp, w, sp, bp, K, N, clip, gid);
      } else if (bits == 4 && group == 32) {
        affine_quant_w4_g32(xp, w, sp, bp, K, N, clip, gid);
      } else {
        return -1;
      }
    }
  }
  return 0;
}

// The reference's dequantizers: w4g64, w8g64, w8g32, w4g32.
int REF_FN(ref_affine_dequant)(const uint32_t* w, const void* s, const void* b, void* out, int K, int N,
                               int bits, int group) {
  if (N <= 0 || K <= 0 || (K % group) != 0) { return -1; }
  const unsigned words = (unsigned)(K * bits / 32);
  for (unsigned n = 0; n < (unsigned)N; ++n) {
    for (unsigned word = 0; word < words; ++word) {
      const VPIPE_ELT* sp = static_cast<const VPIPE_ELT*>(s);
      const VPIPE_ELT* bp = static_cast<const VPIPE_ELT*>(b);
      VPIPE_ELT* op = static_cast<VPIPE_ELT*>(out);
      const metal::uint2 gid(word, n);
      if (bits == 4 && group == 64) {
        affine_dequant_w4g64(w, sp, bp, op, K, N, gid);
      } else if (bits == 8 && group == 64) {
        affine_dequant_w8g64(w, sp, bp, op, K, N, gid);
      } else if (bits == 8 && group == 32) {
        affine_dequant_w8g32(w, sp, bp, op, K, N, gid);
      } else if (bits == 4 && group == 32) {
        affine_dequant_w4g32(w, sp, bp, op, K, N, gid);
      } else {
        return -1;
      }
    }
  }
  return 0;
}

// 8-bit group-64 weights requantised to 4 bits: grid {K/64, N, 1}
// (gpu-kernels/metal/quant/affine_dequant.metal:143).
int REF_FN(ref_affine_requant_w8_to_w4_g64)(const uint32_t* w8, const void* s8, const void* b8, uint32_t* w4,
                                            void* s4, void* b4, int K, int N) {
  if (N <= 0 || K <= 0 || (K % 64) != 0) { return -1; }
  for (unsigned n = 0; n < (unsigned)N; ++n) {
    for (unsigned g = 0; g < (unsigned)(K / 64); ++g) {
      affine_requant_w8_to_w4_g64(w8, static_cast<const VPIPE_ELT*>(s8), static_cast<const VPIPE_ELT*>(b8), w4,
                                  static_cast<VPIPE_ELT*>(s4), static_cast<VPIPE_ELT*>(b4), K, N, metal::uint2(g, n));
    }
  }
  return 0;
}

}  // extern "C"
