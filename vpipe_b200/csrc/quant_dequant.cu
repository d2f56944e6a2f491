// quant_dequant.cu -- forward quantizer, dequantizer and the load-time dtype
// conversions of the 4-bit affine group-64 format. All bit-exact with the
// reference shaders; all pure HBM streams.
#include "vpq_common.cuh"

namespace vpq {

// ---------------------------------------------------------------- quantize
// One thread owns 8 consecutive values (one packed word); the 8 threads of a
// group reduce min / max with shuffles. Replaces affine_quant_impl<4,64>
// (gpu-kernels/metal/quant/affine_dequant.metal:243-301), which uses one
// thread per group with strided reads.
//
// The reference scans the group in index order with min(a,b) = (b<a)?b:a, so
// among equal values (+0 / -0) the FIRST one is kept; that decides the sign
// bit of a zero bias. The butterfly keeps that rule: on a tie the lower lane
// (lower indices) wins.
template <bool SRC_BF16>
__global__ void __launch_bounds__(256)
affine_quant_w4_g64_kernel(const uint16_t* __restrict__ x, uint32_t* __restrict__ w,
                           __half* __restrict__ s, __half* __restrict__ b,
                           int64_t total_words, float clip) {
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  const unsigned lane = threadIdx.x & 31u;
  // The loop bound is warp-uniform (all 32 lanes take part in every shuffle);
  // total_words is a multiple of 8, so the 8 lanes of a group are valid together.
  for (int64_t word = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; word - lane < total_words;
       word += stride) {
    const bool valid = word < total_words;
    const uint4 raw = valid ? *reinterpret_cast<const uint4*>(x + word * 8) : make_uint4(0, 0, 0, 0);
    const uint32_t r[4] = {raw.x, raw.y, raw.z, raw.w};
    float v[8];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      if (SRC_BF16) {
        v[2 * i] = __uint_as_float(r[i] << 16);
        v[2 * i + 1] = __uint_as_float(r[i] & 0xffff0000u);
      } else {
        v[2 * i] = __half2float(__ushort_as_half((unsigned short)(r[i] & 0xffffu)));
        v[2 * i + 1] = __half2float(__ushort_as_half((unsigned short)(r[i] >> 16)));
      }
    }
    float mn = __int_as_float(0x7f800000), mx = __int_as_float(0xff800000);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      mn = (v[i] < mn) ? v[i] : mn;
      mx = (mx < v[i]) ? v[i] : mx;
    }
#pragma unroll
    for (int d = 1; d < 8; d <<= 1) {
      const float omn = __shfl_xor_sync(0xffffffffu, mn, d);
      const float omx = __shfl_xor_sync(0xffffffffu, mx, d);
      if (lane & d) {  // partner holds lower indices: it wins ties
        mn = (mn < omn) ? mn : omn;
        mx = (omx < mx) ? mx : omx;
      } else {
        mn = (omn < mn) ? omn : mn;
        mx = (mx < omx) ? omx : mx;
      }
    }
    if (clip < 1.0f) {  // one rounding per operator, never contracted
      const float mid = __fmul_rn(0.5f, __fadd_rn(mn, mx));
      mn = __fadd_rn(mid, __fmul_rn(__fsub_rn(mn, mid), clip));
      mx = __fadd_rn(mid, __fmul_rn(__fsub_rn(mx, mid), clip));
    }
    const float scale = __fdiv_rn(__fsub_rn(mx, mn), 15.0f);
    const float inv = (scale > 0.0f) ? __fdiv_rn(1.0f, scale) : 0.0f;
    uint32_t packed = 0;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      int q = (int)roundf(__fmul_rn(__fsub_rn(v[i], mn), inv));  // half away from zero
      q = min(max(q, 0), 15);
      packed |= (uint32_t)q << (4 * i);
    }
    if (!valid) { continue; }
    w[word] = packed;
    if ((word & 7) == 0) {
      s[word >> 3] = __float2half_rn(scale);
      b[word >> 3] = __float2half_rn(mn);
    }
  }
}

// -------------------------------------------------------------- dequantize
// One thread expands one packed word into 8 bf16 (one 16-byte store), so a
// warp reads 128 B and writes 512 B, both fully coalesced.
// Replaces affine_dequant_w4g64 (gpu-kernels/metal/quant/affine_dequant.metal:25-58).
__global__ void __launch_bounds__(256)
affine_dequant_w4g64_kernel(const uint32_t* __restrict__ w, const uint16_t* __restrict__ scales,
                            const uint16_t* __restrict__ biases, uint4* __restrict__ ydeq,
                            int64_t total_words) {
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t word = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; word < total_words;
       word += stride) {
    const uint32_t packed = __ldg(w + word);
    const float s = bf16_bits_to_f32(__ldg(scales + (word >> 3)));
    const float b = bf16_bits_to_f32(__ldg(biases + (word >> 3)));
    uint32_t o[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const uint32_t lo = f32_to_bf16_bits(dequant_f32(s, (packed >> (8 * i)) & 0xfu, b));
      const uint32_t hi = f32_to_bf16_bits(dequant_f32(s, (packed >> (8 * i + 4)) & 0xfu, b));
      o[i] = lo | (hi << 16);
    }
    ydeq[word] = make_uint4(o[0], o[1], o[2], o[3]);
  }
}

// ------------------------------------------------------------- conversions
__global__ void __launch_bounds__(256)
f16_to_bf16_kernel(const __half* __restrict__ src, uint16_t* __restrict__ dst, int64_t n) {
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
    dst[i] = (uint16_t)f32_to_bf16_bits(__half2float(src[i]));
  }
}

__global__ void __launch_bounds__(256)
f32_to_bf16_kernel(const float* __restrict__ src, uint16_t* __restrict__ dst, int64_t n) {
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
    dst[i] = (uint16_t)f32_to_bf16_bits(src[i]);
  }
}

static int stream_grid(int64_t items, int threads) {
  const int64_t want = (items + threads - 1) / threads;
  const int64_t cap = (int64_t)num_sms() * 16;  // 16 resident 256-thread CTAs cover a wave
  return (int)(want < 1 ? 1 : (want > cap ? cap : want));
}

}  // namespace vpq

using namespace vpq;

extern "C" int vpq_affine_quant_w4_g64(const void* w_elt, int src_is_bf16, uint32_t* codes,
                                       void* scales_f16, void* biases_f16, int64_t K, int64_t N,
                                       float clip, void* stream) {
  clear_error();
  if (!w_elt || !codes || !scales_f16 || !biases_f16) {
    return fail(VPQ_ERR_INVALID_ARG, "affine_quant_w4_g64: null pointer");
  }
  if (N <= 0 || K <= 0 || (K % 64) != 0) {  // affine-quantizer.cc:57
    return fail(VPQ_ERR_INVALID_ARG, "affine_quant_w4_g64: need N>0, K>0, K%%64==0 (K=%lld N=%lld)",
                (long long)K, (long long)N);
  }
  if (!aligned16(w_elt) || !aligned16(codes)) {
    return fail(VPQ_ERR_ALIGNMENT, "affine_quant_w4_g64: w_elt and codes must be 16-byte aligned");
  }
  if (int rc = require_sm100()) { return rc; }
  const int64_t words = N * (K / 8);
  const int grid = stream_grid(words, 256);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (src_is_bf16) {
    affine_quant_w4_g64_kernel<true><<<grid, 256, 0, st>>>(
        static_cast<const uint16_t*>(w_elt), codes, static_cast<__half*>(scales_f16),
        static_cast<__half*>(biases_f16), words, clip);
  } else {
    affine_quant_w4_g64_kernel<false><<<grid, 256, 0, st>>>(
        static_cast<const uint16_t*>(w_elt), codes, static_cast<__half*>(scales_f16),
        static_cast<__half*>(biases_f16), words, clip);
  }
  VPQ_LAUNCH_OK("affine_quant_w4_g64");
  return VPQ_OK;
}

extern "C" int vpq_affine_dequant_w4g64_bf16(const uint32_t* w, const void* scales,
                                             const void* biases, void* ydeq, int64_t K, int64_t N,
                                             void* stream) {
  clear_error();
  if (!w || !scales || !biases || !ydeq) {
    return fail(VPQ_ERR_INVALID_ARG, "affine_dequant_w4g64: null pointer");
  }
  if (N <= 0 || K <= 0 || (K % 64) != 0) {
    return fail(VPQ_ERR_INVALID_ARG, "affine_dequant_w4g64: need N>0, K>0, K%%64==0");
  }
  if (!aligned16(ydeq) || !aligned16(w)) {
    return fail(VPQ_ERR_ALIGNMENT, "affine_dequant_w4g64: w and ydeq must be 16-byte aligned");
  }
  if (int rc = require_sm100()) { return rc; }
  const int64_t words = N * (K / 8);
  affine_dequant_w4g64_kernel<<<stream_grid(words, 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      w, static_cast<const uint16_t*>(scales), static_cast<const uint16_t*>(biases),
      static_cast<uint4*>(ydeq), words);
  VPQ_LAUNCH_OK("affine_dequant_w4g64");
  return VPQ_OK;
}

extern "C" int vpq_scales_f16_to_bf16(const void* src_f16, void* dst_bf16, int64_t n, void* stream) {
  clear_error();
  if (!src_f16 || !dst_bf16 || n <= 0) {
    return fail(VPQ_ERR_INVALID_ARG, "scales_f16_to_bf16: null pointer or n<=0");
  }
  if (int rc = require_sm100()) { return rc; }
  f16_to_bf16_kernel<<<stream_grid(n, 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __half*>(src_f16), static_cast<uint16_t*>(dst_bf16), n);
  VPQ_LAUNCH_OK("scales_f16_to_bf16");
  return VPQ_OK;
}

extern "C" int vpq_narrow_f32_bf16(const float* src, void* dst_bf16, int64_t n, void* stream) {
  clear_error();
  if (!src || !dst_bf16 || n <= 0) {
    return fail(VPQ_ERR_INVALID_ARG, "narrow_f32_bf16: null pointer or n<=0");
  }
  if (int rc = require_sm100()) { return rc; }
  f32_to_bf16_kernel<<<stream_grid(n, 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      src, static_cast<uint16_t*>(dst_bf16), n);
  VPQ_LAUNCH_OK("narrow_f32_bf16");
  return VPQ_OK;
}
