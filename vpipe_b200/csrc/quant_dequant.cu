// quant_dequant.cu -- forward quantizer, dequantizer and the load-time dtype
// conversions of the affine group-quantized formats: 4-bit group-64 (the hot
// path's format) and its twins w8g64, w8g32, w4g32. All bit-exact with the
// reference shaders; all pure HBM streams.
#include "vpq_common.cuh"

namespace vpq {

// clamp(round(t), 0, qmax) with round() = nearest, halves away from zero, as a float holding the
// integer. A profile of the quantizer showed the ALU pipe (compares, selects, min / max, shifts, logic:
// half the rate of the FMA pipe) 78 % busy and the DRAM 22 %, so the arithmetic is arranged to sit on
// the FMA pipe where it can: the clamp comes first, in floating point (monotonic, so the result is the
// same; a NaN becomes 0); adding and subtracting 2^23 rounds to an integer with ties to even; a tie that
// went down shows as value - rounded == 0.5 exactly and is moved up.
__device__ __forceinline__ float round_clamp_f(float t, float qmax) {
  const float tc = fminf(fmaxf(t, 0.0f), qmax);
  const float r = __fsub_rn(__fadd_rn(tc, 8388608.0f), 8388608.0f);
  return __fadd_rn(r, (__fsub_rn(tc, r) == 0.5f) ? 1.0f : 0.0f);
}

// Eight such integers (each <= 15, or <= 255) packed into one or two words. The weighted sums are
// formed in f32 (exact: every partial sum is an integer below 2^24) and converted once per half.
__device__ __forceinline__ uint32_t pack4_nibbles(float q0, float q1, float q2, float q3) {
  return __float2uint_rz(__fmaf_rn(q3, 4096.0f, __fmaf_rn(q2, 256.0f, __fmaf_rn(q1, 16.0f, q0))));
}
__device__ __forceinline__ uint32_t pack4_bytes(float q0, float q1, float q2, float q3) {
  return __float2uint_rz(__fmaf_rn(q2, 65536.0f, __fmaf_rn(q1, 256.0f, q0))) | (__float2uint_rz(q3) << 24);
}

// ---------------------------------------------------------------- quantize
// One thread owns 8 consecutive values (one packed word at 4 bits, two at 8);
// the GROUP / 8 threads of a group reduce min / max with shuffles. Replaces
// affine_quant_impl<BITS,GROUP> (gpu-kernels/metal/quant/affine_dequant.metal:243-301,
// instantiated as affine_quant_w4_g64, _w8_g64, _w8_g32, _w4_g32), which uses
// one thread per group with strided reads.
//
// The reference scans the group in index order with min(a,b) = (b<a)?b:a, so
// among equal values (+0 / -0) the FIRST one is kept; that decides the sign
// bit of a zero bias. The butterfly keeps that rule: on a tie the lower lane
// (lower indices) wins.
template <bool SRC_BF16, int BITS, int GROUP>
__global__ void __launch_bounds__(256)
affine_quant_kernel(const uint16_t* __restrict__ x, uint32_t* __restrict__ w,
                    __half* __restrict__ s, __half* __restrict__ b,
                    int64_t total_words, float clip) {  // total_words: octets of values (N * K / 8)
  constexpr int TPG = GROUP / 8;             // threads per group
  constexpr float QMAX = (float)((1 << BITS) - 1);
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  const unsigned lane = threadIdx.x & 31u;
  // The loop bound is warp-uniform (all 32 lanes take part in every shuffle);
  // total_words is a multiple of TPG, so the lanes of a group are valid together.
  // kInFlight independent 16-byte loads per thread are issued before the first is used: one load per
  // thread in flight (64 KB per SM at full occupancy) left the quantizer at a third of the HBM rate.
  constexpr int kInFlight = 4;
  for (int64_t word0 = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; word0 - lane < total_words;
       word0 += stride * kInFlight) {
    uint4 raws[kInFlight];
#pragma unroll
    for (int u = 0; u < kInFlight; ++u) {
      const int64_t wd = word0 + u * stride;
      raws[u] = wd < total_words ? ldg_stream_v4(x + wd * 8) : make_uint4(0, 0, 0, 0);
    }
#pragma unroll
    for (int u = 0; u < kInFlight; ++u) {
    const int64_t word = word0 + u * stride;
    if (word - lane >= total_words) { break; }  // warp-uniform: the whole warp is past the end
    const bool valid = word < total_words;
    const uint4 raw = raws[u];
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
    // Fast form: hardware min / max. It differs from the reference's ordered scan only in which zero
    // it keeps when +0 and -0 meet, so a warp in which some group's minimum or maximum is a zero takes
    // the ordered form below instead (rare on real weights; the tests have such groups).
    float mn = fminf(fminf(fminf(v[0], v[1]), fminf(v[2], v[3])), fminf(fminf(v[4], v[5]), fminf(v[6], v[7])));
    float mx = fmaxf(fmaxf(fmaxf(v[0], v[1]), fmaxf(v[2], v[3])), fmaxf(fmaxf(v[4], v[5]), fmaxf(v[6], v[7])));
#pragma unroll
    for (int d = 1; d < TPG; d <<= 1) {
      mn = fminf(mn, __shfl_xor_sync(0xffffffffu, mn, d));
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, d));
    }
    if (__any_sync(0xffffffffu, mn == 0.0f || mx == 0.0f)) {
      mn = __int_as_float(0x7f800000), mx = __int_as_float(0xff800000);
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        mn = (v[i] < mn) ? v[i] : mn;
        mx = (mx < v[i]) ? v[i] : mx;
      }
#pragma unroll
      for (int d = 1; d < TPG; d <<= 1) {
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
    }
    if (clip < 1.0f) {  // one rounding per operator, never contracted
      const float mid = __fmul_rn(0.5f, __fadd_rn(mn, mx));
      mn = __fadd_rn(mid, __fmul_rn(__fsub_rn(mn, mid), clip));
      mx = __fadd_rn(mid, __fmul_rn(__fsub_rn(mx, mid), clip));
    }
    const float scale = __fdiv_rn(__fsub_rn(mx, mn), QMAX);
    const float inv = (scale > 0.0f) ? __fdiv_rn(1.0f, scale) : 0.0f;
    float q[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) { q[i] = round_clamp_f(__fmul_rn(__fsub_rn(v[i], mn), inv), QMAX); }
    uint32_t packed[2];
    if (BITS == 4) {
      packed[0] = pack4_nibbles(q[0], q[1], q[2], q[3]) | (pack4_nibbles(q[4], q[5], q[6], q[7]) << 16);
      packed[1] = 0;
    } else {
      packed[0] = pack4_bytes(q[0], q[1], q[2], q[3]);
      packed[1] = pack4_bytes(q[4], q[5], q[6], q[7]);
    }
    if (!valid) { continue; }
    if (BITS == 4) {
      w[word] = packed[0];
    } else {
      *reinterpret_cast<uint2*>(w + 2 * word) = make_uint2(packed[0], packed[1]);
    }
    if ((word % TPG) == 0) {
      s[word / TPG] = __float2half_rn(scale);
      b[word / TPG] = __float2half_rn(mn);
    }
    }
  }
}

// -------------------------------------------------------------- dequantize
// One thread expands 8 values (one packed word at 4 bits, two at 8) into 8 bf16 (one 16-byte
// store): fully coalesced reads and writes. Replaces affine_dequant_w4g64, _w8g64 and _w8g32
// and affine_dequant_w4g32 (gpu-kernels/metal/quant/affine_dequant.metal:25-58, 69-98, 107-135,
// 191-225).
template <int BITS, int GROUP>
__global__ void __launch_bounds__(256)
affine_dequant_kernel(const uint32_t* __restrict__ w, const uint16_t* __restrict__ scales,
                      const uint16_t* __restrict__ biases, uint4* __restrict__ ydeq,
                      int64_t total_octets) {
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  // kInFlight octets per thread, all loads first: a thread's 4-byte (8-byte) code load is far too
  // little in flight on its own.
  constexpr int kInFlight = BITS == 4 ? 8 : 4;
  for (int64_t oct0 = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; oct0 < total_octets; oct0 += stride * kInFlight) {
    uint2 packed[kInFlight];
    float sc[kInFlight], bi[kInFlight];
#pragma unroll
    for (int u = 0; u < kInFlight; ++u) {
      const int64_t oct = oct0 + u * stride;
      packed[u] = make_uint2(0, 0);
      sc[u] = bi[u] = 0.0f;
      if (oct < total_octets) {
        const int64_t g = oct / (GROUP / 8);
        if (BITS == 4) {
          packed[u].x = __ldg(w + oct);
        } else {
          packed[u] = __ldg(reinterpret_cast<const uint2*>(w) + oct);
        }
        sc[u] = bf16_bits_to_f32(__ldg(scales + g));
        bi[u] = bf16_bits_to_f32(__ldg(biases + g));
      }
    }
#pragma unroll
    for (int u = 0; u < kInFlight; ++u) {
      const int64_t oct = oct0 + u * stride;
      if (oct >= total_octets) { break; }
      uint32_t q[8];
      if (BITS == 4) {
#pragma unroll
        for (int i = 0; i < 8; ++i) { q[i] = (packed[u].x >> (4 * i)) & 0xfu; }
      } else {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          q[i] = (packed[u].x >> (8 * i)) & 0xffu;
          q[4 + i] = (packed[u].y >> (8 * i)) & 0xffu;
        }
      }
      uint32_t o[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        // cvt.rn.bf16x2: the same rounding as the integer form for every finite value
        o[i] = pack_bf16x2(dequant_f32(sc[u], q[2 * i], bi[u]), dequant_f32(sc[u], q[2 * i + 1], bi[u]));
      }
      ydeq[oct] = make_uint4(o[0], o[1], o[2], o[3]);
    }
  }
}

// ---------------------------------------------------------------- requantize 8 -> 4 bits
// Replaces affine_requant_w8_to_w4_g64 (gpu-kernels/metal/quant/affine_dequant.metal:135-189): per
// group of 64, v = s8 * q8 + b8 in f32, scale4 = (max v - min v) / 15, bias4 = min v,
// q4 = clamp(round((v - min) * (1 / scale4)), 0, 15) with the UNROUNDED f32 scale (the stored scale and
// bias are narrowed to the element type afterwards) and round() to nearest, halves away from zero.
// The reference runs one thread per group; here eight lanes share a group (8 values = one 8-byte
// load and one packed output word each, min / max by shuffles), so a warp reads 256 and writes 128
// contiguous bytes. Division and reciprocal are IEEE-rounded here; Metal does not promise that for
// its own, and the reference has no test that pins them.
__global__ void __launch_bounds__(256)
affine_requant_w8_to_w4_g64_kernel(const uint2* __restrict__ w8, const uint16_t* __restrict__ s8,
                                   const uint16_t* __restrict__ b8, uint32_t* __restrict__ w4,
                                   uint16_t* __restrict__ s4, uint16_t* __restrict__ b4, int64_t total_octets) {
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  const int64_t first = (int64_t)blockIdx.x * blockDim.x + (threadIdx.x & ~31);  // the warp's first octet
  constexpr int kInFlight = 4;   // octets per thread whose loads are issued together
  for (int64_t base0 = first; base0 < total_octets; base0 += stride * kInFlight) {
    uint2 packs[kInFlight];
    float ss[kInFlight], bs[kInFlight];
#pragma unroll
    for (int u = 0; u < kInFlight; ++u) {
      const int64_t oct = base0 + u * stride + (threadIdx.x & 31);
      packs[u] = make_uint2(0, 0);
      ss[u] = bs[u] = 0.0f;
      if (oct < total_octets) {
        packs[u] = __ldg(w8 + oct);
        ss[u] = bf16_bits_to_f32(__ldg(s8 + (oct >> 3)));
        bs[u] = bf16_bits_to_f32(__ldg(b8 + (oct >> 3)));
      }
    }
#pragma unroll
    for (int u = 0; u < kInFlight; ++u) {
    const int64_t base = base0 + u * stride;
    if (base >= total_octets) { break; }    // warp-uniform
    const int64_t oct = base + (threadIdx.x & 31);
    const bool live = oct < total_octets;   // whole groups of 8 lanes are live or not
    const int64_t g = oct >> 3;
    float v[8];
    float mn = INFINITY, mx = -INFINITY;
    if (live) {
      const float s = ss[u];
      const float b = bs[u];
      const uint2 packed = packs[u];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        v[i] = dequant_f32(s, (packed.x >> (8 * i)) & 0xffu, b);
        v[4 + i] = dequant_f32(s, (packed.y >> (8 * i)) & 0xffu, b);
      }
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        mn = fminf(mn, v[i]);
        mx = fmaxf(mx, v[i]);
      }
    }
#pragma unroll
    for (int o = 1; o < 8; o <<= 1) {
      mn = fminf(mn, __shfl_xor_sync(0xffffffffu, mn, o));
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    }
    if (live) {
      const float scale = __fdiv_rn(__fsub_rn(mx, mn), 15.0f);
      const float inv = scale > 0.0f ? __fdiv_rn(1.0f, scale) : 0.0f;
      float q[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) { q[i] = round_clamp_f(__fmul_rn(__fsub_rn(v[i], mn), inv), 15.0f); }
      w4[oct] = pack4_nibbles(q[0], q[1], q[2], q[3]) | (pack4_nibbles(q[4], q[5], q[6], q[7]) << 16);
      if ((oct & 7) == 0) {
        s4[g] = (uint16_t)f32_to_bf16_bits(scale);
        b4[g] = (uint16_t)f32_to_bf16_bits(mn);
      }
    }
    }
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

// VEC: eight values per thread and step (two 16-byte loads, one 16-byte store) for 16-byte aligned
// arrays; the last n % 8 values, and unaligned arrays, go one by one. The rounding is the integer form
// in both (bit-exact with the reference for every input, NaNs included).
template <bool VEC>
__global__ void __launch_bounds__(256)
f32_to_bf16_kernel(const float* __restrict__ src, uint16_t* __restrict__ dst, int64_t n) {
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  const int64_t tid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  int64_t done = 0;
  if (VEC) {
    const int64_t octets = n >> 3;
    const float4* s4 = reinterpret_cast<const float4*>(src);
    uint4* d4 = reinterpret_cast<uint4*>(dst);
    for (int64_t o = tid; o < octets; o += stride) {
      const float4 a = __ldg(s4 + 2 * o), b = __ldg(s4 + 2 * o + 1);
      d4[o] = make_uint4(f32_to_bf16_bits(a.x) | (f32_to_bf16_bits(a.y) << 16),
                         f32_to_bf16_bits(a.z) | (f32_to_bf16_bits(a.w) << 16),
                         f32_to_bf16_bits(b.x) | (f32_to_bf16_bits(b.y) << 16),
                         f32_to_bf16_bits(b.z) | (f32_to_bf16_bits(b.w) << 16));
    }
    done = octets << 3;
  }
  for (int64_t i = done + tid; i < n; i += stride) { dst[i] = (uint16_t)f32_to_bf16_bits(src[i]); }
}

static int stream_grid(int64_t items, int threads) {
  const int64_t want = (items + threads - 1) / threads;
  const int64_t cap = (int64_t)num_sms() * 16;  // 16 resident 256-thread CTAs cover a wave
  return (int)(want < 1 ? 1 : (want > cap ? cap : want));
}

}  // namespace vpq

using namespace vpq;

namespace {
template <int BITS, int GROUP>
void launch_quant(bool bf16, const void* w_elt, uint32_t* codes, void* s16, void* b16, int64_t octets, float clip,
                  cudaStream_t st) {
  const int grid = stream_grid(octets, 256);
  if (bf16) {
    affine_quant_kernel<true, BITS, GROUP><<<grid, 256, 0, st>>>(static_cast<const uint16_t*>(w_elt), codes,
                                                                 static_cast<__half*>(s16),
                                                                 static_cast<__half*>(b16), octets, clip);
  } else {
    affine_quant_kernel<false, BITS, GROUP><<<grid, 256, 0, st>>>(static_cast<const uint16_t*>(w_elt), codes,
                                                                  static_cast<__half*>(s16),
                                                                  static_cast<__half*>(b16), octets, clip);
  }
}
bool known_format(int bits, int group) { return (bits == 4 || bits == 8) && (group == 64 || group == 32); }
}  // namespace

extern "C" int vpq_affine_quant(const void* w_elt, int src_is_bf16, uint32_t* codes, void* scales_f16,
                                void* biases_f16, int64_t K, int64_t N, int bits, int group, float clip,
                                void* stream) {
  clear_error();
  if (!w_elt || !codes || !scales_f16 || !biases_f16) {
    return fail(VPQ_ERR_INVALID_ARG, "affine_quant: null pointer");
  }
  if (!known_format(bits, group)) {  // affine-quantizer.cc:55-56
    return fail(VPQ_ERR_UNSUPPORTED, "affine_quant: bits must be 4 or 8 and group 64 or 32 (bits=%d group=%d)", bits,
                group);
  }
  if (N <= 0 || K <= 0 || (K % group) != 0) {  // affine-quantizer.cc:57
    return fail(VPQ_ERR_INVALID_ARG, "affine_quant: need N>0, K>0, K%%%d==0 (K=%lld N=%lld)", group, (long long)K,
                (long long)N);
  }
  if (!aligned16(w_elt) || !aligned16(codes)) {
    return fail(VPQ_ERR_ALIGNMENT, "affine_quant: w_elt and codes must be 16-byte aligned");
  }
  if (int rc = require_sm100()) { return rc; }
  const int64_t octets = N * (K / 8);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const bool bf = src_is_bf16 != 0;
  if (bits == 4 && group == 64) {
    launch_quant<4, 64>(bf, w_elt, codes, scales_f16, biases_f16, octets, clip, st);
  } else if (bits == 8 && group == 64) {
    launch_quant<8, 64>(bf, w_elt, codes, scales_f16, biases_f16, octets, clip, st);
  } else if (bits == 8 && group == 32) {
    launch_quant<8, 32>(bf, w_elt, codes, scales_f16, biases_f16, octets, clip, st);
  } else {
    launch_quant<4, 32>(bf, w_elt, codes, scales_f16, biases_f16, octets, clip, st);
  }
  VPQ_LAUNCH_OK("affine_quant");
  return VPQ_OK;
}

extern "C" int vpq_affine_quant_w4_g64(const void* w_elt, int src_is_bf16, uint32_t* codes,
                                       void* scales_f16, void* biases_f16, int64_t K, int64_t N,
                                       float clip, void* stream) {
  return vpq_affine_quant(w_elt, src_is_bf16, codes, scales_f16, biases_f16, K, N, 4, 64, clip, stream);
}

extern "C" int vpq_affine_dequant_bf16(const uint32_t* w, const void* scales, const void* biases, void* ydeq,
                                       int64_t K, int64_t N, int bits, int group, void* stream) {
  clear_error();
  if (!w || !scales || !biases || !ydeq) { return fail(VPQ_ERR_INVALID_ARG, "affine_dequant: null pointer"); }
  if (!known_format(bits, group)) {
    return fail(VPQ_ERR_UNSUPPORTED, "affine_dequant: bits must be 4 or 8 and group 64 or 32 (bits=%d group=%d)", bits,
                group);
  }
  if (N <= 0 || K <= 0 || (K % group) != 0) {
    return fail(VPQ_ERR_INVALID_ARG, "affine_dequant: need N>0, K>0, K%%%d==0", group);
  }
  if (!aligned16(ydeq) || !aligned16(w)) {
    return fail(VPQ_ERR_ALIGNMENT, "affine_dequant: w and ydeq must be 16-byte aligned");
  }
  if (int rc = require_sm100()) { return rc; }
  const int64_t octets = N * (K / 8);
  const int grid = stream_grid(octets, 256);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const uint16_t* sp = static_cast<const uint16_t*>(scales);
  const uint16_t* bp = static_cast<const uint16_t*>(biases);
  uint4* out = static_cast<uint4*>(ydeq);
  if (bits == 4 && group == 64) {
    affine_dequant_kernel<4, 64><<<grid, 256, 0, st>>>(w, sp, bp, out, octets);
  } else if (bits == 8 && group == 64) {
    affine_dequant_kernel<8, 64><<<grid, 256, 0, st>>>(w, sp, bp, out, octets);
  } else if (bits == 8 && group == 32) {
    affine_dequant_kernel<8, 32><<<grid, 256, 0, st>>>(w, sp, bp, out, octets);
  } else {
    affine_dequant_kernel<4, 32><<<grid, 256, 0, st>>>(w, sp, bp, out, octets);
  }
  VPQ_LAUNCH_OK("affine_dequant");
  return VPQ_OK;
}

extern "C" int vpq_affine_dequant_w4g64_bf16(const uint32_t* w, const void* scales,
                                             const void* biases, void* ydeq, int64_t K, int64_t N,
                                             void* stream) {
  return vpq_affine_dequant_bf16(w, scales, biases, ydeq, K, N, 4, 64, stream);
}

extern "C" int vpq_affine_requant_w8_to_w4_g64_bf16(const uint32_t* w8, const void* s8, const void* b8, uint32_t* w4,
                                                    void* s4, void* b4, int64_t K, int64_t N, void* stream) {
  clear_error();
  if (!w8 || !s8 || !b8 || !w4 || !s4 || !b4) { return fail(VPQ_ERR_INVALID_ARG, "affine_requant_w8_to_w4_g64: null pointer"); }
  if (N <= 0 || K <= 0 || (K % 64) != 0) { return fail(VPQ_ERR_INVALID_ARG, "affine_requant_w8_to_w4_g64: need N>0, K>0, K%%64==0"); }
  if ((reinterpret_cast<uintptr_t>(w8) & 7) || (reinterpret_cast<uintptr_t>(w4) & 3) ||
      (reinterpret_cast<uintptr_t>(s8) & 1) || (reinterpret_cast<uintptr_t>(b8) & 1) ||
      (reinterpret_cast<uintptr_t>(s4) & 1) || (reinterpret_cast<uintptr_t>(b4) & 1)) {
    return fail(VPQ_ERR_ALIGNMENT, "affine_requant_w8_to_w4_g64: w8 must be 8-byte aligned, w4 4-byte, scales and biases 2-byte");
  }
  if (int rc = require_sm100()) { return rc; }
  const int64_t octets = N * (K / 8);
  affine_requant_w8_to_w4_g64_kernel<<<stream_grid(octets, 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      reinterpret_cast<const uint2*>(w8), static_cast<const uint16_t*>(s8), static_cast<const uint16_t*>(b8), w4,
      static_cast<uint16_t*>(s4), static_cast<uint16_t*>(b4), octets);
  VPQ_LAUNCH_OK("affine_requant_w8_to_w4_g64");
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
  if (aligned16(src) && aligned16(dst_bf16) && n >= 8) {
    f32_to_bf16_kernel<true><<<stream_grid(n / 8, 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(
        src, static_cast<uint16_t*>(dst_bf16), n);
  } else {
    f32_to_bf16_kernel<false><<<stream_grid(n, 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(
        src, static_cast<uint16_t*>(dst_bf16), n);
  }
  VPQ_LAUNCH_OK("narrow_f32_bf16");
  return VPQ_OK;
}
