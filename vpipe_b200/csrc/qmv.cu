// qmv.cu -- decode GEMV over 4-bit affine group-64 weights (M = 1 path).
//
// y[m,n] = sum_k x[m,k] * (s[n,k/64] * q[n,k] + b[n,k/64]),  f32 accumulate.
// Replaces affine_qmv_w4g64 (qmv_fast_impl<T,64,4,false,4,2,2>,
// gpu-kernels/metal/quant/affine_qmv.metal:186-301).
//
// The kernel is a pure HBM stream of the packed weights:
//  * each lane reads 16 bytes (32 nibbles, half a quantization group) per row
//    per step with a 128-bit non-allocating load, so a warp covers 1024
//    consecutive k of one row (512 contiguous bytes) per load instruction;
//  * a warp keeps R rows in flight and prefetches the next step's words while
//    it works on the current ones;
//  * nibbles become f32 without a convert instruction: PRMT drops the nibble
//    into mantissa bits 16..19 of 0x43000000, which is the float 128 + q;
//    packed f32x2 FMAs accumulate x*(128+q), and the 128*sum(x) surplus is
//    removed per 32-value chunk with the chunk sums of x that the CTA computes
//    once. Everything is f32: products are exact and the surplus is at most
//    2^7 times a 32-term partial sum, so the result carries f32 rounding noise
//    only (no bf16 / fp16 intermediate anywhere);
//  * x lives in shared memory as f32, transposed so that lane l's 32 values
//    of a step are eight conflict-free 128-bit reads, shared by the R rows;
//  * one shuffle butterfly per row at the end.
// The grid is persistent (2 CTAs per SM); the launch opts into programmatic
// dependent launch so the next GEMV's first weight words are already in
// flight while this one drains.
#include "vpq_common.cuh"

namespace vpq {

namespace {

constexpr int kThreads = 256;
constexpr int kWarps = kThreads / 32;
constexpr int kStepK = 1024;  // k covered by one warp-wide 16-byte load

__device__ __forceinline__ void fma2(float& acc_lo, float& acc_hi, float a_lo, float a_hi,
                                     float b_lo, float b_hi) {
  asm("{\n\t"
      ".reg .b64 ra, rb, rc;\n\t"
      "mov.b64 ra, {%2, %3};\n\t"
      "mov.b64 rb, {%4, %5};\n\t"
      "mov.b64 rc, {%0, %1};\n\t"
      "fma.rn.f32x2 rc, ra, rb, rc;\n\t"
      "mov.b64 {%0, %1}, rc;\n\t"
      "}"
      : "+f"(acc_lo), "+f"(acc_hi)
      : "f"(a_lo), "f"(a_hi), "f"(b_lo), "f"(b_hi));
}

__device__ __forceinline__ float nibble_f32(uint32_t bytes, uint32_t selector) {
  uint32_t r;
  asm("prmt.b32 %0, %1, %2, %3;" : "=r"(r) : "r"(bytes), "r"(0x43000000u), "r"(selector));
  return __uint_as_float(r);  // 128 + q
}

// sum over the 8 nibbles of `word` of x[k] * (128 + q[k]); x0 = k 0..3, x1 = k 4..7
__device__ __forceinline__ void word_fma(uint32_t word, const float4& x0, const float4& x1,
                                         float& acc_lo, float& acc_hi) {
  const uint32_t e = word & 0x0f0f0f0fu;         // nibbles 0,2,4,6 as bytes
  const uint32_t o = (word >> 4) & 0x0f0f0f0fu;  // nibbles 1,3,5,7 as bytes
  fma2(acc_lo, acc_hi, nibble_f32(e, 0x7054u), nibble_f32(o, 0x7054u), x0.x, x0.y);
  fma2(acc_lo, acc_hi, nibble_f32(e, 0x7154u), nibble_f32(o, 0x7154u), x0.z, x0.w);
  fma2(acc_lo, acc_hi, nibble_f32(e, 0x7254u), nibble_f32(o, 0x7254u), x1.x, x1.y);
  fma2(acc_lo, acc_hi, nibble_f32(e, 0x7354u), nibble_f32(o, 0x7354u), x1.z, x1.w);
}

template <int R>
struct Fetch {
  uint4 w[R];
  uint32_t s[R], b[R];
};

template <int R>
__device__ __forceinline__ void fetch(Fetch<R>& f, const uint32_t* __restrict__ w,
                                      const uint16_t* __restrict__ scales,
                                      const uint16_t* __restrict__ biases, int64_t row0, int N,
                                      int K, int step, int lane) {
  const int kk = step * kStepK + lane * 32;
  const bool live = kk < K;
#pragma unroll
  for (int r = 0; r < R; ++r) {
    int64_t row = row0 + r;
    row = row < N ? row : N - 1;  // tail rows re-read the last row; never stored
    if (live) {
      f.w[r] = ldg_stream_v4(w + row * (K >> 3) + (kk >> 3));
      f.s[r] = ldg_nc_u16(scales + row * (K >> 6) + (kk >> 6));
      f.b[r] = ldg_nc_u16(biases + row * (K >> 6) + (kk >> 6));
    } else {
      f.w[r] = make_uint4(0, 0, 0, 0);
      f.s[r] = 0;
      f.b[r] = 0;
    }
  }
}

template <int R>
__global__ void __launch_bounds__(kThreads, 2)
affine_qmv_w4g64_kernel(const uint32_t* __restrict__ w, const uint16_t* __restrict__ scales,
                        const uint16_t* __restrict__ biases, const uint16_t* __restrict__ x,
                        __nv_bfloat16* __restrict__ y, int K, int N, int steps) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  float4* xs = reinterpret_cast<float4*>(smem_raw);                // [steps][8][32] float4
  float* xsum = reinterpret_cast<float*>(xs + (size_t)steps * 256);  // [steps][32]

  const int lane = threadIdx.x & 31;
  const int warp = threadIdx.x >> 5;
  const int m = blockIdx.y;
  const int num_row_blocks = (N + R - 1) / R;
  const int total_warps = gridDim.x * kWarps;
  const int gw = blockIdx.x * kWarps + warp;

  // Let the next kernel in the stream start its own weight prefetch now.
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

  // First weight words: they do not depend on the previous kernel.
  Fetch<R> cur;
  int rb = gw, step = 0;
  const bool have_work = rb < num_row_blocks;
  if (have_work) { fetch<R>(cur, w, scales, biases, (int64_t)rb * R, N, K, 0, lane); }

  // x (and y) may be produced / consumed by the previous kernel.
  asm volatile("griddepcontrol.wait;" ::: "memory");

  // Stage x as f32, transposed: element k = 1024 j + 32 l + 4 i + e lives in
  // xs[(j*8 + i)*32 + l].e ; xsum[j*32 + l] = sum of lane l's 32 values.
  {
    const uint16_t* xr = x + (int64_t)m * K;
    const int chunks = steps * (kStepK / 8);
    for (int t = threadIdx.x; t < chunks; t += kThreads) {
      const int k0 = t * 8;
      uint4 raw = make_uint4(0, 0, 0, 0);
      if (k0 < K) { raw = *reinterpret_cast<const uint4*>(xr + k0); }
      const float4 lo = make_float4(__uint_as_float(raw.x << 16), __uint_as_float(raw.x & 0xffff0000u),
                                    __uint_as_float(raw.y << 16), __uint_as_float(raw.y & 0xffff0000u));
      const float4 hi = make_float4(__uint_as_float(raw.z << 16), __uint_as_float(raw.z & 0xffff0000u),
                                    __uint_as_float(raw.w << 16), __uint_as_float(raw.w & 0xffff0000u));
      const int j = k0 / kStepK, l = (k0 % kStepK) / 32, i0 = (k0 % 32) / 4;
      xs[(j * 8 + i0) * 32 + l] = lo;
      xs[(j * 8 + i0 + 1) * 32 + l] = hi;
      float part = ((lo.x + lo.y) + (lo.z + lo.w)) + ((hi.x + hi.y) + (hi.z + hi.w));
      part += __shfl_xor_sync(0xffffffffu, part, 1);
      part += __shfl_xor_sync(0xffffffffu, part, 2);
      if ((t & 3) == 0) { xsum[j * 32 + l] = part; }
    }
  }
  __syncthreads();

  if (!have_work) { return; }

  float res[R];
#pragma unroll
  for (int r = 0; r < R; ++r) { res[r] = 0.0f; }

  while (true) {
    // prefetch the next (row block, step)
    int nrb = rb, nstep = step + 1;
    if (nstep == steps) {
      nstep = 0;
      nrb = rb + total_warps;
    }
    const bool more = nrb < num_row_blocks;
    Fetch<R> nxt;
    if (more) { fetch<R>(nxt, w, scales, biases, (int64_t)nrb * R, N, K, nstep, lane); }

    // consume the current step
    {
      float acc_lo[R], acc_hi[R];
#pragma unroll
      for (int r = 0; r < R; ++r) { acc_lo[r] = 0.0f, acc_hi[r] = 0.0f; }
      const float4* xp = xs + step * 256 + lane;
#pragma unroll
      for (int wd = 0; wd < 4; ++wd) {
        const float4 x0 = xp[(2 * wd) * 32];
        const float4 x1 = xp[(2 * wd + 1) * 32];
#pragma unroll
        for (int r = 0; r < R; ++r) {
          const uint32_t word = wd == 0 ? cur.w[r].x : wd == 1 ? cur.w[r].y : wd == 2 ? cur.w[r].z : cur.w[r].w;
          word_fma(word, x0, x1, acc_lo[r], acc_hi[r]);
        }
      }
      const float xsc = xsum[step * 32 + lane];
#pragma unroll
      for (int r = 0; r < R; ++r) {
        const float s = bf16_bits_to_f32(cur.s[r]);
        const float b = bf16_bits_to_f32(cur.b[r]);
        const float t = __fmaf_rn(-128.0f, xsc, acc_lo[r] + acc_hi[r]);  // sum x*q over the chunk
        res[r] = __fmaf_rn(s, t, res[r]);
        res[r] = __fmaf_rn(b, xsc, res[r]);
      }
    }

    if (nstep == 0) {  // the row block is complete: reduce over lanes and store
#pragma unroll
      for (int r = 0; r < R; ++r) {
        float v = res[r];
#pragma unroll
        for (int off = 16; off >= 1; off >>= 1) { v += __shfl_xor_sync(0xffffffffu, v, off); }
        const int64_t row = (int64_t)rb * R + r;
        if (lane == 0 && row < N) { y[(int64_t)m * N + row] = __float2bfloat16_rn(v); }
        res[r] = 0.0f;
      }
    }
    if (!more) { break; }
    cur = nxt;
    rb = nrb;
    step = nstep;
  }
}

template <int R>
int launch_qmv(const uint32_t* w, const uint16_t* scales, const uint16_t* biases, const uint16_t* x,
               __nv_bfloat16* y, int K, int N, int M, cudaStream_t st) {
  const int steps = (K + kStepK - 1) / kStepK;
  const size_t smem = (size_t)steps * (256 * sizeof(float4) + 32 * sizeof(float));
  auto kern = affine_qmv_w4g64_kernel<R>;
  if (smem > 48 * 1024) {
    VPQ_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  }
  const int row_blocks = (N + R - 1) / R;
  int ctas = (row_blocks + kWarps - 1) / kWarps;
  const int cap = 2 * num_sms();
  if (ctas > cap) { ctas = cap; }

  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)ctas, (unsigned)M, 1);
  cfg.blockDim = dim3(kThreads, 1, 1);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  VPQ_CUDA_OK(cudaLaunchKernelEx(&cfg, kern, w, scales, biases, x, y, K, N, steps));
  return VPQ_OK;
}

}  // namespace
}  // namespace vpq

using namespace vpq;

extern "C" int vpq_affine_qmv_w4g64_bf16(const uint32_t* w, const void* scales, const void* biases,
                                         const void* x, void* y, int64_t K, int64_t N, int64_t M,
                                         void* stream) {
  clear_error();
  if (!w || !scales || !biases || !x || !y) {
    return fail(VPQ_ERR_INVALID_ARG, "affine_qmv_w4g64: null pointer");
  }
  if (K <= 0 || N <= 0 || M <= 0 || (K % 64) != 0) {
    return fail(VPQ_ERR_INVALID_ARG, "affine_qmv_w4g64: need K>0, N>0, M>0, K%%64==0 (K=%lld N=%lld M=%lld)",
                (long long)K, (long long)N, (long long)M);
  }
  if (K > 32768 || N > (1 << 30) || M > 65535) {
    return fail(VPQ_ERR_UNSUPPORTED, "affine_qmv_w4g64: K<=32768, M<=65535 supported (K=%lld M=%lld)",
                (long long)K, (long long)M);
  }
  if (!aligned16(w) || !aligned16(x) || (reinterpret_cast<uintptr_t>(scales) & 1) ||
      (reinterpret_cast<uintptr_t>(biases) & 1) || (reinterpret_cast<uintptr_t>(y) & 1)) {
    return fail(VPQ_ERR_ALIGNMENT, "affine_qmv_w4g64: w and x must be 16-byte aligned");
  }
  if (int rc = require_sm100()) { return rc; }
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const uint16_t* sc = static_cast<const uint16_t*>(scales);
  const uint16_t* bi = static_cast<const uint16_t*>(biases);
  const uint16_t* xx = static_cast<const uint16_t*>(x);
  __nv_bfloat16* yy = static_cast<__nv_bfloat16*>(y);
  // Rows per warp: more rows share each x read; fewer rows spread a small
  // matrix over more warps.
  if (N >= 8192) { return launch_qmv<4>(w, sc, bi, xx, yy, (int)K, (int)N, (int)M, st); }
  if (N >= 2048) { return launch_qmv<2>(w, sc, bi, xx, yy, (int)K, (int)N, (int)M, st); }
  return launch_qmv<1>(w, sc, bi, xx, yy, (int)K, (int)N, (int)M, st);
}

extern "C" int vpq_affine_qmv_w4g64_bf16_batch(const vpq_linear_desc* d, int count, void* stream) {
  clear_error();
  if (!d || count <= 0) { return fail(VPQ_ERR_INVALID_ARG, "affine_qmv_w4g64_batch: null or empty set"); }
  for (int i = 0; i < count; ++i) {
    if (int rc = vpq_affine_qmv_w4g64_bf16(d[i].w, d[i].scales, d[i].biases, d[i].x, d[i].y, d[i].K,
                                           d[i].N, d[i].M, stream)) {
      return rc;
    }
  }
  return VPQ_OK;
}
