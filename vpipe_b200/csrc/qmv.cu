// qmv.cu -- decode GEMV over 4-bit affine group-64 weights (M = 1 path).
//
// y[m,n] = sum_k x[m,k] * (s[n,k/64] * q[n,k] + b[n,k/64]),  f32 accumulate.
// Replaces affine_qmv_w4g64 (qmv_fast_impl<T,64,4,false,4,2,2>,
// gpu-kernels/metal/quant/affine_qmv.metal:186-301).
//
// The kernel is a stream of the packed weights out of HBM; everything else is
// arranged so that the SM keeps up with 23 bytes (46 nibbles) per clock:
//  * a CTA owns tiles of 16 output rows and its 8 warps split K (warp w takes
//    a contiguous run of 128-wide k tiles), so even a 4096 x 4096 matrix gives
//    every warp work and all loads of a warp are independent;
//  * lane (g, t) of a warp reads 16 bytes of row g and 16 bytes of row g+8 per
//    k tile (a quad covers 64 contiguous bytes of a row) with 128-bit
//    non-allocating loads; four k tiles (8 loads per lane) are kept in flight;
//  * nibbles are widened in registers to bf16 128+q with one LOP3 per two
//    nibbles (0x4300 | q is exactly 128 + q) and fed, unscaled, to
//    mma.sync.m16n8k16 against x; products are exact and the accumulation is
//    f32. A first SIMT version of this kernel (one PRMT and half an f32x2 FMA
//    per nibble) was bound by the integer pipe at under a quarter of the HBM
//    rate; the tensor-core form needs about a third of the instructions;
//  * the two quantization groups of a k tile go to different accumulator
//    columns (even columns see only the first 64 k of x, odd columns the last
//    64), so each group's sum comes out separately and is scaled once:
//    res += s * (acc - 128 * sum(x_group)) + b * sum(x_group), in f32;
//  * x is staged once per CTA in shared memory, already permuted into the
//    B-fragment order that matches the nibble pairing (k, k+4);
//  * per row tile: one shuffle, one shared-memory reduction over the 8 warps.
// The launch opts into programmatic dependent launch: the first weight loads
// are issued before griddepcontrol.wait, so the next GEMV's stream starts
// while this one drains.
#include "vpq_common.cuh"

namespace vpq {

namespace {

constexpr int kThreads = 256;
constexpr int kWarps = kThreads / 32;
constexpr int kSlots = 6;     // k tiles in flight per warp
constexpr int kTileK = 128;   // k per tile: 64 bytes of a row, two quantization groups

struct Slot {
  uint4 ra, rb;     // 32 nibbles of row g and of row g+8
  uint32_t s, z;    // scale and bias (bf16 bits) of this lane's (row, group) item
};

__device__ __forceinline__ void mma_bf16_16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2,
                                               uint32_t a3, uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 "
      "{%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// (v & 0x000f000f) | 0x43004300 in one LOP3: the bf16 pair (128 + lo nibble, 128 + hi nibble)
__device__ __forceinline__ uint32_t and_or_magic(uint32_t v) {
  uint32_t r;
  asm("lop3.b32 %0, %1, 0x000f000f, 0x43004300, 0xEA;" : "=r"(r) : "r"(v));
  return r;
}

// 8 MMAs of one k tile: rows g / g+8 words wa / wb against the staged x fragments
__device__ __forceinline__ void unit_mma(float (&c)[4], float (&d)[4], const uint4& ra, const uint4& rb,
                                         const uint4* __restrict__ xb, int xb_q) {
  const uint32_t wa[4] = {ra.x, ra.y, ra.z, ra.w};
  const uint32_t wb[4] = {rb.x, rb.y, rb.z, rb.w};
#pragma unroll
  for (int wd = 0; wd < 4; ++wd) {
    const uint4 xv = xb[wd * xb_q];
    const uint32_t a = wa[wd], b = wb[wd];
    // nibble pairs (n0,n4) (n1,n5) (n2,n6) (n3,n7) of each word
    mma_bf16_16816(c, and_or_magic(a), and_or_magic(b), and_or_magic(a >> 4), and_or_magic(b >> 4),
                   xv.x, xv.y);
    mma_bf16_16816(d, and_or_magic(a >> 8), and_or_magic(b >> 8), and_or_magic(a >> 12),
                   and_or_magic(b >> 12), xv.z, xv.w);  // second accumulator: two shorter dependency chains
  }
}

__global__ void __launch_bounds__(kThreads, 2)
affine_qmv_w4g64_kernel(const uint32_t* __restrict__ w, const uint16_t* __restrict__ scales,
                        const uint16_t* __restrict__ biases, const uint16_t* __restrict__ x,
                        __nv_bfloat16* __restrict__ y, int K, int N) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  const int KT = (K + kTileK - 1) / kTileK;  // k tiles (the last may hold one group only)
  const int G = K >> 6;                      // groups per row
  const int KW = K >> 3;                     // packed words per row
  uint4* xperm = reinterpret_cast<uint4*>(smem_raw);            // [KT][4 quarters][4 t] x 16 B
  uint4* zero16 = xperm + (size_t)KT * 16;                      // 16 bytes of zeros
  float* xg = reinterpret_cast<float*>(zero16 + 1);             // [2*KT] group sums of x
  float* red = xg + 2 * KT;                                     // [2][kWarps][16]

  const int lane = threadIdx.x & 31;
  const int warp = threadIdx.x >> 5;
  const int g = lane >> 2, t = lane & 3;
  const int m = blockIdx.y;
  const int row_tiles = (N + 15) >> 4;
  // this warp's contiguous run of k tiles: [kt0, kt0 + n_kt)
  const int n_kt = KT / kWarps + (warp < KT % kWarps ? 1 : 0);
  const int kt0 = warp * (KT / kWarps) + min(warp, KT % kWarps);
  const int item_row = g + ((t >> 1) << 3);  // the row whose (group t&1) sum this lane scales
  const int my_tiles = blockIdx.x < row_tiles ? (row_tiles - blockIdx.x + gridDim.x - 1) / gridDim.x : 0;
  const int total_units = my_tiles * n_kt;

  // Let the next kernel in the stream start its own weight prefetch now.
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

  // ---- fetch side: walks the units (row tile, k tile) in the order they are consumed.
  // Offsets past the end of a row (K % 128 == 64) or of the matrix (N % 16 != 0) are clamped
  // onto valid data; what they fetch meets x == 0 or is never stored.
  const uint32_t* f_pa = w;
  const uint32_t* f_pb = w;
  const uint16_t* f_ps = scales;
  const uint16_t* f_pz = biases;
  int f_tile = blockIdx.x, f_i = 0, f_units = 0;
  auto fetch_tile_setup = [&]() {
    const int r0 = f_tile << 4;
    f_pa = w + (int64_t)min(r0 + g, N - 1) * KW;
    f_pb = w + (int64_t)min(r0 + g + 8, N - 1) * KW;
    const int64_t ri = min(r0 + item_row, N - 1);
    f_ps = scales + ri * G;
    f_pz = biases + ri * G;
  };
  auto fetch = [&](Slot& sl) {
    if (f_units < total_units) {
      const int kt = kt0 + f_i;
      const int woff = min(kt * 16 + t * 4, KW - 4);
      const int goff = min(2 * kt + (t & 1), G - 1);
      sl.ra = ldg_stream_v4(f_pa + woff);
      sl.rb = ldg_stream_v4(f_pb + woff);
      sl.s = ldg_nc_u16(f_ps + goff);
      sl.z = ldg_nc_u16(f_pz + goff);
      ++f_units;
      if (++f_i == n_kt) {
        f_i = 0;
        f_tile += gridDim.x;
        fetch_tile_setup();
      }
    }
  };

  // First weight words: they do not depend on the previous kernel.
  Slot slot[kSlots];
  fetch_tile_setup();
#pragma unroll
  for (int j = 0; j < kSlots; ++j) { fetch(slot[j]); }

  // x (and y) may be produced / consumed by the previous kernel.
  asm volatile("griddepcontrol.wait;" ::: "memory");

  // ---- stage x: 8 consecutive values (x0..x7) become the four B-fragment
  // registers (x0,x4) (x1,x5) (x2,x6) (x3,x7); group sums in f32.
  {
    const uint16_t* xr = x + (int64_t)m * K;
    const int chunks = KT * 16;  // 16-byte chunks of the padded x
    // warp-uniform bound: every lane takes part in the shuffles below
    for (int i = threadIdx.x; i - lane < chunks; i += kThreads) {
      const bool live = i < chunks;
      const int k0 = i * 8;
      uint4 in = make_uint4(0, 0, 0, 0);
      if (live && k0 < K) { in = *reinterpret_cast<const uint4*>(xr + k0); }
      uint4 out;
      asm("prmt.b32 %0, %1, %2, 0x5410;" : "=r"(out.x) : "r"(in.x), "r"(in.z));
      asm("prmt.b32 %0, %1, %2, 0x7632;" : "=r"(out.y) : "r"(in.x), "r"(in.z));
      asm("prmt.b32 %0, %1, %2, 0x5410;" : "=r"(out.z) : "r"(in.y), "r"(in.w));
      asm("prmt.b32 %0, %1, %2, 0x7632;" : "=r"(out.w) : "r"(in.y), "r"(in.w));
      const int kt = i >> 4, tt = (i >> 2) & 3, q = i & 3;
      if (live) { xperm[(kt * 4 + q) * 4 + tt] = out; }
      float part = ((bf16_bits_to_f32(in.x & 0xffffu) + __uint_as_float(in.x & 0xffff0000u)) +
                    (bf16_bits_to_f32(in.y & 0xffffu) + __uint_as_float(in.y & 0xffff0000u))) +
                   ((bf16_bits_to_f32(in.z & 0xffffu) + __uint_as_float(in.z & 0xffff0000u)) +
                    (bf16_bits_to_f32(in.w & 0xffffu) + __uint_as_float(in.w & 0xffff0000u)));
      part += __shfl_xor_sync(0xffffffffu, part, 1);
      part += __shfl_xor_sync(0xffffffffu, part, 2);
      part += __shfl_xor_sync(0xffffffffu, part, 4);
      if (live && (i & 7) == 0) { xg[i >> 3] = part; }
    }
    if (threadIdx.x == 0) { *zero16 = make_uint4(0, 0, 0, 0); }
  }
  __syncthreads();

  // Even accumulator columns see the first group of a k tile (chunks t = 0, 1),
  // odd columns the second (t = 2, 3); column c is supplied by the lanes with g == c.
  const bool real = ((g & 1) == 0) ? (t < 2) : (t >= 2);
  const uint4* xb_base = real ? xperm + t : zero16;
  const int xb_kt = real ? 16 : 0, xb_q = real ? 4 : 0;

  // ---- consume side
  int buf = 0, c_i = 0, tile = blockIdx.x;
  float res = 0.0f;
  auto finish_tile = [&]() {  // both groups of a row, then the 8 warps' K slices
    res += __shfl_xor_sync(0xffffffffu, res, 1);
    if ((t & 1) == 0) { red[(buf * kWarps + warp) * 16 + item_row] = res; }
    __syncthreads();
    if (warp == 0 && lane < 16) {
      float v = 0.0f;
#pragma unroll
      for (int ww = 0; ww < kWarps; ++ww) { v += red[(buf * kWarps + ww) * 16 + lane]; }
      const int row = (tile << 4) + lane;
      if (row < N) { y[(int64_t)m * N + row] = __float2bfloat16_rn(v); }
    }
    buf ^= 1;
    res = 0.0f;
    tile += gridDim.x;
  };

  if (n_kt == 0) {  // K < 1024: this warp holds no k tile but still joins every reduction
    for (int i = 0; i < my_tiles; ++i) { finish_tile(); }
    return;
  }

  for (int u = 0; u < total_units; u += kSlots) {
#pragma unroll
    for (int j = 0; j < kSlots; ++j) {
      if (u + j < total_units) {
        const int kt = kt0 + c_i;
        float c[4] = {0.0f, 0.0f, 0.0f, 0.0f}, d[4] = {0.0f, 0.0f, 0.0f, 0.0f};
        unit_mma(c, d, slot[j].ra, slot[j].rb, xb_base + kt * xb_kt, xb_q);
        // c0 = (row g, first group) c1 = (row g, second) c2 = (row g+8, first) c3 = (row g+8, second)
        const float val = t == 0 ? c[0] + d[0] : t == 1 ? c[1] + d[1] : t == 2 ? c[2] + d[2] : c[3] + d[3];
        const float xs = xg[2 * kt + (t & 1)];
        res = __fmaf_rn(bf16_bits_to_f32(slot[j].s), __fmaf_rn(-128.0f, xs, val), res);
        res = __fmaf_rn(bf16_bits_to_f32(slot[j].z), xs, res);
        fetch(slot[j]);  // refill with the unit four ahead
        if (++c_i == n_kt) {
          c_i = 0;
          finish_tile();
        }
      }
    }
  }
}

int launch_qmv(const uint32_t* w, const uint16_t* scales, const uint16_t* biases, const uint16_t* x,
               __nv_bfloat16* y, int K, int N, int M, cudaStream_t st) {
  const int KT = (K + kTileK - 1) / kTileK;
  const size_t smem = (size_t)KT * 256 + 16 + (size_t)2 * KT * sizeof(float) + 2 * kWarps * 16 * sizeof(float);
  auto kern = affine_qmv_w4g64_kernel;
  if (smem > 48 * 1024) {
    VPQ_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  }
  const int row_tiles = (N + 15) / 16;
  const int cap = 2 * num_sms();
  const int ctas = row_tiles < cap ? row_tiles : cap;

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
  VPQ_CUDA_OK(cudaLaunchKernelEx(&cfg, kern, w, scales, biases, x, y, K, N));
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
  return launch_qmv(w, sc, bi, xx, yy, (int)K, (int)N, (int)M, st);
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
