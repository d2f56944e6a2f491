// qmv.cu -- decode GEMV over 4-bit affine group-64 weights (M = 1 path).
//
// y[m,n] = sum_k x[m,k] * (s[n,k/64] * q[n,k] + b[n,k/64]),  f32 accumulate.
// Replaces affine_qmv_w4g64 (qmv_fast_impl<T,64,4,false,4,2,2>,
// gpu-kernels/metal/quant/affine_qmv.metal:186-301).
//
// The kernel is a stream of the packed weights out of HBM; everything else is
// arranged so that an SM keeps up with 23 bytes (46 nibbles) per clock:
//  * the weights never pass through the load/store unit: a producer warp
//    streams them with TMA, as [16 rows x 128 bytes] boxes (128-byte swizzle),
//    into a ring of 16 KB stages (16 rows x 2048 k, plus that span's scales and
//    biases), so up to ~190 KB per SM are in flight with no register cost.
//    Two earlier versions that loaded nibbles with per-lane 128-bit loads
//    saturated near 2.5 TB/s, stalled on outstanding L1 requests;
//  * a CTA owns tiles of 16 output rows; consumer warp w of 8 takes box w of
//    every stage (two 128-wide k tiles), so K is split across the warps;
//  * lane (g, t) reads 16 bytes of two rows per k tile from the stage
//    (conflict-free through the swizzle), widens the nibbles in registers to
//    bf16 128+q with one LOP3 per two nibbles (0x4300 | q is exactly 128 + q)
//    and feeds them, unscaled, to mma.sync.m16n8k16 against x; products are
//    exact and the accumulation is f32. A first SIMT version (one PRMT and half
//    an f32x2 FMA per nibble) was bound by the integer pipe;
//  * the two quantization groups of a k tile go to different accumulator
//    columns (even columns see only the first 64 k of x, odd columns the last
//    64), so each group's sum comes out separately and is scaled once:
//    res += s * (acc - 128 * sum(x_group)) + b * sum(x_group), in f32;
//  * x is staged once per CTA in shared memory, already permuted into the
//    B-fragment order that matches the nibble pairing (k, k+4);
//  * per row tile: one shuffle, one shared-memory reduction over the 8 warps.
// One launch can run a whole list of GEMVs (a "plan"): the CTAs walk the concatenated row tiles
// of all problems, the producer keeps streaming across problem boundaries, and the consumers
// re-stage x only when the next problem reads a different x. A single GEMV is a one-problem list
// passed in the kernel parameters.
// The launch opts into programmatic dependent launch: the producer starts
// streaming weights before griddepcontrol.wait, so the next launch's stream is
// already running while this one drains. Every barrier wait is bounded.
#include "vpq_sm100.cuh"

#include <cstdlib>
#include <cstring>

namespace vpq {

// 0, or (site << 8) | role of the first bounded wait that gave up in this kernel.
__device__ uint32_t g_qmv_status;

namespace {

constexpr int kConsWarps = 8;
constexpr int kConsThreads = kConsWarps * 32;
constexpr int kThreads = kConsThreads + 32;  // + producer warp
constexpr int kTileK = 128;                  // k per MMA unit: 64 bytes of a row, two groups
constexpr int kBoxBytes = 16 * 128;          // one TMA box: 16 rows x 128 bytes (256 k)
constexpr int kBoxesPerStage = 8;            // a stage spans 2048 k
constexpr int kStageW = kBoxesPerStage * kBoxBytes;  // 16 KB of nibbles
constexpr int kStageSZ = 2 * 16 * 64;        // scales + biases of the span: 2 x [16 rows x 32 groups]
constexpr int kMaxStages = 6;
constexpr int kRedSlots = 8;                 // row tiles whose cross-warp sums may be pending

// D = A * B + C on fp16 operands, f32 accumulate.
__device__ __forceinline__ void mma_f16_16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2,
                                              uint32_t a3, uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 "
      "{%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// D = A * B: starts an accumulator chain without first clearing four registers.
__device__ __forceinline__ void mma_f16_16816_first(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2,
                                                    uint32_t a3, uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 "
      "{%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
      : "=f"(c[0]), "=f"(c[1]), "=f"(c[2]), "=f"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "f"(0.0f));
}

// fp16 pairs straight out of a packed word, one LOP3 each:
//   lo_magic(v) = (v & 0x000f000f) | 0x64006400 -> (1024 + nibble 0, 1024 + nibble 4) of v
//   hi_magic(v) = (v & 0x00f000f0) | 0x54005400 -> (  64 + nibble 1,   64 + nibble 5) of v
__device__ __forceinline__ uint32_t lo_magic(uint32_t v) {
  uint32_t r;
  asm("lop3.b32 %0, %1, 0x000f000f, 0x64006400, 0xEA;" : "=r"(r) : "r"(v));
  return r;
}
__device__ __forceinline__ uint32_t hi_magic(uint32_t v) {
  uint32_t r;
  asm("lop3.b32 %0, %1, 0x00f000f0, 0x54005400, 0xEA;" : "=r"(r) : "r"(v));
  return r;
}

enum : uint32_t { kRoleProducer = 1, kRoleConsumer = 2 };

// One GEMV of a launch. Lives in the kernel parameters (single GEMV) or in caller-provided
// device memory (plan). Tensor maps need 64-byte alignment.
struct alignas(64) QmvProblem {
  CUtensorMap mw, ms, mz;      // packed weights [N, K/8] u32; scales, biases [N, K/64] (valid if scales_tma)
  const uint16_t* scales;
  const uint16_t* biases;
  const uint16_t* x;           // one row of K bf16
  __nv_bfloat16* y;            // N outputs
  int K, N;
  int tile_begin, row_tiles;   // this problem's range in the launch's global list of 16-row tiles
  int scales_tma;              // scale / bias rows are TMA boxes (pitch and base 16-byte aligned)
  int pad[3];
};
static_assert(sizeof(QmvProblem) % 64 == 0, "problem records are laid out back to back");

__global__ void __launch_bounds__(kThreads, 2)
affine_qmv_w4g64_kernel(const __grid_constant__ QmvProblem single, const QmvProblem* __restrict__ list,
                        int total_tiles, int stages, int cap_kt) {
  extern __shared__ unsigned char smem_dyn[];
  const uint32_t raw = smem_u32(smem_dyn);
  const uint32_t base = (raw + 1023u) & ~1023u;  // swizzled boxes need 1024-byte alignment
  unsigned char* base_ptr = smem_dyn + (base - raw);
  constexpr int kStageBytes = kStageW + kStageSZ;
  const QmvProblem* probs = list ? list : &single;

  unsigned char* p0 = base_ptr + (size_t)stages * kStageBytes;
  uint4* xperm = reinterpret_cast<uint4*>(p0);                   // [cap_kt][4 quarters][4 t] x 16 B
  uint4* zero256 = xperm + (size_t)cap_kt * 16;                  // 320 bytes of zeros
  float2* xg = reinterpret_cast<float2*>(zero256 + 20);          // [2*cap_kt] per group: surplus, sum of x
  float* red = reinterpret_cast<float*>(xg + 2 * cap_kt);        // [kRedSlots][kConsWarps][16]
  uint32_t* red_cnt = reinterpret_cast<uint32_t*>(red + kRedSlots * kConsWarps * 16);  // [kRedSlots]
  uint32_t* amax_buf = red_cnt + kRedSlots;                      // [kConsWarps]
  uint64_t* bars = reinterpret_cast<uint64_t*>(amax_buf + kConsWarps);
  volatile uint32_t* abort_flag = reinterpret_cast<volatile uint32_t*>(bars + 2 * kMaxStages);
  const uint32_t bar0 = smem_u32(bars);
  auto bar_full = [&](int s) { return bar0 + 8u * s; };
  auto bar_empty = [&](int s) { return bar0 + 8u * (kMaxStages + s); };

  const int lane = threadIdx.x & 31;
  const int warp = threadIdx.x >> 5;

  // Let the next kernel in the stream start its own weight stream now.
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

  if (threadIdx.x == 0) {
    for (int s = 0; s < stages; ++s) {
      mbar_init(bar_full(s), 1);
      mbar_init(bar_empty(s), kConsWarps);
    }
    *abort_flag = 0;
    for (int i = 0; i < kRedSlots; ++i) { red_cnt[i] = 0; }
    fence_mbar_init();
  }
  if (threadIdx.x < 20) { zero256[threadIdx.x] = make_uint4(0, 0, 0, 0); }
  __syncthreads();

  if (warp == kConsWarps) {
    // ------------------------------------------------------------ producer
    // Weights, scales and biases are constants of the model: streaming them
    // does not wait for the previous kernel.
    if (lane == 0) {
      uint32_t it = 0;
      bool ok = true;
      int pi = 0;
      const QmvProblem* P = probs;
      int tb = P->tile_begin, rt = P->row_tiles;
      for (int gt = blockIdx.x; gt < total_tiles && ok; gt += gridDim.x) {
        while (gt >= tb + rt) {
          P = probs + (++pi);
          tb = P->tile_begin;
          rt = P->row_tiles;
        }
        const int tile = gt - tb;
        const int NB = (P->K + 255) >> 8;                              // 128-byte boxes per row
        const int SPT = (NB + kBoxesPerStage - 1) / kBoxesPerStage;    // stages per row tile
        const bool sz_tma = P->scales_tma != 0;
        for (int st = 0; st < SPT; ++st, ++it) {
          const int s = it % stages;
          const uint32_t ph = (it / stages) & 1u;
          if (!mbar_wait(bar_empty(s), ph ^ 1u, (1u << 8) | kRoleProducer, abort_flag, &g_qmv_status)) {
            ok = false;
            break;
          }
          const int nb = min(kBoxesPerStage, NB - st * kBoxesPerStage);
          const uint32_t dst = base + (uint32_t)s * kStageBytes;
          mbar_expect_tx(bar_full(s), (uint32_t)nb * kBoxBytes + (sz_tma ? kStageSZ : 0));
          for (int b = 0; b < nb; ++b) {
            tma_load_2d(dst + b * kBoxBytes, &P->mw, bar_full(s), (st * kBoxesPerStage + b) * 32, tile * 16);
          }
          if (sz_tma) {
            tma_load_2d(dst + kStageW, &P->ms, bar_full(s), st * 32, tile * 16);
            tma_load_2d(dst + kStageW + kStageSZ / 2, &P->mz, bar_full(s), st * 32, tile * 16);
          }
        }
      }
      // Never leave with a copy still in flight: wait for the last load of every stage.
      for (int s = 0; s < stages; ++s) {
        if (it > (uint32_t)s) {
          const uint32_t last = ((it - 1 - s) / stages) * stages + s;
          mbar_wait(bar_full(s), (last / stages) & 1u, (2u << 8) | kRoleProducer, abort_flag, &g_qmv_status);
        }
      }
    }
    return;
  }

  // ---------------------------------------------------------------- consumers
  const int g = lane >> 2, t = lane & 3;
  const int rho = (g >> 1) | ((g & 1) << 2);  // stage row of MMA row g (g+8 -> rho+8): bank-conflict-free
  const int item_row = rho + ((t >> 1) << 3); // the row whose (group t&1) sum this lane scales
  const int par = t & 1;

  // x (and y) may be produced / consumed by the previous kernel.
  asm volatile("griddepcontrol.wait;" ::: "memory");

  // ---- staging of one x vector as fp16 (called by all consumer warps together).
  // The tensor-core operands are fp16: a nibble sits in the low mantissa bits of 0x6400 (1024 + q)
  // or, one nibble higher, of 0x5400 (64 + q), so no shift is needed for half of them. x is scaled
  // by a power of two so that its largest magnitude lands in [2^14, 2^15): every bf16 value within
  // 2^-28 of the maximum is then exact in fp16, and the scale is undone exactly at the end.
  // 8 consecutive values (x0..x7) become the four B-fragment registers (x0,x4) (x1,x5) (x2,x6)
  // (x3,x7). Per group of 64: xg[].x = 1024 * sum(even k) + 64 * sum(odd k), the surplus the
  // magic constants add to the accumulator; xg[].y = sum of all 64, for the bias term.
  constexpr int kXRegs = 8;  // chunks a thread keeps in registers between the two passes
  auto stage_x = [&](const uint16_t* xr, int K, int KT) -> float {
    const int chunks = KT * 16;  // 16-byte chunks of the padded x
    uint4 xin[kXRegs];
    uint32_t amax = 0;  // largest |x| as bf16 bits (ordering of magnitudes == ordering of bit patterns)
#pragma unroll
    for (int r = 0; r < kXRegs; ++r) {
      const int i = threadIdx.x + r * kConsThreads;
      xin[r] = make_uint4(0, 0, 0, 0);
      if (i * 8 < K) { xin[r] = *reinterpret_cast<const uint4*>(xr + i * 8); }
    }
#pragma unroll
    for (int r = 0; r < kXRegs; ++r) {
      const uint32_t v[4] = {xin[r].x, xin[r].y, xin[r].z, xin[r].w};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        amax = max(amax, v[j] & 0x7fffu);
        amax = max(amax, (v[j] >> 16) & 0x7fffu);
      }
    }
    for (int i = threadIdx.x + kXRegs * kConsThreads; i * 8 < K; i += kConsThreads) {
      const uint4 in = *reinterpret_cast<const uint4*>(xr + i * 8);
      const uint32_t v[4] = {in.x, in.y, in.z, in.w};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        amax = max(amax, v[j] & 0x7fffu);
        amax = max(amax, (v[j] >> 16) & 0x7fffu);
      }
    }
    amax = __reduce_max_sync(0xffffffffu, amax);
    // the barrier also orders the previous problem's last reads of xperm / xg before the writes below
    if (lane == 0) { amax_buf[warp] = amax; }
    asm volatile("bar.sync 1, %0;" ::"n"(kConsThreads) : "memory");  // consumers only
    amax = 0;
#pragma unroll
    for (int ww = 0; ww < kConsWarps; ++ww) { amax = max(amax, amax_buf[ww]); }
    int e = (int)(amax >> 7);            // biased exponent of the largest magnitude
    e = min(max(e, 16), 240);            // all-zero / denormal / huge x: keep both factors normal
    const float x_scale = __uint_as_float((uint32_t)(268 - e) << 23);  // 2^(141 - e): max |x| -> [2^14, 2^15)
    const float x_unscale = __uint_as_float((uint32_t)(e - 14) << 23); // its exact inverse
    auto convert_chunk = [&](int i, const uint4& in) {  // called by whole warps: shuffles inside
      const bool live = i < chunks;
      const uint32_t v[4] = {in.x, in.y, in.z, in.w};
      uint32_t hb[4];
      float se = 0.0f, so = 0.0f;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const __half2 h = __floats2half2_rn(__uint_as_float(v[j] << 16) * x_scale,
                                            __uint_as_float(v[j] & 0xffff0000u) * x_scale);
        const float2 f = __half22float2(h);  // what the tensor core will see
        se += f.x;
        so += f.y;
        hb[j] = *reinterpret_cast<const uint32_t*>(&h);
      }
      uint4 out;
      asm("prmt.b32 %0, %1, %2, 0x5410;" : "=r"(out.x) : "r"(hb[0]), "r"(hb[2]));
      asm("prmt.b32 %0, %1, %2, 0x7632;" : "=r"(out.y) : "r"(hb[0]), "r"(hb[2]));
      asm("prmt.b32 %0, %1, %2, 0x5410;" : "=r"(out.z) : "r"(hb[1]), "r"(hb[3]));
      asm("prmt.b32 %0, %1, %2, 0x7632;" : "=r"(out.w) : "r"(hb[1]), "r"(hb[3]));
      const int kt = i >> 4, tt = (i >> 2) & 3, q = i & 3;
      if (live) { xperm[(kt * 4 + q) * 4 + tt] = out; }
#pragma unroll
      for (int off = 1; off < 8; off <<= 1) {
        se += __shfl_xor_sync(0xffffffffu, se, off);
        so += __shfl_xor_sync(0xffffffffu, so, off);
      }
      if (live && (i & 7) == 0) { xg[i >> 3] = make_float2(__fmaf_rn(1024.0f, se, 64.0f * so), se + so); }
    };
#pragma unroll
    for (int r = 0; r < kXRegs; ++r) {
      const int i = threadIdx.x + r * kConsThreads;
      if (i - lane < chunks) { convert_chunk(i, xin[r]); }  // warp-uniform
    }
    for (int i = threadIdx.x + kXRegs * kConsThreads; i - lane < chunks; i += kConsThreads) {
      uint4 in = make_uint4(0, 0, 0, 0);
      if (i * 8 < K) { in = *reinterpret_cast<const uint4*>(xr + i * 8); }
      convert_chunk(i, in);
    }
    asm volatile("bar.sync 1, %0;" ::"n"(kConsThreads) : "memory");
    return x_unscale;
  };

  // Even accumulator columns see the first group of a k tile (chunks t = 0, 1),
  // odd columns the second (t = 2, 3); column c is supplied by the lanes with g == c.
  // The other lanes read zeros from a block laid out like one k tile of xperm
  // (+4: quarter q of the zero block sits in the banks quarter q+1 of the data uses, so the two
  // halves of a warp never collide).
  const bool real = ((g & 1) == 0) ? (t < 2) : (t >= 2);
  const uint4* xb_base = real ? xperm + t : zero256 + 4;
  const int xb_kt = real ? 16 : 0;

  // byte offsets of this lane's two 16-byte reads inside its box, per half (k tile) of the box
  const uint32_t off_h0 = (uint32_t)rho * 128u + (uint32_t)(((0 + t) ^ rho) << 4);
  const uint32_t off_h1 = (uint32_t)rho * 128u + (uint32_t)(((4 + t) ^ rho) << 4);
  const uint32_t sz_off = (uint32_t)kStageW + (uint32_t)item_row * 64u + (uint32_t)warp * 8u;
  const uint32_t sel = par ? 0x3244u : 0x1044u;  // PRMT: this lane's bf16 of a pair -> f32 bits

  uint32_t tile_seq = 0, ph = 0;
  int s = 0;
  bool ok = true;
  int pi = 0;
  const QmvProblem* P = probs;
  int tb = P->tile_begin, rt = P->row_tiles;
  const uint16_t* staged_x = nullptr;
  int staged_K = -1;
  float x_unscale = 1.0f;
  // per-problem values, refreshed when the walk enters a new problem
  int K = 0, N = 0, G = 0, KT = 0, SPT = 0;
  bool sz_tma = false;
  const uint16_t* scales = nullptr;
  const uint16_t* biases = nullptr;
  __nv_bfloat16* y = nullptr;
  bool fresh = true;
  for (int gt = blockIdx.x; gt < total_tiles && ok; gt += gridDim.x, ++tile_seq) {
    while (gt >= tb + rt) {
      P = probs + (++pi);
      tb = P->tile_begin;
      rt = P->row_tiles;
      fresh = true;
    }
    if (fresh) {
      fresh = false;
      K = P->K;
      N = P->N;
      G = K >> 6;
      KT = ((K + 255) >> 8) * 2;  // k tiles per row, padded to whole 256-k boxes (x is zero there)
      SPT = (((K + 255) >> 8) + kBoxesPerStage - 1) / kBoxesPerStage;
      sz_tma = P->scales_tma != 0;
      scales = P->scales;
      biases = P->biases;
      y = P->y;
      const uint16_t* xr = P->x;
      if (xr != staged_x || K != staged_K) {  // q|k|v or gate|up of a layer share one staging
        x_unscale = stage_x(xr, K, KT);
        staged_x = xr;
        staged_K = K;
      }
    }
    const int tile = gt - tb;
    float res = 0.0f;
    for (int st = 0; st < SPT; ++st) {
      if (!warp_wait(bar_full(s), ph, (1u << 8) | kRoleConsumer, abort_flag, &g_qmv_status)) {
        ok = false;
        break;
      }
      const unsigned char* sb = base_ptr + (size_t)s * kStageBytes;
      const int kt0 = st * 16 + warp * 2;  // this warp's box holds k tiles kt0 and kt0 + 1
      if (kt0 < KT) {
        const unsigned char* box = sb + warp * kBoxBytes;
        // both k tiles of the box at once: four independent accumulator chains
        const uint4 ra0 = *reinterpret_cast<const uint4*>(box + off_h0);
        const uint4 rb0 = *reinterpret_cast<const uint4*>(box + off_h0 + 1024);
        const uint4 ra1 = *reinterpret_cast<const uint4*>(box + off_h1);
        const uint4 rb1 = *reinterpret_cast<const uint4*>(box + off_h1 + 1024);
        uint2 sw = make_uint2(0, 0), zw = make_uint2(0, 0);
        if (sz_tma) {
          sw = *reinterpret_cast<const uint2*>(sb + sz_off);
          zw = *reinterpret_cast<const uint2*>(sb + sz_off + kStageSZ / 2);
        }
        const int kt1 = kt0 + 1;
        float c0[4], d0[4], c1[4], d1[4];
        const uint4* xb0 = xb_base + kt0 * xb_kt;
        const uint4* xb1 = xb_base + kt1 * xb_kt;
        const uint32_t a0[4] = {ra0.x, ra0.y, ra0.z, ra0.w}, b0[4] = {rb0.x, rb0.y, rb0.z, rb0.w};
        const uint32_t a1[4] = {ra1.x, ra1.y, ra1.z, ra1.w}, b1[4] = {rb1.x, rb1.y, rb1.z, rb1.w};
#pragma unroll
        for (int wd = 0; wd < 4; ++wd) {
          const uint4 x0 = xb0[wd * 4];
          const uint4 x1 = xb1[wd * 4];
          const uint32_t a0h = a0[wd] >> 8, b0h = b0[wd] >> 8, a1h = a1[wd] >> 8, b1h = b1[wd] >> 8;
          // nibble pairs (n0,n4) (n1,n5) of each word, then (n2,n6) (n3,n7) from the word >> 8
          if (wd == 0) {
            mma_f16_16816_first(c0, lo_magic(a0[wd]), lo_magic(b0[wd]), hi_magic(a0[wd]), hi_magic(b0[wd]), x0.x, x0.y);
            mma_f16_16816_first(c1, lo_magic(a1[wd]), lo_magic(b1[wd]), hi_magic(a1[wd]), hi_magic(b1[wd]), x1.x, x1.y);
            mma_f16_16816_first(d0, lo_magic(a0h), lo_magic(b0h), hi_magic(a0h), hi_magic(b0h), x0.z, x0.w);
            mma_f16_16816_first(d1, lo_magic(a1h), lo_magic(b1h), hi_magic(a1h), hi_magic(b1h), x1.z, x1.w);
          } else {
            mma_f16_16816(c0, lo_magic(a0[wd]), lo_magic(b0[wd]), hi_magic(a0[wd]), hi_magic(b0[wd]), x0.x, x0.y);
            mma_f16_16816(c1, lo_magic(a1[wd]), lo_magic(b1[wd]), hi_magic(a1[wd]), hi_magic(b1[wd]), x1.x, x1.y);
            mma_f16_16816(d0, lo_magic(a0h), lo_magic(b0h), hi_magic(a0h), hi_magic(b0h), x0.z, x0.w);
            mma_f16_16816(d1, lo_magic(a1h), lo_magic(b1h), hi_magic(a1h), hi_magic(b1h), x1.z, x1.w);
          }
        }
        // per unit: [0] = (row g, first group) [1] = (row g, second) [2] = (row g+8, first) [3] = (row g+8, second)
        const float v0 = (t == 0 ? c0[0] : t == 1 ? c0[1] : t == 2 ? c0[2] : c0[3]) +
                         (t == 0 ? d0[0] : t == 1 ? d0[1] : t == 2 ? d0[2] : d0[3]);
        const float v1 = (t == 0 ? c1[0] : t == 1 ? c1[1] : t == 2 ? c1[2] : c1[3]) +
                         (t == 0 ? d1[0] : t == 1 ? d1[1] : t == 2 ? d1[2] : d1[3]);
        const float2 xs0 = xg[2 * kt0 + par];
        const float2 xs1 = xg[2 * kt1 + par];
        uint32_t s0, z0, s1, z1;
        if (sz_tma) {
          asm("prmt.b32 %0, %1, %2, %3;" : "=r"(s0) : "r"(sw.x), "r"(0u), "r"(sel));
          asm("prmt.b32 %0, %1, %2, %3;" : "=r"(z0) : "r"(zw.x), "r"(0u), "r"(sel));
          asm("prmt.b32 %0, %1, %2, %3;" : "=r"(s1) : "r"(sw.y), "r"(0u), "r"(sel));
          asm("prmt.b32 %0, %1, %2, %3;" : "=r"(z1) : "r"(zw.y), "r"(0u), "r"(sel));
        } else {
          // clamped onto valid data: a clamped group meets x == 0, a clamped row is never stored
          const int64_t ri = min(tile * 16 + item_row, N - 1);
          const int g0 = min(2 * kt0 + par, G - 1), g1 = min(2 * kt1 + par, G - 1);
          s0 = ldg_nc_u16(scales + ri * G + g0) << 16;
          z0 = ldg_nc_u16(biases + ri * G + g0) << 16;
          s1 = ldg_nc_u16(scales + ri * G + g1) << 16;
          z1 = ldg_nc_u16(biases + ri * G + g1) << 16;
        }
        res = __fmaf_rn(__uint_as_float(s0), v0 - xs0.x, res);
        res = __fmaf_rn(__uint_as_float(z0), xs0.y, res);
        res = __fmaf_rn(__uint_as_float(s1), v1 - xs1.x, res);
        res = __fmaf_rn(__uint_as_float(z1), xs1.y, res);
      }
      __syncwarp();
      if (lane == 0) { mbar_arrive(bar_empty(s)); }  // this warp's part of the stage is in registers
      if (++s == stages) {
        s = 0;
        ph ^= 1u;
      }
    }
    if (!ok) { break; }
    // Both groups of a row, then the 8 warps' K slices: every warp posts its 16 partial sums and
    // moves on; the warp that posts last adds them in warp order (so the result does not depend
    // on arrival order) and stores. The ring of kRedSlots tiles is deeper than a warp can run ahead.
    res += __shfl_xor_sync(0xffffffffu, res, 1);
    const int slot = tile_seq % kRedSlots;
    if (par == 0) { red[(slot * kConsWarps + warp) * 16 + item_row] = res; }
    __syncwarp();
    uint32_t last = 0;
    if (lane == 0) {
      __threadfence_block();
      last = atomicAdd(&red_cnt[slot], 1u) == (uint32_t)(kConsWarps - 1);
    }
    last = __shfl_sync(0xffffffffu, last, 0);
    if (last) {
      __threadfence_block();
      if (lane < 16) {
        float v = 0.0f;
#pragma unroll
        for (int ww = 0; ww < kConsWarps; ++ww) {
          v += *reinterpret_cast<volatile float*>(&red[(slot * kConsWarps + ww) * 16 + lane]);
        }
        const int row = (tile << 4) + lane;
        if (row < N) { y[row] = __float2bfloat16_rn(v * x_unscale); }
      }
      __syncwarp();
      if (lane == 0) { red_cnt[slot] = 0; }
    }
  }
}

// ------------------------------------------------------------------ host side
struct LaunchShape {
  int stages;
  size_t smem;
};

LaunchShape shape_for(int cap_kt) {
  const size_t stage_bytes = kStageW + kStageSZ;
  const size_t fixed = 1024 /*alignment slack*/ + (size_t)cap_kt * 256 + 320 + (size_t)2 * cap_kt * 8 +
                       kRedSlots * kConsWarps * 16 * 4 + kRedSlots * 4 + kConsWarps * 4 +
                       2 * kMaxStages * 8 + 16;
  const size_t budget = 112 * 1024;  // two CTAs per SM
  int stages = fixed + 2 * stage_bytes <= budget ? (int)((budget - fixed) / stage_bytes) : 2;
  if (stages > kMaxStages) { stages = kMaxStages; }
  return {stages, fixed + (size_t)stages * stage_bytes};
}

int fill_problem(QmvProblem* p, const uint32_t* w, const uint16_t* scales, const uint16_t* biases,
                 const uint16_t* x, __nv_bfloat16* y, int K, int N, int tile_begin) {
  std::memset(p, 0, sizeof(*p));
  if (int rc = make_map_2d(&p->mw, CU_TENSOR_MAP_DATA_TYPE_UINT32, 4, w, (uint64_t)(K / 8), (uint64_t)N, 32,
                           16, CU_TENSOR_MAP_SWIZZLE_128B, "w")) {
    return rc;
  }
  // The scale / bias rows can be TMA boxes only if their pitch and base are multiples of 16 bytes.
  p->scales_tma = ((K % 512) == 0 && aligned16(scales) && aligned16(biases)) ? 1 : 0;
  if (p->scales_tma) {
    const int G = K / 64;
    if (int rc = make_map_2d(&p->ms, CU_TENSOR_MAP_DATA_TYPE_UINT16, 2, scales, (uint64_t)G, (uint64_t)N, 32,
                             16, CU_TENSOR_MAP_SWIZZLE_NONE, "scales")) {
      return rc;
    }
    if (int rc = make_map_2d(&p->mz, CU_TENSOR_MAP_DATA_TYPE_UINT16, 2, biases, (uint64_t)G, (uint64_t)N, 32,
                             16, CU_TENSOR_MAP_SWIZZLE_NONE, "biases")) {
      return rc;
    }
  }
  p->scales = scales;
  p->biases = biases;
  p->x = x;
  p->y = y;
  p->K = K;
  p->N = N;
  p->tile_begin = tile_begin;
  p->row_tiles = (N + 15) / 16;
  return VPQ_OK;
}

int launch_list(const QmvProblem& single, const QmvProblem* list, int total_tiles, int cap_kt,
                cudaStream_t st) {
  const LaunchShape ls = shape_for(cap_kt);
  auto kern = affine_qmv_w4g64_kernel;
  VPQ_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)ls.smem));
  const int cap = 2 * num_sms();
  const int ctas = total_tiles < cap ? total_tiles : cap;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)ctas, 1, 1);
  cfg.blockDim = dim3(kThreads, 1, 1);
  cfg.dynamicSmemBytes = ls.smem;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  VPQ_CUDA_OK(cudaLaunchKernelEx(&cfg, kern, single, list, total_tiles, ls.stages, cap_kt));
  return VPQ_OK;
}

int check_qmv_args(const char* who, const void* w, const void* scales, const void* biases, const void* x,
                   const void* y, int64_t K, int64_t N, int64_t M) {
  if (!w || !scales || !biases || !x || !y) { return fail(VPQ_ERR_INVALID_ARG, "%s: null pointer", who); }
  if (K <= 0 || N <= 0 || M <= 0 || (K % 64) != 0) {
    return fail(VPQ_ERR_INVALID_ARG, "%s: need K>0, N>0, M>0, K%%64==0 (K=%lld N=%lld M=%lld)", who,
                (long long)K, (long long)N, (long long)M);
  }
  if (K > 32768 || N > (1 << 30) || M > 65535) {
    return fail(VPQ_ERR_UNSUPPORTED, "%s: K<=32768, M<=65535 supported (K=%lld M=%lld)", who, (long long)K,
                (long long)M);
  }
  if (!aligned16(w) || !aligned16(x) || (reinterpret_cast<uintptr_t>(scales) & 1) ||
      (reinterpret_cast<uintptr_t>(biases) & 1) || (reinterpret_cast<uintptr_t>(y) & 1)) {
    return fail(VPQ_ERR_ALIGNMENT, "%s: w and x must be 16-byte aligned", who);
  }
  return VPQ_OK;
}

}  // namespace

int qmv_status_read(cudaStream_t st, uint32_t* out) {
  uint32_t v = 0;
  VPQ_CUDA_OK(cudaMemcpyFromSymbolAsync(&v, g_qmv_status, sizeof(v), 0, cudaMemcpyDeviceToHost, st));
  VPQ_CUDA_OK(cudaStreamSynchronize(st));
  if (v != 0) {
    const uint32_t zero = 0;
    VPQ_CUDA_OK(cudaMemcpyToSymbolAsync(g_qmv_status, &zero, sizeof(zero), 0, cudaMemcpyHostToDevice, st));
    VPQ_CUDA_OK(cudaStreamSynchronize(st));
  }
  *out = v;
  return VPQ_OK;
}
}  // namespace vpq

using namespace vpq;

struct vpq_qmv_plan_s {
  const QmvProblem* list_dev;
  int count;        // problems (one per GEMV row)
  int total_tiles;
  int cap_kt;
};

extern "C" int vpq_affine_qmv_w4g64_bf16(const uint32_t* w, const void* scales, const void* biases,
                                         const void* x, void* y, int64_t K, int64_t N, int64_t M,
                                         void* stream) {
  clear_error();
  if (int rc = check_qmv_args("affine_qmv_w4g64", w, scales, biases, x, y, K, N, M)) { return rc; }
  if (int rc = require_sm100()) { return rc; }
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int cap_kt = (int)((K + 255) / 256) * 2;
  for (int64_t m = 0; m < M; ++m) {  // every row streams the weight again, as in the reference
    QmvProblem p;
    if (int rc = fill_problem(&p, w, static_cast<const uint16_t*>(scales), static_cast<const uint16_t*>(biases),
                              static_cast<const uint16_t*>(x) + m * K, static_cast<__nv_bfloat16*>(y) + m * N,
                              (int)K, (int)N, 0)) {
      return rc;
    }
    if (int rc = launch_list(p, nullptr, p.row_tiles, cap_kt, st)) { return rc; }
  }
  return VPQ_OK;
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

extern "C" size_t vpq_qmv_plan_bytes(const vpq_linear_desc* d, int count) {
  if (!d || count <= 0) { return 0; }
  size_t rows = 0;
  for (int i = 0; i < count; ++i) { rows += d[i].M > 0 ? (size_t)d[i].M : 0; }
  return rows * sizeof(QmvProblem) + 64;
}

extern "C" int vpq_qmv_plan_create(const vpq_linear_desc* d, int count, void* workspace, size_t bytes,
                                   void* stream, vpq_qmv_plan** out) {
  clear_error();
  if (!d || count <= 0 || !workspace || !out) {
    return fail(VPQ_ERR_INVALID_ARG, "qmv_plan_create: null or empty arguments");
  }
  if (bytes < vpq_qmv_plan_bytes(d, count)) {
    return fail(VPQ_ERR_INVALID_ARG, "qmv_plan_create: workspace of %zu bytes, %zu needed", bytes,
                vpq_qmv_plan_bytes(d, count));
  }
  for (int i = 0; i < count; ++i) {
    if (int rc = check_qmv_args("qmv_plan_create", d[i].w, d[i].scales, d[i].biases, d[i].x, d[i].y,
                                d[i].K, d[i].N, d[i].M)) {
      return rc;
    }
  }
  if (int rc = require_sm100()) { return rc; }
  size_t rows = 0;
  for (int i = 0; i < count; ++i) { rows += (size_t)d[i].M; }
  QmvProblem* host = static_cast<QmvProblem*>(std::aligned_alloc(64, rows * sizeof(QmvProblem)));
  if (!host) { return fail(VPQ_ERR_INVALID_ARG, "qmv_plan_create: out of host memory"); }
  int tiles = 0, cap_kt = 0;
  size_t r = 0;
  for (int i = 0; i < count; ++i) {
    for (int64_t m = 0; m < d[i].M; ++m, ++r) {
      const int rc = fill_problem(&host[r], d[i].w, static_cast<const uint16_t*>(d[i].scales),
                                  static_cast<const uint16_t*>(d[i].biases),
                                  static_cast<const uint16_t*>(d[i].x) + m * d[i].K,
                                  static_cast<__nv_bfloat16*>(d[i].y) + m * d[i].N, (int)d[i].K, (int)d[i].N,
                                  tiles);
      if (rc) {
        std::free(host);
        return rc;
      }
      tiles += host[r].row_tiles;
      const int kt = (int)((d[i].K + 255) / 256) * 2;
      cap_kt = kt > cap_kt ? kt : cap_kt;
    }
  }
  const uintptr_t dev = (reinterpret_cast<uintptr_t>(workspace) + 63) & ~(uintptr_t)63;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  cudaError_t e = cudaMemcpyAsync(reinterpret_cast<void*>(dev), host, rows * sizeof(QmvProblem),
                                  cudaMemcpyHostToDevice, st);
  if (e == cudaSuccess) { e = cudaStreamSynchronize(st); }
  std::free(host);
  if (e != cudaSuccess) { return fail(VPQ_ERR_CUDA, "qmv_plan_create: copy failed: %s", cudaGetErrorString(e)); }
  vpq_qmv_plan* plan = new vpq_qmv_plan_s();
  plan->list_dev = reinterpret_cast<const QmvProblem*>(dev);
  plan->count = (int)rows;
  plan->total_tiles = tiles;
  plan->cap_kt = cap_kt;
  *out = plan;
  return VPQ_OK;
}

extern "C" int vpq_qmv_plan_run(const vpq_qmv_plan* plan, void* stream) {
  clear_error();
  if (!plan) { return fail(VPQ_ERR_INVALID_ARG, "qmv_plan_run: null plan"); }
  if (int rc = require_sm100()) { return rc; }
  QmvProblem unused;
  std::memset(&unused, 0, sizeof(unused));
  return launch_list(unused, plan->list_dev, plan->total_tiles, plan->cap_kt, static_cast<cudaStream_t>(stream));
}

// ---------------------------------------------------------------- no-allocation variant
// The plan kernel needs its list of problem descriptors in device memory. This variant keeps that
// list in a fixed array that is part of the library image, so the call neither allocates nor needs
// a caller workspace. Every GPU that loads the library carries the array (28 KB) until exit.
constexpr int kNoAllocMaxRows = 64;  // GEMV rows (sum of M over the set) one call can take
static __device__ __align__(256) unsigned char g_noalloc_descs[kNoAllocMaxRows * sizeof(QmvProblem)];

extern "C" int vpq_affine_qmv_w4g64_bf16_set_noalloc(const vpq_linear_desc* d, int count, void* stream) {
  clear_error();
  if (!d || count <= 0) { return fail(VPQ_ERR_INVALID_ARG, "qmv_set_noalloc: null or empty set"); }
  int64_t rows = 0;
  for (int i = 0; i < count; ++i) {
    if (int rc = check_qmv_args("qmv_set_noalloc", d[i].w, d[i].scales, d[i].biases, d[i].x, d[i].y, d[i].K,
                                d[i].N, d[i].M)) {
      return rc;
    }
    rows += d[i].M;
  }
  if (rows > kNoAllocMaxRows) {
    return fail(VPQ_ERR_UNSUPPORTED,
                "qmv_set_noalloc: %lld GEMV rows in the set, the built-in descriptor array holds %d; "
                "split the set or use vpq_qmv_plan_create with a workspace",
                (long long)rows, kNoAllocMaxRows);
  }
  if (int rc = require_sm100()) { return rc; }
  // Device address of the array, looked up once per device with that device current. In host code
  // the array's name is only a handle for this lookup, never a pointer a kernel could use.
  static void* dev_addr[64] = {};
  int dev = 0;
  VPQ_CUDA_OK(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64) { return fail(VPQ_ERR_CUDA, "qmv_set_noalloc: device index %d", dev); }
  if (!dev_addr[dev]) {
    void* ptr = nullptr;
    VPQ_CUDA_OK(cudaGetSymbolAddress(&ptr, g_noalloc_descs));
    dev_addr[dev] = ptr;
  }
  QmvProblem host[kNoAllocMaxRows];
  int tiles = 0, cap_kt = 0, r = 0;
  for (int i = 0; i < count; ++i) {
    for (int64_t m = 0; m < d[i].M; ++m, ++r) {
      if (int rc = fill_problem(&host[r], d[i].w, static_cast<const uint16_t*>(d[i].scales),
                                static_cast<const uint16_t*>(d[i].biases),
                                static_cast<const uint16_t*>(d[i].x) + m * d[i].K,
                                static_cast<__nv_bfloat16*>(d[i].y) + m * d[i].N, (int)d[i].K, (int)d[i].N,
                                tiles)) {
        return rc;
      }
      tiles += host[r].row_tiles;
      const int kt = (int)((d[i].K + 255) / 256) * 2;
      cap_kt = kt > cap_kt ? kt : cap_kt;
    }
  }
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  // every descriptor the kernel will read is rewritten here, so nothing stale from the previous
  // call is ever used; the copy is ordered before the launch on the same stream
  VPQ_CUDA_OK(cudaMemcpyAsync(dev_addr[dev], host, (size_t)r * sizeof(QmvProblem), cudaMemcpyHostToDevice, st));
  QmvProblem unused;
  std::memset(&unused, 0, sizeof(unused));
  return launch_list(unused, static_cast<const QmvProblem*>(dev_addr[dev]), tiles, cap_kt, st);
}

extern "C" int vpq_qmv_plan_destroy(vpq_qmv_plan* plan) {
  delete plan;
  return VPQ_OK;
}
