// qmv_w8.cu -- decode GEMV over 8-bit affine group-64 weights (M = 1 per launch).
//
// y[n] = sum_k x[k] * (s[n,k/64] * q[n,k] + b[n,k/64]),  q one byte per value, f32 accumulate.
// Replaces affine_qmv_w8g64 (qmv_fast_impl<T,64,8,...>, gpu-kernels/metal/quant/affine_qmv.metal:186-301
// instantiated at :3027-3070): the 8-bit linears of mixed-precision checkpoints.
//
// The skeleton of the 4-bit kernel (qmv.cu): a producer warp streams [16 rows x 128 bytes] TMA
// boxes (here 128 k each) plus the span's scales and biases into a ring of stages (8 boxes =
// 1024 k); eight consumer warps split K, warp w takes box w of every stage; exact integer
// arithmetic on mma.sync.m16n8k32.u8.s8 with x as three signed base-256 digits. With one byte per
// weight no unpacking is left: the bytes a lane loads ARE its A fragments. One MMA takes 16 k
// of the k tile's first group (k columns 0..15) and 16 k of its second (16..31); accumulator
// column (digit, parity) gets the digit's bytes in the half of B that belongs to its group and
// zeros in the other, so a lane ends up with digit t's sums for both groups and both of its rows
// and folds them with the groups' scales (lane 3 of a quad folds the bias term b * sum(x)).
// Every warp stages the part of x it multiplies as digit bytes in natural k order, each 128-k box with
// its own power-of-two scale. Every barrier wait is bounded.
#include "vpq_sm100.cuh"

#include <cstring>

namespace vpq {

__device__ uint32_t g_qmv8_status;  // 0, or (site << 8) | role of the first bounded wait that gave up

namespace {

constexpr int kConsWarps = 8;
constexpr int kConsThreads = kConsWarps * 32;
constexpr int kThreads = kConsThreads + 32;  // + producer warp
constexpr int kBoxBytes = 16 * 128;          // one TMA box: 16 rows x 128 bytes (128 k, two groups)
constexpr int kBoxesPerStage = 8;            // a stage spans 1024 k
constexpr int kStageW = kBoxesPerStage * kBoxBytes;
// GS: quantization group, 64 or 32 (the reference's affine_qmv_w8g32, affine_qmv.metal:3050-3066). A 128-k
// box holds 128 / GS groups.
template <int GS>
struct Cfg {
  static constexpr int kGroupsPerKt = 128 / GS;
  static constexpr int kStageGroups = kBoxesPerStage * kGroupsPerKt;   // groups a stage spans
  static constexpr int kStageSZ = 2 * 16 * kStageGroups * 2;           // scales + biases: 2 x [16 rows x groups] bf16
  static constexpr int kStageBytes = kStageW + kStageSZ;
};
constexpr int kMaxStages = 6;
constexpr int kRedSlots = 8;
constexpr int kXBytesPerKt = 3 * 128;        // staged x per 128-k tile: 3 digit planes of 128 bytes

constexpr int kAccInit = 0x4B400000;         // bits of 12582912.0f: an s32 sum |v| < 2^22 added to it reads as a float
constexpr float kAccInitF = 12582912.0f;

__device__ __forceinline__ void mma_u8s8(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                         uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 "
      "{%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void mma_u8s8_first(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                               uint32_t b0, uint32_t b1, int init) {
  asm volatile(
      "mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 "
      "{%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
      : "=r"(c[0]), "=r"(c[1]), "=r"(c[2]), "=r"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "r"(init));
}

enum : uint32_t { kRoleProducer = 1, kRoleConsumer = 2 };

struct alignas(64) Problem8 {
  CUtensorMap mw, ms, mz;      // weights [N, K/4] u32; scales, biases [N, K/64] (valid if scales_tma)
  const uint16_t* scales;
  const uint16_t* biases;
  const uint16_t* x;           // K bf16
  __nv_bfloat16* y;            // N outputs
  int K, N;
  int row_tiles;
  int scales_tma;
  int epilogue;                // kEpi*: what the store does with a row's sum (see fused_store)
  int q_rows, k_rows;
  const uint16_t* aux;
  __nv_bfloat16* y3;
  const int32_t* eid;          // not null: *eid is the expert whose [N, K] slab of w / scales / biases is used
  int experts;                 // slabs in w (eid is clamped to it)
  float eps;                   // RMSNorm epsilon
  const uint16_t* norm_w;      // not null: x is RMS-normalised with these K weights while it is staged
  const int32_t* xrow;         // not null: x is row max(*xrow, 0) of the matrix x points at (sorted-slot gather)
  const int32_t* vrow;         // not null: the slot's outputs are stored only if *vrow >= 0 (and *eid >= 0)
};

template <int GS>
__global__ void __launch_bounds__(kThreads, 2)
affine_qmv_w8g64_kernel(const __grid_constant__ Problem8 P, int stages, int cap_kt) {
  constexpr int kStageSZ = Cfg<GS>::kStageSZ;
  constexpr int kStageBytes = Cfg<GS>::kStageBytes;
  constexpr int GPK = Cfg<GS>::kGroupsPerKt;    // groups per 128-k tile: 2 or 4
  extern __shared__ unsigned char smem_dyn[];
  const uint32_t raw = smem_u32(smem_dyn);
  const uint32_t base = (raw + 1023u) & ~1023u;  // swizzled boxes need 1024-byte alignment
  unsigned char* base_ptr = smem_dyn + (base - raw);
  const int K = P.K, N = P.N;

  unsigned char* p0 = base_ptr + (size_t)stages * kStageBytes;
  uint4* zero128 = reinterpret_cast<uint4*>(p0);                 // 128 bytes of zeros, 128-byte aligned
  unsigned char* xq = p0 + 128;                                  // [cap_kt][3 digits][128 B]: digit bytes in k order
  float* xg = reinterpret_cast<float*>(xq + (size_t)cap_kt * kXBytesPerKt);  // [GPK * cap_kt] sum of X per group
  float* zero16 = xg + ((GPK * cap_kt + 3) & ~3);                // 16 bytes of zeros, 16-byte aligned (cap_kt may be odd)
  float* red = zero16 + 4;                                       // [kRedSlots][kConsWarps][16]
  uint32_t* red_cnt = reinterpret_cast<uint32_t*>(red + kRedSlots * kConsWarps * 16);
  float* xu = reinterpret_cast<float*>(red_cnt + kRedSlots);     // [cap_kt] 1 / scale of every 128-k box of x
  uint64_t* bars = reinterpret_cast<uint64_t*>(xu + ((cap_kt + 1) & ~1));
  volatile uint32_t* abort_flag = reinterpret_cast<volatile uint32_t*>(bars + 2 * kMaxStages);
  uint32_t* sq_cnt = const_cast<uint32_t*>(abort_flag) + 1;      // consumer warps that posted their sum of squares
  float* sq_part = reinterpret_cast<float*>(sq_cnt + 3);         // [kConsWarps]
  const uint32_t bar0 = smem_u32(bars);
  auto bar_full = [&](int s) { return bar0 + 8u * s; };
  auto bar_empty = [&](int s) { return bar0 + 8u * (kMaxStages + s); };

  const int lane = threadIdx.x & 31;
  const int warp = threadIdx.x >> 5;
  const int NB = (K + 127) >> 7;                               // boxes (128-k tiles) per row
  const int SPT = (NB + kBoxesPerStage - 1) / kBoxesPerStage;  // stages per row tile
  const int gt_begin = (int)(((int64_t)P.row_tiles * blockIdx.x) / gridDim.x);
  const int gt_end = (int)(((int64_t)P.row_tiles * (blockIdx.x + 1)) / gridDim.x);

  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

  if (threadIdx.x == 0) {
    for (int s = 0; s < stages; ++s) {
      mbar_init(bar_full(s), 1);
      mbar_init(bar_empty(s), kConsWarps);
    }
    *abort_flag = 0;
    *sq_cnt = 0;
    for (int i = 0; i < kRedSlots; ++i) { red_cnt[i] = 0; }
    fence_mbar_init();
  }
  if (threadIdx.x < 8) { zero128[threadIdx.x] = make_uint4(0, 0, 0, 0); }
  if (threadIdx.x == 8) { *reinterpret_cast<uint4*>(zero16) = make_uint4(0, 0, 0, 0); }
  __syncthreads();

  if (warp == kConsWarps) {
    // ------------------------------------------------------------ producer
    if (lane == 0) {
      uint32_t it = 0;
      bool ok = true;
      const bool sz_tma = P.scales_tma != 0;
      int row0 = 0;
      if (P.eid) {
        // the routed expert is an output of an earlier kernel: unlike the weights it must be waited for
        // (the reference's affine_gather_qmv_swiglu_w8g64 / _geglu_ / affine_gather_down_qmv_w8g64 read it
        // the same way, gpu-kernels/metal/quant/affine_qmv.metal:957-994,1290-1322,1519-1548)
        asm volatile("griddepcontrol.wait;" ::: "memory");
        row0 = min(max(__ldg(P.eid), 0), P.experts - 1) * N;
      }
      for (int tile = gt_begin; tile < gt_end && ok; ++tile) {
        for (int st = 0; st < SPT; ++st, ++it) {
          const int s = it % stages;
          const uint32_t ph = (it / stages) & 1u;
          if (!mbar_wait(bar_empty(s), ph ^ 1u, (1u << 8) | kRoleProducer, abort_flag, &g_qmv8_status)) {
            ok = false;
            break;
          }
          const int nb = min(kBoxesPerStage, NB - st * kBoxesPerStage);
          const uint32_t dst = base + (uint32_t)s * kStageBytes;
          mbar_expect_tx(bar_full(s), (uint32_t)nb * kBoxBytes + (sz_tma ? kStageSZ : 0));
          for (int b = 0; b < nb; ++b) {
            tma_load_2d(dst + b * kBoxBytes, &P.mw, bar_full(s), (st * kBoxesPerStage + b) * 32, row0 + tile * 16);
          }
          if (sz_tma) {
            tma_load_2d(dst + kStageW, &P.ms, bar_full(s), st * Cfg<GS>::kStageGroups, row0 + tile * 16);
            tma_load_2d(dst + kStageW + kStageSZ / 2, &P.mz, bar_full(s), st * Cfg<GS>::kStageGroups, row0 + tile * 16);
          }
        }
      }
      // Never leave with a copy still in flight: wait for the last load of every stage.
      for (int s = 0; s < stages; ++s) {
        if (it > (uint32_t)s) {
          const uint32_t last = ((it - 1 - s) / stages) * stages + s;
          mbar_wait(bar_full(s), (last / stages) & 1u, (2u << 8) | kRoleProducer, abort_flag, &g_qmv8_status);
        }
      }
    }
    return;
  }

  // ---------------------------------------------------------------- consumers
  const int g = lane >> 2, t = lane & 3;
  const int rho = (g >> 1) | ((g & 1) << 2);  // stage row of MMA row g (g+8 -> rho+8): bank-conflict-free

  asm volatile("griddepcontrol.wait;" ::: "memory");  // x may come from the previous kernel

  // ---- staging of x as signed digit bytes. Warp w converts exactly the 128-k boxes it will
  // multiply (box w of every stage), a quarter warp per box, so no CTA barrier is involved. Every
  // box carries its own power-of-two scale: its largest magnitude lands in [2^21, 2^22) and every
  // value is rounded to an integer X (exact within 2^-14 of the box's maximum, off by at most
  // 2^-22 of it otherwise), X = d0 + 256 d1 + 65536 d2 with digits in [-128, 127]; digit plane d
  // of k tile kt holds the 128 bytes d(X[128 kt .. 128 kt + 127]) in order. xu[kt] = 1 / scale.
  // With norm_w the vector is first RMS-normalised as the reference's fused kernel does
  // (affine_qmv_qkv_rms_w8g64, the 8-bit instantiation of gpu-kernels/metal/quant/affine_qmv.metal:570-694):
  // sum of squares in f32 over the whole vector (the eight consumer warps exchange partial sums through
  // shared memory: post, count, bounded wait), x <- bf16(x * rsqrt(mean + eps) * norm_w).
  const uint16_t* xrow_ptr = P.x + (P.xrow ? (size_t)max(__ldg(P.xrow), 0) * (size_t)K : 0);  // a dead slot reads row 0
  float inv = 1.0f;
  if (P.norm_w) {
    float sq = 0.0f;
    for (int k0 = (warp * 32 + lane) * 8; k0 < K; k0 += kConsThreads * 8) {
      const uint4 in = *reinterpret_cast<const uint4*>(xrow_ptr + k0);
      const uint32_t v[4] = {in.x, in.y, in.z, in.w};
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        const float lo = __uint_as_float(v[q] << 16), hi = __uint_as_float(v[q] & 0xffff0000u);
        sq = __fmaf_rn(lo, lo, sq);
        sq = __fmaf_rn(hi, hi, sq);
      }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) { sq += __shfl_xor_sync(0xffffffffu, sq, o); }
    uint32_t all = 1;
    if (lane == 0) {
      sq_part[warp] = sq;
      __threadfence_block();
      atomicAdd(sq_cnt, 1u);
      all = 0;
      for (uint32_t i = 0; i < (1u << 28); ++i) {
        if (*reinterpret_cast<volatile uint32_t*>(sq_cnt) >= (uint32_t)kConsWarps) {
          all = 1;
          break;
        }
        if (*abort_flag) { break; }
      }
      if (!all) {
        *abort_flag = 1;
        atomicCAS(&g_qmv8_status, 0u, (4u << 8) | kRoleConsumer);
      }
      __threadfence_block();
    }
    all = __shfl_sync(0xffffffffu, all, 0);
    if (!all) { return; }
    float total = 0.0f;
#pragma unroll
    for (int ww = 0; ww < kConsWarps; ++ww) { total += *reinterpret_cast<volatile float*>(&sq_part[ww]); }
    inv = __frsqrt_rn(__fadd_rn(__fdiv_rn(total, (float)K), P.eps));
  }
  {
    const int quarter = lane >> 3, sub = lane & 7;
    const int passes = (SPT + 3) >> 2;  // four boxes of this warp per pass
    for (int j = 0; j < passes; ++j) {
      const int kt = (4 * j + quarter) * kBoxesPerStage + warp;
      const bool live = kt < NB;
      const int k0 = kt * 128 + sub * 16;
      uint4 in0 = make_uint4(0, 0, 0, 0), in1 = in0;
      if (k0 < K) {
        in0 = *reinterpret_cast<const uint4*>(xrow_ptr + k0);
        in1 = *reinterpret_cast<const uint4*>(xrow_ptr + k0 + 8);
      }
      uint32_t v[8] = {in0.x, in0.y, in0.z, in0.w, in1.x, in1.y, in1.z, in1.w};
      if (P.norm_w) {
        uint4 n0 = make_uint4(0, 0, 0, 0), n1 = n0;
        if (k0 < K) {
          n0 = __ldg(reinterpret_cast<const uint4*>(P.norm_w + k0));
          n1 = __ldg(reinterpret_cast<const uint4*>(P.norm_w + k0 + 8));
        }
        const uint32_t nv[8] = {n0.x, n0.y, n0.z, n0.w, n1.x, n1.y, n1.z, n1.w};
#pragma unroll
        for (int q = 0; q < 8; ++q) {
          const float lo = __fmul_rn(__fmul_rn(__uint_as_float(v[q] << 16), inv), __uint_as_float(nv[q] << 16));
          const float hi = __fmul_rn(__fmul_rn(__uint_as_float(v[q] & 0xffff0000u), inv),
                                     __uint_as_float(nv[q] & 0xffff0000u));
          v[q] = pack_bf16x2(lo, hi);
        }
      }
      uint32_t amax = 0;  // largest |x| of the box as bf16 bits
#pragma unroll
      for (int q = 0; q < 8; ++q) { amax = max(amax, max(v[q] & 0x7fffu, (v[q] >> 16) & 0x7fffu)); }
#pragma unroll
      for (int o = 4; o > 0; o >>= 1) { amax = max(amax, __shfl_xor_sync(0xffffffffu, amax, o)); }
      int e = (int)(amax >> 7);            // biased exponent of the largest magnitude
      e = min(max(e, 22), 254);            // all-zero / denormal box: keep both factors normal
      const float x_scale = __uint_as_float((uint32_t)(275 - e) << 23);  // 2^(148 - e)
      // round(x * scale) on the FMA pipe: the low bits of fma(x, scale, 1.5 * 2^23) are
      // 0x4B400000 + X; one add turns that into X + 0x808080 (bytes 0..2 = digits + 128).
      uint32_t z[16];
      uint32_t sum = 0;
#pragma unroll
      for (int q = 0; q < 8; ++q) {
        const uint32_t lo = __float_as_uint(__fmaf_rn(__uint_as_float(v[q] << 16), x_scale, kAccInitF));
        const uint32_t hi = __float_as_uint(__fmaf_rn(__uint_as_float(v[q] & 0xffff0000u), x_scale, kAccInitF));
        sum += lo + hi;
        z[2 * q] = lo + (0x808080u - (uint32_t)kAccInit);
        z[2 * q + 1] = hi + (0x808080u - (uint32_t)kAccInit);
      }
      sum -= 16u * (uint32_t)kAccInit;  // = sum of the 16 X, modulo 2^32
      uint32_t plane[3][4];             // digit d of values 4 q .. 4 q + 3 -> plane[d][q]
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        const uint32_t za = z[4 * q], zb = z[4 * q + 1], zc = z[4 * q + 2], zd = z[4 * q + 3];
        const uint32_t t0 = __byte_perm(za, zb, 0x5140), t1 = __byte_perm(zc, zd, 0x5140);
        const uint32_t t2 = __byte_perm(za, zb, 0x0062), t3 = __byte_perm(zc, zd, 0x0062);
        plane[0][q] = __byte_perm(t0, t1, 0x5410) ^ 0x80808080u;
        plane[1][q] = __byte_perm(t0, t1, 0x7632) ^ 0x80808080u;
        plane[2][q] = __byte_perm(t2, t3, 0x5410) ^ 0x80808080u;
      }
      if (live) {
        unsigned char* dst = xq + (size_t)kt * kXBytesPerKt + sub * 16;
#pragma unroll
        for (int d = 0; d < 3; ++d) {
          *reinterpret_cast<uint4*>(dst + d * 128) = make_uint4(plane[d][0], plane[d][1], plane[d][2], plane[d][3]);
        }
      }
      sum += __shfl_xor_sync(0xffffffffu, sum, 1);
      if (GS == 64) {
        sum += __shfl_xor_sync(0xffffffffu, sum, 2);
        if (live && (sub & 3) == 0) { xg[kt * 2 + (sub >> 2)] = (float)(int)sum; }
      } else {  // a group is 32 values = two lanes' pieces
        if (live && (sub & 1) == 0) { xg[kt * 4 + (sub >> 1)] = (float)(int)sum; }
      }
      if (live && sub == 0) { xu[kt] = __uint_as_float((uint32_t)(e - 21) << 23); }  // exact inverse of x_scale
    }
    __syncwarp();
  }

  // Accumulator column c (fed by the lanes with g == c) = (digit c >> 1, group parity c & 1).
  // An MMA's first 16 k columns come from the k tile's first group, the last 16 from its second:
  // B register 0 of a lane carries its digit's bytes if the column's parity is 0, register 1 if
  // it is 1; the other register reads zeros (from a zero line, at the chunks the real reads of
  // the same quarter warp do not use).
  // Group 32: a box has four groups, two in each 64-byte half (chunks t = 0, 1 / t = 2, 3 of a half), so
  // every A fragment meets two B operands: one with this lane's digit bytes in the first half only (and
  // only if its chunk lies in the column's group of that half), one likewise for the second half; the
  // accumulator columns (digit, parity) then hold groups 0 | 1 after the first MMA, 2 | 3 after the second.
  const int digit = g >> 1, parity = g & 1;
  const bool has_digit = digit < 3;
  const unsigned char* zline = reinterpret_cast<const unsigned char*>(zero128);
  const bool b0_real = has_digit && (GS == 64 ? parity == 0 : (t >> 1) == parity);
  const bool b1_real = has_digit && (GS == 64 ? parity == 1 : (t >> 1) == parity);
  const unsigned char* b0_ptr = b0_real ? xq + digit * 128 + t * 16 : zline + (4 + t) * 16;
  const unsigned char* b1_ptr = b1_real ? xq + digit * 128 + 64 + t * 16 : zline + t * 16;
  const int b0_kt = b0_real ? kXBytesPerKt : 0;
  const int b1_kt = b1_real ? kXBytesPerKt : 0;
  const bool bias_lane = t == 3;  // folds b * sum(x) where the others fold s * (digit sum)
  const float* xs_base = bias_lane ? xg : zero16;
  const int xs_kt = bias_lane ? GPK : 0;
  const float digit_weight = t == 1 ? 256.0f : t == 2 ? 65536.0f : 1.0f;

  const uint32_t off_lo = (uint32_t)rho * 128u + (uint32_t)(((0 + t) ^ rho) << 4);  // k 16 t .. of the first group
  const uint32_t off_hi = (uint32_t)rho * 128u + (uint32_t)(((4 + t) ^ rho) << 4);  // k 64 + 16 t .. of the second
  // 4 (8) bytes = the 2 (4) groups of this warp's box, row rho, in the stage's scales or biases
  constexpr uint32_t kSzRow = (uint32_t)Cfg<GS>::kStageGroups * 2u;   // bytes of one row of the stage's scales
  const uint32_t sz_off = (uint32_t)kStageW + (bias_lane ? (uint32_t)kStageSZ / 2 : 0u) + (uint32_t)rho * kSzRow +
                          (uint32_t)warp * (2u * GPK);
  const bool sz_tma = P.scales_tma != 0;
  const int G = K / GS;

  uint32_t tile_seq = 0, ph = 0;
  int s = 0;
  bool ok = true;
  for (int tile = gt_begin; tile < gt_end && ok; ++tile, ++tile_seq) {
    float res_a = 0.0f, res_b = 0.0f;  // W rows rho and rho + 8: this lane's digit (or bias) share
    for (int st = 0; st < SPT; ++st) {
      if (!warp_wait(bar_full(s), ph, (1u << 8) | kRoleConsumer, abort_flag, &g_qmv8_status)) {
        ok = false;
        break;
      }
      const unsigned char* sb = base_ptr + (size_t)s * kStageBytes;
      const int kt = st * kBoxesPerStage + warp;  // this warp's box = k tile kt
      if (kt < NB) {
        const unsigned char* box = sb + warp * kBoxBytes;
        const uint4 ra_lo = *reinterpret_cast<const uint4*>(box + off_lo);
        const uint4 ra_hi = *reinterpret_cast<const uint4*>(box + off_hi);
        const uint4 rb_lo = *reinterpret_cast<const uint4*>(box + off_lo + 1024);
        const uint4 rb_hi = *reinterpret_cast<const uint4*>(box + off_hi + 1024);
        const uint4 x0 = *reinterpret_cast<const uint4*>(b0_ptr + (size_t)kt * b0_kt);
        const uint4 x1 = *reinterpret_cast<const uint4*>(b1_ptr + (size_t)kt * b1_kt);
        uint2 sa, sb2;  // the groups' scales (or biases) of rows rho, rho + 8: 2 in .x (group 64), 4 in .x .y (group 32)
        sa.y = sb2.y = 0;
        if (sz_tma) {
          if (GS == 64) {
            sa.x = *reinterpret_cast<const uint32_t*>(sb + sz_off);
            sb2.x = *reinterpret_cast<const uint32_t*>(sb + sz_off + 8 * kSzRow);
          } else {
            sa = *reinterpret_cast<const uint2*>(sb + sz_off);
            sb2 = *reinterpret_cast<const uint2*>(sb + sz_off + 8 * kSzRow);
          }
        } else {
          // clamped onto valid data: a clamped group meets x == 0, a clamped row is never stored
          const uint16_t* src = bias_lane ? P.biases : P.scales;
          const int64_t slab = P.eid ? (int64_t)min(max(__ldg(P.eid), 0), P.experts - 1) * N : 0;
          const int64_t r_a = slab + min(tile * 16 + rho, N - 1), r_b = slab + min(tile * 16 + rho + 8, N - 1);
          const int g0 = min(GPK * kt, G - 1), g1 = min(GPK * kt + 1, G - 1);
          sa.x = ldg_nc_u16(src + r_a * G + g0) | (ldg_nc_u16(src + r_a * G + g1) << 16);
          sb2.x = ldg_nc_u16(src + r_b * G + g0) | (ldg_nc_u16(src + r_b * G + g1) << 16);
          if (GS == 32) {
            const int g2 = min(4 * kt + 2, G - 1), g3 = min(4 * kt + 3, G - 1);
            sa.y = ldg_nc_u16(src + r_a * G + g2) | (ldg_nc_u16(src + r_a * G + g3) << 16);
            sb2.y = ldg_nc_u16(src + r_b * G + g2) | (ldg_nc_u16(src + r_b * G + g3) << 16);
          }
        }
        auto val = [](int a, int b, float k) { return (__int_as_float(a) - kAccInitF) + (__int_as_float(b) - k); };
        const float xu_box = xu[kt];
        float box_a, box_b;
        if (GS == 64) {
          const float2 xs = *reinterpret_cast<const float2*>(xs_base + kt * xs_kt);
          int ca[4], cb[4];  // two independent chains
          mma_u8s8_first(ca, ra_lo.x, rb_lo.x, ra_hi.x, rb_hi.x, x0.x, x1.x, kAccInit);
          mma_u8s8_first(cb, ra_lo.y, rb_lo.y, ra_hi.y, rb_hi.y, x0.y, x1.y, kAccInit);
          mma_u8s8(ca, ra_lo.z, rb_lo.z, ra_hi.z, rb_hi.z, x0.z, x1.z);
          mma_u8s8(cb, ra_lo.w, rb_lo.w, ra_hi.w, rb_hi.w, x0.w, x1.w);
          // c[0] = (row rho, first group) c[1] = (rho, second) c[2] = (rho + 8, first) c[3] = (rho + 8, second);
          // value = chain a + chain b without the two initial values (+ sum of x in a bias lane,
          // whose accumulators hold the bare initial value)
          const float k0 = kAccInitF - xs.x, k1 = kAccInitF - xs.y;
          // the box's two groups folded with their scales, then its 1 / x-scale brings the sum to true units
          box_a = __fmul_rn(__uint_as_float(sa.x << 16), val(ca[0], cb[0], k0));
          box_a = __fmaf_rn(__uint_as_float(sa.x & 0xffff0000u), val(ca[1], cb[1], k1), box_a);
          box_b = __fmul_rn(__uint_as_float(sb2.x << 16), val(ca[2], cb[2], k0));
          box_b = __fmaf_rn(__uint_as_float(sb2.x & 0xffff0000u), val(ca[3], cb[3], k1), box_b);
        } else {
          const float4 xs = *reinterpret_cast<const float4*>(xs_base + kt * xs_kt);
          int la[4], lb[4], ha[4], hb[4];  // first / second half of the box, two chains each
          mma_u8s8_first(la, ra_lo.x, rb_lo.x, ra_hi.x, rb_hi.x, x0.x, 0u, kAccInit);
          mma_u8s8_first(lb, ra_lo.y, rb_lo.y, ra_hi.y, rb_hi.y, x0.y, 0u, kAccInit);
          mma_u8s8_first(ha, ra_lo.x, rb_lo.x, ra_hi.x, rb_hi.x, 0u, x1.x, kAccInit);
          mma_u8s8_first(hb, ra_lo.y, rb_lo.y, ra_hi.y, rb_hi.y, 0u, x1.y, kAccInit);
          mma_u8s8(la, ra_lo.z, rb_lo.z, ra_hi.z, rb_hi.z, x0.z, 0u);
          mma_u8s8(lb, ra_lo.w, rb_lo.w, ra_hi.w, rb_hi.w, x0.w, 0u);
          mma_u8s8(ha, ra_lo.z, rb_lo.z, ra_hi.z, rb_hi.z, 0u, x1.z);
          mma_u8s8(hb, ra_lo.w, rb_lo.w, ra_hi.w, rb_hi.w, 0u, x1.w);
          // c[0] / c[1] = row rho, groups 0 | 1 (first half) or 2 | 3 (second half); c[2] / c[3] = row rho + 8
          const float k0 = kAccInitF - xs.x, k1 = kAccInitF - xs.y, k2 = kAccInitF - xs.z, k3 = kAccInitF - xs.w;
          box_a = __fmul_rn(__uint_as_float(sa.x << 16), val(la[0], lb[0], k0));
          box_a = __fmaf_rn(__uint_as_float(sa.x & 0xffff0000u), val(la[1], lb[1], k1), box_a);
          box_a = __fmaf_rn(__uint_as_float(sa.y << 16), val(ha[0], hb[0], k2), box_a);
          box_a = __fmaf_rn(__uint_as_float(sa.y & 0xffff0000u), val(ha[1], hb[1], k3), box_a);
          box_b = __fmul_rn(__uint_as_float(sb2.x << 16), val(la[2], lb[2], k0));
          box_b = __fmaf_rn(__uint_as_float(sb2.x & 0xffff0000u), val(la[3], lb[3], k1), box_b);
          box_b = __fmaf_rn(__uint_as_float(sb2.y << 16), val(ha[2], hb[2], k2), box_b);
          box_b = __fmaf_rn(__uint_as_float(sb2.y & 0xffff0000u), val(ha[3], hb[3], k3), box_b);
        }
        res_a = __fmaf_rn(xu_box, box_a, res_a);
        res_b = __fmaf_rn(xu_box, box_b, res_b);
      }
      __syncwarp();
      if (lane == 0) { mbar_arrive(bar_empty(s)); }
      if (++s == stages) {
        s = 0;
        ph ^= 1u;
      }
    }
    if (!ok) { break; }
    // quad: digits + bias -> even lanes end with row rho, odd lanes with row rho + 8; then the 8
    // warps' K slices: the warp that posts last adds them in warp order and stores.
    res_a *= digit_weight;
    res_b *= digit_weight;
    float keep = (t & 1) ? res_b : res_a;
    keep += __shfl_xor_sync(0xffffffffu, (t & 1) ? res_a : res_b, 1);
    keep += __shfl_xor_sync(0xffffffffu, keep, 2);
    const int slot = tile_seq % kRedSlots;
    if (t < 2) { red[(slot * kConsWarps + warp) * 16 + rho + 8 * t] = keep; }
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
        const bool live = !P.vrow || (__ldg(P.vrow) >= 0 && (!P.eid || __ldg(P.eid) >= 0));
        if (live) { fused_store(P.epilogue, v, row, N, lane, P.y, P.aux, P.y3, P.q_rows, P.k_rows); }
      }
      __syncwarp();
      if (lane == 0) { red_cnt[slot] = 0; }
    }
  }
}

size_t fixed_smem(int cap_kt, int groups_per_kt) {
  return 1024 /*alignment slack*/ + 128 + (size_t)cap_kt * kXBytesPerKt + (size_t)((groups_per_kt * cap_kt + 3) & ~3) * 4 + 16 +
         (size_t)kRedSlots * kConsWarps * 16 * 4 + kRedSlots * 4 + (size_t)((cap_kt + 1) & ~1) * 4 + 2 * kMaxStages * 8 + 16 +
         kConsWarps * 4 /* partial sums of squares */;
}

}  // namespace

int qmv8_status_read(cudaStream_t st, uint32_t* out) {
  uint32_t v = 0;
  VPQ_CUDA_OK(cudaMemcpyFromSymbolAsync(&v, g_qmv8_status, sizeof(v), 0, cudaMemcpyDeviceToHost, st));
  VPQ_CUDA_OK(cudaStreamSynchronize(st));
  if (v != 0) {
    const uint32_t zero = 0;
    VPQ_CUDA_OK(cudaMemcpyToSymbolAsync(g_qmv8_status, &zero, sizeof(zero), 0, cudaMemcpyHostToDevice, st));
    VPQ_CUDA_OK(cudaStreamSynchronize(st));
  }
  *out = v;
  return VPQ_OK;
}
}  // namespace vpq

using namespace vpq;

namespace {
template <int GS>
int launch_w8(const char* who, const vpq_linear_desc& d, void* stream) {
  constexpr int kStageBytes = Cfg<GS>::kStageBytes;
  const uint32_t* w = d.w;
  const void *scales = d.scales, *biases = d.biases, *x = d.x;
  void* y = d.y;
  const int64_t K = d.K, N = d.N, M = d.M;
  if (!w || !scales || !biases || !x || !y) { return fail(VPQ_ERR_INVALID_ARG, "%s: null pointer", who); }
  if (K <= 0 || N <= 0 || M <= 0 || (K % GS) != 0) {
    return fail(VPQ_ERR_INVALID_ARG, "%s: need K>0, N>0, M>0, K%%%d==0 (K=%lld N=%lld M=%lld)", who, GS,
                (long long)K, (long long)N, (long long)M);
  }
  if (K > 16384 || N > (1 << 30) || M > 65535) {
    return fail(VPQ_ERR_UNSUPPORTED, "%s: K<=16384, M<=65535 supported (K=%lld M=%lld)", who, (long long)K,
                (long long)M);
  }
  if (!aligned16(w) || !aligned16(x) || (reinterpret_cast<uintptr_t>(scales) & 1) ||
      (reinterpret_cast<uintptr_t>(biases) & 1) || (reinterpret_cast<uintptr_t>(y) & 1)) {
    return fail(VPQ_ERR_ALIGNMENT, "%s: w and x must be 16-byte aligned", who);
  }
  if (int rc = qmv_check_gather(who, d, /*allow_norm=*/true)) { return rc; }
  if (int rc = require_sm100()) { return rc; }
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  Problem8 p;
  std::memset(&p, 0, sizeof(p));
  const uint64_t rows = (uint64_t)N * (uint64_t)(d.expert ? d.experts : 1);  // expert slabs are stacked along the rows
  if (int rc = make_map_2d(&p.mw, CU_TENSOR_MAP_DATA_TYPE_UINT32, 4, w, (uint64_t)(K / 4), rows, 32, 16,
                           CU_TENSOR_MAP_SWIZZLE_128B, "w")) {
    return rc;
  }
  // scale / bias rows as TMA boxes: their pitch (K / GS values of 2 bytes) and base multiples of 16 bytes
  p.scales_tma = ((K % (8 * GS)) == 0 && aligned16(scales) && aligned16(biases)) ? 1 : 0;
  if (p.scales_tma) {
    if (int rc = make_map_2d(&p.ms, CU_TENSOR_MAP_DATA_TYPE_UINT16, 2, scales, (uint64_t)(K / GS), rows,
                             Cfg<GS>::kStageGroups, 16, CU_TENSOR_MAP_SWIZZLE_NONE, "scales")) {
      return rc;
    }
    if (int rc = make_map_2d(&p.mz, CU_TENSOR_MAP_DATA_TYPE_UINT16, 2, biases, (uint64_t)(K / GS), rows,
                             Cfg<GS>::kStageGroups, 16, CU_TENSOR_MAP_SWIZZLE_NONE, "biases")) {
      return rc;
    }
  }
  p.scales = static_cast<const uint16_t*>(scales);
  p.biases = static_cast<const uint16_t*>(biases);
  p.K = (int)K;
  p.N = (int)N;
  p.row_tiles = (int)((N + 15) / 16);
  p.epilogue = d.epilogue;
  p.q_rows = (int)d.q_rows;
  p.k_rows = (int)d.k_rows;
  const bool gated = d.epilogue == VPQ_EPILOGUE_SWIGLU || d.epilogue == VPQ_EPILOGUE_GEGLU;
  const int64_t y_pitch = gated ? N / 2 : d.epilogue == VPQ_EPILOGUE_QKV ? d.q_rows : N;
  const int cap_kt = (int)((K + 127) / 128);
  const size_t fixed = fixed_smem(cap_kt, Cfg<GS>::kGroupsPerKt);
  const size_t budget = 112 * 1024;  // two CTAs per SM
  int stages = fixed + 2 * (size_t)kStageBytes <= budget ? (int)((budget - fixed) / kStageBytes) : 2;
  if (stages > kMaxStages) { stages = kMaxStages; }
  const size_t smem = fixed + (size_t)stages * kStageBytes;
  auto kern = affine_qmv_w8g64_kernel<GS>;
  static int granted[64] = {};
  if (int rc = ensure_dynamic_smem(reinterpret_cast<const void*>(kern), granted, smem)) { return rc; }
  const int cap = 2 * num_sms();
  p.experts = d.expert ? (int)d.experts : 1;
  p.norm_w = static_cast<const uint16_t*>(d.norm_w);
  p.eps = d.eps;
  for (int64_t m = 0; m < M; ++m) {  // every row streams the weight again, as in the reference
    // expert gather: row m is a (token, expert) pair; the pairs of one token share its x row
    const bool row_gather = d.row_map && d.row_gather;   // the x row is read on the GPU (row_map[m])
    const int64_t x_row = row_gather ? 0 : (d.expert && d.x_div > 1) ? m / d.x_div : m;
    p.x = static_cast<const uint16_t*>(x) + x_row * K;
    p.eid = d.expert ? d.expert + (d.expert_div > 1 ? m / d.expert_div : m) : nullptr;
    p.vrow = d.row_map ? d.row_map + m : nullptr;
    p.xrow = row_gather ? d.row_map + m : nullptr;
    p.y = static_cast<__nv_bfloat16*>(y) + m * y_pitch;
    if (d.epilogue == VPQ_EPILOGUE_ADD || d.epilogue == VPQ_EPILOGUE_GELU_MUL || d.epilogue == VPQ_EPILOGUE_SILU_MUL) {
      p.aux = static_cast<const uint16_t*>(d.aux) + m * N;
    } else if (d.epilogue == VPQ_EPILOGUE_QKV) {
      p.aux = static_cast<const uint16_t*>(d.aux) + m * d.k_rows;
      p.y3 = static_cast<__nv_bfloat16*>(d.y3) + m * (N - d.q_rows - d.k_rows);
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)(p.row_tiles < cap ? p.row_tiles : cap), 1, 1);
    cfg.blockDim = dim3(kThreads, 1, 1);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    VPQ_CUDA_OK(cudaLaunchKernelEx(&cfg, kern, p, stages, cap_kt));
  }
  return VPQ_OK;
}
}  // namespace

// The shared-expert gate of a mixture-of-experts block: g[m] = sigmoid(dequant(w[1, K]) . x[m]), w one
// 8-bit group-64 row. Replaces affine_moe_gate_w8g64 (gpu-kernels/metal/quant/affine_qmv.metal:1323-1347),
// which has the same decomposition: one warp per row of x, lanes striding over k (here four consecutive k
// = one packed word per step), a warp sum, lane 0 writes. Latency-bound by construction (K bytes of
// weight): a dozen microseconds of HBM time saved by nothing cleverer.
namespace vpq {
__global__ void __launch_bounds__(128)
affine_moe_gate_w8g64_kernel(const uint32_t* __restrict__ w, const uint16_t* __restrict__ scales,
                             const uint16_t* __restrict__ biases, const uint16_t* __restrict__ x,
                             __nv_bfloat16* __restrict__ out, int K, int M) {
  asm volatile("griddepcontrol.wait;" ::: "memory");  // x may come from the previous kernel
  const int lane = threadIdx.x & 31;
  const int row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (row >= M) { return; }
  const uint2* xr = reinterpret_cast<const uint2*>(x + (size_t)row * K);
  float acc = 0.0f;
  for (int wd = lane; wd < (K >> 2); wd += 32) {   // word wd = k 4 wd .. 4 wd + 3, all in group wd / 16
    const float s = __uint_as_float((uint32_t)__ldg(scales + (wd >> 4)) << 16);
    const float b = __uint_as_float((uint32_t)__ldg(biases + (wd >> 4)) << 16);
    const uint32_t q = __ldg(w + wd);
    const uint2 xv = xr[wd];
    acc = __fmaf_rn(dequant_f32(s, q & 0xffu, b), __uint_as_float(xv.x << 16), acc);
    acc = __fmaf_rn(dequant_f32(s, (q >> 8) & 0xffu, b), __uint_as_float(xv.x & 0xffff0000u), acc);
    acc = __fmaf_rn(dequant_f32(s, (q >> 16) & 0xffu, b), __uint_as_float(xv.y << 16), acc);
    acc = __fmaf_rn(dequant_f32(s, q >> 24, b), __uint_as_float(xv.y & 0xffff0000u), acc);
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) { acc += __shfl_xor_sync(0xffffffffu, acc, o); }
  if (lane == 0) { out[row] = __float2bfloat16_rn(1.0f / (1.0f + expf(-acc))); }
}
}  // namespace vpq

extern "C" int vpq_affine_moe_gate_w8g64_bf16(const uint32_t* w, const void* scales, const void* biases, const void* x,
                                              void* out, int64_t K, int64_t M, void* stream) {
  clear_error();
  if (!w || !scales || !biases || !x || !out) { return fail(VPQ_ERR_INVALID_ARG, "affine_moe_gate_w8g64: null pointer"); }
  if (K <= 0 || M <= 0 || (K % 64) != 0 || K > (1 << 24) || M > (1 << 24)) {
    return fail(VPQ_ERR_INVALID_ARG, "affine_moe_gate_w8g64: need K>0, M>0, K%%64==0 (K=%lld M=%lld)", (long long)K, (long long)M);
  }
  if ((reinterpret_cast<uintptr_t>(w) & 3) || (reinterpret_cast<uintptr_t>(x) & 7) || (reinterpret_cast<uintptr_t>(scales) & 1) ||
      (reinterpret_cast<uintptr_t>(biases) & 1) || (reinterpret_cast<uintptr_t>(out) & 1)) {
    return fail(VPQ_ERR_ALIGNMENT, "affine_moe_gate_w8g64: w must be 4-byte aligned, x 8-byte");
  }
  if (int rc = require_sm100()) { return rc; }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)((M + 3) / 4), 1, 1);
  cfg.blockDim = dim3(128, 1, 1);
  cfg.stream = static_cast<cudaStream_t>(stream);
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  VPQ_CUDA_OK(cudaLaunchKernelEx(&cfg, affine_moe_gate_w8g64_kernel, w, static_cast<const uint16_t*>(scales),
                                 static_cast<const uint16_t*>(biases), static_cast<const uint16_t*>(x),
                                 static_cast<__nv_bfloat16*>(out), (int)K, (int)M));
  return VPQ_OK;
}

extern "C" int vpq_affine_qmv_w8g64_bf16(const uint32_t* w, const void* scales, const void* biases, const void* x,
                                         void* y, int64_t K, int64_t N, int64_t M, void* stream) {
  clear_error();
  vpq_linear_desc d;
  std::memset(&d, 0, sizeof(d));
  d.w = w;
  d.scales = scales;
  d.biases = biases;
  d.x = x;
  d.y = y;
  d.K = K;
  d.N = N;
  d.M = M;
  return launch_w8<64>("affine_qmv_w8g64", d, stream);
}

extern "C" int vpq_affine_qmv_w8g64_bf16_fused(const vpq_linear_desc* desc_host, void* stream) {
  clear_error();
  if (!desc_host) { return fail(VPQ_ERR_INVALID_ARG, "affine_qmv_w8g64 (fused store): null descriptor"); }
  return launch_w8<64>("affine_qmv_w8g64 (fused store)", *desc_host, stream);
}

// 8-bit weights in groups of 32 (scales / biases [N, K/32]): one descriptor, any VPQ_EPILOGUE_*.
extern "C" int vpq_affine_qmv_w8g32_bf16_fused(const vpq_linear_desc* desc_host, void* stream) {
  clear_error();
  if (!desc_host) { return fail(VPQ_ERR_INVALID_ARG, "affine_qmv_w8g32: null descriptor"); }
  return launch_w8<32>("affine_qmv_w8g32", *desc_host, stream);
}
