// qmv_batch.cu -- small-batch decode GEMV: M = 2..4 rows of x against one stream of the weights
// (group 64), and the group-32 GEMV (1..2 rows per stream), one kernel templated over the group size.
//
// y[m,n] = sum_k x[m,k] * (s[n,k/64] * q[n,k] + b[n,k/64]),  f32 accumulate, weights read once.
// Replaces affine_qmv_batch_w4g64 / affine_qmv_batch4_w4g64 (qmv_batch_impl<T,64,4,MAXM>,
// gpu-kernels/metal/quant/affine_qmv.metal:1553-1705): decode of several branches / MTP verify.
//
// Same skeleton as the M = 1 kernel in qmv.cu (a producer warp streams [16 rows x 128 bytes] TMA
// boxes of packed nibbles plus the span's scales and biases into a ring of 18 KB stages; eight
// consumer warps split K, warp w takes box w of every stage), but the arithmetic is arranged so
// that extra rows of x are nearly free:
//  * nibbles become fp16 1024 + q / 64 + q with one LOP3 per two nibbles (plus one shift per
//    word) and go, unscaled, through mma.sync.m16n8k16 against x in fp16 (each row of x scaled by
//    its own power of two so that max |x| lands in [2^14, 2^15): products are exact, accumulation
//    is f32, the scale is undone exactly at the end);
//  * the eight accumulator columns are (row of x, group parity): column c is fed by the lanes
//    with g == c, with row c >> 1 of x where the lane's k chunk lies in group c & 1 of the k tile
//    and zeros elsewhere. Lane t of a quad then holds, for row t of x, the sums of both groups of
//    a k tile for both of its W rows, and folds them with the groups' scales and biases:
//    res += s * (acc - surplus) + b * sum(x), where surplus is what the 1024 / 64 offsets added.
// The M = 1 kernel uses exact integer arithmetic instead (three digit columns per group); there
// every further row of x would cost about half of the first. Here four rows cost what one does,
// so a batch of 4 streams the weights at ~0.6 of the M = 1 rate: ~2.5x over four serial GEMVs.
// Rows are not bit-identical to the M = 1 kernel's (f32 rounding level differences).
// x rows live in shared memory (2 bytes per value per row, per CTA): the rows per pass are
// limited by that (4 up to K = 5120, 2 up to K = 8192; longer rows go through the M = 1 kernel
// one at a time); larger batches run several passes.
#include "vpq_sm100.cuh"

#include <cstring>

namespace vpq {

__device__ uint32_t g_qmvb_status;  // 0, or (site << 8) | role of the first bounded wait that gave up

namespace {

constexpr int kConsWarps = 8;
constexpr int kConsThreads = kConsWarps * 32;
constexpr int kThreads = kConsThreads + 32;  // + producer warp
constexpr int kBoxBytes = 16 * 128;          // one TMA box: 16 rows x 128 bytes (256 k)
constexpr int kBoxesPerStage = 8;            // a stage spans 2048 k
constexpr int kStageW = kBoxesPerStage * kBoxBytes;
// scales + biases of a stage's span: 2 x [16 rows x 2048 / GROUP groups] bf16
template <int GROUP> constexpr int stage_sz() { return 2 * 16 * (2048 / GROUP) * 2; }
template <int GROUP> constexpr int stage_bytes() { return kStageW + stage_sz<GROUP>(); }
constexpr int kMaxStages = 6;
constexpr int kRedSlots = 8;                 // row tiles whose cross-warp sums may be pending
constexpr int kMaxRows = 4;                  // rows of x per pass

__device__ __forceinline__ void mma_f16_16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                              uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 "
      "{%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void mma_f16_16816_first(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2,
                                                    uint32_t a3, uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 "
      "{%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
      : "=f"(c[0]), "=f"(c[1]), "=f"(c[2]), "=f"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "f"(0.0f));
}
// fp16 pairs straight out of a packed word:
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

struct alignas(64) BatchProblem {
  CUtensorMap mw, ms, mz;      // packed weights [N, K/8] u32; scales, biases [N, K/64] (valid if scales_tma)
  const uint16_t* scales;
  const uint16_t* biases;
  const uint16_t* x;           // M rows of K bf16
  __nv_bfloat16* y;            // M rows of N outputs
  int K, N, M;
  int row_tiles;
  int scales_tma;
  int scale_only;              // 1: no biases are read, every group's bias is -8 * its scale (GGUF Q4_0 repacks)
  int epilogue;                // kEpi*: what the store does with a row's sums (see fused_store)
  int q_rows, k_rows;
  int y_pitch, aux_pitch, y3_pitch;  // elements between consecutive rows of x in y / aux / y3
  const uint16_t* aux;
  __nv_bfloat16* y3;
  const uint16_t* norm_w;      // not null: every row of x is RMS-normalised with these K weights while it is staged
  float eps;                   // RMSNorm epsilon
};

// GROUP = 64: columns = (row of x 0..3, group parity). GROUP = 32 (the reference's affine_qmv_w4g32,
// gpu-kernels/metal/quant/affine_qmv.metal:303-320: GGUF Q4_0 repacks): a k tile of 128 has four
// groups and a lane's 32-nibble chunk is exactly one of them, so columns = (row of x 0..1, group
// 0..3); lanes t and t ^ 1 of a quad then hold the two halves of a row's sum.
// XREGS: 16-byte chunks of x a thread keeps in registers between the staging passes. 8 covers four
// rows of K = 4096 but spills 140 bytes per thread, 6 (three rows) spills 48, 4 does not spill and
// covers one or two rows of K = 4096 (the group-32 GEMVs and the two-row batch), whose launches are
// short enough for the spill traffic to show (an SM running two of these CTAs has less L1 than the
// spills need).
template <int GROUP, int XREGS>
__global__ void __launch_bounds__(kThreads, 2)
affine_qmv_batch_w4_kernel(const __grid_constant__ BatchProblem P, int stages, int cap_kt) {
  constexpr int GPT = 128 / GROUP;            // groups per k tile
  constexpr int GPS = 2048 / GROUP;           // groups per stage
  constexpr int kStageSZ = stage_sz<GROUP>();
  constexpr int kStageBytes = stage_bytes<GROUP>();
  extern __shared__ unsigned char smem_dyn[];
  const uint32_t raw = smem_u32(smem_dyn);
  const uint32_t base = (raw + 1023u) & ~1023u;  // swizzled boxes need 1024-byte alignment
  unsigned char* base_ptr = smem_dyn + (base - raw);
  const int M = P.M, K = P.K, N = P.N;

  unsigned char* p0 = base_ptr + (size_t)stages * kStageBytes;
  uint4* xperm = reinterpret_cast<uint4*>(p0);                   // [M][cap_kt][4 quarters][4 t] x 16 B
  uint4* zero256 = xperm + (size_t)M * cap_kt * 16;              // 320 bytes of zeros (also read as float2 zeros)
  float2* xg = reinterpret_cast<float2*>(zero256 + 20);          // [M][2*cap_kt] per group: surplus, sum of x
  float* unscale = reinterpret_cast<float*>(xg + (size_t)M * GPT * cap_kt);  // [kMaxRows]
  float* red = unscale + kMaxRows;                               // [kRedSlots][kConsWarps][kMaxRows][16]
  uint32_t* red_cnt = reinterpret_cast<uint32_t*>(red + kRedSlots * kConsWarps * kMaxRows * 16);
  uint32_t* amax_buf = red_cnt + kRedSlots;                      // [kConsWarps][kMaxRows]
  uint64_t* bars = reinterpret_cast<uint64_t*>(amax_buf + kConsWarps * kMaxRows);
  volatile uint32_t* abort_flag = reinterpret_cast<volatile uint32_t*>(bars + 2 * kMaxStages);
  const uint32_t bar0 = smem_u32(bars);
  auto bar_full = [&](int s) { return bar0 + 8u * s; };
  auto bar_empty = [&](int s) { return bar0 + 8u * (kMaxStages + s); };

  const int lane = threadIdx.x & 31;
  const int warp = threadIdx.x >> 5;
  const int NB = (K + 255) >> 8;                               // 128-byte boxes per row
  const int SPT = (NB + kBoxesPerStage - 1) / kBoxesPerStage;  // stages per row tile
  const int KT = NB * 2;                                       // k tiles per row (x is zero past K)
  // every CTA takes one contiguous run of row tiles
  const int gt_begin = (int)(((int64_t)P.row_tiles * blockIdx.x) / gridDim.x);
  const int gt_end = (int)(((int64_t)P.row_tiles * (blockIdx.x + 1)) / gridDim.x);

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
    if (lane == 0) {
      uint32_t it = 0;
      bool ok = true;
      const bool sz_tma = P.scales_tma != 0;
      const uint32_t sz_bytes = sz_tma ? (P.scale_only ? kStageSZ / 2 : kStageSZ) : 0;
      for (int tile = gt_begin; tile < gt_end && ok; ++tile) {
        for (int st = 0; st < SPT; ++st, ++it) {
          const int s = it % stages;
          const uint32_t ph = (it / stages) & 1u;
          if (!mbar_wait(bar_empty(s), ph ^ 1u, (1u << 8) | kRoleProducer, abort_flag, &g_qmvb_status)) {
            ok = false;
            break;
          }
          const int nb = min(kBoxesPerStage, NB - st * kBoxesPerStage);
          const uint32_t dst = base + (uint32_t)s * kStageBytes;
          mbar_expect_tx(bar_full(s), (uint32_t)nb * kBoxBytes + sz_bytes);
          for (int b = 0; b < nb; ++b) {
            tma_load_2d(dst + b * kBoxBytes, &P.mw, bar_full(s), (st * kBoxesPerStage + b) * 32, tile * 16);
          }
          if (sz_tma) {
            tma_load_2d(dst + kStageW, &P.ms, bar_full(s), st * GPS, tile * 16);
            if (!P.scale_only) { tma_load_2d(dst + kStageW + kStageSZ / 2, &P.mz, bar_full(s), st * GPS, tile * 16); }
          }
        }
      }
      // Never leave with a copy still in flight: wait for the last load of every stage.
      for (int s = 0; s < stages; ++s) {
        if (it > (uint32_t)s) {
          const uint32_t last = ((it - 1 - s) / stages) * stages + s;
          mbar_wait(bar_full(s), (last / stages) & 1u, (2u << 8) | kRoleProducer, abort_flag, &g_qmvb_status);
        }
      }
    }
    return;
  }

  // ---------------------------------------------------------------- consumers
  const int g = lane >> 2, t = lane & 3;
  const int rho = (g >> 1) | ((g & 1) << 2);  // stage row of MMA row g (g+8 -> rho+8): bank-conflict-free

  asm volatile("griddepcontrol.wait;" ::: "memory");  // x may come from the previous kernel

  // ---- staging of the M rows of x as fp16 (all consumer warps together). Per row: the scale
  // 2^(141 - e) puts max |x| into [2^14, 2^15) (every bf16 value within 2^-28 of the maximum is
  // then exact in fp16). 8 consecutive values x0..x7 become the B-fragment registers (x0,x4)
  // (x1,x5) (x2,x6) (x3,x7). Per group of 64: xg.x = 1024 * sum(even k) + 64 * sum(odd k), the
  // surplus the nibble offsets add to the accumulator; xg.y = sum of all 64, for the bias term.
  {
    const int chunks = KT * 16;          // 16-byte chunks of one padded row
    const int total = M * chunks;
    uint32_t amax[kMaxRows] = {0, 0, 0, 0};
    constexpr int kXRegs = XREGS;
    uint4 xin[kXRegs];
    auto load_raw = [&](int i) {
      const int m = i / chunks, ci = i - m * chunks;
      uint4 in = make_uint4(0, 0, 0, 0);
      if (i < total && ci * 8 < K) { in = *reinterpret_cast<const uint4*>(P.x + (size_t)m * K + ci * 8); }
      return in;
    };
    // With norm_w every row is first RMS-normalised as the reference's fused kernel does
    // (affine_qmv_qkv_rms_w4g32 / _w4g64, gpu-kernels/metal/quant/affine_qmv.metal:570-694): sum of
    // squares in f32 over the row (partial sums of the warps through shared memory, the consumers'
    // barrier), x <- bf16(x * rsqrt(mean + eps) * norm_w); scales and digits are taken from that.
    const uint16_t* nw = P.norm_w;
    float inv[kMaxRows] = {1.0f, 1.0f, 1.0f, 1.0f};
    auto normalise = [&](int i, uint4 in) {
      const int m = i / chunks, ci = i - m * chunks;
      if (!(i < total && ci * 8 < K)) { return in; }
      const float r = m == 0 ? inv[0] : m == 1 ? inv[1] : m == 2 ? inv[2] : inv[3];
      const uint4 n = __ldg(reinterpret_cast<const uint4*>(nw + ci * 8));
      const uint32_t v[4] = {in.x, in.y, in.z, in.w}, w4[4] = {n.x, n.y, n.z, n.w};
      uint32_t o[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float lo = __fmul_rn(__fmul_rn(__uint_as_float(v[j] << 16), r), __uint_as_float(w4[j] << 16));
        const float hi = __fmul_rn(__fmul_rn(__uint_as_float(v[j] & 0xffff0000u), r), __uint_as_float(w4[j] & 0xffff0000u));
        asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(o[j]) : "f"(hi), "f"(lo));
      }
      return make_uint4(o[0], o[1], o[2], o[3]);
    };
    auto load_chunk = [&](int i) { return nw ? normalise(i, load_raw(i)) : load_raw(i); };
    auto fold_amax = [&](int i, const uint4& in) {
      const int m = i / chunks;
      const uint32_t v[4] = {in.x, in.y, in.z, in.w};
      uint32_t a = 0;
#pragma unroll
      for (int j = 0; j < 4; ++j) { a = max(a, max(v[j] & 0x7fffu, (v[j] >> 16) & 0x7fffu)); }
#pragma unroll
      for (int r = 0; r < kMaxRows; ++r) { amax[r] = (r == m) ? max(amax[r], a) : amax[r]; }
    };
#pragma unroll
    for (int r = 0; r < kXRegs; ++r) { xin[r] = load_raw(threadIdx.x + r * kConsThreads); }
    if (nw) {
      float sq[kMaxRows] = {0.0f, 0.0f, 0.0f, 0.0f};
      auto fold_sq = [&](int i, const uint4& in) {
        const int m = i / chunks;
        const uint32_t v[4] = {in.x, in.y, in.z, in.w};
        float a = 0.0f;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float lo = __uint_as_float(v[j] << 16), hi = __uint_as_float(v[j] & 0xffff0000u);
          a = __fmaf_rn(lo, lo, a);
          a = __fmaf_rn(hi, hi, a);
        }
#pragma unroll
        for (int r = 0; r < kMaxRows; ++r) { sq[r] += (r == m) ? a : 0.0f; }
      };
#pragma unroll
      for (int r = 0; r < kXRegs; ++r) { fold_sq(threadIdx.x + r * kConsThreads, xin[r]); }
      for (int i = threadIdx.x + kXRegs * kConsThreads; i < total; i += kConsThreads) { fold_sq(i, load_raw(i)); }
      float* sq_buf = reinterpret_cast<float*>(amax_buf);   // [kConsWarps][kMaxRows], free until the amax pass
#pragma unroll
      for (int r = 0; r < kMaxRows; ++r) {
        float a = sq[r];
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) { a += __shfl_xor_sync(0xffffffffu, a, o); }
        if (lane == 0) { sq_buf[warp * kMaxRows + r] = a; }
      }
      asm volatile("bar.sync 1, %0;" ::"n"(kConsThreads) : "memory");
#pragma unroll
      for (int r = 0; r < kMaxRows; ++r) {
        float tot = 0.0f;
#pragma unroll
        for (int ww = 0; ww < kConsWarps; ++ww) { tot += sq_buf[ww * kMaxRows + r]; }
        inv[r] = __frsqrt_rn(__fadd_rn(__fdiv_rn(tot, (float)K), P.eps));
      }
      asm volatile("bar.sync 1, %0;" ::"n"(kConsThreads) : "memory");  // sq_buf is read: the amax pass may reuse it
#pragma unroll
      for (int r = 0; r < kXRegs; ++r) { xin[r] = normalise(threadIdx.x + r * kConsThreads, xin[r]); }
    }
#pragma unroll
    for (int r = 0; r < kXRegs; ++r) { fold_amax(threadIdx.x + r * kConsThreads, xin[r]); }
    for (int i = threadIdx.x + kXRegs * kConsThreads; i < total; i += kConsThreads) { fold_amax(i, load_chunk(i)); }
#pragma unroll
    for (int r = 0; r < kMaxRows; ++r) {
      const uint32_t a = __reduce_max_sync(0xffffffffu, amax[r]);
      if (lane == 0) { amax_buf[warp * kMaxRows + r] = a; }
    }
    asm volatile("bar.sync 1, %0;" ::"n"(kConsThreads) : "memory");  // consumers only
    float x_scale[kMaxRows];
#pragma unroll
    for (int r = 0; r < kMaxRows; ++r) {
      uint32_t a = 0;
#pragma unroll
      for (int ww = 0; ww < kConsWarps; ++ww) { a = max(a, amax_buf[ww * kMaxRows + r]); }
      int e = (int)(a >> 7);               // biased exponent of the largest magnitude
      e = min(max(e, 16), 240);            // all-zero / denormal / huge x: keep both factors normal
      x_scale[r] = __uint_as_float((uint32_t)(268 - e) << 23);  // 2^(141 - e)
      if (threadIdx.x == r) { unscale[r] = __uint_as_float((uint32_t)(e - 14) << 23); }  // its exact inverse
    }
    auto convert_chunk = [&](int i, const uint4& in) {  // called by whole warps: shuffles inside
      const bool live = i < total;
      const int m = live ? i / chunks : 0, ci = live ? i - m * chunks : 0;
      const float sc = m == 0 ? x_scale[0] : m == 1 ? x_scale[1] : m == 2 ? x_scale[2] : x_scale[3];
      const uint32_t v[4] = {in.x, in.y, in.z, in.w};
      uint32_t hb[4];
      float se = 0.0f, so = 0.0f;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const __half2 h = __floats2half2_rn(__uint_as_float(v[j] << 16) * sc, __uint_as_float(v[j] & 0xffff0000u) * sc);
        const float2 f = __half22float2(h);  // what the tensor core will see
        se += f.x;
        so += f.y;
        hb[j] = *reinterpret_cast<const uint32_t*>(&h);
      }
      uint4 out;
      out.x = __byte_perm(hb[0], hb[2], 0x5410);
      out.y = __byte_perm(hb[0], hb[2], 0x7632);
      out.z = __byte_perm(hb[1], hb[3], 0x5410);
      out.w = __byte_perm(hb[1], hb[3], 0x7632);
      const int kt = ci >> 4, tt = (ci >> 2) & 3, q = ci & 3;
      if (live) { xperm[(size_t)m * cap_kt * 16 + (kt * 4 + q) * 4 + tt] = out; }
#pragma unroll
      for (int off = 1; off < GROUP / 8; off <<= 1) {
        se += __shfl_xor_sync(0xffffffffu, se, off);
        so += __shfl_xor_sync(0xffffffffu, so, off);
      }
      if (live && (ci % (GROUP / 8)) == 0) {
        xg[(size_t)m * GPT * cap_kt + ci / (GROUP / 8)] = make_float2(__fmaf_rn(1024.0f, se, 64.0f * so), se + so);
      }
    };
#pragma unroll
    for (int r = 0; r < kXRegs; ++r) {
      const int i = threadIdx.x + r * kConsThreads;
      if (i - lane < total) { convert_chunk(i, xin[r]); }  // warp-uniform
    }
    for (int i = threadIdx.x + kXRegs * kConsThreads; i - lane < total; i += kConsThreads) {
      convert_chunk(i, load_chunk(i));
    }
    asm volatile("bar.sync 1, %0;" ::"n"(kConsThreads) : "memory");
  }

  // Column c of an MMA (fed by the lanes with g == c) stands for (row c >> 1 of x, group c & 1 of
  // the k tile): those lanes read that row's fragments where their chunk t lies in that group
  // (chunks 0, 1 -> first group, 2, 3 -> second) and zeros otherwise, from a block laid out like
  // one k tile of xperm (+4: its quarter q sits in the banks quarter q+1 of the data uses).
  const int col_row = g / GPT;                        // row of x this lane's column stands for
  const int chunk_group = GPT == 2 ? (t >> 1) : t;    // group of the k tile this lane's chunk lies in
  const bool real = col_row < M && ((g % GPT) == chunk_group);
  const uint4* xb_base = real ? xperm + (size_t)col_row * cap_kt * 16 + t : zero256 + 4;
  const int xb_kt = real ? 16 : 0;
  // Lane t of a quad folds its accumulator columns 2t, 2t+1: row t of x, both groups (GROUP 64);
  // row t >> 1 of x, groups 2 (t & 1) and 2 (t & 1) + 1 of the k tile (GROUP 32).
  const int m_lane = GPT == 2 ? t : (t >> 1);
  const int gbase = GPT == 2 ? 0 : 2 * (t & 1);
  const bool row_live = m_lane < M;
  const float2* xg_row = row_live ? xg + (size_t)m_lane * GPT * cap_kt : reinterpret_cast<const float2*>(zero256);
  const int xg_step = row_live ? 1 : 0;

  // byte offsets of this lane's two 16-byte reads inside its box, per half (k tile) of the box
  const uint32_t off_h0 = (uint32_t)rho * 128u + (uint32_t)(((0 + t) ^ rho) << 4);
  const uint32_t off_h1 = (uint32_t)rho * 128u + (uint32_t)(((4 + t) ^ rho) << 4);
  // this lane's two groups of the box's first k tile, row rho, in the stage's scales (the second
  // k tile: + 2 GPT bytes; row rho + 8: + 8 rows; biases: + kStageSZ / 2)
  const uint32_t sz_off = (uint32_t)kStageW + (uint32_t)rho * (GPS * 2) + (uint32_t)(warp * 2 * GPT + gbase) * 2u;
  constexpr uint32_t kRow8 = 8u * GPS * 2u;
  const bool sz_tma = P.scales_tma != 0;
  const bool scale_only = P.scale_only != 0;
  const int G = K / GROUP;
  // a pair of bf16 scales -> the pair of biases -8 * scale (exact: a power of two times a bf16 value)
  auto neg8 = [](uint32_t s2) {
    const float a = -8.0f * __uint_as_float(s2 << 16), b = -8.0f * __uint_as_float(s2 & 0xffff0000u);
    return (__float_as_uint(a) >> 16) | (__float_as_uint(b) & 0xffff0000u);
  };

  uint32_t tile_seq = 0, ph = 0;
  int s = 0;
  bool ok = true;
  for (int tile = gt_begin; tile < gt_end && ok; ++tile, ++tile_seq) {
    float res_a = 0.0f, res_b = 0.0f;  // W rows rho and rho + 8 of the tile, row t of x
    for (int st = 0; st < SPT; ++st) {
      if (!warp_wait(bar_full(s), ph, (1u << 8) | kRoleConsumer, abort_flag, &g_qmvb_status)) {
        ok = false;
        break;
      }
      const unsigned char* sb = base_ptr + (size_t)s * kStageBytes;
      const int kt0 = st * 16 + warp * 2;  // this warp's box holds k tiles kt0 and kt0 + 1
      if (kt0 < KT) {
        const unsigned char* box = sb + warp * kBoxBytes;
        const uint4 ra0 = *reinterpret_cast<const uint4*>(box + off_h0);
        const uint4 rb0 = *reinterpret_cast<const uint4*>(box + off_h0 + 1024);
        const uint4 ra1 = *reinterpret_cast<const uint4*>(box + off_h1);
        const uint4 rb1 = *reinterpret_cast<const uint4*>(box + off_h1 + 1024);
        uint32_t sa[2], sb2[2], za[2], zb[2];  // per k tile: this lane's two groups' scales / biases, rows rho, rho + 8
        if (sz_tma) {
          if constexpr (GROUP == 64) {  // the two k tiles' pairs are adjacent: one 8-byte load each
            const unsigned char* q = sb + sz_off;
            const uint2 a = *reinterpret_cast<const uint2*>(q), b = *reinterpret_cast<const uint2*>(q + kRow8);
            sa[0] = a.x, sa[1] = a.y, sb2[0] = b.x, sb2[1] = b.y;
            if (!scale_only) {
              const uint2 c = *reinterpret_cast<const uint2*>(q + kStageSZ / 2);
              const uint2 e = *reinterpret_cast<const uint2*>(q + kStageSZ / 2 + kRow8);
              za[0] = c.x, za[1] = c.y, zb[0] = e.x, zb[1] = e.y;
            }
          } else {
#pragma unroll
            for (int h = 0; h < 2; ++h) {
              const unsigned char* q = sb + sz_off + h * (2 * GPT);
              sa[h] = *reinterpret_cast<const uint32_t*>(q);
              sb2[h] = *reinterpret_cast<const uint32_t*>(q + kRow8);
              if (!scale_only) {
                za[h] = *reinterpret_cast<const uint32_t*>(q + kStageSZ / 2);
                zb[h] = *reinterpret_cast<const uint32_t*>(q + kStageSZ / 2 + kRow8);
              }
            }
          }
        } else {
          // clamped onto valid data: a clamped group meets x == 0, a clamped row is never stored
          const int64_t r_a = min(tile * 16 + rho, N - 1), r_b = min(tile * 16 + rho + 8, N - 1);
          auto pair = [](const uint16_t* p, int64_t i, int64_t j) { return ldg_nc_u16(p + i) | (ldg_nc_u16(p + j) << 16); };
#pragma unroll
          for (int h = 0; h < 2; ++h) {
            const int g0 = min((kt0 + h) * GPT + gbase, G - 1), g1 = min((kt0 + h) * GPT + gbase + 1, G - 1);
            sa[h] = pair(P.scales, r_a * G + g0, r_a * G + g1);
            sb2[h] = pair(P.scales, r_b * G + g0, r_b * G + g1);
            if (!scale_only) {
              za[h] = pair(P.biases, r_a * G + g0, r_a * G + g1);
              zb[h] = pair(P.biases, r_b * G + g0, r_b * G + g1);
            }
          }
        }
        if (scale_only) {
#pragma unroll
          for (int h = 0; h < 2; ++h) { za[h] = neg8(sa[h]), zb[h] = neg8(sb2[h]); }
        }
        const int kt1 = kt0 + 1;
        float c0[4], d0[4], c1[4], d1[4];  // four independent accumulator chains
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
        // [0] = (W row rho, first group) [1] = (rho, second) [2] = (rho + 8, first) [3] = (rho + 8, second)
        const float4 xs0 = *reinterpret_cast<const float4*>(xg_row + (kt0 * GPT + gbase) * xg_step);  // this lane's two groups
        const float4 xs1 = *reinterpret_cast<const float4*>(xg_row + (kt1 * GPT + gbase) * xg_step);
        auto lo = [](uint32_t v) { return __uint_as_float(v << 16); };
        auto hi = [](uint32_t v) { return __uint_as_float(v & 0xffff0000u); };
        res_a = __fmaf_rn(lo(sa[0]), (c0[0] + d0[0]) - xs0.x, res_a);
        res_a = __fmaf_rn(lo(za[0]), xs0.y, res_a);
        res_a = __fmaf_rn(hi(sa[0]), (c0[1] + d0[1]) - xs0.z, res_a);
        res_a = __fmaf_rn(hi(za[0]), xs0.w, res_a);
        res_a = __fmaf_rn(lo(sa[1]), (c1[0] + d1[0]) - xs1.x, res_a);
        res_a = __fmaf_rn(lo(za[1]), xs1.y, res_a);
        res_a = __fmaf_rn(hi(sa[1]), (c1[1] + d1[1]) - xs1.z, res_a);
        res_a = __fmaf_rn(hi(za[1]), xs1.w, res_a);
        res_b = __fmaf_rn(lo(sb2[0]), (c0[2] + d0[2]) - xs0.x, res_b);
        res_b = __fmaf_rn(lo(zb[0]), xs0.y, res_b);
        res_b = __fmaf_rn(hi(sb2[0]), (c0[3] + d0[3]) - xs0.z, res_b);
        res_b = __fmaf_rn(hi(zb[0]), xs0.w, res_b);
        res_b = __fmaf_rn(lo(sb2[1]), (c1[2] + d1[2]) - xs1.x, res_b);
        res_b = __fmaf_rn(lo(zb[1]), xs1.y, res_b);
        res_b = __fmaf_rn(hi(sb2[1]), (c1[3] + d1[3]) - xs1.z, res_b);
        res_b = __fmaf_rn(hi(zb[1]), xs1.w, res_b);
      }
      __syncwarp();
      if (lane == 0) { mbar_arrive(bar_empty(s)); }  // this warp's part of the stage is in registers
      if (++s == stages) {
        s = 0;
        ph ^= 1u;
      }
    }
    if (!ok) { break; }
    // The 8 warps' K slices: every warp posts its 16 x kMaxRows partial sums and moves on; the
    // warp that posts last adds them in warp order (the result does not depend on arrival order)
    // and stores. The ring of kRedSlots tiles is deeper than a warp can run ahead.
    const int slot = tile_seq % kRedSlots;
    if (GPT == 4) {  // lanes t and t ^ 1 hold the two halves (groups 0 1 / 2 3 of every k tile) of one row of x
      res_a += __shfl_xor_sync(0xffffffffu, res_a, 1);
      res_b += __shfl_xor_sync(0xffffffffu, res_b, 1);
    }
    if (GPT == 2 || (t & 1) == 0) {
      float* mine = red + ((size_t)(slot * kConsWarps + warp) * kMaxRows + m_lane) * 16;
      const float us = unscale[m_lane];
      mine[rho] = res_a * us;
      mine[rho + 8] = res_b * us;
    }
    __syncwarp();
    uint32_t last = 0;
    if (lane == 0) {
      __threadfence_block();
      last = atomicAdd(&red_cnt[slot], 1u) == (uint32_t)(kConsWarps - 1);
    }
    last = __shfl_sync(0xffffffffu, last, 0);
    if (last) {
      __threadfence_block();
#pragma unroll
      for (int half = 0; half < 2; ++half) {
        const int idx = lane + 32 * half, m = idx >> 4, r = idx & 15;
        float v = 0.0f;
#pragma unroll
        for (int ww = 0; ww < kConsWarps; ++ww) {
          v += *reinterpret_cast<volatile float*>(&red[((size_t)(slot * kConsWarps + ww) * kMaxRows + m) * 16 + r]);
        }
        const int row = (tile << 4) + r;
        const bool live = m < M;  // every lane takes part in the store's shuffles; idle ones store nothing
        fused_store(P.epilogue, v, row, live ? N : 0, r, P.y + (size_t)m * P.y_pitch, P.aux + (size_t)m * P.aux_pitch,
                    P.y3 + (size_t)m * P.y3_pitch, live ? P.q_rows : 0, live ? P.k_rows : 0, 0xffffffffu);
      }
      __syncwarp();
      if (lane == 0) { red_cnt[slot] = 0; }
    }
  }
}

// ------------------------------------------------------------------ host side
template <int GROUP>
size_t fixed_smem(int rows, int cap_kt) {
  return 1024 /*alignment slack*/ + (size_t)rows * cap_kt * 256 + 320 + (size_t)rows * (128 / GROUP) * cap_kt * 8 +
         kMaxRows * 4 + (size_t)kRedSlots * kConsWarps * kMaxRows * 16 * 4 + kRedSlots * 4 +
         kConsWarps * kMaxRows * 4 + 2 * kMaxStages * 8 + 16;
}
constexpr size_t kSmemBudget = 112 * 1024;  // two CTAs per SM

// Rows of x one pass can hold next to at least three ring stages (with fewer the stream stalls
// and M serial GEMVs are faster); at most 4 (group 64) or 2 (group 32: four groups per k tile
// take the accumulator columns of two rows).
template <int GROUP>
int rows_per_pass(int cap_kt) {
  int rows = GROUP == 64 ? kMaxRows : 2;
  while (rows > 1 && fixed_smem<GROUP>(rows, cap_kt) + 3 * (size_t)stage_bytes<GROUP>() > kSmemBudget) { --rows; }
  return rows;
}

// Passes of `per_pass` rows over one weight stream each. min_rows: the fewest rows this kernel
// takes itself (group 64 hands single rows to the exact M = 1 kernel through `single`).
template <int GROUP>
int launch_batch(const char* who, const vpq_linear_desc& d, int per_pass, cudaStream_t st, bool single_rows_exact,
                 bool scale_only = false) {
  const uint32_t* w = d.w;
  const void *scales = d.scales, *biases = scale_only ? d.scales : d.biases, *x = d.x;
  void* y = d.y;
  const int64_t K = d.K, N = d.N, M = d.M;
  const bool gated = d.epilogue == VPQ_EPILOGUE_SWIGLU || d.epilogue == VPQ_EPILOGUE_GEGLU;
  const int64_t y_pitch = gated ? N / 2 : d.epilogue == VPQ_EPILOGUE_QKV ? d.q_rows : N;
  const int64_t aux_pitch = (d.epilogue == VPQ_EPILOGUE_ADD || d.epilogue == VPQ_EPILOGUE_GELU_MUL || d.epilogue == VPQ_EPILOGUE_SILU_MUL) ? N
                            : d.epilogue == VPQ_EPILOGUE_QKV                                         ? d.k_rows
                                                                                                     : 0;
  const int64_t y3_pitch = d.epilogue == VPQ_EPILOGUE_QKV ? N - d.q_rows - d.k_rows : 0;
  const int cap_kt = (int)((K + 255) / 256) * 2;
  BatchProblem p;
  std::memset(&p, 0, sizeof(p));
  if (int rc = make_map_2d(&p.mw, CU_TENSOR_MAP_DATA_TYPE_UINT32, 4, w, (uint64_t)(K / 8), (uint64_t)N, 32, 16,
                           CU_TENSOR_MAP_SWIZZLE_128B, "w")) {
    return rc;
  }
  constexpr int GPS = 2048 / GROUP;
  // scale / bias rows as TMA boxes: pitch and base multiples of 16 bytes
  p.scales_tma = ((K / GROUP) % 8 == 0 && aligned16(scales) && aligned16(biases)) ? 1 : 0;
  p.scale_only = scale_only ? 1 : 0;
  p.norm_w = static_cast<const uint16_t*>(d.norm_w);
  p.eps = d.eps;
  if (p.scales_tma) {
    if (int rc = make_map_2d(&p.ms, CU_TENSOR_MAP_DATA_TYPE_UINT16, 2, scales, (uint64_t)(K / GROUP), (uint64_t)N, GPS,
                             16, CU_TENSOR_MAP_SWIZZLE_NONE, "scales")) {
      return rc;
    }
    if (int rc = make_map_2d(&p.mz, CU_TENSOR_MAP_DATA_TYPE_UINT16, 2, biases, (uint64_t)(K / GROUP), (uint64_t)N, GPS,
                             16, CU_TENSOR_MAP_SWIZZLE_NONE, "biases")) {
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
  p.y_pitch = (int)y_pitch;
  p.aux_pitch = (int)aux_pitch;
  p.y3_pitch = (int)y3_pitch;
  for (int64_t m0 = 0; m0 < M; m0 += per_pass) {
    const int rows = (int)((M - m0) < per_pass ? (M - m0) : per_pass);
    // chunks of x per thread in this pass: the instantiation that holds just that many (4: no stack
    // frame, 6: 48 bytes, 8: 140 bytes)
    const int64_t per_thread = ((int64_t)rows * cap_kt * 16 + kConsThreads - 1) / kConsThreads;
    const int held = per_thread <= 4 ? 0 : per_thread <= 6 ? 1 : 2;
    auto kern = held == 0   ? affine_qmv_batch_w4_kernel<GROUP, 4>
                : held == 1 ? affine_qmv_batch_w4_kernel<GROUP, 6>
                            : affine_qmv_batch_w4_kernel<GROUP, 8>;
    p.x = static_cast<const uint16_t*>(x) + m0 * K;
    p.y = static_cast<__nv_bfloat16*>(y) + m0 * y_pitch;
    p.aux = d.aux ? static_cast<const uint16_t*>(d.aux) + m0 * aux_pitch : nullptr;
    p.y3 = d.y3 ? static_cast<__nv_bfloat16*>(d.y3) + m0 * y3_pitch : nullptr;
    p.M = rows;
    if (rows == 1 && single_rows_exact) {  // a single row left over: the exact M = 1 kernel
      vpq_linear_desc one = d;
      one.x = p.x;
      one.y = p.y;
      one.aux = p.aux;
      one.y3 = p.y3;
      one.M = 1;
      if (int rc = vpq_affine_qmv_w4g64_bf16_batch(&one, 1, st)) { return rc; }
      continue;
    }
    const size_t fixed = fixed_smem<GROUP>(rows, cap_kt);
    int stages = fixed < kSmemBudget ? (int)((kSmemBudget - fixed) / stage_bytes<GROUP>()) : 0;
    if (stages > kMaxStages) { stages = kMaxStages; }
    if (stages < 2) { return fail(VPQ_ERR_UNSUPPORTED, "%s: K=%lld does not fit in shared memory", who, (long long)K); }
    const size_t smem = fixed + (size_t)stages * stage_bytes<GROUP>();
    static int granted[3][64] = {};
    if (int rc = ensure_dynamic_smem(reinterpret_cast<const void*>(kern), granted[held], smem)) { return rc; }
    const int cap = 2 * num_sms();
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

int check_batch_args(const char* who, const void* w, const void* scales, const void* biases, const void* x,
                     const void* y, int64_t K, int64_t N, int64_t M, int group) {
  if (!w || !scales || !biases || !x || !y) { return fail(VPQ_ERR_INVALID_ARG, "%s: null pointer", who); }
  if (K <= 0 || N <= 0 || M <= 0 || (K % group) != 0 || (K % 8) != 0) {
    return fail(VPQ_ERR_INVALID_ARG, "%s: need K>0, N>0, M>0, K%%%d==0 (K=%lld N=%lld M=%lld)", who, group,
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

int qmvb_status_read(cudaStream_t st, uint32_t* out) {
  uint32_t v = 0;
  VPQ_CUDA_OK(cudaMemcpyFromSymbolAsync(&v, g_qmvb_status, sizeof(v), 0, cudaMemcpyDeviceToHost, st));
  VPQ_CUDA_OK(cudaStreamSynchronize(st));
  if (v != 0) {
    const uint32_t zero = 0;
    VPQ_CUDA_OK(cudaMemcpyToSymbolAsync(g_qmvb_status, &zero, sizeof(zero), 0, cudaMemcpyHostToDevice, st));
    VPQ_CUDA_OK(cudaStreamSynchronize(st));
  }
  *out = v;
  return VPQ_OK;
}
}  // namespace vpq

using namespace vpq;

namespace {
vpq_linear_desc plain_desc(const uint32_t* w, const void* scales, const void* biases, const void* x, void* y, int64_t K,
                           int64_t N, int64_t M) {
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
  return d;
}

int batch_g64(const char* who, const vpq_linear_desc& d, void* stream) {
  if (int rc = check_batch_args(who, d.w, d.scales, d.biases, d.x, d.y, d.K, d.N, d.M, 64)) { return rc; }
  if (int rc = qmv_check_plain(who, d, /*allow_norm=*/true)) { return rc; }
  if (int rc = require_sm100()) { return rc; }
  const int per_pass = rows_per_pass<64>((int)((d.K + 255) / 256) * 2);
  if (per_pass < 2 || d.M == 1) {  // long rows (K > 8192) do not fit twice in shared memory: one row at a time
    return vpq_affine_qmv_w4g64_bf16_batch(&d, 1, stream);
  }
  return launch_batch<64>(who, d, per_pass, static_cast<cudaStream_t>(stream), true);
}

// scale_only: the descriptor's biases are ignored (may be null)
int gemv_g32(const char* who, const vpq_linear_desc& d, void* stream, bool scale_only = false) {
  if (int rc = check_batch_args(who, d.w, d.scales, scale_only ? d.scales : d.biases, d.x, d.y, d.K, d.N, d.M, 32)) {
    return rc;
  }
  if (int rc = qmv_check_plain(who, d, /*allow_norm=*/true)) { return rc; }
  if (int rc = require_sm100()) { return rc; }
  const int per_pass = rows_per_pass<32>((int)((d.K + 255) / 256) * 2);  // 2 rows per weight stream where they fit
  return launch_batch<32>(who, d, per_pass, static_cast<cudaStream_t>(stream), false, scale_only);
}
}  // namespace

extern "C" int vpq_affine_qmv_batch_w4g64_bf16(const uint32_t* w, const void* scales, const void* biases,
                                               const void* x, void* y, int64_t K, int64_t N, int64_t M,
                                               void* stream) {
  clear_error();
  return batch_g64("affine_qmv_batch_w4g64", plain_desc(w, scales, biases, x, y, K, N, M), stream);
}

extern "C" int vpq_affine_qmv_batch_w4g64_bf16_fused(const vpq_linear_desc* desc_host, void* stream) {
  clear_error();
  if (!desc_host) { return fail(VPQ_ERR_INVALID_ARG, "affine_qmv_batch_w4g64 (fused store): null descriptor"); }
  return batch_g64("affine_qmv_batch_w4g64 (fused store)", *desc_host, stream);
}

extern "C" int vpq_affine_qmv_w4g32_bf16(const uint32_t* w, const void* scales, const void* biases, const void* x,
                                         void* y, int64_t K, int64_t N, int64_t M, void* stream) {
  clear_error();
  return gemv_g32("affine_qmv_w4g32", plain_desc(w, scales, biases, x, y, K, N, M), stream);
}

extern "C" int vpq_affine_qmv_w4g32_bf16_fused(const vpq_linear_desc* desc_host, void* stream) {
  clear_error();
  if (!desc_host) { return fail(VPQ_ERR_INVALID_ARG, "affine_qmv_w4g32 (fused store): null descriptor"); }
  return gemv_g32("affine_qmv_w4g32 (fused store)", *desc_host, stream);
}

extern "C" int vpq_affine_qmv_w4g32_q40_bf16_fused(const vpq_linear_desc* desc_host, void* stream) {
  clear_error();
  if (!desc_host) { return fail(VPQ_ERR_INVALID_ARG, "affine_qmv_w4g32_q40: null descriptor"); }
  return gemv_g32("affine_qmv_w4g32_q40", *desc_host, stream, true);
}
