// qmm.cu -- prefill / DiT GEMM over 4-bit affine group-64 weights on the
// sm_100a tensor cores:  y[M,N] = x[M,K] @ dequant(W)[N,K]^T.
//
// Replaces affine_qmm_steel_w4g64[_bm64|_bm128] (qmm_t_impl,
// gpu-kernels/metal/quant/affine_qmm_steel.metal:318-561) and
// affine_qmm_mma_w4g64 (gpu-kernels/metal/quant/affine_qmm_mma.metal:50-128).
// Same numerics as those kernels: the weight tile is dequantised to bf16
// (f32 multiply-add, one rounding to bf16; bit-identical to
// affine_dequant_w4g64) before the multiply, f32 accumulation, one rounding
// of the result to bf16.
//
// One persistent CTA per SM, 448 threads in four roles:
//   warps 0-3   epilogue: tcgen05.ld the finished 128 x BN f32 accumulator out
//               of tensor memory, round to bf16, store to y
//   warp  4     TMA producer: per 64-wide k block, one bf16 x tile [128 x 64]
//               (128-byte swizzle) and one packed-nibble W tile [BN x 32 B]
//   warp  5     MMA issuer: one thread issues 4 tcgen05.mma (128 x BN x 16)
//               per k block; allocates / frees tensor memory
//   warps 6-13  dequantisers: thread t owns W-tile row t; per k block it turns
//               that row's 32 bytes of nibbles (exactly one quantization
//               group) into 64 bf16 and writes them into the K-major,
//               128-byte-swizzled operand tile the MMA descriptor expects
// linked by mbarrier rings (x+codes stages, dequantised-B stages, two
// accumulator buffers in tensor memory so the epilogue of tile i overlaps the
// main loop of tile i+1). Every wait is bounded: a wait that gives up records
// a code in a device status word and the kernel drains and returns.
//
// No TMA multicast is used anywhere; each CTA issues plain TMA loads and tile
// reuse between CTAs comes from L2.
#include "vpq_sm100.cuh"

#include <algorithm>
#include <cstdlib>

namespace vpq {

// Status word of the tensor-core kernels: 0, or (site << 8) | role of the
// first bounded wait that gave up.
__device__ uint32_t g_qmm_status;

namespace {

constexpr int BM = 128;       // x rows per tile  (MMA M)
constexpr int BK = 64;        // k per stage = one quantization group
constexpr int kStages = 4;    // x + codes ring
constexpr int kBStages = 3;   // dequantised B ring
constexpr int kEpiWarps = 4;
constexpr int kDqWarpsMax = 8;

template <int BN, int BITS = 4>
struct SmemLayout {
  static constexpr int kXBytes = BM * BK * 2;       // 16 KB, 128B-swizzled
  static constexpr int kCodeBytes = BN * (BK * BITS / 8);  // BN rows x 32 B (64 B at 8 bits)
  static constexpr int kBBytes = BN * BK * 2;       // 128B-swizzled K-major
  static constexpr int kOffX = 0;
  static constexpr int kOffB = kOffX + kStages * kXBytes;
  static constexpr int kOffCode = kOffB + kBStages * kBBytes;
  static constexpr int kOffBar = kOffCode + kStages * kCodeBytes;
  static constexpr int kNumBars = 2 * kStages + 2 * kBStages + 4;
  static constexpr int kOffTmem = kOffBar + kNumBars * 8;
  static constexpr int kTotal = kOffTmem + 16;
  static constexpr int kAlloc = kTotal + 1024;  // slack to align the base to 1024 B
};

// ------------------------------------------------------------ PTX wrappers
__device__ __forceinline__ void tc_fence_before() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}

__device__ __forceinline__ void umma_bf16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc,
                                          uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t"
      "}"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}

// Arrives on `bar` once every tcgen05.mma issued so far by this thread is done.
__device__ __forceinline__ void umma_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];"
               ::"r"(bar)
               : "memory");
}

// Shared-memory matrix descriptor: K-major operand, 128-byte swizzle, rows of
// 128 bytes, 8-row groups 1024 bytes apart.
__device__ __forceinline__ uint64_t make_sw128_desc(uint32_t smem_addr) {
  uint64_t d = 0;
  d |= (uint64_t)((smem_addr >> 4) & 0x3fffu);  // start address
  d |= (uint64_t)1 << 16;                       // leading byte offset (unused for swizzled K-major)
  d |= (uint64_t)(1024 >> 4) << 32;             // stride byte offset between 8-row groups
  d |= (uint64_t)1 << 46;                       // descriptor version (sm_100)
  d |= (uint64_t)2 << 61;                       // SWIZZLE_128B
  return d;
}

// Instruction descriptor: D f32, A/B bf16, both K-major, M = 128, N = BN.
template <int BN>
__device__ __forceinline__ constexpr uint32_t make_idesc() {
  return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);
}

__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,"
      "%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
        "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
        "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]),
        "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]),
        "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() {
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// 8 nibbles of one packed word -> 8 bf16 (4 packed registers), bit-identical to
// bf16_rne(fmaf(s, q, b)). A nibble moved into bits 16..23 of a zero word is, read as a float,
// the subnormal (or first-binade) number n * 2^-133, n the integer in those bits: the even
// nibbles arrive as q, the odd ones (left in the high half of their byte) as 16 q. Then
// fmaf(n * 2^-133, s * 2^133 (or s * 2^129 for the odd ones), b) rounds the same real number
// s q + b once. The two multiply-adds of a nibble pair share one packed f32x2 instruction;
// s2 holds (s * 2^133, s * 2^129), b2 holds (b, b). Valid while s * 2^133 is a normal float
// (2^-126 <= |s| < 2^-5); dequant_scale_up() says so, other scales take dequant_word_exact.
// One nibble pair (byte J of the even / odd nibble words) -> one packed bf16x2.
#define VPQ_DEQUANT_PAIR(J, SEL)                                                     \
  asm("{\n\t"                                                                        \
      ".reg .b32 fe, fo, ve, vo;\n\t"                                                \
      ".reg .b64 q2, v2;\n\t"                                                        \
      "prmt.b32 fe, %1, 0, " SEL ";\n\t"                                             \
      "prmt.b32 fo, %2, 0, " SEL ";\n\t"                                             \
      "mov.b64 q2, {fe, fo};\n\t"                                                    \
      "fma.rn.f32x2 v2, %3, q2, %4;\n\t"                                             \
      "mov.b64 {ve, vo}, v2;\n\t"                                                    \
      "cvt.rn.bf16x2.f32 %0, vo, ve;\n\t"                                            \
      "}"                                                                            \
      : "=r"(out[J])                                                                 \
      : "r"(e), "r"(o), "l"(s2), "l"(b2))

__device__ __forceinline__ void dequant_word_fast(uint32_t word, uint64_t s2, uint64_t b2, uint32_t* out) {
  const uint32_t e = word & 0x0f0f0f0fu;  // nibbles 0,2,4,6 in the low halves of the bytes
  const uint32_t o = word & 0xf0f0f0f0u;  // nibbles 1,3,5,7 times 16
  VPQ_DEQUANT_PAIR(0, "0x4044");
  VPQ_DEQUANT_PAIR(1, "0x4144");
  VPQ_DEQUANT_PAIR(2, "0x4244");
  VPQ_DEQUANT_PAIR(3, "0x4344");
}
#undef VPQ_DEQUANT_PAIR

// s * 2^shift by exponent arithmetic; false if s is zero / subnormal or s * 2^133 would overflow.
__device__ __forceinline__ bool dequant_scale_up(float s, float& s_133, float& s_129) {
  const uint32_t bits = __float_as_uint(s);
  const uint32_t e = (bits >> 23) & 0xffu;
  s_133 = __uint_as_float(bits + (133u << 23));
  s_129 = __uint_as_float(bits + (129u << 23));
  return e >= 1u && e <= 121u;
}

// 8-bit codes: the two byte pairs of a word -> two packed bf16x2. The byte goes to bits 16..23
// of a zero word (PRMT), which as a float is q * 2^-133; s2 holds (s * 2^133, s * 2^133).
#define VPQ_DEQUANT_PAIR8(J, SEL_LO, SEL_HI)                                         \
  asm("{\n\t"                                                                        \
      ".reg .b32 fe, fo, ve, vo;\n\t"                                                \
      ".reg .b64 q2, v2;\n\t"                                                        \
      "prmt.b32 fe, %1, 0, " SEL_LO ";\n\t"                                          \
      "prmt.b32 fo, %1, 0, " SEL_HI ";\n\t"                                          \
      "mov.b64 q2, {fe, fo};\n\t"                                                    \
      "fma.rn.f32x2 v2, %2, q2, %3;\n\t"                                             \
      "mov.b64 {ve, vo}, v2;\n\t"                                                    \
      "cvt.rn.bf16x2.f32 %0, vo, ve;\n\t"                                            \
      "}"                                                                            \
      : "=r"(out[J])                                                                 \
      : "r"(word), "l"(s2), "l"(b2))

__device__ __forceinline__ void dequant_word8_fast(uint32_t word, uint64_t s2, uint64_t b2, uint32_t* out) {
  VPQ_DEQUANT_PAIR8(0, "0x4044", "0x4144");  // bytes 0, 1
  VPQ_DEQUANT_PAIR8(1, "0x4244", "0x4344");  // bytes 2, 3
}
#undef VPQ_DEQUANT_PAIR8

__device__ __forceinline__ void dequant_word8_exact(uint32_t word, float s, float b, uint32_t* out) {
#pragma unroll
  for (int j = 0; j < 2; ++j) {
    const float ve = dequant_f32(s, (word >> (16 * j)) & 0xffu, b);
    const float vo = dequant_f32(s, (word >> (16 * j + 8)) & 0xffu, b);
    out[j] = pack_bf16x2(ve, vo);
  }
}

__device__ __forceinline__ uint64_t pack_f32x2(float lo, float hi) {
  uint64_t r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
  return r;
}

__device__ __forceinline__ void dequant_word_exact(uint32_t word, float s, float b, uint32_t* out) {
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const float ve = dequant_f32(s, (word >> (8 * j)) & 0xfu, b);
    const float vo = dequant_f32(s, (word >> (8 * j + 4)) & 0xfu, b);
    out[j] = pack_bf16x2(ve, vo);
  }
}

// One row's scales and biases along K: eight groups (16 bytes) per load, fetched one block of
// eight k blocks ahead, so the latency of these small loads never sits in the dequant loop.
// Rows whose pitch or base is not 16-byte aligned fall back to one 2-byte load per k block.
struct ScaleStream {
  const uint16_t* s;
  const uint16_t* b;
  int groups;
  bool vec;
  uint4 s_cur, b_cur, s_nxt, b_nxt;
  int blk;
  __device__ __forceinline__ ScaleStream(const uint16_t* srow, const uint16_t* brow, int g)
      : s(srow), b(brow), groups(g) {
    vec = ((g & 7) == 0) && ((reinterpret_cast<uintptr_t>(srow) | reinterpret_cast<uintptr_t>(brow)) & 15u) == 0;
    s_cur = b_cur = s_nxt = b_nxt = make_uint4(0, 0, 0, 0);
    blk = -1;
    if (vec) {
      s_nxt = __ldg(reinterpret_cast<const uint4*>(s));
      b_nxt = __ldg(reinterpret_cast<const uint4*>(b));
    }
  }
  __device__ __forceinline__ static float pick(const uint4& v, int i) {
    const uint32_t w = i < 4 ? (i < 2 ? v.x : v.y) : (i < 6 ? v.z : v.w);
    return __uint_as_float((i & 1) ? (w & 0xffff0000u) : (w << 16));
  }
  // Works for any increasing sequence of kb (a warp group may take every other k block).
  __device__ __forceinline__ void get(int kb, float& sc, float& bi) {
    if (vec) {
      const int i = kb & 7;
      if ((kb >> 3) != blk) {
        blk = kb >> 3;
        s_cur = s_nxt;
        b_cur = b_nxt;
        if (blk * 8 + 8 < groups) {
          s_nxt = __ldg(reinterpret_cast<const uint4*>(s + blk * 8 + 8));
          b_nxt = __ldg(reinterpret_cast<const uint4*>(b + blk * 8 + 8));
        }
      }
      sc = pick(s_cur, i);
      bi = pick(b_cur, i);
    } else {
      sc = bf16_bits_to_f32(ldg_nc_u16(s + kb));
      bi = bf16_bits_to_f32(ldg_nc_u16(b + kb));
    }
  }
};

enum Role : uint32_t { kRoleEpi = 1, kRoleTma = 2, kRoleMma = 3, kRoleDq = 4, kRoleSend = 5 };

// Grouped (mixture-of-experts) form of the GEMM, the reference's affine_qmm_grouped_w4g64 /
// affine_qmm_grouped_swiglu_w4g64 (affine_qmm_steel.metal:1026-1176,1371-1440): the rows of x are
// (token, expert) pairs sorted by expert and padded per expert to whole row tiles; row tile i
// multiplies expert tile2e[i]'s slab of w ([E, N, K/8], scales [E, N, K/64]); a negative (or out of
// range) entry is an all-padding tile and is skipped by every role. sdst, when given, scatters
// row m of the product to row sdst[m] of y (negative or >= y_rows: not stored).
struct GroupSpec {
  const int* tile2e;  // null: one weight for all row tiles
  const int* sdst;    // null: row m of the product is row m of y
  int experts;
  int y_rows;
};

__device__ __forceinline__ float gelu_tanh_f(float x) {
  const float t = tanhf(0.7978845608028654f * (x + 0.044715f * x * x * x));
  return 0.5f * x * (1.0f + t);
}

// kAct 0: y [.., N]; 1 / 2: columns 2j, 2j + 1 are gate j, up j, y [.., N / 2] = silu / gelu(gate) * up.
template <int BN, int kAct, int BITS>
__global__ void __launch_bounds__(32 * (kEpiWarps + 2 + BN / 32), 1)
affine_qmm_w4g64_kernel(const __grid_constant__ CUtensorMap tmap_x,
                        const __grid_constant__ CUtensorMap tmap_w,
                        const uint16_t* __restrict__ scales, const uint16_t* __restrict__ biases,
                        __nv_bfloat16* __restrict__ y, int M, int N, int K, const GroupSpec G) {
  using L = SmemLayout<BN, BITS>;
  static_assert(L::kAlloc <= 227 * 1024, "shared memory of the single-CTA kernel");
  constexpr int kDqWarps = BN / 32;
  static_assert(kDqWarps <= kDqWarpsMax, "tile too wide");
  constexpr uint32_t kTmemCols = 2 * BN;  // two accumulator buffers (power of two >= 32)
  static_assert(kTmemCols == 512 || kTmemCols == 256 || kTmemCols == 128, "tensor memory columns");

  extern __shared__ unsigned char smem_dyn[];
  const uint32_t raw = smem_u32(smem_dyn);
  const uint32_t base = (raw + 1023u) & ~1023u;  // swizzled tiles need 1024-byte alignment
  unsigned char* base_ptr = smem_dyn + (base - raw);

  const uint32_t bar0 = base + L::kOffBar;
  auto bar_full = [&](int s) { return bar0 + 8u * s; };
  auto bar_empty = [&](int s) { return bar0 + 8u * (kStages + s); };
  auto bar_bfull = [&](int t) { return bar0 + 8u * (2 * kStages + t); };
  auto bar_bempty = [&](int t) { return bar0 + 8u * (2 * kStages + kBStages + t); };
  auto bar_accfull = [&](int a) { return bar0 + 8u * (2 * kStages + 2 * kBStages + a); };
  auto bar_accempty = [&](int a) { return bar0 + 8u * (2 * kStages + 2 * kBStages + 2 + a); };
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(base_ptr + L::kOffTmem);
  volatile uint32_t* abort_flag = tmem_slot + 1;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  const int tiles_m = (M + BM - 1) / BM;
  const int tiles_n = (N + BN - 1) / BN;
  const int num_tiles = tiles_m * tiles_n;
  const int num_kb = K / BK;
  // expert of a tile's row tile; -1: skip the tile (the same answer in every role)
  auto expert_of = [&](int tile) -> int {
    if (G.tile2e == nullptr) { return 0; }
    const int e = __ldg(G.tile2e + tile / tiles_n);
    return (e >= 0 && e < G.experts) ? e : -1;
  };

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      mbar_init(bar_full(s), 1);
      mbar_init(bar_empty(s), 1 + kDqWarps);
    }
    for (int t = 0; t < kBStages; ++t) {
      mbar_init(bar_bfull(t), kDqWarps);
      mbar_init(bar_bempty(t), 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(bar_accfull(a), 1);
      mbar_init(bar_accempty(a), kEpiWarps);
    }
    *abort_flag = 0;
    fence_mbar_init();
  }
  if (warp == 5) {  // tensor memory: whole warp allocates, address lands in shared memory
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                 ::"r"(smem_u32((const void*)tmem_slot)), "r"(kTmemCols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 4) {
    // ------------------------------------------------------- TMA producer
    if (lane == 0) {
      uint32_t it = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
        const int e = expert_of(tile);
        if (e < 0) { continue; }
        const int m0 = (tile / tiles_n) * BM;
        const int n0 = (tile % tiles_n) * BN;
        const int w_row0 = e * N + n0;  // expert e's slab starts at row e * N of the [E * N, K / 8] map
        for (int kb = 0; kb < num_kb; ++kb, ++it) {
          const int s = it % kStages;
          const uint32_t ph = (it / kStages) & 1u;
          if (!mbar_wait(bar_empty(s), ph ^ 1u, (1u << 8) | kRoleTma, abort_flag, &g_qmm_status)) { ok = false; break; }
          mbar_expect_tx(bar_full(s), L::kXBytes + L::kCodeBytes);
          tma_load_2d(base + L::kOffX + s * L::kXBytes, &tmap_x, bar_full(s), kb * BK, m0);
          tma_load_2d(base + L::kOffCode + s * L::kCodeBytes, &tmap_w, bar_full(s), kb * (BK * BITS / 32), w_row0);
        }
      }
      // Never leave with a copy still in flight: wait for the last load of every stage.
      const uint32_t issued = it;
      for (int s = 0; s < kStages; ++s) {
        // index of the last iteration that used stage s, if any
        if (issued > (uint32_t)s) {
          const uint32_t last = ((issued - 1 - s) / kStages) * kStages + s;
          mbar_wait(bar_full(s), (last / kStages) & 1u, (2u << 8) | kRoleTma, abort_flag, &g_qmm_status);
        }
      }
    }
  } else if (warp == 5) {
    // --------------------------------------------------------- MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc = make_idesc<BN>();
      uint32_t it = 0, ti = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
        if (expert_of(tile) < 0) { continue; }
        const int a = ti & 1;
        const uint32_t aph = (ti >> 1) & 1u;
        ++ti;
        if (!mbar_wait(bar_accempty(a), aph ^ 1u, (1u << 8) | kRoleMma, abort_flag, &g_qmm_status)) { ok = false; break; }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + (uint32_t)(a * BN);
        for (int kb = 0; kb < num_kb; ++kb, ++it) {
          const int s = it % kStages;
          const uint32_t ph = (it / kStages) & 1u;
          const int t = it % kBStages;
          const uint32_t bph = (it / kBStages) & 1u;
          if (!mbar_wait(bar_full(s), ph, (2u << 8) | kRoleMma, abort_flag, &g_qmm_status)) { ok = false; break; }
          if (!mbar_wait(bar_bfull(t), bph, (3u << 8) | kRoleMma, abort_flag, &g_qmm_status)) { ok = false; break; }
          tc_fence_after();
          const uint64_t a_desc = make_sw128_desc(base + L::kOffX + s * L::kXBytes);
          const uint64_t b_desc = make_sw128_desc(base + L::kOffB + t * L::kBBytes);
#pragma unroll
          for (int k16 = 0; k16 < BK / 16; ++k16) {
            // 16 bf16 = 32 bytes further along K inside the swizzle atom: +2 in the address field
            umma_bf16(d_tmem, a_desc + 2u * k16, b_desc + 2u * k16, idesc, (kb | k16) ? 1u : 0u);
          }
          umma_commit(bar_empty(s));   // x stage free once these MMAs have read it
          umma_commit(bar_bempty(t));  // dequantised tile free likewise
        }
        if (ok) { umma_commit(bar_accfull(a)); }
      }
    }
  } else if (warp >= 6) {
    // ------------------------------------------------------- dequantisers
    const int t_row = threadIdx.x - 6 * 32;  // 0 .. BN-1 : row of the W tile
    const uint32_t row_off = (uint32_t)(t_row >> 3) * 1024u + (uint32_t)(t_row & 7) * 128u;
    const uint32_t sw = (uint32_t)(t_row & 7);
    const int groups = K >> 6;
    uint32_t it = 0;
    bool ok = true;
    for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
      const int e = expert_of(tile);
      if (e < 0) { continue; }
      const int n0 = (tile % tiles_n) * BN;
      int row = n0 + t_row;
      row = row < N ? row : N - 1;  // tail rows: any valid scale; their columns are never stored
      const int64_t srow_i = (int64_t)e * N + row;
      const uint16_t* srow = scales + srow_i * groups;
      const uint16_t* brow = biases + srow_i * groups;
      ScaleStream sst(srow, brow, groups);
      for (int kb = 0; kb < num_kb; ++kb, ++it) {
        const int s = it % kStages;
        const uint32_t ph = (it / kStages) & 1u;
        const int t = it % kBStages;
        const uint32_t bph = (it / kBStages) & 1u;
        float sc, bi;
        sst.get(kb, sc, bi);
        if (!warp_wait(bar_full(s), ph, (1u << 8) | kRoleDq, abort_flag, &g_qmm_status)) { ok = false; break; }
        const uint4* cp = reinterpret_cast<const uint4*>(base_ptr + L::kOffCode + s * L::kCodeBytes +
                                                         t_row * (BK * BITS / 8));
        uint32_t o[32];
        float s_133, s_129;
        if (BITS == 4) {
          const uint4 c0 = cp[0], c1 = cp[1];
          __syncwarp();
          if (lane == 0) { mbar_arrive(bar_empty(s)); }  // codes are in registers
          const uint32_t cw[8] = {c0.x, c0.y, c0.z, c0.w, c1.x, c1.y, c1.z, c1.w};
          if (dequant_scale_up(sc, s_133, s_129)) {
            const uint64_t s2 = pack_f32x2(s_133, s_129), b2 = pack_f32x2(bi, bi);
#pragma unroll
            for (int wd = 0; wd < 8; ++wd) { dequant_word_fast(cw[wd], s2, b2, o + 4 * wd); }
          } else {
#pragma unroll
            for (int wd = 0; wd < 8; ++wd) { dequant_word_exact(cw[wd], sc, bi, o + 4 * wd); }
          }
        } else {  // a byte per value: 16 words (see dequant_word8_fast)
          const uint4 c0 = cp[0], c1 = cp[1], c2 = cp[2], c3 = cp[3];
          __syncwarp();
          if (lane == 0) { mbar_arrive(bar_empty(s)); }
          const uint32_t cw[16] = {c0.x, c0.y, c0.z, c0.w, c1.x, c1.y, c1.z, c1.w,
                                   c2.x, c2.y, c2.z, c2.w, c3.x, c3.y, c3.z, c3.w};
          if (dequant_scale_up(sc, s_133, s_129)) {
            const uint64_t s2 = pack_f32x2(s_133, s_133), b2 = pack_f32x2(bi, bi);
#pragma unroll
            for (int wd = 0; wd < 16; ++wd) { dequant_word8_fast(cw[wd], s2, b2, o + 2 * wd); }
          } else {
#pragma unroll
            for (int wd = 0; wd < 16; ++wd) { dequant_word8_exact(cw[wd], sc, bi, o + 2 * wd); }
          }
        }

        if (!warp_wait(bar_bempty(t), bph ^ 1u, (2u << 8) | kRoleDq, abort_flag, &g_qmm_status)) { ok = false; break; }
        unsigned char* bt = base_ptr + L::kOffB + t * L::kBBytes + row_off;
#pragma unroll
        for (int c = 0; c < 8; ++c) {  // 16-byte chunk c of the row lands at chunk (c ^ row%8)
          *reinterpret_cast<uint4*>(bt + ((c ^ sw) << 4)) =
              make_uint4(o[4 * c], o[4 * c + 1], o[4 * c + 2], o[4 * c + 3]);
        }
        fence_proxy_async();  // make the generic-proxy writes visible to the tensor core
        __syncwarp();
        if (lane == 0) { mbar_arrive(bar_bfull(t)); }
      }
    }
  } else {
    // ------------------------------------------------------------ epilogue
    uint32_t ti = 0;
    bool ok = true;
    const int n_out = kAct ? N / 2 : N;  // width of y
    const bool vec_ok = (n_out % 8) == 0;
    for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
      if (expert_of(tile) < 0) { continue; }
      const int m0 = (tile / tiles_n) * BM;
      const int n0 = (tile % tiles_n) * BN;
      const int a = ti & 1;
      const uint32_t aph = (ti >> 1) & 1u;
      ++ti;
      if (!warp_wait(bar_accfull(a), aph, (1u << 8) | kRoleEpi, abort_flag, &g_qmm_status)) { ok = false; break; }
      tc_fence_after();
      const int m = m0 + warp * 32 + lane;  // warp w reads tensor-memory lanes 32w .. 32w+31
      const uint32_t taddr = tmem_base + ((uint32_t)(warp * 32) << 16) + (uint32_t)(a * BN);
      int dr = -1;  // row of y this lane's row goes to
      if (m < M) {
        dr = G.sdst ? __ldg(G.sdst + m) : m;
        if (dr >= G.y_rows) { dr = -1; }
      }
      __nv_bfloat16* yrow = y + (int64_t)(dr < 0 ? 0 : dr) * n_out + (kAct ? n0 / 2 : n0);
#pragma unroll 1
      for (int c = 0; c < BN / 32; ++c) {
        uint32_t r[32];
        tmem_ld32(taddr + (uint32_t)(c * 32), r);
        tmem_ld_wait();
        const int nc = n0 + c * 32;
        if (dr >= 0 && nc < N) {
          if (kAct) {
            float o[16];
#pragma unroll
            for (int i = 0; i < 16; ++i) {
              const float g = __uint_as_float(r[2 * i]), u = __uint_as_float(r[2 * i + 1]);
              o[i] = (kAct == 2 ? gelu_tanh_f(g) : __fdividef(g, 1.0f + __expf(-g))) * u;
            }
            const int oc = nc / 2;  // first output column of these 16
            if (vec_ok) {
#pragma unroll
              for (int v = 0; v < 2; ++v) {
                if (oc + v * 8 < n_out) {
                  uint4 pk;
                  pk.x = pack_bf16x2(o[8 * v + 0], o[8 * v + 1]);
                  pk.y = pack_bf16x2(o[8 * v + 2], o[8 * v + 3]);
                  pk.z = pack_bf16x2(o[8 * v + 4], o[8 * v + 5]);
                  pk.w = pack_bf16x2(o[8 * v + 6], o[8 * v + 7]);
                  *reinterpret_cast<uint4*>(yrow + c * 16 + v * 8) = pk;
                }
              }
            } else {
#pragma unroll
              for (int j = 0; j < 16; ++j) {
                if (oc + j < n_out) { yrow[c * 16 + j] = __float2bfloat16_rn(o[j]); }
              }
            }
          } else if (vec_ok) {
#pragma unroll
            for (int v = 0; v < 4; ++v) {
              if (nc + v * 8 < N) {
                uint4 pk;
                pk.x = pack_bf16x2(__uint_as_float(r[8 * v + 0]), __uint_as_float(r[8 * v + 1]));
                pk.y = pack_bf16x2(__uint_as_float(r[8 * v + 2]), __uint_as_float(r[8 * v + 3]));
                pk.z = pack_bf16x2(__uint_as_float(r[8 * v + 4]), __uint_as_float(r[8 * v + 5]));
                pk.w = pack_bf16x2(__uint_as_float(r[8 * v + 6]), __uint_as_float(r[8 * v + 7]));
                *reinterpret_cast<uint4*>(yrow + c * 32 + v * 8) = pk;
              }
            }
          } else {
#pragma unroll
            for (int j = 0; j < 32; ++j) {
              if (nc + j < N) { yrow[c * 32 + j] = __float2bfloat16_rn(__uint_as_float(r[j])); }
            }
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) { mbar_arrive(bar_accempty(a)); }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 5) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kTmemCols)
                 : "memory");
  }
}

#include "qmm_2cta.cuh"

// ------------------------------------------------------------- host side
template <int BN, int kAct, int BITS = 4>
int launch_qmm_act(const uint32_t* w, const uint16_t* scales, const uint16_t* biases, const void* x,
                   __nv_bfloat16* y, int K, int N, int M, const GroupSpec& G, cudaStream_t st) {
  using L = SmemLayout<BN, BITS>;
  CUtensorMap map_x, map_w;
  if (int rc = make_map_2d(&map_x, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, x, (uint64_t)K, (uint64_t)M,
                           BK, BM, CU_TENSOR_MAP_SWIZZLE_128B, "x")) {
    return rc;
  }
  if (int rc = make_map_2d(&map_w, CU_TENSOR_MAP_DATA_TYPE_UINT32, 4, w, (uint64_t)(K * BITS / 32),
                           (uint64_t)N * (uint64_t)G.experts, BK * BITS / 32, BN, CU_TENSOR_MAP_SWIZZLE_NONE, "w")) {
    return rc;
  }
  auto kern = affine_qmm_w4g64_kernel<BN, kAct, BITS>;
  VPQ_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, L::kAlloc));
  const int tiles = ((M + BM - 1) / BM) * ((N + BN - 1) / BN);
  const int sms = num_sms();
  const int grid = tiles < sms ? tiles : sms;
  constexpr int threads = 32 * (kEpiWarps + 2 + BN / 32);
  kern<<<grid, threads, L::kAlloc, st>>>(map_x, map_w, scales, biases, y, M, N, K, G);
  VPQ_LAUNCH_OK("affine_qmm_w4g64");
  return VPQ_OK;
}

template <int BN>
int launch_qmm(const uint32_t* w, const uint16_t* scales, const uint16_t* biases, const void* x,
               __nv_bfloat16* y, int K, int N, int M, cudaStream_t st) {
  const GroupSpec G = {nullptr, nullptr, 1, M};
  return launch_qmm_act<BN, 0>(w, scales, biases, x, y, K, N, M, G, st);
}

// Rows of a [rows, K] bf16 matrix gathered into sorted order: out[i] = src[srow[i]], zeros where
// srow[i] is negative or out of range (padding slots). 16-byte copies; K % 8 == 0.
__global__ void gather_rows_kernel(const uint4* __restrict__ src, const int* __restrict__ srow,
                                   uint4* __restrict__ out, int n_out, int src_rows, int row_vecs) {
  const int64_t total = (int64_t)n_out * row_vecs;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    const int r = (int)(i / row_vecs), c = (int)(i % row_vecs);
    const int sr = __ldg(srow + r);
    out[i] = (sr >= 0 && sr < src_rows) ? __ldg(src + (int64_t)sr * row_vecs + c) : make_uint4(0, 0, 0, 0);
  }
}

// Width of the CTA pair's tile. A 256 x 128 tile costs about 0.6 of a 256 x 256 one (it moves
// more shared-memory bytes per flop), so it pays only where the wide tiles would leave CTA pairs
// idle: few tiles (small N), or a last round that is mostly empty.
int pick_tile_width(int M, int N, int pairs) {
  const int tm = (M + two_cta::TM - 1) / two_cta::TM;
  const int wide = tm * ((N + 255) / 256), narrow = tm * ((N + 127) / 128);
  const double t_wide = (double)((wide + pairs - 1) / pairs);
  const double t_narrow = 0.6 * (double)((narrow + pairs - 1) / pairs);
  return t_narrow < 0.95 * t_wide ? 128 : 256;
}

template <int BITS>
int launch_qmm_2cta_bits(const uint32_t* w, const uint16_t* scales, const uint16_t* biases, const void* x,
                         const two_cta::OutSpec& out, int K, int N, int M, cudaStream_t st, int reserve_sms,
                         int group = 64) {
  int pairs = (num_sms() - reserve_sms) / 2;  // SMs left free run a concurrent collective
  if (pairs < 1) { pairs = 1; }
  const bool two_widths = BITS == 4 && out.swiglu == 0 && group == 64 && out.split0 == 0;
  int comm_pairs = out.comm_pairs > 0 ? out.comm_pairs : 0;
  if (comm_pairs > 0 && out.direct_last) {
    // Column split with at most one tile per pair: every pair sends its own tile, no SM is set aside.
    const int w = two_widths ? pick_tile_width(M, N, pairs) : 256;
    if (((M + two_cta::TM - 1) / two_cta::TM) * ((N + w - 1) / w) <= pairs) { comm_pairs = 0; }
  }
  const int tnt = two_widths ? pick_tile_width(M, N, pairs - comm_pairs) : 256;
  CUtensorMap map_x, map_w;
  if (int rc = make_map_2d(&map_x, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, x, (uint64_t)K, (uint64_t)M,
                           BK, 128, CU_TENSOR_MAP_SWIZZLE_128B, "x")) {
    return rc;
  }
  if (int rc = make_map_2d(&map_w, CU_TENSOR_MAP_DATA_TYPE_UINT32, 4, w, (uint64_t)(K * BITS / 32),
                           (uint64_t)N, BK * BITS / 32, tnt / 2, CU_TENSOR_MAP_SWIZZLE_NONE, "w")) {
    return rc;
  }
  using KernelT = void (*)(const CUtensorMap, const CUtensorMap, const uint16_t*, const uint16_t*, const two_cta::OutSpec,
                           const two_cta::DestMaps, int, int, int);
  KernelT kern;
  int smem;
  if (tnt == 128) {
    kern = two_cta::affine_qmm_w4g64_2cta_kernel<0, 4, 128, 64>;
    smem = two_cta::SmemT<4, 128>::kAlloc;
  } else if (group == 32) {  // the group-32 twins the reference has: plain (4 and 8 bits) and GeGLU (4 bits)
    if (out.swiglu == 1 || (out.swiglu == 2 && BITS == 8)) {
      return fail(VPQ_ERR_UNSUPPORTED, "affine_qmm (group 32): gated stores exist for 4-bit GeGLU only");
    }
    kern = out.swiglu == 2 ? two_cta::affine_qmm_w4g64_2cta_kernel<2, 4, 256, 32>
                           : two_cta::affine_qmm_w4g64_2cta_kernel<0, BITS, 256, 32>;
    smem = two_cta::SmemT<BITS, 256>::kAlloc;
  } else {
    kern = out.swiglu == 2   ? two_cta::affine_qmm_w4g64_2cta_kernel<2, BITS, 256, 64>
           : out.swiglu == 1 ? two_cta::affine_qmm_w4g64_2cta_kernel<1, BITS, 256, 64>
                             : two_cta::affine_qmm_w4g64_2cta_kernel<0, BITS, 256, 64>;
    smem = two_cta::SmemT<BITS, 256>::kAlloc;
  }
  VPQ_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
  const int tiles = ((M + two_cta::TM - 1) / two_cta::TM) * ((N + tnt - 1) / tnt);
  two_cta::OutSpec spec = out;
  spec.comm_pairs = comm_pairs;
  int compute = pairs;
  if (spec.comm_pairs > 0) {  // column split: the last pairs of the grid only send
    if (spec.comm_pairs > pairs / 2) { spec.comm_pairs = pairs / 2; }
    compute = pairs - spec.comm_pairs;
  }
  const int grid = 2 * ((tiles < compute ? tiles : compute) + spec.comm_pairs);
  two_cta::DestMaps maps = {};
  for (int d = 0; spec.comm_pairs > 0 && d < spec.count; ++d) {
    // this rank's column block of destination d: [M rows x N columns] at column col0 of a row-major [M, ld]
    if (int rc = make_map_2d(&maps.m[d], CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, spec.base[d] + spec.col0, (uint64_t)N,
                             (uint64_t)M, (uint32_t)tnt, 16, CU_TENSOR_MAP_SWIZZLE_NONE, "y (column split)",
                             (uint64_t)spec.ld * 2)) {
      return rc;
    }
  }
  kern<<<grid, two_cta::kThreads2, smem, st>>>(map_x, map_w, scales, biases, spec, maps, M, N, K);
  VPQ_LAUNCH_OK("affine_qmm (2-CTA)");
  return VPQ_OK;
}

int launch_qmm_2cta(const uint32_t* w, const uint16_t* scales, const uint16_t* biases, const void* x,
                    const two_cta::OutSpec& out, int K, int N, int M, cudaStream_t st, int reserve_sms) {
  return launch_qmm_2cta_bits<4>(w, scales, biases, x, out, K, N, M, st, reserve_sms);
}

}  // namespace
}  // namespace vpq

using namespace vpq;

namespace vpq {
int qmm_launch_reserved(const uint32_t* w, const void* scales, const void* biases, const void* x, void* y,
                        int64_t K, int64_t N, int64_t M, void* stream, int reserve_sms) {
  clear_error();
  if (!w || !scales || !biases || !x || !y) {
    return fail(VPQ_ERR_INVALID_ARG, "affine_qmm_w4g64: null pointer");
  }
  if (K <= 0 || N <= 0 || M <= 0 || (K % 64) != 0) {
    return fail(VPQ_ERR_INVALID_ARG, "affine_qmm_w4g64: need K>0, N>0, M>0, K%%64==0 (K=%lld N=%lld M=%lld)",
                (long long)K, (long long)N, (long long)M);
  }
  if (K > (1 << 20) || N > (1 << 24) || M > (1 << 24)) {
    return fail(VPQ_ERR_UNSUPPORTED, "affine_qmm_w4g64: shape too large (K=%lld N=%lld M=%lld)",
                (long long)K, (long long)N, (long long)M);
  }
  if (!aligned16(w) || !aligned16(x) || !aligned16(y) ||
      (reinterpret_cast<uintptr_t>(scales) & 1) || (reinterpret_cast<uintptr_t>(biases) & 1)) {
    return fail(VPQ_ERR_ALIGNMENT, "affine_qmm_w4g64: w, x and y must be 16-byte aligned");
  }
  if (int rc = require_sm100()) { return rc; }
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  // 256 x 256 tiles on CTA pairs when there are at least two row tiles' worth of rows; the
  // single-CTA 128 x 256 kernel otherwise.
  if (M > 128) {
    two_cta::OutSpec out = {};
    out.base[0] = static_cast<__nv_bfloat16*>(y);
    out.count = 1;
    out.col0 = 0;
    out.ld = N;
    return launch_qmm_2cta(w, static_cast<const uint16_t*>(scales), static_cast<const uint16_t*>(biases),
                           x, out, (int)K, (int)N, (int)M, st, reserve_sms);
  }
  return launch_qmm<256>(w, static_cast<const uint16_t*>(scales), static_cast<const uint16_t*>(biases),
                         x, static_cast<__nv_bfloat16*>(y), (int)K, (int)N, (int)M, st);
}

// Column block [M, N] of a wider row-major output, stored into `count` destinations (this GPU's
// and its peers' copies of y): the fused epilogue of the column-split. Needs M > 128.
int qmm_launch_multi_dest(const uint32_t* w, const void* scales, const void* biases, const void* x,
                          void* const* dests, int count, int64_t ld, int64_t col0, int64_t K, int64_t N,
                          int64_t M, void* stream, const PeerSync* sync) {
  if (!w || !scales || !biases || !x || !dests || count < 1 || count > 8) {
    return fail(VPQ_ERR_INVALID_ARG, "qmm (fused split): null pointer or more than 8 destinations");
  }
  if (K <= 0 || N <= 0 || M <= 128 || (K % 64) != 0 || (ld % 8) != 0 || (col0 % 8) != 0) {
    return fail(VPQ_ERR_UNSUPPORTED, "qmm (fused split): needs M > 128, K %% 64 == 0, ld and col0 %% 8 == 0");
  }
  if (!aligned16(w) || !aligned16(x)) { return fail(VPQ_ERR_ALIGNMENT, "qmm (fused split): w, x alignment"); }
  if (int rc = require_sm100()) { return rc; }
  two_cta::OutSpec out = {};
  for (int d = 0; d < count; ++d) {
    if (!dests[d] || !aligned16(dests[d])) { return fail(VPQ_ERR_ALIGNMENT, "qmm (fused split): destination %d", d); }
    out.base[d] = static_cast<__nv_bfloat16*>(dests[d]);
  }
  out.count = count;
  out.col0 = (int)col0;
  out.ld = ld;
  if (count > 1) {
    if (!sync || !sync->tile_flags) { return fail(VPQ_ERR_INVALID_ARG, "qmm (fused split): the tile flags are missing"); }
    const int64_t tiles = ((M + 255) / 256) * ((N + 127) / 128);
    if (tiles > sync->tile_flag_count) {
      return fail(VPQ_ERR_UNSUPPORTED, "qmm (fused split): %lld tiles, the communicator's flag array holds %d", (long long)tiles,
                  sync->tile_flag_count);
    }
    // Sender pairs: 12 SMs with one peer, 16 with more. More do not help (24 or 32 sender SMs gave the
    // same times for the exchange-bound shapes at 4 GPUs, and cost the others a round of tiles).
    out.comm_pairs = count <= 2 ? 6 : 8;
    out.direct_last = 1;
    out.tile_flags = sync->tile_flags;
    out.handshake = sync->my_flags != nullptr;
    out.sync = *sync;
  }
  return launch_qmm_2cta(w, static_cast<const uint16_t*>(scales), static_cast<const uint16_t*>(biases), x, out,
                         (int)K, (int)N, (int)M, static_cast<cudaStream_t>(stream), 0);
}
}  // namespace vpq

extern "C" int vpq_affine_qmm_w4g64_bf16(const uint32_t* w, const void* scales, const void* biases,
                                         const void* x, void* y, int64_t K, int64_t N, int64_t M,
                                         void* stream) {
  return qmm_launch_reserved(w, scales, biases, x, y, K, N, M, stream, 0);
}

namespace {
// Gated GEMMs: gate / up rows interleaved in w, y = act(gate) * up, [M, N / 2].
int qmm_gated(const char* who, int bits, int act, const uint32_t* w, const void* scales, const void* biases,
              const void* x, void* y, int64_t K, int64_t N, int64_t M, void* stream, int64_t out_stride = 0,
              int64_t out_off = 0) {
  clear_error();
  if (out_stride < 0 || out_off < 0 || (out_stride > 0 && out_off + N / 2 > out_stride) ||
      (out_stride == 0 && out_off != 0) || out_stride > (1ll << 30)) {
    return fail(VPQ_ERR_INVALID_ARG, "%s: the block [out_off, out_off + N/2) must lie inside a row of out_stride", who);
  }
  if (!w || !scales || !biases || !x || !y) { return fail(VPQ_ERR_INVALID_ARG, "%s: null pointer", who); }
  if (K <= 0 || N <= 0 || M <= 0 || (K % 64) != 0 || (N % 2) != 0) {
    return fail(VPQ_ERR_INVALID_ARG, "%s: need K>0, M>0, K%%64==0 and an even N>0 (K=%lld N=%lld M=%lld)", who,
                (long long)K, (long long)N, (long long)M);
  }
  if (K > (1 << 20) || N > (1 << 24) || M > (1 << 24)) {
    return fail(VPQ_ERR_UNSUPPORTED, "%s: shape too large (K=%lld N=%lld M=%lld)", who, (long long)K, (long long)N,
                (long long)M);
  }
  if (!aligned16(w) || !aligned16(x) || !aligned16(y) || (reinterpret_cast<uintptr_t>(scales) & 1) ||
      (reinterpret_cast<uintptr_t>(biases) & 1)) {
    return fail(VPQ_ERR_ALIGNMENT, "%s: w, x and y must be 16-byte aligned", who);
  }
  if (int rc = require_sm100()) { return rc; }
  two_cta::OutSpec out = {};
  out.base[0] = static_cast<__nv_bfloat16*>(y);
  out.count = 1;
  out.col0 = (int)out_off;
  out.ld = out_stride > 0 ? out_stride : N / 2;
  out.swiglu = act;
  const uint16_t* s16 = static_cast<const uint16_t*>(scales);
  const uint16_t* b16 = static_cast<const uint16_t*>(biases);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (bits == 8) { return launch_qmm_2cta_bits<8>(w, s16, b16, x, out, (int)K, (int)N, (int)M, st, 0); }
  return launch_qmm_2cta_bits<4>(w, s16, b16, x, out, (int)K, (int)N, (int)M, st, 0);
}
}  // namespace

extern "C" int vpq_affine_qmm_swiglu_w4g64_bf16(const uint32_t* w, const void* scales, const void* biases,
                                                const void* x, void* y, int64_t K, int64_t N, int64_t M,
                                                void* stream) {
  return qmm_gated("affine_qmm_swiglu_w4g64", 4, 1, w, scales, biases, x, y, K, N, M, stream);
}

extern "C" int vpq_affine_qmm_swiglu_bf16_rs(const uint32_t* w, const void* scales, const void* biases,
                                            const void* x, void* y, int64_t K, int64_t N, int64_t M, int bits,
                                            int64_t out_stride, int64_t out_off, void* stream) {
  if (bits != 4 && bits != 8) {
    clear_error();
    return fail(VPQ_ERR_INVALID_ARG, "affine_qmm_swiglu (strided store): bits must be 4 or 8");
  }
  return qmm_gated(bits == 8 ? "affine_qmm_swiglu_w8g64_rs" : "affine_qmm_swiglu_w4g64_rs", bits, 1, w, scales, biases,
                   x, y, K, N, M, stream, out_stride, out_off);
}

extern "C" int vpq_affine_qmm_geglu_w4g64_bf16(const uint32_t* w, const void* scales, const void* biases,
                                               const void* x, void* y, int64_t K, int64_t N, int64_t M,
                                               void* stream) {
  return qmm_gated("affine_qmm_geglu_w4g64", 4, 2, w, scales, biases, x, y, K, N, M, stream);
}

extern "C" int vpq_affine_qmm_swiglu_w8g64_bf16(const uint32_t* w, const void* scales, const void* biases,
                                                const void* x, void* y, int64_t K, int64_t N, int64_t M,
                                                void* stream) {
  return qmm_gated("affine_qmm_swiglu_w8g64", 8, 1, w, scales, biases, x, y, K, N, M, stream);
}

extern "C" int vpq_affine_qmm_geglu_w8g64_bf16(const uint32_t* w, const void* scales, const void* biases,
                                               const void* x, void* y, int64_t K, int64_t N, int64_t M,
                                               void* stream) {
  return qmm_gated("affine_qmm_geglu_w8g64", 8, 2, w, scales, biases, x, y, K, N, M, stream);
}

// q | k | v in one GEMM over the row-concatenated weight, three outputs.
extern "C" int vpq_affine_qmm_qkv_w4g64_bf16(const uint32_t* w, const void* scales, const void* biases, const void* x,
                                             void* q_out, void* k_out, void* v_out, int64_t K, int64_t q_rows,
                                             int64_t k_rows, int64_t v_rows, int64_t M, void* stream) {
  clear_error();
  if (!w || !scales || !biases || !x || !q_out || !k_out || !v_out) {
    return fail(VPQ_ERR_INVALID_ARG, "affine_qmm_qkv_w4g64: null pointer");
  }
  if (K <= 0 || M <= 0 || (K % 64) != 0 || q_rows <= 0 || k_rows <= 0 || v_rows <= 0) {
    return fail(VPQ_ERR_INVALID_ARG, "affine_qmm_qkv_w4g64: need K>0, M>0, K%%64==0 and positive q / k / v row counts");
  }
  if ((q_rows % 128) != 0 || (k_rows % 128) != 0 || (v_rows % 8) != 0) {
    return fail(VPQ_ERR_UNSUPPORTED,
                "affine_qmm_qkv_w4g64: q_rows and k_rows must be multiples of 128 and v_rows of 8 (got %lld, %lld, %lld); "
                "run three GEMMs on the row slices of w instead",
                (long long)q_rows, (long long)k_rows, (long long)v_rows);
  }
  const int64_t N = q_rows + k_rows + v_rows;
  if (K > (1 << 20) || N > (1 << 24) || M > (1 << 24)) {
    return fail(VPQ_ERR_UNSUPPORTED, "affine_qmm_qkv_w4g64: shape too large (K=%lld N=%lld M=%lld)", (long long)K,
                (long long)N, (long long)M);
  }
  if (!aligned16(w) || !aligned16(x) || !aligned16(q_out) || !aligned16(k_out) || !aligned16(v_out) ||
      (reinterpret_cast<uintptr_t>(scales) & 1) || (reinterpret_cast<uintptr_t>(biases) & 1)) {
    return fail(VPQ_ERR_ALIGNMENT, "affine_qmm_qkv_w4g64: w, x and the outputs must be 16-byte aligned");
  }
  if (int rc = require_sm100()) { return rc; }
  two_cta::OutSpec out = {};
  out.base[0] = static_cast<__nv_bfloat16*>(q_out);
  out.base[1] = static_cast<__nv_bfloat16*>(k_out);
  out.base[2] = static_cast<__nv_bfloat16*>(v_out);
  out.count = 1;
  out.col0 = 0;
  out.ld = N;
  out.split0 = (int)q_rows;
  out.split1 = (int)(q_rows + k_rows);
  return launch_qmm_2cta_bits<4>(w, static_cast<const uint16_t*>(scales), static_cast<const uint16_t*>(biases), x, out,
                                 (int)K, (int)N, (int)M, static_cast<cudaStream_t>(stream), 0);
}

// The GEMM for any of the format twins: bits 4 | 8, group 64 | 32; act 0 plain, 2 GeGLU (4 bits).
extern "C" int vpq_affine_qmm_bf16(const uint32_t* w, const void* scales, const void* biases, const void* x, void* y,
                                   int64_t K, int64_t N, int64_t M, int bits, int group, int act, void* stream) {
  clear_error();
  if ((bits != 4 && bits != 8) || (group != 64 && group != 32) || (act != 0 && act != 2)) {
    return fail(VPQ_ERR_INVALID_ARG, "affine_qmm: bits must be 4 or 8, group 64 or 32, act 0 or 2 (got %d, %d, %d)", bits,
                group, act);
  }
  if (!w || !scales || !biases || !x || !y) { return fail(VPQ_ERR_INVALID_ARG, "affine_qmm: null pointer"); }
  if (K <= 0 || N <= 0 || M <= 0 || (K % 64) != 0 || (act && (N % 2))) {
    return fail(VPQ_ERR_INVALID_ARG, "affine_qmm: need K>0, N>0 (even for a gated store), M>0, K%%64==0 (K=%lld N=%lld M=%lld)",
                (long long)K, (long long)N, (long long)M);
  }
  if (K > (1 << 20) || N > (1 << 24) || M > (1 << 24)) {
    return fail(VPQ_ERR_UNSUPPORTED, "affine_qmm: shape too large (K=%lld N=%lld M=%lld)", (long long)K, (long long)N,
                (long long)M);
  }
  if (!aligned16(w) || !aligned16(x) || !aligned16(y) || (reinterpret_cast<uintptr_t>(scales) & 1) ||
      (reinterpret_cast<uintptr_t>(biases) & 1)) {
    return fail(VPQ_ERR_ALIGNMENT, "affine_qmm: w, x and y must be 16-byte aligned");
  }
  if (int rc = require_sm100()) { return rc; }
  two_cta::OutSpec out = {};
  out.base[0] = static_cast<__nv_bfloat16*>(y);
  out.count = 1;
  out.col0 = 0;
  out.ld = act ? N / 2 : N;
  out.swiglu = act;
  const uint16_t* s16 = static_cast<const uint16_t*>(scales);
  const uint16_t* b16 = static_cast<const uint16_t*>(biases);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (bits == 8) { return launch_qmm_2cta_bits<8>(w, s16, b16, x, out, (int)K, (int)N, (int)M, st, 0, group); }
  return launch_qmm_2cta_bits<4>(w, s16, b16, x, out, (int)K, (int)N, (int)M, st, 0, group);
}

extern "C" int vpq_affine_qmm_w8g64_bf16(const uint32_t* w, const void* scales, const void* biases, const void* x,
                                         void* y, int64_t K, int64_t N, int64_t M, void* stream) {
  clear_error();
  if (!w || !scales || !biases || !x || !y) { return fail(VPQ_ERR_INVALID_ARG, "affine_qmm_w8g64: null pointer"); }
  if (K <= 0 || N <= 0 || M <= 0 || (K % 64) != 0) {
    return fail(VPQ_ERR_INVALID_ARG, "affine_qmm_w8g64: need K>0, N>0, M>0, K%%64==0 (K=%lld N=%lld M=%lld)",
                (long long)K, (long long)N, (long long)M);
  }
  if (K > (1 << 20) || N > (1 << 24) || M > (1 << 24)) {
    return fail(VPQ_ERR_UNSUPPORTED, "affine_qmm_w8g64: shape too large (K=%lld N=%lld M=%lld)", (long long)K,
                (long long)N, (long long)M);
  }
  if (!aligned16(w) || !aligned16(x) || !aligned16(y) || (reinterpret_cast<uintptr_t>(scales) & 1) ||
      (reinterpret_cast<uintptr_t>(biases) & 1)) {
    return fail(VPQ_ERR_ALIGNMENT, "affine_qmm_w8g64: w, x and y must be 16-byte aligned");
  }
  if (int rc = require_sm100()) { return rc; }
  two_cta::OutSpec out = {};
  out.base[0] = static_cast<__nv_bfloat16*>(y);
  out.count = 1;
  out.col0 = 0;
  out.ld = N;
  return launch_qmm_2cta_bits<8>(w, static_cast<const uint16_t*>(scales), static_cast<const uint16_t*>(biases), x, out,
                                 (int)K, (int)N, (int)M, static_cast<cudaStream_t>(stream), 0);
}

namespace {
int qmm_grouped(const char* who, int act, const uint32_t* w, const void* scales, const void* biases, const void* x,
                void* y, int64_t K, int64_t N, int64_t M, const int* tile2e, const int* srow, const int* sdst,
                int64_t experts, int64_t x_rows, int64_t y_rows, void* x_sorted, void* stream, int bits = 4) {
  clear_error();
  if (!w || !scales || !biases || !x || !y || !tile2e) { return fail(VPQ_ERR_INVALID_ARG, "%s: null pointer", who); }
  if (K <= 0 || N <= 0 || M <= 0 || (K % 64) != 0 || experts <= 0 || y_rows <= 0 || (act && (N % 2) != 0)) {
    return fail(VPQ_ERR_INVALID_ARG,
                "%s: need K>0, N>0 (even for a gated store), M>0, K%%64==0, experts>0, y_rows>0 "
                "(K=%lld N=%lld M=%lld experts=%lld)",
                who, (long long)K, (long long)N, (long long)M, (long long)experts);
  }
  if (K > (1 << 20) || N > (1 << 24) || M > (1 << 24) || N * experts > (1ll << 30) || y_rows > (1ll << 30)) {
    return fail(VPQ_ERR_UNSUPPORTED, "%s: shape too large (K=%lld N=%lld M=%lld experts=%lld)", who, (long long)K,
                (long long)N, (long long)M, (long long)experts);
  }
  if (srow && (!x_sorted || x_rows <= 0)) {
    return fail(VPQ_ERR_INVALID_ARG, "%s: a row gather needs x_rows > 0 and an [M, K] scratch buffer", who);
  }
  if (!aligned16(w) || !aligned16(x) || !aligned16(y) || (srow && !aligned16(x_sorted)) ||
      (reinterpret_cast<uintptr_t>(scales) & 1) || (reinterpret_cast<uintptr_t>(biases) & 1) ||
      (reinterpret_cast<uintptr_t>(tile2e) & 3) || (reinterpret_cast<uintptr_t>(srow) & 3) ||
      (reinterpret_cast<uintptr_t>(sdst) & 3)) {
    return fail(VPQ_ERR_ALIGNMENT, "%s: w, x, y (and the scratch) must be 16-byte aligned, index arrays 4-byte", who);
  }
  if (int rc = require_sm100()) { return rc; }
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const void* xs = x;
  if (srow) {  // the gather the reference fuses into its x loader, as one pass over [M, K]
    const int row_vecs = (int)(K / 8);
    const int64_t total = M * row_vecs;
    const int blocks = (int)std::min<int64_t>((total + 255) / 256, (int64_t)num_sms() * 8);
    gather_rows_kernel<<<blocks, 256, 0, st>>>(static_cast<const uint4*>(x), srow, static_cast<uint4*>(x_sorted),
                                               (int)M, (int)x_rows, row_vecs);
    VPQ_LAUNCH_OK("moe row gather");
    xs = x_sorted;
  }
  const GroupSpec G = {tile2e, sdst, (int)experts, (int)y_rows};
  const uint16_t* s16 = static_cast<const uint16_t*>(scales);
  const uint16_t* b16 = static_cast<const uint16_t*>(biases);
  __nv_bfloat16* yb = static_cast<__nv_bfloat16*>(y);
  if (bits == 8) {
    switch (act) {
      case 0: return launch_qmm_act<256, 0, 8>(w, s16, b16, xs, yb, (int)K, (int)N, (int)M, G, st);
      case 1: return launch_qmm_act<256, 1, 8>(w, s16, b16, xs, yb, (int)K, (int)N, (int)M, G, st);
      default: return launch_qmm_act<256, 2, 8>(w, s16, b16, xs, yb, (int)K, (int)N, (int)M, G, st);
    }
  }
  switch (act) {
    case 0: return launch_qmm_act<256, 0>(w, s16, b16, xs, yb, (int)K, (int)N, (int)M, G, st);
    case 1: return launch_qmm_act<256, 1>(w, s16, b16, xs, yb, (int)K, (int)N, (int)M, G, st);
    default: return launch_qmm_act<256, 2>(w, s16, b16, xs, yb, (int)K, (int)N, (int)M, G, st);
  }
}
}  // namespace

// The grouped GEMMs over 8-bit experts (w u32 [experts * N, K/4]): act 0 down (scatter through sdst),
// 1 SwiGLU, 2 GeGLU (row gather through srow). Replace affine_qmm_grouped_w8g64, _grouped_swiglu_w8g64,
// _grouped_geglu_w8g64 (the 8-bit instantiations, gpu-kernels/metal/quant/affine_qmm_steel.metal:1069-1094,
// 1290-1312,1341-1367).
extern "C" int vpq_affine_qmm_grouped_w8g64_bf16(int act, const uint32_t* w, const void* scales, const void* biases,
                                                 const void* x, void* y, int64_t K, int64_t N, int64_t M,
                                                 const int* tile2e, const int* rows_map, int64_t experts,
                                                 int64_t rows, void* x_sorted, void* stream) {
  if (act < 0 || act > 2) {
    clear_error();
    return fail(VPQ_ERR_INVALID_ARG, "affine_qmm_grouped_w8g64: act must be 0 (down), 1 (swiglu) or 2 (geglu)");
  }
  if (act == 0) {
    return qmm_grouped("affine_qmm_grouped_w8g64", 0, w, scales, biases, x, y, K, N, M, tile2e, nullptr, rows_map, experts, 0,
                       rows_map ? rows : M, nullptr, stream, 8);
  }
  return qmm_grouped(act == 1 ? "affine_qmm_grouped_swiglu_w8g64" : "affine_qmm_grouped_geglu_w8g64", act, w, scales, biases,
                     x, y, K, N, M, tile2e, rows_map, nullptr, experts, rows, M, x_sorted, stream, 8);
}

extern "C" int vpq_qmm_grouped_tile_rows(void) { return BM; }

extern "C" int vpq_affine_qmm_grouped_w4g64_bf16(const uint32_t* w, const void* scales, const void* biases,
                                                 const void* x_sorted, void* y, int64_t K, int64_t N, int64_t M,
                                                 const int* tile2e, const int* sdst, int64_t experts,
                                                 int64_t y_rows, void* stream) {
  return qmm_grouped("affine_qmm_grouped_w4g64", 0, w, scales, biases, x_sorted, y, K, N, M, tile2e, nullptr, sdst,
                     experts, 0, sdst ? y_rows : M, nullptr, stream);
}

extern "C" int vpq_affine_qmm_grouped_swiglu_w4g64_bf16(const uint32_t* w, const void* scales, const void* biases,
                                                        const void* x, void* y, int64_t K, int64_t N, int64_t M,
                                                        const int* tile2e, const int* srow, int64_t experts,
                                                        int64_t x_rows, void* x_sorted, void* stream) {
  return qmm_grouped("affine_qmm_grouped_swiglu_w4g64", 1, w, scales, biases, x, y, K, N, M, tile2e, srow, nullptr,
                     experts, x_rows, M, x_sorted, stream);
}

extern "C" int vpq_affine_qmm_grouped_geglu_w4g64_bf16(const uint32_t* w, const void* scales, const void* biases,
                                                       const void* x, void* y, int64_t K, int64_t N, int64_t M,
                                                       const int* tile2e, const int* srow, int64_t experts,
                                                       int64_t x_rows, void* x_sorted, void* stream) {
  return qmm_grouped("affine_qmm_grouped_geglu_w4g64", 2, w, scales, biases, x, y, K, N, M, tile2e, srow, nullptr,
                     experts, x_rows, M, x_sorted, stream);
}

namespace vpq {
namespace {
// One thread waits, with the kernels' own bounded wait and a caller-chosen poll limit, on an
// mbarrier that nobody arrives at. The wait must run out, record (0x7f << 8) | 0x7f in the status
// word and return: the path every device-side wait takes when its partner never shows up.
__global__ void wait_probe_kernel(uint32_t polls, uint32_t hint_ns) {
  __shared__ uint64_t bar;
  __shared__ uint32_t abort_flag;
  if (threadIdx.x == 0) {
    mbar_init(smem_u32(&bar), 1);
    abort_flag = 0;
    fence_mbar_init();
    mbar_wait_limited(smem_u32(&bar), 0u, (0x7fu << 8) | 0x7fu, &abort_flag, &g_qmm_status, polls, hint_ns);
  }
}
}  // namespace
}  // namespace vpq

extern "C" int vpq_wait_probe(uint32_t polls, uint32_t hint_ns, void* stream) {
  clear_error();
  if (polls == 0 || polls > (1u << 16) || hint_ns > 100000u) {
    return fail(VPQ_ERR_INVALID_ARG, "wait_probe: 0 < polls <= 65536, hint_ns <= 100000 (the probe must end in well under a second)");
  }
  if (int rc = require_sm100()) { return rc; }
  wait_probe_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(polls, hint_ns);
  VPQ_LAUNCH_OK("wait_probe");
  return VPQ_OK;
}

extern "C" int vpq_device_status(void* stream, uint32_t* detail) {
  clear_error();
  if (int rc = require_sm100()) { return rc; }
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  uint32_t v = 0;
  VPQ_CUDA_OK(cudaMemcpyFromSymbolAsync(&v, g_qmm_status, sizeof(v), 0, cudaMemcpyDeviceToHost, st));
  VPQ_CUDA_OK(cudaStreamSynchronize(st));
  uint32_t vq = 0;
  if (int rc = qmv_status_read(st, &vq)) { return rc; }
  if (vq == 0) {
    if (int rc = qmvb_status_read(st, &vq)) { return rc; }  // the small-batch GEMV reports like the GEMV
  }
  if (vq == 0) {
    if (int rc = qmv8_status_read(st, &vq)) { return rc; }  // and the 8-bit one
  }
  if (detail) { *detail = v ? v : (vq ? (vq | 0x10000u) : 0u); }
  uint32_t vn = 0;
  if (int rc = nsplit_status_read(st, &vn)) { return rc; }
  if (vn != 0 && v == 0 && vq == 0) {
    if (detail) { *detail = vn | 0x20000u; }
    return fail(VPQ_ERR_TIMEOUT, "the cross-GPU barrier gave up waiting for rank %u", vn & 0xffu);
  }
  if (vq != 0 && v == 0) {
    return fail(VPQ_ERR_TIMEOUT, "a bounded device-side wait gave up in the GEMV kernel (site %u, role %u)",
                vq >> 8, vq & 0xffu);
  }
  if (v != 0) {
    const uint32_t zero = 0;
    VPQ_CUDA_OK(cudaMemcpyToSymbolAsync(g_qmm_status, &zero, sizeof(zero), 0, cudaMemcpyHostToDevice, st));
    VPQ_CUDA_OK(cudaStreamSynchronize(st));
    return fail(VPQ_ERR_TIMEOUT, "a bounded device-side wait gave up (site %u, role %u)", v >> 8, v & 0xffu);
  }
  return VPQ_OK;
}
