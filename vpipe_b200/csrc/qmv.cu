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
//  * the arithmetic is integer and exact. x is scaled by a power of two, rounded to a 23-bit
//    integer and split into three signed base-256 digits; a packed word becomes tensor-core
//    operands with two LOP3 and no shift: (w & 0x0f0f0f0f) holds its even nibbles as bytes,
//    (w & 0xf0f0f0f0) its odd nibbles times 16, and the two kinds go to separate
//    mma.sync.m16n8k32.u8.s8 accumulators (the second is divided by 16 afterwards). Earlier
//    versions were bound by the integer pipe: a SIMT one (one PRMT and half an f32x2 FMA per
//    nibble), then an fp16 mma.sync one (four LOP3 and a shift per word);
//  * the eight accumulator columns are (digit, group parity): lane t of a quad ends up with the
//    sums of digit t for both quantization groups of a k tile and both of its rows, so every
//    lane folds four (row, group) sums per k tile with that group's scale -- and lane 3, whose
//    digit does not exist, folds the bias term b * sum(x) instead. Accumulators start from the
//    bit pattern of 12582912.0f, so the integer sum reads back as a float with no conversion;
//  * x is staged once per CTA in shared memory, already as digit bytes in B-fragment order; the raw
//    values get there by asynchronous copies, so the staging holds nothing in registers across its
//    passes. The kernel must not have a stack frame: two CTAs of 112 KB shared memory leave an SM
//    less L1 than sixteen warps' spill slots, and a spilled value then costs a trip to L2 (measured:
//    2 us per dependent launch with 176 bytes of frame per thread);
//  * per row tile: two shuffles, one shared-memory reduction over the 8 warps.
// One launch can run a whole list of GEMVs (a "plan"): the CTAs walk the concatenated row tiles
// of all problems, the producer keeps streaming across problem boundaries, and the consumers
// re-stage x only when the next problem reads a different x. A single GEMV is a one-problem list
// passed in the kernel parameters.
// The launch opts into programmatic dependent launch: the producer starts
// streaming weights before griddepcontrol.wait, so the next launch's stream is
// already running while this one drains, and the consumers wait only in front of
// their first read of x, with the problem record already fetched. Every barrier wait is bounded.
#include "vpq_sm100.cuh"

#include <cstdlib>
#include <cstring>
#include <vector>

namespace vpq {

// 0, or (site << 8) | role of the first bounded wait that gave up in this kernel.
__device__ uint32_t g_qmv_status;

namespace {

constexpr int kConsWarps = 8;
constexpr int kConsThreads = kConsWarps * 32;
constexpr int kThreads = kConsThreads + 32;  // + producer warp
constexpr int kBoxBytes = 16 * 128;          // one TMA box: 16 rows x 128 bytes (256 k)
constexpr int kBoxesPerStage = 8;            // a stage spans 2048 k
constexpr int kStageW = kBoxesPerStage * kBoxBytes;  // 16 KB of nibbles
constexpr int kStageSZ = 2 * 16 * 64;        // scales + biases of the span: 2 x [16 rows x 32 groups]
constexpr int kMaxStages = 6;
constexpr int kRedSlots = 8;                 // row tiles whose cross-warp sums may be pending
constexpr int kDynSlots = 8;                 // chunks the producer may have posted ahead of the slowest consumer warp (> ring depth)

// D = A * B + C: A unsigned bytes [16 x 32], B signed bytes [32 x 8], s32 accumulate.
__device__ __forceinline__ void mma_u8s8_16832(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                               uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 "
      "{%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// D = A * B + init: starts an accumulator chain from a constant. The constant sits in four
// registers of its own that only these instructions read, so the hardware's accumulator-input quad
// is there already and no moves are needed to seed the four chains of every stage (16 of ~240
// instructions per stage otherwise).
struct AccInit {
  int c0, c1, c2, c3;
};
__device__ __forceinline__ AccInit make_acc_init(int v) {
  AccInit a;
  // opaque to the compiler on purpose: four equal constants would be merged into one register again
  asm volatile("mov.b32 %0, %4;\n\tmov.b32 %1, %4;\n\tmov.b32 %2, %4;\n\tmov.b32 %3, %4;"
               : "=r"(a.c0), "=r"(a.c1), "=r"(a.c2), "=r"(a.c3)
               : "r"(v));
  return a;
}
__device__ __forceinline__ void mma_u8s8_16832_first(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2,
                                                     uint32_t a3, uint32_t b0, uint32_t b1, const AccInit& init) {
  asm volatile(
      "mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 "
      "{%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%11,%12,%13};"
      : "=r"(c[0]), "=r"(c[1]), "=r"(c[2]), "=r"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "r"(init.c0), "r"(init.c1), "r"(init.c2), "r"(init.c3));
}

// Accumulators start at the bits of 12582912.0f (1.5 * 2^23): while |sum| < 2^22 the integer
// result, read as a float, is exactly 12582912 + sum.
constexpr int kAccInit = 0x4B400000;
constexpr float kAccInitF = 12582912.0f;
// Odd nibbles enter the tensor core as 16 * q: their accumulator, read as a float and divided by
// 16, carries kAccInitF / 16; that and the even accumulator's kAccInitF are removed together.
constexpr float kAccSurplus = kAccInitF / 16.0f + kAccInitF;  // 13369344, exact
constexpr uint32_t kEvenNibbles = 0x0f0f0f0fu;
constexpr uint32_t kOddNibbles = 0xf0f0f0f0u;
constexpr int kXBytesPerKt = 3 * 128;  // staged x per k tile: 3 digits x [4 chunks x 32 bytes]

enum : uint32_t { kRoleProducer = 1, kRoleConsumer = 2 };

// Fused stores (the reference's affine_qmv_w4g64_add, affine_qmv_swiglu_w4g64 and
// affine_qmv_qkv_w4g64, gpu-kernels/metal/quant/affine_qmv.metal:347-363, 806-906, 405-516).

// One GEMV of a launch. Lives in the kernel parameters (single GEMV) or in caller-provided
// device memory (plan). Tensor maps need 64-byte alignment.
struct alignas(64) QmvProblem {
  CUtensorMap mw, ms, mz;      // packed weights [rows, K/8] u32; scales, biases [rows, K/64] (valid if scales_tma)
  const uint16_t* scales;
  const uint16_t* biases;
  const uint16_t* x;           // one row of K bf16
  __nv_bfloat16* y;            // N outputs
  int K, N;
  int tile_begin, row_tiles;   // this problem's range in the launch's global list of 16-row tiles
  int scales_tma;              // scale / bias rows are TMA boxes (pitch and base 16-byte aligned)
  int epilogue;                // kEpi*: what the store does with a row's sum
  int q_rows, k_rows;          // kEpiQkv: rows [0, q_rows) -> y, [q_rows, q_rows + k_rows) -> aux, the rest -> y3
  const uint16_t* aux;         // kEpiAdd: residual, N values; kEpiGeluMul: the multiplier; kEpiQkv: the second output
  __nv_bfloat16* y3;           // kEpiQkv: the third output
  const uint16_t* norm_w;      // not null: x is RMS-normalised with these K weights while it is staged
  const int32_t* eid;          // not null: *eid is the expert whose [N, K] slab of w / scales / biases is used
  float eps;                   // RMSNorm epsilon
  int wait_tiles;              // > 0: tiles of the launch that must be complete before x (and aux) may be read
  int experts;                 // slabs in w (eid is clamped to it)
  int pad0;
  const int32_t* xrow;         // not null: x is row max(*xrow, 0) of the matrix P.x points at (sorted-slot gather)
  const int32_t* vrow;         // not null: the slot is live, and its outputs are stored, only if *vrow >= 0 (and *eid >= 0)
};
static_assert(sizeof(QmvProblem) == 512, "problem records are laid out back to back");

// How a launch's row tiles are dealt to the CTAs.
//   single: one GEMV in the kernel parameters, tiles split evenly.
//   ranges: a list of independent GEMVs; the host's table gives every CTA one contiguous run of the
//           concatenated tiles. A plan may keep the last tenth of its tiles out of the table, as a
//           pool of chunks (a few tiles of one GEMV each): a CTA that has finished its run takes
//           chunks from the pool until it is empty, so the CTAs of slower SMs end up with less. The
//           producer thread claims a chunk (one atomic add on a counter in the plan's workspace) and
//           posts it to its consumers through a small queue in shared memory.
//   chain:  a list whose GEMVs may read what earlier ones wrote. Every GEMV is spread over the whole
//           grid (as evenly as its tiles go), a
//           counter in global memory counts finished tiles, and a GEMV with wait_tiles > 0 stages its
//           x only once that many tiles are complete. The producer warp does not wait: weights are
//           constants, so the stream of GEMV i + 1 runs while GEMV i drains. The launch must be
//           cooperative (all CTAs resident), since CTAs wait on one another.
struct Walk {
  const QmvProblem* P;  // current problem
  int tile;             // next tile of P for this CTA
  int hi;               // end of this CTA's tiles in P
  int left;             // single / ranges: tiles left in this CTA's run; chain: problems after P
  __device__ __forceinline__ Walk(const QmvProblem* single, const QmvProblem* list, const int2* ranges,
                                  int total_tiles, int count, bool chain) {
    if (chain) {
      P = list - 1;
      tile = hi = 0;
      left = count;
      return;
    }
    int gt, gt_end;
    P = list ? list : single;
    if (ranges) {
      const int2 a = ranges[blockIdx.x], b = ranges[blockIdx.x + 1];
      gt = a.x;
      gt_end = b.x;
      P += a.y;
    } else {
      // as evenly as the tiles go, the extras to the lowest CTAs: those are placed first, one per SM,
      // so no SM gets two of the extras while another has none
      const int grid = (int)gridDim.x, b = (int)blockIdx.x;
      const int q = total_tiles / grid, r = total_tiles - q * grid;
      gt = b * q + min(b, r);
      gt_end = gt + q + (b < r ? 1 : 0);
    }
    tile = gt - P->tile_begin;
    hi = P->row_tiles;
    left = gt_end - gt;
  }
  // The producer thread's way into the pool: claims the next chunk and posts it (or the end mark,
  // a chunk of no tiles) to the consumer warps. False when the pool is empty.
  // `dyn_n`: chunks taken so far.
  __device__ __forceinline__ bool claim_chunk(const QmvProblem* list, uint32_t* dq, uint32_t* dyn, const int4* chunks,
                                              int num_chunks, volatile uint32_t* abort_flag, uint32_t& dyn_n) {
    // The counter belongs to the previous launch of the plan until that launch has ended.
    if (dyn_n == 0) { asm volatile("griddepcontrol.wait;" ::: "memory"); }
    // (after a wait of this CTA has given up its consumers may be gone: claim nothing more)
    const uint32_t c = *abort_flag ? (uint32_t)num_chunks : atomicAdd(dyn, 1u);
    const int4 ch = c < (uint32_t)num_chunks ? __ldg(chunks + c) : make_int4(0, 0, 0, 0);
    volatile uint32_t* e = dq + (dyn_n & (kDynSlots - 1)) * 4;
    e[0] = (uint32_t)ch.x;
    e[1] = (uint32_t)ch.y;
    e[2] = (uint32_t)ch.z;
    __threadfence_block();
    ++dyn_n;
    *reinterpret_cast<volatile uint32_t*>(dq + kDynSlots * 4) = dyn_n;
    if (ch.z == 0) { return false; }
    P = list + ch.y;
    tile = ch.x - P->tile_begin;
    hi = P->row_tiles;
    left = ch.z;
    return true;
  }
  // A consumer warp's way: waits (bounded) for the producer's next post. False at the end mark.
  __device__ __forceinline__ bool receive_chunk(const QmvProblem* list, const uint32_t* dq, volatile uint32_t* abort_flag,
                                                uint32_t& dyn_n) {
    uint32_t gt = 0, prob = 0, cnt = 0;
    if ((threadIdx.x & 31) == 0) {
      const volatile uint32_t* posted = dq + kDynSlots * 4;
      bool got = false;
      for (uint32_t i = 0; i < (1u << 28); ++i) {
        if (*posted > dyn_n) {
          got = true;
          break;
        }
        if (*abort_flag) { break; }
      }
      if (got) {
        __threadfence_block();
        const volatile uint32_t* e = dq + (dyn_n & (kDynSlots - 1)) * 4;
        gt = e[0];
        prob = e[1];
        cnt = e[2];
      } else if (!*abort_flag) {
        *abort_flag = 1;
        atomicCAS(&g_qmv_status, 0u, (5u << 8) | kRoleConsumer);
      }
    }
    gt = __shfl_sync(0xffffffffu, gt, 0);
    prob = __shfl_sync(0xffffffffu, prob, 0);
    cnt = __shfl_sync(0xffffffffu, cnt, 0);
    ++dyn_n;
    if (cnt == 0) { return false; }
    P = list + prob;
    tile = (int)gt - P->tile_begin;
    hi = P->row_tiles;
    left = (int)cnt;
    return true;
  }
  // Advances to this CTA's next run of tiles [lo, hi) inside one problem (P). When it returns false
  // in a launch with a pool, claim_chunk / receive_chunk refill the walk and the caller asks again.
  __device__ __forceinline__ bool next_range(int& lo, int& out_hi, bool chain) {
    if (!chain) {
      if (left <= 0) { return false; }
      if (tile >= hi) {
        ++P;
        tile = 0;
        hi = P->row_tiles;
      }
      lo = tile;
      out_hi = min(hi, tile + left);
      left -= out_hi - lo;
      tile = out_hi;
      return true;
    }
    for (;;) {
      if (left <= 0) { return false; }
      --left;
      ++P;
      // rt tiles over the whole grid as evenly as they go: CTA b takes rt / grid tiles, the first
      // rt % grid CTAs one more (consecutive CTAs sit on different SMs, so no SM gets two of the extras
      // while others have none)
      const int rt = P->row_tiles, grid = (int)gridDim.x, b = (int)blockIdx.x;
      const int q = rt / grid, r = rt - q * grid;
      lo = b * q + min(b, r);
      out_hi = lo + q + (b < r ? 1 : 0);
      if (lo < out_hi) { return true; }
    }
  }
};

__device__ __forceinline__ uint32_t ld_acquire_u32(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

// A tensor map that lives in global memory may have been rewritten since this SM last used the
// address (a plan re-created in the same workspace, the fixed array of the no-allocation entry):
// the acquire fence makes the copy the TMA unit reads current.
__device__ __forceinline__ void tensormap_acquire(const CUtensorMap* m) {
  asm volatile("fence.proxy.tensormap::generic.acquire.gpu [%0], 128;" ::"l"(m) : "memory");
}

// Shared memory behind the stage ring (p0 = its end), in this order; cap_kt = k tiles of the longest x.
struct Scratch {
  uint4* zero128;        // 128 bytes of zeros, 128-byte aligned
  unsigned char* xq;     // [cap_kt][3 digits][4 chunks][32 B]
  float* xg;             // [2 * cap_kt] sum of X per group
  float* zero16;         // four times -kAccSurplus: "no bias term" in the form the fold wants
  float* xu;             // [cap_kt / 2] 1 / scale of every 256-k box of x
  float* red;            // [kRedSlots][kConsWarps][16]
  uint32_t* red_cnt;     // [kRedSlots]
  float* sq_part;        // [2][kConsWarps]
  // [0], [1]: warps that posted their sum of squares; [2]: consumer warps that left; [3]: tiles this CTA
  // finished (chain); [4]: largest dependency a warp of this CTA has claimed the polling of; [5]: largest
  // dependency known to be satisfied
  uint32_t* sq_cnt;
  uint64_t* bars;
  volatile uint32_t* abort_flag;
  // chunks of the launch's shared pool the producer has claimed for this CTA: kDynSlots entries of
  // {first tile, problem, tiles, -}, then the number of entries posted so far
  uint32_t* dq;
  __device__ __forceinline__ Scratch(unsigned char* p0, int cap_kt) {
    zero128 = reinterpret_cast<uint4*>(p0);
    xq = p0 + 128;
    xg = reinterpret_cast<float*>(xq + (size_t)cap_kt * kXBytesPerKt);
    zero16 = xg + 2 * cap_kt;  // cap_kt is even
    xu = zero16 + 4;
    red = xu + ((cap_kt / 2 + 3) & ~3);
    red_cnt = reinterpret_cast<uint32_t*>(red + kRedSlots * kConsWarps * 16);
    sq_part = reinterpret_cast<float*>(red_cnt + kRedSlots);
    sq_cnt = reinterpret_cast<uint32_t*>(sq_part + 2 * kConsWarps);
    bars = reinterpret_cast<uint64_t*>(sq_cnt + 8);
    abort_flag = reinterpret_cast<volatile uint32_t*>(bars + 2 * kMaxStages);
    dq = reinterpret_cast<uint32_t*>(bars + 2 * kMaxStages) + 4;
  }
};

constexpr uint32_t kDepPolls = 1u << 21;  // polls (an L2 round trip each) of the tile counter before a dependent GEMV gives up: seconds

// ---- staging of one x vector as signed digit bytes. Warp w converts exactly the 256-k boxes it
// will multiply (box w of every stage), so no CTA barrier is involved: a half warp takes one
// box, a lane 16 consecutive values. Every box carries its own power-of-two scale: its largest
// magnitude lands in [2^21, 2^22) and every value is rounded to an integer X, so a value is
// exact if it lies within 2^-14 of the largest of its 256 neighbours and is off by at most
// 2^-22 of that neighbour otherwise (one huge activation costs nothing outside its own box).
// X = d0 + 256 d1 + 65536 d2 with digits in [-128, 127] (adding 0x808080 turns the balanced
// digits into plain bytes; an xor takes the offset off again in two's complement). Per digit a
// lane stores the 16 bytes one lane feeds to an even-nibble MMA (x0,x2,x4,x6 of packed word
// w0 | of w1) and an odd-nibble MMA (x1,x3,x5,x7 of w0 | of w1). xg[group] = sum of the 64 X of
// the group (for the bias term), xu[box] = 1 / scale.
// With norm_w the vector is first RMS-normalised as the reference's fused kernel does
// (affine_qmv_qkv_rms_w4g64, gpu-kernels/metal/quant/affine_qmv.metal:570-694): sum of squares
// in f32 over the whole vector (the warps exchange their partial sums through one consumer
// barrier), x <- bf16(x * rsqrt(mean + eps) * norm_w).
__device__ __forceinline__ bool stage_x(const QmvProblem* P, unsigned char* p0, int cap_kt, int sq_gen, int need,
                                     const uint32_t* sync) {
  const Scratch sc(p0, cap_kt);
  unsigned char* xq = sc.xq;
  float* xg = sc.xg;
  float* xu = sc.xu;
  float* sq_part = sc.sq_part;
  uint32_t* sq_cnt = sc.sq_cnt;
  volatile uint32_t* abort_flag = sc.abort_flag;
  const int K = P->K;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int half = lane >> 4, sub = lane & 15;
  const uint16_t* xr = P->x;
  const int32_t* xrow = P->xrow;
  const uint16_t* nw = P->norm_w;
  const int NB = (K + 255) >> 8;
  const int passes = (((NB + kBoxesPerStage - 1) / kBoxesPerStage) + 1) >> 1;  // two boxes of this warp per pass
  auto box_of = [&](int j) { return (2 * j + half) * kBoxesPerStage + warp; };
  auto k_of = [&](int j) { return (box_of(j) << 8) + sub * 16; };
  // This lane's 32 raw bytes of box `box` wait inside the box's own 768 bytes of xq until they are converted.
  auto raw_of = [&](int box) { return xq + (size_t)box * (2 * kXBytesPerKt) + sub * 32; };
  auto load_piece = [&](int j, uint4& a, uint4& b) {
    a = b = make_uint4(0, 0, 0, 0);
    if (box_of(j) < NB) {
      const unsigned char* raw = raw_of(box_of(j));
      a = *reinterpret_cast<const uint4*>(raw);
      b = *reinterpret_cast<const uint4*>(raw + 16);
    }
  };
  if (nw) {  // the norm weights are constants: bring this lane's share into L1 before waiting for x
    for (int j = 0; j < passes; ++j) {
      const int k0 = k_of(j);
      if (k0 < K) { asm volatile("prefetch.global.L1 [%0];" ::"l"(nw + k0)); }
    }
  }
  // Everything above reads the problem record and constants of the model; from here on the kernel
  // touches what the previous kernel in the stream may still be writing (x, the routed rows, and
  // later the residual and y), so this is where it waits for it. The record's fields are in flight
  // during the wait instead of after it.
  asm volatile("griddepcontrol.wait;" ::: "memory");
  if (xrow) { xr += (size_t)max(__ldg(xrow), 0) * (size_t)K; }   // a dead slot reads row 0 and stores nothing
  if (need > 0) {
    // This GEMV reads what earlier GEMVs of the launch wrote: wait (bounded) until their tiles are
    // counted. One warp per CTA polls the counter in global memory (the first to get here claims
    // it), the others watch a flag in shared memory, so a dependency costs the L2 one poller per CTA.
    uint32_t seen = 0;
    if (lane == 0) {
      volatile uint32_t* dep_seen = sq_cnt + 5;
      if (*dep_seen >= (uint32_t)need) {
        seen = 1;
      } else if (atomicMax(sq_cnt + 4, (uint32_t)need) < (uint32_t)need) {  // this warp polls for the CTA
        for (uint32_t i = 0; i < kDepPolls; ++i) {
          if (ld_acquire_u32(sync) >= (uint32_t)need) {
            seen = 1;
            break;
          }
          if (*abort_flag) { break; }
        }
        if (seen) {
          __threadfence_block();
          *dep_seen = (uint32_t)need;
        }
      } else {
        for (uint32_t i = 0; i < 64u * kDepPolls; ++i) {
          if (*dep_seen >= (uint32_t)need) {
            seen = 1;
            break;
          }
          if (*abort_flag) { break; }
        }
      }
      if (!seen) {
        *abort_flag = 1;
        atomicCAS(&g_qmv_status, 0u, (3u << 8) | kRoleConsumer);
      }
      __threadfence_block();  // the poller's acquire reaches the other warps through the flag in shared memory
    }
    seen = __shfl_sync(0xffffffffu, seen, 0);
    if (!seen) { return false; }
  }
  // All of this warp's boxes are fetched at once, asynchronously and past L1 (x may have been written
  // by another SM a moment ago), so a long vector costs one trip to L2 and no registers; past K the
  // copy fills zeros.
  for (int j = 0; j < passes; ++j) {
    if (box_of(j) < NB) {
      const int k0 = k_of(j);
      const uint32_t dst = smem_u32(raw_of(box_of(j)));
      const uint32_t n = k0 < K ? 16u : 0u;
      const uint16_t* src = xr + (k0 < K ? k0 : 0);
      asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(n) : "memory");
      asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst + 16u), "l"(src + 8), "r"(n) : "memory");
    }
  }
  asm volatile("cp.async.wait_all;" ::: "memory");
  float inv = 1.0f;
  if (nw) {
    float sq = 0.0f;
    auto add_sq = [&](const uint4& in) {
      const uint32_t v[4] = {in.x, in.y, in.z, in.w};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float lo = __uint_as_float(v[j] << 16), hi = __uint_as_float(v[j] & 0xffff0000u);
        sq = __fmaf_rn(lo, lo, sq);
        sq = __fmaf_rn(hi, hi, sq);
      }
    };
    for (int j = 0; j < passes; ++j) {
      uint4 a, b;
      load_piece(j, a, b);
      add_sq(a);
      add_sq(b);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) { sq += __shfl_xor_sync(0xffffffffu, sq, o); }
    // The warps exchange their partial sums through shared memory: post, count, wait (bounded, and
    // given up at once if a warp of this CTA has aborted) until all eight have posted. Uses alternate
    // between the two halves of sq_part, so a warp that runs ahead cannot overwrite sums still being read.
    const int sq_par = sq_gen & 1;
    const uint32_t target = (uint32_t)kConsWarps * (uint32_t)(sq_gen / 2 + 1);
    uint32_t all = 1;
    if (lane == 0) {
      sq_part[sq_par * kConsWarps + warp] = sq;
      __threadfence_block();
      atomicAdd(&sq_cnt[sq_par], 1u);
      all = 0;
      for (uint32_t i = 0; i < (1u << 28); ++i) {
        if (*reinterpret_cast<volatile uint32_t*>(&sq_cnt[sq_par]) >= target) {
          all = 1;
          break;
        }
        if (*abort_flag) { break; }
      }
      if (!all) {
        *abort_flag = 1;
        atomicCAS(&g_qmv_status, 0u, (4u << 8) | kRoleConsumer);
      }
      __threadfence_block();
    }
    all = __shfl_sync(0xffffffffu, all, 0);
    if (!all) { return false; }
    float total = 0.0f;
#pragma unroll
    for (int ww = 0; ww < kConsWarps; ++ww) {
      total += *reinterpret_cast<volatile float*>(&sq_part[sq_par * kConsWarps + ww]);
    }
    inv = __frsqrt_rn(__fadd_rn(__fdiv_rn(total, (float)K), P->eps));
  }
  auto convert_piece = [&](int j, const uint4& in0, const uint4& in1) {  // whole warps: shuffles inside
    const int box = (2 * j + half) * kBoxesPerStage + warp;
    const bool live = box < NB;
    uint32_t v[8] = {in0.x, in0.y, in0.z, in0.w, in1.x, in1.y, in1.z, in1.w};
    if (nw) {
      const int k0 = k_of(j);
      uint4 n0 = make_uint4(0, 0, 0, 0), n1 = n0;
      if (k0 < K) {
        n0 = __ldg(reinterpret_cast<const uint4*>(nw + k0));
        n1 = __ldg(reinterpret_cast<const uint4*>(nw + k0 + 8));
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
    uint32_t amax = 0;  // largest |x| of the box as bf16 bits (ordering of magnitudes == ordering of bit patterns)
#pragma unroll
    for (int q = 0; q < 8; ++q) { amax = __vmaxu2(amax, v[q] & 0x7fff7fffu); }  // both halves at once
    amax = max(amax & 0xffffu, amax >> 16);
#pragma unroll
    for (int o = 8; o > 0; o >>= 1) { amax = max(amax, __shfl_xor_sync(0xffffffffu, amax, o)); }
    int e = (int)(amax >> 7);            // biased exponent of the largest magnitude
    e = min(max(e, 22), 254);            // all-zero / denormal box: keep both factors normal
    const float x_scale = __uint_as_float((uint32_t)(275 - e) << 23);   // 2^(148 - e): max |x| -> [2^21, 2^22)
    // round(x * scale) without the conversion unit: the low bits of fma(x, scale, 1.5 * 2^23)
    // are 0x4B400000 + X. One add moves that to X + 0x808080 (bytes 0..2: digits + 128; byte 3
    // is never used); the + 128 is taken off the transposed words below.
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
    // byte d of za, zb, zc, zd -> one word per digit d
    auto digits_of4 = [](uint32_t za, uint32_t zb, uint32_t zc, uint32_t zd, uint32_t (&out)[3]) {
      const uint32_t t0 = __byte_perm(za, zb, 0x5140), t1 = __byte_perm(zc, zd, 0x5140);
      const uint32_t t2 = __byte_perm(za, zb, 0x0062), t3 = __byte_perm(zc, zd, 0x0062);
      out[0] = __byte_perm(t0, t1, 0x5410) ^ 0x80808080u;
      out[1] = __byte_perm(t0, t1, 0x7632) ^ 0x80808080u;
      out[2] = __byte_perm(t2, t3, 0x5410) ^ 0x80808080u;
    };
    uint32_t e0[3], o0[3], e1[3], o1[3];
    digits_of4(z[0], z[2], z[4], z[6], e0);
    digits_of4(z[1], z[3], z[5], z[7], o0);
    digits_of4(z[8], z[10], z[12], z[14], e1);
    digits_of4(z[9], z[11], z[13], z[15], o1);
    const int i = box * 16 + sub;  // index of this 16-value piece in the padded x
    if (live) {
      unsigned char* dst = xq + (size_t)(i >> 3) * kXBytesPerKt + (i & 7) * 16;
#pragma unroll
      for (int d = 0; d < 3; ++d) {
        *reinterpret_cast<uint4*>(dst + d * 128) = make_uint4(e0[d], e1[d], o0[d], o1[d]);
      }
    }
    sum += __shfl_xor_sync(0xffffffffu, sum, 1);
    sum += __shfl_xor_sync(0xffffffffu, sum, 2);
    // (stored with the accumulators' surplus already taken off: the fold then needs no subtraction)
    if (live && (sub & 3) == 0) { xg[i >> 2] = (float)(int)sum - kAccSurplus; }
    if (live && sub == 0) { xu[box] = __uint_as_float((uint32_t)(e - 21) << 23); }  // exact inverse of x_scale
  };
  for (int j = 0; j < passes; ++j) {
    uint4 a, b;
    load_piece(j, a, b);
    __syncwarp();  // every lane holds its raw piece before the digits of the box overwrite it
    convert_piece(j, a, b);
  }
  __syncwarp();
  return true;
}


// The producer: one thread streams the weights, scales and biases of this CTA's tiles into the ring.
// They are constants of the model, so the stream waits neither for the previous kernel nor for an
// earlier GEMV of a chain.
__device__ __noinline__ void produce(const QmvProblem* single, const QmvProblem* list, const int2* ranges,
                                     int total_tiles, int stages, int count, bool chain, uint32_t base, uint32_t bar0,
                                     volatile uint32_t* abort_flag, uint32_t* dq, uint32_t* dyn, const int4* chunks,
                                     int num_chunks) {
  constexpr int kStageBytes = kStageW + kStageSZ;
  auto bar_full = [&](int s) { return bar0 + 8u * s; };
  auto bar_empty = [&](int s) { return bar0 + 8u * (kMaxStages + s); };
  uint32_t it = 0;
  bool ok = true;
  Walk wk(single, list, ranges, total_tiles, count, chain);
  int NB = 0, SPT = 0, row0 = 0;
  bool sz_tma = false;
  const QmvProblem* fenced = nullptr;  // the problem whose tensor maps were made current last
  auto acquire_maps = [&](const QmvProblem* Q) {
    tensormap_acquire(&Q->mw);
    if (Q->scales_tma) {
      tensormap_acquire(&Q->ms);
      tensormap_acquire(&Q->mz);
    }
    fenced = Q;
  };
  int lo = 0, hi = 0;
  uint32_t dyn_n = 0;
  while (ok && (wk.next_range(lo, hi, chain) ||
                (dyn && wk.claim_chunk(list, dq, dyn, chunks, num_chunks, abort_flag, dyn_n) &&
                 wk.next_range(lo, hi, chain)))) {
    const QmvProblem* P = wk.P;
    NB = (P->K + 255) >> 8;                              // 128-byte boxes per row
    SPT = (NB + kBoxesPerStage - 1) / kBoxesPerStage;    // stages per row tile
    sz_tma = P->scales_tma != 0;
    row0 = 0;
    if (P->eid) {
      // the routed expert is an output of an earlier kernel: unlike the weights it must be waited for
      asm volatile("griddepcontrol.wait;" ::: "memory");
      row0 = min(max(__ldg(P->eid), 0), P->experts - 1) * P->N;
    }
    if (list && P != fenced) { acquire_maps(P); }
    for (int tile = lo; tile < hi && ok; ++tile) {
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
          tma_load_2d(dst + b * kBoxBytes, &P->mw, bar_full(s), (st * kBoxesPerStage + b) * 32, row0 + tile * 16);
        }
        if (sz_tma) {
          tma_load_2d(dst + kStageW, &P->ms, bar_full(s), st * 32, row0 + tile * 16);
          tma_load_2d(dst + kStageW + kStageSZ / 2, &P->mz, bar_full(s), st * 32, row0 + tile * 16);
        }
      }
    }
    // The walk moves on to the next problem now: make its tensor maps current while this problem's
    // loads are in flight, instead of in front of its first load.
    if (list && ok && wk.left > 0 && (chain || wk.tile >= wk.hi)) { acquire_maps(P + 1); }
  }
  // Never leave with a copy still in flight: wait for the last load of every stage.
  for (int s = 0; s < stages; ++s) {
    if (it > (uint32_t)s) {
      const uint32_t last = ((it - 1 - s) / stages) * stages + s;
      mbar_wait(bar_full(s), (last / stages) & 1u, (2u << 8) | kRoleProducer, abort_flag, &g_qmv_status);
    }
  }
}

// The tiles [lo, hi) of one GEMV for this CTA's eight consumer warps: the hot loop, in a function
// of its own so that it gets its own register allocation. `state` carries the ring position and
// the tile count between calls: bits 0..2 stage, bit 3 phase, bits 4.. tiles processed; the
// return value is the new state, or kConsumeFailed if a bounded wait gave up.
constexpr uint32_t kConsumeFailed = 0xffffffffu;

__device__ __forceinline__ uint32_t consume_tiles(const QmvProblem* P, int lo, int hi, uint32_t state, unsigned char* base_ptr,
                                               int stages, int cap_kt, uint32_t* sync) {
  constexpr int kStageBytes = kStageW + kStageSZ;
  const Scratch sc(base_ptr + (size_t)stages * kStageBytes, cap_kt);
  uint4* zero128 = sc.zero128;
  unsigned char* xq = sc.xq;
  float* xg = sc.xg;
  float* zero16 = sc.zero16;
  float* xu = sc.xu;
  float* red = sc.red;
  uint32_t* red_cnt = sc.red_cnt;
  uint32_t* sq_cnt = sc.sq_cnt;
  volatile uint32_t* abort_flag = sc.abort_flag;
  const uint32_t bar0 = smem_u32(sc.bars);
  auto bar_full = [&](int s) { return bar0 + 8u * s; };
  auto bar_empty = [&](int s) { return bar0 + 8u * (kMaxStages + s); };
  const int lane = threadIdx.x & 31;
  const int warp = threadIdx.x >> 5;
  const int g = lane >> 2, t = lane & 3;
  const int rho = (g >> 1) | ((g & 1) << 2);  // stage row of MMA row g (g+8 -> rho+8): bank-conflict-free
  const bool chain = sync != nullptr;

  // Accumulator column c of an MMA is supplied by the lanes with g == c and stands for
  // (digit c >> 1, group parity c & 1): those lanes feed the digit's bytes if their chunk t lies
  // in that group (t >> 1 == parity) and zeros otherwise (digit 3 does not exist: always zeros).
  // Zeros come from a block laid out like one digit of one k tile, read at the other 16-byte half
  // of the lane's 32-byte slot, so real and zero lanes of a quarter warp never share a bank.
  const bool real = (g < 6) && ((t >> 1) == (g & 1));
  const unsigned char* xop_base =
      real ? xq + (g >> 1) * 128 + t * 32 : reinterpret_cast<const unsigned char*>(zero128) + t * 32 + 16;
  const int xop_kt = real ? kXBytesPerKt : 0;
  const int xop_second = real ? 16 : -16;
  // Lane 3 of a quad folds the bias term: it reads biases where the others read scales, and the
  // group sums of x where the others read zeros.
  const bool bias_lane = t == 3;
  const float* xs_base = bias_lane ? xg : zero16;
  const int xs_box = bias_lane ? 4 : 0;
  const float digit_weight = t == 1 ? 256.0f : t == 2 ? 65536.0f : 1.0f;

  // byte offsets of this lane's two 16-byte reads inside its box, per half (k tile) of the box
  const uint32_t off_h0 = (uint32_t)rho * 128u + (uint32_t)(((0 + t) ^ rho) << 4);
  const uint32_t off_h1 = (uint32_t)rho * 128u + (uint32_t)(((4 + t) ^ rho) << 4);
  // this lane's 8 bytes (4 groups of the warp's box) of row rho in the stage's scales or biases. The
  // 64-byte rows arrive with the 64-byte swizzle (16-byte chunk ^= (row >> 1) & 3), so the eight
  // rows a warp reads lie in eight different banks instead of two.
  const uint32_t sz_off = (uint32_t)kStageW + (bias_lane ? (uint32_t)kStageSZ / 2 : 0u) + (uint32_t)rho * 64u +
                          (uint32_t)((((warp >> 1) ^ (rho >> 1)) & 3) << 4) + (uint32_t)(warp & 1) * 8u;

  const AccInit acc_init = make_acc_init(kAccInit);
  int s = (int)(state & 7u);
  uint32_t ph = (state >> 3) & 1u;
  uint32_t tile_seq = state >> 4;
  bool ok = true;
  const int KT = ((P->K + 255) >> 8) * 2;  // k tiles per row, padded to whole 256-k boxes (x is zero there)
  const int SPT = ((KT >> 1) + kBoxesPerStage - 1) / kBoxesPerStage;
  const bool sz_tma = P->scales_tma != 0;
  for (int tile = lo; tile < hi; ++tile) {
    float res_a = 0.0f, res_b = 0.0f;  // rows rho and rho + 8 of the tile: this lane's digit (or bias) share
    for (int st = 0; st < SPT; ++st) {
      if (!warp_wait(bar_full(s), ph, (1u << 8) | kRoleConsumer, abort_flag, &g_qmv_status)) {
        ok = false;
        break;
      }
      const unsigned char* sb = base_ptr + (size_t)s * kStageBytes;
      const int kt0 = st * 16 + warp * 2;  // this warp's box holds k tiles kt0 and kt0 + 1
      if (kt0 < KT) {
        const unsigned char* box = sb + warp * kBoxBytes;
        const uint4 ra0 = *reinterpret_cast<const uint4*>(box + off_h0);         // row rho,     k tile kt0
        const uint4 rb0 = *reinterpret_cast<const uint4*>(box + off_h0 + 1024);  // row rho + 8
        const uint4 ra1 = *reinterpret_cast<const uint4*>(box + off_h1);         // row rho,     k tile kt0 + 1
        const uint4 rb1 = *reinterpret_cast<const uint4*>(box + off_h1 + 1024);
        const unsigned char* xop = xop_base + kt0 * xop_kt;
        const uint4 x00 = *reinterpret_cast<const uint4*>(xop);                  // kt0, words 0 1
        const uint4 x01 = *reinterpret_cast<const uint4*>(xop + xop_second);     // kt0, words 2 3
        const uint4 x10 = *reinterpret_cast<const uint4*>(xop + xop_kt);
        const uint4 x11 = *reinterpret_cast<const uint4*>(xop + xop_kt + xop_second);
        uint2 sa, sb2;  // 4 consecutive groups' scales (or biases) of rows rho, rho + 8
        if (sz_tma) {
          sa = *reinterpret_cast<const uint2*>(sb + sz_off);
          sb2 = *reinterpret_cast<const uint2*>(sb + sz_off + 512);
        } else {
          // clamped onto valid data: a clamped group meets x == 0, a clamped row is never stored
          const uint16_t* src = bias_lane ? P->biases : P->scales;
          const int G = P->K >> 6, N = P->N;
          const int64_t row0 = P->eid ? (int64_t)min(max(__ldg(P->eid), 0), P->experts - 1) * N : 0;
          const int64_t r_a = row0 + min(tile * 16 + rho, N - 1), r_b = row0 + min(tile * 16 + rho + 8, N - 1);
          const int g0 = min(2 * kt0, G - 1), g1 = min(2 * kt0 + 1, G - 1);
          const int g2 = min(2 * kt0 + 2, G - 1), g3 = min(2 * kt0 + 3, G - 1);
          sa.x = ldg_nc_u16(src + r_a * G + g0) | (ldg_nc_u16(src + r_a * G + g1) << 16);
          sa.y = ldg_nc_u16(src + r_a * G + g2) | (ldg_nc_u16(src + r_a * G + g3) << 16);
          sb2.x = ldg_nc_u16(src + r_b * G + g0) | (ldg_nc_u16(src + r_b * G + g1) << 16);
          sb2.y = ldg_nc_u16(src + r_b * G + g2) | (ldg_nc_u16(src + r_b * G + g3) << 16);
        }
        const float4 xs = *reinterpret_cast<const float4*>(xs_base + (kt0 >> 1) * xs_box);
        const float xu_box = xu[kt0 >> 1];
        // four independent chains: even / odd nibbles of each k tile
        int ce0[4], co0[4], ce1[4], co1[4];
        mma_u8s8_16832_first(ce0, ra0.x & kEvenNibbles, rb0.x & kEvenNibbles, ra0.y & kEvenNibbles,
                             rb0.y & kEvenNibbles, x00.x, x00.y, acc_init);
        mma_u8s8_16832_first(ce1, ra1.x & kEvenNibbles, rb1.x & kEvenNibbles, ra1.y & kEvenNibbles,
                             rb1.y & kEvenNibbles, x10.x, x10.y, acc_init);
        mma_u8s8_16832_first(co0, ra0.x & kOddNibbles, rb0.x & kOddNibbles, ra0.y & kOddNibbles,
                             rb0.y & kOddNibbles, x00.z, x00.w, acc_init);
        mma_u8s8_16832_first(co1, ra1.x & kOddNibbles, rb1.x & kOddNibbles, ra1.y & kOddNibbles,
                             rb1.y & kOddNibbles, x10.z, x10.w, acc_init);
        mma_u8s8_16832(ce0, ra0.z & kEvenNibbles, rb0.z & kEvenNibbles, ra0.w & kEvenNibbles,
                       rb0.w & kEvenNibbles, x01.x, x01.y);
        mma_u8s8_16832(ce1, ra1.z & kEvenNibbles, rb1.z & kEvenNibbles, ra1.w & kEvenNibbles,
                       rb1.w & kEvenNibbles, x11.x, x11.y);
        mma_u8s8_16832(co0, ra0.z & kOddNibbles, rb0.z & kOddNibbles, ra0.w & kOddNibbles,
                       rb0.w & kOddNibbles, x01.z, x01.w);
        mma_u8s8_16832(co1, ra1.z & kOddNibbles, rb1.z & kOddNibbles, ra1.w & kOddNibbles,
                       rb1.w & kOddNibbles, x11.z, x11.w);
        // c[0] = (row rho, first group of the k tile) c[1] = (rho, second) c[2] = (rho + 8, first)
        // c[3] = (rho + 8, second); value = even + odd / 16 - surplus (+ sum of x in a bias lane,
        // whose accumulators hold the bare initial value). The four groups of the box are folded
        // with their scales first, then the box's 1 / x-scale brings the sum to true units.
        const float k0 = xs.x, k1 = xs.y, k2 = xs.z, k3 = xs.w;  // sum of x (bias lanes) or 0, minus the surplus
        auto val = [](int even, int odd, float k) {
          return __int_as_float(even) + __fmaf_rn(__int_as_float(odd), 0.0625f, k);
        };
        float box_a = __fmul_rn(__uint_as_float(sa.x << 16), val(ce0[0], co0[0], k0));
        box_a = __fmaf_rn(__uint_as_float(sa.x & 0xffff0000u), val(ce0[1], co0[1], k1), box_a);
        box_a = __fmaf_rn(__uint_as_float(sa.y << 16), val(ce1[0], co1[0], k2), box_a);
        box_a = __fmaf_rn(__uint_as_float(sa.y & 0xffff0000u), val(ce1[1], co1[1], k3), box_a);
        float box_b = __fmul_rn(__uint_as_float(sb2.x << 16), val(ce0[2], co0[2], k0));
        box_b = __fmaf_rn(__uint_as_float(sb2.x & 0xffff0000u), val(ce0[3], co0[3], k1), box_b);
        box_b = __fmaf_rn(__uint_as_float(sb2.y << 16), val(ce1[2], co1[2], k2), box_b);
        box_b = __fmaf_rn(__uint_as_float(sb2.y & 0xffff0000u), val(ce1[3], co1[3], k3), box_b);
        res_a = __fmaf_rn(xu_box, box_a, res_a);
        res_b = __fmaf_rn(xu_box, box_b, res_b);
      }
      __syncwarp();
      if (lane == 0) { mbar_arrive(bar_empty(s)); }  // this warp's part of the stage is in registers
      if (++s == stages) {
        s = 0;
        ph ^= 1u;
      }
    }
    if (!ok) { break; }
    // The four lanes of a quad (three digits + bias) are summed so that even lanes end with row
    // rho and odd lanes with row rho + 8; then the 8 warps' K slices: every warp posts its 16
    // partial sums and moves on; the warp that posts last adds them in warp order (so the result
    // does not depend on arrival order) and stores. The ring of kRedSlots tiles is deeper than a
    // warp can run ahead.
    res_a *= digit_weight;
    res_b *= digit_weight;
    float keep = (t & 1) ? res_b : res_a;
    keep += __shfl_xor_sync(0xffffffffu, (t & 1) ? res_a : res_b, 1);
    keep += __shfl_xor_sync(0xffffffffu, keep, 2);
    const int slot = tile_seq % kRedSlots;
    ++tile_seq;
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
        // a dead slot of the sorted form (padding row, or a tile without an expert) stores nothing
        const bool live = !P->vrow || (__ldg(P->vrow) >= 0 && (!P->eid || __ldg(P->eid) >= 0));
        if (live) { fused_store(P->epilogue, v, row, P->N, lane, P->y, P->aux, P->y3, P->q_rows, P->k_rows); }
      }
      __syncwarp();
      if (lane == 0) {
        red_cnt[slot] = 0;
        if (chain) {
          // Publish: the stores above, then the count. Tiles of a CTA finish in order, so the warp that
          // finishes the CTA's last tile of this GEMV reports all of them with one release-add.
          // (the finishers of a CTA are chained at block scope through a counter in shared memory, so the
          // one release below also covers the stores of the tiles that other warps finished)
          __threadfence_block();
          atomicAdd(sq_cnt + 3, 1u);
          if (tile == hi - 1) {
            const uint32_t mine = (uint32_t)(hi - lo);
            __threadfence_block();
            asm volatile("red.release.gpu.global.add.u32 [%0], %1;" ::"l"(sync), "r"(mine) : "memory");
          }
        }
      }
    }
  }
  if (!ok) { return kConsumeFailed; }
  return (uint32_t)s | (ph << 3) | (tile_seq << 4);
}

// kPool: the launch has a pool of chunks (a plan of independent GEMVs). Its own instantiation, and
// the pool's loop after the table's, so that the launches without a pool keep their code.
template <bool kPool>
__global__ void __launch_bounds__(kThreads, 2)
affine_qmv_w4g64_kernel(const __grid_constant__ QmvProblem single, const QmvProblem* __restrict__ list,
                        const int2* __restrict__ ranges, int total_tiles, int stages, int cap_kt, int count,
                        uint32_t* sync, uint32_t* dyn, const int4* __restrict__ chunks, int num_chunks) {
  extern __shared__ unsigned char smem_dyn[];
  const uint32_t raw = smem_u32(smem_dyn);
  const uint32_t base = (raw + 1023u) & ~1023u;  // swizzled boxes need 1024-byte alignment
  unsigned char* base_ptr = smem_dyn + (base - raw);
  constexpr int kStageBytes = kStageW + kStageSZ;
  const bool chain = sync != nullptr;
  unsigned char* p0 = base_ptr + (size_t)stages * kStageBytes;
  const Scratch sc(p0, cap_kt);
  const uint32_t bar0 = smem_u32(sc.bars);
  const int lane = threadIdx.x & 31;
  const int warp = threadIdx.x >> 5;

  // Let the next kernel in the stream start its own weight stream now.
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

  if (threadIdx.x == 0) {
    for (int s = 0; s < stages; ++s) {
      mbar_init(bar0 + 8u * s, 1);
      mbar_init(bar0 + 8u * (kMaxStages + s), kConsWarps);
    }
    *sc.abort_flag = 0;
    for (int i = 0; i < kRedSlots; ++i) { sc.red_cnt[i] = 0; }
    for (int i = 0; i < 8; ++i) { sc.sq_cnt[i] = 0; }
    sc.dq[kDynSlots * 4] = 0;
    fence_mbar_init();
  }
  if (threadIdx.x < 8) { sc.zero128[threadIdx.x] = make_uint4(0, 0, 0, 0); }
  if (threadIdx.x == 8) {  // what the lanes without a bias term read in place of a group sum of x
    sc.zero16[0] = sc.zero16[1] = sc.zero16[2] = sc.zero16[3] = -kAccSurplus;
  }
  __syncthreads();

  if (warp == kConsWarps) {
    if (lane == 0) {
      produce(&single, list, ranges, total_tiles, stages, count, chain, base, bar0, sc.abort_flag, sc.dq,
              kPool ? dyn : nullptr, chunks, num_chunks);
    }
    return;
  }

  // ---------------------------------------------------------------- consumers
  // x (and y) may be produced / consumed by the previous kernel: stage_x waits for it before it
  // touches x, and every range of a CTA starts with a staging or follows one.
  Walk wk(&single, list, ranges, total_tiles, count, chain);
  const uint16_t* staged_x = nullptr;
  int staged_K = -1, sq_gen = 0;
  uint32_t state = 0;
  int lo = 0, hi = 0;
  while (wk.next_range(lo, hi, chain)) {
    const QmvProblem* P = wk.P;
    const int K = P->K;
    const uint16_t* xr = P->x;
    const int need = chain ? P->wait_tiles : 0;
    // q|k|v or gate|up of a layer share one staging; a dependent or normalised x is always staged
    if (need > 0 || P->norm_w != nullptr || P->xrow != nullptr || xr != staged_x || K != staged_K) {
      if (!stage_x(P, p0, cap_kt, sq_gen, need, sync)) { break; }
      staged_x = P->norm_w ? nullptr : xr;
      staged_K = K;
      if (P->norm_w) { ++sq_gen; }
    }
    state = consume_tiles(P, lo, hi, state, base_ptr, stages, cap_kt, sync);
    if (state == kConsumeFailed) { break; }
  }
  if constexpr (kPool) {
    // The pool: chunks the producer claims once the table's run is used up. The loop body is the one
    // above, written out a second time: as one loop over both sources the launches without a pool
    // lost 1 - 2 % (the hot loop's register allocation moved).
    uint32_t dyn_n = 0;
    while (state != kConsumeFailed && !*sc.abort_flag && wk.receive_chunk(list, sc.dq, sc.abort_flag, dyn_n) &&
           wk.next_range(lo, hi, chain)) {
      const QmvProblem* P = wk.P;
      const int K = P->K;
      const uint16_t* xr = P->x;
      if (P->norm_w != nullptr || P->xrow != nullptr || xr != staged_x || K != staged_K) {
        if (!stage_x(P, p0, cap_kt, sq_gen, 0, sync)) { break; }
        staged_x = P->norm_w ? nullptr : xr;
        staged_K = K;
        if (P->norm_w) { ++sq_gen; }
      }
      state = consume_tiles(P, lo, hi, state, base_ptr, stages, cap_kt, sync);
      if (state == kConsumeFailed) { break; }
    }
  }
  if (chain || kPool) {
    // The CTA that leaves last puts both counters back to zero for the next run (every CTA has
    // passed all of its waits by then, also one that gave up, and every producer has made its last
    // claim, since its consumers leave only after the end mark it posts). No barrier: the warp of a
    // CTA that leaves last reports for the CTA.
    uint32_t* ctr = chain ? sync : dyn;
    __syncwarp();
    if (lane == 0) {
      __threadfence();
      if (atomicAdd(&sc.sq_cnt[2], 1u) == (uint32_t)(kConsWarps - 1)) {
        if (atomicAdd(ctr + 1, 1u) == gridDim.x - 1) {
          ctr[0] = 0;
          ctr[1] = 0;
          __threadfence();
        }
      }
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
  const size_t fixed = 1024 /*alignment slack*/ + 128 + (size_t)cap_kt * kXBytesPerKt + (size_t)2 * cap_kt * 4 + 16 +
                       (size_t)((cap_kt / 2 + 3) & ~3) * 4 + kRedSlots * kConsWarps * 16 * 4 + kRedSlots * 4 +
                       2 * kConsWarps * 4 + 32 + 2 * kMaxStages * 8 + 16 + (kDynSlots * 4 + 4) * 4;
  const size_t budget = 112 * 1024;  // two CTAs per SM
  int stages = fixed + 2 * stage_bytes <= budget ? (int)((budget - fixed) / stage_bytes) : 2;
  if (stages > kMaxStages) { stages = kMaxStages; }
  return {stages, fixed + (size_t)stages * stage_bytes};
}

int fill_problem(QmvProblem* p, const uint32_t* w, const uint16_t* scales, const uint16_t* biases,
                 const uint16_t* x, __nv_bfloat16* y, int K, int N, int tile_begin, int experts = 1) {
  std::memset(p, 0, sizeof(*p));
  const uint64_t rows = (uint64_t)N * (uint64_t)experts;  // expert slabs are stacked along the rows
  if (int rc = make_map_2d(&p->mw, CU_TENSOR_MAP_DATA_TYPE_UINT32, 4, w, (uint64_t)(K / 8), rows, 32,
                           16, CU_TENSOR_MAP_SWIZZLE_128B, "w")) {
    return rc;
  }
  // The scale / bias rows can be TMA boxes only if their pitch and base are multiples of 16 bytes.
  p->scales_tma = ((K % 512) == 0 && aligned16(scales) && aligned16(biases)) ? 1 : 0;
  if (p->scales_tma) {
    const int G = K / 64;
    if (int rc = make_map_2d(&p->ms, CU_TENSOR_MAP_DATA_TYPE_UINT16, 2, scales, (uint64_t)G, rows, 32,
                             16, CU_TENSOR_MAP_SWIZZLE_64B, "scales")) {
      return rc;
    }
    if (int rc = make_map_2d(&p->mz, CU_TENSOR_MAP_DATA_TYPE_UINT16, 2, biases, (uint64_t)G, rows, 32,
                             16, CU_TENSOR_MAP_SWIZZLE_64B, "biases")) {
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
  p->experts = experts;
  return VPQ_OK;
}

constexpr int kMaxGrid = 1023;  // CTAs a range table has room for

// CTAs of a launch: two per SM, or one per row tile if there are fewer. With the extra tiles on the
// lowest CTAs an SM's two CTAs differ by at most one tile from any other SM's (384 tiles: 3 or 2 per
// SM; as 192 CTAs x 2 some SMs would hold 4 and others 2). Measured on a chain of dependent decode
// launches: 8.55 us per launch against 8.82 with equal tiles per CTA.
int grid_for(int total_tiles) {
  int cap = 2 * num_sms();
  if (cap > kMaxGrid) { cap = kMaxGrid; }
  return total_tiles <= cap ? total_tiles : cap;
}

// Splits the concatenated row tiles of `count` problems into `grid` contiguous runs of about equal
// cost (a tile costs its stages -- the kernel is bound by the bytes it streams -- plus a small
// fixed share for the reduction and the store).
// out[b] = {first tile of CTA b, index of the problem it belongs to}, out[grid] closes the list.
int64_t tile_cost(const QmvProblem& q) {
  const int nb = (q.K + 255) >> 8;
  return (int64_t)(16 * ((nb + kBoxesPerStage - 1) / kBoxesPerStage) + 3);  // measured: the fixed share is ~0.2 stage
}

void build_ranges(const QmvProblem* p, size_t count, int grid, int2* out) {
  int64_t total = 0;
  for (size_t r = 0; r < count; ++r) { total += tile_cost(p[r]) * p[r].row_tiles; }
  size_t r = 0;
  int64_t before = 0;  // cost of the problems before r
  for (int b = 0; b < grid; ++b) {
    const int64_t target = total * b / grid;
    while (r + 1 < count && before + tile_cost(p[r]) * p[r].row_tiles <= target) {
      before += tile_cost(p[r]) * p[r].row_tiles;
      ++r;
    }
    int t = (int)((target - before) / tile_cost(p[r]));
    if (t > p[r].row_tiles) { t = p[r].row_tiles; }
    out[b] = make_int2(p[r].tile_begin + t, (int)r);
  }
  const QmvProblem& last = p[count - 1];
  out[grid] = make_int2(last.tile_begin + last.row_tiles, (int)(count - 1));
}

int g_granted[64] = {};  // dynamic shared memory already granted to the kernel, per device
int g_granted_pool[64] = {};

// `sync` not null: the list is a dependent chain (two counters in device memory, zero between
// runs); the launch is cooperative because its CTAs wait on one another.
int launch_list(const QmvProblem& single, const QmvProblem* list, const int2* ranges, int total_tiles, int cap_kt,
                cudaStream_t st, int count = 1, uint32_t* sync = nullptr, int chain_grid = 0, uint32_t* dyn = nullptr,
                const int4* chunks = nullptr, int num_chunks = 0) {
  const LaunchShape ls = shape_for(cap_kt);
  auto kern = dyn ? affine_qmv_w4g64_kernel<true> : affine_qmv_w4g64_kernel<false>;
  if (int rc = ensure_dynamic_smem(reinterpret_cast<const void*>(kern), dyn ? g_granted_pool : g_granted, ls.smem)) {
    return rc;
  }
  const int ctas = sync ? chain_grid : grid_for(total_tiles);
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)ctas, 1, 1);
  cfg.blockDim = dim3(kThreads, 1, 1);
  cfg.dynamicSmemBytes = ls.smem;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  if (sync) {
    attr[0].id = cudaLaunchAttributeCooperative;
    attr[0].val.cooperative = 1;
  } else {
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
  }
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  VPQ_CUDA_OK(cudaLaunchKernelEx(&cfg, kern, single, list, ranges, total_tiles, ls.stages, cap_kt, count, sync, dyn,
                                 chunks, num_chunks));
  return VPQ_OK;
}

// CTAs of a dependent chain: all must be resident at once, so at most what the occupancy
// calculator grants for this kernel's shared memory, and no more than the largest GEMV has tiles.
int chain_grid_for(int cap_kt, int max_row_tiles, int* out) {
  const LaunchShape ls = shape_for(cap_kt);
  auto kern = affine_qmv_w4g64_kernel<false>;
  if (int rc = ensure_dynamic_smem(reinterpret_cast<const void*>(kern), g_granted, ls.smem)) { return rc; }
  int per_sm = 0;
  VPQ_CUDA_OK(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kern, kThreads, ls.smem));
  if (per_sm < 1) { return fail(VPQ_ERR_CUDA, "qmv chain: the kernel does not fit an SM"); }
  if (per_sm > 2) { per_sm = 2; }
  int grid = per_sm * num_sms();
  if (grid > max_row_tiles) { grid = max_row_tiles; }
  *out = grid;
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

// Validation of one descriptor: shapes, fused store, RMSNorm prologue, expert gather.
int check_row_map(const char* who, const vpq_linear_desc& d);

int check_desc(const char* who, const vpq_linear_desc& d, bool in_plan) {
  if (int rc = check_qmv_args(who, d.w, d.scales, d.biases, d.x, d.y, d.K, d.N, d.M)) { return rc; }
  if (d.depends != 0 && d.depends != 1) { return fail(VPQ_ERR_INVALID_ARG, "%s: depends must be 0 or 1", who); }
  if (d.depends && !in_plan) {
    return fail(VPQ_ERR_UNSUPPORTED, "%s: depends is honoured by vpq_qmv_plan_create only", who);
  }
  if (d.norm_w) {
    if (!aligned16(d.norm_w)) { return fail(VPQ_ERR_ALIGNMENT, "%s: norm_w must be 16-byte aligned", who); }
    if (!(d.eps >= 0.0f)) { return fail(VPQ_ERR_INVALID_ARG, "%s: eps must be >= 0", who); }
  }
  if (d.expert) {
    if (d.experts <= 0 || d.experts * d.N > (1ll << 30)) {
      return fail(VPQ_ERR_INVALID_ARG, "%s: an expert gather needs 0 < experts, experts * N <= 2^30", who);
    }
    if (reinterpret_cast<uintptr_t>(d.expert) & 3) {
      return fail(VPQ_ERR_ALIGNMENT, "%s: the expert index array must be 4-byte aligned", who);
    }
    if (d.x_div < 0) { return fail(VPQ_ERR_INVALID_ARG, "%s: x_div must be >= 0", who); }
  } else if (d.experts > 1 || d.x_div > 1) {
    return fail(VPQ_ERR_INVALID_ARG, "%s: experts / x_div given without an expert index array", who);
  }
  if (int rc = check_row_map(who, d)) { return rc; }
  return qmv_check_store(who, d);
}
}  // namespace

// The kernels other than the 4-bit group-64 GEMV take plain descriptors only.
int qmv_check_plain(const char* who, const vpq_linear_desc& d, bool allow_norm) {
  if ((d.norm_w && !allow_norm) || d.expert || d.depends || d.experts > 1 || d.x_div > 1 || d.row_map || d.row_gather ||
      d.expert_div > 1) {
    return fail(VPQ_ERR_UNSUPPORTED, "%s: %sexpert and depends are taken by the w4 g64 GEMV entry points only", who,
                allow_norm ? "" : "norm_w, ");
  }
  if (d.norm_w) {
    if (!aligned16(d.norm_w)) { return fail(VPQ_ERR_ALIGNMENT, "%s: norm_w must be 16-byte aligned", who); }
    if (!(d.eps >= 0.0f)) { return fail(VPQ_ERR_INVALID_ARG, "%s: eps must be >= 0", who); }
  }
  return qmv_check_store(who, d);
}

namespace {
int check_row_map(const char* who, const vpq_linear_desc& d) {
  if (d.row_map) {
    if (reinterpret_cast<uintptr_t>(d.row_map) & 3) {
      return fail(VPQ_ERR_ALIGNMENT, "%s: row_map must be 4-byte aligned", who);
    }
    if (d.row_gather != 0 && d.row_gather != 1) { return fail(VPQ_ERR_INVALID_ARG, "%s: row_gather must be 0 or 1", who); }
  } else if (d.row_gather != 0) {
    return fail(VPQ_ERR_INVALID_ARG, "%s: row_gather given without row_map", who);
  }
  if (d.expert_div < 0 || (d.expert_div > 1 && !d.expert)) {
    return fail(VPQ_ERR_INVALID_ARG, "%s: expert_div must be >= 0 and needs an expert index array", who);
  }
  return VPQ_OK;
}
}  // namespace

int qmv_check_gather(const char* who, const vpq_linear_desc& d, bool allow_norm) {
  if (int rc = check_row_map(who, d)) { return rc; }
  if ((d.norm_w && !allow_norm) || d.depends) {
    return fail(VPQ_ERR_UNSUPPORTED, "%s: %s taken by the w4 g64 GEMV entry points only", who,
                allow_norm ? "depends is" : "norm_w and depends are");
  }
  if (d.norm_w) {
    if (!aligned16(d.norm_w)) { return fail(VPQ_ERR_ALIGNMENT, "%s: norm_w must be 16-byte aligned", who); }
    if (!(d.eps >= 0.0f)) { return fail(VPQ_ERR_INVALID_ARG, "%s: eps must be >= 0", who); }
  }
  if (d.expert) {
    if (d.experts <= 0 || d.experts * d.N > (1ll << 30)) {
      return fail(VPQ_ERR_INVALID_ARG, "%s: an expert gather needs 0 < experts, experts * N <= 2^30", who);
    }
    if (reinterpret_cast<uintptr_t>(d.expert) & 3) {
      return fail(VPQ_ERR_ALIGNMENT, "%s: the expert index array must be 4-byte aligned", who);
    }
    if (d.x_div < 0) { return fail(VPQ_ERR_INVALID_ARG, "%s: x_div must be >= 0", who); }
  } else if (d.experts > 1 || d.x_div > 1) {
    return fail(VPQ_ERR_INVALID_ARG, "%s: experts / x_div given without an expert index array", who);
  }
  return qmv_check_store(who, d);
}

int qmv_check_store(const char* who, const vpq_linear_desc& d) {
  switch (d.epilogue) {
    case VPQ_EPILOGUE_NONE:
      return VPQ_OK;
    case VPQ_EPILOGUE_ADD:
      if (!d.aux || (reinterpret_cast<uintptr_t>(d.aux) & 1)) {
        return fail(VPQ_ERR_INVALID_ARG, "%s: the residual is null or not 2-byte aligned", who);
      }
      return VPQ_OK;
    case VPQ_EPILOGUE_GELU_MUL:
    case VPQ_EPILOGUE_SILU_MUL:
      if (!d.aux || (reinterpret_cast<uintptr_t>(d.aux) & 1)) {
        return fail(VPQ_ERR_INVALID_ARG, "%s: the multiplier is null or not 2-byte aligned", who);
      }
      return VPQ_OK;
    case VPQ_EPILOGUE_SWIGLU:
    case VPQ_EPILOGUE_GEGLU:
      if (d.N % 2) { return fail(VPQ_ERR_INVALID_ARG, "%s: a gated store needs an even N (gate / up interleaved)", who); }
      return VPQ_OK;
    case VPQ_EPILOGUE_QKV:
      if (d.q_rows < 0 || d.k_rows < 0 || d.q_rows + d.k_rows > d.N) {
        return fail(VPQ_ERR_INVALID_ARG, "%s: q_rows %lld + k_rows %lld exceed N %lld", who, (long long)d.q_rows,
                    (long long)d.k_rows, (long long)d.N);
      }
      if ((d.k_rows > 0 && !d.aux) || (d.q_rows + d.k_rows < d.N && !d.y3) ||
          (reinterpret_cast<uintptr_t>(d.aux) & 1) || (reinterpret_cast<uintptr_t>(d.y3) & 1)) {
        return fail(VPQ_ERR_INVALID_ARG, "%s: k / v output null or not 2-byte aligned", who);
      }
      return VPQ_OK;
    default:
      return fail(VPQ_ERR_INVALID_ARG, "%s: unknown epilogue %d", who, (int)d.epilogue);
  }
}

namespace {

// Row m of a descriptor as a kernel problem.
int fill_from_desc(QmvProblem* p, const vpq_linear_desc& d, int64_t m, int tile_begin) {
  const bool gated = d.epilogue == VPQ_EPILOGUE_SWIGLU || d.epilogue == VPQ_EPILOGUE_GEGLU;
  const int64_t y_pitch = gated ? d.N / 2
                          : d.epilogue == VPQ_EPILOGUE_QKV  ? d.q_rows
                                                            : d.N;
  const bool row_gather = d.row_map && d.row_gather;   // the x row is read on the GPU (row_map[m])
  const int64_t x_row = row_gather ? 0 : (d.expert && d.x_div > 1) ? m / d.x_div : m;  // pairs of one token share its row
  if (int rc = fill_problem(p, d.w, static_cast<const uint16_t*>(d.scales), static_cast<const uint16_t*>(d.biases),
                            static_cast<const uint16_t*>(d.x) + x_row * d.K,
                            static_cast<__nv_bfloat16*>(d.y) + m * y_pitch, (int)d.K, (int)d.N, tile_begin,
                            d.expert ? (int)d.experts : 1)) {
    return rc;
  }
  p->epilogue = d.epilogue;
  if (d.epilogue == VPQ_EPILOGUE_ADD || d.epilogue == VPQ_EPILOGUE_GELU_MUL || d.epilogue == VPQ_EPILOGUE_SILU_MUL) {
    p->aux = static_cast<const uint16_t*>(d.aux) + m * d.N;
  } else if (d.epilogue == VPQ_EPILOGUE_QKV) {
    p->q_rows = (int)d.q_rows;
    p->k_rows = (int)d.k_rows;
    p->aux = static_cast<const uint16_t*>(d.aux) + m * d.k_rows;
    p->y3 = static_cast<__nv_bfloat16*>(d.y3) + m * (d.N - d.q_rows - d.k_rows);
  }
  p->norm_w = static_cast<const uint16_t*>(d.norm_w);
  p->eps = d.eps;
  p->eid = d.expert ? d.expert + (d.expert_div > 1 ? m / d.expert_div : m) : nullptr;
  p->vrow = d.row_map ? d.row_map + m : nullptr;
  p->xrow = row_gather ? d.row_map + m : nullptr;
  return VPQ_OK;
}

// One launch per row of one descriptor (every row streams the weight again, as in the reference).
int launch_desc_rows(const char* who, const vpq_linear_desc& d, cudaStream_t st) {
  if (int rc = check_desc(who, d, false)) { return rc; }
  if (int rc = require_sm100()) { return rc; }
  const int cap_kt = (int)((d.K + 255) / 256) * 2;
  for (int64_t m = 0; m < d.M; ++m) {
    QmvProblem p;
    if (int rc = fill_from_desc(&p, d, m, 0)) { return rc; }
    if (int rc = launch_list(p, nullptr, nullptr, p.row_tiles, cap_kt, st)) { return rc; }
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
  const int2* ranges_dev;
  uint32_t* sync_dev;  // dependent chain: {finished tiles, CTAs that left}; null for independent GEMVs
  uint32_t* dyn_dev;   // pool of chunks: {chunks claimed, CTAs that left}; null without a pool
  const int4* chunks_dev;  // the pool: {first tile, problem, tiles, 0} per chunk
  int num_chunks;
  int count;           // problems (one per GEMV row)
  int total_tiles;
  int cap_kt;
  int chain_grid;
};

namespace {
vpq_linear_desc make_desc(const uint32_t* w, const void* scales, const void* biases, const void* x, void* y,
                          int64_t K, int64_t N, int64_t M) {
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
}  // namespace

extern "C" int vpq_affine_qmv_w4g64_bf16(const uint32_t* w, const void* scales, const void* biases,
                                         const void* x, void* y, int64_t K, int64_t N, int64_t M,
                                         void* stream) {
  clear_error();
  return launch_desc_rows("affine_qmv_w4g64", make_desc(w, scales, biases, x, y, K, N, M),
                          static_cast<cudaStream_t>(stream));
}

extern "C" int vpq_affine_qmv_w4g64_bf16_add(const uint32_t* w, const void* scales, const void* biases,
                                             const void* x, void* y, int64_t K, int64_t N, int64_t M,
                                             const void* residual, void* stream) {
  clear_error();
  vpq_linear_desc d = make_desc(w, scales, biases, x, y, K, N, M);
  d.epilogue = VPQ_EPILOGUE_ADD;
  d.aux = residual;
  return launch_desc_rows("affine_qmv_w4g64_add", d, static_cast<cudaStream_t>(stream));
}

extern "C" int vpq_affine_qmv_swiglu_w4g64_bf16(const uint32_t* w, const void* scales, const void* biases,
                                                const void* x, void* y, int64_t K, int64_t N, int64_t M,
                                                void* stream) {
  clear_error();
  vpq_linear_desc d = make_desc(w, scales, biases, x, y, K, N, M);
  d.epilogue = VPQ_EPILOGUE_SWIGLU;
  return launch_desc_rows("affine_qmv_swiglu_w4g64", d, static_cast<cudaStream_t>(stream));
}

extern "C" int vpq_affine_qmv_geglu_w4g64_bf16(const uint32_t* w, const void* scales, const void* biases,
                                               const void* x, void* y, int64_t K, int64_t N, int64_t M,
                                               void* stream) {
  clear_error();
  vpq_linear_desc d = make_desc(w, scales, biases, x, y, K, N, M);
  d.epilogue = VPQ_EPILOGUE_GEGLU;
  return launch_desc_rows("affine_qmv_geglu_w4g64", d, static_cast<cudaStream_t>(stream));
}

extern "C" int vpq_affine_qmv_gelu_mul_w4g64_bf16(const uint32_t* w, const void* scales, const void* biases,
                                                  const void* x, void* y, int64_t K, int64_t N, int64_t M,
                                                  const void* mul, void* stream) {
  clear_error();
  vpq_linear_desc d = make_desc(w, scales, biases, x, y, K, N, M);
  d.epilogue = VPQ_EPILOGUE_GELU_MUL;
  d.aux = mul;
  return launch_desc_rows("affine_qmv_gelu_mul_w4g64", d, static_cast<cudaStream_t>(stream));
}

extern "C" int vpq_affine_qmv_qkv_w4g64_bf16(const uint32_t* w, const void* scales, const void* biases,
                                             const void* x, void* q_out, void* k_out, void* v_out, int64_t K,
                                             int64_t q_rows, int64_t k_rows, int64_t v_rows, int64_t M,
                                             void* stream) {
  clear_error();
  if (q_rows <= 0 || k_rows < 0 || v_rows < 0) {
    return fail(VPQ_ERR_INVALID_ARG, "affine_qmv_qkv_w4g64: need q_rows > 0, k_rows >= 0, v_rows >= 0");
  }
  vpq_linear_desc d = make_desc(w, scales, biases, x, q_out, K, q_rows + k_rows + v_rows, M);
  d.epilogue = VPQ_EPILOGUE_QKV;
  d.aux = k_out;
  d.y3 = v_out;
  d.q_rows = q_rows;
  d.k_rows = k_rows;
  return launch_desc_rows("affine_qmv_qkv_w4g64", d, static_cast<cudaStream_t>(stream));
}

extern "C" int vpq_affine_qmv_w4g64_bf16_batch(const vpq_linear_desc* d, int count, void* stream) {
  clear_error();
  if (!d || count <= 0) { return fail(VPQ_ERR_INVALID_ARG, "affine_qmv_w4g64_batch: null or empty set"); }
  for (int i = 0; i < count; ++i) {
    if (int rc = launch_desc_rows("affine_qmv_w4g64_batch", d[i], static_cast<cudaStream_t>(stream))) { return rc; }
  }
  return VPQ_OK;
}

namespace {
// The pool of a plan of independent GEMVs: the share of the launch's cost that is handed out in
// chunks at run time, the cost of one chunk in units of tile_cost (about eight 4096-k tiles: long
// enough to pay for a staging of x, short next to the spread of the CTAs' finishing times, which it
// bounds), and the least work per CTA for a pool to be worth having.
constexpr int kPoolPercent = 10;
constexpr int64_t kChunkCost = 8 * 35;
constexpr int kPoolMinTilesPerCta = 32;

size_t pool_chunks_bound(size_t tiles, size_t rows) { return tiles * (kPoolPercent + 2) / 100 + rows + 8; }
}  // namespace

extern "C" size_t vpq_qmv_plan_bytes(const vpq_linear_desc* d, int count) {
  if (!d || count <= 0) { return 0; }
  size_t rows = 0, tiles = 0;
  for (int i = 0; i < count; ++i) {
    if (d[i].M > 0 && d[i].N > 0) {
      rows += (size_t)d[i].M;
      tiles += (size_t)d[i].M * (size_t)((d[i].N + 15) / 16);
    }
  }
  return rows * sizeof(QmvProblem) + 64 + (kMaxGrid + 1) * sizeof(int2) + 64 /* the chain's counters */ +
         128 /* the pool's counters, alignment */ + pool_chunks_bound(tiles, rows) * sizeof(int4);
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
  bool chain = false;
  for (int i = 0; i < count; ++i) {
    if (int rc = check_desc("qmv_plan_create", d[i], true)) { return rc; }
    chain = chain || d[i].depends != 0;
  }
  if (int rc = require_sm100()) { return rc; }
  size_t rows = 0;
  for (int i = 0; i < count; ++i) { rows += (size_t)d[i].M; }
  QmvProblem* host = static_cast<QmvProblem*>(std::aligned_alloc(64, rows * sizeof(QmvProblem)));
  if (!host) { return fail(VPQ_ERR_INVALID_ARG, "qmv_plan_create: out of host memory"); }
  int tiles = 0, cap_kt = 0, max_rt = 1;
  size_t r = 0;
  for (int i = 0; i < count; ++i) {
    const int first_tile = tiles;  // a dependent descriptor waits for everything before it in the list
    for (int64_t m = 0; m < d[i].M; ++m, ++r) {
      const int rc = fill_from_desc(&host[r], d[i], m, tiles);
      if (rc) {
        std::free(host);
        return rc;
      }
      host[r].wait_tiles = d[i].depends ? first_tile : 0;
      tiles += host[r].row_tiles;
      max_rt = host[r].row_tiles > max_rt ? host[r].row_tiles : max_rt;
      const int kt = (int)((d[i].K + 255) / 256) * 2;
      cap_kt = kt > cap_kt ? kt : cap_kt;
    }
  }
  const uintptr_t dev = (reinterpret_cast<uintptr_t>(workspace) + 63) & ~(uintptr_t)63;
  const uintptr_t dev_ranges = dev + rows * sizeof(QmvProblem);
  const uintptr_t dev_sync = (dev_ranges + (kMaxGrid + 1) * sizeof(int2) + 15) & ~(uintptr_t)15;
  int chain_grid = 0;
  if (chain) {
    if (int rc = chain_grid_for(cap_kt, max_rt, &chain_grid)) {
      std::free(host);
      return rc;
    }
  }
  const int grid = grid_for(tiles);
  int2 host_ranges[kMaxGrid + 1];
  const uintptr_t dev_dyn = dev_sync + 64;
  const uintptr_t dev_chunks = dev_dyn + 64;
  std::vector<int4> pool;
  if (!chain && tiles >= kPoolMinTilesPerCta * grid) {
    // The tail of the list, worth kPoolPercent of the launch's cost, leaves the CTAs' table and
    // becomes the pool: chunks of about kChunkCost, none across two GEMVs, in list order.
    int64_t total = 0;
    for (size_t q = 0; q < rows; ++q) { total += tile_cost(host[q]) * host[q].row_tiles; }
    int64_t want = total * kPoolPercent / 100;
    size_t split = rows;      // first problem with tiles in the pool
    int split_tiles = 0;      // tiles of it that stay in the table
    while (split > 0 && want > 0) {
      --split;
      const int64_t c = tile_cost(host[split]);
      const int64_t take = want / c < host[split].row_tiles ? want / c : host[split].row_tiles;
      split_tiles = host[split].row_tiles - (int)take;
      want -= take * c;
      if (take < host[split].row_tiles) { break; }
    }
    for (size_t q = split; q < rows; ++q) {
      const int per = (int)(kChunkCost / tile_cost(host[q]) > 0 ? kChunkCost / tile_cost(host[q]) : 1);
      for (int t = q == split ? split_tiles : 0; t < host[q].row_tiles; t += per) {
        const int n = host[q].row_tiles - t < per ? host[q].row_tiles - t : per;
        pool.push_back(make_int4(host[q].tile_begin + t, (int)q, n, 0));
      }
    }
    if (pool.empty() || pool.size() > pool_chunks_bound((size_t)tiles, rows) || (split == 0 && split_tiles == 0)) {
      pool.clear();
    } else {
      // the table over what stays: the list up to the split, the split problem cut short
      const int kept = host[split].row_tiles;
      host[split].row_tiles = split_tiles;
      build_ranges(host, split_tiles > 0 ? split + 1 : split, grid, host_ranges);
      host[split].row_tiles = kept;
    }
  }
  if (pool.empty()) { build_ranges(host, rows, grid, host_ranges); }
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  cudaError_t e = cudaMemcpyAsync(reinterpret_cast<void*>(dev), host, rows * sizeof(QmvProblem),
                                  cudaMemcpyHostToDevice, st);
  if (e == cudaSuccess) {
    e = cudaMemcpyAsync(reinterpret_cast<void*>(dev_ranges), host_ranges, (size_t)(grid + 1) * sizeof(int2),
                        cudaMemcpyHostToDevice, st);
  }
  if (e == cudaSuccess && !pool.empty()) {
    e = cudaMemcpyAsync(reinterpret_cast<void*>(dev_chunks), pool.data(), pool.size() * sizeof(int4),
                        cudaMemcpyHostToDevice, st);
  }
  if (e == cudaSuccess) { e = cudaMemsetAsync(reinterpret_cast<void*>(dev_sync), 0, 128, st); }
  if (e == cudaSuccess) { e = cudaStreamSynchronize(st); }
  std::free(host);
  if (e != cudaSuccess) { return fail(VPQ_ERR_CUDA, "qmv_plan_create: copy failed: %s", cudaGetErrorString(e)); }
  vpq_qmv_plan* plan = new vpq_qmv_plan_s();
  plan->list_dev = reinterpret_cast<const QmvProblem*>(dev);
  plan->ranges_dev = reinterpret_cast<const int2*>(dev_ranges);
  plan->sync_dev = chain ? reinterpret_cast<uint32_t*>(dev_sync) : nullptr;
  plan->dyn_dev = pool.empty() ? nullptr : reinterpret_cast<uint32_t*>(dev_dyn);
  plan->chunks_dev = pool.empty() ? nullptr : reinterpret_cast<const int4*>(dev_chunks);
  plan->num_chunks = (int)pool.size();
  plan->count = (int)rows;
  plan->total_tiles = tiles;
  plan->cap_kt = cap_kt;
  plan->chain_grid = chain_grid;
  *out = plan;
  return VPQ_OK;
}

extern "C" int vpq_qmv_plan_run(const vpq_qmv_plan* plan, void* stream) {
  clear_error();
  if (!plan) { return fail(VPQ_ERR_INVALID_ARG, "qmv_plan_run: null plan"); }
  if (int rc = require_sm100()) { return rc; }
  QmvProblem unused;
  std::memset(&unused, 0, sizeof(unused));
  if (plan->sync_dev) {
    return launch_list(unused, plan->list_dev, nullptr, plan->total_tiles, plan->cap_kt,
                       static_cast<cudaStream_t>(stream), plan->count, plan->sync_dev, plan->chain_grid);
  }
  return launch_list(unused, plan->list_dev, plan->ranges_dev, plan->total_tiles, plan->cap_kt,
                     static_cast<cudaStream_t>(stream), plan->count, nullptr, 0, plan->dyn_dev, plan->chunks_dev,
                     plan->num_chunks);
}

// ---------------------------------------------------------------- no-allocation variant
// The plan kernel needs its list of problem descriptors in device memory. This variant keeps that
// list in a fixed array that is part of the library image, so the call neither allocates nor needs
// a caller workspace. Every GPU that loads the library carries the array (40 KB) until exit.
constexpr int kNoAllocMaxRows = 64;  // GEMV rows (sum of M over the set) one call can take
static __device__ __align__(256) unsigned char
    g_noalloc_descs[kNoAllocMaxRows * sizeof(QmvProblem) + (kMaxGrid + 1) * sizeof(int2)];  // records, then the CTA ranges

extern "C" int vpq_affine_qmv_w4g64_bf16_set_noalloc(const vpq_linear_desc* d, int count, void* stream) {
  clear_error();
  if (!d || count <= 0) { return fail(VPQ_ERR_INVALID_ARG, "qmv_set_noalloc: null or empty set"); }
  int64_t rows = 0;
  for (int i = 0; i < count; ++i) {
    if (int rc = check_desc("qmv_set_noalloc", d[i], false)) { return rc; }
    rows += d[i].M;
  }
  if (rows > kNoAllocMaxRows) {
    return fail(VPQ_ERR_UNSUPPORTED,
                "qmv_set_noalloc: %lld GEMV rows in the set, the built-in descriptor array holds %d; "
                "split the set or use vpq_qmv_plan_create with a workspace",
                (long long)rows, kNoAllocMaxRows);
  }
  if (int rc = require_sm100()) { return rc; }
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  // The descriptors travel from this call's stack by stream-ordered copies: a captured copy node
  // would keep pointers into a dead stack frame and replay them, so the call refuses to be captured.
  cudaStreamCaptureStatus capturing = cudaStreamCaptureStatusNone;
  VPQ_CUDA_OK(cudaStreamIsCapturing(st, &capturing));
  if (capturing != cudaStreamCaptureStatusNone) {
    return fail(VPQ_ERR_UNSUPPORTED, "qmv_set_noalloc: the stream is being captured; this entry point cannot be "
                                     "recorded into a CUDA graph (use vpq_qmv_plan_create / vpq_qmv_plan_run)");
  }
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
      if (int rc = fill_from_desc(&host[r], d[i], m, tiles)) { return rc; }
      tiles += host[r].row_tiles;
      const int kt = (int)((d[i].K + 255) / 256) * 2;
      cap_kt = kt > cap_kt ? kt : cap_kt;
    }
  }
  // every descriptor the kernel will read is rewritten here, so nothing stale from the previous
  // call is ever used; the copy is ordered before the launch on the same stream
  VPQ_CUDA_OK(cudaMemcpyAsync(dev_addr[dev], host, (size_t)r * sizeof(QmvProblem), cudaMemcpyHostToDevice, st));
  const int grid = grid_for(tiles);
  int2 host_ranges[kMaxGrid + 1];
  build_ranges(host, (size_t)r, grid, host_ranges);
  void* dev_ranges = static_cast<unsigned char*>(dev_addr[dev]) + kNoAllocMaxRows * sizeof(QmvProblem);
  VPQ_CUDA_OK(cudaMemcpyAsync(dev_ranges, host_ranges, (size_t)(grid + 1) * sizeof(int2), cudaMemcpyHostToDevice, st));
  QmvProblem unused;
  std::memset(&unused, 0, sizeof(unused));
  return launch_list(unused, static_cast<const QmvProblem*>(dev_addr[dev]), static_cast<const int2*>(dev_ranges), tiles,
                     cap_kt, st, r);
}

extern "C" int vpq_qmv_plan_destroy(vpq_qmv_plan* plan) {
  delete plan;
  return VPQ_OK;
}
