// qmm_ta.cuh -- the QMM with the dequantised weight tile as the TENSOR-MEMORY operand.
// Included by qmm.cu (uses its helpers and those of qmm_2cta.cuh).
//
// The CTA-pair kernel of qmm_2cta.cuh is bound by shared-memory bandwidth: per 64-wide k block
// every CTA writes its dequantised 128 x 64 W tile to shared memory (16 KB), and the tensor cores
// of both SMs read it back (32 KB), next to the x operand and the TMA writes. Here the product is
// computed transposed, y^T = W x^T: the dequantised W tile is the A operand of tcgen05.mma and A
// may live in tensor memory. The dequantiser threads own one W row each, which is exactly one
// tensor-memory lane, so they store their 64 bf16 straight into it with tcgen05.st: no shared-memory
// store, no operand read, no fence.proxy.async. What remains in shared memory per k block and CTA is
// the x tile (12 KB written by TMA, 24 KB read by the two tensor cores) and the packed codes
// (4 KB + 4 KB): 44 KB against 88 KB before.
//
// Tile of a CTA pair: 256 W rows (output columns n; 128 per CTA = its tensor-memory lanes) x 192
// rows of x (output rows m; 96 per CTA as the B operand, K-major, 128-byte swizzle). Tensor memory
// (512 columns): two accumulators of 192 columns (the epilogue of tile i overlaps the main loop of
// tile i + 1) + a ring of four 32-column A tiles. The accumulator holds y^T: lane = n, column = m;
// the epilogue stores one bf16 per lane, 32 consecutive n = 64 contiguous bytes per instruction.
//
// Roles per CTA, 448 threads: warps 0-3 epilogue, warp 4 TMA producer, warp 5 tensor-memory
// allocation (+ MMA issue in the leader CTA), warps 6-13 dequantisers in two groups that take
// alternate k blocks; a dequantiser thread's W row is its tensor-memory lane (warp % 4 selects the
// 32-lane quarter a warp may access). Barriers as in qmm_2cta.cuh; every wait is bounded.
#pragma once

namespace ta {

constexpr int TW = 256;         // W rows (output columns) per tile, 128 per CTA
constexpr int TX = 192;         // x rows (output rows) per tile, 96 per CTA
constexpr int kXStages = 6;     // x + codes ring
constexpr int kATiles = 4;      // dequantised-A ring in tensor memory
constexpr int kDqWarps = 8;
constexpr int kDqGroups = 2;
constexpr int kDqGroupWarps = kDqWarps / kDqGroups;
constexpr int kThreadsTa = 32 * (kEpiWarps + 2 + kDqWarps);
constexpr uint32_t kAccCols = TX;                  // columns of one accumulator
constexpr uint32_t kAColBase = 2 * kAccCols;       // first column of the A ring (384)
constexpr uint32_t kAColsPerTile = BK / 2;         // 64 bf16 = 32 columns
static_assert(kAColBase + kATiles * kAColsPerTile <= 512, "tensor memory columns");

struct SmemTa {
  static constexpr int kXBytes = (TX / 2) * BK * 2;     // 96 rows x 128 B = 12 KB, 128B-swizzled
  static constexpr int kCodeBytes = 128 * (BK / 2);     // 128 rows x 32 B
  static constexpr int kOffX = 0;
  static constexpr int kOffCode = kOffX + kXStages * kXBytes;
  static constexpr int kOffBar = kOffCode + kXStages * kCodeBytes;
  static constexpr int kNumBars = 3 * kXStages + 2 * kATiles + 4;
  static constexpr int kOffTmem = kOffBar + kNumBars * 8;
  static constexpr int kTotal = kOffTmem + 16;
  static constexpr int kAlloc = kTotal + 1024;
};

// D[tmem] (+)= A[tmem] * B[smem]: A is the dequantised W tile in tensor memory.
__device__ __forceinline__ void umma_bf16_pair_ta(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc,
                                                  uint32_t accumulate) {
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], [%1], %2, %3, p;\n\t"
      "}"
      ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}

// 32 consecutive 32-bit columns of this thread's tensor-memory lane.
__device__ __forceinline__ void tmem_st32(uint32_t taddr, const uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,"
      "%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};"
      ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]),
        "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]),
        "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]),
        "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
      : "memory");
}
__device__ __forceinline__ void tmem_st_wait() {
  asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}

// Instruction descriptor: D f32, A/B bf16, K-major, M = 256 (pair), N = TX.
__device__ __forceinline__ constexpr uint32_t make_idesc_ta() {
  return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(TX >> 3) << 17) | ((uint32_t)(TW >> 4) << 24);
}

__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kThreadsTa, 1)
affine_qmm_w4g64_ta_kernel(const __grid_constant__ CUtensorMap tmap_x, const __grid_constant__ CUtensorMap tmap_w,
                           const uint16_t* __restrict__ scales, const uint16_t* __restrict__ biases,
                           __nv_bfloat16* __restrict__ y, int64_t ld, int M, int N, int K) {
  using L = SmemTa;
  constexpr uint32_t kTmemCols = 512;

  extern __shared__ unsigned char smem_dyn[];
  const uint32_t raw = smem_u32(smem_dyn);
  const uint32_t base = (raw + 1023u) & ~1023u;
  unsigned char* base_ptr = smem_dyn + (base - raw);

  const uint32_t bar0 = base + L::kOffBar;
  auto bar_xfull = [&](int s) { return bar0 + 8u * s; };
  auto bar_cfull = [&](int s) { return bar0 + 8u * (kXStages + s); };
  auto bar_empty = [&](int s) { return bar0 + 8u * (2 * kXStages + s); };
  auto bar_afull = [&](int t) { return bar0 + 8u * (3 * kXStages + t); };
  auto bar_aempty = [&](int t) { return bar0 + 8u * (3 * kXStages + kATiles + t); };
  auto bar_accfull = [&](int a) { return bar0 + 8u * (3 * kXStages + 2 * kATiles + a); };
  auto bar_accempty = [&](int a) { return bar0 + 8u * (3 * kXStages + 2 * kATiles + 2 + a); };
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(base_ptr + L::kOffTmem);
  volatile uint32_t* abort_flag = tmem_slot + 1;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = two_cta::cluster_ctarank();  // 0 = leader (issues the MMAs)
  const int cluster_id = blockIdx.x >> 1;
  const int num_clusters = gridDim.x >> 1;

  // tiles: W-row tiles fastest, so that the CTA pairs working at the same time share x tiles in L2
  const int tiles_w = (N + TW - 1) / TW;
  const int tiles_x = (M + TX - 1) / TX;
  const int num_tiles = tiles_w * tiles_x;
  const int num_kb = K / BK;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kXStages; ++s) {
      mbar_init(bar_xfull(s), 1);
      mbar_init(bar_cfull(s), 1);
      mbar_init(bar_empty(s), 1 + kDqGroupWarps);
    }
    for (int t = 0; t < kATiles; ++t) {
      mbar_init(bar_afull(t), 2 * kDqGroupWarps);
      mbar_init(bar_aempty(t), 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(bar_accfull(a), 1);
      mbar_init(bar_accempty(a), 2 * kEpiWarps);
    }
    *abort_flag = 0;
    fence_mbar_init();
  }
  if (warp == 5) {  // the same warp of both CTAs allocates the pair's tensor memory
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;"
                 ::"r"(smem_u32((const void*)tmem_slot)), "r"(kTmemCols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  two_cta::cluster_sync_all();  // both CTAs' barriers exist before anybody signals across
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 4) {
    // ------------------------------------------------------- TMA producer (both CTAs)
    if (lane == 0) {
      uint32_t it = 0;
      bool ok = true;
      for (int tile = cluster_id; tile < num_tiles && ok; tile += num_clusters) {
        const int m0 = (tile / tiles_w) * TX + (int)rank * (TX / 2);   // this CTA's half of the x rows (B operand)
        const int n0 = (tile % tiles_w) * TW + (int)rank * 128;        // this CTA's W rows (A operand)
        for (int kb = 0; kb < num_kb; ++kb, ++it) {
          const int s = it % kXStages;
          const uint32_t ph = (it / kXStages) & 1u;
          if (!mbar_wait(bar_empty(s), ph ^ 1u, (1u << 8) | kRoleTma, abort_flag, &g_qmm_status)) { ok = false; break; }
          // the leader expects the x bytes of both CTAs; each CTA expects its own codes
          if (rank == 0) { mbar_expect_tx(bar_xfull(s), 2 * L::kXBytes); }
          mbar_expect_tx(bar_cfull(s), L::kCodeBytes);
          two_cta::tma_load_2d_pair(base + L::kOffX + s * L::kXBytes, &tmap_x, two_cta::map_to_cta(bar_xfull(s), 0),
                                    kb * BK, m0);
          tma_load_2d(base + L::kOffCode + s * L::kCodeBytes, &tmap_w, bar_cfull(s), kb * (BK / 8), n0);
        }
      }
      // Never leave with a copy still in flight (as in qmm_2cta.cuh).
      for (int s = 0; s < kXStages; ++s) {
        if (it > (uint32_t)s) {
          const uint32_t last = ((it - 1 - s) / kXStages) * kXStages + s;
          mbar_wait(bar_cfull(s), (last / kXStages) & 1u, (2u << 8) | kRoleTma, abort_flag, &g_qmm_status);
          if (rank == 0) {
            mbar_wait(bar_xfull(s), (last / kXStages) & 1u, (3u << 8) | kRoleTma, abort_flag, &g_qmm_status);
          }
        }
      }
    }
  } else if (warp == 5) {
    // --------------------------------------------------------- MMA issuer (leader only)
    if (lane == 0 && rank == 0) {
      constexpr uint32_t idesc = make_idesc_ta();
      uint32_t it = 0, ti = 0;
      bool ok = true;
      for (int tile = cluster_id; tile < num_tiles && ok; tile += num_clusters, ++ti) {
        const int a = ti & 1;
        const uint32_t aph = (ti >> 1) & 1u;
        if (!mbar_wait(bar_accempty(a), aph ^ 1u, (1u << 8) | kRoleMma, abort_flag, &g_qmm_status)) { ok = false; break; }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + (uint32_t)a * kAccCols;
        for (int kb = 0; kb < num_kb; ++kb, ++it) {
          const int s = it % kXStages;
          const uint32_t ph = (it / kXStages) & 1u;
          const int t = it % kATiles;
          const uint32_t tph = (it / kATiles) & 1u;
          if (!mbar_wait(bar_xfull(s), ph, (2u << 8) | kRoleMma, abort_flag, &g_qmm_status)) { ok = false; break; }
          if (!mbar_wait(bar_afull(t), tph, (3u << 8) | kRoleMma, abort_flag, &g_qmm_status)) { ok = false; break; }
          tc_fence_after();
          const uint32_t a_tmem = tmem_base + kAColBase + (uint32_t)t * kAColsPerTile;
          const uint64_t b_desc = make_sw128_desc(base + L::kOffX + s * L::kXBytes);
#pragma unroll
          for (int k16 = 0; k16 < BK / 16; ++k16) {
            // 16 bf16 further along K: 8 columns of the A tile, 32 bytes inside the swizzle atom of B
            umma_bf16_pair_ta(d_tmem, a_tmem + 8u * k16, b_desc + 2u * k16, idesc, (kb | k16) ? 1u : 0u);
          }
          two_cta::umma_commit_pair(bar_empty(s));    // x stage free in both CTAs
          two_cta::umma_commit_pair(bar_aempty(t));   // A tile free in both CTAs
        }
        if (ok) { two_cta::umma_commit_pair(bar_accfull(a)); }
      }
    }
  } else if (warp >= 6) {
    // ------------------------------------------------------- dequantisers (both CTAs)
    // A warp may touch only the tensor-memory lanes 32 (warp % 4) .. + 31; a thread's W row is its lane.
    const int grp = (warp - 6) / kDqGroupWarps;
    const int t_row = (warp & 3) * 32 + lane;   // row of the CTA's 128 W rows = tensor-memory lane
    const uint32_t lane_base = (uint32_t)((warp & 3) * 32) << 16;
    const int groups = K >> 6;
    const uint32_t afull_leader = two_cta::map_to_cta(bar0, 0);  // cluster address of the leader's barrier block
    uint32_t it = 0;
    bool ok = true;
    for (int tile = cluster_id; tile < num_tiles && ok; tile += num_clusters) {
      const int n0 = (tile % tiles_w) * TW + (int)rank * 128;
      int row = n0 + t_row;
      row = row < N ? row : N - 1;  // tail rows: any valid scale; their columns are never stored
      ScaleStream sst(scales + (int64_t)row * groups, biases + (int64_t)row * groups, groups);
      for (int kb = 0; kb < num_kb; ++kb, ++it) {
        const int s = it % kXStages;
        const uint32_t ph = (it / kXStages) & 1u;
        const int t = it % kATiles;
        const uint32_t tph = (it / kATiles) & 1u;
        if ((kb & (kDqGroups - 1)) != grp) { continue; }  // the other group's k block
        float sc, bi;
        sst.get(kb, sc, bi);
        if (!warp_wait(bar_cfull(s), ph, (1u << 8) | kRoleDq, abort_flag, &g_qmm_status)) { ok = false; break; }
        const uint4* cp = reinterpret_cast<const uint4*>(base_ptr + L::kOffCode + s * L::kCodeBytes + t_row * (BK / 2));
        const uint4 c0 = cp[0], c1 = cp[1];
        __syncwarp();
        if (lane == 0) { mbar_arrive(bar_empty(s)); }  // codes are in registers
        uint32_t o[32];
        const uint32_t cw[8] = {c0.x, c0.y, c0.z, c0.w, c1.x, c1.y, c1.z, c1.w};
        float s_133, s_129;
        if (dequant_scale_up(sc, s_133, s_129)) {
          const uint64_t s2 = pack_f32x2(s_133, s_129), b2 = pack_f32x2(bi, bi);
#pragma unroll
          for (int wd = 0; wd < 8; ++wd) { dequant_word_fast(cw[wd], s2, b2, o + 4 * wd); }
        } else {  // a zero, subnormal or large scale: the plain way
#pragma unroll
          for (int wd = 0; wd < 8; ++wd) { dequant_word_exact(cw[wd], sc, bi, o + 4 * wd); }
        }
        if (!warp_wait(bar_aempty(t), tph ^ 1u, (2u << 8) | kRoleDq, abort_flag, &g_qmm_status)) { ok = false; break; }
        tc_fence_after();
        // o[c] = (k = 2c, 2c + 1): column c of the A tile, low half first
        tmem_st32(tmem_base + lane_base + kAColBase + (uint32_t)t * kAColsPerTile, o);
        tmem_st_wait();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) {
          if (rank == 0) {
            mbar_arrive(bar_afull(t));
          } else {
            two_cta::mbar_arrive_cluster(afull_leader + 8u * (3 * kXStages + t));
          }
        }
      }
    }
  } else {
    // ------------------------------------------------------------ epilogue (both CTAs)
    // Accumulator = y^T: this thread's lane is output column n, its 32 registers of a load are 32
    // consecutive output rows m. A store instruction writes 32 consecutive n of one row: 64 bytes.
    uint32_t ti = 0;
    bool ok = true;
    const uint32_t accempty_leader = two_cta::map_to_cta(bar0, 0) + 8u * (3 * kXStages + 2 * kATiles + 2);
    for (int tile = cluster_id; tile < num_tiles && ok; tile += num_clusters, ++ti) {
      const int m0 = (tile / tiles_w) * TX;
      const int n = (tile % tiles_w) * TW + (int)rank * 128 + warp * 32 + lane;
      const int a = ti & 1;
      const uint32_t aph = (ti >> 1) & 1u;
      if (!warp_wait(bar_accfull(a), aph, (1u << 8) | kRoleEpi, abort_flag, &g_qmm_status)) { ok = false; break; }
      tc_fence_after();
      const uint32_t taddr = tmem_base + ((uint32_t)(warp * 32) << 16) + (uint32_t)a * kAccCols;
      __nv_bfloat16* ycol = y + n;
      const bool n_ok = n < N;
#pragma unroll 1
      for (int c = 0; c < TX / 32; ++c) {
        uint32_t r[32];
        tmem_ld32(taddr + (uint32_t)(c * 32), r);
        tmem_ld_wait();
        const int mb = m0 + c * 32;
        if (mb < M && n_ok) {
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            if (mb + j < M) { ycol[(int64_t)(mb + j) * ld] = __float2bfloat16_rn(__uint_as_float(r[j])); }
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) {
        if (rank == 0) {
          mbar_arrive(bar_accempty(a));
        } else {
          two_cta::mbar_arrive_cluster(accempty_leader + 8u * a);
        }
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  two_cta::cluster_sync_all();  // nobody leaves while its partner may still read its shared memory or signal it
  if (warp == 5) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kTmemCols)
                 : "memory");
  }
}

}  // namespace ta
