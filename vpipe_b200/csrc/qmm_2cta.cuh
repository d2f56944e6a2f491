// qmm_2cta.cuh -- the QMM as a 2-CTA (cta_group::2) kernel: a cluster of two CTAs on one TPC
// computes a 256 x 256 output tile. Included by qmm.cu (uses its helpers).
//
// Why two CTAs: with a 128-row tile, every 64-wide k block costs one SM the dequantisation of
// 256 W rows and the shared-memory traffic of a full B operand. In a CTA pair each SM keeps its
// own 128 x rows (A operand) but only HALF of the W tile (128 rows of B); the tensor cores of
// both SMs read both halves. Dequant work and shared-memory bytes per flop halve.
//
// Per CTA, 448 threads: warps 0-3 epilogue (tensor-memory lanes = this CTA's 128 output rows),
// warp 4 TMA producer, warp 5 tensor-memory allocation (+ MMA issue in the leader CTA only), warps
// 6-13 dequantisers: groups of warps with one W row (64 values) per thread, the groups taking
// k blocks in turn so one block's latency hides behind the others'.
//
// Column split over several GPUs: the last `comm_pairs` CTA pairs of the grid compute nothing. They
// are SENDER CTAs: the computing pairs store every tile into this GPU's y and count it in a flag
// array; a sender CTA waits for its next tile's count, reads the tile back (from L2) and stores it
// into every peer's y with the TMA unit over NVLink. Keeping the peer stores on SMs of their
// own matters: a store that waits for link credit holds up everything behind it on its SM's way to
// the memory system. Issued from the computing SMs (first from the epilogue warps, then from two
// extra warps per CTA) the exchange did not overlap the GEMM, it added to it. The exception is a
// pair's LAST tile (direct_last): nothing follows it on those SMs, so its epilogue warps store it
// into the peers themselves, and the end of the exchange runs on every SM instead of the senders'.
//
// Two tile widths: 256 x 256 (TNT = 256: 128 W rows per CTA, two dequant groups of four warps) and
// 256 x 128 (TNT = 128: 64 W rows per CTA, four groups of two warps), the narrow one for shapes
// whose 256-wide tiles would leave most CTA pairs idle.
//
// Barriers. Local to each CTA: cfull[s] (packed W landed here), empty[s] (x + codes slot free:
// one multicast tcgen05.commit + the local dequant warps), bempty[t] (dequantised tile free:
// multicast commit), accfull[a] (accumulator done: multicast commit). In the leader CTA only:
// xfull[s] (x tiles of BOTH CTAs landed: the peer's TMA signals it through cta_group::2),
// bfull[t] (both halves dequantised: local + remote arrivals), accempty[a] (both CTAs' epilogues
// drained). No TMA load is a multicast load. Every wait is bounded.
#pragma once

namespace two_cta {

constexpr int TM = 256;        // tile rows (128 per CTA)
constexpr int kXStages4 = 5;   // x + codes ring, 4-bit weights
constexpr int kXStages8 = 4;   // ... 8-bit weights (the codes of a stage are twice as large)
constexpr int kDqWarps = 8;
constexpr int kThreads2 = 32 * (kEpiWarps + 2 + kDqWarps);

// Where a CTA pair's output tile goes: `count` row-major destinations (this GPU's y and, in the
// fused column-split, every peer's y mapped into this address space), leading dimension `ld`,
// and the column at which this GPU's block starts. Peer destinations are written with ordinary
// stores over NVLink.
struct OutSpec {
  __nv_bfloat16* base[8];
  int count;
  int col0;
  int64_t ld;
  int swiglu;  // 1, 2: columns 2j, 2j+1 of the product are gate j, up j: store act(gate) * up, half as
               // wide; act = silu (1) or the tanh form of gelu (2). Selects the kernel instantiation.
  // q | k | v GEMM: split0 > 0 routes output columns [0, split0) to base[0] (row pitch split0),
  // [split0, split1) to base[1] (pitch split1 - split0) and the rest to base[2] (pitch N - split1);
  // both splits are multiples of 128, so a 128-column pass never straddles two outputs.
  int split0, split1;
  int handshake;      // 1: `sync` is valid (column split with the cross-GPU handshake inside the kernel)
  int comm_pairs;     // column split: CTA pairs at the end of the grid that only send (0: nothing is sent)
  int direct_last;    // column split: a computing pair stores its LAST tile into the peers itself (nothing
                      // is queued behind that tile on its SMs, and the tail of the exchange runs on all SMs)
  uint32_t* tile_flags;  // column split: per tile, epilogue warps that have stored it locally (zero between calls)
  vpq::PeerSync sync;
};

// Column split: tensor maps over this rank's column block of every destination's y (m[0] = this
// GPU's copy, the source of the senders; m[1..] = the peers'), boxes of [tile width x 16 rows].
struct DestMaps {
  CUtensorMap m[8];
};

template <int BITS, int TNT = 256>
struct SmemT {
  static constexpr int kWRows = TNT / 2;              // W rows dequantised per CTA
  static constexpr int kDqGroups = 256 / kWRows;      // warp groups that take k blocks in turn (a group = kWRows threads)
  static constexpr int kDqGroupWarps = kDqWarps / kDqGroups;
  static constexpr int kXStages = TNT == 128 ? 6 : (BITS == 8 ? kXStages8 : kXStages4);
  static constexpr int kBTiles = TNT == 128 ? 8 : 5;  // dequantised-B ring
  static constexpr int kXBytes = 128 * BK * 2;        // 16 KB, 128B-swizzled
  static constexpr int kCodeBytes = kWRows * (BK * BITS / 8);  // rows x 32 B (64 B at 8 bits)
  static constexpr int kBBytes = kWRows * BK * 2;     // 128B-swizzled K-major
  static constexpr int kOffX = 0;
  static constexpr int kOffB = kOffX + kXStages * kXBytes;
  static constexpr int kOffCode = kOffB + kBTiles * kBBytes;
  static constexpr int kEpiBytes = 32 * 256;          // per epilogue warp: 32 rows x 128 bf16
  static constexpr int kOffEpi = kOffCode + kXStages * kCodeBytes;
  static constexpr int kOffBar = kOffEpi + kEpiWarps * kEpiBytes;
  static constexpr int kNumBars = 3 * kXStages + 2 * kBTiles + 4;
  static constexpr int kOffTmem = kOffBar + kNumBars * 8;
  static constexpr int kTotal = kOffTmem + 16;
  static constexpr int kAlloc = kTotal + 1024;
};
static_assert(SmemT<4>::kAlloc <= 227 * 1024 && SmemT<8>::kAlloc <= 227 * 1024 && SmemT<4, 128>::kAlloc <= 227 * 1024,
              "shared memory of the pair kernel");

__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}

__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}

// shared::cluster address of `local_addr` (a shared::cta address) in CTA `rank` of the cluster
__device__ __forceinline__ uint32_t map_to_cta(uint32_t local_addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(local_addr), "r"(rank));
  return r;
}

__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}

// The leader's MMA thread waits on barriers the partner CTA also arrives on with the ordinary
// bounded wait: the partner's shared-memory writes are published to the async proxy by its
// fence.proxy.async before its remote arrive, and the tensor core reads them only afterwards.
__device__ __forceinline__ bool mbar_wait_cluster(uint32_t bar, uint32_t parity, uint32_t code,
                                                  volatile uint32_t* abort_flag, uint32_t* status_word) {
  return mbar_wait(bar, parity, code, abort_flag, status_word);
}

// x tile of a CTA pair: lands in this CTA's shared memory, completes bytes on the LEADER's barrier.
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst, const CUtensorMap* map,
                                                 uint32_t leader_bar_cluster_addr, int c0, int c1) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%3, %4}], [%2];"
      ::"r"(dst), "l"(map), "r"(leader_bar_cluster_addr), "r"(c0), "r"(c1)
      : "memory");
}

__device__ __forceinline__ void umma_bf16_pair(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc,
                                               uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t"
      "}"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}

// Arrives on the barrier at this shared-memory offset in BOTH CTAs once the MMAs issued so far are done.
__device__ __forceinline__ void umma_commit_pair(uint32_t bar) {
  asm volatile(
      "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
      ::"r"(bar), "h"((uint16_t)3)
      : "memory");
}

// Instruction descriptor: D f32, A/B bf16, both K-major, M = 256 (pair), N = TNT.
template <int TNT>
__device__ __forceinline__ constexpr uint32_t make_idesc_pair() {
  return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(TNT >> 3) << 17) | ((uint32_t)(TM >> 4) << 24);
}

__device__ __forceinline__ uint4 ld_cg_v4(const void* p) {  // from L2: written moments ago by another warp
  uint4 r;
  asm volatile("ld.global.cg.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w) : "l"(p) : "memory");
  return r;
}


// GS: quantization group along K, 64 (one group per k block) or 32 (two).
template <int kAct, int BITS, int TNT, int GS>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kThreads2, 1)
affine_qmm_w4g64_2cta_kernel(const __grid_constant__ CUtensorMap tmap_x,
                             const __grid_constant__ CUtensorMap tmap_w,
                             const uint16_t* __restrict__ scales, const uint16_t* __restrict__ biases,
                             const OutSpec out, const __grid_constant__ DestMaps maps, int M, int N, int K) {
  using L = SmemT<BITS, TNT>;
  constexpr int kXStages = L::kXStages;
  constexpr int kBTiles = L::kBTiles;
  constexpr int kDqGroups = L::kDqGroups;
  constexpr int kDqGroupWarps = L::kDqGroupWarps;
  constexpr int kWRows = L::kWRows;
  constexpr int TN = TNT;
  constexpr uint32_t kTmemCols = 2 * TNT;  // two accumulator buffers

  extern __shared__ unsigned char smem_dyn[];
  const uint32_t raw = smem_u32(smem_dyn);
  const uint32_t base = (raw + 1023u) & ~1023u;
  unsigned char* base_ptr = smem_dyn + (base - raw);

  const uint32_t bar0 = base + L::kOffBar;
  auto bar_xfull = [&](int s) { return bar0 + 8u * s; };
  auto bar_cfull = [&](int s) { return bar0 + 8u * (kXStages + s); };
  auto bar_empty = [&](int s) { return bar0 + 8u * (2 * kXStages + s); };
  auto bar_bfull = [&](int t) { return bar0 + 8u * (3 * kXStages + t); };
  auto bar_bempty = [&](int t) { return bar0 + 8u * (3 * kXStages + kBTiles + t); };
  auto bar_accfull = [&](int a) { return bar0 + 8u * (3 * kXStages + 2 * kBTiles + a); };
  auto bar_accempty = [&](int a) { return bar0 + 8u * (3 * kXStages + 2 * kBTiles + 2 + a); };
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(base_ptr + L::kOffTmem);
  volatile uint32_t* abort_flag = tmem_slot + 1;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();  // 0 = leader (issues the MMAs)
  const int cluster_id = blockIdx.x >> 1;
  const int num_clusters = (gridDim.x >> 1) - out.comm_pairs;  // the pairs that compute

  const int tiles_m = (M + TM - 1) / TM;
  const int tiles_n = (N + TN - 1) / TN;
  const int num_tiles = tiles_m * tiles_n;
  const int num_kb = K / BK;

  if (out.comm_pairs > 0 && cluster_id >= num_clusters) {
    // -------------------------------------------------- sender CTAs (column split only)
    // Both CTAs of a sender pair work alone: sender CTA c of C takes tiles c, c + C, ... in the
    // order the computing pairs finish them. No barriers of the pipeline, no tensor memory.
    const int C = 2 * out.comm_pairs;
    // tiles the senders move: all, or all but the last tile of every computing pair (the last num_clusters)
    const int send_tiles = out.direct_last ? max(0, num_tiles - num_clusters) : num_tiles;
    __shared__ uint32_t comm_ok;
    if (threadIdx.x == 0) { comm_ok = 1; }
    __syncthreads();
    if (out.handshake && threadIdx.x >= 1 && threadIdx.x < (unsigned)out.count) {
      // No store into a peer's y before that peer's stream has reached this call (bounded wait).
      bool seen = false;
      volatile uint32_t* f = out.sync.my_flags + out.sync.src_rank[threadIdx.x];
      for (uint32_t i = 0; i < (1u << 24); ++i) {
        if ((int32_t)(*f - out.sync.epoch) >= 0) {
          seen = true;
          break;
        }
        __nanosleep(100);
      }
      if (!seen) {
        comm_ok = 0;
        atomicCAS(&g_qmm_status, 0u, (2u << 8) | kRoleSend);
      }
    }
    __threadfence_system();
    __syncthreads();
    // One thread drives the copy with the TMA unit, nothing passes through registers: a tile travels
    // as chunks of kChunkRows rows; a chunk is loaded from this GPU's y into a ring slot of shared
    // memory (tensor-map load, completion on the slot's mbarrier) and stored from there into every
    // peer's y (tensor-map stores, one bulk group per chunk). Loads run kSlots - 1 chunks ahead of
    // the stores. The maps cover exactly this rank's column block, so a tile that overhangs the block
    // is clipped by the hardware on both sides.
    // kDrivers threads of a sender CTA (lane 0 of the first warps) each run such a pipeline of their
    // own on their own share of the tiles: one thread's load -> store -> wait chain keeps the TMA unit
    // busy only part of the time.
    constexpr int kDrivers = 4;
    constexpr int kChunkRows = 16;
    constexpr int kChunkBytes = kChunkRows * TN * 2;   // 8 KB (4 KB for the 128-wide tile)
    constexpr int kSlots = 6;
    constexpr int kChunksPerTile = TM / kChunkRows;
    static_assert(kDrivers * (kSlots * kChunkBytes + kSlots * 8) <= L::kTotal, "sender rings fit the kernel's shared memory");
    __shared__ uint32_t comm_abort;
    if (lane == 0 && warp < kDrivers) {
      const uint32_t ring = base + (uint32_t)warp * (kSlots * kChunkBytes);              // the pipeline's shared memory is free here
      const uint32_t sbar = base + kDrivers * kSlots * kChunkBytes + (uint32_t)warp * kSlots * 8u;  // one mbarrier per slot
      const int C = kDrivers * 2 * out.comm_pairs;   // (shadows: tiles are dealt over all drivers of all sender CTAs)
      const int c = ((cluster_id - num_clusters) * 2 + (int)rank) * kDrivers + warp;
      for (int i = 0; i < kSlots; ++i) { mbar_init(sbar + 8u * i, 1); }
      fence_mbar_init();
      int my_tiles = 0;
      for (int tile = c; tile < send_tiles; tile += C) { ++my_tiles; }
      const int total = my_tiles * kChunksPerTile;
      int loaded = 0, ready_tiles = 0;   // chunks whose load was issued; tiles of this CTA's list known to be complete
      bool ok = comm_ok != 0;
      // Is tile number ti of this CTA's list stored locally by all eight epilogue warps of its pair?
      // block: wait for it (bounded; false = gave up); otherwise just look.
      auto tile_ready = [&](int ti, bool block) -> bool {
        if (ti < ready_tiles) { return true; }
        volatile uint32_t* f = out.tile_flags + (c + ti * C);
        bool seen = *f >= 2u * kEpiWarps;
        for (uint32_t i = 0; block && !seen && i < (1u << 24); ++i) {
          __nanosleep(64);
          seen = *f >= 2u * kEpiWarps;
        }
        if (seen) {
          __threadfence();
          asm volatile("fence.proxy.async.global;" ::: "memory");  // generic-proxy stores -> the TMA unit's reads
          ready_tiles = ti + 1;
        }
        return seen;
      };
      auto issue_load = [&](int q) {   // chunk q of this CTA's list
        const int ti = q / kChunksPerTile, ch = q % kChunksPerTile;
        const int tile = c + ti * C;
        const int slot = q % kSlots;
        mbar_expect_tx(sbar + 8u * slot, kChunkBytes);
        tma_load_2d(ring + slot * kChunkBytes, &maps.m[0], sbar + 8u * slot, (tile % tiles_n) * TN,
                    (tile / tiles_n) * TM + ch * kChunkRows);
      };
      for (int q = 0; q < total && ok; ++q) {
        // loads run up to kSlots chunks ahead, as far as finished tiles allow; the chunk that is due
        // now is waited for
        while (loaded < total && loaded < q + kSlots) {
          const bool must = loaded == q;
          if (!tile_ready(loaded / kChunksPerTile, must)) {
            if (must) {
              atomicCAS(&g_qmm_status, 0u, (1u << 8) | kRoleSend);
              ok = false;
            }
            break;
          }
          issue_load(loaded);
          ++loaded;
        }
        if (!ok) { break; }
        const int slot = q % kSlots;
        if (!mbar_wait(sbar + 8u * slot, (uint32_t)(q / kSlots) & 1u, (3u << 8) | kRoleSend, &comm_abort, &g_qmm_status)) {
          ok = false;
          break;
        }
        const int ti = q / kChunksPerTile, ch = q % kChunksPerTile;
        const int tile = c + ti * C;
        for (int d = 1; d < out.count; ++d) {
          tma_store_2d(&maps.m[d], ring + slot * kChunkBytes, (tile % tiles_n) * TN, (tile / tiles_n) * TM + ch * kChunkRows);
        }
        bulk_commit();
        if (ch == kChunksPerTile - 1) { out.tile_flags[tile] = 0; }  // all of the tile's loads have landed: ready for the next call
        bulk_wait_read<0>();  // the slot may be loaded again (the stores themselves drain behind)
      }
      bulk_wait_all();  // every store of this driver has been performed
      if (!ok) { comm_ok = 0; }
    }
    // All stores of this CTA are out: the CTA that finishes last on this GPU (of the senders, or of the
    // whole grid when the computing pairs store their last tiles themselves) tells every peer that this
    // rank's column block is complete in the peer's y.
    __threadfence_system();
    __syncthreads();
    if (out.handshake && threadIdx.x == 0) {
      const uint32_t parties = out.direct_last ? gridDim.x : (uint32_t)C;
      if (atomicAdd(out.sync.warps_done, 1u) == parties - 1u) {
        __threadfence_system();
        for (int d = 1; d < out.count; ++d) {
          *reinterpret_cast<volatile uint32_t*>(out.sync.flag_of[d] + 8 + out.sync.rank) = out.sync.epoch;
        }
        *out.sync.warps_done = 0;
        __threadfence_system();
      }
    }
    return;
  }

  if (threadIdx.x == 0) {
    for (int s = 0; s < kXStages; ++s) {
      mbar_init(bar_xfull(s), 1);
      mbar_init(bar_cfull(s), 1);
      mbar_init(bar_empty(s), 1 + kDqGroupWarps);
    }
    for (int t = 0; t < kBTiles; ++t) {
      mbar_init(bar_bfull(t), 2 * kDqGroupWarps);
      mbar_init(bar_bempty(t), 1);
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
  cluster_sync_all();  // both CTAs' barriers exist before anybody signals across
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (out.handshake && blockIdx.x == 0 && threadIdx.x < (unsigned)out.count && threadIdx.x >= 1) {
    // this rank's stream has reached the call: tell every peer (its senders wait for this before they
    // write into our y, which an earlier kernel of ours may have been reading until now)
    *reinterpret_cast<volatile uint32_t*>(out.sync.flag_of[threadIdx.x] + out.sync.rank) = out.sync.epoch;
  }

  if (warp == 4) {
    // ------------------------------------------------------- TMA producer (both CTAs)
    if (lane == 0) {
      uint32_t it = 0;
      bool ok = true;
      for (int tile = cluster_id; tile < num_tiles && ok; tile += num_clusters) {
        const int m0 = (tile / tiles_n) * TM + (int)rank * 128;
        const int n0 = (tile % tiles_n) * TN + (int)rank * kWRows;
        for (int kb = 0; kb < num_kb; ++kb, ++it) {
          const int s = it % kXStages;
          const uint32_t ph = (it / kXStages) & 1u;
          if (!mbar_wait(bar_empty(s), ph ^ 1u, (1u << 8) | kRoleTma, abort_flag, &g_qmm_status)) { ok = false; break; }
          // the leader expects the x bytes of both CTAs; each CTA expects its own codes
          if (rank == 0) { mbar_expect_tx(bar_xfull(s), 2 * L::kXBytes); }
          mbar_expect_tx(bar_cfull(s), L::kCodeBytes);
          tma_load_2d_pair(base + L::kOffX + s * L::kXBytes, &tmap_x, map_to_cta(bar_xfull(s), 0), kb * BK, m0);
          tma_load_2d(base + L::kOffCode + s * L::kCodeBytes, &tmap_w, bar_cfull(s), kb * (BK * BITS / 32), n0);
        }
      }
      // Never leave with a copy still in flight: the codes barriers are local; the x copies of
      // the last uses of each stage are covered by the final cluster barrier below, which the
      // leader reaches only after its MMAs (hence these loads) completed or its waits gave up.
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
      constexpr uint32_t idesc = make_idesc_pair<TNT>();
      uint32_t it = 0, ti = 0;
      bool ok = true;
      for (int tile = cluster_id; tile < num_tiles && ok; tile += num_clusters, ++ti) {
        const int a = ti & 1;
        const uint32_t aph = (ti >> 1) & 1u;
        if (!mbar_wait_cluster(bar_accempty(a), aph ^ 1u, (1u << 8) | kRoleMma, abort_flag, &g_qmm_status)) { ok = false; break; }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + (uint32_t)(a * TN);
        for (int kb = 0; kb < num_kb; ++kb, ++it) {
          const int s = it % kXStages;
          const uint32_t ph = (it / kXStages) & 1u;
          const int t = it % kBTiles;
          const uint32_t bph = (it / kBTiles) & 1u;
          if (!mbar_wait_cluster(bar_xfull(s), ph, (2u << 8) | kRoleMma, abort_flag, &g_qmm_status)) { ok = false; break; }
          if (!mbar_wait_cluster(bar_bfull(t), bph, (3u << 8) | kRoleMma, abort_flag, &g_qmm_status)) { ok = false; break; }
          tc_fence_after();
          const uint64_t a_desc = make_sw128_desc(base + L::kOffX + s * L::kXBytes);
          const uint64_t b_desc = make_sw128_desc(base + L::kOffB + t * L::kBBytes);
#pragma unroll
          for (int k16 = 0; k16 < BK / 16; ++k16) {
            umma_bf16_pair(d_tmem, a_desc + 2u * k16, b_desc + 2u * k16, idesc, (kb | k16) ? 1u : 0u);
          }
          umma_commit_pair(bar_empty(s));   // x stage free in both CTAs
          umma_commit_pair(bar_bempty(t));  // dequantised tiles free in both CTAs
        }
        if (ok) { umma_commit_pair(bar_accfull(a)); }
      }
    }
  } else if (warp >= 6) {
    // ------------------------------------------------------- dequantisers (both CTAs)
    // Groups of kWRows threads take the k blocks in turn, one W row (a whole group of 64 values)
    // per thread: a group has kDqGroups MMA periods to turn a tile around instead of one.
    const int grp = (warp - 6) / kDqGroupWarps;
    const int t_row = threadIdx.x - 6 * 32 - grp * (kDqGroupWarps * 32);  // 0 .. kWRows - 1
    const uint32_t row_off = (uint32_t)(t_row >> 3) * 1024u + (uint32_t)(t_row & 7) * 128u;
    const uint32_t sw = (uint32_t)(t_row & 7);
    const int groups = K / GS;
    const uint32_t bfull_leader = map_to_cta(bar0, 0);  // cluster address of the leader's barrier block
    uint32_t it = 0;
    bool ok = true;
    for (int tile = cluster_id; tile < num_tiles && ok; tile += num_clusters) {
      const int n0 = (tile % tiles_n) * TN + (int)rank * kWRows;
      int row = n0 + t_row;
      row = row < N ? row : N - 1;  // tail rows: any valid scale; their columns are never stored
      const uint16_t* srow = scales + (int64_t)row * groups;
      const uint16_t* brow = biases + (int64_t)row * groups;
      ScaleStream sst(srow, brow, groups);
      for (int kb = 0; kb < num_kb; ++kb, ++it) {
        const int s = it % kXStages;
        const uint32_t ph = (it / kXStages) & 1u;
        const int t = it % kBTiles;
        const uint32_t bph = (it / kBTiles) & 1u;
        if ((kb & (kDqGroups - 1)) != grp) { continue; }  // another group's k block
        float sc, bi, sc_hi, bi_hi;  // group 32: the scales of the two halves of the k block
        if (GS == 64) {
          sst.get(kb, sc, bi);
          sc_hi = sc;
          bi_hi = bi;
        } else {
          sst.get(2 * kb, sc, bi);
          sst.get(2 * kb + 1, sc_hi, bi_hi);
        }
        if (!warp_wait(bar_cfull(s), ph, (1u << 8) | kRoleDq, abort_flag, &g_qmm_status)) { ok = false; break; }
        const uint4* cp = reinterpret_cast<const uint4*>(base_ptr + L::kOffCode + s * L::kCodeBytes +
                                                         t_row * (BK * BITS / 8));
        uint32_t o[32];
        if (BITS == 4) {
          const uint4 c0 = cp[0], c1 = cp[1];
          __syncwarp();
          if (lane == 0) { mbar_arrive(bar_empty(s)); }  // codes are in registers

          const uint32_t cw[8] = {c0.x, c0.y, c0.z, c0.w, c1.x, c1.y, c1.z, c1.w};
#pragma unroll
          for (int hf = 0; hf < (GS == 64 ? 1 : 2); ++hf) {  // per scale: the whole k block, or each half of it
            constexpr int kWords = GS == 64 ? 8 : 4;
            const float sh = hf ? sc_hi : sc, bh = hf ? bi_hi : bi;
            float s_133, s_129;
            if (dequant_scale_up(sh, s_133, s_129)) {
              const uint64_t s2 = pack_f32x2(s_133, s_129), b2 = pack_f32x2(bh, bh);
#pragma unroll
              for (int wd = 0; wd < kWords; ++wd) { dequant_word_fast(cw[hf * kWords + wd], s2, b2, o + 4 * (hf * kWords + wd)); }
            } else {  // a zero, subnormal or large scale: the plain way
#pragma unroll
              for (int wd = 0; wd < kWords; ++wd) { dequant_word_exact(cw[hf * kWords + wd], sh, bh, o + 4 * (hf * kWords + wd)); }
            }
          }
        } else {
          const uint4 c0 = cp[0], c1 = cp[1], c2 = cp[2], c3 = cp[3];
          __syncwarp();
          if (lane == 0) { mbar_arrive(bar_empty(s)); }  // codes are in registers
          const uint32_t cw[16] = {c0.x, c0.y, c0.z, c0.w, c1.x, c1.y, c1.z, c1.w,
                                   c2.x, c2.y, c2.z, c2.w, c3.x, c3.y, c3.z, c3.w};
          // A byte placed in bits 16..23 of an otherwise zero word is the float q * 2^-133
          // (subnormals and the first binade are linear in their bit pattern), so
          // fma(that, s * 2^133, b) rounds the same real number as fma(s, q, b): bit-exact,
          // as long as s * 2^133 is a normal float (2^-126 <= |s| < 2^-5; else the plain way).
#pragma unroll
          for (int hf = 0; hf < (GS == 64 ? 1 : 2); ++hf) {
            constexpr int kWords = GS == 64 ? 16 : 8;
            const float sh = hf ? sc_hi : sc, bh = hf ? bi_hi : bi;
            float s_133, s_129;
            if (dequant_scale_up(sh, s_133, s_129)) {
              const uint64_t s2 = pack_f32x2(s_133, s_133), b2 = pack_f32x2(bh, bh);
#pragma unroll
              for (int wd = 0; wd < kWords; ++wd) { dequant_word8_fast(cw[hf * kWords + wd], s2, b2, o + 2 * (hf * kWords + wd)); }
            } else {
#pragma unroll
              for (int wd = 0; wd < kWords; ++wd) { dequant_word8_exact(cw[hf * kWords + wd], sh, bh, o + 2 * (hf * kWords + wd)); }
            }
          }
        }

        if (!warp_wait(bar_bempty(t), bph ^ 1u, (2u << 8) | kRoleDq, abort_flag, &g_qmm_status)) { ok = false; break; }
        unsigned char* bt = base_ptr + L::kOffB + t * L::kBBytes + row_off;
#pragma unroll
        for (int c = 0; c < 8; ++c) {  // 16-byte chunk c of the row lands at chunk (c ^ row%8)
          *reinterpret_cast<uint4*>(bt + ((((uint32_t)c) ^ sw) << 4)) =
              make_uint4(o[4 * c], o[4 * c + 1], o[4 * c + 2], o[4 * c + 3]);
        }
        fence_proxy_async();  // generic-proxy writes -> visible to the tensor cores' async reads
        __syncwarp();
        if (lane == 0) {
          if (rank == 0) {
            mbar_arrive(bar_bfull(t));
          } else {
            mbar_arrive_cluster(bfull_leader + 8u * (3 * kXStages + t));
          }
        }
      }
    }
  } else {
    // ------------------------------------------------------------ epilogue (both CTAs)
    uint32_t ti = 0;
    bool ok = true;
    // Fused SwiGLU / GeGLU (the reference's affine_qmm_swiglu_w4g64, affine_qmm_steel.metal:641-800,
    // and affine_qmm_geglu_w4g64, :1451-1547): the 256 columns of a tile become 128 outputs, one
    // pass of the same store path.
    constexpr bool swiglu = kAct != 0;
    const int n_out = swiglu ? N / 2 : N;                 // width of the stored block
    constexpr int passes = swiglu ? 1 : TN / 128;
    constexpr int loads = swiglu ? 8 : 4;                 // 32-column accumulator reads per pass
    const bool vec_ok = (n_out % 8) == 0 && (out.ld % 8) == 0 && (out.col0 % 8) == 0;
    const uint32_t accempty_leader = map_to_cta(bar0, 0) + 8u * (3 * kXStages + 2 * kBTiles + 2);
    for (int tile = cluster_id; tile < num_tiles && ok; tile += num_clusters, ++ti) {
      const int m0 = (tile / tiles_n) * TM + (int)rank * 128;
      const int n0 = (tile % tiles_n) * TN;
      const int a = ti & 1;
      const uint32_t aph = (ti >> 1) & 1u;
      // this pair's last tile goes to the peers from here (column split)
      bool direct = kAct == 0 && out.direct_last != 0 && out.count > 1 && tile + num_clusters >= num_tiles;
      if (direct && out.handshake) {
        // no store into a peer's y before that peer's stream has reached this call (bounded wait; by the
        // last tile the flags have long arrived)
        bool seen = true;
        if (lane >= 1 && lane < out.count) {
          volatile uint32_t* f = out.sync.my_flags + out.sync.src_rank[lane];
          seen = false;
          for (uint32_t i = 0; i < (1u << 24); ++i) {
            if ((int32_t)(*f - out.sync.epoch) >= 0) {
              seen = true;
              break;
            }
            __nanosleep(100);
          }
        }
        if (!__all_sync(0xffffffffu, seen)) {
          if (lane == 0) { atomicCAS(&g_qmm_status, 0u, (4u << 8) | kRoleSend); }
          direct = false;  // this GPU's y is still written; the peers' stay untouched
        }
        __threadfence_system();
      }
      if (!warp_wait(bar_accfull(a), aph, (1u << 8) | kRoleEpi, abort_flag, &g_qmm_status)) { ok = false; break; }
      tc_fence_after();
      const uint32_t taddr = tmem_base + ((uint32_t)(warp * 32) << 16) + (uint32_t)(a * TN);
      // The accumulator comes out of tensor memory one row per lane; it is transposed through a
      // warp-private, XOR-swizzled staging block so that 16 lanes store 256 contiguous bytes of
      // one output row (what remote stores over NVLink, and local ones, want).
      unsigned char* stg = base_ptr + L::kOffEpi + warp * L::kEpiBytes;
      const int mrow0 = m0 + warp * 32;
#pragma unroll 1
      for (int h = 0; h < passes; ++h) {
#pragma unroll 1
        for (int c = 0; c < loads; ++c) {
          uint32_t r[32];
          tmem_ld32(taddr + (uint32_t)(h * 128 + c * 32), r);
          tmem_ld_wait();
          if (swiglu) {
#pragma unroll
            for (int v = 0; v < 2; ++v) {
              float o[8];
#pragma unroll
              for (int i = 0; i < 8; ++i) {
                const float g = __uint_as_float(r[16 * v + 2 * i]), u = __uint_as_float(r[16 * v + 2 * i + 1]);
                if (kAct == 2) {  // gelu_pytorch_tanh(g) * u
                  const float th = tanhf(0.7978845608028654f * (g + 0.044715f * g * g * g));
                  o[i] = 0.5f * g * (1.0f + th) * u;
                } else {
                  o[i] = __fdividef(g, 1.0f + __expf(-g)) * u;
                }
              }
              uint4 pk;
              pk.x = pack_bf16x2(o[0], o[1]);
              pk.y = pack_bf16x2(o[2], o[3]);
              pk.z = pack_bf16x2(o[4], o[5]);
              pk.w = pack_bf16x2(o[6], o[7]);
              const int j = c * 2 + v;
              *reinterpret_cast<uint4*>(stg + lane * 256 + ((j ^ (lane & 15)) << 4)) = pk;
            }
          } else {
#pragma unroll
            for (int v = 0; v < 4; ++v) {
              uint4 pk;
              pk.x = pack_bf16x2(__uint_as_float(r[8 * v + 0]), __uint_as_float(r[8 * v + 1]));
              pk.y = pack_bf16x2(__uint_as_float(r[8 * v + 2]), __uint_as_float(r[8 * v + 3]));
              pk.z = pack_bf16x2(__uint_as_float(r[8 * v + 4]), __uint_as_float(r[8 * v + 5]));
              pk.w = pack_bf16x2(__uint_as_float(r[8 * v + 6]), __uint_as_float(r[8 * v + 7]));
              const int j = c * 4 + v;  // 16-byte chunk of the 256-byte row
              *reinterpret_cast<uint4*>(stg + lane * 256 + ((j ^ (lane & 15)) << 4)) = pk;
            }
          }
        }
        __syncwarp();
        int nc0 = swiglu ? n0 / 2 : n0 + h * 128;  // first stored column of this pass (within the block)
        const int j = lane & 15;               // this lane's 16-byte chunk = 8 columns
        const bool col_ok = nc0 + j * 8 < n_out;
        if (out.split0 > 0) {
          // three outputs (q | k | v): this pass's 128 columns belong to exactly one of them
          const int seg = nc0 < out.split0 ? 0 : nc0 < out.split1 ? 1 : 2;
          const int seg0 = seg == 0 ? 0 : seg == 1 ? out.split0 : out.split1;
          const int seg_w = (seg == 0 ? out.split0 : seg == 1 ? out.split1 : N) - seg0;
          __nv_bfloat16* dst = out.base[seg];
#pragma unroll 4
          for (int i = 0; i < 16; ++i) {
            const int row = 2 * i + (lane >> 4);
            const uint4 pk = *reinterpret_cast<const uint4*>(stg + row * 256 + ((j ^ (row & 15)) << 4));
            const int mm = mrow0 + row;
            if (mm < M && col_ok) { *reinterpret_cast<uint4*>(dst + (int64_t)mm * seg_w + (nc0 - seg0) + j * 8) = pk; }
          }
        } else if (vec_ok) {
#pragma unroll 4
          for (int i = 0; i < 16; ++i) {
            const int row = 2 * i + (lane >> 4);
            const uint4 pk = *reinterpret_cast<const uint4*>(stg + row * 256 + ((j ^ (row & 15)) << 4));
            const int mm = mrow0 + row;
            if (mm < M && col_ok) {
              const int64_t off = (int64_t)mm * out.ld + out.col0 + nc0 + j * 8;
              *reinterpret_cast<uint4*>(out.base[0] + off) = pk;  // this GPU's y; the senders feed the peers
              if (kAct != 0 || direct) {
                for (int d = 1; d < out.count; ++d) { *reinterpret_cast<uint4*>(out.base[d] + off) = pk; }
              }
            }
          }
        } else {  // ragged widths: element-wise
          for (int i = 0; i < 16; ++i) {
            const int row = 2 * i + (lane >> 4);
            const uint4 pk = *reinterpret_cast<const uint4*>(stg + row * 256 + ((j ^ (row & 15)) << 4));
            const __nv_bfloat16* e = reinterpret_cast<const __nv_bfloat16*>(&pk);
            const int mm = mrow0 + row;
            if (mm < M) {
              for (int d = 0; d < out.count; ++d) {
                __nv_bfloat16* yrow = out.base[d] + (int64_t)mm * out.ld + out.col0 + nc0 + j * 8;
                for (int q = 0; q < 8; ++q) {
                  if (nc0 + j * 8 + q < n_out) { yrow[q] = e[q]; }
                }
              }
            }
          }
        }
        __syncwarp();
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) {
        if (rank == 0) {
          mbar_arrive(bar_accempty(a));
        } else {
          mbar_arrive_cluster(accempty_leader + 8u * a);
        }
      }
      if (out.comm_pairs > 0 && !direct) {  // hand the tile to the sender CTAs: stores first, then the count
        __threadfence();
        __syncwarp();
        if (lane == 0) { atomicAdd(out.tile_flags + tile, 1u); }
      }
      if (direct) { __threadfence_system(); }  // this warp's peer stores, before the CTA reports below
    }
  }

  tc_fence_before();
  __syncthreads();
  if (kAct == 0 && out.direct_last != 0 && out.handshake && threadIdx.x == 0) {
    // this CTA's peer stores are out (fenced by their warps, ordered before this thread by the barrier):
    // the CTA of the grid that reports last tells every peer that the column block is complete
    __threadfence_system();
    if (atomicAdd(out.sync.warps_done, 1u) == gridDim.x - 1u) {
      __threadfence_system();
      for (int d = 1; d < out.count; ++d) {
        *reinterpret_cast<volatile uint32_t*>(out.sync.flag_of[d] + 8 + out.sync.rank) = out.sync.epoch;
      }
      *out.sync.warps_done = 0;
      __threadfence_system();
    }
  }
  cluster_sync_all();  // nobody leaves while its partner may still read its shared memory or signal it
  if (warp == 5) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kTmemCols)
                 : "memory");
  }
}

}  // namespace two_cta
