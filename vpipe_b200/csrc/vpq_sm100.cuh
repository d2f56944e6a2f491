// vpq_sm100.cuh -- mbarrier / TMA / proxy-fence helpers shared by the kernels,
// and the host helper that encodes 2-D tensor maps.
#pragma once

#include <cuda.h>

#include "vpq_common.cuh"

namespace vpq {

// Encodes a row-major 2-D tensor map (inner extent first); row_pitch_bytes 0 = rows back to back.
// Host side, api.cu.
int make_map_2d(CUtensorMap* map, CUtensorMapDataType dt, int elt_bytes, const void* ptr,
                uint64_t inner, uint64_t outer, uint32_t box_inner, uint32_t box_outer,
                CUtensorMapSwizzle swz, const char* what, uint64_t row_pitch_bytes = 0);

#ifdef __CUDACC__


__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return (uint32_t)__cvta_generic_to_shared(p);
}

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}

__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}

__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes)
               : "memory");
}

__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t"
      "}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}

// Bounded wait. The poll loop is four instructions of PTX around mbarrier.try_wait with a
// suspend-time hint (the thread sleeps in hardware instead of taking issue slots from the warps
// that are working; a profile of the first QMM showed most issued instructions were polls).
// On giving up it raises the CTA's abort flag, records `code` in the kernel's device status word
// (first failure wins) and returns false.
constexpr uint32_t kWaitHintNs = 1000;     // how long one try_wait may sleep
constexpr uint32_t kWaitPolls = 1u << 21;  // polls before a wait gives up (about 2 s of sleeping)

__device__ __forceinline__ bool mbar_wait_limited(uint32_t bar, uint32_t parity, uint32_t code,
                                                  volatile uint32_t* abort_flag, uint32_t* status_word,
                                                  uint32_t polls, uint32_t hint_ns) {
  uint32_t done;
  asm volatile(
      "{\n\t"
      ".reg .pred p, q;\n\t"
      ".reg .u32 n;\n\t"
      "mov.u32 n, 0;\n\t"
      "mov.u32 %0, 1;\n"
      "VPQ_WAIT_LOOP:\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
      "@p bra VPQ_WAIT_DONE;\n\t"
      "add.u32 n, n, 1;\n\t"
      "setp.lt.u32 q, n, %4;\n\t"
      "@q bra VPQ_WAIT_LOOP;\n\t"
      "mov.u32 %0, 0;\n"
      "VPQ_WAIT_DONE:\n\t"
      "}"
      : "=r"(done)
      : "r"(bar), "r"(parity), "r"(hint_ns), "r"(polls)
      : "memory");
  if (done) { return true; }
  *abort_flag = 1;
  atomicCAS(status_word, 0u, code);
  return false;
}

__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, uint32_t code,
                                          volatile uint32_t* abort_flag, uint32_t* status_word) {
  return mbar_wait_limited(bar, parity, code, abort_flag, status_word, kWaitPolls, kWaitHintNs);
}

// The same wait for a whole warp: every lane polls, then the lanes agree, so a
// warp never splits around the __syncwarp / .sync.aligned operations that follow.
__device__ __forceinline__ bool warp_wait(uint32_t bar, uint32_t parity, uint32_t code,
                                          volatile uint32_t* abort_flag, uint32_t* status_word) {
  const bool mine = mbar_wait(bar, parity, code, abort_flag, status_word);
  return __all_sync(0xffffffffu, mine);
}

// Plain (non-multicast) 2-D TMA load into this CTA's shared memory.
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, uint32_t bar,
                                            int c0, int c1) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%3, %4}], [%2];"
      ::"r"(dst), "l"(map), "r"(bar), "r"(c0), "r"(c1)
      : "memory");
}

// 2-D TMA store of a shared-memory tile (no swizzle) into global memory -- this GPU's or, in the
// column split, a peer's; elements outside the tensor are not written. Completion is tracked with
// bulk groups: commit, then wait for the group's READS of shared memory before reusing the tile.
__device__ __forceinline__ void tma_store_2d(const CUtensorMap* map, uint32_t src, int c0, int c1) {
  asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];"
               ::"l"(map), "r"(src), "r"(c0), "r"(c1)
               : "memory");
}
__device__ __forceinline__ void bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
template <int kPending>
__device__ __forceinline__ void bulk_wait_read() {
  asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(kPending) : "memory");
}
__device__ __forceinline__ void bulk_wait_all() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }

__device__ __forceinline__ void fence_proxy_async() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

__device__ __forceinline__ void fence_mbar_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}

#endif  // __CUDACC__

}  // namespace vpq
