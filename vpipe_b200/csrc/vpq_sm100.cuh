// vpq_sm100.cuh -- mbarrier / TMA / proxy-fence helpers shared by the kernels,
// and the host helper that encodes 2-D tensor maps.
#pragma once

#include <cuda.h>

#include "vpq_common.cuh"

namespace vpq {

// Encodes a row-major 2-D tensor map (inner extent first). Host side, api.cu.
int make_map_2d(CUtensorMap* map, CUtensorMapDataType dt, int elt_bytes, const void* ptr,
                uint64_t inner, uint64_t outer, uint32_t box_inner, uint32_t box_outer,
                CUtensorMapSwizzle swz, const char* what);

#ifdef __CUDACC__

constexpr uint32_t kSpinLimit = 1u << 22;  // polls (with back-off) before a wait gives up

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

// Bounded wait. On giving up it raises the CTA's abort flag, records `code`
// in the kernel's device status word (first failure wins) and returns false.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, uint32_t code,
                                          volatile uint32_t* abort_flag, uint32_t* status_word) {
  for (uint32_t i = 0; i < kSpinLimit; ++i) {
    if (mbar_try_wait(bar, parity)) { return true; }
    if (i > 64) {
      __nanosleep(i > 4096 ? 256 : 32);
      if (*abort_flag) { return false; }
    }
  }
  *abort_flag = 1;
  atomicCAS(status_word, 0u, code);
  return false;
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

__device__ __forceinline__ void fence_proxy_async() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

__device__ __forceinline__ void fence_mbar_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}

#endif  // __CUDACC__

}  // namespace vpq
