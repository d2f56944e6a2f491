// vpq_common.cuh -- shared host/device helpers for the sm_100a kernels.
#pragma once

#include <cuda_runtime.h>
#include <cuda_fp16.h>
#include <cuda_bf16.h>
#include <stdint.h>

#include "../../include/vpq.h"

namespace vpq {

// ----------------------------------------------------------------- host side
// Records a message for vpq_last_error() and returns `code`.
int fail(int code, const char* fmt, ...);
void clear_error();

// Makes sure the current device can run sm_100a code (cached per device).
int require_sm100();

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

#define VPQ_CUDA_OK(expr)                                                          \
  do {                                                                             \
    cudaError_t _e = (expr);                                                       \
    if (_e != cudaSuccess) {                                                       \
      return ::vpq::fail(VPQ_ERR_CUDA, "%s: %s", #expr, cudaGetErrorString(_e));   \
    }                                                                              \
  } while (0)

#define VPQ_LAUNCH_OK(what)                                                        \
  do {                                                                             \
    cudaError_t _e = cudaGetLastError();                                           \
    if (_e != cudaSuccess) {                                                       \
      return ::vpq::fail(VPQ_ERR_CUDA, "%s launch: %s", what, cudaGetErrorString(_e)); \
    }                                                                              \
  } while (0)

int num_sms();

// The QMM with `reserve_sms` SMs left idle for a collective running beside it (qmm.cu).
int qmm_launch_reserved(const uint32_t* w, const void* scales, const void* biases, const void* x, void* y,
                        int64_t K, int64_t N, int64_t M, void* stream, int reserve_sms);

// The QMM whose epilogue stores its [M, N] column block into several row-major outputs of leading
// dimension ld at column col0 (this GPU's y and its peers' y); qmm.cu.
int qmm_launch_multi_dest(const uint32_t* w, const void* scales, const void* biases, const void* x,
                          void* const* dests, int count, int64_t ld, int64_t col0, int64_t K, int64_t N,
                          int64_t M, void* stream);

// Reads and clears the GEMV kernel's device status word (qmv.cu).
int ensure_dynamic_smem(const void* func, int* granted, size_t bytes);
int qmv_status_read(cudaStream_t st, uint32_t* out);
int qmvb_status_read(cudaStream_t st, uint32_t* out);
int qmv8_status_read(cudaStream_t st, uint32_t* out);
// Same for the cross-GPU barrier of the fused column-split (nsplit.cu).
int nsplit_status_read(cudaStream_t st, uint32_t* out);

// --------------------------------------------------------------- device side
#ifdef __CUDACC__

// f32 -> bf16 bits, the reference's integer round-to-nearest-even form
// (generative-models/quantize/model-quantizer.cc:56-60). Equal to
// cvt.rn.bf16.f32 for every finite input.
__device__ __forceinline__ uint32_t f32_to_bf16_bits(float f) {
  const uint32_t u = __float_as_uint(f);
  return (u + 0x7fffu + ((u >> 16) & 1u)) >> 16;
}

__device__ __forceinline__ float bf16_bits_to_f32(uint32_t b) {
  return __uint_as_float(b << 16);
}

// Two f32 -> packed bf16x2 (lo = a, hi = b), round to nearest even.
__device__ __forceinline__ uint32_t pack_bf16x2(float a, float b) {
  uint32_t r;
  asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(b), "f"(a));
  return r;
}

// The dequantised weight, exactly as the reference computes it: s*q is exact
// in f32 (8-bit x 4-bit significands), one f32 rounding on the add, then RNE
// to bf16 (gpu-kernels/metal/quant/affine_dequant.metal:49-52).
__device__ __forceinline__ float dequant_f32(float s, uint32_t q, float b) {
  return __fmaf_rn(s, (float)q, b);
}

__device__ __forceinline__ uint4 ldg_stream_v4(const void* p) {
  uint4 r;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w)
               : "l"(p));
  return r;
}

__device__ __forceinline__ uint32_t ldg_nc_u16(const void* p) {
  uint16_t r;
  asm volatile("ld.global.nc.u16 %0, [%1];" : "=h"(r) : "l"(p));
  return r;
}

#endif  // __CUDACC__

}  // namespace vpq
