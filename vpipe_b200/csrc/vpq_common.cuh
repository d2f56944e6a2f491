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

// Cross-GPU handshake of the fused column split, carried out inside the GEMM kernel itself.
// Every rank has a flag table (uint32 [16], mapped by all peers): slot r = "rank r has started call
// number `epoch`" (so whatever it enqueued earlier to read y is done), slot 8 + r = "rank r has
// finished storing its column block of call `epoch` everywhere". flag_of[d] is the table of the
// peer behind destination d (d >= 1; the order of `dests`), src_rank[d] that peer's rank.
struct PeerSync {
  uint32_t* flag_of[8];
  int src_rank[8];
  uint32_t* my_flags;   // this rank's own table
  uint32_t* warps_done; // this GPU's count of sender CTAs that finished (zero between calls)
  uint32_t* tile_flags; // per tile of the GEMM: epilogue warps that stored it locally (zero between calls)
  int tile_flag_count;  // entries of tile_flags
  uint32_t epoch;
  int rank;
};

// The QMM that stores its [M, N] column block into this GPU's row-major output dests[0] (leading
// dimension ld, first column col0) and whose sender CTAs copy every finished tile on to the peers'
// outputs dests[1..count); qmm.cu. `sync` carries the tile flags; its handshake part is used when
// sync->my_flags is not null.
int qmm_launch_multi_dest(const uint32_t* w, const void* scales, const void* biases, const void* x,
                          void* const* dests, int count, int64_t ld, int64_t col0, int64_t K, int64_t N,
                          int64_t M, void* stream, const PeerSync* sync);

// Reads and clears the GEMV kernel's device status word (qmv.cu).
int ensure_dynamic_smem(const void* func, int* granted, size_t bytes);
int qmv_status_read(cudaStream_t st, uint32_t* out);
int qmvb_status_read(cudaStream_t st, uint32_t* out);
int qmv8_status_read(cudaStream_t st, uint32_t* out);
// The fused-store part of a GEMV descriptor's validation (epilogue code, aux / y3 / row counts).
int qmv_check_store(const char* who, const vpq_linear_desc& d);
// Same, and rejects the RMSNorm prologue, expert gather and plan dependency of the w4 g64 GEMV.
int qmv_check_plain(const char* who, const vpq_linear_desc& d, bool allow_norm = false);
// Same, but the expert gather (expert, experts, x_div) is allowed and validated; allow_norm: norm_w too.
int qmv_check_gather(const char* who, const vpq_linear_desc& d, bool allow_norm = false);
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
  // (float)q without the conversion unit: q < 2^23 sits in the mantissa of 2^23 + q, exactly
  const float qf = __fsub_rn(__uint_as_float(0x4B000000u | q), 8388608.0f);
  return __fmaf_rn(s, qf, b);
}

// gelu_pytorch_tanh: 0.5 x (1 + tanh(sqrt(2 / pi) (x + 0.044715 x^3))), the activation of the
// reference's geglu stores (affine_qmv.metal:1421-1429, ops/llm_elementwise.metal:388-407).
__device__ __forceinline__ float gelu_tanh(float x) {
  const float t = tanhf(0.7978845608028654f * (x + 0.044715f * x * x * x));
  return 0.5f * x * (1.0f + t);
}

// What a GEMV does with a row's f32 sum: the reference's fused decode stores (VPQ_EPILOGUE_*;
// affine_qmv.metal:265-283,347-363,405-516,806-906,1352-1448). Called by lanes 0..15 of a warp,
// lane = row within the 16-row tile; the gated stores pair lanes 2j, 2j + 1.
enum : int { kEpiNone = 0, kEpiAdd = 1, kEpiSwiglu = 2, kEpiQkv = 3, kEpiGeglu = 4, kEpiGeluMul = 5, kEpiSiluMul = 6 };

// A residual or multiplier may have been written by another SM earlier in the same launch (a chain of
// dependent GEMVs over buffers that the layers reuse), so it is read past L1.
__device__ __forceinline__ uint32_t ld_cg_u16(const uint16_t* p) {
  uint16_t r;
  asm volatile("ld.global.cg.u16 %0, [%1];" : "=h"(r) : "l"(p) : "memory");
  return r;
}

// `mask` names the lanes that make the call together (the gated stores shuffle among them).
__device__ __forceinline__ void fused_store(int epi, float v, int row, int N, int lane, __nv_bfloat16* y,
                                            const uint16_t* aux, __nv_bfloat16* y3, int q_rows, int k_rows,
                                            unsigned mask = 0x0000ffffu) {
  if (epi == kEpiNone) {
    if (row < N) { y[row] = __float2bfloat16_rn(v); }
  } else if (epi == kEpiAdd) {
    // the sum is rounded to bf16 first, then added to the residual in bf16, as the reference does
    if (row < N) {
      const float r = __uint_as_float(ld_cg_u16(aux + row) << 16);
      y[row] = __float2bfloat16_rn(__bfloat162float(__float2bfloat16_rn(v)) + r);
    }
  } else if (epi == kEpiSwiglu) {
    // rows 2j, 2j+1 are gate j, up j: one output silu(gate) * up from the unrounded sums
    const float up = __shfl_down_sync(mask, v, 1);
    if ((lane & 1) == 0 && row + 1 < N) { y[row >> 1] = __float2bfloat16_rn(v / (1.0f + expf(-v)) * up); }
  } else if (epi == kEpiGeglu) {
    // as above with the tanh form of gelu on the gate
    const float up = __shfl_down_sync(mask, v, 1);
    if ((lane & 1) == 0 && row + 1 < N) { y[row >> 1] = __float2bfloat16_rn(gelu_tanh(v) * up); }
  } else if (epi == kEpiGeluMul) {
    // gelu of the bf16-rounded sum, times the multiplier: what a separate pass over y would compute
    if (row < N) {
      const float m = __uint_as_float(ld_cg_u16(aux + row) << 16);
      y[row] = __float2bfloat16_rn(gelu_tanh(__bfloat162float(__float2bfloat16_rn(v))) * m);
    }
  } else if (epi == kEpiSiluMul) {
    // silu of the unrounded sum, times the multiplier (the up projection of a split-width SwiGLU)
    if (row < N) {
      const float m = __uint_as_float(ld_cg_u16(aux + row) << 16);
      y[row] = __float2bfloat16_rn(v / (1.0f + expf(-v)) * m);
    }
  } else {
    const int qk = q_rows + k_rows;
    if (row < q_rows) {
      y[row] = __float2bfloat16_rn(v);
    } else if (row < qk) {
      reinterpret_cast<__nv_bfloat16*>(const_cast<uint16_t*>(aux))[row - q_rows] = __float2bfloat16_rn(v);
    } else if (row < N) {
      y3[row - qk] = __float2bfloat16_rn(v);
    }
  }
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
