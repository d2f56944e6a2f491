/* vpq_oracle.h -- CPU restatement of vpipe's 4-bit affine group-quantized linear.
 *
 * TEST INFRASTRUCTURE ONLY. This is the checker the CUDA path is compared
 * against and the timed CPU baseline; it is never linked into, called from or
 * used as a fallback by the shipped library.
 *
 * Every function cites the reference source (path inside tgo-app-dev/vpipe)
 * whose arithmetic it restates. Parity status: the quantize / dequantize
 * functions are pinned bit-for-bit against the reference's own shader source
 * compiled as C++ (oracle/_ref, built by oracle/Makefile); QMV / QMM follow
 * the reference's CPU test oracles (fp32 dequantise-then-matmul). Rounding
 * behaviour of Apple GPU hardware itself is unpinned: the contract is the
 * IEEE semantics of the shader source.
 *
 * Layout (all row-major):
 *   codes  u32 [N, K/8]   nibble i of word j of row n is k = 8j+i, low first
 *   scales     [N, K/64]  f16 on disk, bf16 after load
 *   biases     [N, K/64]  the affine zero point (group minimum), same types
 *   x      bf16 [M, K],  y bf16 [M, N]
 * 16-bit floats are passed as raw uint16_t bit patterns.
 */
#ifndef VPQ_ORACLE_H
#define VPQ_ORACLE_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* scalar conversions */
uint16_t vpq_o_f32_to_bf16(float f);      /* model-quantizer.cc:56-60 (integer RNE form) */
float    vpq_o_bf16_to_f32(uint16_t b);
uint16_t vpq_o_f32_to_f16(float f);       /* IEEE RNE, the MSL (half) cast */
float    vpq_o_f16_to_f32(uint16_t h);

/* F32 checkpoint tensor -> BF16 before quantizing. model-quantizer.cc:48-62 */
void vpq_o_narrow_f32_bf16(const float* src, uint16_t* dst, size_t n);

/* On-disk F16 scales/biases -> bf16 at load (RNE through f32).
 * flux2/metal-flux2-transformer.cc:55-58,84-86 ; qwen3/metal-qwen-model.cc:203-213 */
void vpq_o_f16_to_bf16(const uint16_t* src, uint16_t* dst, size_t n);

/* Forward quantizer, one (row, group) at a time exactly as the shader does.
 * gpu-kernels/metal/quant/affine_dequant.metal:243-301 (affine_quant_impl<4,64>)
 * w_elt: [N,K] f16 (src_is_bf16=0) or bf16 (src_is_bf16=1) bit patterns.
 * Returns 0, or -1 on bad arguments (K % 64 != 0, N <= 0), mirroring
 * AffineQuantizer::quantize_linear's checks (affine-quantizer.cc:57). */
int vpq_o_quant_w4_g64(const uint16_t* w_elt, int src_is_bf16, uint32_t* codes,
                       uint16_t* scales_f16, uint16_t* biases_f16,
                       int K, int N, float clip);

/* Dequantize to bf16: bf16_rne(float(s)*float(q) + float(b)).
 * gpu-kernels/metal/quant/affine_dequant.metal:25-58 */
/* Any of the reference's (bits, group) pairs: (4|8, 64|32). */
int vpq_o_quant(const uint16_t* w_elt, int src_is_bf16, uint32_t* codes, uint16_t* scales_f16,
                uint16_t* biases_f16, int K, int N, int bits, int group, float clip);
int vpq_o_dequant_bf16(const uint32_t* codes, const uint16_t* s_bf16, const uint16_t* b_bf16,
                       uint16_t* out_bf16, int K, int N, int bits, int group);
void vpq_o_dequant_w4g64_bf16(const uint32_t* codes, const uint16_t* s_bf16,
                              const uint16_t* b_bf16, uint16_t* out_bf16,
                              int K, int N);

/* Dequantize to f32 without the bf16 rounding: deq = s*v + b.
 * tests/unit-tests/metal-compute-gemm-mma.cc:253-288 (make_qweight) ;
 * generative-models/quantize/model-quantizer.cc:252-258 */
void vpq_o_dequant_w4g64_f32(const uint32_t* codes, const uint16_t* s_bf16,
                             const uint16_t* b_bf16, float* out_f32,
                             int K, int N);

/* fp32 dequantise-then-matmul reference, sequential f32 accumulate over k:
 * y_f32[m,n] = sum_k float(x[m,k]) * deq[n,k].
 * tests/unit-tests/metal-compute-gemm-mma.cc:337-347,441-451 */
void vpq_o_matmul_f32_seq(const uint16_t* x_bf16, const float* deq,
                          float* y_f32, int M, int N, int K);

/* Same contraction with a double accumulator.
 * tests/unit-tests/metal-lm/quant-gemv.cc:255-265 */
void vpq_o_matmul_f64(const uint16_t* x_bf16, const float* deq,
                      double* y_f64, int M, int N, int K);

/* Same contraction, f32 accumulate, blocked and multithreaded (OpenMP). The
 * summation order differs from _seq (8 interleaved partial sums per output),
 * so results agree with it to f32 rounding noise only. Used for the larger
 * parity cases and as the timed CPU baseline. threads <= 0: all cores. */
void vpq_o_matmul_f32_fast(const uint16_t* x_bf16, const float* deq,
                           float* y_f32, int M, int N, int K, int threads);

/* Restatement of the reference QMV kernel's own arithmetic order
 * (qmv_fast_impl<T,64,4,false,4,2,2>): 32 lanes x 16 values per 512-k block,
 * x pre-divided by 1/16/256/4096 against unshifted nibble masks, per lane
 * chunk scale*sum(x*q) + bias*sum(x) in f32 where the 4-term sum(x) partial is
 * formed in the storage type on full blocks, butterfly lane reduction, one
 * rounding to bf16. gpu-kernels/metal/quant/affine_qmv.metal:57-111,151-174,186-284 */
void vpq_o_qmv_kernel_order(const uint32_t* codes, const uint16_t* s_bf16,
                            const uint16_t* b_bf16, const uint16_t* x_bf16,
                            uint16_t* y_bf16, int K, int N, int M);

/* Restatement of the reference QMM numerics: W rounded to bf16 before the
 * multiply, f32 accumulate, one rounding at store.
 * gpu-kernels/metal/quant/affine_qmm_steel.metal:78-96,231-242,401-455 */
void vpq_o_qmm_kernel_numerics(const uint32_t* codes, const uint16_t* s_bf16,
                               const uint16_t* b_bf16, const uint16_t* x_bf16,
                               uint16_t* y_bf16, int K, int N, int M, int threads);

/* Output byte sizes. generative-models/quantize/affine-quantizer.h:37-40 */
size_t vpq_o_weight_bytes(int N, int K, int bits);
size_t vpq_o_scale_bytes(int N, int K, int group);

/* Timed CPU baseline: dequantise (reference f32 routine) then fp32 GEMM then
 * bf16 store, all host cores. Returns seconds of wall time for the call. */
double vpq_o_cpu_linear(const uint32_t* codes, const uint16_t* s_bf16,
                        const uint16_t* b_bf16, const uint16_t* x_bf16,
                        uint16_t* y_bf16, float* deq_scratch,
                        int K, int N, int M, int threads);

int vpq_o_max_threads(void);

#ifdef __cplusplus
}
#endif
#endif
