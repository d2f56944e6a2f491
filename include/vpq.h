/* vpq.h -- C ABI of the B200 (sm_100a) 4-bit affine group-quantized linear.
 *
 * Drop-in boundary for the one operator family vpipe (tgo-app-dev/vpipe)
 * dispatches for every quantized Linear: the weight-only int4, group-64
 * affine QMV (decode) / QMM (prefill, DiT), its dequantizer and its forward
 * quantizer. The reference reaches these through its metal-compute kernel
 * calling convention (bind buffer slots, set int constants, dispatch); each
 * entry point below takes exactly those slots as plain device pointers and
 * sizes, and cites the reference interface it replaces.
 *
 * Conventions (all entry points)
 *  - Pointers are CUDA device pointers unless a name ends in _host. The caller
 *    owns every buffer; nothing here allocates, frees or synchronises unless
 *    stated. Work is enqueued on `stream` (a cudaStream_t passed as void*; NULL
 *    is the legacy default stream) and is asynchronous, like an encoded but
 *    uncommitted Metal dispatch (apple-silicon/metal-compute/compute-encoder.h:188,
 *    command-stream.h:144).
 *  - Layout, row-major:  w u32 [N, K/8]  (nibble i of word j of row n is
 *    k = 8j+i, low nibble first);  scales, biases [N, K/64]  (biases is the
 *    affine zero point, not a Linear bias);  x [M, K];  y [M, N].
 *    gpu-kernels/metal/quant/affine_qmv.metal:8-26, affine_dequant.metal:46-47.
 *  - 16-bit floats are raw bit patterns (bf16 unless stated f16).
 *  - Return value: VPQ_OK or an error code; nothing is launched on error and
 *    vpq_last_error() gives a message. There is no CPU fallback: on a machine
 *    without a usable sm_100 device the compute entry points return
 *    VPQ_ERR_CUDA. The reference signals the same conditions with
 *    valid()==false / bool returns (compute-library.h:134, affine-quantizer.cc:57).
 *  - Alignment: w and x must be 16-byte aligned (the GEMMs also want y so); scales, biases and a
 *    GEMV's y need 2 bytes only, but scales / biases ride on TMA (faster) when 16-byte aligned with
 *    K % 512 == 0. K % 64 == 0. Violations return VPQ_ERR_ALIGNMENT.
 */
#ifndef VPQ_H
#define VPQ_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define VPQ_VERSION 100

typedef enum vpq_status {
  VPQ_OK = 0,
  VPQ_ERR_INVALID_ARG = 1, /* null pointer, non-positive size, K % 64 != 0 ...   */
  VPQ_ERR_ALIGNMENT = 2,   /* a pointer is not 16-byte aligned                    */
  VPQ_ERR_UNSUPPORTED = 3, /* shape outside what the kernel handles               */
  VPQ_ERR_CUDA = 4,        /* CUDA runtime / driver error, or no sm_100 device    */
  VPQ_ERR_NCCL = 5,        /* NCCL missing or returned an error                   */
  VPQ_ERR_TIMEOUT = 6,     /* a bounded device-side wait gave up                  */
  VPQ_ERR_NOT_FOUND = 7    /* vpq_function(): unknown (library, entry) pair       */
} vpq_status;

int vpq_version(void);
const char* vpq_status_string(int status);
/* Message for the calling thread's most recent failing call ("" if none). */
const char* vpq_last_error(void);

/* Byte sizes of the quantizer's three outputs.
 * Replaces AffineQuantizer::weight_bytes / scale_bytes,
 * generative-models/quantize/affine-quantizer.h:37-40. */
size_t vpq_weight_bytes(int N, int K, int bits);
size_t vpq_scale_bytes(int N, int K, int group);

/* Forward quantizer: dense W[N,K] (f16 or bf16) -> codes u32 [N,K/8],
 * scales f16 [N,K/64], biases f16 [N,K/64]; clip 1.0 = plain min/max.
 * Bit-exact with the reference shader.
 * Replaces kernel affine_quant_w4_g64 (slots 0:x 1:w 2:s 3:b 4:K 5:N 6:clip),
 * gpu-kernels/metal/quant/affine_dequant.metal:243-301, and the dispatch in
 * AffineQuantizer::quantize_linear, generative-models/quantize/affine-quantizer.cc:52-84. */
int vpq_affine_quant_w4_g64(const void* w_elt, int src_is_bf16, uint32_t* codes,
                            void* scales_f16, void* biases_f16,
                            int64_t K, int64_t N, float clip, void* stream);

/* FP32 checkpoint tensor -> BF16 (round to nearest even) before quantizing.
 * Replaces narrow_f32_bf16_, generative-models/quantize/model-quantizer.cc:48-62. */
int vpq_narrow_f32_bf16(const float* src, void* dst_bf16, int64_t n, void* stream);

/* On-disk F16 scales / biases -> bf16 at load (RNE through f32).
 * Replaces the F16 branch of to_f16_, generative-models/flux2/metal-flux2-transformer.cc:65-91
 * (same conversion in generative-models/qwen3/metal-qwen-model.cc:203-213). */
int vpq_scales_f16_to_bf16(const void* src_f16, void* dst_bf16, int64_t n, void* stream);

/* The quantizer and dequantizer for the format twins the reference's mixed-precision and
 * GGUF-repacked checkpoints use: bits 4 or 8, group 64 or 32 (codes u32 [N, K*bits/32], 8-bit
 * codes one byte per value, little-endian in the word; scales / biases [N, K/group]). Bit-exact
 * with kernels affine_quant_w8_g64 / _w4_g64 / _w8_g32 / _w4_g32 and affine_dequant_w4g64 / _w8g64
 * / _w8g32 / _w4g32, gpu-kernels/metal/quant/affine_dequant.metal:25-135,191-225,243-301; validated as
 * AffineQuantizer::quantize_linear does, generative-models/quantize/affine-quantizer.cc:55-57.
 * Besides w4 g64 the library has a fused GEMV and GEMM for w8 g64 (vpq_affine_qmv_w8g64_bf16,
 * vpq_affine_qmm_w8g64_bf16) and a fused GEMV for w4 g32 (vpq_affine_qmv_w4g32_bf16); the remaining
 * combinations are dequantised once and multiplied densely, as the reference itself does for its codec weights
 * (affine_dequant.metal:100-106). */
int vpq_affine_quant(const void* w_elt, int src_is_bf16, uint32_t* codes, void* scales_f16, void* biases_f16,
                     int64_t K, int64_t N, int bits, int group, float clip, void* stream);
int vpq_affine_dequant_bf16(const uint32_t* w, const void* scales, const void* biases, void* ydeq, int64_t K,
                            int64_t N, int bits, int group, void* stream);

/* 8-bit group-64 weights requantised to 4 bits (the draft copy of a vocabulary matrix that a
 * speculative head reads at half the bandwidth): per group of 64, v = s8 * q8 + b8 in f32,
 * s4 = (max v - min v) / 15, b4 = min v, q4 = clamp(round((v - min v) / s4), 0, 15) computed with the
 * f32 scale, scales and biases then narrowed to bf16. w8 u32 [N, K/4] -> w4 u32 [N, K/8]; s8, b8, s4, b4
 * bf16 [N, K/64]; slots 0..5 in this order, K and N as constants. Replaces affine_requant_w8_to_w4_g64
 * (gpu-kernels/metal/quant/affine_dequant.metal:135-189). Division and reciprocal are IEEE-rounded;
 * the reference's are Metal's, which no test of the reference pins. */
int vpq_affine_requant_w8_to_w4_g64_bf16(const uint32_t* w8, const void* s8, const void* b8, uint32_t* w4, void* s4,
                                         void* b4, int64_t K, int64_t N, void* stream);

/* Dequantize to dense bf16 [N,K]: bf16_rne(float(s)*q + float(b)). Bit-exact.
 * Replaces kernel affine_dequant_w4g64 (slots 0:w 1:scales 2:biases 3:ydeq 4:K 5:N),
 * gpu-kernels/metal/quant/affine_dequant.metal:25-58. */
int vpq_affine_dequant_w4g64_bf16(const uint32_t* w, const void* scales, const void* biases,
                                  void* ydeq, int64_t K, int64_t N, void* stream);

/* Decode GEMV: y[m,n] = sum_k x[m,k] * (s*q + b), f32 accumulate, bf16 out.
 * Every row m streams the whole weight again, as in the reference; meant for
 * M = 1 (small M works, M >= 16 belongs to vpq_affine_qmm_w4g64_bf16).
 * K <= 32768. Replaces kernel affine_qmv_w4g64 in library affine_qmv_bf16
 * (slots 0:w 1:scales 2:biases 3:x 4:y 5:K 6:N; M from the dispatch grid),
 * gpu-kernels/metal/quant/affine_qmv.metal:286-301, dispatched at
 * generative-models/qwen3/metal-qwen-model.cc:3033-3048. */
int vpq_affine_qmv_w4g64_bf16(const uint32_t* w, const void* scales, const void* biases,
                              const void* x, void* y, int64_t K, int64_t N, int64_t M,
                              void* stream);

/* The fused decode GEMVs as single calls (see VPQ_EPILOGUE_* below for the arithmetic).
 * _add: slot 7 of the reference kernel is `residual` [M, N]. _swiglu: N = 2 * ffn, y is [M, N/2].
 * _qkv: slots 4..6 of the reference kernel are the three outputs, 8..10 the row counts. */
int vpq_affine_qmv_w4g64_bf16_add(const uint32_t* w, const void* scales, const void* biases, const void* x,
                                  void* y, int64_t K, int64_t N, int64_t M, const void* residual,
                                  void* stream);
int vpq_affine_qmv_swiglu_w4g64_bf16(const uint32_t* w, const void* scales, const void* biases, const void* x,
                                     void* y, int64_t K, int64_t N, int64_t M, void* stream);
int vpq_affine_qmv_qkv_w4g64_bf16(const uint32_t* w, const void* scales, const void* biases, const void* x,
                                  void* q_out, void* k_out, void* v_out, int64_t K, int64_t q_rows,
                                  int64_t k_rows, int64_t v_rows, int64_t M, void* stream);
/* _geglu: as _swiglu with gelu_pytorch_tanh on the gate (affine_qmv_geglu_w4g64,
 * gpu-kernels/metal/quant/affine_qmv.metal:1352-1448). _gelu_mul: slot 7 of the reference kernel is
 * `mul` [M, N]; y = gelu(bf16(sum)) * mul (affine_qmv_gelu_mul_w4g64, affine_qmv.metal:265-283,745-765). */
int vpq_affine_qmv_geglu_w4g64_bf16(const uint32_t* w, const void* scales, const void* biases, const void* x,
                                    void* y, int64_t K, int64_t N, int64_t M, void* stream);
int vpq_affine_qmv_gelu_mul_w4g64_bf16(const uint32_t* w, const void* scales, const void* biases, const void* x,
                                       void* y, int64_t K, int64_t N, int64_t M, const void* mul,
                                       void* stream);

/* Decode GEMV over 8-bit group-64 weights (w u32 [N, K/4], one byte per value): the 8-bit linears
 * of mixed-precision checkpoints. Exact integer tensor-core arithmetic as the 4-bit kernel, with
 * no unpacking at all. K <= 16384. Replaces affine_qmv_w8g64 (slots as affine_qmv_w4g64),
 * gpu-kernels/metal/quant/affine_qmv.metal:186-301,3027-3070. */
int vpq_affine_qmv_w8g64_bf16(const uint32_t* w, const void* scales, const void* biases, const void* x,
                              void* y, int64_t K, int64_t N, int64_t M, void* stream);

/* Decode GEMV over 4-bit group-32 weights (scales / biases [N, K/32]): GGUF Q4_0 repacks. The
 * small-batch kernel with the accumulator columns = (row of x, group 0..3 of a 128-k tile): up to
 * two rows of x share one stream of the weights. K % 32 == 0, K <= 32768. Replaces affine_qmv_w4g32
 * (slots as affine_qmv_w4g64), gpu-kernels/metal/quant/affine_qmv.metal:303-320. */
int vpq_affine_qmv_w4g32_bf16(const uint32_t* w, const void* scales, const void* biases, const void* x,
                              void* y, int64_t K, int64_t N, int64_t M, void* stream);

/* Small-batch decode GEMV: the M rows of x (M = 2..8: decode of several branches, MTP verify)
 * share ONE stream of the weights, up to 4 rows per pass (4 up to K = 5120, 2 up to K = 8192: the
 * rows live in shared memory; longer rows, and a single left-over row, run on the M = 1 kernel). fp16 tensor-core arithmetic with exact products and f32 accumulation; the rows agree
 * with vpq_affine_qmv_w4g64_bf16 to f32 rounding, not bit for bit (the reference's batched rows
 * are bit-identical to its M = 1 kernel). Replaces affine_qmv_batch_w4g64 / affine_qmv_batch4_w4g64
 * (slots as QMV, 7: total rows), gpu-kernels/metal/quant/affine_qmv.metal:1553-1705. */
int vpq_affine_qmv_batch_w4g64_bf16(const uint32_t* w, const void* scales, const void* biases, const void* x,
                                    void* y, int64_t K, int64_t N, int64_t M, void* stream);

/* A set of independent GEMVs enqueued back to back (one launch each, in order),
 * e.g. the q | k | v or gate | up projections of one decoder layer. descs_host
 * is a host array read during the call. Each launch opts into programmatic
 * dependent launch, so the weight stream of launch i+1 starts while launch i
 * drains. Replaces ComputeEncoder::concurrent_scope around the per-projection
 * dispatches, apple-silicon/metal-compute/compute-encoder.h:156-181, as used in
 * encode_decode_step_, generative-models/qwen3/metal-qwen-model.cc:3004-3074. */
typedef struct vpq_linear_desc {
  const uint32_t* w;
  const void* scales;
  const void* biases;
  const void* x;
  void* y;
  int64_t K, N, M;
  /* Fused store, VPQ_EPILOGUE_*; zero-initialised descriptors store y = x W^T as is. */
  int32_t epilogue;
  int32_t depends;      /* plans only: 1 = this GEMV reads (x, residual) what GEMVs earlier in the list write */
  const void* aux;      /* ADD: residual [M, N]; GELU_MUL, SILU_MUL: multiplier [M, N]; QKV: the k output [M, k_rows] (written) */
  void* y3;             /* QKV: the v output [M, N - q_rows - k_rows] */
  int64_t q_rows, k_rows;
  /* RMSNorm prologue (w4 g64 GEMV only): with norm_w [K] (bf16, 16-byte aligned) every row of x is
   * replaced, while it is staged on chip, by bf16(x * rsqrt(mean(x^2) + eps) * norm_w); the normed row
   * never touches device memory. Replaces affine_qmv_qkv_rms_w4g64 (slot 4 = norm_w, 12 = eps),
   * gpu-kernels/metal/quant/affine_qmv.metal:570-694; works with every store, not only QKV. */
  const void* norm_w;
  /* Expert gather (w4 g64 GEMV only): w / scales / biases are `experts` slabs [experts, N, ..] and row
   * m (a (token, expert) pair) multiplies slab expert[m], an index the GPU reads when the kernel runs
   * (the router's output never visits the host). Row m reads x row m / x_div (x_div = top_k for the
   * gate|up GEMV, whose pairs of one token share its row; 0 or 1: row m) and writes y row m.
   * Replaces affine_gather_qmv_swiglu_w4g64, affine_gather_qmv_geglu_w4g64 and
   * affine_gather_down_qmv_w4g64 (slot 7 = pair_eid, 8 = top_k), affine_qmv.metal:908-955,1262-1291,1488-1521. */
  const int32_t* expert;
  int64_t experts;
  int32_t x_div;
  float eps;
  /* Sorted-slot form of the expert gather (the 4- and 8-bit GEMVs): the M rows are slots of (token,
   * expert) pairs sorted by expert and padded per expert to tiles of expert_div slots. row_map [M]
   * (device int32) is the reference's srow: slot m is live iff row_map[m] >= 0, and also only if its
   * tile's expert is >= 0; a dead slot's y row is not written. With row_gather = 1 slot m reads x row
   * row_map[m] (the gate|up GEMV, which gathers from the hidden states), with 0 it reads x row m (the
   * down GEMV over the sorted activations). Slot m multiplies slab expert[m / expert_div] (expert is then
   * the reference's tile2e; 0 or 1: expert[m]). Replaces affine_grouped_swiglu_w4g64, affine_grouped_down_w4g64
   * and their _w8g64 twins (slot 7 = srow, 8 = tile2e; tiles of 2 slots), gpu-kernels/metal/quant/
   * affine_qmv.metal:2551-2719. Every live slot is one GEMV over its expert's slab here (the reference
   * shares one weight read between the two slots of a tile). */
  const int32_t* row_map;
  int32_t row_gather;
  int32_t expert_div;
} vpq_linear_desc;

/* What the GEMV does with each row's f32 sum (the reference's fused decode kernels):
 * ADD     y[n] = bf16(bf16(sum) + residual[n])                  affine_qmv_w4g64_add,
 *         gpu-kernels/metal/quant/affine_qmv.metal:265-270,347-363 (o_proj / down_proj + residual)
 * SWIGLU  W rows interleaved (2j = gate j, 2j+1 = up j), N = 2 ffn, y is [M, N/2]:
 *         y[j] = bf16(silu(sum[2j]) * sum[2j+1]), from the unrounded sums    affine_qmv_swiglu_w4g64,
 *         affine_qmv.metal:806-906
 * QKV     W is q | k | v row-concatenated; rows land in three buffers: y (q), aux (k), y3 (v)
 *         affine_qmv_qkv_w4g64, affine_qmv.metal:405-516
 * GEGLU   as SWIGLU with gelu(g) = 0.5 g (1 + tanh(sqrt(2/pi) (g + 0.044715 g^3))) on the gate
 *         affine_qmv_geglu_w4g64, affine_qmv.metal:1352-1448
 * GELU_MUL y[n] = bf16(gelu(bf16(sum)) * mul[n])                 affine_qmv_gelu_mul_w4g64,
 *         affine_qmv.metal:265-283,745-765 (Gemma per-layer-input gate)
 * SILU_MUL y[n] = bf16(silu(sum) * mul[n]), mul [M, N] in aux (may be y itself: each element is read, then
 *         written, by one thread). The second half of a SwiGLU whose gate and up matrices are separate and of
 *         different widths: run the up GEMV into y, then the gate GEMV with this store and aux = y
 *         (affine_gather_qmv_swiglu_w4w8g64 / _w8w4g64, affine_qmv.metal:1153-1259; up reaches the product
 *         rounded to bf16 here, unrounded there) */
enum {
  VPQ_EPILOGUE_NONE = 0,
  VPQ_EPILOGUE_ADD = 1,
  VPQ_EPILOGUE_SWIGLU = 2,
  VPQ_EPILOGUE_QKV = 3,
  VPQ_EPILOGUE_GEGLU = 4,
  VPQ_EPILOGUE_GELU_MUL = 5,
  VPQ_EPILOGUE_SILU_MUL = 6
};
int vpq_affine_qmv_w4g64_bf16_batch(const vpq_linear_desc* descs_host, int count, void* stream);

/* The 8-bit GEMV with a fused store: one descriptor (w u32 [N, K/4]), any VPQ_EPILOGUE_*. Replaces
 * affine_qmv_w8g64_add, affine_qmv_swiglu_w8g64, affine_qmv_qkv_w8g64 and affine_qmv_gelu_mul_w8g64
 * (the 8-bit instantiations of the kernels cited above, gpu-kernels/metal/quant/affine_qmv.metal:
 * 540-560,789-805,3122-3160), affine_qmv_geglu_w8g64, and, with expert / experts / x_div set as for the
 * 4-bit GEMV (w then holds the experts' slabs, u32 [experts * N, K/4]), the 8-bit expert-gather GEMVs
 * affine_gather_qmv_swiglu_w8g64, affine_gather_qmv_geglu_w8g64 and affine_gather_down_qmv_w8g64
 * (affine_qmv.metal:957-994,1290-1322,1519-1548). norm_w and depends are not taken. */
int vpq_affine_qmv_w8g64_bf16_fused(const vpq_linear_desc* desc_host, void* stream);

/* The same GEMV over 8-bit weights in groups of 32 (scales / biases [N, K/32], K % 32 == 0): the 8-bit
 * layers of GGUF repacks. One descriptor, any VPQ_EPILOGUE_*, norm_w and the expert gather as above.
 * Replaces affine_qmv_w8g32 (gpu-kernels/metal/quant/affine_qmv.metal:3050-3066). */
int vpq_affine_qmv_w8g32_bf16_fused(const vpq_linear_desc* desc_host, void* stream);

/* The shared-expert gate of a mixture-of-experts block: out[m] = sigmoid(dequant(w) . x[m]) for ONE
 * 8-bit group-64 weight row (w u32 [K/4], scales / biases [K/64]) and M rows of x; out bf16 [M].
 * Slots 0..4 = w, scales, biases, x, out; K as a constant. Replaces affine_moe_gate_w8g64
 * (gpu-kernels/metal/quant/affine_qmv.metal:1323-1347). x must be 8-byte aligned. */
int vpq_affine_moe_gate_w8g64_bf16(const uint32_t* w, const void* scales, const void* biases, const void* x,
                                   void* out, int64_t K, int64_t M, void* stream);

/* The small-batch GEMV (w4 g64, rows of x share one stream of the weights) and the group-32 GEMV with
 * a fused store: one descriptor, any VPQ_EPILOGUE_*. Replace affine_qmv_batch_swiglu_w4g64,
 * affine_qmv_w4g32_add, affine_qmv_geglu_w4g32, affine_qmv_gelu_mul_w4g32
 * (gpu-kernels/metal/quant/affine_qmv.metal:367-385,770-787,1451-1470,2871). */
int vpq_affine_qmv_batch_w4g64_bf16_fused(const vpq_linear_desc* desc_host, void* stream);
int vpq_affine_qmv_w4g32_bf16_fused(const vpq_linear_desc* desc_host, void* stream);

/* The scale-only group-32 GEMV for GGUF Q4_0 repacks: every group's bias is -8 * its scale (exact in
 * bf16), so the biases are neither passed nor read (desc->biases is ignored and may be null): one
 * ninth less weight traffic. Results are bit-identical to vpq_affine_qmv_w4g32_bf16_fused given
 * biases = -8 * scales. Any VPQ_EPILOGUE_*. Replaces affine_qmv_w4g32_q40, affine_qmv_w4g32_add_q40
 * and affine_qmv_geglu_w4g32_q40 (gpu-kernels/metal/quant/affine_qmv.metal:322-341,384-403,1472-1487). */
int vpq_affine_qmv_w4g32_q40_bf16_fused(const vpq_linear_desc* desc_host, void* stream);

/* A list of independent GEMVs run as ONE launch: the kernel walks the row tiles of all problems
 * back to back, so there is no launch gap and no per-problem ramp-up, and problems that read the
 * same x (q | k | v, gate | up) stage it once. "Encode once, commit many": the analogue of
 * encoding a decode step's dispatches into one command buffer and re-committing it,
 * apple-silicon/metal-compute/command-stream.h:144, generative-models/qwen3/metal-qwen-model.cc:3004-3074.
 * Descriptors with depends == 0 must be independent of each other (none reads another's y). A
 * descriptor with depends == 1 may read (x, residual) what ANY earlier descriptor of the list
 * writes: the list then runs as a dependent chain inside one cooperative launch -- every GEMV is
 * spread over the whole grid, a counter in the workspace counts finished tiles, and a dependent
 * GEMV stages its x only when everything before it is complete, while its weights are already
 * streaming. That is a whole decode step between two attention calls as one launch: o_proj +
 * residual -> norm + gate|up (SwiGLU) -> down + residual -> norm + q|k|v; bit-identical to one
 * launch per GEMV. An expert index array (`expert`) must be complete before the launch. Pointers
 * are captured at creation, their contents may change between runs. `workspace` is caller-owned device memory
 * of vpq_qmv_plan_bytes() bytes holding the per-problem descriptors; it must outlive the plan.
 * vpq_qmv_plan_create copies into it and synchronises `stream`; vpq_qmv_plan_run only launches.
 * A large list of independent GEMVs keeps the last tenth of its row tiles as a pool that the CTAs
 * draw from as they finish (the SMs of a GPU do not stream at one rate); whoever computes a tile,
 * its bytes are the same. The pool's counter and the chain's counters live in the workspace and go
 * back to zero at the end of every run, so runs of one plan must follow one another on the GPU:
 * one stream, or streams ordered by events -- never two runs of the same plan at once. */
typedef struct vpq_qmv_plan_s vpq_qmv_plan;
size_t vpq_qmv_plan_bytes(const vpq_linear_desc* descs_host, int count);
int vpq_qmv_plan_create(const vpq_linear_desc* descs_host, int count, void* workspace, size_t bytes,
                        void* stream, vpq_qmv_plan** out);
int vpq_qmv_plan_run(const vpq_qmv_plan* plan, void* stream);
int vpq_qmv_plan_destroy(vpq_qmv_plan* plan);

/* The same one-launch set of independent GEMVs for callers that must not allocate device memory
 * and have no workspace to lend: code running inside someone else's memory budget (a host
 * application whose allocator owns every byte of HBM, a plugin entry point that is handed
 * buffers and nothing else) or on a latency path where a cudaMalloc, which can synchronise the
 * whole device, is not acceptable. No counterpart in the reference. The descriptor list the
 * kernel needs lives in a fixed 40 KB array inside the library image (held by every GPU that
 * loads the library until exit), so at most 64 GEMV rows (sum of M over the set) fit in one call;
 * larger sets are rejected with VPQ_ERR_UNSUPPORTED. The call performs no cudaMalloc / cudaFree
 * and uses no allocating library routine. The first call on each device looks up the array's
 * device address; make that first call outside any stream capture. All calls share the one
 * array: a call rewrites every descriptor it uses (nothing is read from a previous call), but
 * two calls that overlap on the GPU (different streams) race on it -- keep calls to this entry
 * point ordered on one stream per device. The call cannot be recorded into a CUDA graph: its
 * descriptors are copied from the call's stack, so a stream that is being captured is refused with
 * VPQ_ERR_UNSUPPORTED (use vpq_qmv_plan_create / vpq_qmv_plan_run there). */
int vpq_affine_qmv_w4g64_bf16_set_noalloc(const vpq_linear_desc* descs_host, int count, void* stream);

/* Prefill / DiT GEMM: y[M,N] = x[M,K] @ dequant(W)[N,K]^T. W is dequantised
 * to bf16 tile by tile in shared memory (bit-identical to
 * vpq_affine_dequant_w4g64_bf16), multiplied on the tcgen05 tensor cores with
 * f32 accumulation in tensor memory, rounded once to bf16. M and N tails are
 * handled; K % 64 == 0. Replaces kernels affine_qmm_steel_w4g64[_bm64|_bm128]
 * in library affine_qmm_steel_bf16 (slots 0..4 as QMV, 5:K 6:N 7:M),
 * gpu-kernels/metal/quant/affine_qmm_steel.metal:461-561, and
 * affine_qmm_mma_w4g64, gpu-kernels/metal/quant/affine_qmm_mma.metal:50-128;
 * dispatched at generative-models/flux2/metal-flux2-transformer.cc:1291-1330. */
int vpq_affine_qmm_w4g64_bf16(const uint32_t* w, const void* scales, const void* biases,
                              const void* x, void* y, int64_t K, int64_t N, int64_t M,
                              void* stream);

/* Fused SwiGLU GEMM: W rows interleaved by output feature (row 2j = gate j, row 2j+1 = up j),
 * N = 2 * ffn; y[M, N/2] = bf16(silu(x.gate_j) * (x.up_j)) computed in f32 from the accumulators,
 * so the [M, N] intermediate is never written. Replaces affine_qmm_swiglu_w4g64[_bm64|_bm128]
 * (same slots as the GEMM, y half as wide), gpu-kernels/metal/quant/affine_qmm_steel.metal:641-850;
 * unlike those, any even N is accepted (tails are masked). */
int vpq_affine_qmm_swiglu_w4g64_bf16(const uint32_t* w, const void* scales, const void* biases,
                                     const void* x, void* y, int64_t K, int64_t N, int64_t M,
                                     void* stream);

/* GEMM over 8-bit group-64 weights (w u32 [N, K/4]): the same CTA-pair tcgen05 kernel, the W tile
 * dequantised from bytes (bit-identical to vpq_affine_dequant_bf16 at bits 8). Replaces
 * affine_qmm_steel_w8g64[_bm64|_bm128], gpu-kernels/metal/quant/affine_qmm_steel.metal:1595-1675. */
int vpq_affine_qmm_w8g64_bf16(const uint32_t* w, const void* scales, const void* biases, const void* x,
                              void* y, int64_t K, int64_t N, int64_t M, void* stream);

/* q | k | v as ONE GEMM over the row-concatenated weight (the way the reference keeps these three
 * projections, generative-models/qwen3/metal-qwen-model.cc:214-250), with three outputs q [M, q_rows],
 * k [M, k_rows], v [M, v_rows]: narrow k / v projections (N = 1024 in an 8B decoder) alone fill a
 * quarter of the GPU's tiles, together with q they fill it. q_rows and k_rows must be multiples of
 * 128, v_rows of 8 (otherwise run three GEMMs on row slices of w). The prefill counterpart of
 * affine_qmv_qkv_w4g64 (gpu-kernels/metal/quant/affine_qmv.metal:405-516); in the reference prefill
 * runs affine_qmm_steel_w4g64 on the concatenated weight and slices the output afterwards. */
int vpq_affine_qmm_qkv_w4g64_bf16(const uint32_t* w, const void* scales, const void* biases, const void* x,
                                  void* q_out, void* k_out, void* v_out, int64_t K, int64_t q_rows,
                                  int64_t k_rows, int64_t v_rows, int64_t M, void* stream);

/* The GEMM over any of the format twins: bits 4 | 8, group 64 | 32 (scales / biases [N, K/group]), act 0
 * (y [M, N]) or 2 (GeGLU over interleaved gate | up rows, y [M, N/2]; 4-bit only at group 32). The
 * group-32 forms are the same CTA-pair kernel with two scales per 64-wide k block. Replaces
 * affine_qmm_steel_w4g32, affine_qmm_geglu_w4g32 and affine_qmm_steel_w8g32 (slots as the GEMM),
 * gpu-kernels/metal/quant/affine_qmm_steel.metal:618-639,1573-1593,1677-1697. */
int vpq_affine_qmm_bf16(const uint32_t* w, const void* scales, const void* biases, const void* x, void* y,
                        int64_t K, int64_t N, int64_t M, int bits, int group, int act, void* stream);

/* The other gated GEMMs, same slots and layout as the SwiGLU one: gelu_pytorch_tanh on the gate
 * (affine_qmm_geglu_w4g64, gpu-kernels/metal/quant/affine_qmm_steel.metal:1451-1569), and both
 * activations over 8-bit weights (affine_qmm_swiglu_w8g64, :1700-1790; affine_qmm_geglu_w8g64,
 * :1864-1885). */
int vpq_affine_qmm_geglu_w4g64_bf16(const uint32_t* w, const void* scales, const void* biases, const void* x,
                                    void* y, int64_t K, int64_t N, int64_t M, void* stream);
int vpq_affine_qmm_swiglu_w8g64_bf16(const uint32_t* w, const void* scales, const void* biases, const void* x,
                                     void* y, int64_t K, int64_t N, int64_t M, void* stream);
int vpq_affine_qmm_geglu_w8g64_bf16(const uint32_t* w, const void* scales, const void* biases, const void* x,
                                    void* y, int64_t K, int64_t N, int64_t M, void* stream);

/* SwiGLU GEMM writing into a column block of a wider buffer: y[m * out_stride + out_off + j], j in
 * [0, N/2); out_stride 0 means the contiguous N/2 (then out_off must be 0). Lets a block write its
 * MLP activations next to other columns with no concat. bits 4 or 8. Replaces
 * affine_qmm_swiglu_w4g64_bm64_rs / affine_qmm_swiglu_w8g64_bm64_rs (slot 8 = out_stride, 9 = out_off),
 * gpu-kernels/metal/quant/affine_qmm_steel.metal:657-770,920-947,1815-1837. Stores are 16-byte
 * vectors when out_stride, out_off and N/2 are multiples of 8, element-wise otherwise. */
int vpq_affine_qmm_swiglu_bf16_rs(const uint32_t* w, const void* scales, const void* biases, const void* x,
                                  void* y, int64_t K, int64_t N, int64_t M, int bits, int64_t out_stride,
                                  int64_t out_off, void* stream);

/* Grouped (mixture-of-experts) GEMMs for prefill. The (token, expert) pairs are sorted by expert
 * and each expert's block is padded to whole row tiles of vpq_qmm_grouped_tile_rows() rows (128;
 * the reference pads to its BM of 32 / 64): M is the padded row count, tile2e [ceil(M / tile)] the
 * expert of each row tile (negative: an all-padding tile, skipped). w is [experts, N, K/8], scales /
 * biases [experts, N, K/64].
 * _grouped_: the down GEMM. x_sorted [M, K]; row m of the product is stored to row sdst[m] of
 *   y [y_rows, N] (negative: a padding row, not stored; sdst null: y is [M, N] in sorted order).
 *   Replaces affine_qmm_grouped_w4g64 (slots 0:w 1:scales 2:biases 3:x 4:y 5:K 6:N 7:M 8:tile2e
 *   9:sdst), gpu-kernels/metal/quant/affine_qmm_steel.metal:1042-1064,1371-1440.
 * _grouped_swiglu_ / _grouped_geglu_: the gate|up GEMM, rows of w interleaved gate / up, y [M, N/2]
 *   in sorted order. With srow, x is the hidden [x_rows, K] and sorted row m reads row srow[m] of it
 *   (negative: zeros); the reference fuses that gather into its x loader, here it is one pass into
 *   the caller's scratch x_sorted [M, K] ahead of the GEMM, which reads x through TMA. With srow
 *   null, x is already sorted and x_sorted is unused. Replaces affine_qmm_grouped_swiglu_w4g64 /
 *   affine_qmm_grouped_geglu_w4g64 (slot 9 = srow), affine_qmm_steel.metal:1098-1176,1186-1288,1314-1336. */
int vpq_qmm_grouped_tile_rows(void);
int vpq_affine_qmm_grouped_w4g64_bf16(const uint32_t* w, const void* scales, const void* biases,
                                      const void* x_sorted, void* y, int64_t K, int64_t N, int64_t M,
                                      const int* tile2e, const int* sdst, int64_t experts, int64_t y_rows,
                                      void* stream);
int vpq_affine_qmm_grouped_swiglu_w4g64_bf16(const uint32_t* w, const void* scales, const void* biases,
                                             const void* x, void* y, int64_t K, int64_t N, int64_t M,
                                             const int* tile2e, const int* srow, int64_t experts,
                                             int64_t x_rows, void* x_sorted, void* stream);
int vpq_affine_qmm_grouped_geglu_w4g64_bf16(const uint32_t* w, const void* scales, const void* biases,
                                            const void* x, void* y, int64_t K, int64_t N, int64_t M,
                                            const int* tile2e, const int* srow, int64_t experts,
                                            int64_t x_rows, void* x_sorted, void* stream);

/* The grouped GEMMs over 8-bit experts (w u32 [experts * N, K/4]). act 0: the down GEMM (rows_map = sdst,
 * rows = y_rows, x_sorted unused); act 1 / 2: gate|up with the SwiGLU / GeGLU store (rows_map = srow,
 * rows = x_rows, x_sorted the [M, K] scratch), arguments otherwise as for the 4-bit entries above.
 * Replace affine_qmm_grouped_w8g64, affine_qmm_grouped_swiglu_w8g64, affine_qmm_grouped_geglu_w8g64
 * (gpu-kernels/metal/quant/affine_qmm_steel.metal:1069-1094,1341-1367,1290-1312). */
int vpq_affine_qmm_grouped_w8g64_bf16(int act, const uint32_t* w, const void* scales, const void* biases,
                                      const void* x, void* y, int64_t K, int64_t N, int64_t M, const int* tile2e,
                                      const int* rows_map, int64_t experts, int64_t rows, void* x_sorted,
                                      void* stream);

/* Device-side status of the tensor-core kernels: every wait inside them is
 * bounded; one that gives up records where and the kernel returns. Reads the
 * status word of the current device back to the host (synchronises `stream`),
 * clears it, and returns VPQ_OK or VPQ_ERR_TIMEOUT with *detail set to the
 * recorded code. The analogue of Fence::wait_ok(&reason),
 * apple-silicon/metal-compute/command-stream.h:92-99. */
int vpq_device_status(void* stream, uint32_t* detail);

/* Two probes of that reporting path, for tests and bring-up: each makes ONE bounded wait run out
 * on purpose (nothing faults or hangs; the GPU stays usable) so that vpq_device_status can be seen
 * to return VPQ_ERR_TIMEOUT and then clear. No counterpart in the reference beyond the
 * Fence::wait_ok contract cited above.
 * vpq_wait_probe: one thread waits on an mbarrier nobody arrives at, with the kernels' own wait
 *   and `polls` polls of `hint_ns` each (polls <= 65536, hint_ns <= 100000); detail 0x7f7f.
 * vpq_peer_barrier_probe: the cross-GPU flag barrier of the fused column split, run on one GPU
 *   with `workspace` (256 bytes of device memory, 16-byte aligned) standing in for every rank's flag
 *   table and rank `absent_rank` never publishing; the wait ends after max_polls polls of about
 *   100 ns (max_polls <= 2^20); detail 0x20000 | 0x7700 | absent_rank. Synchronises `stream` once. */
int vpq_wait_probe(uint32_t polls, uint32_t hint_ns, void* stream);
int vpq_peer_barrier_probe(void* workspace, int world, int absent_rank, uint32_t max_polls, void* stream);

/* --- calling by the reference's (library, entry) strings ------------------
 * Replaces MetalCompute::load_library(name).function(entry),
 * apple-silicon/metal-compute/metal-compute.h:301, compute-library.h:134.
 * Returns NULL for an unknown pair (the reference returns an invalid handle).
 * Known libraries: affine_qmv_bf16 (entries affine_qmv_w4g64, affine_qmv_w4g64_add,
 * affine_qmv_swiglu_w4g64, affine_qmv_qkv_w4g64, affine_qmv_qkv_rms_w4g64, affine_gather_qmv_swiglu_w4g64,
 * affine_gather_qmv_geglu_w4g64, affine_gather_down_qmv_w4g64, ...), affine_qmm_steel_bf16, affine_qmm_mma_bf16,
 * affine_dequant_bf16, affine_dequant (quantizer, f16 source). */
typedef struct vpq_function_s vpq_function;
const vpq_function* vpq_function_lookup(const char* library, const char* entry);
const char* vpq_function_name(const vpq_function* fn);

/* One dispatch with the reference's slot numbering: buffers[i] is what
 * set_buffer(i, ...) bound (byte offsets already applied), K / N / M / clip are
 * what set_constant bound. The grid is derived from the shapes, so the
 * reference's grid / threadgroup arguments have no counterpart. Slot layouts:
 *   QMV, QMM : 0:w 1:scales 2:biases 3:x 4:y            affine_qmv.metal:19-26
 *   QMV add  : as QMV, 7:residual                       affine_qmv.metal:347-363
 *   QMV / QMM swiglu: as QMV / QMM (N = 2 ffn, y is [M, N/2])   affine_qmv.metal:891-906, affine_qmm_steel.metal:801-827
 *   QMV qkv  : 0:w 1:scales 2:biases 3:x 4:q 5:k 6:v; K, q_rows, k_rows, v_rows   affine_qmv.metal:492-511
 *   QMV norm + qkv: 0:w 1:scales 2:biases 3:x 4:norm_w 5:q 6:k 7:v; K, q_rows, k_rows, v_rows, eps   affine_qmv.metal:671-694
 *   gathered expert QMV (gate|up with swiglu / geglu, down): as QMV, 7:pair_eid; experts, top_k (gate|up)   affine_qmv.metal:928-955,1265-1291
 *   QMM swiglu, strided store: as QMM swiglu; out_stride, out_off (the reference's slots 8, 9)   affine_qmm_steel.metal:925-947
 *   grouped QMM (down): as QMM (x sorted), 8:tile2e 9:sdst; experts, rows = rows of y   affine_qmm_steel.metal:1042-1064
 *   grouped QMM swiglu / geglu: as QMM (x the hidden), 8:tile2e 9:srow 10:scratch [M, K]; experts, rows = rows of x
 *                                                       affine_qmm_steel.metal:1266-1336
 *   dequant  : 0:w 1:scales 2:biases 3:ydeq             affine_dequant.metal:14
 *   quant    : 0:x 1:w 2:scales_f16 3:biases_f16        affine_dequant.metal:288-296
 * Replaces ComputeEncoder::set_function/set_buffer/set_constant/dispatch,
 * apple-silicon/metal-compute/compute-encoder.h:80-83,188. */
typedef struct vpq_dispatch_args {
  const void* buffers[12];
  int64_t K, N, M;
  float clip;
  int64_t q_rows, k_rows, v_rows; /* QMV qkv only */
  int64_t out_stride, out_off;    /* QMM swiglu with a strided store only */
  int64_t experts, rows;          /* grouped QMM / gathered QMV: experts in w; grouped QMM: rows of y (down) or of the hidden (gate|up) */
  int64_t top_k;                  /* gathered gate|up QMV only: pairs per token */
  float eps;                      /* QMV norm + qkv only */
} vpq_dispatch_args;
int vpq_dispatch(const vpq_function* fn, const vpq_dispatch_args* args, void* stream);

/* --- column-split over the GPUs of one box --------------------------------
 * No counterpart in the reference (it is single-GPU). Rank r of `world` owns
 * rows [r*N/world, (r+1)*N/world) of w / scales / biases (contiguous slices of
 * all three arrays), x is replicated, and the ranks' output column blocks are
 * all-gathered with NCCL. NCCL is loaded with dlopen at first use. */
typedef struct vpq_comm_s vpq_comm;
#define VPQ_UNIQUE_ID_BYTES 128
/* Rank 0 fills id (host memory) and ships it to the other ranks by any means. */
int vpq_comm_unique_id(void* id_host);
int vpq_comm_create(const void* id_host, int rank, int world, vpq_comm** out);
int vpq_comm_destroy(vpq_comm* comm);
int vpq_comm_rank(const vpq_comm* comm);
int vpq_comm_world(const vpq_comm* comm);

/* y_shards: device buffer [world, M, N/world] bf16 (shard-major); each rank
 * computes its own block in place and receives the others'. If y_rowmajor is
 * not NULL the gathered blocks are also written as row-major [M, N].
 * N % world == 0. m_chunks >= 1 splits M so that the gather of one chunk
 * overlaps the GEMM of the next (uses two internal streams ordered after and
 * before `stream` with events created at vpq_comm_create). */
int vpq_affine_qmm_w4g64_bf16_nsplit(vpq_comm* comm,
                                     const uint32_t* w_shard, const void* scales_shard,
                                     const void* biases_shard, const void* x,
                                     void* y_shards, void* y_rowmajor,
                                     int64_t K, int64_t N, int64_t M, int m_chunks,
                                     void* stream);

/* Fused form: no separate collective. y lives in a symmetric buffer that every rank has mapped
 * (CUDA IPC, one process per GPU). Each rank's GEMM stores its column block into its own row-major
 * y[M, N]; a few CTAs of the same kernel compute nothing and instead copy every finished tile on to
 * the peers' y over NVLink (TMA load from the local y, TMA stores to the peers) while the tensor
 * cores of the other SMs work on the next tiles; the last tile of every computing CTA pair goes to
 * the peers straight from its epilogue. The handshake between the ranks runs inside the kernel as well:
 *   started  - the kernel announces its start to every peer, and nothing is stored into a peer's y
 *              until that peer has announced its own start, i.e. until
 *              whatever the peer enqueued earlier to read y (the previous step's result) is done;
 *   finished - the CTA whose peer stores complete last on a GPU announces it to every peer, and a small
 *              kernel behind the GEMM on the stream waits for all peers' announcements, so that
 *              later work on the stream finds every column block in y.
 * Ordering is therefore by stream order alone: enqueue the consumers of y after the call and the
 * next call after them, on the same stream, on every rank; no host synchronisation and no second
 * buffer are needed. All ranks must make the same sequence of calls on a communicator. Every wait
 * is bounded; a rank that never shows up ends in VPQ_ERR_TIMEOUT from vpq_device_status.
 * vpq_comm_alloc_symmetric is collective (all ranks, same order) and is the one place this library
 * allocates device memory; it owns the buffer until vpq_comm_free_symmetric / vpq_comm_destroy.
 * Needs M > 128, N % (8*world) == 0. */
int vpq_comm_alloc_symmetric(vpq_comm* comm, size_t bytes, void** local_ptr);
int vpq_comm_free_symmetric(vpq_comm* comm, void* local_ptr);
int vpq_affine_qmm_w4g64_bf16_nsplit_fused(vpq_comm* comm, const uint32_t* w_shard,
                                           const void* scales_shard, const void* biases_shard,
                                           const void* x, void* y_sym, int64_t K, int64_t N, int64_t M,
                                           void* stream);

#ifdef __cplusplus
}
#endif
#endif /* VPQ_H */
