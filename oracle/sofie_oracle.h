/*
 * TEST INFRASTRUCTURE -- not product code.  A plain-C, CPU restatement of the arithmetic of the
 * code SOFIE emits for the inference hot path, used only as the checker in tests/, in
 * __graft_entry__.smoke() and as the timed CPU baseline of bench.py.  Nothing under sofie_b200/
 * may link or call it.
 *
 * It takes the same descriptor structs as the product's C ABI (include/sofie_b200.h) so a test can
 * hand one description to both sides.  Floating-point contractions accumulate in double and round
 * once, so the result is a tight centre for any fp32 summation order (BLAS, tensor cores); integer
 * contractions accumulate in int32 exactly.  The epilogue applies the documented steps one fp32
 * rounding at a time (this file must be compiled with -ffp-contract=off).
 *
 * Parity status: the fp32 operators are pinned against the reference's checked-in expected vectors
 * and against the reference's own emitted CPU code (oracle/_ref), see tests/golden/.  The int8
 * (QLinearMatMul / QLinearConv), FP8 and bf16 paths have NO counterpart in the reference
 * (core/inc/SOFIE/operators/ROperator_Gemm.hxx:67-68 static_asserts float): for those this file
 * follows the ONNX operator definitions and says so -- "parity unpinned" by the reference.
 */
#ifndef SOFIE_ORACLE_H
#define SOFIE_ORACLE_H
#include "../include/sofie_b200.h"

#ifdef __cplusplus
extern "C" {
#endif

/* Number of threads the contraction loops use (OpenMP if compiled with it, else 1). */
int so_threads(void);
void so_set_threads(int n);

/* Y = epilogue(op(A) x op(B)), batched; semantics of sofie_b200_gemm_desc / sofie_b200_epilogue.
 * Host pointers.  Gemm: ROperator_Gemm.hxx:419-741 + Gemm_Call (SOFIE_common_helpers.cxx:296-323):
 * bias broadcast pre-written into Y, then sgemm with beta = 1, then Relu.  QLinearMatMul and the
 * FP8 GEMM: ONNX definitions (no reference implementation). */
int so_gemm(const sofie_b200_gemm_desc *d, const void *A, const void *B, void *Y, const sofie_b200_epilogue *ep);

/* NCHW convolution with the same epilogue (channels = epilogue columns); shape rules of
 * ROperator_Conv.hxx:123-262, K order (c, r, s) of ROperator_Conv.hxx:456-476. */
int so_conv(const sofie_b200_conv_desc *d, const void *X, const void *W, void *Y, const sofie_b200_epilogue *ep);
int so_conv_out_shape(const sofie_b200_conv_desc *d, int64_t *Ho, int64_t *Wo);

/* ROperator_LayerNormalization.hxx:257-312 (two-pass, biased variance). dtype F32 or BF16. */
int so_layernorm(const void *x, void *y, int x_dtype, int y_dtype, int64_t rows, int64_t cols, const float *scale,
                 const float *bias, float eps, float *mean_out, float *invstd_out);
/* ROperator_Softmax.hxx:97-118 (max, exp, sum, multiply by reciprocal). */
int so_softmax(const void *x, void *y, int x_dtype, int y_dtype, int64_t rows, int64_t cols, int log_softmax);
/* ROperator_SDPA.hxx:141-200, fp32, step for step: per (batch, head, query) dot * scale (+ mask), max, exp(s - max), / sum,
 * weighted sum over V.  folded = 0: Q, K [B,H,S,D], V, Y [B,H,S,Dv]; folded = 1: [B,S,H*D] (ROperator_SDPA.hxx:103-129).
 * mask [B,H,S,S] or NULL; scale 0 = 1/sqrt(D).  With softmax over an axis other than the last (so_softmax_axis) this is
 * the general-axis path of ROperator_Softmax.hxx:120-200, which divides by the sum. */
int so_sdpa(const float *q, const float *k, const float *v, const float *mask, float *y, int64_t B, int64_t H, int64_t S, int64_t D,
            int64_t Dv, float scale, int folded);
int so_softmax_axis(const float *x, float *y, int64_t outer, int64_t axis_len, int64_t inner, int log_softmax);
/* ROperator_Relu.hxx / ROperator_Gelu.hxx:62-98 / LeakyRelu / Sigmoid, elementwise, F32 or BF16. */
int so_unary(const void *x, void *y, int dtype, int64_t n, int act, float act_alpha);
/* ROperator_BasicBinary.hxx:520-636 with trailing broadcast; op 0 Add 1 Sub 2 Mul 3 Div. */
int so_binary(const void *a, const void *b, void *y, int dtype, int64_t n, int64_t nb, int op, int act);
/* ROperator_BatchNormalization.hxx:136-153: (x - mean[c]) * fused_scale[c] + bias[c]. */
int so_batchnorm(const float *x, float *y, int64_t outer, int64_t channels, int64_t inner, const float *fused_scale,
                 const float *bias, const float *mean, int act);
/* fused_scale = scale / sqrt(var + eps) in fp32, ROperator_BatchNormalization.hxx:100-109. */
void so_batchnorm_fold(const float *scale, const float *var, float eps, int64_t channels, float *fused_scale);
/* ROperator_Pool.hxx:531-536,590-607: sum then divide by the window size. */
int so_global_avgpool(const void *x, float *y, int x_dtype, int64_t nc, int64_t inner);
/* ONNX QuantizeLinear / DequantizeLinear. */
int so_quantize(const float *x, void *q, int q_dtype, int64_t n, const float *scale, const int32_t *zp,
                int64_t channels, int64_t inner);
int so_dequantize(const void *q, float *x, int q_dtype, int64_t n, const float *scale, const int32_t *zp,
                  int64_t channels, int64_t inner);
/* Conversions (round to nearest even; e4m3fn saturates to +-448, NaN stays NaN). */
uint8_t so_f32_to_e4m3(float v);
float so_e4m3_to_f32(uint8_t v);
uint16_t so_f32_to_bf16(float v);
float so_bf16_to_f32(uint16_t v);
int so_convert(const void *x, void *y, int x_dtype, int y_dtype, int64_t rows, int64_t cols, const float *row_scale);
/* Best-fit-with-coalescing arena policy of MemoryPlanner.inc:47-132 (sizes rounded to 256). */
int so_plan_arena(const sofie_b200_tensor_life *lives, int64_t n, int64_t *offsets, int64_t *total);

#ifdef __cplusplus
}
#endif
#endif
