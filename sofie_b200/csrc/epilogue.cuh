// The fused epilogue of every contraction kernel (tcgen05 and SIMT): one definition so that
// all kernels round identically.  Each step is a separately rounded fp32 operation
// (__fmul_rn/__fadd_rn block FMA contraction), which is what makes the int8 requantisation
// reproducible bit for bit by a host restatement compiled with -ffp-contract=off.  The activations that call a
// transcendental function (erff, tanhf, expf) are reproducible only as far as the two math libraries agree (a few
// units in the last place): integer outputs behind Gelu or Sigmoid are held to one step of the output type,
// everything behind Relu / LeakyRelu / no activation to exact equality.
#pragma once
#include "common.cuh"

namespace sb200 {

// Device copy of sofie_b200_epilogue plus what the kernel needs to address Y.
struct EpiParams {
  const float *row_scale;
  const float *col_scale;
  const void *bias;
  const void *residual;
  void *Y;
  long long ldy, ldc, ldr;
  long long stride_y, stride_c, stride_r;  // batch strides (elements)
  float alpha, beta, act_alpha, out_scale;
  int bias_mode, act, out_zp, y_dtype, residual_dtype;
  int acc_is_int;
  int params_aligned;  // col_scale and a per-column bias are 16-byte aligned (vector loads allowed)
  int y_peers;           // further outputs (peers' copies of Y) that every bulk-stored row segment also goes to (tcgen05 kernel)
  int residual_aligned;  // residual base, pitch and batch stride are multiples of 16 bytes (1) or of 32 bytes (2); 0: neither
  int fast;            // store_chunk_fast() applies: aligned per-column vectors, no full-matrix bias
  int seg_chunks;      // tcgen05 epilogue: 32-column chunks per flushed row segment (0: a whole 128-byte segment)
  int split_out;       // fp32 output written as a TF32 pair: hi = tf32(v) at column j, lo = tf32(v - hi) at column N + j
};

__device__ __forceinline__ float act_apply(float v, int act, float act_alpha) {
  switch (act) {
    case SOFIE_B200_ACT_RELU:
      // x > 0 ? x : 0, the CPU helper's form (SOFIE_common_helpers.cxx:325-332)
      return v > 0.f ? v : 0.f;
    case SOFIE_B200_ACT_GELU_ERF:
      // 0.5*x*(1+erf(x/sqrt(2))), ROperator_Gelu.hxx:67
      return __fmul_rn(__fmul_rn(0.5f, v), __fadd_rn(1.f, erff(__fmul_rn(v, 0.7071067811865475f))));
    case SOFIE_B200_ACT_GELU_TANH: {
      // 0.5*x*(1+tanh(sqrt(2/pi)*(x+0.044715*x^3))), ROperator_Gelu.hxx:64-66
      // every product and sum rounded on its own, in the order the expression is written in
      const float x3 = __fmul_rn(__fmul_rn(v, v), v);
      const float t = tanhf(__fmul_rn(0.7978845608028654f, __fadd_rn(v, __fmul_rn(0.044715f, x3))));
      return __fmul_rn(__fmul_rn(0.5f, v), __fadd_rn(1.f, t));
    }
    case SOFIE_B200_ACT_LEAKY_RELU:
      return v >= 0.f ? v : __fmul_rn(act_alpha, v);
    case SOFIE_B200_ACT_SIGMOID:
      return __fdiv_rn(1.f, __fadd_rn(1.f, expf(-v)));
    default:
      return v;
  }
}

// Everything between the raw accumulator and the value that is converted to the output type.
__device__ __forceinline__ float epi_value(const EpiParams &p, uint32_t raw, long long b, long long i,
                                           long long j) {
  float v;
  if (p.acc_is_int) {
    int a = (int)raw;
    if (p.bias_mode == SOFIE_B200_BIAS_COL_I32) a += ((const int *)p.bias)[j];
    else if (p.bias_mode == SOFIE_B200_BIAS_ROW_I32) a += ((const int *)p.bias)[i];
    v = (float)a;
  } else {
    v = __uint_as_float(raw);
  }
  if (p.row_scale) v = __fmul_rn(v, p.row_scale[i]);
  if (p.col_scale) v = __fmul_rn(v, p.col_scale[j]);
  if (p.alpha != 1.f) v = __fmul_rn(v, p.alpha);
  switch (p.bias_mode) {
    case SOFIE_B200_BIAS_COL_F32: v = __fadd_rn(v, ((const float *)p.bias)[j]); break;
    case SOFIE_B200_BIAS_ROW_F32: v = __fadd_rn(v, ((const float *)p.bias)[i]); break;
    case SOFIE_B200_BIAS_SCALAR_F32: v = __fadd_rn(v, ((const float *)p.bias)[0]); break;
    case SOFIE_B200_BIAS_FULL_F32:
      v = __fadd_rn(v, __fmul_rn(p.beta, ((const float *)p.bias)[b * p.stride_c + i * p.ldc + j]));
      break;
    default: break;
  }
  if (p.residual) {
    long long off = b * p.stride_r + i * p.ldr + j;
    float r = p.residual_dtype == SOFIE_B200_BF16 ? __bfloat162float(((const __nv_bfloat16 *)p.residual)[off])
                                                  : ((const float *)p.residual)[off];
    v = __fadd_rn(v, r);
  }
  return act_apply(v, p.act, p.act_alpha);
}

// ONNX QuantizeLinear rounding: half to even, add zero point, saturate.
__device__ __forceinline__ int quantize_i(float v, float out_scale, int zp, int lo, int hi) {
  float q = out_scale == 1.f ? v : __fdiv_rn(v, out_scale);
  q = rintf(q) + (float)zp;
  q = fminf(fmaxf(q, (float)lo), (float)hi);
  return (int)q;
}

// Scalar store of one output element (edges and the SIMT kernel).
__device__ __forceinline__ void epi_store_one(const EpiParams &p, uint32_t raw, long long b, long long i,
                                              long long j) {
  long long off = b * p.stride_y + i * p.ldy + j;
  if (p.y_dtype == SOFIE_B200_I32) {
    int a = (int)raw;
    if (p.bias_mode == SOFIE_B200_BIAS_COL_I32) a += ((const int *)p.bias)[j];
    else if (p.bias_mode == SOFIE_B200_BIAS_ROW_I32) a += ((const int *)p.bias)[i];
    ((int *)p.Y)[off] = a;
    return;
  }
  float v = epi_value(p, raw, b, i, j);
  switch (p.y_dtype) {
    case SOFIE_B200_F32: ((float *)p.Y)[off] = v; break;
    case SOFIE_B200_BF16: ((__nv_bfloat16 *)p.Y)[off] = __float2bfloat16_rn(v); break;
    case SOFIE_B200_I8: ((int8_t *)p.Y)[off] = (int8_t)quantize_i(v, p.out_scale, p.out_zp, -128, 127); break;
    case SOFIE_B200_U8: ((uint8_t *)p.Y)[off] = (uint8_t)quantize_i(v, p.out_scale, p.out_zp, 0, 255); break;
    default: break;
  }
}

}  // namespace sb200
