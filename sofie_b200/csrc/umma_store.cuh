// Epilogue store of the tcgen05 contraction kernels (single-CTA and CTA-pair): one 32-column chunk of
// one accumulator row through the fused epilogue to global memory.
#pragma once
#include "gemm.cuh"
#include "ptx.cuh"

namespace sb200 {

__device__ __forceinline__ void raise_abort(volatile int *abort_flag, int *status, int code) {
  *abort_flag = 1;
  atomicCAS(status, 0, code);
}

__device__ __forceinline__ void st_v4(void *p, uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
  *reinterpret_cast<uint4 *>(p) = make_uint4(a, b, c, d);
}

// Applies the fused epilogue to one 32-column chunk of one accumulator row and stores it.
//
// The work is staged as passes over a register array, with every data-independent decision
// (which scales exist, which activation, which output type) taken once per chunk OUTSIDE the
// unrolled per-element loops: a warp cannot overlap instructions across a branch, so uniform
// branches inside the element loop would serialise the whole epilogue.  Absent scales multiply
// by 1.0f and an absent bias adds 0.0f; both are exact, so the value equals the documented
// step-by-step formula (sofie_b200_epilogue) bit for bit.
__device__ __forceinline__ void store_chunk(const EpiParams &ep, const uint32_t (&raw)[32], long long b, long long row,
                                            int col0, int ncols, bool vec) {
  const bool full = ncols == 32;
  const long long off = b * ep.stride_y + row * ep.ldy + col0;

  if (ep.y_dtype == SOFIE_B200_I32) {  // raw integer accumulator (+ int32 bias)
    int a[32];
#pragma unroll
    for (int c = 0; c < 32; ++c) a[c] = (int)raw[c];
    if (ep.bias_mode == SOFIE_B200_BIAS_COL_I32) {
#pragma unroll
      for (int c = 0; c < 32; ++c) a[c] += (full || c < ncols) ? ((const int *)ep.bias)[col0 + c] : 0;
    } else if (ep.bias_mode == SOFIE_B200_BIAS_ROW_I32) {
      const int br = ((const int *)ep.bias)[row];
#pragma unroll
      for (int c = 0; c < 32; ++c) a[c] += br;
    }
    int *y = (int *)ep.Y + off;
    if (vec && full) {
#pragma unroll
      for (int c = 0; c < 32; c += 4) st_v4(y + c, a[c], a[c + 1], a[c + 2], a[c + 3]);
    } else {
#pragma unroll
      for (int c = 0; c < 32; ++c)
        if (c < ncols) y[c] = a[c];
    }
    return;
  }

  float v[32];
  // 1. accumulator -> fp32
  if (ep.acc_is_int) {
    if (ep.bias_mode == SOFIE_B200_BIAS_COL_I32) {
#pragma unroll
      for (int c = 0; c < 32; ++c) v[c] = (float)((int)raw[c] + ((full || c < ncols) ? ((const int *)ep.bias)[col0 + c] : 0));
    } else {
      const int br = ep.bias_mode == SOFIE_B200_BIAS_ROW_I32 ? ((const int *)ep.bias)[row] : 0;
#pragma unroll
      for (int c = 0; c < 32; ++c) v[c] = (float)((int)raw[c] + br);
    }
  } else {
#pragma unroll
    for (int c = 0; c < 32; ++c) v[c] = __uint_as_float(raw[c]);
  }
  // 2. scales, in the documented order: row, column, alpha
  if (ep.row_scale) {
    const float rs = ep.row_scale[row];
#pragma unroll
    for (int c = 0; c < 32; ++c) v[c] = __fmul_rn(v[c], rs);
  }
  if (ep.col_scale) {
    if (full && ep.params_aligned) {
#pragma unroll
      for (int c = 0; c < 32; c += 4) {
        const float4 s4 = *reinterpret_cast<const float4 *>(ep.col_scale + col0 + c);  // col0 % 32 == 0
        v[c] = __fmul_rn(v[c], s4.x); v[c + 1] = __fmul_rn(v[c + 1], s4.y);
        v[c + 2] = __fmul_rn(v[c + 2], s4.z); v[c + 3] = __fmul_rn(v[c + 3], s4.w);
      }
    } else {
#pragma unroll
      for (int c = 0; c < 32; ++c) v[c] = __fmul_rn(v[c], c < ncols ? ep.col_scale[col0 + c] : 1.f);
    }
  }
  if (ep.alpha != 1.f) {
#pragma unroll
    for (int c = 0; c < 32; ++c) v[c] = __fmul_rn(v[c], ep.alpha);
  }
  // 3. additive terms
  switch (ep.bias_mode) {
    case SOFIE_B200_BIAS_COL_F32:
      if (full && ep.params_aligned) {
#pragma unroll
        for (int c = 0; c < 32; c += 4) {
          const float4 b4 = *reinterpret_cast<const float4 *>((const float *)ep.bias + col0 + c);
          v[c] = __fadd_rn(v[c], b4.x); v[c + 1] = __fadd_rn(v[c + 1], b4.y);
          v[c + 2] = __fadd_rn(v[c + 2], b4.z); v[c + 3] = __fadd_rn(v[c + 3], b4.w);
        }
      } else {
#pragma unroll
        for (int c = 0; c < 32; ++c)
          if (c < ncols) v[c] = __fadd_rn(v[c], ((const float *)ep.bias)[col0 + c]);
      }
      break;
    case SOFIE_B200_BIAS_ROW_F32: {
      const float br = ((const float *)ep.bias)[row];
#pragma unroll
      for (int c = 0; c < 32; ++c) v[c] = __fadd_rn(v[c], br);
      break;
    }
    case SOFIE_B200_BIAS_SCALAR_F32: {
      const float bs = ((const float *)ep.bias)[0];
#pragma unroll
      for (int c = 0; c < 32; ++c) v[c] = __fadd_rn(v[c], bs);
      break;
    }
    case SOFIE_B200_BIAS_FULL_F32: {
      const float *cr = (const float *)ep.bias + b * ep.stride_c + row * ep.ldc + col0;
#pragma unroll
      for (int c = 0; c < 32; ++c)
        if (full || c < ncols) v[c] = __fadd_rn(v[c], __fmul_rn(ep.beta, cr[c]));
      break;
    }
    default: break;
  }
  if (ep.residual) {
    const long long roff = b * ep.stride_r + row * ep.ldr + col0;
    if (ep.residual_dtype == SOFIE_B200_BF16) {
      const __nv_bfloat16 *r = (const __nv_bfloat16 *)ep.residual + roff;
#pragma unroll
      for (int c = 0; c < 32; ++c)
        if (full || c < ncols) v[c] = __fadd_rn(v[c], __bfloat162float(r[c]));
    } else {
      const float *r = (const float *)ep.residual + roff;
#pragma unroll
      for (int c = 0; c < 32; ++c)
        if (full || c < ncols) v[c] = __fadd_rn(v[c], r[c]);
    }
  }
  // 4. activation
  switch (ep.act) {
    case SOFIE_B200_ACT_NONE: break;
    case SOFIE_B200_ACT_RELU:
#pragma unroll
      for (int c = 0; c < 32; ++c) v[c] = act_apply(v[c], SOFIE_B200_ACT_RELU, 0.f);
      break;
    case SOFIE_B200_ACT_GELU_ERF:
#pragma unroll
      for (int c = 0; c < 32; ++c) v[c] = act_apply(v[c], SOFIE_B200_ACT_GELU_ERF, 0.f);
      break;
    default:
#pragma unroll
      for (int c = 0; c < 32; ++c) v[c] = act_apply(v[c], ep.act, ep.act_alpha);
      break;
  }
  // 5. convert and store
  if (ep.y_dtype == SOFIE_B200_F32) {
    float *y = (float *)ep.Y + off;
    if (vec && full) {
#pragma unroll
      for (int c = 0; c < 32; c += 4)
        st_v4(y + c, __float_as_uint(v[c]), __float_as_uint(v[c + 1]), __float_as_uint(v[c + 2]), __float_as_uint(v[c + 3]));
    } else {
#pragma unroll
      for (int c = 0; c < 32; ++c)
        if (c < ncols) y[c] = v[c];
    }
  } else if (ep.y_dtype == SOFIE_B200_BF16) {
    __nv_bfloat16 *y = (__nv_bfloat16 *)ep.Y + off;
    if (vec && full) {
#pragma unroll
      for (int c = 0; c < 32; c += 8) {
        uint32_t w[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          __nv_bfloat162 h2 = __floats2bfloat162_rn(v[c + 2 * u], v[c + 2 * u + 1]);
          w[u] = *reinterpret_cast<uint32_t *>(&h2);
        }
        st_v4(y + c, w[0], w[1], w[2], w[3]);
      }
    } else {
#pragma unroll
      for (int c = 0; c < 32; ++c)
        if (c < ncols) y[c] = __float2bfloat16_rn(v[c]);
    }
  } else {  // I8 / U8: ONNX rounding (half to even), zero point, saturate
    const float lo = ep.y_dtype == SOFIE_B200_I8 ? -128.f : 0.f;
    const float hi = ep.y_dtype == SOFIE_B200_I8 ? 127.f : 255.f;
    const float zp = (float)ep.out_zp;
    if (ep.out_scale != 1.f) {
#pragma unroll
      for (int c = 0; c < 32; ++c) v[c] = __fdiv_rn(v[c], ep.out_scale);
    }
    uint32_t q[32];
#pragma unroll
    for (int c = 0; c < 32; ++c) q[c] = (uint32_t)(int)fminf(fmaxf(rintf(v[c]) + zp, lo), hi) & 0xffu;
    uint8_t *y = (uint8_t *)ep.Y + off;
    if (vec && full) {
#pragma unroll
      for (int c = 0; c < 32; c += 16) {
        uint32_t w[4];
#pragma unroll
        for (int u = 0; u < 4; ++u)
          w[u] = q[c + 4 * u] | (q[c + 4 * u + 1] << 8) | (q[c + 4 * u + 2] << 16) | (q[c + 4 * u + 3] << 24);
        st_v4(y + c, w[0], w[1], w[2], w[3]);
      }
    } else {
#pragma unroll
      for (int c = 0; c < 32; ++c)
        if (c < ncols) y[c] = (uint8_t)q[c];
    }
  }
}

}  // namespace sb200
