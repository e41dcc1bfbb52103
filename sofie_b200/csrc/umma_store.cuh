// Epilogue store of the tcgen05 contraction kernels: one 32-column chunk of
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

// Coalesced stores of the epilogue.  In the accumulator a lane owns a ROW, so a direct 16-byte store per lane
// touches 32 different 128-byte lines per instruction, the L1 spends 32 cycles on it, and rows are written in
// pieces shorter than a line.  Instead the finished 16-byte units of up to 128 bytes per row (one 32-column
// chunk of 4-byte outputs, two of 2-byte, four of 1-byte outputs) are collected in a per-warp staging buffer in
// shared memory (32 rows x 128 bytes, XOR-swizzled: conflict-free both ways) and flushed with consecutive lanes
// holding consecutive units of the same row: one store instruction then writes four whole 128-byte lines.
//
// The row pitch of the buffer is 128 bytes, or 64 or 32 where a warp flushes shorter row segments (so that both warps of
// a lane quarter have segments to work on when the tile is narrow).  The two low bits of the buffer's address -- it is
// 1024-byte aligned -- carry the pitch: 128 >> code bytes.  Byte a of the buffer lives at a ^ (((a >> 7) & m) << 4) with
// m = 7, 3, 1: the TMA unit's swizzle whose span equals the pitch (128B, 64B, 32B), so a bulk tensor store of a
// (pitch x 32 rows) box through a map with that swizzle reads the rows back in order.
__device__ __forceinline__ uint32_t stage_swizzle(uint32_t a, uint32_t code) { return a ^ (((a >> 7) & (7u >> code)) << 4); }

// stage_units: lane (= row) writes its U units of the chunk at unit offset `slot * U` of its row.
template <int U>
__device__ __forceinline__ void stage_units(uint32_t stage, const uint32_t (&w)[4 * U], int slot) {
  const int lane = threadIdx.x & 31;
  const uint32_t code = stage & 3u, base = stage & ~3u;
  const uint32_t a0 = (uint32_t)lane * (128u >> code) + (uint32_t)(slot * U) * 16u;
#pragma unroll
  for (int u = 0; u < U; ++u) {
    asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(base + stage_swizzle(a0 + u * 16, code)), "r"(w[4 * u]),
                 "r"(w[4 * u + 1]), "r"(w[4 * u + 2]), "r"(w[4 * u + 3])
                 : "memory");
  }
}

// flush_staged: writes the first `units` 16-byte units of each of the first `rows_valid` rows of the buffer to
// y_row0 + row * ldy_bytes.  All lanes of the warp call it; the buffer may be refilled right after it returns.
__device__ __forceinline__ void flush_staged(uint32_t stage, uint8_t *y_row0, long long ldy_bytes, int rows_valid, int units) {
  const int lane = threadIdx.x & 31;
  __syncwarp();   // every lane's units are in the buffer
  const uint32_t code = stage & 3u, base = stage & ~3u;
  const int lg = 3 - (int)code;   // log2 of the units per buffer row
  for (int i = 0; i < (8 >> code); ++i) {
    const int idx = i * 32 + lane, r = idx >> lg, u = idx & ((1 << lg) - 1);
    uint32_t a, b, c, d;
    asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];" : "=r"(a), "=r"(b), "=r"(c), "=r"(d) : "r"(base + stage_swizzle((uint32_t)(r * (128 >> code) + u * 16), code)) : "memory");
    if (r < rows_valid && u < units) st_v4(y_row0 + r * ldy_bytes + u * 16, a, b, c, d);
  }
  __syncwarp();   // reads done before anyone overwrites the buffer
}

// Chunks per 128-byte row segment for an output type: the group a warp stages before it flushes.
__device__ __forceinline__ int chunks_per_flush(int y_dtype) {
  return (y_dtype == SOFIE_B200_F32 || y_dtype == SOFIE_B200_I32) ? 1 : (y_dtype == SOFIE_B200_BF16 ? 2 : 4);
}
__device__ __forceinline__ int out_elem_bytes(int y_dtype) {
  return (y_dtype == SOFIE_B200_F32 || y_dtype == SOFIE_B200_I32) ? 4 : (y_dtype == SOFIE_B200_BF16 ? 2 : 1);
}

// Applies the fused epilogue to one 32-column chunk of one accumulator row and stores it.
//
// The work is staged as passes over a register array, with every data-independent decision
// (which scales exist, which activation, which output type) taken once per chunk OUTSIDE the
// unrolled per-element loops: a warp cannot overlap instructions across a branch, so uniform
// branches inside the element loop would serialise the whole epilogue.  Absent scales multiply
// by 1.0f and an absent bias adds 0.0f; both are exact, so the value equals the documented
// step-by-step formula (sofie_b200_epilogue) bit for bit.
//
// `row` is this lane's row; lane 0 of the warp holds row `row - lane`.  With `stage` != 0 (shared-memory address of
// the warp's 4 KB staging buffer) a full, aligned chunk is not stored but staged at position `slot` of the row's
// 128-byte segment, the function returns true, and the caller flushes the buffer with flush_staged() once the
// segment is complete; then EVERY lane of the warp must make the call (rows at or past `rows_total` are computed
// but never stored).  Otherwise the chunk is stored directly and the function returns false.
template <int W = 32>
__device__ __forceinline__ bool store_chunk(const EpiParams &ep, const uint32_t (&raw)[W], long long b, long long row,
                                            int col0, int ncols, bool vec, uint32_t stage = 0, long long rows_total = 0,
                                            int slot = 0, int split_part = 0) {
  const bool full = ncols == W;
  // split_part (fp32 output as a TF32 pair, EpiParams::split_out): 1 stores hi = tf32(v) at the element's own column,
  // 2 stores lo = tf32(v - hi) at column N + j; the caller makes both calls (and flushes at the matching address)
  const long long off = b * ep.stride_y + row * ep.ldy + col0 + (split_part == 2 ? ep.ldy / 2 : 0);
  const bool staged = stage != 0 && vec && full;       // warp-uniform
  if (!staged && stage != 0 && row >= rows_total) return false;   // direct path: rows past the end store nothing
  const long long rr = (stage != 0 && row >= rows_total) ? rows_total - 1 : row;   // row whose per-row operands are read

  if (ep.y_dtype == SOFIE_B200_I32) {  // raw integer accumulator (+ int32 bias)
    int a[W];
#pragma unroll
    for (int c = 0; c < W; ++c) a[c] = (int)raw[c];
    if (ep.bias_mode == SOFIE_B200_BIAS_COL_I32) {
#pragma unroll
      for (int c = 0; c < W; ++c) a[c] += (full || c < ncols) ? ((const int *)ep.bias)[col0 + c] : 0;
    } else if (ep.bias_mode == SOFIE_B200_BIAS_ROW_I32) {
      const int br = ((const int *)ep.bias)[rr];
#pragma unroll
      for (int c = 0; c < W; ++c) a[c] += br;
    }
    int *y = (int *)ep.Y + off;
    if (staged) {
      uint32_t w[W];
#pragma unroll
      for (int c = 0; c < W; ++c) w[c] = (uint32_t)a[c];
      stage_units<W / 4>(stage, w, slot);
      return true;
    } else if (vec && full) {
#pragma unroll
      for (int c = 0; c < W; c += 4) st_v4(y + c, a[c], a[c + 1], a[c + 2], a[c + 3]);
    } else {
#pragma unroll
      for (int c = 0; c < W; ++c)
        if (c < ncols) y[c] = a[c];
    }
    return false;
  }

  float v[W];
  // 1. accumulator -> fp32
  if (ep.acc_is_int) {
    if (ep.bias_mode == SOFIE_B200_BIAS_COL_I32) {
#pragma unroll
      for (int c = 0; c < W; ++c) v[c] = (float)((int)raw[c] + ((full || c < ncols) ? ((const int *)ep.bias)[col0 + c] : 0));
    } else {
      const int br = ep.bias_mode == SOFIE_B200_BIAS_ROW_I32 ? ((const int *)ep.bias)[rr] : 0;
#pragma unroll
      for (int c = 0; c < W; ++c) v[c] = (float)((int)raw[c] + br);
    }
  } else {
#pragma unroll
    for (int c = 0; c < W; ++c) v[c] = __uint_as_float(raw[c]);
  }
  // 2. scales, in the documented order: row, column, alpha
  if (ep.row_scale) {
    const float rs = ep.row_scale[rr];
#pragma unroll
    for (int c = 0; c < W; ++c) v[c] = __fmul_rn(v[c], rs);
  }
  if (ep.col_scale) {
    if (full && ep.params_aligned) {
#pragma unroll
      for (int c = 0; c < W; c += 4) {
        const float4 s4 = *reinterpret_cast<const float4 *>(ep.col_scale + col0 + c);  // col0 % 32 == 0
        v[c] = __fmul_rn(v[c], s4.x); v[c + 1] = __fmul_rn(v[c + 1], s4.y);
        v[c + 2] = __fmul_rn(v[c + 2], s4.z); v[c + 3] = __fmul_rn(v[c + 3], s4.w);
      }
    } else {
#pragma unroll
      for (int c = 0; c < W; ++c) v[c] = __fmul_rn(v[c], c < ncols ? ep.col_scale[col0 + c] : 1.f);
    }
  }
  if (ep.alpha != 1.f) {
#pragma unroll
    for (int c = 0; c < W; ++c) v[c] = __fmul_rn(v[c], ep.alpha);
  }
  // 3. additive terms
  switch (ep.bias_mode) {
    case SOFIE_B200_BIAS_COL_F32:
      if (full && ep.params_aligned) {
#pragma unroll
        for (int c = 0; c < W; c += 4) {
          const float4 b4 = *reinterpret_cast<const float4 *>((const float *)ep.bias + col0 + c);
          v[c] = __fadd_rn(v[c], b4.x); v[c + 1] = __fadd_rn(v[c + 1], b4.y);
          v[c + 2] = __fadd_rn(v[c + 2], b4.z); v[c + 3] = __fadd_rn(v[c + 3], b4.w);
        }
      } else {
#pragma unroll
        for (int c = 0; c < W; ++c)
          if (c < ncols) v[c] = __fadd_rn(v[c], ((const float *)ep.bias)[col0 + c]);
      }
      break;
    case SOFIE_B200_BIAS_ROW_F32: {
      const float br = ((const float *)ep.bias)[rr];
#pragma unroll
      for (int c = 0; c < W; ++c) v[c] = __fadd_rn(v[c], br);
      break;
    }
    case SOFIE_B200_BIAS_SCALAR_F32: {
      const float bs = ((const float *)ep.bias)[0];
#pragma unroll
      for (int c = 0; c < W; ++c) v[c] = __fadd_rn(v[c], bs);
      break;
    }
    case SOFIE_B200_BIAS_FULL_F32: {
      const float *cr = (const float *)ep.bias + b * ep.stride_c + rr * ep.ldc + col0;
#pragma unroll
      for (int c = 0; c < W; ++c)
        if (full || c < ncols) v[c] = __fadd_rn(v[c], __fmul_rn(ep.beta, cr[c]));
      break;
    }
    default: break;
  }
  if (ep.residual) {
    const long long roff = b * ep.stride_r + rr * ep.ldr + col0;
    if (ep.residual_dtype == SOFIE_B200_BF16) {
      const __nv_bfloat16 *r = (const __nv_bfloat16 *)ep.residual + roff;
#pragma unroll
      for (int c = 0; c < W; ++c)
        if (full || c < ncols) v[c] = __fadd_rn(v[c], __bfloat162float(r[c]));
    } else {
      const float *r = (const float *)ep.residual + roff;
#pragma unroll
      for (int c = 0; c < W; ++c)
        if (full || c < ncols) v[c] = __fadd_rn(v[c], r[c]);
    }
  }
  // 4. activation
  switch (ep.act) {
    case SOFIE_B200_ACT_NONE: break;
    case SOFIE_B200_ACT_RELU:
#pragma unroll
      for (int c = 0; c < W; ++c) v[c] = act_apply(v[c], SOFIE_B200_ACT_RELU, 0.f);
      break;
    case SOFIE_B200_ACT_GELU_ERF:
#pragma unroll
      for (int c = 0; c < W; ++c) v[c] = act_apply(v[c], SOFIE_B200_ACT_GELU_ERF, 0.f);
      break;
    default:
#pragma unroll
      for (int c = 0; c < W; ++c) v[c] = act_apply(v[c], ep.act, ep.act_alpha);
      break;
  }
  // 5. convert and store
  if (split_part != 0) {
#pragma unroll
    for (int c = 0; c < W; ++c) {
      const float h = tf32_rn(v[c]);
      v[c] = split_part == 1 ? h : tf32_rn(__fsub_rn(v[c], h));
    }
  }
  if (ep.y_dtype == SOFIE_B200_F32) {
    float *y = (float *)ep.Y + off;
    if (staged) {
      uint32_t w[W];
#pragma unroll
      for (int c = 0; c < W; ++c) w[c] = __float_as_uint(v[c]);
      stage_units<W / 4>(stage, w, slot);
      return true;
    } else if (vec && full) {
#pragma unroll
      for (int c = 0; c < W; c += 4)
        st_v4(y + c, __float_as_uint(v[c]), __float_as_uint(v[c + 1]), __float_as_uint(v[c + 2]), __float_as_uint(v[c + 3]));
    } else {
#pragma unroll
      for (int c = 0; c < W; ++c)
        if (c < ncols) y[c] = v[c];
    }
  } else if (ep.y_dtype == SOFIE_B200_BF16) {
    __nv_bfloat16 *y = (__nv_bfloat16 *)ep.Y + off;
    if (staged) {
      uint32_t w[W / 2];
#pragma unroll
      for (int u = 0; u < W / 2; ++u) {
        __nv_bfloat162 h2 = __floats2bfloat162_rn(v[2 * u], v[2 * u + 1]);
        w[u] = *reinterpret_cast<uint32_t *>(&h2);
      }
      stage_units<W / 8>(stage, w, slot);
      return true;
    } else if (vec && full) {
#pragma unroll
      for (int c = 0; c < W; c += 8) {
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
      for (int c = 0; c < W; ++c)
        if (c < ncols) y[c] = __float2bfloat16_rn(v[c]);
    }
  } else {  // I8 / U8: ONNX rounding (half to even), zero point, saturate
    const float lo = ep.y_dtype == SOFIE_B200_I8 ? -128.f : 0.f;
    const float hi = ep.y_dtype == SOFIE_B200_I8 ? 127.f : 255.f;
    const float zp = (float)ep.out_zp;
    if (ep.out_scale != 1.f) {
#pragma unroll
      for (int c = 0; c < W; ++c) v[c] = __fdiv_rn(v[c], ep.out_scale);
    }
    uint32_t q[W];
#pragma unroll
    for (int c = 0; c < W; ++c) q[c] = (uint32_t)(int)fminf(fmaxf(rintf(v[c]) + zp, lo), hi) & 0xffu;
    uint8_t *y = (uint8_t *)ep.Y + off;
    if (staged) {
      uint32_t w[W / 4];
#pragma unroll
      for (int u = 0; u < W / 4; ++u) w[u] = q[4 * u] | (q[4 * u + 1] << 8) | (q[4 * u + 2] << 16) | (q[4 * u + 3] << 24);
      stage_units<W / 16>(stage, w, slot);
      return true;
    } else if (vec && full) {
#pragma unroll
      for (int c = 0; c < W; c += 16) {
        uint32_t w[4];
#pragma unroll
        for (int u = 0; u < 4; ++u)
          w[u] = q[c + 4 * u] | (q[c + 4 * u + 1] << 8) | (q[c + 4 * u + 2] << 16) | (q[c + 4 * u + 3] << 24);
        st_v4(y + c, w[0], w[1], w[2], w[3]);
      }
    } else {
#pragma unroll
      for (int c = 0; c < W; ++c)
        if (c < ncols) y[c] = (uint8_t)q[c];
    }
  }
  return false;
}

// Neutral operands for features a launch does not use: the fast path below always multiplies by a column scale
// and adds a column bias, and reads these instead of branching.  x * 1.0f and x + (-0.0f) return x bit for bit
// (also for x = -0.0f, which + 0.0f would turn into +0.0f).
__device__ __align__(16) const float g_epi_ones[32] = {1.f, 1.f, 1.f, 1.f, 1.f, 1.f, 1.f, 1.f, 1.f, 1.f, 1.f, 1.f, 1.f, 1.f, 1.f, 1.f,
                                                       1.f, 1.f, 1.f, 1.f, 1.f, 1.f, 1.f, 1.f, 1.f, 1.f, 1.f, 1.f, 1.f, 1.f, 1.f, 1.f};
__device__ __align__(16) const float g_epi_negzero[32] = {-0.f, -0.f, -0.f, -0.f, -0.f, -0.f, -0.f, -0.f, -0.f, -0.f, -0.f, -0.f, -0.f, -0.f, -0.f, -0.f,
                                                          -0.f, -0.f, -0.f, -0.f, -0.f, -0.f, -0.f, -0.f, -0.f, -0.f, -0.f, -0.f, -0.f, -0.f, -0.f, -0.f};
__device__ __align__(16) const int g_epi_izero[32] = {};

// The fast path (epi_values_fast + epi_finish_fast): the same epilogue as store_chunk() for the common case -- a full 32-column chunk, staged, with 16-byte aligned
// per-column vectors and no full-matrix bias -- written so that a launch takes almost no branches.  Every taken
// branch costs an epilogue warp an instruction-fetch bubble that nothing hides (one or two warps per scheduler),
// and a dozen "skip this feature" jumps per chunk made the epilogue slower than the main loop of a K = 512 tile.
// Scales and biases are therefore always applied, with neutral operands when absent; only the residual, the
// activation and the output type branch, and the rare cases are marked unlikely so they sit out of line.
// Operation order and rounding are those of store_chunk(): the results are bit-identical.
// Packed fp32 arithmetic of sm_100 (two values per instruction, each half rounded exactly as the scalar instruction
// would round it) on float2, which lets the compiler keep the pairs in aligned register pairs without moves.
__device__ __forceinline__ float2 fmul2(float2 a, float2 b) { return __fmul2_rn(a, b); }
__device__ __forceinline__ float2 fadd2(float2 a, float2 b) { return __fadd2_rn(a, b); }
__device__ __forceinline__ float2 ffma2(float2 a, float2 b, float2 c) { return __ffma2_rn(a, b, c); }
__device__ __forceinline__ float2 dup2(float x) { return make_float2(x, x); }

// Gelu (erf form) of two values for outputs that are rounded to bf16 afterwards.  erff() costs some thirty instructions
// per element and the Abramowitz & Stegun 7.1.28 form used before twenty per pair, which kept a Gelu epilogue longer than
// the main loop it follows.  x Phi(x) is x / (1 + exp(-l(x))) with l the logit of the normal distribution function, an odd
// function close to 1.5958 x + 0.0715 x^3; here l(x) = x q(x^2) with a cubic q fitted (minimax, relative) to the erf form:
// |error| <= 7.6e-4 of the value wherever |Gelu| > 1e-3 (a third of half a bf16 ulp) and 8e-5 absolute, against the
// 2e-2 relative + 1e-2 absolute bar of the bf16 paths.  -log2(e) is folded into the coefficients; six packed fp32
// instructions and two special-function ones (ex2, rcp) per pair.  Large |x|: q stays negative for every x^2, so
// x -> +inf gives exp2(-inf) = 0 and the value x, x -> -inf gives 1 / inf = 0 and the value -0.
__device__ __forceinline__ float2 gelu_erf_pair_lowp(float2 x) {
  const float2 s = fmul2(x, x);
  float2 q = ffma2(s, dup2(-4.490078936214559e-06f), dup2(0.0012212033616378903f));
  q = ffma2(q, s, dup2(-0.10808564722537994f));
  q = ffma2(q, s, dup2(-2.29966402053833f));
  const float2 w = fmul2(x, q);
  float2 e, r;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e.x) : "f"(w.x));
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e.y) : "f"(w.y));
  const float2 d = fadd2(e, dup2(1.f));
  asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(r.x) : "f"(d.x));
  asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(r.y) : "f"(d.y));
  return fmul2(x, r);
}

// First half of the fast path: everything that reads the raw accumulator -- integer bias, conversion, the three
// scales and the additive bias terms -- into v[32].  When it returns, `raw` is dead and the caller may already
// load the next chunk into it.  Returns false when the chunk was finished here (int32 output: staged as is).
template <bool ACC_INT, int W>   // W columns handled together (16, 32 or 64): independent chains for the scheduler to interleave
__device__ __forceinline__ bool epi_values_fast(const EpiParams &ep, const uint32_t (&raw)[W], float2 (&v)[W / 2], long long rr, int col0,
                                                uint32_t stage, int slot) {
  const int mode = ep.bias_mode;
  const int4 *bip = reinterpret_cast<const int4 *>(g_epi_izero);
  int rbi = 0;
  int bi_step = 0;             // the neutral arrays are 32 entries long: they are re-read for every group of four columns
  if (ACC_INT) {
    if (mode == SOFIE_B200_BIAS_COL_I32) { bip = reinterpret_cast<const int4 *>((const int *)ep.bias + col0); bi_step = 1; }
    if (mode == SOFIE_B200_BIAS_ROW_I32) rbi = ((const int *)ep.bias)[rr];
  }
  if (__builtin_expect(ep.y_dtype == SOFIE_B200_I32, 0)) {  // raw integer accumulator (+ int32 bias)
    constexpr int CW = W < 32 ? W : 32;   // columns per staging call
#pragma unroll
    for (int i = 0; i < W / CW; ++i) {
      uint32_t w[CW];
#pragma unroll
      for (int c = 0; c < CW; c += 4) {
        const int4 bi = bip[((CW * i + c) >> 2) * bi_step];
        w[c] = (uint32_t)((int)raw[CW * i + c] + bi.x + rbi); w[c + 1] = (uint32_t)((int)raw[CW * i + c + 1] + bi.y + rbi);
        w[c + 2] = (uint32_t)((int)raw[CW * i + c + 2] + bi.z + rbi); w[c + 3] = (uint32_t)((int)raw[CW * i + c + 3] + bi.w + rbi);
      }
      stage_units<CW / 4>(stage, w, slot + i);
    }
    return false;
  }
  float rs = 1.f;
  if (ep.row_scale) rs = ep.row_scale[rr];
  const bool has_cs = ep.col_scale != nullptr, has_bf = mode == SOFIE_B200_BIAS_COL_F32;
  const float4 *csp = reinterpret_cast<const float4 *>(has_cs ? ep.col_scale + col0 : g_epi_ones);
  const float4 *bfp = reinterpret_cast<const float4 *>(has_bf ? (const float *)ep.bias + col0 : g_epi_negzero);
  const int cs_step = has_cs ? 1 : 0, bf_step = has_bf ? 1 : 0;
  float rbf = -0.f;
  if (mode == SOFIE_B200_BIAS_ROW_F32) rbf = ((const float *)ep.bias)[rr];
  if (mode == SOFIE_B200_BIAS_SCALAR_F32) rbf = ((const float *)ep.bias)[0];
  const float2 rs2 = dup2(rs), alpha2 = dup2(ep.alpha), rbf2 = dup2(rbf);
#pragma unroll
  for (int c = 0; c < W; c += 4) {
    const float4 cs = csp[(c >> 2) * cs_step], bf = bfp[(c >> 2) * bf_step];
    float2 xa, xb;
    if (ACC_INT) {
      const int4 bi = bip[(c >> 2) * bi_step];
      xa = make_float2((float)((int)raw[c] + bi.x + rbi), (float)((int)raw[c + 1] + bi.y + rbi));
      xb = make_float2((float)((int)raw[c + 2] + bi.z + rbi), (float)((int)raw[c + 3] + bi.w + rbi));
    } else {
      xa = make_float2(__uint_as_float(raw[c]), __uint_as_float(raw[c + 1]));
      xb = make_float2(__uint_as_float(raw[c + 2]), __uint_as_float(raw[c + 3]));
    }
    v[c >> 1] = fadd2(fadd2(fmul2(fmul2(fmul2(xa, rs2), make_float2(cs.x, cs.y)), alpha2), make_float2(bf.x, bf.y)), rbf2);
    v[(c >> 1) + 1] = fadd2(fadd2(fmul2(fmul2(fmul2(xb, rs2), make_float2(cs.z, cs.w)), alpha2), make_float2(bf.z, bf.w)), rbf2);
  }
  return true;
}

// Second half of the fast path: residual, activation, conversion to the output type, staging.
// split_part (fp32 output as a TF32 pair, EpiParams::split_out): 1 stages hi = tf32(v); 2, called right after 1 on the same
// v, stages lo = tf32(v - hi) and skips the residual and the activation, which call 1 has already applied to v.
template <int W>
__device__ __forceinline__ void epi_finish_fast(const EpiParams &ep, float2 (&v)[W / 2], long long b, long long rr, int col0, uint32_t stage,
                                                int slot, int split_part = 0) {
  constexpr int P = W / 2, CW = W < 32 ? W : 32, NC = W / CW;   // pairs; columns per staging call; staging calls
  if (ep.residual && split_part != 2) {
    const long long roff = b * ep.stride_r + rr * ep.ldr + col0;
    if (ep.residual_dtype == SOFIE_B200_BF16) {
      if (ep.residual_aligned) {
        const uint4 *r = reinterpret_cast<const uint4 *>((const __nv_bfloat16 *)ep.residual + roff);
#pragma unroll
        for (int c = 0; c < W; c += 8) {
          const uint4 q = r[c >> 3];
          const uint32_t ww[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
          for (int u = 0; u < 4; ++u)   // a bf16 is the upper half of the fp32 with the same value
            v[(c >> 1) + u] = fadd2(v[(c >> 1) + u], make_float2(__uint_as_float(ww[u] << 16), __uint_as_float(ww[u] & 0xffff0000u)));
        }
      } else {
        const __nv_bfloat16 *r1 = (const __nv_bfloat16 *)ep.residual + roff;
#pragma unroll
        for (int u = 0; u < P; ++u) v[u] = fadd2(v[u], make_float2(__bfloat162float(r1[2 * u]), __bfloat162float(r1[2 * u + 1])));
      }
    } else {
      const float *r = (const float *)ep.residual + roff;
#pragma unroll
      for (int u = 0; u < P; ++u) v[u] = fadd2(v[u], make_float2(r[2 * u], r[2 * u + 1]));
    }
  }
  if (ep.act != SOFIE_B200_ACT_NONE && split_part != 2) {
    if (ep.act == SOFIE_B200_ACT_RELU) {
#pragma unroll
      for (int u = 0; u < P; ++u) v[u] = make_float2(act_apply(v[u].x, SOFIE_B200_ACT_RELU, 0.f), act_apply(v[u].y, SOFIE_B200_ACT_RELU, 0.f));
    } else if (ep.act == SOFIE_B200_ACT_GELU_ERF) {
      if (ep.y_dtype == SOFIE_B200_BF16) {
#pragma unroll
        for (int u = 0; u < P; ++u) v[u] = gelu_erf_pair_lowp(v[u]);
      } else {
#pragma unroll
        for (int u = 0; u < P; ++u)
          v[u] = make_float2(act_apply(v[u].x, SOFIE_B200_ACT_GELU_ERF, 0.f), act_apply(v[u].y, SOFIE_B200_ACT_GELU_ERF, 0.f));
      }
    } else {
#pragma unroll
      for (int u = 0; u < P; ++u) v[u] = make_float2(act_apply(v[u].x, ep.act, ep.act_alpha), act_apply(v[u].y, ep.act, ep.act_alpha));
    }
  }
  if (ep.y_dtype == SOFIE_B200_BF16) {
#pragma unroll
    for (int i = 0; i < NC; ++i) {
      uint32_t w[CW / 2];
#pragma unroll
      for (int u = 0; u < CW / 2; ++u) {
        __nv_bfloat162 h2 = __floats2bfloat162_rn(v[CW / 2 * i + u].x, v[CW / 2 * i + u].y);
        w[u] = *reinterpret_cast<uint32_t *>(&h2);
      }
      stage_units<CW / 8>(stage, w, slot + i);
    }
  } else if (ep.y_dtype == SOFIE_B200_F32) {
#pragma unroll
    for (int i = 0; i < NC; ++i) {
      uint32_t w[CW];
#pragma unroll
      for (int u = 0; u < CW / 2; ++u) {
        float x = v[CW / 2 * i + u].x, y = v[CW / 2 * i + u].y;
        if (split_part != 0) {
          const float hx = tf32_rn(x), hy = tf32_rn(y);
          x = split_part == 1 ? hx : tf32_rn(__fsub_rn(x, hx));
          y = split_part == 1 ? hy : tf32_rn(__fsub_rn(y, hy));
        }
        w[2 * u] = __float_as_uint(x); w[2 * u + 1] = __float_as_uint(y);
      }
      stage_units<CW / 4>(stage, w, slot + i);
    }
  } else {  // I8 / U8: ONNX rounding (half to even), zero point, saturate
    const int lo = ep.y_dtype == SOFIE_B200_I8 ? -128 : 0, hi = ep.y_dtype == SOFIE_B200_I8 ? 127 : 255;
    const int zp = ep.out_zp;
    if (__builtin_expect(ep.out_scale != 1.f, 0)) {
#pragma unroll
      for (int u = 0; u < P; ++u) v[u] = make_float2(__fdiv_rn(v[u].x, ep.out_scale), __fdiv_rn(v[u].y, ep.out_scale));
    }
    // rint(v) + zp saturated to [lo, hi].  Rounding is monotonic and the bounds are integers, so v is clamped FIRST, to
    // [lo - zp, hi - zp] (NaN goes to the lower bound as fmaxf drops it, like the float formula's saturation), and then
    // rounded half-to-even by adding 1.5 * 2^23: the sum's low mantissa bits are the integer.  Full-rate instructions only
    // (a float-to-int conversion issues at a quarter of the rate).  |lo - zp|, |hi - zp| < 2^22 for any 8-bit zero point.
    const float flo = (float)(lo - zp), fhi = (float)(hi - zp);
    const int unmagic = zp - 0x4B400000;
#pragma unroll
    for (int i = 0; i < NC; ++i) {
      int q[CW];
#pragma unroll
      for (int u = 0; u < CW / 2; ++u) {
        q[2 * u] = __float_as_int(__fadd_rn(fminf(fmaxf(v[CW / 2 * i + u].x, flo), fhi), 12582912.f)) + unmagic;
        q[2 * u + 1] = __float_as_int(__fadd_rn(fminf(fmaxf(v[CW / 2 * i + u].y, flo), fhi), 12582912.f)) + unmagic;
      }
      uint32_t w[CW / 4];
#pragma unroll
      for (int u = 0; u < CW / 4; ++u) {
        const uint32_t lo2 = __byte_perm((uint32_t)q[4 * u], (uint32_t)q[4 * u + 1], 0x0040);      // bytes q0, q1
        const uint32_t hi2 = __byte_perm((uint32_t)q[4 * u + 2], (uint32_t)q[4 * u + 3], 0x0040);  // bytes q2, q3
        w[u] = __byte_perm(lo2, hi2, 0x5410);
      }
      stage_units<CW / 16>(stage, w, slot + i);
    }
  }
}

// Address of element (row0, col) of batch b of Y, in bytes.
__device__ __forceinline__ uint8_t *y_address(const EpiParams &ep, long long b, long long row0, long long col) {
  return (uint8_t *)ep.Y + (b * ep.stride_y + row0 * ep.ldy + col) * out_elem_bytes(ep.y_dtype);
}

}  // namespace sb200
