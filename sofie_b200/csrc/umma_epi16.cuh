// Epilogue of the tcgen05 contraction kernel (gemm_umma.cu): an epilogue warp drains its 32 tensor-memory lanes of a
// finished accumulator in steps of 16 columns through the fused epilogue into a staging buffer in shared memory, and a
// complete 64-byte row segment leaves as one bulk tensor store.
//
// The epilogue is bound by instruction issue (ncu: two thirds of the issue slots busy, no memory unit near its limit), so
// this file is about instructions per element:
//   - the output type is a template argument of the drain loop, chosen once per tile;
//   - which parts of the epilogue formula exist is a bit mask taken once per kernel (EPI16_*): an absent part is skipped
//     behind one warp-uniform branch instead of multiplying by 1.0f or adding -0.0f (both exact: same bits);
//   - 8-bit outputs are rounded, shifted by the zero point and saturated in three instructions per pair of elements;
//   - the staging address of a lane is a base and an XOR term fixed for the kernel.
// Everything the fast path does not cover (unaligned Y, a full-matrix bias, ragged tile edges) goes through store_chunk().
#pragma once
#include "umma_store.cuh"

namespace sb200 {

enum : uint32_t {
  EPI16_RS = 1u, EPI16_CS = 2u, EPI16_ALPHA = 4u, EPI16_BF = 8u, EPI16_RBF_ROW = 16u, EPI16_RBF_SCALAR = 32u,
  EPI16_BI = 64u, EPI16_RBI = 128u, EPI16_RES = 256u, EPI16_ACT = 512u, EPI16_OUT_SCALE = 1024u
};
__device__ __forceinline__ uint32_t epi16_flags(const EpiParams &ep) {
  uint32_t f = 0;
  if (ep.row_scale) f |= EPI16_RS;
  if (ep.col_scale) f |= EPI16_CS;
  if (ep.alpha != 1.f) f |= EPI16_ALPHA;
  if (ep.bias_mode == SOFIE_B200_BIAS_COL_F32) f |= EPI16_BF;
  if (ep.bias_mode == SOFIE_B200_BIAS_ROW_F32) f |= EPI16_RBF_ROW;
  if (ep.bias_mode == SOFIE_B200_BIAS_SCALAR_F32) f |= EPI16_RBF_SCALAR;
  if (ep.bias_mode == SOFIE_B200_BIAS_COL_I32) f |= EPI16_BI;
  if (ep.bias_mode == SOFIE_B200_BIAS_ROW_I32) f |= EPI16_RBI;
  if (ep.residual) f |= EPI16_RES;
  if (ep.act != SOFIE_B200_ACT_NONE) f |= EPI16_ACT;
  if (ep.out_scale != 1.f) f |= EPI16_OUT_SCALE;
  return f;
}

constexpr uint32_t EPI16_DYNAMIC = 0x80000000u;

enum { OUT16_F32 = 0, OUT16_BF16 = 1, OUT16_I8 = 2, OUT16_U8 = 3, OUT16_I32 = 4 };
__device__ __forceinline__ int out16_class(int y_dtype) {
  return y_dtype == SOFIE_B200_F32 ? OUT16_F32 : y_dtype == SOFIE_B200_BF16 ? OUT16_BF16 : y_dtype == SOFIE_B200_I8 ? OUT16_I8
       : y_dtype == SOFIE_B200_U8 ? OUT16_U8 : OUT16_I32;
}

// What an epilogue warp keeps for the whole kernel.
struct Epi16Warp {
  uint32_t fl;        // EPI16_* of the plan's epilogue
  uint32_t stage;     // staging buffer of the warp (shared-memory address) | pitch code (stage_units)
  uint32_t row_addr;  // this lane's row of the buffer
  uint32_t row_xor;   // swizzle term of that row: unit at byte offset o of the row lives at row_addr + (o ^ row_xor)
  int steps_per_seg;  // 16-column steps per flushed row segment
  int seg_units;      // 16-byte units of a complete segment
  int out_class;      // OUT16_*
};
// WIDE: 128-byte segments in a 4 KB buffer (twice the steps of a 64-byte segment; pitch code 0).
template <bool WIDE = false>
__device__ __forceinline__ Epi16Warp epi16_warp_init(const EpiParams &ep, uint32_t stage_base) {
  Epi16Warp w;
  w.fl = epi16_flags(ep);
  w.out_class = out16_class(ep.y_dtype);
  const int G_full = chunks_per_flush(ep.y_dtype);   // steps per 64-byte segment: 1 (4-byte), 2 (2-byte), 4 (1-byte outputs)
  const int G = WIDE ? 2 * G_full : (ep.seg_chunks > 0 && ep.seg_chunks < G_full ? ep.seg_chunks : G_full);
  const uint32_t code = WIDE ? 0u : (G == G_full) ? 1u : (2 * G == G_full ? 2u : 3u);   // row pitch 128, 64, 32 or 16 bytes
  w.stage = stage_base | code;
  w.steps_per_seg = G;
  w.seg_units = 4 * G / G_full;
  const uint32_t a = (threadIdx.x & 31u) * (128u >> code);
  w.row_addr = stage_base + a;
  w.row_xor = ((a >> 7) & (7u >> code)) << 4;
  return w;
}

__device__ __forceinline__ void st_shared_v4(uint32_t addr, uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
  asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(a), "r"(b), "r"(c), "r"(d) : "memory");
}

// rint(v) + zp, saturated to the 8-bit output type, for four values -> four bytes (v0 lowest).  v is first bounded below
// by `lower`: -2^22 (which also sends a NaN there, as the float formula's saturation does), or 0 when a Relu precedes the
// quantisation -- max(v, 0) is that Relu (a NaN and -0 both end as the integer 0 either way), so the activation costs no
// instruction of its own; then v + 1.5 * 2^23 holds rint(v) in
// its low mantissa bits for |v| < 2^22 and is monotonic in v above that, as are the bits of a positive float read as an
// integer; the integer addition takes the exponent bits away and adds the zero point, and the packing conversion
// saturates to [-128, 127] or [0, 255].  Full-rate instructions only: 2.5 per element.  (A saturating integer subtraction
// instead of the lower bound costs eight instructions: the target has none.)
template <bool SIGNED>
__device__ __forceinline__ uint32_t quantize4(float2 lo, float2 hi, int unmagic, float lower) {
  const float2 m = dup2(12582912.f);
  const float2 a = fadd2(make_float2(fmaxf(lo.x, lower), fmaxf(lo.y, lower)), m);
  const float2 b = fadd2(make_float2(fmaxf(hi.x, lower), fmaxf(hi.y, lower)), m);
  const int q0 = __float_as_int(a.x) - unmagic, q1 = __float_as_int(a.y) - unmagic, q2 = __float_as_int(b.x) - unmagic, q3 = __float_as_int(b.y) - unmagic;
  uint32_t out;
  if (SIGNED) {
    asm("{\n"
        ".reg .b32 h;\n"
        "cvt.pack.sat.s8.s32.b32 h, %4, %3, 0;\n"
        "cvt.pack.sat.s8.s32.b32 %0, %2, %1, h;\n"
        "}\n"
        : "=r"(out)
        : "r"(q0), "r"(q1), "r"(q2), "r"(q3));
  } else {
    asm("{\n"
        ".reg .b32 h;\n"
        "cvt.pack.sat.u8.s32.b32 h, %4, %3, 0;\n"
        "cvt.pack.sat.u8.s32.b32 %0, %2, %1, h;\n"
        "}\n"
        : "=r"(out)
        : "r"(q0), "r"(q1), "r"(q2), "r"(q3));
  }
  return out;
}

// One 16-column step of the fast path: raw accumulator -> output type -> staging buffer, at position `j` of the row
// segment.  The next step's accumulator columns are requested into `raw` as soon as `raw` is dead.
//
// FL: the plan's EPI16_* mask as a compile-time constant, or EPI16_DYNAMIC to read it from `w`.  With the mask in a
// register the compiler turns the short optional parts into predicated code, and a predicated-off instruction still
// takes its issue slot: a step with only alpha set executed the loads and arithmetic of every other part as well, half
// of its instructions.  The masks of the common epilogues are therefore instantiated (drain16_any picks per tile).
template <bool ACC_INT, int OUT, uint32_t FL>
__device__ __forceinline__ void epi16_step(const EpiParams &ep, const Epi16Warp &w, uint32_t (&raw)[16], uint32_t next_taddr, bool has_next,
                                           long long b, long long rr, int col0, int j) {
  const uint32_t fl = FL == EPI16_DYNAMIC ? w.fl : FL;
  constexpr int UNITS = OUT == OUT16_BF16 ? 2 : (OUT == OUT16_I8 || OUT == OUT16_U8) ? 1 : 4;   // 16-byte units per step
  const uint32_t o0 = ((uint32_t)(j * UNITS * 16)) ^ w.row_xor;
  if (ACC_INT) {
    if (fl & EPI16_BI) {
      const int4 *bip = reinterpret_cast<const int4 *>((const int *)ep.bias + col0);
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        const int4 bi = bip[q];
        raw[4 * q] += (uint32_t)bi.x; raw[4 * q + 1] += (uint32_t)bi.y; raw[4 * q + 2] += (uint32_t)bi.z; raw[4 * q + 3] += (uint32_t)bi.w;
      }
    }
    if (fl & EPI16_RBI) {
      const uint32_t rbi = (uint32_t)((const int *)ep.bias)[rr];
#pragma unroll
      for (int c = 0; c < 16; ++c) raw[c] += rbi;
    }
  }
  if (OUT == OUT16_I32) {
#pragma unroll
    for (int u = 0; u < 4; ++u) st_shared_v4(w.row_addr + (o0 ^ (16u * u)), raw[4 * u], raw[4 * u + 1], raw[4 * u + 2], raw[4 * u + 3]);
    if (has_next) ptx::tmem_ld_x16(next_taddr, raw);
    return;
  }
  float2 v[8];
  if (ACC_INT) {
#pragma unroll
    for (int u = 0; u < 8; ++u) v[u] = make_float2((float)(int)raw[2 * u], (float)(int)raw[2 * u + 1]);
  } else {
#pragma unroll
    for (int u = 0; u < 8; ++u) v[u] = make_float2(__uint_as_float(raw[2 * u]), __uint_as_float(raw[2 * u + 1]));
  }
  if (fl & EPI16_RS) {
    const float2 rs2 = dup2(ep.row_scale[rr]);
#pragma unroll
    for (int u = 0; u < 8; ++u) v[u] = fmul2(v[u], rs2);
  }
  if (fl & EPI16_CS) {
    const float4 *csp = reinterpret_cast<const float4 *>(ep.col_scale + col0);
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      const float4 cs = csp[q];
      v[2 * q] = fmul2(v[2 * q], make_float2(cs.x, cs.y));
      v[2 * q + 1] = fmul2(v[2 * q + 1], make_float2(cs.z, cs.w));
    }
  }
  if (fl & EPI16_ALPHA) {
    const float2 alpha2 = dup2(ep.alpha);
#pragma unroll
    for (int u = 0; u < 8; ++u) v[u] = fmul2(v[u], alpha2);
  }
  if (fl & EPI16_BF) {
    const float4 *bfp = reinterpret_cast<const float4 *>((const float *)ep.bias + col0);
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      const float4 bf = bfp[q];
      v[2 * q] = fadd2(v[2 * q], make_float2(bf.x, bf.y));
      v[2 * q + 1] = fadd2(v[2 * q + 1], make_float2(bf.z, bf.w));
    }
  }
  if (fl & (EPI16_RBF_ROW | EPI16_RBF_SCALAR)) {
    const float2 rbf2 = dup2(((const float *)ep.bias)[(fl & EPI16_RBF_ROW) ? rr : 0]);
#pragma unroll
    for (int u = 0; u < 8; ++u) v[u] = fadd2(v[u], rbf2);
  }
  if (has_next) ptx::tmem_ld_x16(next_taddr, raw);   // flies during the rest of the step
  if (fl & EPI16_RES) {
    const long long roff = b * ep.stride_r + rr * ep.ldr + col0;
    if (ep.residual_dtype == SOFIE_B200_BF16) {
      if (ep.residual_aligned == 2) {
        // one 256-bit load: a lane reads its own row, so every load instruction touches 32 lines, and the load unit's
        // time per line -- not latency -- made two 128-bit loads per step cost a third of a short-K tile's time
        uint32_t ww[8];
        asm volatile("ld.global.v8.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
                     : "=r"(ww[0]), "=r"(ww[1]), "=r"(ww[2]), "=r"(ww[3]), "=r"(ww[4]), "=r"(ww[5]), "=r"(ww[6]), "=r"(ww[7])
                     : "l"((const __nv_bfloat16 *)ep.residual + roff));
#pragma unroll
        for (int u = 0; u < 8; ++u)   // a bf16 is the upper half of the fp32 with the same value
          v[u] = fadd2(v[u], make_float2(__uint_as_float(ww[u] << 16), __uint_as_float(ww[u] & 0xffff0000u)));
      } else if (ep.residual_aligned) {
        const uint4 *r = reinterpret_cast<const uint4 *>((const __nv_bfloat16 *)ep.residual + roff);
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          const uint4 q = r[h];
          const uint32_t ww[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
          for (int u = 0; u < 4; ++u)   // a bf16 is the upper half of the fp32 with the same value
            v[4 * h + u] = fadd2(v[4 * h + u], make_float2(__uint_as_float(ww[u] << 16), __uint_as_float(ww[u] & 0xffff0000u)));
        }
      } else {
        const __nv_bfloat16 *r1 = (const __nv_bfloat16 *)ep.residual + roff;
#pragma unroll
        for (int u = 0; u < 8; ++u) v[u] = fadd2(v[u], make_float2(__bfloat162float(r1[2 * u]), __bfloat162float(r1[2 * u + 1])));
      }
    } else {
      const float *r = (const float *)ep.residual + roff;
#pragma unroll
      for (int u = 0; u < 8; ++u) v[u] = fadd2(v[u], make_float2(r[2 * u], r[2 * u + 1]));
    }
  }
  constexpr bool OUT8 = OUT == OUT16_I8 || OUT == OUT16_U8;
  float q_lower = -4194304.f;   // lower bound of the 8-bit quantiser
  if (fl & EPI16_ACT) {
    if (ep.act == SOFIE_B200_ACT_RELU) {
      if (OUT8 && !(fl & EPI16_OUT_SCALE)) {
        q_lower = 0.f;          // the quantiser's lower bound is the Relu
      } else {
#pragma unroll
        for (int u = 0; u < 8; ++u) v[u] = make_float2(act_apply(v[u].x, SOFIE_B200_ACT_RELU, 0.f), act_apply(v[u].y, SOFIE_B200_ACT_RELU, 0.f));
      }
    } else if (ep.act == SOFIE_B200_ACT_GELU_ERF) {
      if (OUT == OUT16_BF16) {
#pragma unroll
        for (int u = 0; u < 8; ++u) v[u] = gelu_erf_pair_lowp(v[u]);
      } else {
#pragma unroll
        for (int u = 0; u < 8; ++u)
          v[u] = make_float2(act_apply(v[u].x, SOFIE_B200_ACT_GELU_ERF, 0.f), act_apply(v[u].y, SOFIE_B200_ACT_GELU_ERF, 0.f));
      }
    } else {
#pragma unroll
      for (int u = 0; u < 8; ++u) v[u] = make_float2(act_apply(v[u].x, ep.act, ep.act_alpha), act_apply(v[u].y, ep.act, ep.act_alpha));
    }
  }
  if (OUT == OUT16_BF16) {
    uint32_t p[8];
#pragma unroll
    for (int u = 0; u < 8; ++u) {
      __nv_bfloat162 h2 = __floats2bfloat162_rn(v[u].x, v[u].y);
      p[u] = *reinterpret_cast<uint32_t *>(&h2);
    }
    st_shared_v4(w.row_addr + o0, p[0], p[1], p[2], p[3]);
    st_shared_v4(w.row_addr + (o0 ^ 16u), p[4], p[5], p[6], p[7]);
  } else if (OUT == OUT16_F32) {
#pragma unroll
    for (int u = 0; u < 4; ++u)
      st_shared_v4(w.row_addr + (o0 ^ (16u * u)), __float_as_uint(v[2 * u].x), __float_as_uint(v[2 * u].y), __float_as_uint(v[2 * u + 1].x),
                   __float_as_uint(v[2 * u + 1].y));
  } else {  // I8 / U8: ONNX rounding (half to even), zero point, saturate
    if (__builtin_expect((fl & EPI16_OUT_SCALE) != 0, 0)) {
#pragma unroll
      for (int u = 0; u < 8; ++u) v[u] = make_float2(__fdiv_rn(v[u].x, ep.out_scale), __fdiv_rn(v[u].y, ep.out_scale));
    }
    const int unmagic = 0x4B400000 - ep.out_zp;
    uint32_t p[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) p[u] = quantize4<OUT == OUT16_I8>(v[2 * u], v[2 * u + 1], unmagic, q_lower);
    st_shared_v4(w.row_addr + o0, p[0], p[1], p[2], p[3]);
  }
}

// One epilogue warp drains its share of a finished accumulator: the 32 tensor-memory lanes at `taddr` (lane = row `row` of
// Y), columns [0, c_end) of the tile that starts at column n0 of Y.  Steps of 16 columns are taken in groups of
// w.steps_per_seg consecutive steps (one row segment); this warp takes groups first_group, first_group + group_stride, ...
//
// With a tensor map of Y (`tm_y`; box = one segment x 32 rows, swizzle = the segment's width: exactly the staging buffer's
// layout) a complete row segment leaves as ONE bulk tensor store issued by lane 0: the TMA unit clips rows past the end.
// The buffer is reused only after the store has read it (bulk_wait_read_all before the next segment is staged, and before
// the function returns).
template <bool ACC_INT, int OUT, uint32_t FL>
__device__ __forceinline__ void drain16(const EpiParams &ep, const Epi16Warp &w, uint32_t taddr, int c_end, int first_group, int group_stride,
                                        long long b, long long row, int n0, bool vec, long long rows_total, const CUtensorMap *tm_y, const CUtensorMap *tm_peers) {
  const int G = w.steps_per_seg;
  const int nst = (c_end + 15) >> 4;
  int st = first_group * G, j = 0;   // current step and its position in its segment
  if (st >= nst) return;
  constexpr int UNITS = OUT == OUT16_BF16 ? 2 : (OUT == OUT16_I8 || OUT == OUT16_U8) ? 1 : 4;
  const long long row0 = row - (threadIdx.x & 31);
  const long long left = rows_total - row0;
  const int rows_valid = left < 0 ? 0 : (left > 32 ? 32 : (int)left);
  const bool fast = vec && ep.fast && rows_valid > 0;
  const long long rr = row < rows_total ? row : rows_total - 1;   // rows past the end compute on the last row's operands
  int units = 0, seg_col = 0;
  bool store_pending = false;
  uint32_t raw[16];
  ptx::tmem_ld_x16(taddr + 16 * st, raw);
#pragma unroll 1
  while (true) {
    int st2 = st + 1, j2 = j + 1;
    if (j2 >= G) { j2 = 0; st2 += (group_stride - 1) * G; }
    const bool has_next = st2 < nst;
    const int c = 16 * st;
    if (j == 0) {
      units = 0; seg_col = c;
      if (store_pending) {   // the previous segment's bulk store must have read the buffer before it is refilled
        if ((threadIdx.x & 31) == 0) ptx::bulk_wait_read_all();
        __syncwarp();
        store_pending = false;
      }
    }
    ptx::tmem_ld_wait();
    if (fast && c_end - c >= 16) {
      epi16_step<ACC_INT, OUT, FL>(ep, w, raw, taddr + 16 * st2, has_next, b, rr, n0 + c, j);
      units += UNITS;
    } else {
      if (store_chunk<16>(ep, raw, b, row, n0 + c, min(16, c_end - c), vec, w.stage, rows_total, j)) units += UNITS;
      if (has_next) ptx::tmem_ld_x16(taddr + 16 * st2, raw);
    }
    if ((j == G - 1 || !has_next) && units > 0) {
      if (tm_y != nullptr && units == w.seg_units) {
        ptx::fence_proxy_async();   // this lane's staging writes become visible to the TMA unit
        __syncwarp();
        if ((threadIdx.x & 31) == 0) {
          ptx::tma_store_3d(tm_y, w.stage & ~3u, n0 + seg_col, (int)row0, (int)b);
          if constexpr (!ACC_INT)   // the int8 kernels sit at the register limit: the peer stores exist for the floating kinds only
            for (int q = 0; q < ep.y_peers; ++q)   // the same segment into every peer's copy of Y (over NVLink when it is another GPU's)
            ptx::tma_store_3d(tm_peers + q, w.stage & ~3u, n0 + seg_col, (int)row0, (int)b);
          ptx::bulk_commit_group();
        }
        store_pending = true;
      } else {
        flush_staged(w.stage, y_address(ep, b, row0, n0 + seg_col), ep.ldy * out_elem_bytes(ep.y_dtype), rows_valid, units);
      }
    }
    st = st2; j = j2;
    if (!has_next) break;
  }
  if (store_pending) {
    if ((threadIdx.x & 31) == 0) ptx::bulk_wait_read_all();
    __syncwarp();
  }
}

// drain16 with the plan's mask as a constant where it is one of the common ones, else with the mask in a register.
template <bool ACC_INT, int OUT>
__device__ __forceinline__ void drain16_masks(const EpiParams &ep, const Epi16Warp &w, uint32_t taddr, int c_end, int first_group, int group_stride,
                                              long long b, long long row, int n0, bool vec, long long rows_total, const CUtensorMap *tm_y, const CUtensorMap *tm_peers) {
#define SB200_DRAIN16(MASK)                                                                                                  \
  if (w.fl == (MASK)) return drain16<ACC_INT, OUT, (MASK)>(ep, w, taddr, c_end, first_group, group_stride, b, row, n0, vec, rows_total, tm_y, tm_peers)
  if (ACC_INT && (OUT == OUT16_I8 || OUT == OUT16_BF16)) {
    SB200_DRAIN16(EPI16_ALPHA);                                   // QLinearMatMul with per-tensor scales
    SB200_DRAIN16(EPI16_CS | EPI16_BI);                           // QLinearConv
    SB200_DRAIN16(EPI16_CS | EPI16_BI | EPI16_ACT);               // ... with a fused activation
  }
  if (!ACC_INT && OUT == OUT16_BF16) {
    SB200_DRAIN16(0u);
    SB200_DRAIN16(EPI16_ALPHA);
    SB200_DRAIN16(EPI16_CS | EPI16_BF);                           // dequantised weights, bias
    SB200_DRAIN16(EPI16_CS | EPI16_BF | EPI16_ACT);
    SB200_DRAIN16(EPI16_CS | EPI16_BF | EPI16_RES);
    SB200_DRAIN16(EPI16_RS | EPI16_CS | EPI16_BF | EPI16_ACT);    // FP8 with row and column scales
  }
#undef SB200_DRAIN16
  drain16<ACC_INT, OUT, EPI16_DYNAMIC>(ep, w, taddr, c_end, first_group, group_stride, b, row, n0, vec, rows_total, tm_y, tm_peers);
}

template <bool ACC_INT>
__device__ __forceinline__ void drain16_any(const EpiParams &ep, const Epi16Warp &w, uint32_t taddr, int c_end, int first_group, int group_stride,
                                            long long b, long long row, int n0, bool vec, long long rows_total, const CUtensorMap *tm_y, const CUtensorMap *tm_peers) {
  switch (w.out_class) {
    case OUT16_F32: drain16_masks<ACC_INT, OUT16_F32>(ep, w, taddr, c_end, first_group, group_stride, b, row, n0, vec, rows_total, tm_y, tm_peers); break;
    case OUT16_BF16: drain16_masks<ACC_INT, OUT16_BF16>(ep, w, taddr, c_end, first_group, group_stride, b, row, n0, vec, rows_total, tm_y, tm_peers); break;
    case OUT16_I8: drain16_masks<ACC_INT, OUT16_I8>(ep, w, taddr, c_end, first_group, group_stride, b, row, n0, vec, rows_total, tm_y, tm_peers); break;
    case OUT16_U8: drain16_masks<ACC_INT, OUT16_U8>(ep, w, taddr, c_end, first_group, group_stride, b, row, n0, vec, rows_total, tm_y, tm_peers); break;
    default:
      if (ACC_INT) drain16_masks<true, OUT16_I32>(ep, w, taddr, c_end, first_group, group_stride, b, row, n0, vec, rows_total, tm_y, tm_peers);
      break;
  }
}

}  // namespace sb200
