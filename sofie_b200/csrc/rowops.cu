// LayerNormalization and Softmax: the row-wise memory-bound operators the fusion pass leaves.
//
// Each row is read from HBM exactly once with 128-bit loads into registers, reduced with warp
// shuffles, and written once with 128-bit stores.  A row is owned by a group of G lanes
// (G = 4..32, the smallest power of two whose 16-byte chunks cover the row), so short rows
// (Softmax over 128 attention scores) keep every lane busy and long rows (LayerNorm over
// d_model) use a whole warp.  Rows too long for the register cache, or not 16-byte aligned,
// take a CTA-per-row kernel that re-reads through L2.
//
// Arithmetic follows the reference's CPU code: LayerNorm is two-pass (mean, then biased
// variance of x-mean), invStd = 1/sqrt(var+eps), y = scale*invStd*(x-mean)+bias
// (ROperator_LayerNormalization.hxx:257-312); Softmax is max, exp(x-max), sum, multiply by the
// reciprocal of the sum (ROperator_Softmax.hxx:97-118).
#include <algorithm>

#include "common.cuh"

namespace sb200 {

template <typename T> struct Vec16;  // one 16-byte chunk of T as floats
template <> struct Vec16<float> {
  static constexpr int E = 4;
  static __device__ __forceinline__ void load(const float *p, float *v) {
    float4 t = *reinterpret_cast<const float4 *>(p);
    v[0] = t.x; v[1] = t.y; v[2] = t.z; v[3] = t.w;
  }
  static __device__ __forceinline__ void store(float *p, const float *v) {
    *reinterpret_cast<float4 *>(p) = make_float4(v[0], v[1], v[2], v[3]);
  }
};
template <> struct Vec16<__nv_bfloat16> {
  static constexpr int E = 8;
  static __device__ __forceinline__ void load(const __nv_bfloat16 *p, float *v) {
    uint4 t = *reinterpret_cast<const uint4 *>(p);
    const uint32_t w[4] = {t.x, t.y, t.z, t.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      v[2 * i] = __uint_as_float(w[i] << 16);
      v[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
    }
  }
  static __device__ __forceinline__ void store(__nv_bfloat16 *p, const float *v) {
    uint32_t w[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      __nv_bfloat162 h = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
      w[i] = *reinterpret_cast<uint32_t *>(&h);
    }
    *reinterpret_cast<uint4 *>(p) = make_uint4(w[0], w[1], w[2], w[3]);
  }
};

// Stores E floats (E = elements of one input chunk) as TOut; may take one or two 16-byte stores.
template <typename TOut, int E>
__device__ __forceinline__ void store_chunk_as(TOut *p, const float *v) {
  if constexpr (std::is_same<TOut, float>::value) {
#pragma unroll
    for (int i = 0; i < E; i += 4) Vec16<float>::store(p + i, v + i);
  } else {
    if constexpr (E == 8) {
      Vec16<__nv_bfloat16>::store(p, v);
    } else {  // 4 bf16 = 8 bytes
      __nv_bfloat162 a = __floats2bfloat162_rn(v[0], v[1]), b = __floats2bfloat162_rn(v[2], v[3]);
      *reinterpret_cast<uint2 *>(p) = make_uint2(*reinterpret_cast<uint32_t *>(&a), *reinterpret_cast<uint32_t *>(&b));
    }
  }
}

__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ float group_sum(float v, int G) {
  for (int o = G >> 1; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float group_max(float v, int G) {
  for (int o = G >> 1; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// A 16-byte chunk kept as loaded (bf16 stays packed: two values per register), unpacked at each use.
// Holding the row packed halves the registers a lane needs, which doubles the CTAs per SM and with
// them the bytes in flight -- the kernel is bound by memory latency, not by arithmetic.
__device__ __forceinline__ uint4 ld_raw16(const void *p) { return *reinterpret_cast<const uint4 *>(p); }
template <typename T> __device__ __forceinline__ void unpack16(const uint4 &r, float *v);
template <> __device__ __forceinline__ void unpack16<float>(const uint4 &r, float *v) {
  v[0] = __uint_as_float(r.x); v[1] = __uint_as_float(r.y); v[2] = __uint_as_float(r.z); v[3] = __uint_as_float(r.w);
}
template <> __device__ __forceinline__ void unpack16<__nv_bfloat16>(const uint4 &r, float *v) {
  const uint32_t w[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    v[2 * i] = __uint_as_float(w[i] << 16);
    v[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
  }
}
// The same chunk as pairs of fp32 (the operands of the packed f32x2 instructions).
template <typename T> __device__ __forceinline__ void unpack16_pairs(const uint4 &r, float2 *v);
template <> __device__ __forceinline__ void unpack16_pairs<float>(const uint4 &r, float2 *v) {
  v[0] = make_float2(__uint_as_float(r.x), __uint_as_float(r.y));
  v[1] = make_float2(__uint_as_float(r.z), __uint_as_float(r.w));
}
template <> __device__ __forceinline__ void unpack16_pairs<__nv_bfloat16>(const uint4 &r, float2 *v) {
  const uint32_t w[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) v[i] = make_float2(__uint_as_float(w[i] << 16), __uint_as_float(w[i] & 0xffff0000u));
}
template <typename T> __device__ __forceinline__ uint4 fill16(bool minus_inf);
template <> __device__ __forceinline__ uint4 fill16<float>(bool mi) { const uint32_t u = mi ? 0xff800000u : 0u; return make_uint4(u, u, u, u); }
template <> __device__ __forceinline__ uint4 fill16<__nv_bfloat16>(bool mi) { const uint32_t u = mi ? 0xff80ff80u : 0u; return make_uint4(u, u, u, u); }

// MODE 0: LayerNorm, 1: Softmax, 2: LogSoftmax.  CH = 16-byte chunks cached per lane.
template <typename TIn, typename TOut, int CH, int MODE>
__global__ void __launch_bounds__(256, (MODE == 0 ? (CH >= 16 ? 2 : (CH >= 8 && sizeof(TIn) == 4 ? 3 : 4)) : (CH >= 8 ? 2 : (CH >= 4 && sizeof(TIn) == 4 ? 3 : 4)))) row_group_kernel(const TIn *__restrict__ x, TOut *__restrict__ y, long long rows,
                                                        int cols, int G, const float *__restrict__ scale,
                                                        const float *__restrict__ bias, float eps,
                                                        float *__restrict__ mean_out, float *__restrict__ invstd_out) {
  constexpr int E = Vec16<TIn>::E;
  const int lane = threadIdx.x & 31;
  const int gl = lane & (G - 1);                   // lane within the group
  const int groups_per_cta = blockDim.x / G;
  const long long gid0 = (long long)blockIdx.x * groups_per_cta + threadIdx.x / G;
  const long long gstride = (long long)gridDim.x * groups_per_cta;
  const float inv_n = 1.f / (float)cols;
  const long long iters = (rows + gstride - 1) / gstride;  // same trip count for every thread
  for (long long it = 0; it < iters; ++it) {
    // all lanes of a warp must reach the shuffles: rows beyond the end compute on filler values
    const long long row = gid0 + it * gstride;
    const bool live = row < rows;
    const TIn *xr = x + row * (long long)cols;
    uint4 r[CH];
#pragma unroll
    for (int c = 0; c < CH; ++c) {
      const int col = (c * G + gl) * E;
      r[c] = (live && col < cols) ? ld_raw16(xr + col) : fill16<TIn>(MODE != 0);
    }
    if constexpr (MODE == 0) {
      // LayerNorm on pairs (packed fp32 arithmetic, two values per instruction, each half rounded as the scalar
      // instruction would): the kernel kept the row packed to stay at 4 CTAs per SM and was half issue-bound
      // from unpacking and scalar arithmetic in three passes.
      constexpr int P = E / 2;
      float2 s2 = make_float2(0.f, 0.f);
#pragma unroll
      for (int c = 0; c < CH; ++c) {
        float2 v[P];
        unpack16_pairs<TIn>(r[c], v);
#pragma unroll
        for (int e = 0; e < P; ++e) s2 = __fadd2_rn(s2, v[e]);
      }
      const float mean = group_sum(s2.x + s2.y, G) * inv_n;
      const float2 nmean2 = make_float2(-mean, -mean);
      float2 q2 = make_float2(0.f, 0.f);
#pragma unroll
      for (int c = 0; c < CH; ++c) {
        const int col = (c * G + gl) * E;
        if (col < cols) {
          float2 v[P];
          unpack16_pairs<TIn>(r[c], v);
#pragma unroll
          for (int e = 0; e < P; ++e) { const float2 d = __fadd2_rn(v[e], nmean2); q2 = __ffma2_rn(d, d, q2); }
        }
      }
      const float var = group_sum(q2.x + q2.y, G) * inv_n;
      const float inv = 1.f / sqrtf(var + eps);
      const float2 inv2 = make_float2(inv, inv);
      if (live) {
        TOut *yr = y + row * (long long)cols;
#pragma unroll
        for (int c = 0; c < CH; ++c) {
          const int col = (c * G + gl) * E;
          if (col < cols) {
            float2 v[P];
            float o[E];
            unpack16_pairs<TIn>(r[c], v);
#pragma unroll
            for (int e = 0; e < E; e += 4) {  // scale / bias: 128-bit loads (cols % E == 0 and 16-byte aligned, checked by the host)
              const float4 s4 = scale ? *reinterpret_cast<const float4 *>(scale + col + e) : make_float4(1.f, 1.f, 1.f, 1.f);
              const float4 b4 = bias ? *reinterpret_cast<const float4 *>(bias + col + e) : make_float4(0.f, 0.f, 0.f, 0.f);
              // scale * invStd * (x - mean) + bias, left to right, each step rounded
              float2 t0 = __fadd2_rn(v[e / 2], nmean2), t1 = __fadd2_rn(v[e / 2 + 1], nmean2);
              if (scale) {
                t0 = __fmul2_rn(__fmul2_rn(make_float2(s4.x, s4.y), inv2), t0);
                t1 = __fmul2_rn(__fmul2_rn(make_float2(s4.z, s4.w), inv2), t1);
              } else {
                t0 = __fmul2_rn(inv2, t0);
                t1 = __fmul2_rn(inv2, t1);
              }
              if (bias) {
                t0 = __fadd2_rn(t0, make_float2(b4.x, b4.y));
                t1 = __fadd2_rn(t1, make_float2(b4.z, b4.w));
              }
              o[e] = t0.x; o[e + 1] = t0.y; o[e + 2] = t1.x; o[e + 3] = t1.y;
            }
            store_chunk_as<TOut, E>(yr + col, o);
          }
        }
        if (gl == 0) {
          if (mean_out) mean_out[row] = mean;
          if (invstd_out) invstd_out[row] = inv;
        }
      }
    } else {
      // Softmax keeps the row unpacked: exp(x - max) is computed once and reused for the output
      float v[CH][E];
      float m = -INFINITY;
#pragma unroll
      for (int c = 0; c < CH; ++c) {
        unpack16<TIn>(r[c], v[c]);
#pragma unroll
        for (int e = 0; e < E; ++e) m = fmaxf(m, v[c][e]);
      }
      m = group_max(m, G);
      float s = 0.f;
#pragma unroll
      for (int c = 0; c < CH; ++c) {
        const int col = (c * G + gl) * E;
        if (col < cols) {
#pragma unroll
          for (int e = 0; e < E; ++e) {
            if constexpr (MODE == 1) {
              // a result that is rounded to bf16 (8 significand bits) takes the hardware's base-2 exponential directly
              // (2 ulp of fp32); fp32 results keep expf
              if constexpr (sizeof(TOut) == 2) v[c][e] = fast_exp2(__fmaf_rn(v[c][e], 1.4426950408889634f, -m * 1.4426950408889634f));
              else v[c][e] = expf(v[c][e] - m);
              s += v[c][e];
            } else { v[c][e] = v[c][e] - m; s += expf(v[c][e]); }
          }
        }
      }
      s = group_sum(s, G);
      const float rr = MODE == 1 ? 1.f / s : logf(s);
      if (live) {
        TOut *yr = y + row * (long long)cols;
#pragma unroll
        for (int c = 0; c < CH; ++c) {
          const int col = (c * G + gl) * E;
          if (col < cols) {
            float o[E];
#pragma unroll
            for (int e = 0; e < E; ++e) o[e] = MODE == 1 ? v[c][e] * rr : v[c][e] - rr;
            store_chunk_as<TOut, E>(yr + col, o);
          }
        }
      }
    }
  }
}

// LayerNorm, one warp per row, R rows per trip.  A lane owns the same CH 16-byte chunks of every row it sees, so its scale
// and bias values are loaded ONCE into registers (the group kernel above re-loads them for every chunk of every row:
// four 16-byte loads of parameters per 16-byte load of data, which made it issue-bound at half the memory bandwidth).
// All 16-byte loads of the R rows of a trip are issued before the first use; the rows are unpacked to fp32 once and
// the three passes (sum, squared deviations, output) run on registers; the R reductions of a pass interleave.
template <typename TIn, typename TOut, int CH, int R>
__global__ void __launch_bounds__(256, 2) layernorm_warp_kernel(const TIn *__restrict__ x, TOut *__restrict__ y, long long rows, int cols,
                                                                const float *__restrict__ scale, const float *__restrict__ bias, float eps,
                                                                float *__restrict__ mean_out, float *__restrict__ invstd_out) {
  constexpr int E = Vec16<TIn>::E, P = E / 2;   // elements and fp32 pairs per 16-byte chunk
  const int lane = threadIdx.x & 31;
  const long long warp0 = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const long long nwarps = ((long long)gridDim.x * blockDim.x) >> 5;
  const float inv_n = 1.f / (float)cols;
  // Arithmetic on pairs (packed fp32 instructions: two values per instruction, each half rounded as the scalar instruction
  // rounds it): the kernel was bound by instruction issue at 0.77 of the copy bandwidth with scalar arithmetic.
  float2 sc[CH][P], bi[CH][P];
  bool have[CH];
#pragma unroll
  for (int c = 0; c < CH; ++c) {
    const int col = (c * 32 + lane) * E;
    have[c] = col < cols;
#pragma unroll
    for (int e = 0; e < E; e += 4) {
      const float4 s4 = (have[c] && scale) ? *reinterpret_cast<const float4 *>(scale + col + e) : make_float4(1.f, 1.f, 1.f, 1.f);
      const float4 b4 = (have[c] && bias) ? *reinterpret_cast<const float4 *>(bias + col + e) : make_float4(0.f, 0.f, 0.f, 0.f);
      sc[c][e / 2] = make_float2(s4.x, s4.y); sc[c][e / 2 + 1] = make_float2(s4.z, s4.w);
      bi[c][e / 2] = make_float2(b4.x, b4.y); bi[c][e / 2 + 1] = make_float2(b4.z, b4.w);
    }
  }
  // the loads of the next trip are issued before the arithmetic of the current one: a warp always has R * CH 16-byte loads in flight
  uint4 nxt[R][CH];
  auto fetch = [&](long long r0) {
#pragma unroll
    for (int r = 0; r < R; ++r)
#pragma unroll
      for (int c = 0; c < CH; ++c)
        nxt[r][c] = (r0 + r < rows && have[c]) ? ld_raw16(x + (r0 + r) * (long long)cols + (c * 32 + lane) * E) : fill16<TIn>(false);
  };
  fetch(warp0 * R);
  for (long long row0 = warp0 * R; row0 < rows; row0 += nwarps * R) {
    uint4 raw[R][CH];
#pragma unroll
    for (int r = 0; r < R; ++r)
#pragma unroll
      for (int c = 0; c < CH; ++c) raw[r][c] = nxt[r][c];
    fetch(row0 + nwarps * R);
    // rows go through the arithmetic two at a time (registers: the raw rows of the trip stay packed until their turn)
#pragma unroll
    for (int r0 = 0; r0 < R; r0 += 2) {
      float2 v[2][CH][P];
      float s[2];
#pragma unroll
      for (int r = 0; r < 2; ++r) {
        float2 s2 = make_float2(0.f, 0.f);
#pragma unroll
        for (int c = 0; c < CH; ++c) {
          unpack16_pairs<TIn>(raw[r0 + r][c], v[r][c]);
#pragma unroll
          for (int e = 0; e < P; ++e) s2 = __fadd2_rn(s2, v[r][c][e]);
        }
        s[r] = s2.x + s2.y;
      }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1)
#pragma unroll
        for (int r = 0; r < 2; ++r) s[r] += __shfl_xor_sync(0xffffffffu, s[r], o);
      float mean[2], q[2];
#pragma unroll
      for (int r = 0; r < 2; ++r) {
        mean[r] = s[r] * inv_n;
        const float2 nm = make_float2(-mean[r], -mean[r]);
        float2 q2 = make_float2(0.f, 0.f);
#pragma unroll
        for (int c = 0; c < CH; ++c)
          if (have[c]) {
#pragma unroll
            for (int e = 0; e < P; ++e) { v[r][c][e] = __fadd2_rn(v[r][c][e], nm); q2 = __ffma2_rn(v[r][c][e], v[r][c][e], q2); }
          }
        q[r] = q2.x + q2.y;
      }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1)
#pragma unroll
        for (int r = 0; r < 2; ++r) q[r] += __shfl_xor_sync(0xffffffffu, q[r], o);
#pragma unroll
      for (int r = 0; r < 2; ++r) {
        const long long row = row0 + r0 + r;
        if (row < rows) {
          const float inv = 1.f / sqrtf(q[r] * inv_n + eps);
          const float2 inv2 = make_float2(inv, inv);
          TOut *yr = y + row * (long long)cols;
#pragma unroll
          for (int c = 0; c < CH; ++c)
            if (have[c]) {
              float o[E];
              // scale * invStd * (x - mean) + bias, left to right, each step rounded
#pragma unroll
              for (int e = 0; e < P; ++e) {
                float2 t = scale ? __fmul2_rn(__fmul2_rn(sc[c][e], inv2), v[r][c][e]) : __fmul2_rn(inv2, v[r][c][e]);
                if (bias) t = __fadd2_rn(t, bi[c][e]);
                o[2 * e] = t.x; o[2 * e + 1] = t.y;
              }
              store_chunk_as<TOut, E>(yr + (c * 32 + lane) * E, o);
            }
          if (lane == 0) {
            if (mean_out) mean_out[row] = mean[r];
            if (invstd_out) invstd_out[row] = inv;
          }
        }
      }
    }
  }
}

__device__ __forceinline__ float ld_as_float(const float *p) { return *p; }
__device__ __forceinline__ float ld_as_float(const __nv_bfloat16 *p) { return __bfloat162float(*p); }
__device__ __forceinline__ void st_from_float(float *p, float v) { *p = v; }
__device__ __forceinline__ void st_from_float(__nv_bfloat16 *p, float v) { *p = __float2bfloat16_rn(v); }

template <int OP>  // 0 sum, 1 max
__device__ __forceinline__ float block_reduce(float v, float *sh) {
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
  v = OP == 0 ? group_sum(v, 32) : group_max(v, 32);
  __syncthreads();
  if (lane == 0) sh[w] = v;
  __syncthreads();
  float r = OP == 0 ? 0.f : -INFINITY;
  for (int i = 0; i < (int)(blockDim.x >> 5); ++i) r = OP == 0 ? r + sh[i] : fmaxf(r, sh[i]);
  return r;
}

// One CTA per row, scalar accesses, the row re-read through L2: any length, any alignment.
template <typename TIn, typename TOut, int MODE>
__global__ void __launch_bounds__(256) row_block_kernel(const TIn *__restrict__ x, TOut *__restrict__ y, long long rows,
                                                        long long cols, const float *__restrict__ scale,
                                                        const float *__restrict__ bias, float eps,
                                                        float *__restrict__ mean_out, float *__restrict__ invstd_out) {
  __shared__ float sh[8];
  for (long long row = blockIdx.x; row < rows; row += gridDim.x) {
    const TIn *xr = x + row * cols;
    TOut *yr = y + row * cols;
    if constexpr (MODE == 0) {
      float s = 0.f;
      for (long long c = threadIdx.x; c < cols; c += blockDim.x) s += ld_as_float(xr + c);
      const float mean = block_reduce<0>(s, sh) / (float)cols;
      float q = 0.f;
      for (long long c = threadIdx.x; c < cols; c += blockDim.x) { float d = ld_as_float(xr + c) - mean; q += d * d; }
      const float var = block_reduce<0>(q, sh) / (float)cols;
      const float inv = 1.f / sqrtf(var + eps);
      for (long long c = threadIdx.x; c < cols; c += blockDim.x) {
        const float dlt = ld_as_float(xr + c) - mean;
        float t = scale ? (scale[c] * inv) * dlt : inv * dlt;
        if (bias) t += bias[c];
        st_from_float(yr + c, t);
      }
      if (threadIdx.x == 0) {
        if (mean_out) mean_out[row] = mean;
        if (invstd_out) invstd_out[row] = inv;
      }
    } else {
      float m = -INFINITY;
      for (long long c = threadIdx.x; c < cols; c += blockDim.x) m = fmaxf(m, ld_as_float(xr + c));
      m = block_reduce<1>(m, sh);
      float s = 0.f;
      for (long long c = threadIdx.x; c < cols; c += blockDim.x) s += expf(ld_as_float(xr + c) - m);
      s = block_reduce<0>(s, sh);
      const float r = MODE == 1 ? 1.f / s : logf(s);
      for (long long c = threadIdx.x; c < cols; c += blockDim.x) {
        float d = ld_as_float(xr + c) - m;
        st_from_float(yr + c, MODE == 1 ? expf(d) * r : d - r);
      }
    }
  }
}

template <typename TIn, typename TOut, int MODE>
static int launch_rows(sofie_b200_ctx *ctx, const void *x, void *y, long long rows, long long cols, const float *scale,
                       const float *bias, float eps, float *mean_out, float *invstd_out) {
  constexpr int E = Vec16<TIn>::E;
  cudaStream_t st = ctx->stream;
  const bool aligned = (cols % E == 0) && ((uintptr_t)x % 16 == 0) && ((uintptr_t)scale % 16 == 0) && ((uintptr_t)bias % 16 == 0) &&
                       ((uintptr_t)y % (sizeof(TOut) * E > 16 ? 16 : sizeof(TOut) * E) == 0);
  const long long chunks = (cols + E - 1) / E;
  if (MODE == 0 && aligned && chunks > 16 && chunks <= (sizeof(TIn) == 2 ? 64 : 128) && rows >= 4096) {
    // rows of 16 to 128 chunks, enough of them to fill the machine: one warp per row, parameters in registers
    const int ch = (int)((chunks + 31) / 32);
    const unsigned grid = (unsigned)std::min<long long>((rows + 31) / 32, (long long)ctx->sm_count * 2);
    const TIn *xi = (const TIn *)x;
    TOut *yo = (TOut *)y;
    if constexpr (MODE == 0) {
      if (ch <= 1) layernorm_warp_kernel<TIn, TOut, 1, 4><<<grid, 256, 0, st>>>(xi, yo, rows, (int)cols, scale, bias, eps, mean_out, invstd_out);
      else if (ch <= 2) layernorm_warp_kernel<TIn, TOut, 2, 2><<<grid, 256, 0, st>>>(xi, yo, rows, (int)cols, scale, bias, eps, mean_out, invstd_out);
      else if constexpr (sizeof(TIn) == 4) layernorm_warp_kernel<TIn, TOut, 4, 2><<<grid, 256, 0, st>>>(xi, yo, rows, (int)cols, scale, bias, eps, mean_out, invstd_out);
    }
  } else if (aligned && chunks <= 32 * 16) {
    // Lanes per row: as few as keep <= 8 chunks (128 bytes) per lane, so that each lane has several
    // independent 16-byte loads in flight and the reductions stay short; widened again when there
    // are too few rows to fill the machine.
    int G = 4;
    while (G < 32 && (chunks + G - 1) / G > 8) G <<= 1;
    while (G < 32 && G < chunks && rows * G < (long long)ctx->sm_count * 2048) G <<= 1;
    const int ch = (int)((chunks + G - 1) / G);
    const int groups_per_cta = 256 / G;
    long long ctas = (rows + groups_per_cta - 1) / groups_per_cta;
    const long long cap = (long long)ctas > (long long)ctx->sm_count * 32 ? (long long)ctx->sm_count * 32 : ctas;
    const unsigned grid = (unsigned)(cap < 1 ? 1 : cap);
    const TIn *xi = (const TIn *)x;
    TOut *yo = (TOut *)y;
#define SB_ROW_LAUNCH(CHV) \
  row_group_kernel<TIn, TOut, CHV, MODE><<<grid, 256, 0, st>>>(xi, yo, rows, (int)cols, G, scale, bias, eps, mean_out, invstd_out)
    if (ch <= 1) SB_ROW_LAUNCH(1);
    else if (ch <= 2) SB_ROW_LAUNCH(2);
    else if (ch <= 4) SB_ROW_LAUNCH(4);
    else if (ch <= 8) SB_ROW_LAUNCH(8);
    else SB_ROW_LAUNCH(16);
#undef SB_ROW_LAUNCH
  } else {
    long long g = rows < (long long)ctx->sm_count * 16 ? rows : (long long)ctx->sm_count * 16;
    row_block_kernel<TIn, TOut, MODE><<<(unsigned)g, 256, 0, st>>>((const TIn *)x, (TOut *)y, rows, cols, scale, bias,
                                                                    eps, mean_out, invstd_out);
  }
  SB_CUDA(cudaGetLastError());
  ctx->launches++;
  return 0;
}

template <int MODE>
static int dispatch_rows(sofie_b200_ctx *ctx, const void *x, void *y, int xd, int yd, long long rows, long long cols,
                         const float *scale, const float *bias, float eps, float *mo, float *io) {
  if (xd == SOFIE_B200_F32 && yd == SOFIE_B200_F32) return launch_rows<float, float, MODE>(ctx, x, y, rows, cols, scale, bias, eps, mo, io);
  if (xd == SOFIE_B200_BF16 && yd == SOFIE_B200_BF16) return launch_rows<__nv_bfloat16, __nv_bfloat16, MODE>(ctx, x, y, rows, cols, scale, bias, eps, mo, io);
  if (xd == SOFIE_B200_F32 && yd == SOFIE_B200_BF16) return launch_rows<float, __nv_bfloat16, MODE>(ctx, x, y, rows, cols, scale, bias, eps, mo, io);
  if (xd == SOFIE_B200_BF16 && yd == SOFIE_B200_F32) return launch_rows<__nv_bfloat16, float, MODE>(ctx, x, y, rows, cols, scale, bias, eps, mo, io);
  return fail(SOFIE_B200_ERR_INVALID, "row operator: types %d -> %d not supported (F32 and BF16 only)", xd, yd);
}

// Softmax / LogSoftmax along an axis that is not the last one: x viewed as [outer, n, inner], normalised over n.  One thread
// per (outer, inner) column walks the axis three times (maximum, exp and sum, normalise); neighbouring threads hold
// neighbouring inner positions, so every pass is coalesced.  The generic-axis path of the reference divides by the sum
// (ROperator_Softmax.hxx:120-200), as this does.
template <class T>
__global__ void __launch_bounds__(256) softmax_axis_kernel(const T *__restrict__ x, T *__restrict__ y, long long outer, long long n, long long inner,
                                                           int log_softmax) {
  const long long total = outer * inner;
  for (long long t = (long long)blockIdx.x * blockDim.x + threadIdx.x; t < total; t += (long long)gridDim.x * blockDim.x) {
    const long long o = t / inner, i = t - o * inner;
    const T *xs = x + o * n * inner + i;
    T *ys = y + o * n * inner + i;
    float m = ld_as_float(xs);
    for (long long a = 1; a < n; ++a) m = fmaxf(m, ld_as_float(xs + a * inner));
    float sum = 0.f;
    for (long long a = 0; a < n; ++a) sum += expf(ld_as_float(xs + a * inner) - m);
    const float ls = logf(sum);
    for (long long a = 0; a < n; ++a) {
      const float v = ld_as_float(xs + a * inner) - m;
      st_from_float(ys + a * inner, log_softmax ? v - ls : __fdiv_rn(expf(v), sum));
    }
  }
}

}  // namespace sb200

using namespace sb200;

extern "C" {

int sofie_b200_layernorm_enqueue(sofie_b200_ctx *ctx, const void *x, void *y, int32_t x_dtype, int32_t y_dtype,
                                 int64_t rows, int64_t cols, const float *scale, const float *bias, float eps,
                                 float *mean_out, float *invstd_out) {
  if (!ctx) return fail(SOFIE_B200_ERR_INVALID, "layernorm_enqueue: ctx is NULL");
  if (rows < 0 || cols < 0) return fail(SOFIE_B200_ERR_INVALID, "layernorm_enqueue: negative extent");
  if (rows == 0 || cols == 0) return 0;
  if (!x || !y) return fail(SOFIE_B200_ERR_INVALID, "layernorm_enqueue: NULL tensor");
  SB_CUDA(cudaSetDevice(ctx->device));
  return dispatch_rows<0>(ctx, x, y, x_dtype, y_dtype, rows, cols, scale, bias, eps, mean_out, invstd_out);
}

int sofie_b200_softmax_enqueue(sofie_b200_ctx *ctx, const void *x, void *y, int32_t x_dtype, int32_t y_dtype,
                               int64_t rows, int64_t cols, int32_t log_softmax) {
  if (!ctx) return fail(SOFIE_B200_ERR_INVALID, "softmax_enqueue: ctx is NULL");
  if (rows < 0 || cols < 0) return fail(SOFIE_B200_ERR_INVALID, "softmax_enqueue: negative extent");
  if (rows == 0 || cols == 0) return 0;
  if (!x || !y) return fail(SOFIE_B200_ERR_INVALID, "softmax_enqueue: NULL tensor");
  SB_CUDA(cudaSetDevice(ctx->device));
  if (log_softmax) return dispatch_rows<2>(ctx, x, y, x_dtype, y_dtype, rows, cols, nullptr, nullptr, 0.f, nullptr, nullptr);
  return dispatch_rows<1>(ctx, x, y, x_dtype, y_dtype, rows, cols, nullptr, nullptr, 0.f, nullptr, nullptr);
}

int sofie_b200_softmax_axis_enqueue(sofie_b200_ctx *ctx, const void *x, void *y, int32_t dtype, int64_t outer, int64_t n, int64_t inner,
                                    int32_t log_softmax) {
  if (!ctx) return fail(SOFIE_B200_ERR_INVALID, "softmax_axis_enqueue: ctx is NULL");
  if (outer < 0 || n < 0 || inner < 0) return fail(SOFIE_B200_ERR_INVALID, "softmax_axis_enqueue: negative extent");
  if (outer * n * inner == 0) return 0;
  if (!x || !y) return fail(SOFIE_B200_ERR_INVALID, "softmax_axis_enqueue: NULL tensor");
  SB_CUDA(cudaSetDevice(ctx->device));
  if (inner == 1) return sofie_b200_softmax_enqueue(ctx, x, y, dtype, dtype, outer, n, log_softmax);
  const long long total = outer * inner;
  const unsigned grid = (unsigned)std::min<long long>((total + 255) / 256, (long long)ctx->sm_count * 16);
  if (dtype == SOFIE_B200_F32) softmax_axis_kernel<float><<<grid, 256, 0, ctx->stream>>>((const float *)x, (float *)y, outer, n, inner, log_softmax);
  else if (dtype == SOFIE_B200_BF16)
    softmax_axis_kernel<__nv_bfloat16><<<grid, 256, 0, ctx->stream>>>((const __nv_bfloat16 *)x, (__nv_bfloat16 *)y, outer, n, inner, log_softmax);
  else return fail(SOFIE_B200_ERR_INVALID, "softmax_axis_enqueue: type %d not supported (F32, BF16)", dtype);
  SB_CUDA(cudaGetLastError());
  ctx->launches++;
  return 0;
}

}  // extern "C"
