// Standalone elementwise operators: unary activations, broadcast binary ops, inference
// BatchNormalization, GlobalAveragePool, Quantize/DequantizeLinear and type conversion.
// All are HBM-bound: 128-bit accesses on the aligned body, scalar accesses on the ragged tail,
// grid sized to a multiple of the SM count with a grid-stride loop.
#include "epilogue.cuh"

namespace sb200 {

static inline unsigned grid_for(const sofie_b200_ctx *ctx, long long work_items, int threads) {
  long long blocks = (work_items + threads - 1) / threads;
  long long cap = (long long)ctx->sm_count * 16;
  if (blocks > cap) blocks = cap;
  if (blocks < 1) blocks = 1;
  return (unsigned)blocks;
}

__device__ __forceinline__ float binop(float a, float b, int op) {
  switch (op) {
    case 0: return __fadd_rn(a, b);
    case 1: return __fsub_rn(a, b);
    case 2: return __fmul_rn(a, b);
    default: return __fdiv_rn(a, b);
  }
}

// ---- unary --------------------------------------------------------------------------------
__global__ void __launch_bounds__(256) unary_f32_kernel(const float *__restrict__ x, float *__restrict__ y, long long n,
                                                        int act, float aa, int vec) {
  const long long tid = (long long)blockIdx.x * blockDim.x + threadIdx.x, nth = (long long)gridDim.x * blockDim.x;
  long long body = vec ? n / 4 : 0;
  for (long long i = tid; i < body; i += nth) {
    float4 v = reinterpret_cast<const float4 *>(x)[i];
    v.x = act_apply(v.x, act, aa); v.y = act_apply(v.y, act, aa); v.z = act_apply(v.z, act, aa); v.w = act_apply(v.w, act, aa);
    reinterpret_cast<float4 *>(y)[i] = v;
  }
  for (long long i = body * 4 + tid; i < n; i += nth) y[i] = act_apply(x[i], act, aa);
}

__global__ void __launch_bounds__(256) unary_bf16_kernel(const __nv_bfloat16 *__restrict__ x, __nv_bfloat16 *__restrict__ y,
                                                         long long n, int act, float aa, int vec) {
  const long long tid = (long long)blockIdx.x * blockDim.x + threadIdx.x, nth = (long long)gridDim.x * blockDim.x;
  long long body = vec ? n / 8 : 0;
  for (long long i = tid; i < body; i += nth) {
    uint4 t = reinterpret_cast<const uint4 *>(x)[i];
    uint32_t w[4] = {t.x, t.y, t.z, t.w};
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      float lo = act_apply(__uint_as_float(w[k] << 16), act, aa);
      float hi = act_apply(__uint_as_float(w[k] & 0xffff0000u), act, aa);
      __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
      w[k] = *reinterpret_cast<uint32_t *>(&h);
    }
    reinterpret_cast<uint4 *>(y)[i] = make_uint4(w[0], w[1], w[2], w[3]);
  }
  for (long long i = body * 8 + tid; i < n; i += nth) y[i] = __float2bfloat16_rn(act_apply(__bfloat162float(x[i]), act, aa));
}

// ---- binary with trailing broadcast: y[i] = a[i] op b[i % nb] ------------------------------
__global__ void __launch_bounds__(256) binary_f32_kernel(const float *__restrict__ a, const float *__restrict__ b,
                                                         float *__restrict__ y, long long n, long long nb, int op, int act,
                                                         int vec) {
  const long long tid = (long long)blockIdx.x * blockDim.x + threadIdx.x, nth = (long long)gridDim.x * blockDim.x;
  long long body = vec ? n / 4 : 0;
  for (long long i = tid; i < body; i += nth) {
    float4 va = reinterpret_cast<const float4 *>(a)[i];
    float4 vb = reinterpret_cast<const float4 *>(b)[nb == n ? i : (i * 4 % nb) / 4];
    va.x = act_apply(binop(va.x, vb.x, op), act, 0.f); va.y = act_apply(binop(va.y, vb.y, op), act, 0.f);
    va.z = act_apply(binop(va.z, vb.z, op), act, 0.f); va.w = act_apply(binop(va.w, vb.w, op), act, 0.f);
    reinterpret_cast<float4 *>(y)[i] = va;
  }
  for (long long i = body * 4 + tid; i < n; i += nth) y[i] = act_apply(binop(a[i], b[i % nb], op), act, 0.f);
}

__global__ void __launch_bounds__(256) binary_bf16_kernel(const __nv_bfloat16 *__restrict__ a, const __nv_bfloat16 *__restrict__ b,
                                                          __nv_bfloat16 *__restrict__ y, long long n, long long nb, int op,
                                                          int act, int vec) {
  const long long tid = (long long)blockIdx.x * blockDim.x + threadIdx.x, nth = (long long)gridDim.x * blockDim.x;
  long long body = vec ? n / 8 : 0;
  for (long long i = tid; i < body; i += nth) {
    uint4 ta = reinterpret_cast<const uint4 *>(a)[i];
    uint4 tb = reinterpret_cast<const uint4 *>(b)[nb == n ? i : (i * 8 % nb) / 8];
    uint32_t wa[4] = {ta.x, ta.y, ta.z, ta.w}, wb[4] = {tb.x, tb.y, tb.z, tb.w};
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      float lo = act_apply(binop(__uint_as_float(wa[k] << 16), __uint_as_float(wb[k] << 16), op), act, 0.f);
      float hi = act_apply(binop(__uint_as_float(wa[k] & 0xffff0000u), __uint_as_float(wb[k] & 0xffff0000u), op), act, 0.f);
      __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
      wa[k] = *reinterpret_cast<uint32_t *>(&h);
    }
    reinterpret_cast<uint4 *>(y)[i] = make_uint4(wa[0], wa[1], wa[2], wa[3]);
  }
  for (long long i = body * 8 + tid; i < n; i += nth)
    y[i] = __float2bfloat16_rn(act_apply(binop(__bfloat162float(a[i]), __bfloat162float(b[i % nb]), op), act, 0.f));
}

// ---- BatchNormalization (inference), NCHW --------------------------------------------------
// (x - mean[c]) * fused_scale[c] + bias[c], the expression of ROperator_BatchNormalization.hxx:143
__global__ void __launch_bounds__(256) batchnorm_kernel(const float *__restrict__ x, float *__restrict__ y, long long n,
                                                        long long channels, long long inner, const float *__restrict__ fs,
                                                        const float *__restrict__ bias, const float *__restrict__ mean,
                                                        int act, int vec) {
  const long long tid = (long long)blockIdx.x * blockDim.x + threadIdx.x, nth = (long long)gridDim.x * blockDim.x;
  long long body = vec ? n / 4 : 0;  // vec only when inner % 4 == 0: the four lanes share a channel
  for (long long i = tid; i < body; i += nth) {
    const long long c = (i * 4 / inner) % channels;
    const float m = mean[c], s = fs[c], b = bias[c];
    float4 v = reinterpret_cast<const float4 *>(x)[i];
    v.x = act_apply(__fadd_rn(__fmul_rn(__fsub_rn(v.x, m), s), b), act, 0.f);
    v.y = act_apply(__fadd_rn(__fmul_rn(__fsub_rn(v.y, m), s), b), act, 0.f);
    v.z = act_apply(__fadd_rn(__fmul_rn(__fsub_rn(v.z, m), s), b), act, 0.f);
    v.w = act_apply(__fadd_rn(__fmul_rn(__fsub_rn(v.w, m), s), b), act, 0.f);
    reinterpret_cast<float4 *>(y)[i] = v;
  }
  for (long long i = body * 4 + tid; i < n; i += nth) {
    const long long c = (i / inner) % channels;
    y[i] = act_apply(__fadd_rn(__fmul_rn(__fsub_rn(x[i], mean[c]), fs[c]), bias[c]), act, 0.f);
  }
}

// ---- GlobalAveragePool: one warp per (n,c) plane --------------------------------------------
template <typename T> __device__ __forceinline__ float pool_ld(const T *p);
template <> __device__ __forceinline__ float pool_ld<float>(const float *p) { return *p; }
template <> __device__ __forceinline__ float pool_ld<__nv_bfloat16>(const __nv_bfloat16 *p) { return __bfloat162float(*p); }
template <> __device__ __forceinline__ float pool_ld<int8_t>(const int8_t *p) { return (float)*p; }

template <typename T>
__global__ void __launch_bounds__(256) avgpool_kernel(const T *__restrict__ x, float *__restrict__ y, long long nc, long long inner) {
  const int lane = threadIdx.x & 31;
  const long long w0 = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5, nw = ((long long)gridDim.x * blockDim.x) >> 5;
  for (long long r = w0; r < nc; r += nw) {
    const T *xr = x + r * inner;
    float s = 0.f;
    for (long long i = lane; i < inner; i += 32) s += pool_ld<T>(xr + i);
    for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
    if (lane == 0) y[r] = s / (float)inner;
  }
}

// Channels-last planes: one thread per (image, channel); the threads of a warp read consecutive channels of one pixel.
template <typename T>
__global__ void __launch_bounds__(256) avgpool_nhwc_kernel(const T *__restrict__ x, float *__restrict__ y, long long n, long long pixels, long long c) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n * c) return;
  const T *p = x + (i / c) * pixels * c + i % c;
  float s = 0.f;
  for (long long j = 0; j < pixels; ++j) s += pool_ld<T>(p + j * c);
  y[i] = s / (float)pixels;
}

// ---- Quantize / Dequantize -------------------------------------------------------------------
template <typename Q>
__global__ void __launch_bounds__(256) quantize_kernel(const float *__restrict__ x, Q *__restrict__ q, long long n,
                                                       const float *__restrict__ scale, const int *__restrict__ zp,
                                                       long long channels, long long inner, int lo, int hi) {
  const long long tid = (long long)blockIdx.x * blockDim.x + threadIdx.x, nth = (long long)gridDim.x * blockDim.x;
  for (long long i = tid; i < n; i += nth) {
    const long long c = channels == 1 ? 0 : (i / inner) % channels;
    q[i] = (Q)quantize_i(x[i], scale[c], zp ? zp[c] : 0, lo, hi);
  }
}
template <typename Q>
__global__ void __launch_bounds__(256) dequantize_kernel(const Q *__restrict__ q, float *__restrict__ x, long long n,
                                                         const float *__restrict__ scale, const int *__restrict__ zp,
                                                         long long channels, long long inner) {
  const long long tid = (long long)blockIdx.x * blockDim.x + threadIdx.x, nth = (long long)gridDim.x * blockDim.x;
  for (long long i = tid; i < n; i += nth) {
    const long long c = channels == 1 ? 0 : (i / inner) % channels;
    x[i] = __fmul_rn((float)((int)q[i] - (zp ? zp[c] : 0)), scale[c]);
  }
}

// ---- convert ----------------------------------------------------------------------------------
template <typename T> __device__ __forceinline__ float cv_ld(const T *p);
template <> __device__ __forceinline__ float cv_ld<float>(const float *p) { return *p; }
template <> __device__ __forceinline__ float cv_ld<__nv_bfloat16>(const __nv_bfloat16 *p) { return __bfloat162float(*p); }
template <> __device__ __forceinline__ float cv_ld<__nv_fp8_e4m3>(const __nv_fp8_e4m3 *p) { return (float)*p; }
template <> __device__ __forceinline__ float cv_ld<int8_t>(const int8_t *p) { return (float)*p; }
template <typename T> __device__ __forceinline__ void cv_st(T *p, float v);
template <> __device__ __forceinline__ void cv_st<float>(float *p, float v) { *p = v; }
template <> __device__ __forceinline__ void cv_st<__nv_bfloat16>(__nv_bfloat16 *p, float v) { *p = __float2bfloat16_rn(v); }
template <> __device__ __forceinline__ void cv_st<__nv_fp8_e4m3>(__nv_fp8_e4m3 *p, float v) { *p = __nv_fp8_e4m3(v); }

template <typename TI, typename TO>
__global__ void __launch_bounds__(256) convert_kernel(const TI *__restrict__ x, TO *__restrict__ y, long long rows, long long cols,
                                                      const float *__restrict__ row_scale) {
  const long long n = rows * cols;
  const long long tid = (long long)blockIdx.x * blockDim.x + threadIdx.x, nth = (long long)gridDim.x * blockDim.x;
  for (long long i = tid; i < n; i += nth) {
    float v = cv_ld<TI>(x + i);
    if (row_scale) v = __fdiv_rn(v, row_scale[i / cols]);
    cv_st<TO>(y + i, v);
  }
}

template <typename TI>
static int convert_to(sofie_b200_ctx *ctx, const void *x, void *y, int yd, long long rows, long long cols, const float *rs) {
  const unsigned g = grid_for(ctx, rows * cols, 256);
  cudaStream_t st = ctx->stream;
  switch (yd) {
    case SOFIE_B200_F32: convert_kernel<TI, float><<<g, 256, 0, st>>>((const TI *)x, (float *)y, rows, cols, rs); break;
    case SOFIE_B200_BF16: convert_kernel<TI, __nv_bfloat16><<<g, 256, 0, st>>>((const TI *)x, (__nv_bfloat16 *)y, rows, cols, rs); break;
    case SOFIE_B200_F8E4M3: convert_kernel<TI, __nv_fp8_e4m3><<<g, 256, 0, st>>>((const TI *)x, (__nv_fp8_e4m3 *)y, rows, cols, rs); break;
    default: return fail(SOFIE_B200_ERR_INVALID, "convert_enqueue: output type %d not supported", yd);
  }
  return 0;
}

// ---- Transpose (rank <= 4 permutation) --------------------------------------------------------------
// y[o0,o1,o2,o3] = x[...] with output dimension d taken from input dimension perm[d].  Elements are
// moved as opaque words of `es` bytes; when the innermost dimension stays innermost the copy runs on
// 16-byte vectors (contiguous runs on both sides), otherwise element by element with coalesced writes.
struct PermuteParams {
  long long out_dim[4];
  long long in_stride[4];  // stride (in units) of the input dimension feeding each output dimension
  long long total;         // units to move
};

template <typename U>
__global__ void __launch_bounds__(256) permute_kernel(const U *__restrict__ x, U *__restrict__ y, PermuteParams p) {
  const long long tid = (long long)blockIdx.x * blockDim.x + threadIdx.x, nth = (long long)gridDim.x * blockDim.x;
  for (long long i = tid; i < p.total; i += nth) {
    long long r = i;
    const long long i3 = r % p.out_dim[3]; r /= p.out_dim[3];
    const long long i2 = r % p.out_dim[2]; r /= p.out_dim[2];
    const long long i1 = r % p.out_dim[1]; r /= p.out_dim[1];
    y[i] = x[r * p.in_stride[0] + i1 * p.in_stride[1] + i2 * p.in_stride[2] + i3 * p.in_stride[3]];
  }
}

// The depth taps of a 3-D convolution as channels: y[(n, od), (c, t), hw] = x[n, c, od * stride - pad + t * dil, hw], zero
// outside the depth range.  With the taps there, a 3-D convolution over [N,C,D,H,W] is a 2-D one over N * Do slices of C * T
// channels, and its weights [K, C, T, R, S] are the 2-D ones [K, C * T, R, S] as they lie in memory.
template <typename W>
__global__ void __launch_bounds__(256) depth_unfold_kernel(const W *__restrict__ x, W *__restrict__ y, long long total, long long c, long long d, long long hw,
                                                           long long taps, long long d_out, long long stride_d, long long pad_front, long long dil_d) {
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const long long p = i % hw, ct = (i / hw) % (c * taps), nd = i / (hw * c * taps);
    const long long t = ct % taps, ch = ct / taps, od = nd % d_out, n = nd / d_out;
    const long long z = od * stride_d - pad_front + t * dil_d;
    y[i] = (z >= 0 && z < d) ? x[((n * c + ch) * d + z) * hw + p] : (W)0;
  }
}

}  // namespace sb200

using namespace sb200;

#define SB_PRELUDE(name)                                                              \
  if (!ctx) return fail(SOFIE_B200_ERR_INVALID, name ": ctx is NULL");                \
  SB_CUDA(cudaSetDevice(ctx->device));
#define SB_LAUNCHED()               \
  SB_CUDA(cudaGetLastError());      \
  ctx->launches++;                  \
  return 0;

extern "C" {

int sofie_b200_unary_enqueue(sofie_b200_ctx *ctx, const void *x, void *y, int32_t dtype, int64_t n, int32_t act,
                             float act_alpha) {
  SB_PRELUDE("unary_enqueue");
  if (n < 0) return fail(SOFIE_B200_ERR_INVALID, "unary_enqueue: negative length");
  if (n == 0) return 0;
  if (!x || !y) return fail(SOFIE_B200_ERR_INVALID, "unary_enqueue: NULL tensor");
  const int vec = ((uintptr_t)x % 16 == 0) && ((uintptr_t)y % 16 == 0);
  if (dtype == SOFIE_B200_F32)
    unary_f32_kernel<<<grid_for(ctx, n / 4 + 1, 256), 256, 0, ctx->stream>>>((const float *)x, (float *)y, n, act, act_alpha, vec);
  else if (dtype == SOFIE_B200_BF16)
    unary_bf16_kernel<<<grid_for(ctx, n / 8 + 1, 256), 256, 0, ctx->stream>>>((const __nv_bfloat16 *)x, (__nv_bfloat16 *)y, n, act, act_alpha, vec);
  else
    return fail(SOFIE_B200_ERR_INVALID, "unary_enqueue: type %d not supported", dtype);
  SB_LAUNCHED();
}

int sofie_b200_binary_enqueue(sofie_b200_ctx *ctx, const void *a, const void *b, void *y, int32_t dtype, int64_t n,
                              int64_t nb, int32_t op, int32_t act) {
  SB_PRELUDE("binary_enqueue");
  if (n < 0 || nb < 0) return fail(SOFIE_B200_ERR_INVALID, "binary_enqueue: negative length");
  if (n == 0) return 0;
  if (!a || !b || !y) return fail(SOFIE_B200_ERR_INVALID, "binary_enqueue: NULL tensor");
  if (nb == 0 || n % nb) return fail(SOFIE_B200_ERR_INVALID, "binary_enqueue: %lld is not a multiple of the broadcast length %lld", (long long)n, (long long)nb);
  if (op < 0 || op > 3) return fail(SOFIE_B200_ERR_INVALID, "binary_enqueue: op %d unknown", op);
  const int e = dtype == SOFIE_B200_F32 ? 4 : 8;
  const int vec = ((uintptr_t)a % 16 == 0) && ((uintptr_t)b % 16 == 0) && ((uintptr_t)y % 16 == 0) && (nb % e == 0);
  if (dtype == SOFIE_B200_F32)
    binary_f32_kernel<<<grid_for(ctx, n / 4 + 1, 256), 256, 0, ctx->stream>>>((const float *)a, (const float *)b, (float *)y, n, nb, op, act, vec);
  else if (dtype == SOFIE_B200_BF16)
    binary_bf16_kernel<<<grid_for(ctx, n / 8 + 1, 256), 256, 0, ctx->stream>>>((const __nv_bfloat16 *)a, (const __nv_bfloat16 *)b, (__nv_bfloat16 *)y, n, nb, op, act, vec);
  else
    return fail(SOFIE_B200_ERR_INVALID, "binary_enqueue: type %d not supported", dtype);
  SB_LAUNCHED();
}

int sofie_b200_batchnorm_enqueue(sofie_b200_ctx *ctx, const float *x, float *y, int64_t outer, int64_t channels,
                                 int64_t inner, const float *fused_scale, const float *bias, const float *mean,
                                 int32_t act) {
  SB_PRELUDE("batchnorm_enqueue");
  if (outer < 0 || channels < 0 || inner < 0) return fail(SOFIE_B200_ERR_INVALID, "batchnorm_enqueue: negative extent");
  const long long n = outer * channels * inner;
  if (n == 0) return 0;
  if (!x || !y || !fused_scale || !bias || !mean) return fail(SOFIE_B200_ERR_INVALID, "batchnorm_enqueue: NULL tensor");
  const int vec = ((uintptr_t)x % 16 == 0) && ((uintptr_t)y % 16 == 0) && (inner % 4 == 0);
  batchnorm_kernel<<<grid_for(ctx, n / 4 + 1, 256), 256, 0, ctx->stream>>>(x, y, n, channels, inner, fused_scale, bias, mean, act, vec);
  SB_LAUNCHED();
}

int sofie_b200_global_avgpool_enqueue(sofie_b200_ctx *ctx, const void *x, float *y, int32_t x_dtype, int64_t nc,
                                      int64_t inner) {
  SB_PRELUDE("global_avgpool_enqueue");
  if (nc < 0 || inner < 0) return fail(SOFIE_B200_ERR_INVALID, "global_avgpool_enqueue: negative extent");
  if (nc == 0) return 0;
  if (inner == 0) return fail(SOFIE_B200_ERR_INVALID, "global_avgpool_enqueue: empty plane");
  if (!x || !y) return fail(SOFIE_B200_ERR_INVALID, "global_avgpool_enqueue: NULL tensor");
  const unsigned g = grid_for(ctx, nc * 32, 256);
  if (x_dtype == SOFIE_B200_F32) avgpool_kernel<float><<<g, 256, 0, ctx->stream>>>((const float *)x, y, nc, inner);
  else if (x_dtype == SOFIE_B200_BF16) avgpool_kernel<__nv_bfloat16><<<g, 256, 0, ctx->stream>>>((const __nv_bfloat16 *)x, y, nc, inner);
  else if (x_dtype == SOFIE_B200_I8) avgpool_kernel<int8_t><<<g, 256, 0, ctx->stream>>>((const int8_t *)x, y, nc, inner);
  else return fail(SOFIE_B200_ERR_INVALID, "global_avgpool_enqueue: type %d not supported", x_dtype);
  SB_LAUNCHED();
}

int sofie_b200_global_avgpool_nhwc_enqueue(sofie_b200_ctx *ctx, const void *x, float *y, int32_t x_dtype, int64_t n,
                                           int64_t pixels, int64_t channels) {
  SB_PRELUDE("global_avgpool_nhwc_enqueue");
  if (n < 0 || pixels < 0 || channels < 0) return fail(SOFIE_B200_ERR_INVALID, "global_avgpool_nhwc_enqueue: negative extent");
  if (n * channels == 0) return 0;
  if (pixels == 0) return fail(SOFIE_B200_ERR_INVALID, "global_avgpool_nhwc_enqueue: empty plane");
  if (!x || !y) return fail(SOFIE_B200_ERR_INVALID, "global_avgpool_nhwc_enqueue: NULL tensor");
  const unsigned g = (unsigned)((n * channels + 255) / 256);
  if (x_dtype == SOFIE_B200_F32) avgpool_nhwc_kernel<float><<<g, 256, 0, ctx->stream>>>((const float *)x, y, n, pixels, channels);
  else if (x_dtype == SOFIE_B200_BF16) avgpool_nhwc_kernel<__nv_bfloat16><<<g, 256, 0, ctx->stream>>>((const __nv_bfloat16 *)x, y, n, pixels, channels);
  else if (x_dtype == SOFIE_B200_I8) avgpool_nhwc_kernel<int8_t><<<g, 256, 0, ctx->stream>>>((const int8_t *)x, y, n, pixels, channels);
  else return fail(SOFIE_B200_ERR_INVALID, "global_avgpool_nhwc_enqueue: type %d not supported", x_dtype);
  SB_LAUNCHED();
}

int sofie_b200_quantize_enqueue(sofie_b200_ctx *ctx, const float *x, void *q, int32_t q_dtype, int64_t n,
                                const float *scale, const int32_t *zero_point, int64_t channels, int64_t inner) {
  SB_PRELUDE("quantize_enqueue");
  if (n < 0 || channels < 1 || inner < 1) return fail(SOFIE_B200_ERR_INVALID, "quantize_enqueue: bad extent");
  if (n == 0) return 0;
  if (!x || !q || !scale) return fail(SOFIE_B200_ERR_INVALID, "quantize_enqueue: NULL tensor");
  const unsigned g = grid_for(ctx, n, 256);
  if (q_dtype == SOFIE_B200_I8) quantize_kernel<int8_t><<<g, 256, 0, ctx->stream>>>(x, (int8_t *)q, n, scale, zero_point, channels, inner, -128, 127);
  else if (q_dtype == SOFIE_B200_U8) quantize_kernel<uint8_t><<<g, 256, 0, ctx->stream>>>(x, (uint8_t *)q, n, scale, zero_point, channels, inner, 0, 255);
  else return fail(SOFIE_B200_ERR_INVALID, "quantize_enqueue: type %d not supported", q_dtype);
  SB_LAUNCHED();
}

int sofie_b200_dequantize_enqueue(sofie_b200_ctx *ctx, const void *q, float *x, int32_t q_dtype, int64_t n,
                                  const float *scale, const int32_t *zero_point, int64_t channels, int64_t inner) {
  SB_PRELUDE("dequantize_enqueue");
  if (n < 0 || channels < 1 || inner < 1) return fail(SOFIE_B200_ERR_INVALID, "dequantize_enqueue: bad extent");
  if (n == 0) return 0;
  if (!x || !q || !scale) return fail(SOFIE_B200_ERR_INVALID, "dequantize_enqueue: NULL tensor");
  const unsigned g = grid_for(ctx, n, 256);
  if (q_dtype == SOFIE_B200_I8) dequantize_kernel<int8_t><<<g, 256, 0, ctx->stream>>>((const int8_t *)q, x, n, scale, zero_point, channels, inner);
  else if (q_dtype == SOFIE_B200_U8) dequantize_kernel<uint8_t><<<g, 256, 0, ctx->stream>>>((const uint8_t *)q, x, n, scale, zero_point, channels, inner);
  else if (q_dtype == SOFIE_B200_I32) dequantize_kernel<int><<<g, 256, 0, ctx->stream>>>((const int *)q, x, n, scale, zero_point, channels, inner);
  else return fail(SOFIE_B200_ERR_INVALID, "dequantize_enqueue: type %d not supported", q_dtype);
  SB_LAUNCHED();
}

int sofie_b200_depth_unfold_enqueue(sofie_b200_ctx *ctx, const void *x, void *y, int32_t dtype, int64_t n, int64_t c, int64_t d, int64_t hw,
                                    int64_t taps, int64_t d_out, int64_t stride_d, int64_t pad_front, int64_t dil_d) {
  SB_PRELUDE("depth_unfold_enqueue");
  const int es = dtype_size(dtype);
  if (es != 1 && es != 4) return fail(SOFIE_B200_ERR_INVALID, "depth_unfold_enqueue: 1- and 4-byte element types only (type %d)", dtype);
  if (n < 0 || c < 1 || d < 1 || hw < 1 || taps < 1 || d_out < 1 || stride_d < 1 || dil_d < 1 || pad_front < 0)
    return fail(SOFIE_B200_ERR_INVALID, "depth_unfold_enqueue: bad extent");
  const long long total = n * d_out * c * taps * hw;
  if (total == 0) return 0;
  if (!x || !y) return fail(SOFIE_B200_ERR_INVALID, "depth_unfold_enqueue: NULL tensor");
  const unsigned grid = (unsigned)std::min<long long>((total + 255) / 256, (long long)ctx->sm_count * 32);
  if (es == 4)
    depth_unfold_kernel<uint32_t><<<grid, 256, 0, ctx->stream>>>((const uint32_t *)x, (uint32_t *)y, total, c, d, hw, taps, d_out, stride_d, pad_front, dil_d);
  else
    depth_unfold_kernel<uint8_t><<<grid, 256, 0, ctx->stream>>>((const uint8_t *)x, (uint8_t *)y, total, c, d, hw, taps, d_out, stride_d, pad_front, dil_d);
  SB_LAUNCHED();
}

int sofie_b200_transpose_enqueue(sofie_b200_ctx *ctx, const void *x, void *y, int32_t dtype, int32_t rank,
                                 const int64_t *in_shape, const int32_t *perm) {
  SB_PRELUDE("transpose_enqueue");
  if (rank < 1 || rank > 4 || !in_shape || !perm) return fail(SOFIE_B200_ERR_INVALID, "transpose_enqueue: rank 1..4 with shape and permutation expected");
  const int es = dtype_size(dtype);
  if (!es) return fail(SOFIE_B200_ERR_INVALID, "transpose_enqueue: type %d unknown", dtype);
  // left-pad to rank 4
  long long ishape[4] = {1, 1, 1, 1}, istride[4];
  int pm[4] = {0, 1, 2, 3};
  const int pad = 4 - rank;
  bool seen[4] = {false, false, false, false};
  for (int d = 0; d < rank; ++d) {
    if (in_shape[d] < 0 || perm[d] < 0 || perm[d] >= rank || seen[perm[d]]) return fail(SOFIE_B200_ERR_INVALID, "transpose_enqueue: bad shape or permutation");
    seen[perm[d]] = true;
    ishape[pad + d] = in_shape[d];
    pm[pad + d] = pad + perm[d];
  }
  istride[3] = 1;
  for (int d = 2; d >= 0; --d) istride[d] = istride[d + 1] * ishape[d + 1];
  PermuteParams p;
  long long total = 1;
  for (int d = 0; d < 4; ++d) { p.out_dim[d] = ishape[pm[d]]; p.in_stride[d] = istride[pm[d]]; total *= p.out_dim[d]; }
  if (total == 0) return 0;
  if (!x || !y) return fail(SOFIE_B200_ERR_INVALID, "transpose_enqueue: NULL tensor");
  // innermost dimension unchanged: move 16-byte words when everything is aligned to them
  const long long inner_bytes = p.out_dim[3] * es;
  if (pm[3] == 3 && inner_bytes % 16 == 0 && (uintptr_t)x % 16 == 0 && (uintptr_t)y % 16 == 0) {
    const long long w = 16 / es;
    p.out_dim[3] /= w;
    for (int d = 0; d < 3; ++d) p.in_stride[d] /= w;
    p.total = total / w;
    permute_kernel<uint4><<<grid_for(ctx, p.total, 256), 256, 0, ctx->stream>>>((const uint4 *)x, (uint4 *)y, p);
  } else {
    p.total = total;
    const unsigned g = grid_for(ctx, total, 256);
    if (es == 1) permute_kernel<uint8_t><<<g, 256, 0, ctx->stream>>>((const uint8_t *)x, (uint8_t *)y, p);
    else if (es == 2) permute_kernel<uint16_t><<<g, 256, 0, ctx->stream>>>((const uint16_t *)x, (uint16_t *)y, p);
    else permute_kernel<uint32_t><<<g, 256, 0, ctx->stream>>>((const uint32_t *)x, (uint32_t *)y, p);
  }
  SB_LAUNCHED();
}

int sofie_b200_convert_enqueue(sofie_b200_ctx *ctx, const void *x, void *y, int32_t x_dtype, int32_t y_dtype,
                               int64_t rows, int64_t cols, const float *row_scale) {
  SB_PRELUDE("convert_enqueue");
  if (rows < 0 || cols < 0) return fail(SOFIE_B200_ERR_INVALID, "convert_enqueue: negative extent");
  if (rows * cols == 0) return 0;
  if (!x || !y) return fail(SOFIE_B200_ERR_INVALID, "convert_enqueue: NULL tensor");
  int rc;
  switch (x_dtype) {
    case SOFIE_B200_F32: rc = convert_to<float>(ctx, x, y, y_dtype, rows, cols, row_scale); break;
    case SOFIE_B200_BF16: rc = convert_to<__nv_bfloat16>(ctx, x, y, y_dtype, rows, cols, row_scale); break;
    case SOFIE_B200_F8E4M3: rc = convert_to<__nv_fp8_e4m3>(ctx, x, y, y_dtype, rows, cols, row_scale); break;
    case SOFIE_B200_I8: rc = convert_to<int8_t>(ctx, x, y, y_dtype, rows, cols, row_scale); break;
    default: return fail(SOFIE_B200_ERR_INVALID, "convert_enqueue: input type %d not supported", x_dtype);
  }
  if (rc) return rc;
  SB_LAUNCHED();
}

}  // extern "C"
