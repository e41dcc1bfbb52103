/*
 * TEST INFRASTRUCTURE -- not product code (see sofie_oracle.h).  CPU restatement of the arithmetic
 * of SOFIE's emitted inference code for the hot path.  Compile with -ffp-contract=off.
 */
#include "sofie_oracle.h"

#include <math.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

int so_threads(void) {
#ifdef _OPENMP
  return omp_get_max_threads();
#else
  return 1;
#endif
}

void so_set_threads(int n) {
#ifdef _OPENMP
  if (n > 0) omp_set_num_threads(n);
#else
  (void)n;
#endif
}

/* ---------------------------------------------------------------------------------------------
 * element conversions
 * ------------------------------------------------------------------------------------------- */
static float u2f(uint32_t u) { float f; memcpy(&f, &u, 4); return f; }
static uint32_t f2u(float f) { uint32_t u; memcpy(&u, &f, 4); return u; }

float so_bf16_to_f32(uint16_t v) { return u2f((uint32_t)v << 16); }

uint16_t so_f32_to_bf16(float v) {
  uint32_t u = f2u(v);
  if ((u & 0x7fffffffu) > 0x7f800000u) return (uint16_t)((u >> 16) | 0x40); /* quiet NaN */
  u += 0x7fffu + ((u >> 16) & 1u); /* round to nearest even */
  return (uint16_t)(u >> 16);
}

/* e4m3fn: 1 sign, 4 exponent (bias 7), 3 mantissa; no infinities; 0x7f/0xff are NaN; max 448. */
float so_e4m3_to_f32(uint8_t v) {
  const int s = v >> 7, e = (v >> 3) & 0xf, m = v & 7;
  float r;
  if (e == 0xf && m == 7) return NAN;
  if (e == 0) r = ldexpf((float)m, -9);          /* subnormal: m * 2^-3 * 2^-6 */
  else r = ldexpf(1.f + (float)m / 8.f, e - 7);
  return s ? -r : r;
}

uint8_t so_f32_to_e4m3(float v) {
  if (v != v) return 0x7f;
  const uint8_t s = signbit(v) ? 0x80 : 0;
  float a = fabsf(v);
  if (a >= 464.f) return s | 0x7e; /* saturate (464 is the midpoint above 448; ties go to even = 448) */
  if (a > 448.f) return s | 0x7e;
  /* quantum: 2^-9 below 2^-6, else 2^(floor(log2 a) - 3) */
  int ex;
  frexpf(a, &ex); /* a = f * 2^ex, f in [0.5,1) -> floor(log2 a) = ex-1 */
  int q = ex - 1 - 3;
  if (q < -9) q = -9;
  float scaled = ldexpf(a, -q);        /* exact */
  float r = nearbyintf(scaled);        /* round half to even (default rounding mode) */
  float back = ldexpf(r, q);
  if (back == 0.f) return s;
  if (back > 448.f) return s | 0x7e;
  /* encode */
  frexpf(back, &ex);
  int e = ex - 1 + 7;
  if (e <= 0) { /* subnormal */
    int m = (int)ldexpf(back, 9);
    return s | (uint8_t)m;
  }
  int m = (int)(ldexpf(back, -(ex - 1)) * 8.f) - 8;
  return s | (uint8_t)(e << 3) | (uint8_t)m;
}

static double load_elem(const void *p, int dtype, int64_t i) {
  switch (dtype) {
    case SOFIE_B200_F32: return ((const float *)p)[i];
    case SOFIE_B200_BF16: return so_bf16_to_f32(((const uint16_t *)p)[i]);
    case SOFIE_B200_I8: return ((const int8_t *)p)[i];
    case SOFIE_B200_U8: return ((const uint8_t *)p)[i];
    case SOFIE_B200_I32: return ((const int32_t *)p)[i];
    case SOFIE_B200_F8E4M3: return so_e4m3_to_f32(((const uint8_t *)p)[i]);
  }
  return 0;
}

static float load_f(const void *p, int dtype, int64_t i) { return (float)load_elem(p, dtype, i); }

static void store_f(void *p, int dtype, int64_t i, float v) {
  if (dtype == SOFIE_B200_F32) ((float *)p)[i] = v;
  else if (dtype == SOFIE_B200_BF16) ((uint16_t *)p)[i] = so_f32_to_bf16(v);
  else if (dtype == SOFIE_B200_F8E4M3) ((uint8_t *)p)[i] = so_f32_to_e4m3(v);
}

/* ---------------------------------------------------------------------------------------------
 * activations and the fused epilogue (the documented steps of sofie_b200_epilogue)
 * ------------------------------------------------------------------------------------------- */
static float act_apply(float v, int act, float aa) {
  switch (act) {
    case SOFIE_B200_ACT_RELU: return v > 0.f ? v : 0.f;                      /* SOFIE_common_helpers.cxx:325-332 */
    case SOFIE_B200_ACT_GELU_ERF: return (0.5f * v) * (1.f + erff(v * 0.7071067811865475f)); /* ROperator_Gelu.hxx:67 */
    case SOFIE_B200_ACT_GELU_TANH: { float x3 = v * v * v; return 0.5f * v * (1.f + tanhf(0.7978845608028654f * (v + 0.044715f * x3))); }
    case SOFIE_B200_ACT_LEAKY_RELU: return v >= 0.f ? v : aa * v;
    case SOFIE_B200_ACT_SIGMOID: return 1.f / (1.f + expf(-v));
  }
  return v;
}

/* ONNX QuantizeLinear: round half to even, add zero point, saturate. */
static int quantize_i(float v, float out_scale, int zp, int lo, int hi) {
  float q = out_scale == 1.f ? v : v / out_scale;
  q = nearbyintf(q) + (float)zp;
  if (q < (float)lo) q = (float)lo;
  if (q > (float)hi) q = (float)hi;
  return (int)q;
}

typedef struct {
  const sofie_b200_epilogue *ep;
  int y_dtype, int_acc;
  int64_t ldy, stride_y, stride_c, stride_r, ldc, ldr;
} epi_ctx;

/* acc_i is used when int_acc, acc_f otherwise (acc_f already rounded to fp32). */
static void epi_store(const epi_ctx *c, void *Y, int64_t b, int64_t i, int64_t j, int32_t acc_i, float acc_f) {
  const sofie_b200_epilogue *ep = c->ep;
  const int64_t off = b * c->stride_y + i * c->ldy + j;
  const int bm = ep ? ep->bias_mode : SOFIE_B200_BIAS_NONE;
  if (c->int_acc) {
    if (bm == SOFIE_B200_BIAS_COL_I32) acc_i += ((const int32_t *)ep->bias)[j];
    else if (bm == SOFIE_B200_BIAS_ROW_I32) acc_i += ((const int32_t *)ep->bias)[i];
  }
  if (c->y_dtype == SOFIE_B200_I32) { ((int32_t *)Y)[off] = acc_i; return; }
  float v = c->int_acc ? (float)acc_i : acc_f;
  float out_scale = 1.f; int zp = 0;
  if (ep) {
    if (ep->row_scale) v = v * ep->row_scale[i];
    if (ep->col_scale) v = v * ep->col_scale[j];
    if (ep->alpha != 1.f) v = v * ep->alpha;
    switch (bm) {
      case SOFIE_B200_BIAS_COL_F32: v = v + ((const float *)ep->bias)[j]; break;
      case SOFIE_B200_BIAS_ROW_F32: v = v + ((const float *)ep->bias)[i]; break;
      case SOFIE_B200_BIAS_SCALAR_F32: v = v + ((const float *)ep->bias)[0]; break;
      case SOFIE_B200_BIAS_FULL_F32: { float t = ep->beta * ((const float *)ep->bias)[b * c->stride_c + i * c->ldc + j]; v = v + t; break; }
      default: break;
    }
    if (ep->residual) v = v + load_f(ep->residual, ep->residual_dtype, b * c->stride_r + i * c->ldr + j);
    v = act_apply(v, ep->act, ep->act_alpha);
    out_scale = ep->out_scale == 0.f ? 1.f : ep->out_scale;
    zp = ep->out_zero_point;
  }
  switch (c->y_dtype) {
    case SOFIE_B200_F32: ((float *)Y)[off] = v; break;
    case SOFIE_B200_BF16: ((uint16_t *)Y)[off] = so_f32_to_bf16(v); break;
    case SOFIE_B200_I8: ((int8_t *)Y)[off] = (int8_t)quantize_i(v, out_scale, zp, -128, 127); break;
    case SOFIE_B200_U8: ((uint8_t *)Y)[off] = (uint8_t)quantize_i(v, out_scale, zp, 0, 255); break;
    default: break;
  }
}

/* ---------------------------------------------------------------------------------------------
 * contraction
 * ------------------------------------------------------------------------------------------- */
int so_gemm(const sofie_b200_gemm_desc *din, const void *A, const void *B, void *Y, const sofie_b200_epilogue *ep) {
  sofie_b200_gemm_desc d = *din;
  if (d.batch < 1) d.batch = 1;
  if (d.lda == 0) d.lda = d.trans_a ? d.M : d.K;
  if (d.ldb == 0) d.ldb = d.trans_b ? d.K : d.N;
  if (d.ldy == 0) d.ldy = d.N;
  epi_ctx c = {ep, d.y_dtype, d.ab_dtype == SOFIE_B200_I8, d.ldy, d.stride_y, d.stride_c, d.stride_r,
               ep && ep->ldc ? ep->ldc : d.N, ep && ep->ldr ? ep->ldr : d.N};
  const int64_t M = d.M, N = d.N, K = d.K;
  for (int64_t b = 0; b < d.batch; ++b) {
    if (c.int_acc) {
      const int8_t *a = (const int8_t *)A + b * d.stride_a, *bb = (const int8_t *)B + b * d.stride_b;
      /* B as [N][K] contiguous in k for a vectorisable inner loop */
      int8_t *bt = (int8_t *)malloc((size_t)(N * K > 0 ? N * K : 1));
      for (int64_t n = 0; n < N; ++n)
        for (int64_t k = 0; k < K; ++k) bt[n * K + k] = d.trans_b ? bb[n * d.ldb + k] : bb[k * d.ldb + n];
#pragma omp parallel for schedule(static)
      for (int64_t i = 0; i < M; ++i) {
        int8_t *ar = (int8_t *)malloc((size_t)(K > 0 ? K : 1));
        for (int64_t k = 0; k < K; ++k) ar[k] = d.trans_a ? a[k * d.lda + i] : a[i * d.lda + k];
        for (int64_t j = 0; j < N; ++j) {
          const int8_t *br = bt + j * K;
          int32_t acc = 0;
          for (int64_t k = 0; k < K; ++k) acc += (int32_t)ar[k] * (int32_t)br[k];
          epi_store(&c, Y, b, i, j, acc, 0.f);
        }
        free(ar);
      }
      free(bt);
    } else {
      /* decode once to float, accumulate in double, round once to fp32 */
      float *af = (float *)malloc(sizeof(float) * (size_t)(M * K > 0 ? M * K : 1));
      float *bf = (float *)malloc(sizeof(float) * (size_t)(N * K > 0 ? N * K : 1));
      for (int64_t i = 0; i < M; ++i)
        for (int64_t k = 0; k < K; ++k)
          af[i * K + k] = load_f(A, d.ab_dtype, b * d.stride_a + (d.trans_a ? k * d.lda + i : i * d.lda + k));
      for (int64_t n = 0; n < N; ++n)
        for (int64_t k = 0; k < K; ++k)
          bf[n * K + k] = load_f(B, d.ab_dtype, b * d.stride_b + (d.trans_b ? n * d.ldb + k : k * d.ldb + n));
#pragma omp parallel for schedule(static)
      for (int64_t i = 0; i < M; ++i)
        for (int64_t j = 0; j < N; ++j) {
          const float *ar = af + i * K, *br = bf + j * K;
          double acc = 0.0;
          for (int64_t k = 0; k < K; ++k) acc += (double)ar[k] * (double)br[k];
          epi_store(&c, Y, b, i, j, 0, (float)acc);
        }
      free(af);
      free(bf);
    }
  }
  return 0;
}

/* ---------------------------------------------------------------------------------------------
 * convolution (direct loops; K order (c, r, s) as ROperator_Conv.hxx:456-476)
 * ------------------------------------------------------------------------------------------- */
int so_conv_out_shape(const sofie_b200_conv_desc *d, int64_t *Ho, int64_t *Wo) {
  const int64_t er = (d->R - 1) * d->dil_h + 1, es = (d->S - 1) * d->dil_w + 1;
  const int64_t h = d->H + d->pad_top + d->pad_bottom - er, w = d->W + d->pad_left + d->pad_right - es;
  if (h < 0 || w < 0 || d->stride_h < 1 || d->stride_w < 1) return -1;
  *Ho = h / d->stride_h + 1;
  *Wo = w / d->stride_w + 1;
  return 0;
}

int so_conv(const sofie_b200_conv_desc *din, const void *X, const void *W, void *Y, const sofie_b200_epilogue *ep) {
  sofie_b200_conv_desc d = *din;
  if (d.groups < 1) d.groups = 1;
  int64_t Ho, Wo;
  if (so_conv_out_shape(&d, &Ho, &Wo)) return -1;
  const int64_t cg = d.C / d.groups, kg = d.K / d.groups, pix = Ho * Wo;
  /* epilogue with channel as the "column": element (n, k, p) is row p? -- addressed directly below */
  const int int_acc = d.x_dtype == SOFIE_B200_I8;
  sofie_b200_epilogue e;
  memset(&e, 0, sizeof(e));
  e.alpha = 1.f; e.beta = 1.f; e.out_scale = 1.f;
  if (ep) e = *ep;
  /* Treat one image as a [K, pix] matrix: rows = channels.  Per-channel vectors are per-row here. */
  sofie_b200_epilogue er = e;
  er.row_scale = e.col_scale; er.col_scale = NULL;
  if (e.bias_mode == SOFIE_B200_BIAS_COL_F32) er.bias_mode = SOFIE_B200_BIAS_ROW_F32;
  if (e.bias_mode == SOFIE_B200_BIAS_COL_I32) er.bias_mode = SOFIE_B200_BIAS_ROW_I32;
  epi_ctx c = {&er, d.y_dtype, int_acc, pix, d.K * pix, 0, d.K * pix, pix, pix};
#pragma omp parallel for collapse(2) schedule(static)
  for (int64_t n = 0; n < d.N; ++n)
    for (int64_t k = 0; k < d.K; ++k) {
      const int64_t g = k / kg;
      for (int64_t oh = 0; oh < Ho; ++oh)
        for (int64_t ow = 0; ow < Wo; ++ow) {
          double accf = 0.0;
          int32_t acci = 0;
          for (int64_t cc = 0; cc < cg; ++cc)
            for (int64_t r = 0; r < d.R; ++r)
              for (int64_t s = 0; s < d.S; ++s) {
                const int64_t ih = oh * d.stride_h - d.pad_top + r * d.dil_h, iw = ow * d.stride_w - d.pad_left + s * d.dil_w;
                const int64_t wi = ((k * cg + cc) * d.R + r) * d.S + s;
                const int inb = ih >= 0 && ih < d.H && iw >= 0 && iw < d.W;
                const int64_t xi = ((n * d.C + g * cg + cc) * d.H + ih) * d.W + iw;
                if (int_acc) {
                  const int32_t xv = inb ? ((const int8_t *)X)[xi] : d.x_zero_point;
                  acci += xv * (int32_t)((const int8_t *)W)[wi];
                } else if (inb) {
                  accf += (double)((const float *)X)[xi] * (double)((const float *)W)[wi];
                }
              }
          epi_store(&c, Y, n, k, oh * Wo + ow, acci, (float)accf);
        }
    }
  return 0;
}

/* ---------------------------------------------------------------------------------------------
 * row-wise and elementwise operators
 * ------------------------------------------------------------------------------------------- */
int so_layernorm(const void *x, void *y, int xd, int yd, int64_t rows, int64_t cols, const float *scale, const float *bias,
                 float eps, float *mean_out, float *invstd_out) {
  for (int64_t r = 0; r < rows; ++r) {
    /* ROperator_LayerNormalization.hxx:257-312: sum, mean, sum of squared deviations, 1/sqrt(var+eps) */
    float sum = 0.f;
    for (int64_t c = 0; c < cols; ++c) sum += load_f(x, xd, r * cols + c);
    const float mean = sum / (float)cols;
    float sq = 0.f;
    for (int64_t c = 0; c < cols; ++c) { float t = load_f(x, xd, r * cols + c) - mean; sq += t * t; }
    const float inv = 1.f / sqrtf(sq / (float)cols + eps);
    for (int64_t c = 0; c < cols; ++c) {
      /* scale * invStdDev * (x - mean) + bias, evaluated left to right as the emitted expression */
      const float d = load_f(x, xd, r * cols + c) - mean;
      float t = scale ? (scale[c] * inv) * d : inv * d;
      if (bias) t = t + bias[c];
      store_f(y, yd, r * cols + c, t);
    }
    if (mean_out) mean_out[r] = mean;
    if (invstd_out) invstd_out[r] = inv;
  }
  return 0;
}

int so_sdpa(const float *q, const float *k, const float *v, const float *mask, float *y, int64_t B, int64_t H, int64_t S, int64_t D,
            int64_t Dv, float scale, int folded) {
  if (scale == 0.f) scale = 1.f / sqrtf((float)D);
  /* strides of the two layouts, ROperator_SDPA.hxx:118-135 */
  const int64_t qk_b = folded ? S * H * D : H * S * D, qk_h = folded ? D : S * D, qk_s = folded ? H * D : D;
  const int64_t vy_b = folded ? S * H * Dv : H * S * Dv, vy_h = folded ? Dv : S * Dv, vy_s = folded ? H * Dv : Dv;
  float *scores = (float *)malloc(sizeof(float) * (size_t)(S > 0 ? S : 1));
  if (!scores) return -1;
  for (int64_t b = 0; b < B; ++b)
    for (int64_t h = 0; h < H; ++h)
      for (int64_t s = 0; s < S; ++s) {
        const int64_t qb = b * qk_b + h * qk_h + s * qk_s;
        for (int64_t j = 0; j < S; ++j) {
          const int64_t kb = b * qk_b + h * qk_h + j * qk_s;
          float dot = 0;
          for (int64_t d = 0; d < D; ++d) dot += q[qb + d] * k[kb + d];
          scores[j] = dot * scale;
          if (mask) scores[j] += mask[((b * H + h) * S + s) * S + j];
        }
        float mx = scores[0];
        for (int64_t j = 1; j < S; ++j) if (scores[j] > mx) mx = scores[j];
        float sum = 0;
        for (int64_t j = 0; j < S; ++j) { scores[j] = expf(scores[j] - mx); sum += scores[j]; }
        for (int64_t j = 0; j < S; ++j) scores[j] /= sum;
        for (int64_t d = 0; d < Dv; ++d) {
          float acc = 0;
          for (int64_t j = 0; j < S; ++j) acc += scores[j] * v[b * vy_b + h * vy_h + j * vy_s + d];
          y[b * vy_b + h * vy_h + s * vy_s + d] = acc;
        }
      }
  free(scores);
  return 0;
}

int so_softmax_axis(const float *x, float *y, int64_t outer, int64_t n, int64_t inner, int log_softmax) {
  for (int64_t o = 0; o < outer; ++o)
    for (int64_t i = 0; i < inner; ++i) {
      const float *xs = x + o * n * inner + i;
      float *ys = y + o * n * inner + i;
      float m = xs[0];
      for (int64_t a = 1; a < n; ++a) if (xs[a * inner] > m) m = xs[a * inner];
      float sum = 0.f;
      for (int64_t a = 0; a < n; ++a) { ys[a * inner] = expf(xs[a * inner] - m); sum += ys[a * inner]; }
      for (int64_t a = 0; a < n; ++a) ys[a * inner] = log_softmax ? (xs[a * inner] - m) - logf(sum) : ys[a * inner] / sum;
    }
  return 0;
}

int so_softmax(const void *x, void *y, int xd, int yd, int64_t rows, int64_t cols, int log_softmax) {
  for (int64_t r = 0; r < rows; ++r) {
    float m = -INFINITY;
    for (int64_t c = 0; c < cols; ++c) { float v = load_f(x, xd, r * cols + c); if (v > m) m = v; }
    float s = 0.f;
    for (int64_t c = 0; c < cols; ++c) s += expf(load_f(x, xd, r * cols + c) - m);
    const float inv = 1.f / s, ls = logf(s);
    for (int64_t c = 0; c < cols; ++c) {
      float t = load_f(x, xd, r * cols + c) - m;
      store_f(y, yd, r * cols + c, log_softmax ? t - ls : expf(t) * inv);
    }
  }
  return 0;
}

int so_unary(const void *x, void *y, int dtype, int64_t n, int act, float aa) {
  for (int64_t i = 0; i < n; ++i) store_f(y, dtype, i, act_apply(load_f(x, dtype, i), act, aa));
  return 0;
}

int so_binary(const void *a, const void *b, void *y, int dtype, int64_t n, int64_t nb, int op, int act) {
  if (nb <= 0 || n % nb) return -1;
  for (int64_t i = 0; i < n; ++i) {
    const float u = load_f(a, dtype, i), v = load_f(b, dtype, i % nb);
    float r = op == 0 ? u + v : op == 1 ? u - v : op == 2 ? u * v : u / v;
    store_f(y, dtype, i, act_apply(r, act, 0.f));
  }
  return 0;
}

void so_batchnorm_fold(const float *scale, const float *var, float eps, int64_t channels, float *fused) {
  for (int64_t c = 0; c < channels; ++c) fused[c] = scale[c] / sqrtf(var[c] + eps);
}

int so_batchnorm(const float *x, float *y, int64_t outer, int64_t channels, int64_t inner, const float *fs,
                 const float *bias, const float *mean, int act) {
  const int64_t n = outer * channels * inner;
  for (int64_t i = 0; i < n; ++i) {
    const int64_t c = (i / inner) % channels;
    float t = x[i] - mean[c];
    t = t * fs[c];
    t = t + bias[c];
    y[i] = act_apply(t, act, 0.f);
  }
  return 0;
}

int so_global_avgpool(const void *x, float *y, int xd, int64_t nc, int64_t inner) {
  for (int64_t r = 0; r < nc; ++r) {
    float s = 0.f;
    for (int64_t i = 0; i < inner; ++i) s += load_f(x, xd, r * inner + i);
    y[r] = s / (float)inner;
  }
  return 0;
}

int so_quantize(const float *x, void *q, int qd, int64_t n, const float *scale, const int32_t *zp, int64_t channels,
                int64_t inner) {
  for (int64_t i = 0; i < n; ++i) {
    const int64_t c = channels == 1 ? 0 : (i / inner) % channels;
    const int z = zp ? zp[c] : 0;
    if (qd == SOFIE_B200_I8) ((int8_t *)q)[i] = (int8_t)quantize_i(x[i], scale[c], z, -128, 127);
    else if (qd == SOFIE_B200_U8) ((uint8_t *)q)[i] = (uint8_t)quantize_i(x[i], scale[c], z, 0, 255);
    else return -1;
  }
  return 0;
}

int so_dequantize(const void *q, float *x, int qd, int64_t n, const float *scale, const int32_t *zp, int64_t channels,
                  int64_t inner) {
  for (int64_t i = 0; i < n; ++i) {
    const int64_t c = channels == 1 ? 0 : (i / inner) % channels;
    const int z = zp ? zp[c] : 0;
    x[i] = (float)((int)load_elem(q, qd, i) - z) * scale[c];
  }
  return 0;
}

int so_convert(const void *x, void *y, int xd, int yd, int64_t rows, int64_t cols, const float *row_scale) {
  for (int64_t i = 0; i < rows * cols; ++i) {
    float v = load_f(x, xd, i);
    if (row_scale) v = v / row_scale[i / cols];
    store_f(y, yd, i, v);
  }
  return 0;
}

/* ---------------------------------------------------------------------------------------------
 * arena: best fit with coalescing (MemoryPlanner.inc:47-132), arrays and linear scans
 * ------------------------------------------------------------------------------------------- */
typedef struct { int64_t off, size; } blk;

int so_plan_arena(const sofie_b200_tensor_life *lives, int64_t n, int64_t *offsets, int64_t *total_out) {
  int64_t tmin = 0, tmax = 0, total = 0, nfree = 0;
  blk *fl = (blk *)malloc(sizeof(blk) * (size_t)(n + 1));
  for (int64_t i = 0; i < n; ++i) {
    if (!(lives[i].end > lives[i].begin)) { free(fl); return -1; }
    if (i == 0 || lives[i].begin < tmin) tmin = lives[i].begin;
    if (i == 0 || lives[i].end > tmax) tmax = lives[i].end;
  }
  for (int64_t t = tmin; t <= tmax; ++t) {
    for (int64_t i = 0; i < n; ++i) { /* releases first */
      if (lives[i].end != t) continue;
      int64_t sz = (lives[i].size + 255) / 256 * 256;
      if (sz == 0) continue;
      int64_t pos = 0;
      while (pos < nfree && fl[pos].off < offsets[i]) ++pos;
      memmove(fl + pos + 1, fl + pos, sizeof(blk) * (size_t)(nfree - pos));
      fl[pos].off = offsets[i]; fl[pos].size = sz; ++nfree;
      if (pos + 1 < nfree && fl[pos].off + fl[pos].size == fl[pos + 1].off) {
        fl[pos].size += fl[pos + 1].size;
        memmove(fl + pos + 1, fl + pos + 2, sizeof(blk) * (size_t)(nfree - pos - 2)); --nfree;
      }
      if (pos > 0 && fl[pos - 1].off + fl[pos - 1].size == fl[pos].off) {
        fl[pos - 1].size += fl[pos].size;
        memmove(fl + pos, fl + pos + 1, sizeof(blk) * (size_t)(nfree - pos - 1)); --nfree;
      }
    }
    for (int64_t i = 0; i < n; ++i) { /* then allocations, in index order */
      if (lives[i].begin != t) continue;
      int64_t sz = (lives[i].size + 255) / 256 * 256;
      if (sz == 0) { offsets[i] = total; continue; }
      int64_t best = -1;
      for (int64_t f = 0; f < nfree; ++f)
        if (fl[f].size >= sz && (best < 0 || fl[f].size < fl[best].size)) best = f;
      if (best >= 0) {
        offsets[i] = fl[best].off;
        if (fl[best].size == sz) { memmove(fl + best, fl + best + 1, sizeof(blk) * (size_t)(nfree - best - 1)); --nfree; }
        else { fl[best].off += sz; fl[best].size -= sz; }
      } else {
        offsets[i] = total;
        total += sz;
      }
    }
  }
  free(fl);
  *total_out = total;
  return 0;
}
