// Convolution over a whole NCHW batch.
//
// Y[n, k, :, :] (a [Cout, Ho*Wo] matrix per image, which is exactly the NCHW output) is computed
// as  W[Cout, C*R*S] x xcol[n][Ho*Wo, C*R*S]^T : the weights are the K-major A operand as they
// are stored (only padded once, at plan creation, to a 16-byte row pitch), the unfolded input is
// the K-major B operand, the batch index is the image, and output channels are accumulator ROWS.
// One unfold kernel and one batched contraction per group replace the reference's host loop of
// per-image Im2ColKernel + blas.matmul launches (ROperator_Conv.hxx:1002-1103).  The K order
// (c, r, s) is the reference's (ROperator_Conv.hxx:456-476), so weights need no permutation.
#include <mutex>

#include "gemm.cuh"

struct sofie_b200_conv_plan {
  sofie_b200_ctx *ctx = nullptr;
  sofie_b200_conv_desc d{};
  int64_t Ho = 0, Wo = 0;
  int64_t cg = 0, kg = 0;      // input channels / output channels per group
  int64_t kdim = 0, kpad = 0;  // C/g*R*S and its padded pitch
  void *w_padded = nullptr;    // [K, kpad] device copy of the weights ([K, 2*kpad] hi|lo in split mode)
  int split = 0;               // fp32 at fp32 accuracy on the tensor cores: operands stored as hi | lo segments (gemm_split.cu)
  int direct = 0;              // 3-channel 3x3 first layer: direct kernel on the CUDA cores, no unfold, no contraction plan
  sofie_b200_gemm_desc edesc{}; // direct mode: the contraction this convolution stands for (shapes and pitches of its epilogue)
  int pix_rows = 0;            // y_layout = channels-last: output pixels are the accumulator rows, the unfolded input is the A operand
  int nhwc = 0;                // channels-last unfold: the input is first transposed to [N, H, W, C] in the workspace and K runs
                               // (r, s, c), so every 16-byte chunk of the unfolded matrix is one aligned vector copy
  int pair_out = 0;            // y_layout = 2: Y is channels-last TF32 pairs, [N, Ho, Wo, 2K]
  int stem = 0;                // 3-channel 3x3 int8 first layer with a channels-last output: unfold_c3k3_kernel + tensor-core contraction
  int stem_pack = 1;           // output pixels per row of that contraction (1, 2 or 4; see stem_weights_kernel)
  void *stem_vec = nullptr;    // stem_pack > 1: the per-channel epilogue vectors repeated per packed pixel, [2][stem_pack * K] words
  int implicit = 0;            // channels-last in and out on the tensor cores with no unfolded copy: the contraction's TMA producer reads
                               // the input tensor itself in im2col mode (gemm_umma.cu); no workspace
  sofie_b200_gemm_plan *gemm = nullptr;
  // unit-stride convolution over pixel pairs: the odd output columns are a contraction of their own (gemm: the even ones)
  sofie_b200_gemm_plan *gemm_odd = nullptr;
  void *w_odd = nullptr;
};

namespace sb200 {

static int conv_out_shape(const sofie_b200_conv_desc &d, int64_t *Ho, int64_t *Wo) {
  if (d.stride_h < 1 || d.stride_w < 1 || d.dil_h < 1 || d.dil_w < 1) return fail(SOFIE_B200_ERR_INVALID, "conv: strides and dilations must be >= 1");
  const int64_t eff_r = (d.R - 1) * d.dil_h + 1, eff_s = (d.S - 1) * d.dil_w + 1;  // dilated kernel extent
  const int64_t h = d.H + d.pad_top + d.pad_bottom - eff_r, w = d.W + d.pad_left + d.pad_right - eff_s;
  if (h < 0 || w < 0) return fail(SOFIE_B200_ERR_INVALID, "conv: kernel larger than the padded input");
  *Ho = h / d.stride_h + 1;
  *Wo = w / d.stride_w + 1;
  return 0;
}

// Position of one 16-byte chunk of the unfolded matrix: which image / group / output pixel it belongs to and the
// (channel, kernel row, kernel column) of its first element.  One 64-bit division per chunk, the rest in 32 bits;
// the elements of the chunk then step (c, r, s) incrementally instead of dividing k for every element, which is
// what made the first version of these kernels division-bound (233 GB/s on the int8 layers).
struct UnfoldPos {
  long long row;        // (g, n, pix) flattened: row of the B operand
  unsigned ch;          // chunk inside the row
  const void *xg;       // first input channel of the group in image n
  int ih0, iw0;         // input coordinates of kernel element (0, 0)
  unsigned c, r, s;     // decomposition of k = ch * VEC
};
template <typename T, int VEC>
__device__ __forceinline__ UnfoldPos unfold_pos(const T *x, const sofie_b200_conv_desc &d, long long i, unsigned chunks, unsigned pix, unsigned Wo,
                                                unsigned cg) {
  UnfoldPos u;
  u.row = i / chunks;
  u.ch = (unsigned)(i - u.row * chunks);
  const long long gn = u.row / pix;
  const unsigned p = (unsigned)(u.row - gn * pix);
  const unsigned n = (unsigned)(gn % d.N), g = (unsigned)(gn / d.N);
  const unsigned oh = p / Wo, ow = p - oh * Wo;
  u.ih0 = (int)(oh * d.stride_h) - d.pad_top;
  u.iw0 = (int)(ow * d.stride_w) - d.pad_left;
  u.xg = x + ((long long)n * d.C + (long long)g * cg) * d.H * d.W;
  const unsigned S = (unsigned)d.S, rs = (unsigned)(d.R * d.S), k = u.ch * VEC;
  u.c = k / rs;
  const unsigned q = k - u.c * rs;
  u.r = q / S;
  u.s = q - u.r * S;
  return u;
}

// xcol[g][n][pix][kpad]; one thread writes 16 bytes (VEC elements along k).
template <typename T, int VEC>
__global__ void __launch_bounds__(256) unfold_kernel(const T *__restrict__ x, T *__restrict__ xcol, sofie_b200_conv_desc d,
                                                     long long Ho, long long Wo, long long cg, long long kdim, long long kpad,
                                                     T pad_value) {
  const unsigned chunks = (unsigned)(kpad / VEC), pix = (unsigned)(Ho * Wo);
  const long long total = (long long)d.groups * d.N * pix * chunks;
  const int H = (int)d.H, W = (int)d.W, R = (int)d.R, S = (int)d.S;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const UnfoldPos u = unfold_pos<T, VEC>(x, d, i, chunks, pix, (unsigned)Wo, (unsigned)cg);
    const T *xg = (const T *)u.xg;
    int c = (int)u.c, r = (int)u.r, s = (int)u.s;
    __align__(16) T v[VEC];
#pragma unroll
    for (int e = 0; e < VEC; ++e) {
      T val = (T)0;
      if ((long long)u.ch * VEC + e < kdim) {
        const int ih = u.ih0 + r * d.dil_h, iw = u.iw0 + s * d.dil_w;
        val = (ih >= 0 && ih < H && iw >= 0 && iw < W) ? xg[((long long)c * H + ih) * W + iw] : pad_value;
      }
      v[e] = val;
      if (++s == S) { s = 0; if (++r == R) { r = 0; ++c; } }
    }
    *reinterpret_cast<uint4 *>(xcol + i * VEC) = *reinterpret_cast<const uint4 *>(v);
  }
}

// fp32 input unfolded straight into the split form of the operand: xcol[g][n][pix][hi | lo], each segment kpad wide.
__global__ void __launch_bounds__(256) unfold_split_kernel(const float *__restrict__ x, float *__restrict__ xcol, sofie_b200_conv_desc d,
                                                           long long Ho, long long Wo, long long cg, long long kdim, long long kpad) {
  const unsigned chunks = (unsigned)(kpad / 4), pix = (unsigned)(Ho * Wo);
  const long long total = (long long)d.groups * d.N * pix * chunks;
  const int H = (int)d.H, W = (int)d.W, R = (int)d.R, S = (int)d.S;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const UnfoldPos u = unfold_pos<float, 4>(x, d, i, chunks, pix, (unsigned)Wo, (unsigned)cg);
    const float *xg = (const float *)u.xg;
    int c = (int)u.c, r = (int)u.r, s = (int)u.s;
    __align__(16) float hi[4], lo[4];
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      float val = 0.f;
      if ((long long)u.ch * 4 + e < kdim) {
        const int ih = u.ih0 + r * d.dil_h, iw = u.iw0 + s * d.dil_w;
        if (ih >= 0 && ih < H && iw >= 0 && iw < W) val = xg[((long long)c * H + ih) * W + iw];
      }
      hi[e] = tf32_rn(val);
      lo[e] = tf32_rn(__fsub_rn(val, hi[e]));
      if (++s == S) { s = 0; if (++r == R) { r = 0; ++c; } }
    }
    float *o = xcol + u.row * 2 * kpad + u.ch * 4;
    *reinterpret_cast<uint4 *>(o) = *reinterpret_cast<const uint4 *>(hi);
    *reinterpret_cast<uint4 *>(o + kpad) = *reinterpret_cast<const uint4 *>(lo);
  }
}

// ---- channels-last unfold ---------------------------------------------------------------------------------------
// With K ordered (c, r, s) a 16-byte chunk of the unfolded matrix gathers single elements from up to 16 places of an
// NCHW tensor; the int8 layers of the conv-net configuration spent 85 % of their time there.  Ordered (r, s, c) over a
// channels-last copy of the input, the same chunk is 16 consecutive bytes of one input pixel.  The copy costs one pass
// over the input, a ninth of what the unfold writes for a 3x3 kernel.

// [N, C, HW] -> [N, HW, C] through a 32 x 32 shared-memory tile (any element type).
template <typename T>
__global__ void __launch_bounds__(256) nchw_to_nhwc_kernel(const T *__restrict__ x, T *__restrict__ y, int C, int HW) {
  __shared__ T tile[32][33];
  const long long n = blockIdx.z;
  const int c0 = blockIdx.y * 32, p0 = blockIdx.x * 32;
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const int c = c0 + ty + 8 * j, p = p0 + tx;
    if (c < C && p < HW) tile[ty + 8 * j][tx] = x[(n * C + c) * HW + p];
  }
  __syncthreads();
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const int p = p0 + ty + 8 * j, c = c0 + tx;
    if (c < C && p < HW) y[(n * HW + p) * C + c] = tile[tx][ty + 8 * j];
  }
}

// The same for 1-byte elements with 4-byte accesses on both sides: a 64-channel x 128-pixel tile, read as words of 4
// pixels, written as words of 4 channels.  Needs C % 4 == 0 and HW % 4 == 0.
__global__ void __launch_bounds__(256) nchw_to_nhwc_bytes_kernel(const uint8_t *__restrict__ x, uint8_t *__restrict__ y, int C, int HW) {
  __shared__ uint8_t tile[64][132];
  const long long n = blockIdx.z;
  const int c0 = blockIdx.y * 64, p0 = blockIdx.x * 128;
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    const int c = c0 + ty + 8 * j, p = p0 + 4 * tx;
    if (c < C && p < HW) *reinterpret_cast<uint32_t *>(&tile[ty + 8 * j][4 * tx]) = *reinterpret_cast<const uint32_t *>(x + (n * C + c) * HW + p);
  }
  __syncthreads();
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    const int idx = threadIdx.x + 256 * j;   // (pixel, word of 4 channels)
    const int pl = idx >> 4, cw = idx & 15;
    const int p = p0 + pl, c = c0 + 4 * cw;
    if (p < HW && c < C) {
      const uint32_t w = (uint32_t)tile[4 * cw][pl] | ((uint32_t)tile[4 * cw + 1][pl] << 8) | ((uint32_t)tile[4 * cw + 2][pl] << 16) |
                         ((uint32_t)tile[4 * cw + 3][pl] << 24);
      *reinterpret_cast<uint32_t *>(y + (n * HW + p) * C + c) = w;
    }
  }
}

// Weights [K, cg, R, S] -> [K, R, S, cg] (the K order of the channels-last unfold).
template <typename T>
__global__ void __launch_bounds__(256) reorder_weights_kernel(const T *__restrict__ w, T *__restrict__ out, long long filters, int cg, int rs) {
  const long long total = filters * cg * rs;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const long long f = i / ((long long)cg * rs);
    const int k = (int)(i - f * cg * rs);
    const int q = k / cg, c = k - q * cg;   // out index: k = q * cg + c
    out[i] = w[(f * cg + c) * rs + q];
  }
}

// xcol[g][n][pix][(r, s, c)] from the channels-last input; one thread copies 16 bytes.  SPLIT writes hi | lo, each kpad wide
// (kpad = kdim rounded up to a K block of the TF32 kernel, zero filled); otherwise kpad == kdim.
template <typename T, int VEC, bool SPLIT>
__global__ void __launch_bounds__(256) unfold_nhwc_kernel(const T *__restrict__ x, T *__restrict__ xcol, sofie_b200_conv_desc d, long long Ho,
                                                          long long Wo, long long cg, long long kdim, long long kpad, T pad_value) {
  const unsigned chunks = (unsigned)(kpad / VEC), pix = (unsigned)(Ho * Wo), ccg = (unsigned)cg;
  const long long total = (long long)d.groups * d.N * pix * chunks;
  const int H = (int)d.H, W = (int)d.W, S = (int)d.S;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const long long row = i / chunks;
    const unsigned ch = (unsigned)(i - row * chunks);
    const long long gn = row / pix;
    const unsigned p = (unsigned)(row - gn * pix);
    const unsigned n = (unsigned)(gn % d.N), g = (unsigned)(gn / d.N);
    const unsigned oh = p / (unsigned)Wo, ow = p - oh * (unsigned)Wo;
    const unsigned k = ch * VEC, q = k / ccg, c = k - q * ccg;
    const int r = (int)(q / S), s = (int)(q - (q / S) * S);
    const int ih = (int)(oh * d.stride_h) - d.pad_top + r * d.dil_h, iw = (int)(ow * d.stride_w) - d.pad_left + s * d.dil_w;
    __align__(16) T v[VEC];
    if (k >= (unsigned)kdim) {
#pragma unroll
      for (int e = 0; e < VEC; ++e) v[e] = (T)0;
    } else if (ih >= 0 && ih < H && iw >= 0 && iw < W) {
      *reinterpret_cast<uint4 *>(v) = *reinterpret_cast<const uint4 *>(x + (((long long)n * H + ih) * W + iw) * d.C + g * ccg + c);
    } else {
#pragma unroll
      for (int e = 0; e < VEC; ++e) v[e] = pad_value;
    }
    if constexpr (!SPLIT) {
      *reinterpret_cast<uint4 *>(xcol + i * VEC) = *reinterpret_cast<const uint4 *>(v);
    } else {
      __align__(16) float hi[4], lo[4];
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        hi[e] = tf32_rn((float)v[e]);
        lo[e] = tf32_rn(__fsub_rn((float)v[e], hi[e]));
      }
      float *o = (float *)xcol + row * 2 * kpad + ch * 4;
      *reinterpret_cast<uint4 *>(o) = *reinterpret_cast<const uint4 *>(hi);
      *reinterpret_cast<uint4 *>(o + kpad) = *reinterpret_cast<const uint4 *>(lo);
    }
  }
}

// ---- 3-channel 3x3 first layer on the tensor cores ------------------------------------------------------------------
// K = 27 is less than one MMA K step, so as a contraction this layer is all epilogue; the tensor-core kernel's epilogue
// still writes 8-bit outputs several times faster than CUDA-core dot products do.  The unfolded matrix is [pixels][32]
// bytes (K order (c, r, s) as the weights are stored, five bytes of padding): one thread gathers the 27 inputs of its
// output pixel -- neighbouring lanes read neighbouring bytes of the same input rows -- and writes its row as two 16-byte
// stores, so a warp writes 1 KB of consecutive memory.
__global__ void __launch_bounds__(256) unfold_c3k3_kernel(const int8_t *__restrict__ x, uint4 *__restrict__ xcol, sofie_b200_conv_desc d, int Ho, int Wo) {
  const long long pix = (long long)Ho * Wo, total = d.N * pix;
  const long long gp = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (gp >= total) return;
  const long long n = gp / pix;
  const int p = (int)(gp - n * pix), oh = p / Wo, ow = p - oh * Wo;
  const int ih0 = oh * d.stride_h - d.pad_top, iw0 = ow * d.stride_w - d.pad_left;
  const int H = (int)d.H, Wd = (int)d.W;
  const int8_t *xn = x + n * 3 * H * Wd;
  uint32_t w[8] = {0u, 0u, 0u, 0u, 0u, 0u, 0u, 0u};
#pragma unroll
  for (int c = 0; c < 3; ++c)
#pragma unroll
    for (int r = 0; r < 3; ++r)
#pragma unroll
      for (int s2 = 0; s2 < 3; ++s2) {
        const int k = (c * 3 + r) * 3 + s2;
        const int ih = ih0 + r * d.dil_h, iw = iw0 + s2 * d.dil_w;
        const int8_t v = (ih >= 0 && ih < H && iw >= 0 && iw < Wd) ? xn[((long long)c * H + ih) * Wd + iw] : (int8_t)d.x_zero_point;
        w[k >> 2] |= (uint32_t)(uint8_t)v << (8 * (k & 3));
      }
  xcol[2 * gp] = make_uint4(w[0], w[1], w[2], w[3]);
  xcol[2 * gp + 1] = make_uint4(w[4], w[5], w[6], w[7]);
}

// As a contraction with one output pixel per row the first layer is [pixels, 32] x [32, K]: 128 x K tiles with a fraction of
// one K block each, and the kernel's cost per TILE (one TMA load whose 128-byte box is a quarter data, the accumulator hand-over,
// an epilogue warp's fixed work) sets the pace, not its arithmetic.  P consecutive pixels' rows are P * 32 contiguous bytes, and
// their P * K outputs are contiguous in a channels-last Y, so the same memory is also the contraction
// [pixels / P, P * 32] x [P * 32, P * K] with block-diagonal filters: a quarter of the tiles, full 128-byte rows, 256 columns.
// Filters [K][32] -> [P * K][P * 32]: row q * K + k holds filter k in columns [32 q, 32 q + 32), zeros elsewhere.
__global__ void __launch_bounds__(256) stem_weights_kernel(const int8_t *__restrict__ w, int8_t *__restrict__ out, int K, int P) {
  const int total = P * K * P * 32;
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < total; i += gridDim.x * blockDim.x) {
    const int row = i / (P * 32), col = i - row * (P * 32);
    const int q = row / K, k = row - q * K;
    out[i] = (col >> 5) == q ? w[k * 32 + (col & 31)] : (int8_t)0;
  }
}
// A per-channel vector of 4-byte words repeated P times (scale and bias of the packed contraction's P * K columns).
__global__ void __launch_bounds__(256) repeat_words_kernel(const uint32_t *__restrict__ a, const uint32_t *__restrict__ b, uint32_t *__restrict__ out,
                                                           int K, int P) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= P * K) return;
  if (a) out[i] = a[i % K];
  if (b) out[P * K + i] = b[i % K];
}

// ---- stride-2 implicit convolution over pixel pairs -------------------------------------------------------------------
// A pixel of 64 bytes is half a 128-byte K block, and the TMA unit spends its time per ROW it moves, not per byte: a layer
// with 64 int8 channels loaded nine 64-byte rows per output pixel at a quarter of the bandwidth 128-byte rows reach.  With a
// horizontal stride of 2 (3 taps, left padding 1) the channels-last input [N, H, W, C] is read as [N, H, W/2, 2C] instead:
// output column ow needs input columns 2ow-1, 2ow, 2ow+1 = the upper half of pair ow-1 and both halves of pair ow, i.e. a
// two-tap, unit-stride convolution over pairs with zero weights for the lower half of the first tap.  Six 128-byte rows per
// output pixel instead of nine 64-byte ones; a third more MMA work, which this layer has to spare.
// Filters [K, C, R, 3] -> [K][R][2][2C].
//
// With a horizontal stride of 1 (padding 1 on both sides, even W) the same view serves two contractions that each produce
// every other output column, written into the output read as [N, Ho, W/2, 2K]: the even columns 2j need inputs 2j-1, 2j,
// 2j+1 -- the stride-2 pattern, pairs j-1 and j, into channels [0, K) of output pair j -- and the odd columns 2j+1 need
// 2j, 2j+1, 2j+2: pairs j and j+1 with zero weights for the upper half of the second tap (`odd`), into channels [K, 2K).
template <typename T>
__global__ void __launch_bounds__(256) pair_weights_kernel(const T *__restrict__ w, T *__restrict__ out, long long filters, int C, int R, int odd) {
  const long long per = (long long)R * 2 * 2 * C, total = filters * per;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const long long k = i / per;
    const int rem = (int)(i - k * per), r = rem / (4 * C), sp = (rem / (2 * C)) & 1, cc = rem % (2 * C);
    const int c = cc % C, upper = cc / C;
    // original tap, -1: no such tap (zero weight)
    const int s = odd ? (sp == 0 ? (upper ? 1 : 0) : (upper ? -1 : 2)) : (sp == 0 ? (upper ? 0 : -1) : (upper ? 2 : 1));
    out[i] = s < 0 ? (T)0 : w[((k * C + c) * R + r) * 3 + s];
  }
}

// ---- direct convolution for the 3-channel 3x3 first layer ----------------------------------------------------------
// K = 27: as a contraction this layer is one K block per tile and all epilogue (2.9 of the int8 conv net's 8.5 ms for
// 0.4 % of its flops, plus an unfold that writes 10x the image).  Here a thread owns one output pixel: its 27 inputs sit
// in registers (int8: packed four to a word for dp4a), the weights are broadcast from shared memory channel by channel,
// and every output goes through the scalar form of the fused epilogue (epi_value), so results equal the contraction's.
// Channels-last output: 16 bytes of consecutive channels per store; NCHW: one coalesced store per channel.
constexpr int DIRECT_KD = 27;   // K; padded per filter to 32 int8 (8 words: two 16-byte shared-memory loads) or 28 floats (seven)

template <typename T> struct DirectAcc;
template <> struct DirectAcc<int8_t> { using W = int; static constexpr int NW = 8; static constexpr int KW = 32; };
template <> struct DirectAcc<float> { using W = float; static constexpr int NW = 28; static constexpr int KW = 28; };

// Activation chosen at compile time for the direct kernel's inner loops (0 none, 1 Relu, 2 whatever ep.act says): a switch
// on ep.act per output costs several branches, and the loops are issue-bound.
template <int ACT>
__device__ __forceinline__ float direct_act(float v, const EpiParams &ep) {
  if (ACT == 0) return v;
  if (ACT == 1) return v > 0.f ? v : 0.f;
  return act_apply(v, ep.act, ep.act_alpha);
}
template <int V> struct IntTag { static constexpr int value = V; };

template <typename T, bool NHWC_OUT>
__global__ void __launch_bounds__(256) conv_direct_kernel(const T *__restrict__ x, const typename DirectAcc<T>::W *__restrict__ wq,
                                                          sofie_b200_conv_desc d, int Ho, int Wo, EpiParams ep) {
  using W = typename DirectAcc<T>::W;
  constexpr int NW = DirectAcc<T>::NW;
  extern __shared__ __align__(16) unsigned char dsm[];
  W *ws = reinterpret_cast<W *>(dsm);   // [K filters][NW]
  const int filters = (int)d.K;
  for (int i = threadIdx.x; i < filters * NW; i += blockDim.x) ws[i] = wq[i];
  // per-channel epilogue operands, read once per CTA: scale (or 1), additive fp32 bias (or -0: x + -0 = x bit for bit),
  // int32 bias (or 0).  In either output layout exactly one of row_scale / col_scale and of the ROW / COL bias modes
  // carries the per-channel vector, indexed by the channel.
  // One 16-byte record per channel {scale, fp32 bias, int32 bias (as bits), unused}: one shared-memory load per output.
  float4 *prm = reinterpret_cast<float4 *>(ws + (size_t)filters * NW);
  for (int k = threadIdx.x; k < filters; k += blockDim.x) {
    const int m = ep.bias_mode;
    const float sc = ep.row_scale ? ep.row_scale[k] : (ep.col_scale ? ep.col_scale[k] : 1.f);
    const float bf = (m == SOFIE_B200_BIAS_COL_F32 || m == SOFIE_B200_BIAS_ROW_F32) ? ((const float *)ep.bias)[k]
                                                                                     : (m == SOFIE_B200_BIAS_SCALAR_F32 ? ((const float *)ep.bias)[0] : -0.f);
    const int bi = (m == SOFIE_B200_BIAS_COL_I32 || m == SOFIE_B200_BIAS_ROW_I32) ? ((const int *)ep.bias)[k] : 0;
    prm[k] = make_float4(sc, bf, __int_as_float(bi), 0.f);
  }
  __syncthreads();
  // Without a residual or a full-matrix bias the epilogue of output (pixel, channel k) is this, step for step what
  // epi_value() computes; otherwise epi_value() itself is called.
  const bool lean = ep.residual == nullptr && ep.bias_mode != SOFIE_B200_BIAS_FULL_F32;
  const float alpha = ep.alpha;
  const long long pix = (long long)Ho * Wo, total = d.N * pix;
  const long long gp_raw = (long long)blockIdx.x * blockDim.x + threadIdx.x;   // pixel of the whole batch
  const bool valid = gp_raw < total;
  const long long gp = valid ? gp_raw : total - 1;   // lanes past the end recompute the last pixel and store nothing
  const long long n = gp / pix;
  const int p = (int)(gp - n * pix), oh = p / Wo, ow = p - oh * Wo;
  const int ih0 = oh * d.stride_h - d.pad_top, iw0 = ow * d.stride_w - d.pad_left;
  const int H = (int)d.H, Wd = (int)d.W;
  const T *xn = x + n * 3 * H * Wd;
  W xin[NW];
  {
    T v[32];
#pragma unroll
    for (int i = 27; i < 32; ++i) v[i] = (T)0;
#pragma unroll
    for (int c = 0; c < 3; ++c)
#pragma unroll
      for (int r = 0; r < 3; ++r)
#pragma unroll
        for (int s2 = 0; s2 < 3; ++s2) {
          const int ih = ih0 + r * d.dil_h, iw = iw0 + s2 * d.dil_w;
          v[(c * 3 + r) * 3 + s2] = (ih >= 0 && ih < H && iw >= 0 && iw < Wd) ? xn[((long long)c * H + ih) * Wd + iw] : (T)d.x_zero_point;
        }
    if constexpr (sizeof(T) == 1) {
#pragma unroll
      for (int i = 0; i < 8; ++i)
        xin[i] = (int)((uint32_t)(uint8_t)v[4 * i] | ((uint32_t)(uint8_t)v[4 * i + 1] << 8) | ((uint32_t)(uint8_t)v[4 * i + 2] << 16) |
                       ((uint32_t)(uint8_t)v[4 * i + 3] << 24));
    } else {
#pragma unroll
      for (int i = 0; i < 28; ++i) xin[i] = v[i];
    }
  }
  // (b, i, j) of the contraction the epilogue parameters describe: channels-last Y: row = pixel of the batch, column = channel;
  // NCHW Y: batch = image, row = channel, column = pixel
  auto raw_of = [&](int k) -> uint32_t {
    const W *wk = ws + k * NW;
    if constexpr (sizeof(T) == 1) {
      const int4 w0 = *reinterpret_cast<const int4 *>(wk), w1 = *reinterpret_cast<const int4 *>(wk + 4);
      int acc = __dp4a(xin[0], w0.x, 0);
      acc = __dp4a(xin[1], w0.y, acc); acc = __dp4a(xin[2], w0.z, acc); acc = __dp4a(xin[3], w0.w, acc);
      acc = __dp4a(xin[4], w1.x, acc); acc = __dp4a(xin[5], w1.y, acc); acc = __dp4a(xin[6], w1.z, acc);
      return (uint32_t)acc;   // the eighth word is padding
    } else {
      // seven 16-byte loads (a filter's 28 floats are 16-byte aligned), the 27 FMAs in the order of the K index
      const float4 *w4 = reinterpret_cast<const float4 *>(wk);
      float acc = 0.f;
#pragma unroll
      for (int i = 0; i < 7; ++i) {
        const float4 q = w4[i];
        acc = __fmaf_rn(xin[4 * i], q.x, acc);
        acc = __fmaf_rn(xin[4 * i + 1], q.y, acc);
        acc = __fmaf_rn(xin[4 * i + 2], q.z, acc);
        if (i < 6) acc = __fmaf_rn(xin[4 * i + 3], q.w, acc);
      }
      return __float_as_uint(acc);
    }
  };
  // the lean epilogue with the activation fixed at compile time (tag: IntTag<0|1|2>, see direct_act)
  auto lean_value = [&](int k, auto tag) -> float {
    const uint32_t raw = raw_of(k);
    const float4 pr = prm[k];
    float v = sizeof(T) == 1 ? (float)((int)raw + __float_as_int(pr.z)) : __uint_as_float(raw);
    v = __fadd_rn(__fmul_rn(__fmul_rn(v, pr.x), alpha), pr.y);
    return direct_act<decltype(tag)::value>(v, ep);
  };
  auto value_of = [&](int k, long long eb, long long ei, long long ej) -> float {
    if (!lean) return epi_value(ep, raw_of(k), eb, ei, ej);
    return lean_value(k, IntTag<2>{});
  };
  // runs body(tag) with the tag of ep.act
  auto with_act = [&](auto body) {
    if (ep.act == SOFIE_B200_ACT_RELU) body(IntTag<1>{});
    else if (ep.act == SOFIE_B200_ACT_NONE) body(IntTag<0>{});
    else body(IntTag<2>{});
  };
  if constexpr (!NHWC_OUT) {
    if (valid) {
      if (!lean || ep.y_dtype == SOFIE_B200_I32) {
        for (int k = 0; k < filters; ++k) epi_store_one(ep, raw_of(k), n, k, p);
      } else {   // one coalesced store per channel: consecutive lanes are consecutive pixels of the channel's plane
        const long long o0 = n * ep.stride_y + p;
        for (int k = 0; k < filters; ++k) {
          const float v = value_of(k, n, k, p);
          const long long o = o0 + (long long)k * ep.ldy;
          if (ep.y_dtype == SOFIE_B200_F32) ((float *)ep.Y)[o] = v;
          else if (ep.y_dtype == SOFIE_B200_BF16) ((__nv_bfloat16 *)ep.Y)[o] = __float2bfloat16_rn(v);
          else if (ep.y_dtype == SOFIE_B200_I8) ((int8_t *)ep.Y)[o] = (int8_t)quantize_i(v, ep.out_scale, ep.out_zp, -128, 127);
          else ((uint8_t *)ep.Y)[o] = (uint8_t)quantize_i(v, ep.out_scale, ep.out_zp, 0, 255);
        }
      }
    }
  } else {
    const int ys = ep.y_dtype == SOFIE_B200_F32 || ep.y_dtype == SOFIE_B200_I32 ? 4 : (ep.y_dtype == SOFIE_B200_BF16 ? 2 : 1);
    const int per = 16 / ys;   // channels per 16-byte store
    const int pair = ep.split_out ? 2 : 1;   // fp32 output as TF32 pairs: hi channels, then lo channels
    const bool vec = (filters % per == 0) && (((uintptr_t)ep.Y | (uintptr_t)(ep.ldy * ys)) % 16 == 0) && ep.ldy == (long long)filters * pair;
    if (!vec || ep.y_dtype == SOFIE_B200_I32) {
      if (valid)
        for (int k = 0; k < filters; ++k) epi_store_one(ep, raw_of(k), 0, gp, k);
      return;
    }
    // A warp's 32 pixels are 32 * filters * ys CONTIGUOUS bytes of a channels-last Y: each lane puts its pixel's channels
    // into the warp's staging rows in shared memory, then the warp copies the block out 512 contiguous bytes per instruction
    // (a lane storing its own 16-byte pieces wrote half sectors at a 64-byte stride: 0.28 TB/s on the int8 first layer).
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int row_bytes = filters * ys * pair;
    if (pair == 2) {
      // TF32 pairs: 32 channels at a time.  A pixel's staging row is [32 hi | 32 lo] floats; the warp then writes each
      // 128-byte run to its place (hi at channel k, lo at channel filters + k of the pixel's 2 * filters floats).
      constexpr int KC = 32;
      constexpr int PITCH = KC * 8 + 16;   // 16 bytes of padding: lanes 256 bytes apart would all write the same banks
      unsigned char *st = dsm + (size_t)filters * (NW * sizeof(W) + 16) + (size_t)warp * 32 * PITCH;
      const long long gp0 = gp_raw - lane;
      for (int kc0 = 0; kc0 < filters; kc0 += KC) {
        const int nk = min(KC, filters - kc0);
        auto fill = [&](auto tag) {
#pragma unroll 1
          for (int k0 = 0; k0 < nk; k0 += 4) {
            float v[4], h[4];
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              v[e] = lean ? lean_value(kc0 + k0 + e, tag) : value_of(kc0 + k0 + e, 0, gp, kc0 + k0 + e);
              h[e] = tf32_rn(v[e]);
              v[e] = tf32_rn(__fsub_rn(v[e], h[e]));
            }
            *reinterpret_cast<float4 *>(st + (size_t)lane * PITCH + (size_t)k0 * 4) = make_float4(h[0], h[1], h[2], h[3]);
            *reinterpret_cast<float4 *>(st + (size_t)lane * PITCH + (size_t)(KC + k0) * 4) = make_float4(v[0], v[1], v[2], v[3]);
          }
        };
        with_act(fill);
        __syncwarp();
        const int per_run = nk / 4;   // 16-byte pieces per run
        for (int idx = lane; idx < 64 * per_run; idx += 32) {
          const int run = idx / per_run, u = idx - run * per_run, px = run >> 1, which = run & 1;
          if (gp0 + px < total)
            *reinterpret_cast<uint4 *>((unsigned char *)ep.Y + (gp0 + px) * row_bytes + (size_t)(which * filters + kc0) * 4 + (size_t)u * 16) =
                *reinterpret_cast<const uint4 *>(st + (size_t)px * PITCH + (size_t)which * KC * 4 + (size_t)u * 16);
        }
        __syncwarp();
      }
      return;
    }
    const int pitch = row_bytes + 16;   // padded staging rows: a power-of-two pitch puts every lane's store on the same banks
    unsigned char *stage = dsm + (size_t)filters * (NW * sizeof(W) + 16) + (size_t)warp * 32 * pitch;
    unsigned char *srow = stage + (size_t)lane * pitch;
    if (ys == 1) {
      const int lo = ep.y_dtype == SOFIE_B200_I8 ? -128 : 0, hi = ep.y_dtype == SOFIE_B200_I8 ? 127 : 255;
      // sat(rint(v / out_scale) + zp) as in quantize_i(), with the clamp first (the bounds are integers and rounding is
      // monotonic) and the rounding as an addition of 1.5 * 2^23: no quarter-rate conversion instructions
      const float flo = (float)(lo - ep.out_zp), fhi = (float)(hi - ep.out_zp), oscale = ep.out_scale;
      const int unmagic = ep.out_zp - 0x4B400000;
      auto fill = [&](auto tag) {
        const bool plain = lean && oscale == 1.f;   // no division, no general epilogue
#pragma unroll 1
        for (int k0 = 0; k0 < filters; k0 += 16) {
          uint32_t w[4];
#pragma unroll
          for (int u = 0; u < 4; ++u) {
            int q[4];
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              const int k = k0 + 4 * u + e;
              float v = plain ? lean_value(k, tag) : value_of(k, 0, gp, k);
              if (!plain && oscale != 1.f) v = __fdiv_rn(v, oscale);
              q[e] = __float_as_int(__fadd_rn(fminf(fmaxf(v, flo), fhi), 12582912.f)) + unmagic;
            }
            w[u] = __byte_perm(__byte_perm((uint32_t)q[0], (uint32_t)q[1], 0x0040), __byte_perm((uint32_t)q[2], (uint32_t)q[3], 0x0040), 0x5410);
          }
          *reinterpret_cast<uint4 *>(srow + k0) = make_uint4(w[0], w[1], w[2], w[3]);
        }
      };
      with_act(fill);
    } else if (ys == 2) {
      for (int k0 = 0; k0 < filters; k0 += 8) {
        uint32_t w[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          __nv_bfloat162 h2 = __floats2bfloat162_rn(value_of(k0 + 2 * u, 0, gp, k0 + 2 * u), value_of(k0 + 2 * u + 1, 0, gp, k0 + 2 * u + 1));
          w[u] = *reinterpret_cast<uint32_t *>(&h2);
        }
        *reinterpret_cast<uint4 *>(srow + (size_t)k0 * 2) = make_uint4(w[0], w[1], w[2], w[3]);
      }
    } else {
      for (int k0 = 0; k0 < filters; k0 += 4) {
        float v[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) v[e] = value_of(k0 + e, 0, gp, k0 + e);
        *reinterpret_cast<float4 *>(srow + (size_t)k0 * 4) = make_float4(v[0], v[1], v[2], v[3]);
      }
    }
    __syncwarp();
    const long long gp0 = gp_raw - lane;   // first pixel of this warp
    const long long left = total - gp0;
    const long long bytes_valid = (left >= 32 ? 32 : (left > 0 ? left : 0)) * row_bytes;
    unsigned char *ydst = (unsigned char *)ep.Y + gp0 * row_bytes;
    for (long long off = (long long)lane * 16; off < bytes_valid; off += 512) {
      const int r = (int)(off / row_bytes);
      *reinterpret_cast<uint4 *>(ydst + off) = *reinterpret_cast<const uint4 *>(stage + (size_t)r * pitch + (off - (long long)r * row_bytes));
    }
  }
}

// Weights [K, 3, 3, 3] -> [K][32 int8] or [K][28 floats], zero padded.
template <typename T>
__global__ void __launch_bounds__(256) direct_weights_kernel(const T *__restrict__ w, T *__restrict__ out, long long filters) {
  constexpr int DIRECT_KW = DirectAcc<T>::KW;
  const long long total = filters * DIRECT_KW;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const long long f = i / DIRECT_KW;
    const int k = (int)(i - f * DIRECT_KW);
    out[i] = k < DIRECT_KD ? w[f * DIRECT_KD + k] : (T)0;
  }
}

template <typename T>
__global__ void __launch_bounds__(256) pad_weights_kernel(const T *__restrict__ w, T *__restrict__ wp, long long rows, long long kdim,
                                                          long long kpad) {
  const long long total = rows * kpad;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const long long r = i / kpad, k = i % kpad;
    wp[i] = k < kdim ? w[r * kdim + k] : (T)0;
  }
}

// Dynamic shared memory of conv_direct_kernel: the filters with one record of epilogue operands per channel, and for a
// channels-last output a staging block of 32 pixels per warp (TF32 pairs: 32 channels at a time).  A plan takes the
// direct path only when this fits the opt-in limit; wider first layers unfold.
constexpr size_t kDirectSmemLimit = 160 * 1024;
static size_t direct_smem_bytes(const sofie_b200_conv_desc &d, bool pix_rows, bool pair_out) {
  const size_t wsm = (size_t)d.K * ((d.x_dtype == SOFIE_B200_F32 ? 28 * sizeof(float) : 8 * sizeof(int)) + 16);
  const int threads = pix_rows ? 128 : 256;
  return wsm + (pix_rows ? (pair_out ? (size_t)(threads / 32) * 32 * (32 * 8 + 16)
                                     : (size_t)(threads / 32) * 32 * (d.K * dtype_size(d.y_dtype) + 16)) : 0);
}

}  // namespace sb200

using namespace sb200;

extern "C" {

int sofie_b200_conv_out_shape(const sofie_b200_conv_desc *desc, int64_t *Ho, int64_t *Wo) {
  if (!desc || !Ho || !Wo) return fail(SOFIE_B200_ERR_INVALID, "conv_out_shape: NULL argument");
  return conv_out_shape(*desc, Ho, Wo);
}

int sofie_b200_conv_plan_create(sofie_b200_ctx *ctx, const sofie_b200_conv_desc *desc, const void *W,
                                sofie_b200_conv_plan **out) {
  if (!ctx || !desc || !W || !out) return fail(SOFIE_B200_ERR_INVALID, "conv_plan_create: NULL argument");
  *out = nullptr;
  sofie_b200_conv_desc d = *desc;
  if (d.groups < 1) d.groups = 1;
  if (d.N < 0 || d.C < 1 || d.H < 1 || d.W < 1 || d.K < 1 || d.R < 1 || d.S < 1)
    return fail(SOFIE_B200_ERR_INVALID, "conv_plan_create: bad extent");
  if (d.C % d.groups || d.K % d.groups)
    return fail(SOFIE_B200_ERR_INVALID, "conv_plan_create: channels %lld / filters %lld not divisible by groups %d", (long long)d.C, (long long)d.K, d.groups);
  if (d.x_dtype != SOFIE_B200_F32 && d.x_dtype != SOFIE_B200_I8)
    return fail(SOFIE_B200_ERR_INVALID, "conv_plan_create: input type %d not supported (F32, I8)", d.x_dtype);
  if (d.x_layout < 0 || d.x_layout > 2 || d.y_layout < 0 || d.y_layout > 2)
    return fail(SOFIE_B200_ERR_INVALID, "conv_plan_create: layouts are 0 (NCHW), 1 (channels-last) or 2 (channels-last TF32 pairs)");
  if ((d.x_layout == 2 || d.y_layout == 2) && (d.x_dtype != SOFIE_B200_F32 || d.y_dtype != SOFIE_B200_F32 || d.precise == 0 || d.groups != 1))
    return fail(SOFIE_B200_ERR_INVALID, "conv_plan_create: layout 2 (TF32 pairs) is for one-group F32 convolutions at precise = 1");
  if (d.x_layout == 2 && d.C % 32 != 0)
    return fail(SOFIE_B200_ERR_INVALID, "conv_plan_create: x_layout = 2 needs C to be a multiple of 32");
  if (d.y_layout == 2 && d.K % 4 != 0)
    return fail(SOFIE_B200_ERR_INVALID, "conv_plan_create: y_layout = 2 needs K to be a multiple of 4");
  if (d.x_layout == 1 && (d.C / d.groups) % (16 / dtype_size(d.x_dtype)) != 0)
    return fail(SOFIE_B200_ERR_INVALID, "conv_plan_create: a channels-last input needs C/groups to be a whole number of 16-byte vectors");
  int64_t Ho, Wo;
  int rc = conv_out_shape(d, &Ho, &Wo);
  if (rc) return rc;
  SB_CUDA(cudaSetDevice(ctx->device));
  const int es = dtype_size(d.x_dtype);
  sofie_b200_conv_plan *p = new sofie_b200_conv_plan();
  p->pix_rows = d.y_layout != 0;
  p->pair_out = d.y_layout == 2;
  p->ctx = ctx; p->d = d; p->Ho = Ho; p->Wo = Wo;
  p->cg = d.C / d.groups; p->kg = d.K / d.groups;
  p->kdim = p->cg * d.R * d.S;
  const int64_t vec = 16 / es;
  p->kpad = (p->kdim + vec - 1) / vec * vec;
  // The int8 first layer with a channels-last output goes to the tensor cores once there are enough output pixels to fill
  // the machine with 128-pixel tiles (see unfold_c3k3_kernel); small ones and the fp32 layer take the direct kernel.
  const bool first_layer = d.groups == 1 && d.C == 3 && d.R == 3 && d.S == 3 && d.x_layout == 0;
  p->stem = first_layer && d.x_dtype == SOFIE_B200_I8 && d.y_layout == 1 && d.K % 16 == 0 && d.K <= 256 &&
            (d.N > 0 ? d.N : 1) * Ho * Wo >= 16384 && !(d.flags & SOFIE_B200_CONV_UNFOLD);
  if (first_layer && !p->stem && d.K <= 256 && !(d.flags & SOFIE_B200_CONV_UNFOLD) &&
      direct_smem_bytes(d, p->pix_rows, p->pair_out) <= kDirectSmemLimit) {
    // the 3-channel first layer: direct kernel (see conv_direct_kernel); the plan only keeps the padded weights
    p->direct = 1;
    const int DIRECT_KW = es == 4 ? DirectAcc<float>::KW : DirectAcc<int8_t>::KW;
    p->kpad = DIRECT_KW;
    if (cudaMalloc(&p->w_padded, (size_t)(d.K * DIRECT_KW * es)) != cudaSuccess) {
      delete p;
      return fail(SOFIE_B200_ERR_CUDA, "conv_plan_create: allocating padded weights failed: %s", cudaGetErrorString(cudaGetLastError()));
    }
    const unsigned wg = (unsigned)((d.K * DIRECT_KW + 255) / 256);
    if (es == 4) direct_weights_kernel<float><<<wg, 256, 0, ctx->stream>>>((const float *)W, (float *)p->w_padded, d.K);
    else direct_weights_kernel<int8_t><<<wg, 256, 0, ctx->stream>>>((const int8_t *)W, (int8_t *)p->w_padded, d.K);
    ctx->launches++;
    sofie_b200_gemm_desc &e = p->edesc;   // the contraction whose epilogue is applied
    e.ab_dtype = d.x_dtype; e.y_dtype = d.y_dtype; e.K = DIRECT_KD;
    const int64_t imgs = d.N > 0 ? d.N : 1;
    if (p->pix_rows) { e.M = imgs * Ho * Wo; e.N = d.K; e.batch = 1; e.ldy = p->pair_out ? 2 * d.K : d.K; }
    else { e.M = d.K; e.N = Ho * Wo; e.batch = imgs; e.ldy = Ho * Wo; e.stride_y = d.K * Ho * Wo; e.stride_r = d.K * Ho * Wo; }
    *out = p;
    return 0;
  }
  // fp32 at fp32 accuracy without an unfold: X is a channels-last tensor of TF32 pairs (written by a convolution with
  // y_layout = 2), read in im2col mode by the chunk-promotion kernel; the filters are split once here.
  if (d.x_layout == 2) {
    if (d.y_layout == 0) { delete p; return fail(SOFIE_B200_ERR_INVALID, "conv_plan_create: x_layout = 2 needs a channels-last output (y_layout 1 or 2)"); }
    const int64_t rows = (d.N > 0 ? d.N : 1) * Ho * Wo;
    Im2colDesc ic;
    ic.on = 1; ic.N = d.N > 0 ? d.N : 1; ic.H = d.H; ic.W = d.W; ic.C = d.C; ic.Cs = 2 * d.C; ic.Ho = Ho; ic.Wo = Wo;
    ic.R = (int)d.R; ic.S = (int)d.S; ic.pt = (int)d.pad_top; ic.pl = (int)d.pad_left; ic.pb = (int)d.pad_bottom; ic.pr = (int)d.pad_right;
    ic.sh = (int)d.stride_h; ic.sw = (int)d.stride_w; ic.dh = (int)d.dil_h; ic.dw = (int)d.dil_w;
    sofie_b200_gemm_desc g{};
    g.trans_a = 0; g.trans_b = 1; g.ab_dtype = SOFIE_B200_F32; g.y_dtype = SOFIE_B200_F32;
    g.M = rows; g.N = d.K; g.K = 3 * p->kdim; g.batch = 1; g.lda = 2 * p->kdim; g.ldb = 2 * p->kdim;
    g.ldy = p->pair_out ? 2 * d.K : d.K; g.precise = 0;
    rc = (rows < 0x7fffffffLL && 3 * p->kdim < 0x7fffffffLL) ? gemm_plan_create_promote_im2col(ctx, g, ic, p->pair_out, &p->gemm) : 1;
    if (rc) { delete p; return rc < 0 ? rc : fail(SOFIE_B200_ERR_INVALID, "conv_plan_create: this convolution cannot run from a tensor of TF32 pairs (x_layout = 2)"); }
    p->implicit = 1; p->nhwc = 1; p->split = 1; p->kpad = p->kdim;
    void *w_perm = nullptr;
    if (cudaMalloc(&w_perm, (size_t)(d.K * p->kdim * es)) != cudaSuccess || cudaMalloc(&p->w_padded, (size_t)(d.K * 2 * p->kdim * es)) != cudaSuccess) {
      cudaGetLastError();
      if (w_perm) cudaFree(w_perm);
      sofie_b200_gemm_plan_destroy(p->gemm);
      delete p;
      return fail(SOFIE_B200_ERR_CUDA, "conv_plan_create: allocating the filter buffers failed");
    }
    const long long wt = d.K * p->kdim;
    const unsigned wg = (unsigned)std::min<long long>((wt + 255) / 256, (long long)ctx->sm_count * 16);
    reorder_weights_kernel<float><<<wg, 256, 0, ctx->stream>>>((const float *)W, (float *)w_perm, d.K, (int)p->cg, (int)(d.R * d.S));
    ctx->launches++;
    rc = split2_enqueue(ctx, (const float *)w_perm, (float *)p->w_padded, d.K, p->kdim, p->kdim, p->kdim, 1, 0, 0);
    cudaStreamSynchronize(ctx->stream);
    cudaFree(w_perm);
    if (rc) { sofie_b200_gemm_plan_destroy(p->gemm); cudaFree(p->w_padded); delete p; return rc; }
    *out = p;
    return 0;
  }
  if (d.y_layout == 2 && !p->direct) { delete p; return fail(SOFIE_B200_ERR_INVALID, "conv_plan_create: y_layout = 2 needs x_layout = 2 or the 3-channel first layer"); }
  // Implicit convolution: both tensors channels-last, one group, the channels of a pixel a whole number of 64-byte K
  // blocks, and padding that reads as zero (TMA fills out-of-range pixels with zeros, so a non-zero input zero point
  // needs an unpadded convolution).  int8, or fp32 where single-pass TF32 was asked for.
  {
    const bool has_pad = d.pad_top || d.pad_bottom || d.pad_left || d.pad_right;
    const bool type_ok = d.x_dtype == SOFIE_B200_I8 ? (d.x_zero_point == 0 || !has_pad) : d.precise == 0;
    const int64_t rows = (d.N > 0 ? d.N : 1) * Ho * Wo;
    if (d.groups == 1 && d.x_layout == 1 && d.y_layout == 1 && type_ok && (d.C * es) % 64 == 0 && rows < 0x7fffffffLL &&
        d.K * p->kdim < 0x7fffffffLL && !(d.flags & SOFIE_B200_CONV_UNFOLD)) {
      Im2colDesc ic;
      ic.on = 1; ic.N = d.N > 0 ? d.N : 1; ic.H = d.H; ic.W = d.W; ic.C = d.C; ic.Ho = Ho; ic.Wo = Wo;
      ic.R = (int)d.R; ic.S = (int)d.S; ic.pt = (int)d.pad_top; ic.pl = (int)d.pad_left; ic.pb = (int)d.pad_bottom; ic.pr = (int)d.pad_right;
      ic.sh = (int)d.stride_h; ic.sw = (int)d.stride_w; ic.dh = (int)d.dil_h; ic.dw = (int)d.dil_w;
      // pixels of 64 bytes under a horizontal stride of 2: read pixel pairs (see pair_weights_kernel)
      const bool pairs = d.C * es == 64 && d.stride_w == 2 && d.S == 3 && d.dil_w == 1 && d.pad_left == 1 && d.pad_right <= 1 && d.W % 2 == 0 &&
                         Wo == d.W / 2;
      // ... and under a horizontal stride of 1: two contractions over the pairs, for the even and the odd output columns
      const bool pairs1 = d.C * es == 64 && d.stride_w == 1 && d.S == 3 && d.dil_w == 1 && d.pad_left == 1 && d.pad_right == 1 && d.W % 2 == 0 &&
                          Wo == d.W && (d.K * dtype_size(d.y_dtype)) % 16 == 0 && rows >= 16384;
      int64_t kimp = p->kdim;
      if (pairs || pairs1) {
        ic.W = d.W / 2; ic.C = 2 * d.C; ic.S = 2; ic.sw = 1; ic.pl = 1; ic.pr = 0;
        kimp = d.R * 2 * 2 * d.C;
      }
      if (pairs1) ic.Wo = Wo / 2;
      sofie_b200_gemm_desc g{};
      g.trans_a = 0; g.trans_b = 1; g.ab_dtype = d.x_dtype; g.y_dtype = d.y_dtype;
      g.M = pairs1 ? rows / 2 : rows; g.N = d.K; g.K = kimp; g.batch = 1; g.lda = kimp; g.ldb = kimp; g.ldy = pairs1 ? 2 * d.K : d.K; g.precise = 0;
      const bool y_ok = d.y_dtype == SOFIE_B200_F32 || d.y_dtype == SOFIE_B200_BF16 || d.y_dtype == SOFIE_B200_I8 || d.y_dtype == SOFIE_B200_U8 ||
                        (d.y_dtype == SOFIE_B200_I32 && d.x_dtype == SOFIE_B200_I8);
      rc = y_ok ? gemm_plan_create_im2col(ctx, g, ic, &p->gemm) : 1;
      if (rc < 0) { delete p; return rc; }
      if (rc == 0 && pairs1) {
        Im2colDesc io = ic;
        io.pl = 0; io.pr = 1;   // odd columns: pairs j and j + 1
        rc = gemm_plan_create_im2col(ctx, g, io, &p->gemm_odd);
        if (rc) { sofie_b200_gemm_plan_destroy(p->gemm); p->gemm = nullptr; delete p; return rc < 0 ? rc : fail(SOFIE_B200_ERR_INVALID, "conv_plan_create: no plan for the odd columns"); }
      }
      if (rc == 0) {
        p->implicit = 1; p->nhwc = 1; p->kpad = p->kdim;
        if (cudaMalloc(&p->w_padded, (size_t)(d.K * kimp * es)) != cudaSuccess || (pairs1 && cudaMalloc(&p->w_odd, (size_t)(d.K * kimp * es)) != cudaSuccess)) {
          sofie_b200_gemm_plan_destroy(p->gemm);
          if (p->gemm_odd) sofie_b200_gemm_plan_destroy(p->gemm_odd);
          if (p->w_padded) cudaFree(p->w_padded);
          delete p;
          return fail(SOFIE_B200_ERR_CUDA, "conv_plan_create: allocating the filter buffer failed: %s", cudaGetErrorString(cudaGetLastError()));
        }
        const long long wt = d.K * kimp;
        const unsigned wg = (unsigned)std::min<long long>((wt + 255) / 256, (long long)ctx->sm_count * 16);
        if (pairs1 && es == 4) {
          pair_weights_kernel<float><<<wg, 256, 0, ctx->stream>>>((const float *)W, (float *)p->w_padded, d.K, (int)d.C, (int)d.R, 0);
          pair_weights_kernel<float><<<wg, 256, 0, ctx->stream>>>((const float *)W, (float *)p->w_odd, d.K, (int)d.C, (int)d.R, 1);
        } else if (pairs1) {
          pair_weights_kernel<int8_t><<<wg, 256, 0, ctx->stream>>>((const int8_t *)W, (int8_t *)p->w_padded, d.K, (int)d.C, (int)d.R, 0);
          pair_weights_kernel<int8_t><<<wg, 256, 0, ctx->stream>>>((const int8_t *)W, (int8_t *)p->w_odd, d.K, (int)d.C, (int)d.R, 1);
        }
        else if (pairs && es == 4) pair_weights_kernel<float><<<wg, 256, 0, ctx->stream>>>((const float *)W, (float *)p->w_padded, d.K, (int)d.C, (int)d.R, 0);
        else if (pairs) pair_weights_kernel<int8_t><<<wg, 256, 0, ctx->stream>>>((const int8_t *)W, (int8_t *)p->w_padded, d.K, (int)d.C, (int)d.R, 0);
        else if (es == 4) reorder_weights_kernel<float><<<wg, 256, 0, ctx->stream>>>((const float *)W, (float *)p->w_padded, d.K, (int)p->cg, (int)(d.R * d.S));
        else reorder_weights_kernel<int8_t><<<wg, 256, 0, ctx->stream>>>((const int8_t *)W, (int8_t *)p->w_padded, d.K, (int)p->cg, (int)(d.R * d.S));
        cudaError_t e = cudaGetLastError();
        if (e != cudaSuccess) {
          sofie_b200_gemm_plan_destroy(p->gemm);
          if (p->gemm_odd) sofie_b200_gemm_plan_destroy(p->gemm_odd);
          cudaFree(p->w_padded);
          if (p->w_odd) cudaFree(p->w_odd);
          delete p;
          return fail(SOFIE_B200_ERR_CUDA, "conv_plan_create: %s", cudaGetErrorString(e));
        }
        ctx->launches += pairs1 ? 2 : 1;
        *out = p;
        return 0;
      }
    }
  }
  // fp32 at fp32 accuracy: large convolutions run as 3xTF32 on the tensor cores, with the weights split once here and
  // the input split by the unfold kernel; small ones stay on the fp32 FMA kernel.
  const int64_t images = d.N > 0 ? d.N : 1;
  sofie_b200_gemm_desc g{};
  g.trans_a = 0; g.trans_b = 1;
  g.ab_dtype = d.x_dtype; g.y_dtype = d.y_dtype;
  if (!p->pix_rows) {   // Y[n] = W x xcol[n]^T: channels are rows, one contraction per image (batched)
    g.M = p->kg; g.N = Ho * Wo; g.batch = images;
    g.ldy = Ho * Wo; g.stride_a = 0; g.stride_y = d.K * Ho * Wo; g.stride_r = d.K * Ho * Wo;
  } else {              // Y = xcol x W^T: all output pixels of the batch are the rows, channels the columns (channels-last Y)
    g.M = images * Ho * Wo; g.N = p->kg; g.batch = 1;
    g.ldy = d.K;
  }
  if (d.x_dtype == SOFIE_B200_F32 && d.precise != 0 && images <= 65535 &&
      2.0 * (double)p->kg * (double)(Ho * Wo) * (double)p->kpad * (double)images >= SPLIT_MIN_FLOPS) {
    const int64_t ks = split_ks(p->kdim);   // operands stored hi | lo, each segment ks wide; the contraction runs over 3 * ks
    g.K = 3 * ks; g.lda = g.ldb = 2 * ks; g.stride_b = p->pix_rows ? 0 : Ho * Wo * 2 * ks; g.precise = 0;
    rc = gemm_plan_create_promote(ctx, g, &p->gemm);
    if (rc < 0) { delete p; return rc; }
    p->split = (rc == 0);
    if (p->split) p->kpad = ks;
  }
  // channels-last unfold when the per-group channel count is a whole number of 16-byte vectors (then kpad == kdim)
  p->nhwc = (d.x_layout == 1 || (p->cg % vec == 0 && d.N <= 65535)) ? 1 : 0;
  const void *w_src = W;
  void *w_perm = nullptr;
  if (p->nhwc) {
    if (cudaMalloc(&w_perm, (size_t)(d.K * p->kdim * es)) != cudaSuccess) {
      if (p->gemm) sofie_b200_gemm_plan_destroy(p->gemm);
      delete p;
      return fail(SOFIE_B200_ERR_CUDA, "conv_plan_create: allocating the weight re-layout buffer failed: %s", cudaGetErrorString(cudaGetLastError()));
    }
    const long long wt = d.K * p->kdim;
    const unsigned wg = (unsigned)std::min<long long>((wt + 255) / 256, (long long)ctx->sm_count * 16);
    if (es == 4) reorder_weights_kernel<float><<<wg, 256, 0, ctx->stream>>>((const float *)W, (float *)w_perm, d.K, (int)p->cg, (int)(d.R * d.S));
    else reorder_weights_kernel<int8_t><<<wg, 256, 0, ctx->stream>>>((const int8_t *)W, (int8_t *)w_perm, d.K, (int)p->cg, (int)(d.R * d.S));
    ctx->launches++;
    w_src = w_perm;
  }
  // the re-layout buffer is only read by kernels enqueued below; it is freed once they have run
  auto free_perm = [&]() { if (w_perm) { cudaStreamSynchronize(ctx->stream); cudaFree(w_perm); w_perm = nullptr; } };
  const int64_t kw = p->split ? 2 * p->kpad : p->kpad;   // pitch of one weight row / one unfolded pixel
  if (cudaMalloc(&p->w_padded, (size_t)(d.K * kw * es)) != cudaSuccess) {
    free_perm();
    if (p->gemm) sofie_b200_gemm_plan_destroy(p->gemm);
    delete p;
    return fail(SOFIE_B200_ERR_CUDA, "conv_plan_create: allocating padded weights failed: %s", cudaGetErrorString(cudaGetLastError()));
  }
  const long long total = d.K * p->kpad;
  const unsigned grid = (unsigned)std::min<long long>((total + 255) / 256, (long long)ctx->sm_count * 16);
  if (p->split) {
    rc = split2_enqueue(ctx, (const float *)w_src, (float *)p->w_padded, d.K, p->kdim, p->kpad, p->kdim, 1, 0, 0);
    free_perm();
    if (rc) { sofie_b200_gemm_plan_destroy(p->gemm); cudaFree(p->w_padded); delete p; return rc; }
    *out = p;
    return 0;
  }
  if (d.x_dtype == SOFIE_B200_F32)
    pad_weights_kernel<float><<<grid, 256, 0, ctx->stream>>>((const float *)w_src, (float *)p->w_padded, d.K, p->kdim, p->kpad);
  else
    pad_weights_kernel<int8_t><<<grid, 256, 0, ctx->stream>>>((const int8_t *)w_src, (int8_t *)p->w_padded, d.K, p->kdim, p->kpad);
  cudaError_t e = cudaGetLastError();
  free_perm();
  if (e != cudaSuccess) { cudaFree(p->w_padded); delete p; return fail(SOFIE_B200_ERR_CUDA, "conv_plan_create: %s", cudaGetErrorString(e)); }
  ctx->launches++;

  g.K = p->kpad; g.lda = p->kpad; g.ldb = p->kpad; g.stride_b = p->pix_rows ? 0 : Ho * Wo * p->kpad;
  g.precise = d.precise;
  if (p->stem) {
    // P output pixels per row of the contraction (see stem_weights_kernel): as many as keep P * K columns within one tile
    int P = 4;
    while (P > 1 && (d.K * P > 256 || (images * Ho * Wo) % P != 0)) P >>= 1;
    if (P > 1) {
      void *wb = nullptr;
      if (cudaMalloc(&wb, (size_t)(P * d.K) * (size_t)(P * 32)) != cudaSuccess || cudaMalloc(&p->stem_vec, (size_t)(2 * P * d.K) * 4) != cudaSuccess) {
        cudaGetLastError();
        if (wb) cudaFree(wb);
        cudaFree(p->w_padded);
        delete p;
        return fail(SOFIE_B200_ERR_CUDA, "conv_plan_create: allocating the packed first-layer filters failed");
      }
      stem_weights_kernel<<<(unsigned)((P * d.K * P * 32 + 255) / 256), 256, 0, ctx->stream>>>((const int8_t *)p->w_padded, (int8_t *)wb, (int)d.K, P);
      ctx->launches++;
      cudaStreamSynchronize(ctx->stream);   // the unpacked copy is read by the kernel above
      cudaFree(p->w_padded);
      p->w_padded = wb;
      p->stem_pack = P;
      g.M = images * Ho * Wo / P; g.N = P * d.K; g.K = P * 32; g.lda = g.ldb = P * 32; g.ldy = P * d.K;
    }
  }
  rc = sofie_b200_gemm_plan_create(ctx, &g, &p->gemm);
  if (rc) { cudaFree(p->w_padded); if (p->stem_vec) cudaFree(p->stem_vec); delete p; return rc; }
  *out = p;
  return 0;
}

int sofie_b200_conv_plan_destroy(sofie_b200_conv_plan *plan) {
  if (!plan) return 0;
  cudaSetDevice(plan->ctx->device);
  if (plan->gemm) sofie_b200_gemm_plan_destroy(plan->gemm);
  if (plan->gemm_odd) sofie_b200_gemm_plan_destroy(plan->gemm_odd);
  if (plan->w_padded) cudaFree(plan->w_padded);
  if (plan->w_odd) cudaFree(plan->w_odd);
  if (plan->stem_vec) cudaFree(plan->stem_vec);
  delete plan;
  return 0;
}

const char *sofie_b200_conv_plan_kernel(const sofie_b200_conv_plan *plan) {
  if (!plan) return "";
  if (plan->gemm_odd) return "umma_im2col_x2";   // implicit convolution over pixel pairs, even and odd output columns: two launches
  return plan->direct ? "direct" : sofie_b200_gemm_plan_kernel(plan->gemm);   // "umma_im2col": implicit convolution
}

int64_t sofie_b200_conv_workspace_bytes(const sofie_b200_conv_plan *plan) {
  if (!plan) return 0;
  if (plan->direct || plan->implicit) return 0;
  const int64_t es = dtype_size(plan->d.x_dtype);
  const int64_t xcol = (int64_t)plan->d.groups * plan->d.N * plan->Ho * plan->Wo * plan->kpad * (plan->split ? 2 : 1) * es;
  if (!plan->nhwc || plan->d.x_layout == 1) return xcol;   // a channels-last input needs no copy
  return (xcol + 255) / 256 * 256 + plan->d.N * plan->d.C * plan->d.H * plan->d.W * es;   // + the channels-last copy of the input
}

int sofie_b200_conv_enqueue(sofie_b200_conv_plan *plan, const void *X, void *Y, void *workspace,
                            const sofie_b200_epilogue *ep) {
  if (!plan) return fail(SOFIE_B200_ERR_INVALID, "conv_enqueue: plan is NULL");
  const sofie_b200_conv_desc &d = plan->d;
  if (d.N == 0) return 0;
  if (plan->pair_out && ((uintptr_t)Y % 16) != 0) return fail(SOFIE_B200_ERR_INVALID, "conv_enqueue: a TF32-pair output must be 16-byte aligned");
  if (plan->direct) {
    if (!X || !Y) return fail(SOFIE_B200_ERR_INVALID, "conv_enqueue: NULL tensor");
    sofie_b200_ctx *ctx = plan->ctx;
    SB_CUDA(cudaSetDevice(ctx->device));
    const long long pix = plan->Ho * plan->Wo;
    sofie_b200_epilogue e{};
    e.alpha = 1.f; e.beta = 1.f; e.out_scale = 1.f;
    if (ep) {
      if (ep->row_scale) return fail(SOFIE_B200_ERR_INVALID, "conv_enqueue: row_scale has no meaning for a convolution");
      e = *ep;
      if (plan->pix_rows) {
        if (ep->bias_mode == SOFIE_B200_BIAS_ROW_F32 || ep->bias_mode == SOFIE_B200_BIAS_ROW_I32 || ep->bias_mode == SOFIE_B200_BIAS_FULL_F32)
          return fail(SOFIE_B200_ERR_INVALID, "conv_enqueue: bias_mode %d not supported for a convolution", ep->bias_mode);
        e.ldr = d.K;
      } else {   // channels are the rows of the contraction this convolution stands for
        e.row_scale = ep->col_scale;
        e.col_scale = nullptr;
        switch (ep->bias_mode) {
          case SOFIE_B200_BIAS_NONE: case SOFIE_B200_BIAS_SCALAR_F32: break;
          case SOFIE_B200_BIAS_COL_F32: e.bias_mode = SOFIE_B200_BIAS_ROW_F32; break;
          case SOFIE_B200_BIAS_COL_I32: e.bias_mode = SOFIE_B200_BIAS_ROW_I32; break;
          default: return fail(SOFIE_B200_ERR_INVALID, "conv_enqueue: bias_mode %d not supported for a convolution", ep->bias_mode);
        }
        e.ldr = pix;
      }
    }
    EpiParams epi;
    int rc = gemm_make_epi(plan->edesc, Y, &e, &epi);
    if (rc) return rc;
    const long long total = d.N * pix;
    // channels-last output: 128 threads and a staging block of 32 pixels x K channels per warp behind the weights
    const int threads = plan->pix_rows ? 128 : 256;
    const unsigned grid = (unsigned)((total + threads - 1) / threads);
    const size_t sm = direct_smem_bytes(d, plan->pix_rows, plan->pair_out);
    epi.split_out = plan->pair_out;
    if (d.x_dtype == SOFIE_B200_F32) {
      if (plan->pix_rows) {
        SB_CUDA(cudaFuncSetAttribute(conv_direct_kernel<float, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kDirectSmemLimit));
        conv_direct_kernel<float, true><<<grid, threads, sm, ctx->stream>>>((const float *)X, (const float *)plan->w_padded, d, (int)plan->Ho, (int)plan->Wo, epi);
      } else conv_direct_kernel<float, false><<<grid, threads, sm, ctx->stream>>>((const float *)X, (const float *)plan->w_padded, d, (int)plan->Ho, (int)plan->Wo, epi);
    } else {
      if (plan->pix_rows) {
        SB_CUDA(cudaFuncSetAttribute(conv_direct_kernel<int8_t, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kDirectSmemLimit));
        conv_direct_kernel<int8_t, true><<<grid, threads, sm, ctx->stream>>>((const int8_t *)X, (const int *)plan->w_padded, d, (int)plan->Ho, (int)plan->Wo, epi);
      } else conv_direct_kernel<int8_t, false><<<grid, threads, sm, ctx->stream>>>((const int8_t *)X, (const int *)plan->w_padded, d, (int)plan->Ho, (int)plan->Wo, epi);
    }
    SB_CUDA(cudaGetLastError());
    ctx->launches++;
    return 0;
  }
  if (plan->implicit) {
    if (!X || !Y) return fail(SOFIE_B200_ERR_INVALID, "conv_enqueue: NULL tensor");
    sofie_b200_epilogue e{};
    e.alpha = 1.f; e.beta = 1.f; e.out_scale = 1.f;
    if (ep) {
      if (ep->row_scale) return fail(SOFIE_B200_ERR_INVALID, "conv_enqueue: row_scale has no meaning for a convolution");
      if (ep->bias_mode == SOFIE_B200_BIAS_ROW_F32 || ep->bias_mode == SOFIE_B200_BIAS_ROW_I32 || ep->bias_mode == SOFIE_B200_BIAS_FULL_F32)
        return fail(SOFIE_B200_ERR_INVALID, "conv_enqueue: bias_mode %d not supported for a convolution", ep->bias_mode);
      e = *ep;
      e.ldr = d.K;
    }
    if (plan->gemm_odd) {
      // even output columns, then the odd ones: the output (and a residual) read as [N, Ho, W/2, 2K], channels [0, K) and [K, 2K)
      e.ldr = 2 * d.K;
      int rc = sofie_b200_gemm_enqueue(plan->gemm, X, plan->w_padded, Y, &e);
      if (rc) return rc;
      if (e.residual) e.residual = (const char *)e.residual + d.K * dtype_size(e.residual_dtype);
      return sofie_b200_gemm_enqueue(plan->gemm_odd, X, plan->w_odd, (char *)Y + d.K * dtype_size(d.y_dtype), &e);
    }
    return sofie_b200_gemm_enqueue(plan->gemm, X, plan->w_padded, Y, &e);
  }
  if (!X || !Y || !workspace) return fail(SOFIE_B200_ERR_INVALID, "conv_enqueue: NULL tensor or workspace");
  if ((uintptr_t)workspace % 16) return fail(SOFIE_B200_ERR_INVALID, "conv_enqueue: workspace must be 16-byte aligned");
  sofie_b200_ctx *ctx = plan->ctx;
  SB_CUDA(cudaSetDevice(ctx->device));
  const int es = dtype_size(d.x_dtype);
  const long long pix = plan->Ho * plan->Wo;
  const long long total = (long long)d.groups * d.N * pix * (plan->kpad / (16 / es));
  const unsigned grid = (unsigned)std::min<long long>((total + 255) / 256, (long long)ctx->sm_count * 32);
  if (plan->nhwc) {
    const long long xcol_bytes = (long long)d.groups * d.N * pix * plan->kpad * (plan->split ? 2 : 1) * es;
    void *xl = (char *)workspace + (xcol_bytes + 255) / 256 * 256;
    const int HW = (int)(d.H * d.W), C_ = (int)d.C;
    if (d.x_layout == 1) {
      xl = const_cast<void *>(X);
    } else {
    if (es == 1 && C_ % 4 == 0 && HW % 4 == 0)
      nchw_to_nhwc_bytes_kernel<<<dim3((HW + 127) / 128, (C_ + 63) / 64, (unsigned)d.N), 256, 0, ctx->stream>>>((const uint8_t *)X, (uint8_t *)xl, C_, HW);
    else if (es == 1)
      nchw_to_nhwc_kernel<uint8_t><<<dim3((HW + 31) / 32, (C_ + 31) / 32, (unsigned)d.N), 256, 0, ctx->stream>>>((const uint8_t *)X, (uint8_t *)xl, C_, HW);
    else
      nchw_to_nhwc_kernel<uint32_t><<<dim3((HW + 31) / 32, (C_ + 31) / 32, (unsigned)d.N), 256, 0, ctx->stream>>>((const uint32_t *)X, (uint32_t *)xl, C_, HW);
    SB_CUDA(cudaGetLastError());
    ctx->launches++;
    }
    if (plan->split)
      unfold_nhwc_kernel<float, 4, true><<<grid, 256, 0, ctx->stream>>>((const float *)xl, (float *)workspace, d, plan->Ho, plan->Wo, plan->cg, plan->kdim, plan->kpad, 0.f);
    else if (es == 4)
      unfold_nhwc_kernel<float, 4, false><<<grid, 256, 0, ctx->stream>>>((const float *)xl, (float *)workspace, d, plan->Ho, plan->Wo, plan->cg, plan->kdim, plan->kpad, 0.f);
    else
      unfold_nhwc_kernel<int8_t, 16, false><<<grid, 256, 0, ctx->stream>>>((const int8_t *)xl, (int8_t *)workspace, d, plan->Ho, plan->Wo, plan->cg, plan->kdim, plan->kpad, (int8_t)d.x_zero_point);
  } else if (plan->split)
    unfold_split_kernel<<<grid, 256, 0, ctx->stream>>>((const float *)X, (float *)workspace, d, plan->Ho, plan->Wo, plan->cg, plan->kdim, plan->kpad);
  else if (d.x_dtype == SOFIE_B200_F32)
    unfold_kernel<float, 4><<<grid, 256, 0, ctx->stream>>>((const float *)X, (float *)workspace, d, plan->Ho, plan->Wo, plan->cg, plan->kdim, plan->kpad, 0.f);
  else if (plan->stem)
    unfold_c3k3_kernel<<<(unsigned)((d.N * pix + 255) / 256), 256, 0, ctx->stream>>>((const int8_t *)X, (uint4 *)workspace, d, (int)plan->Ho, (int)plan->Wo);
  else
    unfold_kernel<int8_t, 16><<<grid, 256, 0, ctx->stream>>>((const int8_t *)X, (int8_t *)workspace, d, plan->Ho, plan->Wo, plan->cg, plan->kdim, plan->kpad, (int8_t)d.x_zero_point);
  SB_CUDA(cudaGetLastError());
  ctx->launches++;

  // Output channels are accumulator rows here: per-channel vectors of the caller's epilogue
  // (documented per column = per channel) become per-row vectors.
  sofie_b200_epilogue e{};
  e.alpha = 1.f; e.beta = 1.f; e.out_scale = 1.f;
  const int ys = dtype_size(d.y_dtype);
  if (plan->pix_rows) {
    // Channels are accumulator columns: the caller's per-channel vectors apply as they are.
    if (ep) {
      if (ep->row_scale) return fail(SOFIE_B200_ERR_INVALID, "conv_enqueue: row_scale has no meaning for a convolution");
      if (ep->bias_mode == SOFIE_B200_BIAS_ROW_F32 || ep->bias_mode == SOFIE_B200_BIAS_ROW_I32 || ep->bias_mode == SOFIE_B200_BIAS_FULL_F32)
        return fail(SOFIE_B200_ERR_INVALID, "conv_enqueue: bias_mode %d not supported for a convolution", ep->bias_mode);
      e = *ep;
      e.ldr = d.K;
    }
    const long long kw = plan->split ? 2 * plan->kpad : plan->kpad;
    if (plan->stem_pack > 1) {
      // the packed contraction has stem_pack * K columns: its per-channel vectors are the caller's, repeated
      const int P = plan->stem_pack, K = (int)d.K;
      const bool per_channel_bias = e.bias && (e.bias_mode == SOFIE_B200_BIAS_COL_F32 || e.bias_mode == SOFIE_B200_BIAS_COL_I32);
      if (e.col_scale || per_channel_bias) {
        repeat_words_kernel<<<(unsigned)((P * K + 255) / 256), 256, 0, ctx->stream>>>((const uint32_t *)e.col_scale, per_channel_bias ? (const uint32_t *)e.bias : nullptr,
                                                                                   (uint32_t *)plan->stem_vec, K, P);
        SB_CUDA(cudaGetLastError());
        ctx->launches++;
        if (e.col_scale) e.col_scale = (const float *)plan->stem_vec;
        if (per_channel_bias) e.bias = (const uint32_t *)plan->stem_vec + P * K;
      }
      e.ldr = (long long)P * K;
      return sofie_b200_gemm_enqueue(plan->gemm, workspace, plan->w_padded, Y, &e);
    }
    for (int g = 0; g < d.groups; ++g) {
      sofie_b200_epilogue eg = e;
      if (eg.col_scale) eg.col_scale += g * plan->kg;
      if (eg.bias && eg.bias_mode != SOFIE_B200_BIAS_SCALAR_F32) eg.bias = (const char *)eg.bias + (size_t)g * plan->kg * 4;
      if (eg.residual) eg.residual = (const char *)eg.residual + (size_t)g * plan->kg * dtype_size(eg.residual_dtype);
      const char *a = (const char *)workspace + (size_t)g * d.N * pix * kw * es;
      const char *b = (const char *)plan->w_padded + (size_t)g * plan->kg * kw * es;
      char *y = (char *)Y + (size_t)g * plan->kg * ys;
      int rc = sofie_b200_gemm_enqueue(plan->gemm, a, b, y, &eg);
      if (rc) return rc;
    }
    return 0;
  }
  if (ep) {
    if (ep->row_scale) return fail(SOFIE_B200_ERR_INVALID, "conv_enqueue: row_scale has no meaning for a convolution");
    e = *ep;
    e.row_scale = ep->col_scale;
    e.col_scale = nullptr;
    switch (ep->bias_mode) {
      case SOFIE_B200_BIAS_NONE: case SOFIE_B200_BIAS_SCALAR_F32: break;
      case SOFIE_B200_BIAS_COL_F32: e.bias_mode = SOFIE_B200_BIAS_ROW_F32; break;
      case SOFIE_B200_BIAS_COL_I32: e.bias_mode = SOFIE_B200_BIAS_ROW_I32; break;
      default: return fail(SOFIE_B200_ERR_INVALID, "conv_enqueue: bias_mode %d not supported for a convolution", ep->bias_mode);
    }
    e.ldr = pix;
  }
  for (int g = 0; g < d.groups; ++g) {
    sofie_b200_epilogue eg = e;
    if (eg.row_scale) eg.row_scale += g * plan->kg;
    if (eg.bias && eg.bias_mode != SOFIE_B200_BIAS_SCALAR_F32) eg.bias = (const char *)eg.bias + (size_t)g * plan->kg * 4;
    if (eg.residual) eg.residual = (const char *)eg.residual + (size_t)g * plan->kg * pix * dtype_size(eg.residual_dtype);
    const long long kw = plan->split ? 2 * plan->kpad : plan->kpad;
    const char *a = (const char *)plan->w_padded + (size_t)g * plan->kg * kw * es;
    const char *b = (const char *)workspace + (size_t)g * d.N * pix * kw * es;
    char *y = (char *)Y + (size_t)g * plan->kg * pix * ys;
    int rc = sofie_b200_gemm_enqueue(plan->gemm, a, b, y, &eg);
    if (rc) return rc;
  }
  return 0;
}

}  // extern "C"

// -----------------------------------------------------------------------------------------------
// Convolution for callers that must not allocate
// -----------------------------------------------------------------------------------------------
// Some hosts of this library run their inference loop under a rule of "no device allocation after
// configuration": online event filters and other fixed-budget services partition GPU memory once,
// at start-up, and treat any later cudaMalloc as a fault, because it serialises the device, can
// fail from fragmentation hours into a run, and is not allowed from the callback contexts they
// call us from.  The regular path needs two device buffers per convolution (the padded weights
// owned by the plan, and the unfolded-input workspace the caller provides).  The entry point below
// needs neither: both live in one fixed array that is part of the library image.
//
// Cost and limits: every GPU on which the library is loaded carries the array (16 MiB) from load to
// exit, used or not.  A call whose padded weights plus unfolded input exceed it is refused.  All
// calls on a device share the array, so two calls that can overlap on the GPU (different streams,
// different contexts) race on it; calls on one stream are ordered and safe.  The array keeps the
// previous call's bytes: nothing in it is assumed to be zero, each call writes every byte it later
// reads (padding columns included).
namespace sb200 {

constexpr size_t kConvStaticScratchBytes = size_t(16) << 20;
static __device__ __align__(256) unsigned char g_conv_static_scratch[kConvStaticScratchBytes];

// In host code `g_conv_static_scratch` is only a handle for the symbol, not a device address.  The
// address is looked up once per device, with that device current, and cached.
constexpr int kMaxDevices = 64;
static void *g_conv_static_ptr[kMaxDevices] = {};
static std::mutex g_conv_static_mutex;

static int conv_static_scratch(int device, unsigned char **out) {
  if (device < 0 || device >= kMaxDevices) return fail(SOFIE_B200_ERR_INVALID, "conv_enqueue_noalloc: device index %d out of range", device);
  std::lock_guard<std::mutex> lock(g_conv_static_mutex);
  if (!g_conv_static_ptr[device]) {
    void *p = nullptr;
    cudaError_t e = cudaGetSymbolAddress(&p, g_conv_static_scratch);
    if (e != cudaSuccess || !p)
      return fail(SOFIE_B200_ERR_CUDA, "conv_enqueue_noalloc: cudaGetSymbolAddress failed on device %d: %s", device, cudaGetErrorString(e));
    g_conv_static_ptr[device] = p;
  }
  *out = static_cast<unsigned char *>(g_conv_static_ptr[device]);
  return 0;
}

}  // namespace sb200

extern "C" int sofie_b200_conv_enqueue_noalloc(sofie_b200_ctx *ctx, const sofie_b200_conv_desc *desc, const void *X,
                                               const void *W, void *Y, const sofie_b200_epilogue *ep) {
  if (!ctx || !desc) return fail(SOFIE_B200_ERR_INVALID, "conv_enqueue_noalloc: NULL argument");
  if (desc->x_layout != 0 || desc->y_layout != 0) return fail(SOFIE_B200_ERR_INVALID, "conv_enqueue_noalloc: only the NCHW layouts are supported");
  sofie_b200_conv_desc d = *desc;
  if (d.groups < 1) d.groups = 1;
  if (d.N < 0 || d.C < 1 || d.H < 1 || d.W < 1 || d.K < 1 || d.R < 1 || d.S < 1)
    return fail(SOFIE_B200_ERR_INVALID, "conv_enqueue_noalloc: bad extent");
  if (d.C % d.groups || d.K % d.groups)
    return fail(SOFIE_B200_ERR_INVALID, "conv_enqueue_noalloc: channels %lld / filters %lld not divisible by groups %d", (long long)d.C, (long long)d.K, d.groups);
  if (d.x_dtype != SOFIE_B200_F32 && d.x_dtype != SOFIE_B200_I8)
    return fail(SOFIE_B200_ERR_INVALID, "conv_enqueue_noalloc: input type %d not supported (F32, I8)", d.x_dtype);
  int64_t Ho, Wo;
  int rc = conv_out_shape(d, &Ho, &Wo);
  if (rc) return rc;
  if (d.N == 0) return 0;
  if (!X || !W || !Y) return fail(SOFIE_B200_ERR_INVALID, "conv_enqueue_noalloc: NULL tensor");

  const int es = dtype_size(d.x_dtype);
  const int64_t cg = d.C / d.groups, kg = d.K / d.groups, pix = Ho * Wo;
  const int64_t kdim = cg * d.R * d.S, vec = 16 / es;
  const int64_t kpad = (kdim + vec - 1) / vec * vec;
  const size_t w_bytes = (size_t)((d.K * kpad * es + 255) / 256 * 256);
  const size_t x_bytes = (size_t)((int64_t)d.groups * d.N * pix * kpad * es);
  if (w_bytes + x_bytes > kConvStaticScratchBytes)
    return fail(SOFIE_B200_ERR_TOO_LARGE,
                "conv_enqueue_noalloc: this convolution needs %zu bytes of scratch (padded weights %zu + unfolded input %zu); "
                "the static scratch holds %zu bytes -- use the plan-based entry points with a caller workspace",
                w_bytes + x_bytes, w_bytes, x_bytes, kConvStaticScratchBytes);

  // Every argument check comes before the first launch: a refused call enqueues nothing and leaves the shared array alone.
  switch (d.y_dtype) {
    case SOFIE_B200_F32: case SOFIE_B200_BF16: case SOFIE_B200_I8: case SOFIE_B200_U8: break;
    case SOFIE_B200_I32:
      if (d.x_dtype != SOFIE_B200_I8) return fail(SOFIE_B200_ERR_INVALID, "conv_enqueue_noalloc: I32 output needs I8 input");
      break;
    default: return fail(SOFIE_B200_ERR_INVALID, "conv_enqueue_noalloc: output type %d not supported", d.y_dtype);
  }
  sofie_b200_epilogue e{};
  e.alpha = 1.f; e.beta = 1.f; e.out_scale = 1.f;
  if (ep) {
    if (ep->row_scale) return fail(SOFIE_B200_ERR_INVALID, "conv_enqueue_noalloc: row_scale has no meaning for a convolution");
    e = *ep;
    e.row_scale = ep->col_scale;  // output channels are accumulator rows, as in sofie_b200_conv_enqueue
    e.col_scale = nullptr;
    switch (ep->bias_mode) {
      case SOFIE_B200_BIAS_NONE: case SOFIE_B200_BIAS_SCALAR_F32: break;
      case SOFIE_B200_BIAS_COL_F32: e.bias_mode = SOFIE_B200_BIAS_ROW_F32; break;
      case SOFIE_B200_BIAS_COL_I32: e.bias_mode = SOFIE_B200_BIAS_ROW_I32; break;
      default: return fail(SOFIE_B200_ERR_INVALID, "conv_enqueue_noalloc: bias_mode %d not supported for a convolution", ep->bias_mode);
    }
    e.ldr = pix;
  }

  SB_CUDA(cudaSetDevice(ctx->device));
  unsigned char *scratch = nullptr;
  if ((rc = conv_static_scratch(ctx->device, &scratch))) return rc;
  unsigned char *w_padded = scratch, *xcol = scratch + w_bytes;

  // the contraction, planned on the stack (no heap, no device memory); planning can still refuse, so it also precedes the launches
  sofie_b200_gemm_plan gp;
  gp.ctx = ctx;
  sofie_b200_gemm_desc &g = gp.desc;
  g.M = kg; g.N = pix; g.K = kpad; g.batch = d.N;
  g.trans_a = 0; g.trans_b = 1;
  g.ab_dtype = d.x_dtype; g.y_dtype = d.y_dtype;
  g.lda = kpad; g.ldb = kpad; g.ldy = pix;
  g.stride_a = 0; g.stride_b = pix * kpad; g.stride_y = d.K * pix;
  g.stride_c = 0; g.stride_r = d.K * pix;
  g.precise = d.precise;
  if (!(d.x_dtype == SOFIE_B200_F32 && d.precise != 0)) {
    rc = umma_plan_init(&gp);
    if (rc < 0) return rc;
    gp.use_umma = (rc == 0);
  }
  {
    EpiParams probe;   // the per-group epilogues below differ from this one only by pointer offsets
    if ((rc = gemm_make_epi(g, Y, &e, &probe))) return rc;
  }

  // 1. weights to a 16-byte row pitch, 2. unfold the whole batch; both rewrite every byte the contraction reads
  const long long wtotal = d.K * kpad;
  const unsigned wgrid = (unsigned)std::min<long long>((wtotal + 255) / 256, (long long)ctx->sm_count * 16);
  const long long xtotal = (long long)d.groups * d.N * pix * (kpad / vec);
  const unsigned xgrid = (unsigned)std::min<long long>((xtotal + 255) / 256, (long long)ctx->sm_count * 32);
  if (d.x_dtype == SOFIE_B200_F32) {
    pad_weights_kernel<float><<<wgrid, 256, 0, ctx->stream>>>((const float *)W, (float *)w_padded, d.K, kdim, kpad);
    unfold_kernel<float, 4><<<xgrid, 256, 0, ctx->stream>>>((const float *)X, (float *)xcol, d, Ho, Wo, cg, kdim, kpad, 0.f);
  } else {
    pad_weights_kernel<int8_t><<<wgrid, 256, 0, ctx->stream>>>((const int8_t *)W, (int8_t *)w_padded, d.K, kdim, kpad);
    unfold_kernel<int8_t, 16><<<xgrid, 256, 0, ctx->stream>>>((const int8_t *)X, (int8_t *)xcol, d, Ho, Wo, cg, kdim, kpad, (int8_t)d.x_zero_point);
  }
  SB_CUDA(cudaGetLastError());
  ctx->launches += 2;

  // 3. the contraction
  const int ys = dtype_size(d.y_dtype);
  for (int grp = 0; grp < d.groups; ++grp) {
    sofie_b200_epilogue eg = e;
    if (eg.row_scale) eg.row_scale += grp * kg;
    if (eg.bias && eg.bias_mode != SOFIE_B200_BIAS_SCALAR_F32) eg.bias = (const char *)eg.bias + (size_t)grp * kg * 4;
    if (eg.residual) eg.residual = (const char *)eg.residual + (size_t)grp * kg * pix * dtype_size(eg.residual_dtype);
    const unsigned char *a = w_padded + (size_t)grp * kg * kpad * es;
    const unsigned char *b = xcol + (size_t)grp * d.N * pix * kpad * es;
    char *y = (char *)Y + (size_t)grp * kg * pix * ys;
    rc = sofie_b200_gemm_enqueue(&gp, a, b, y, &eg);
    if (rc) return rc;
  }
  return 0;
}
