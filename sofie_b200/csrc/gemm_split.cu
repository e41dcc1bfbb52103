// fp32 contractions on the tensor cores at fp32 accuracy: error-compensated 3xTF32.
//
// A TF32 multiply keeps 11 significand bits of each operand, far from the 1e-5 bar the fp32 models
// are held to.  Each operand is therefore split as x = hi + lo with hi = x rounded to the nearest TF32
// value (low 13 bits clear, so the tensor core reads it exactly) and lo = x - hi, itself rounded to TF32
// (|lo| <= 2^-12 |x|, so what is dropped is below 2^-23 |x| and unbiased), and the product is formed
// as  A_hi*B_hi + A_lo*B_hi + A_hi*B_lo  (the A_lo*B_lo term is below 2^-24 relative).  The
// three partial products are one contraction over K' = 3*Ks with the operands laid out as
//     A' = [ A_hi | A_lo | A_hi ]     B' = [ B_hi | B_hi | B_lo ]        (Ks = K rounded up to 4, zero filled)
// so one TF32 tcgen05 contraction (gemm_umma3x.cu, which sums short K chunks in registers) does the work.  The split
// kernels also bring every operand to K-major order, whatever the transposition flags.
#include "gemm.cuh"

namespace sb200 {

// dst [rows, 3*Ks] K-major; element (r, k) comes from src[k*ld + r] when `mn` (source stored [K, rows]) else src[r*ld + k].
// pattern 0: hi | lo | hi (A side), 1: hi | hi | lo (B side)
__global__ void __launch_bounds__(256) split3_kernel(const float *__restrict__ src, float *__restrict__ dst, long long rows, long long K,
                                                     long long Ks, long long ld, long long batch_stride, int mn, int pattern) {
  const long long per_batch = rows * Ks;
  const long long b = blockIdx.y;
  const float *s = src + b * batch_stride;
  float *d = dst + b * rows * 3 * Ks;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < per_batch; i += (long long)gridDim.x * blockDim.x) {
    // when the source is MN-major walk rows fastest so that reads coalesce; else k fastest (reads and writes coalesce)
    long long r, k;
    if (mn) { r = i % rows; k = i / rows; } else { k = i % Ks; r = i / Ks; }
    float x = 0.f;
    if (k < K) x = mn ? s[k * ld + r] : s[r * ld + k];
    const float hi = tf32_rn(x);
    const float lo = tf32_rn(__fsub_rn(x, hi));
    float *o = d + r * 3 * Ks + k;
    o[0] = hi;
    o[Ks] = pattern == 0 ? lo : hi;
    o[2 * Ks] = pattern == 0 ? hi : lo;
  }
}

int split3_enqueue(sofie_b200_ctx *ctx, const float *src, float *dst, long long rows, long long K, long long Ks, long long ld,
                   long long batch, long long batch_stride, int mn, int pattern) {
  const long long per_batch = rows * Ks;
  long long blocks = (per_batch + 255) / 256;
  const long long cap = (long long)ctx->sm_count * 16;
  if (blocks > cap) blocks = cap;
  if (blocks < 1) blocks = 1;
  dim3 grid((unsigned)blocks, (unsigned)batch);
  split3_kernel<<<grid, 256, 0, ctx->stream>>>(src, dst, rows, K, Ks, ld, batch_stride, mn, pattern);
  SB_CUDA(cudaGetLastError());
  ctx->launches++;
  return 0;
}

}  // namespace sb200
