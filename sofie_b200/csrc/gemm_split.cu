// fp32 contractions on the tensor cores at fp32 accuracy: error-compensated 3xTF32.
//
// A TF32 multiply keeps 11 significand bits of each operand, far from the 1e-5 bar the fp32 models
// are held to.  Each operand is therefore split as x = hi + lo with hi = x rounded to the nearest TF32
// value (low 13 bits clear, so the tensor core reads it exactly) and lo = x - hi, itself rounded to TF32
// (|lo| <= 2^-12 |x|, so what is dropped is below 2^-23 |x| and unbiased), and the product is formed
// as  A_hi*B_hi + A_lo*B_hi + A_hi*B_lo  (the A_lo*B_lo term is below 2^-24 relative).  The
// three partial products are one contraction over K' = 3*Ks (Ks = K rounded up to a K block of 32, zero filled) whose
// segments read   A: hi, lo, hi   and   B: hi, hi, lo.   Each operand is STORED once as [ hi | lo ] (2*Ks per row); the
// producer of the TF32 kernel (gemm_umma3x.cu, which sums short K chunks in registers) looks the K coordinate of each
// segment up per operand.  The split kernels also bring every operand to K-major order, whatever the transposition flags.
#include "gemm.cuh"

namespace sb200 {

// dst [rows, 2*Ks] K-major, hi | lo; element (r, k) comes from src[k*ld + r] when `mn` (source stored [K, rows]) else src[r*ld + k].
__global__ void __launch_bounds__(256) split2_kernel(const float *__restrict__ src, float *__restrict__ dst, long long rows, long long K,
                                                     long long Ks, long long ld, long long batch_stride, int mn) {
  const long long per_batch = rows * Ks;
  const long long b = blockIdx.y;
  const float *s = src + b * batch_stride;
  float *d = dst + b * rows * 2 * Ks;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < per_batch; i += (long long)gridDim.x * blockDim.x) {
    // when the source is MN-major walk rows fastest so that reads coalesce; else k fastest (reads and writes coalesce)
    long long r, k;
    if (mn) { r = i % rows; k = i / rows; } else { k = i % Ks; r = i / Ks; }
    float x = 0.f;
    if (k < K) x = mn ? s[k * ld + r] : s[r * ld + k];
    const float hi = tf32_rn(x);
    const float lo = tf32_rn(__fsub_rn(x, hi));
    float *o = d + r * 2 * Ks + k;
    o[0] = hi;
    o[Ks] = lo;
  }
}

int split2_enqueue(sofie_b200_ctx *ctx, const float *src, float *dst, long long rows, long long K, long long Ks, long long ld,
                   long long batch, long long batch_stride, int mn) {
  const long long per_batch = rows * Ks;
  long long blocks = (per_batch + 255) / 256;
  const long long cap = (long long)ctx->sm_count * 16;
  if (blocks > cap) blocks = cap;
  if (blocks < 1) blocks = 1;
  dim3 grid((unsigned)blocks, (unsigned)batch);
  split2_kernel<<<grid, 256, 0, ctx->stream>>>(src, dst, rows, K, Ks, ld, batch_stride, mn);
  SB_CUDA(cudaGetLastError());
  ctx->launches++;
  return 0;
}

}  // namespace sb200
