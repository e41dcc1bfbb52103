// General-shape contraction on the CUDA cores.  It covers what the tcgen05 path cannot take:
// operands whose pitches or base addresses are not 16-byte multiples (TMA's rule), and fp32
// products that must stay within 1e-5 of an fp32 BLAS (plain fp32 FMA, no TF32 rounding).
// 64x64 output tile per CTA, 256 threads, 4x4 outputs per thread, K stepped by 16 through
// shared memory with the next step's operands prefetched into registers.  The epilogue is the shared one (epilogue.cuh).
#include "gemm.cuh"

namespace sb200 {

template <typename T> struct SimtIn;
template <> struct SimtIn<float> { using acc_t = float; static __device__ __forceinline__ float cvt(float v) { return v; } };
template <> struct SimtIn<__nv_bfloat16> { using acc_t = float; static __device__ __forceinline__ float cvt(__nv_bfloat16 v) { return __bfloat162float(v); } };
template <> struct SimtIn<int8_t> { using acc_t = int; static __device__ __forceinline__ int cvt(int8_t v) { return (int)v; } };
template <> struct SimtIn<__nv_fp8_e4m3> { using acc_t = float; static __device__ __forceinline__ float cvt(__nv_fp8_e4m3 v) { return (float)v; } };

constexpr int ST = 64, SK = 16;

template <typename T>
__global__ void __launch_bounds__(256) simt_gemm_kernel(const SimtParams p) {
  using acc_t = typename SimtIn<T>::acc_t;
  __shared__ acc_t sA[SK][ST + 1];
  __shared__ acc_t sB[SK][ST + 1];
  const int b = blockIdx.z;
  const long long m0 = (long long)blockIdx.y * ST, n0 = (long long)blockIdx.x * ST;
  const T *A = (const T *)p.A + (long long)b * p.stride_a;
  const T *B = (const T *)p.B + (long long)b * p.stride_b;
  const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
  acc_t acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = 0;

  // The global loads of K step k0 + SK are issued before the products of step k0 and land in registers meanwhile
  // (four elements of each operand per thread and step).
  constexpr int PER = ST * SK / 256;
  acc_t ra[PER], rb[PER];
  auto fetch = [&](long long k0) {
#pragma unroll
    for (int q = 0; q < PER; ++q) {
      const int e = threadIdx.x + q * 256;
      int kk, mm;
      if (p.trans_a) { mm = e % ST; kk = e / ST; } else { kk = e % SK; mm = e / SK; }
      const long long m = m0 + mm, k = k0 + kk;
      ra[q] = (m < p.M && k < p.K) ? SimtIn<T>::cvt(p.trans_a ? A[k * p.lda + m] : A[m * p.lda + k]) : (acc_t)0;
      int nn;
      if (p.trans_b) { kk = e % SK; nn = e / SK; } else { nn = e % ST; kk = e / ST; }
      const long long n = n0 + nn, kb = k0 + kk;
      rb[q] = (n < p.N && kb < p.K) ? SimtIn<T>::cvt(p.trans_b ? B[n * p.ldb + kb] : B[kb * p.ldb + n]) : (acc_t)0;
    }
  };
  fetch(0);
  for (long long k0 = 0; k0 < p.K; k0 += SK) {
#pragma unroll
    for (int q = 0; q < PER; ++q) {
      const int e = threadIdx.x + q * 256;
      int kk, mm, nn;
      if (p.trans_a) { mm = e % ST; kk = e / ST; } else { kk = e % SK; mm = e / SK; }
      sA[kk][mm] = ra[q];
      if (p.trans_b) { kk = e % SK; nn = e / SK; } else { nn = e % ST; kk = e / ST; }
      sB[kk][nn] = rb[q];
    }
    if (k0 + SK < p.K) fetch(k0 + SK);
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < SK; ++kk) {
      acc_t a[4], bb[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) a[i] = sA[kk][ty * 4 + i];
#pragma unroll
      for (int j = 0; j < 4; ++j) bb[j] = sB[kk][tx + 16 * j];
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          if constexpr (sizeof(acc_t) == 4 && !std::is_same<acc_t, int>::value) acc[i][j] = fmaf(a[i], bb[j], acc[i][j]);
          else acc[i][j] += a[i] * bb[j];
        }
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    long long m = m0 + ty * 4 + i;
    if (m >= p.M) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      long long n = n0 + tx + 16 * j;
      if (n >= p.N) continue;
      uint32_t raw;
      if constexpr (std::is_same<acc_t, int>::value) raw = (uint32_t)acc[i][j];
      else raw = __float_as_uint(acc[i][j]);
      epi_store_one(p.ep, raw, b, m, n);
    }
  }
}

int simt_enqueue(sofie_b200_gemm_plan *plan, const void *A, const void *B, const EpiParams &ep) {
  const sofie_b200_gemm_desc &d = plan->desc;
  SimtParams p;
  p.A = A; p.B = B;
  p.M = (int)d.M; p.N = (int)d.N; p.K = (int)d.K; p.batch = (int)d.batch;
  p.lda = d.lda; p.ldb = d.ldb; p.stride_a = d.stride_a; p.stride_b = d.stride_b;
  p.trans_a = d.trans_a; p.trans_b = d.trans_b;
  p.ep = ep;
  dim3 grid((unsigned)((d.N + ST - 1) / ST), (unsigned)((d.M + ST - 1) / ST), (unsigned)d.batch);
  if (grid.y > 65535 || grid.z > 65535) return fail(SOFIE_B200_ERR_TOO_LARGE, "simt gemm: grid too large");
  cudaStream_t st = plan->ctx->stream;
  switch (d.ab_dtype) {
    case SOFIE_B200_F32: simt_gemm_kernel<float><<<grid, 256, 0, st>>>(p); break;
    case SOFIE_B200_BF16: simt_gemm_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>(p); break;
    case SOFIE_B200_I8: simt_gemm_kernel<int8_t><<<grid, 256, 0, st>>>(p); break;
    case SOFIE_B200_F8E4M3: simt_gemm_kernel<__nv_fp8_e4m3><<<grid, 256, 0, st>>>(p); break;
    default: return fail(SOFIE_B200_ERR_INVALID, "simt gemm: unsupported operand type %d", d.ab_dtype);
  }
  SB_CUDA(cudaGetLastError());
  plan->ctx->launches++;
  return 0;
}

}  // namespace sb200
