// Self-test of the bounded-wait protocol of the contraction kernels: a wait that nothing ever satisfies must end by
// itself, report through the context's status word and leave the context usable.
#include "gemm.cuh"
#include "ptx.cuh"
#include "umma_store.cuh"

namespace sb200 {

// One thread waits on an mbarrier phase that no one arrives on, with the kernels' own mbar_wait() and a short limit,
// then takes the kernels' own abort path (raise_abort) and returns normally.
__global__ void wait_timeout_kernel(int *status, unsigned long long limit_ns) {
  __shared__ uint64_t bar;
  __shared__ int abort_flag;
  if (threadIdx.x == 0) {
    abort_flag = 0;
    ptx::mbar_init(ptx::smem_u32(&bar), 1);
    ptx::fence_barrier_init();
    if (!ptx::mbar_wait(ptx::smem_u32(&bar), 0, &abort_flag, limit_ns)) raise_abort(&abort_flag, status, DEV_WAIT_SMEM_FULL);
  }
}

}  // namespace sb200

extern "C" int sofie_b200_selftest_wait_timeout(sofie_b200_ctx *ctx, int64_t limit_us) {
  using namespace sb200;
  if (!ctx) return fail(SOFIE_B200_ERR_INVALID, "selftest_wait_timeout: ctx is NULL");
  if (limit_us < 1 || limit_us > 100000) return fail(SOFIE_B200_ERR_INVALID, "selftest_wait_timeout: limit must be 1 .. 100000 microseconds");
  SB_CUDA(cudaSetDevice(ctx->device));
  wait_timeout_kernel<<<1, 32, 0, ctx->stream>>>(ctx->d_status, (unsigned long long)limit_us * 1000ull);
  SB_CUDA(cudaGetLastError());
  ctx->launches++;
  return 0;
}
