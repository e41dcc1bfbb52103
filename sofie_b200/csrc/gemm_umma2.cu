// CTA-pair variant of the tcgen05 contraction kernel: a thread-block cluster of two CTAs on two SMs
// computes one 256 x bn tile with tcgen05.mma.cta_group::2.
//
// Why: with one CTA per 128 x 256 tile every SM pulls 48 KB of operands per 128-byte K step, and the
// shared-memory ring (4 stages) covers only about one microsecond of tensor-pipe work -- less than the
// L2 latency under load, so the pipe idles.  In a pair each CTA stages its own 128 rows of A and only
// HALF of the B slice (bn/2 columns); the MMA unit reads A and B from both CTAs' shared memory.  Per SM
// that is 32 KB per K step: 7 stages, 1.75x the lookahead, and a third less L2 traffic.
//
// Protocol (rank 0 = leader; both CTAs use identical shared-memory offsets)
//   full[s]    lives in the leader.  The leader's producer arrives with expect_tx for the bytes of BOTH
//              CTAs; each CTA's TMA loads (cta_group::2 form, never multicast) count on that barrier.
//   empty[s]   one per CTA.  The leader's MMA thread commits twice, to its own and to the peer's barrier,
//              so each producer waits only on local memory.
//   tfull[a]   one per CTA, committed twice by the leader the same way.
//   tempty[a]  lives in the leader; the four epilogue warps of each CTA arrive (remotely from the peer).
// The accumulator of rows [128 r, 128 r + 128) sits in the tensor memory of CTA r, so each CTA runs the
// epilogue of its own rows.  Every wait is bounded; the cluster barrier at the end keeps either CTA's
// shared and tensor memory alive until the other is done with it.
#include <cudaTypedefs.h>

#include "gemm.cuh"
#include "ptx.cuh"
#include "umma_store.cuh"

namespace sb200 {
using namespace ptx;

template <int KIND>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(UMMA_PAIR_THREADS, 1)
umma_pair_gemm_kernel(const __grid_constant__ CUtensorMap tm_a, const __grid_constant__ CUtensorMap tm_b,
                      const __grid_constant__ UmmaParams p) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw_addr = smem_u32(smem_raw);
  const uint32_t pad = (1024u - (raw_addr & 1023u)) & 1023u;
  uint8_t *smem = smem_raw + pad;

  const int stages = p.stages;
  const uint32_t smem_a = smem_u32(smem);
  const uint32_t smem_b = smem_a + stages * p.a_stage_bytes;
  uint8_t *tail = smem + stages * (p.a_stage_bytes + p.b_stage_bytes);
  const uint32_t bar_full = smem_u32(tail);
  const uint32_t bar_empty = bar_full + 8 * stages;
  const uint32_t bar_tfull = bar_empty + 8 * stages;
  const uint32_t bar_tempty = bar_tfull + 16;
  uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(tail + 16 * stages + 32);
  volatile int *abort_flag = reinterpret_cast<volatile int *>(tmem_slot + 1);
  const uint32_t epi_stage = smem_u32(tail) + UMMA_TAIL_BYTES;   // 4 KB per epilogue warp (coalesced_store)

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();
  const bool leader = rank == 0;
  const uint32_t peer = rank ^ 1u;

  if (threadIdx.x == 0) {
    for (int s = 0; s < stages; ++s) {
      mbar_init(bar_full + 8 * s, 1);
      mbar_init(bar_empty + 8 * s, 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(bar_tfull + 8 * i, 1);
      mbar_init(bar_tempty + 8 * i, 8);  // four epilogue warps of each CTA
    }
    *abort_flag = 0;
    fence_barrier_init();
    prefetch_tensormap(&tm_a);
    prefetch_tensormap(&tm_b);
  }
  if (warp == 1) {
    tmem_alloc_pair(smem_u32(tmem_slot), p.tmem_cols);
    tmem_relinquish_pair();
  }
  tc_fence_before();
  __syncthreads();
  // both CTAs' barriers must exist before either signals the other's
  cluster_arrive();
  cluster_wait();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  const long long tiles_per_batch = (long long)p.tiles_m * p.tiles_n;
  const long long first = blockIdx.x >> 1, step = gridDim.x >> 1;

  if (warp == 0) {
    // ------------------------------ TMA producer (one per CTA) -------------------------
    if (lane == 0) {
      uint32_t stage = 0, phase = 0;
      bool ok = true;
      ROLE_TIMER(w_empty);
      ROLE_TIMER(t_begin);
#ifdef SB200_ROLE_TIMERS
      t_begin = clock64();
#endif
      const uint32_t full_leader = mapa(bar_full, 0);
      const uint32_t group = p.commit_group;
      uint32_t gpos = 0;
      for (long long t = first; t < p.num_tiles && ok; t += step) {
        const int b = (int)(t / tiles_per_batch);
        const int r = (int)(t % tiles_per_batch);
        const int m0 = (r % p.tiles_m) * (2 * UMMA_BM) + (int)rank * UMMA_BM;
        const int n0 = (r / p.tiles_m) * p.bn + (int)rank * p.b_rows;
        const int ba = p.a_bcast ? 0 : b, bb = p.b_bcast ? 0 : b;
        for (int kb = 0; kb < p.num_kb; ++kb) {
          // the empty barrier of a release group is that of its first stage (see the MMA issuer)
          if (gpos == 0 && !ROLE_WAIT(w_empty, mbar_wait(bar_empty + 8 * stage, phase ^ 1u, abort_flag))) {
            raise_abort(abort_flag, p.status, DEV_WAIT_SMEM_EMPTY);
            ok = false;
            break;
          }
          if (++gpos == group) gpos = 0;
          const uint32_t full = full_leader + 8 * stage;
          if (leader) mbar_arrive_expect_tx(bar_full + 8 * stage, 2u * (p.a_stage_bytes + p.b_stage_bytes));
          const int k0 = kb * p.kb_elems;
          const uint32_t sa = smem_a + stage * p.a_stage_bytes;
          const uint32_t sb = smem_b + stage * p.b_stage_bytes;
          if (!p.a_mn) {
            tma_load_3d_pair(sa, &tm_a, full, k0, m0, ba);
          } else {
            for (int x = 0; x < p.a_boxes; ++x) tma_load_3d_pair(sa + x * p.a_box_bytes, &tm_a, full, m0 + x * p.a_box_mn, k0, ba);
          }
          if (!p.b_mn) {
            tma_load_3d_pair(sb, &tm_b, full, k0, n0, bb);
          } else {
            for (int x = 0; x < p.b_boxes; ++x) tma_load_3d_pair(sb + x * p.b_box_bytes, &tm_b, full, n0 + x * p.b_box_mn, k0, bb);
          }
          if (++stage == (uint32_t)stages) { stage = 0; phase ^= 1u; }
        }
      }
      ROLE_REPORT("[cta %d] producer: total %lld, waiting for a free stage %lld\n", blockIdx.x, clock64() - t_begin, w_empty);
      if (!ok) {
        const uint64_t t0 = globaltimer();
        while (globaltimer() - t0 < 200000ull) {}
      }
    }
  } else if (warp == 1) {
    // ------------------------------ MMA issuer (leader CTA only) ------------------------
    if (lane == 0 && leader) {
      uint32_t stage = 0, phase = 0;
      uint32_t acc = 0, acc_phase = 0;
      bool ok = true;
      ROLE_TIMER(w_full);
      ROLE_TIMER(w_tempty);
      ROLE_TIMER(c_fence);
      ROLE_TIMER(c_mma);
      ROLE_TIMER(c_commit);
      ROLE_TIMER(sec_t0);
      ROLE_TIMER(t_begin);
#ifdef SB200_ROLE_TIMERS
      t_begin = clock64();
#endif
      const uint32_t empty_peer = mapa(bar_empty, peer), tfull_peer = mapa(bar_tfull, peer);
      uint32_t gpos = 0;   // position of the current stage inside its release group
      // descriptor words that do not change inside the loop, kept in registers
      const uint64_t a_hi = (uint64_t)p.a_desc_hi << 32, b_hi = (uint64_t)p.b_desc_hi << 32;
      const uint32_t a_lo0 = p.a_desc_lo | ((smem_a >> 4) & 0x3fffu), b_lo0 = p.b_desc_lo | ((smem_b >> 4) & 0x3fffu);
      const uint32_t a_step = p.a_stage_bytes >> 4, b_step = p.b_stage_bytes >> 4;
      const uint32_t a_kadv = p.a_kadv, b_kadv = p.b_kadv, idesc = p.idesc;
      const int num_kb = p.num_kb;
      const uint32_t group = p.commit_group;
      for (long long t = first; t < p.num_tiles && ok; t += step) {
        if (!ROLE_WAIT(w_tempty, mbar_wait(bar_tempty + 8 * acc, acc_phase ^ 1u, abort_flag))) {
          raise_abort(abort_flag, p.status, DEV_WAIT_TMEM_EMPTY);
          break;
        }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * p.bn;
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!ROLE_WAIT(w_full, mbar_wait(bar_full + 8 * stage, phase, abort_flag))) {
            raise_abort(abort_flag, p.status, DEV_WAIT_SMEM_FULL);
            ok = false;
            break;
          }
          ROLE_SECTION_BEGIN();
          tc_fence_after();
          ROLE_SECTION_END(c_fence);
          const uint32_t a_lo = a_lo0 + stage * a_step;
          const uint32_t b_lo = b_lo0 + stage * b_step;
          ROLE_SECTION_BEGIN();
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            const uint64_t ad = a_hi | (uint64_t)(a_lo + k * a_kadv);
            const uint64_t bd = b_hi | (uint64_t)(b_lo + k * b_kadv);
            umma_pair<KIND>(d_tmem, ad, bd, idesc, (kb | k) != 0 ? 1u : 0u);
          }
          ROLE_SECTION_END(c_mma);
          ROLE_SECTION_BEGIN();
          // Stages are released in groups of `commit_group` consecutive stages that share the empty barrier of the
          // group's first stage: a commit of a CTA pair is expensive for the tensor pipes of both SMs.
          if (++gpos == group) {
            const uint32_t first = bar_empty + 8 * (stage + 1 - group);
            tc_commit_pair(first);                              // this CTA's producer may refill the group
            tc_commit_pair(first + (empty_peer - bar_empty));    // and so may the peer's
            gpos = 0;
          }
          ROLE_SECTION_END(c_commit);
          if (++stage == (uint32_t)stages) { stage = 0; phase ^= 1u; }
        }
        if (!ok) break;
        tc_commit_pair(bar_tfull + 8 * acc);
        tc_commit_pair(tfull_peer + 8 * acc);
        if (++acc == 2) { acc = 0; acc_phase ^= 1u; }
      }
      ROLE_REPORT("[cta %d] mma issuer: total %lld, waiting for operands %lld, for a drained accumulator %lld\n", blockIdx.x,
                  clock64() - t_begin, w_full, w_tempty);
      ROLE_REPORT("[cta %d] mma issuer sections: fence %lld, issuing MMAs %lld, commits %lld\n", blockIdx.x, c_fence, c_mma, c_commit);
    }
  } else {
    // ------------------------------ epilogue (each CTA: its own 128 rows) ------------------
    const int quad = warp & 3;
    uint32_t acc = 0, acc_phase = 0;
    const uint32_t tempty_leader = mapa(bar_tempty, 0);
    ROLE_TIMER(w_tfull);
    ROLE_TIMER(t_begin);
#ifdef SB200_ROLE_TIMERS
    t_begin = clock64();
#endif
    for (long long t = first; t < p.num_tiles; t += step) {
      const int b = (int)(t / tiles_per_batch);
      const int r = (int)(t % tiles_per_batch);
      const int m0 = (r % p.tiles_m) * (2 * UMMA_BM) + (int)rank * UMMA_BM;
      const int n0 = (r / p.tiles_m) * p.bn;
      if (!ROLE_WAIT(w_tfull, mbar_wait(bar_tfull + 8 * acc, acc_phase, abort_flag))) {
        raise_abort(abort_flag, p.status, DEV_WAIT_TMEM_FULL);
        break;
      }
      tc_fence_after();
      const int row = m0 + quad * 32 + lane;
      const uint32_t taddr = tmem_base + ((uint32_t)(quad * 32) << 16) + acc * p.bn;
      drain_accumulator<KIND == KIND_I8>(p.ep, taddr, min(p.bn, p.N - n0), 0, 1, b, row, n0, p.vec_ok != 0, epi_stage + (uint32_t)(warp - 2) * 4096u, p.M);
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(tempty_leader + 8 * acc);
      if (++acc == 2) { acc = 0; acc_phase ^= 1u; }
    }
    if (threadIdx.x == 64) { ROLE_REPORT("[cta %d] epilogue: total %lld, waiting for an accumulator %lld\n", blockIdx.x, clock64() - t_begin, w_tfull); }
  }

  tc_fence_before();
  __syncthreads();
  // neither CTA may leave while the other can still signal its barriers or write its tensor memory
  cluster_arrive();
  cluster_wait();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc_pair(tmem_base, p.tmem_cols);
  }
}

int umma_pair_set_smem(int kind, size_t smem_bytes) {
  cudaError_t e = cudaSuccess;
  switch (kind) {
    case KIND_I8: e = cudaFuncSetAttribute(umma_pair_gemm_kernel<KIND_I8>, cudaFuncAttributeMaxDynamicSharedMemorySize, UMMA_MAX_DYN_SMEM); break;
    case KIND_F8: e = cudaFuncSetAttribute(umma_pair_gemm_kernel<KIND_F8>, cudaFuncAttributeMaxDynamicSharedMemorySize, UMMA_MAX_DYN_SMEM); break;
    case KIND_F16: e = cudaFuncSetAttribute(umma_pair_gemm_kernel<KIND_F16>, cudaFuncAttributeMaxDynamicSharedMemorySize, UMMA_MAX_DYN_SMEM); break;
    default: e = cudaFuncSetAttribute(umma_pair_gemm_kernel<KIND_TF32>, cudaFuncAttributeMaxDynamicSharedMemorySize, UMMA_MAX_DYN_SMEM); break;
  }
  if (e != cudaSuccess) return fail(SOFIE_B200_ERR_CUDA, "cudaFuncSetAttribute(pair kernel, smem=%zu): %s", smem_bytes, cudaGetErrorString(e));
  return 0;
}

// How many CTA pairs the device can hold at once with this much shared memory: the persistent tile
// schedule needs every pair of the grid resident from the start.
int umma_pair_max_clusters(int kind, size_t smem_bytes, int *out) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(2, 1, 1);
  cfg.blockDim = dim3(UMMA_PAIR_THREADS, 1, 1);
  cfg.dynamicSmemBytes = smem_bytes;
  cudaLaunchAttribute attr;
  attr.id = cudaLaunchAttributeClusterDimension;
  attr.val.clusterDim.x = 2; attr.val.clusterDim.y = 1; attr.val.clusterDim.z = 1;
  cfg.attrs = &attr;
  cfg.numAttrs = 1;
  int n = 0;
  cudaError_t e = cudaSuccess;
  switch (kind) {
    case KIND_I8: e = cudaOccupancyMaxActiveClusters(&n, umma_pair_gemm_kernel<KIND_I8>, &cfg); break;
    case KIND_F8: e = cudaOccupancyMaxActiveClusters(&n, umma_pair_gemm_kernel<KIND_F8>, &cfg); break;
    case KIND_F16: e = cudaOccupancyMaxActiveClusters(&n, umma_pair_gemm_kernel<KIND_F16>, &cfg); break;
    default: e = cudaOccupancyMaxActiveClusters(&n, umma_pair_gemm_kernel<KIND_TF32>, &cfg); break;
  }
  if (e != cudaSuccess) return fail(SOFIE_B200_ERR_CUDA, "cudaOccupancyMaxActiveClusters: %s", cudaGetErrorString(e));
  *out = n;
  return 0;
}

int umma_pair_launch(sofie_b200_gemm_plan *plan, const UmmaParams &u) {
  // the cluster shape is part of the kernel (__cluster_dims__), so a plain launch forms the pairs
  cudaStream_t st = plan->ctx->stream;
  dim3 grid(plan->grid), block(UMMA_PAIR_THREADS);
  switch (plan->kind) {
    case KIND_I8: umma_pair_gemm_kernel<KIND_I8><<<grid, block, plan->smem_bytes, st>>>(plan->tm_a, plan->tm_b, u); break;
    case KIND_F8: umma_pair_gemm_kernel<KIND_F8><<<grid, block, plan->smem_bytes, st>>>(plan->tm_a, plan->tm_b, u); break;
    case KIND_F16: umma_pair_gemm_kernel<KIND_F16><<<grid, block, plan->smem_bytes, st>>>(plan->tm_a, plan->tm_b, u); break;
    default: umma_pair_gemm_kernel<KIND_TF32><<<grid, block, plan->smem_bytes, st>>>(plan->tm_a, plan->tm_b, u); break;
  }
  SB_CUDA(cudaGetLastError());
  plan->ctx->launches++;
  return 0;
}

}  // namespace sb200
