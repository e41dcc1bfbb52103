// TF32 contraction with chunk promotion, the kernel behind the fp32-accurate ("umma3x") path.
//
// The tensor core adds into its fp32 accumulator with truncation, so a long K accumulates a bias that
// grows linearly with the number of MMA steps (measured: 2e-5 relative at K' = 3000), too much for the
// 1e-5 bar of the fp32 models.  Here the MMA issuer accumulates only CHUNK K-blocks (16 MMA steps) at
// a time into one of two tensor-memory accumulators; the epilogue warps drain each finished chunk into
// registers and add the chunks there with round-to-nearest, overlapping the next chunk's MMAs.  The error
// no longer depends on K.  Same roles, rings and bounded waits as umma_gemm_kernel; operands are the
// K-major split matrices written by split2_kernel (each stored once as hi | lo; the producer maps the K blocks of the
// three products hi*hi, lo*hi, hi*lo onto them).  The tile is 128 x bn, bn in {64, 128, 256}; eight
// epilogue warps (two per tensor-memory lane quarter, each owning half of the columns) keep one fp32
// register per accumulator element, so bn = 256 fits and the shared-memory operand traffic per MMA
// stays that of the plain kernel.
#include <cudaTypedefs.h>

#include "gemm.cuh"
#include "ptx.cuh"
#include "umma_store.cuh"

namespace sb200 {
using namespace ptx;

// warp 0: TMA producer of A (with fused stages: of the hi block of A), warp 1: MMA issuer, warps 2-9: epilogue,
// warp 10: producer of the lo block of A (fused stages only), warp 11: producer of B.  A thread is held by every TMA
// instruction until the unit has taken it (400 cycles for an im2col-mode load of 128 pixels x 128 bytes), and one thread
// issuing the four loads of a fused stage (1030 cycles) was slower than the stage's twelve MMAs (768 at 128 columns).
constexpr int PROMOTE_THREADS = 384;
constexpr int PROMOTE_HALF_MAX = 128; // accumulator columns (= fp32 sum registers) per epilogue thread

// Final step of a tile for one epilogue warp: the fused epilogue over this thread's `half_cols` sums (row `row`, columns
// col0 ...), staged per 32-column chunk and written by bulk tensor stores (or coalesced vector stores without a map of Y).
__device__ __noinline__ void promote_finish(const UmmaParams &p, const CUtensorMap *tm_y, const float *sum, int b, int row, int col0, int half_cols,
                                            uint32_t my_stage) {
  const int lane = threadIdx.x & 31;
  bool store_pending = false;   // a bulk tensor store of the staging buffer may still be reading it
  auto buffer_free = [&]() {
    if (store_pending) {
      if (lane == 0) bulk_wait_read_all();
      __syncwarp();
      store_pending = false;
    }
  };
  for (int c = 0; c < half_cols; c += 32) {
    const int col = col0 + c;
    if (col >= p.N) break;   // warp-uniform
    uint32_t raw[32];
#pragma unroll
    for (int u = 0; u < 32; ++u) raw[u] = __float_as_uint(sum[c + u]);
    const int parts = p.ep.split_out ? 2 : 1;   // a TF32 pair: the hi pass, then the lo pass N columns further
    const int rows_valid = (int)max(0LL, min(32LL, (long long)p.M - (row - lane)));
    const long long ldy_bytes = p.ep.ldy * out_elem_bytes(p.ep.y_dtype);
    if (p.vec_ok && p.ep.fast && p.N - col >= 32 && rows_valid > 0 && p.ep.y_dtype == SOFIE_B200_F32) {
      // the branch-light epilogue of the plain kernel (same arithmetic, step for step)
      const long long rr = row < p.M ? row : (long long)p.M - 1;
      float2 v[16];
      epi_values_fast<false, 32>(p.ep, raw, v, rr, col, my_stage, 0);
      for (int part = 0; part < parts; ++part) {
        buffer_free();
        epi_finish_fast<32>(p.ep, v, b, rr, col, my_stage, 0, p.ep.split_out ? part + 1 : 0);
        if (p.y_tma) {   // the 32 rows x 128 bytes leave as one bulk tensor store (rows past the end are clipped)
          fence_proxy_async();
          __syncwarp();
          if (lane == 0) {
            tma_store_3d(tm_y, my_stage, col + part * p.N, row - lane, b);
            bulk_commit_group();
          }
          store_pending = true;
        } else {
          flush_staged(my_stage, y_address(p.ep, b, row - lane, col + part * p.N), ldy_bytes, rows_valid, 8);
        }
      }
    } else {
      buffer_free();
      for (int part = 0; part < parts; ++part) {
        const int sp = p.ep.split_out ? part + 1 : 0;
        if (store_chunk(p.ep, raw, b, row, col, min(32, p.N - col), p.vec_ok != 0, my_stage, p.M, 0, sp))
          flush_staged(my_stage, y_address(p.ep, b, row - lane, col + part * p.N), ldy_bytes, rows_valid, 2 * out_elem_bytes(p.ep.y_dtype));
      }
    }
  }
  buffer_free();
}

__global__ void __launch_bounds__(PROMOTE_THREADS, 1)
umma_tf32_promote_kernel(const __grid_constant__ CUtensorMap tm_a, const __grid_constant__ CUtensorMap tm_b,
                         const __grid_constant__ CUtensorMap tm_y, const __grid_constant__ UmmaParams p) {
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

  if (threadIdx.x == 0) {
    for (int s = 0; s < stages; ++s) {
      mbar_init(bar_full + 8 * s, p.fused3 ? 3 : 2);   // one arrival (with its byte count) per active producer
      mbar_init(bar_empty + 8 * s, 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(bar_tfull + 8 * i, 1);
      mbar_init(bar_tempty + 8 * i, 8);
    }
    *abort_flag = 0;
    fence_barrier_init();
    prefetch_tensormap(&tm_a);
    prefetch_tensormap(&tm_b);
    if (p.y_tma) prefetch_tensormap(&tm_y);
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(tmem_slot), p.tmem_cols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const long long tiles_per_batch = (long long)p.tiles_m * p.tiles_n;
  // K-blocks (of 32 floats) per tensor-memory accumulation; with fused stages a step is one K block of all three products
  const int chunk = p.fused3 ? max(1, p.promote_chunk / 3) : p.promote_chunk;
  const int num_steps = p.fused3 ? p.seg_kb : p.num_kb;
  const int num_chunks = (num_steps + chunk - 1) / chunk;
  const uint32_t a_half = p.a_stage_bytes >> 1, b_half = p.b_stage_bytes >> 1;   // fused stages: hi block, then lo block

  if (warp == 0 || warp >= 10) {
    // ---- TMA producers.  role 0: A (fused stages: its hi block), 1: the lo block of A (fused stages only), 2: B
    const int role = warp == 0 ? 0 : warp - 9;
    if (lane == 0 && (role != 1 || p.fused3)) {
      uint32_t stage = 0, phase = 0;
      bool ok = true;
      ROLE_TIMER(w_empty);
      ROLE_TIMER(c_load_a);
      ROLE_TIMER(c_load_b);
      ROLE_TIMER(sec_t0);
      ROLE_TIMER(t_begin);
#ifdef SB200_ROLE_TIMERS
      t_begin = clock64();
#endif
      for (long long t = blockIdx.x; t < p.num_tiles && ok; t += gridDim.x) {
        const int b = (int)(t / tiles_per_batch);
        const int r = (int)(t % tiles_per_batch);
        int tm, tn;
        tile_mn(p, r, tm, tn);
        const int m0 = tm * UMMA_BM;
        const int n0 = tn * p.bn;
        const int ba = p.a_bcast ? 0 : b, bb = p.b_bcast ? 0 : b;
        // implicit convolution (A is a channels-last tensor of TF32 pairs, read in im2col mode): the tile's first output
        // pixel -> image and base pixel (tap (0, 0)) of its filter window
        int ic_n = 0, ic_w = 0, ic_h = 0;
        if (p.im2col) {
          ic_n = m0 / p.ic_pix;
          const int rem = m0 - ic_n * p.ic_pix, oh = rem / p.ic_wo;
          ic_h = oh * p.ic_sh - p.ic_pt;
          ic_w = (rem - oh * p.ic_wo) * p.ic_sw - p.ic_pl;
        }
        for (int kb = 0; kb < num_steps; ++kb) {
          if (!ROLE_WAIT(w_empty, mbar_wait(bar_empty + 8 * stage, phase ^ 1u, abort_flag))) {
            raise_abort(abort_flag, p.status, DEV_WAIT_SMEM_EMPTY);
            ok = false;
            break;
          }
          const uint32_t full = bar_full + 8 * stage;
          mbar_arrive_expect_tx(full, role == 2 ? p.b_stage_bytes : (p.fused3 ? a_half : p.a_stage_bytes));
          if (p.fused3) {   // K block kb of the stored operands: hi and lo of A, hi and lo of B
            const uint32_t sa = smem_a + stage * p.a_stage_bytes, sb = smem_b + stage * p.b_stage_bytes;
            ROLE_SECTION_BEGIN();
            if (role == 2) {
            } else if (p.im2col) {
              const int tap = kb / p.ic_cblocks, cb = kb - tap * p.ic_cblocks;
              const int tap_r = tap / p.ic_s, tap_s = tap - tap_r * p.ic_s;
              const uint16_t wo = (uint16_t)(tap_s * p.ic_dw), ho = (uint16_t)(tap_r * p.ic_dh);
              if (role == 0) tma_load_im2col_4d(sa, &tm_a, full, cb * p.kb_elems, ic_w, ic_h, ic_n, wo, ho);
              else tma_load_im2col_4d(sa + a_half, &tm_a, full, p.ic_c + cb * p.kb_elems, ic_w, ic_h, ic_n, wo, ho);
            } else {
              if (role == 0) tma_load_3d(sa, &tm_a, full, kb * p.kb_elems, m0, ba);
              else tma_load_3d(sa + a_half, &tm_a, full, (p.seg_kb + kb) * p.kb_elems, m0, ba);
            }
            ROLE_SECTION_END(c_load_a);
            ROLE_SECTION_BEGIN();
            if (role == 2) {
              tma_load_3d(sb, &tm_b, full, kb * p.kb_elems, n0, bb);
              tma_load_3d(sb + b_half, &tm_b, full, (p.seg_kb + kb) * p.kb_elems, n0, bb);
            }
            ROLE_SECTION_END(c_load_b);
            if (++stage == (uint32_t)stages) { stage = 0; phase ^= 1u; }
            continue;
          }
          // K block kb of the three-product contraction -> K block of the stored [hi | lo] operand
          const int seg = kb / p.seg_kb, off = kb - seg * p.seg_kb;
          ROLE_SECTION_BEGIN();
          if (role != 0) {
          } else if (p.im2col) {
            // K block `off` of a segment is (filter tap off / cblocks, channel block off % cblocks); the lo channels of a
            // pixel follow its ic_c hi channels
            const int tap = off / p.ic_cblocks, cb = off - tap * p.ic_cblocks;
            const int tap_r = tap / p.ic_s, tap_s = tap - tap_r * p.ic_s;
            tma_load_im2col_4d(smem_a + stage * p.a_stage_bytes, &tm_a, full, (p.a_seg_kb[seg] != 0 ? p.ic_c : 0) + cb * p.kb_elems, ic_w, ic_h,
                               ic_n, (uint16_t)(tap_s * p.ic_dw), (uint16_t)(tap_r * p.ic_dh));
          } else
          tma_load_3d(smem_a + stage * p.a_stage_bytes, &tm_a, full, (p.a_seg_kb[seg] + off) * p.kb_elems, m0, ba);
          ROLE_SECTION_END(c_load_a);
          ROLE_SECTION_BEGIN();
          if (role == 2) tma_load_3d(smem_b + stage * p.b_stage_bytes, &tm_b, full, (p.b_seg_kb[seg] + off) * p.kb_elems, n0, bb);
          ROLE_SECTION_END(c_load_b);
          if (++stage == (uint32_t)stages) { stage = 0; phase ^= 1u; }
        }
      }
      ROLE_REPORT("[cta %d] promote producer: total %lld, waiting for a free stage %lld, issuing A loads %lld, B loads %lld\n", blockIdx.x, clock64() - t_begin, w_empty, c_load_a, c_load_b);
      if (!ok) {
        const uint64_t t0 = globaltimer();
        while (globaltimer() - t0 < 200000ull) {}
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {  // ---- MMA issuer: one tensor-memory accumulation per chunk of K-blocks
      uint32_t stage = 0, phase = 0, acc = 0, acc_phase = 0;
      bool ok = true;
      ROLE_TIMER(w_full);
      ROLE_TIMER(w_tempty);
      ROLE_TIMER(t_begin);
#ifdef SB200_ROLE_TIMERS
      t_begin = clock64();
#endif
      for (long long t = blockIdx.x; t < p.num_tiles && ok; t += gridDim.x) {
        for (int ch = 0; ch < num_chunks && ok; ++ch) {
          if (!ROLE_WAIT(w_tempty, mbar_wait(bar_tempty + 8 * acc, acc_phase ^ 1u, abort_flag))) {
            raise_abort(abort_flag, p.status, DEV_WAIT_TMEM_EMPTY);
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t d_tmem = tmem_base + acc * p.bn;
          const int kb0 = ch * chunk, kb_end = min(num_steps, kb0 + chunk);
          for (int kb = kb0; kb < kb_end; ++kb) {
            if (!ROLE_WAIT(w_full, mbar_wait(bar_full + 8 * stage, phase, abort_flag))) {
              raise_abort(abort_flag, p.status, DEV_WAIT_SMEM_FULL);
              ok = false;
              break;
            }
            tc_fence_after();
            const uint32_t a_lo = p.a_desc_lo | (((smem_a + stage * p.a_stage_bytes) >> 4) & 0x3fffu);
            const uint32_t b_lo = p.b_desc_lo | (((smem_b + stage * p.b_stage_bytes) >> 4) & 0x3fffu);
            if (p.fused3) {   // hi x hi, lo x hi, hi x lo from the four blocks of the stage
              const uint32_t a_l2 = p.a_desc_lo | (((smem_a + stage * p.a_stage_bytes + a_half) >> 4) & 0x3fffu);
              const uint32_t b_l2 = p.b_desc_lo | (((smem_b + stage * p.b_stage_bytes + b_half) >> 4) & 0x3fffu);
              const uint64_t ah = (uint64_t)p.a_desc_hi << 32, bh = (uint64_t)p.b_desc_hi << 32;
#pragma unroll
              for (int k = 0; k < 4; ++k)
                umma<KIND_TF32>(d_tmem, ah | (uint64_t)(a_lo + k * p.a_kadv), bh | (uint64_t)(b_lo + k * p.b_kadv), p.idesc, (kb != kb0 || k != 0) ? 1u : 0u);
#pragma unroll
              for (int k = 0; k < 4; ++k)
                umma<KIND_TF32>(d_tmem, ah | (uint64_t)(a_l2 + k * p.a_kadv), bh | (uint64_t)(b_lo + k * p.b_kadv), p.idesc, 1u);
#pragma unroll
              for (int k = 0; k < 4; ++k)
                umma<KIND_TF32>(d_tmem, ah | (uint64_t)(a_lo + k * p.a_kadv), bh | (uint64_t)(b_l2 + k * p.b_kadv), p.idesc, 1u);
              tc_commit(bar_empty + 8 * stage);
              if (++stage == (uint32_t)stages) { stage = 0; phase ^= 1u; }
              continue;
            }
#pragma unroll
            for (int k = 0; k < 4; ++k) {
              const uint64_t ad = ((uint64_t)p.a_desc_hi << 32) | (uint64_t)(a_lo + k * p.a_kadv);
              const uint64_t bd = ((uint64_t)p.b_desc_hi << 32) | (uint64_t)(b_lo + k * p.b_kadv);
              umma<KIND_TF32>(d_tmem, ad, bd, p.idesc, (kb != kb0 || k != 0) ? 1u : 0u);
            }
            tc_commit(bar_empty + 8 * stage);
            if (++stage == (uint32_t)stages) { stage = 0; phase ^= 1u; }
          }
          if (!ok) break;
          tc_commit(bar_tfull + 8 * acc);
          if (++acc == 2) { acc = 0; acc_phase ^= 1u; }
        }
      }
      ROLE_REPORT("[cta %d] promote mma issuer: total %lld, waiting for operands %lld, for a drained accumulator %lld\n", blockIdx.x, clock64() - t_begin, w_full, w_tempty);
    }
  } else {
    // ---- epilogue: sum the chunks in registers (round to nearest), then the fused epilogue
    const int quad = warp & 3;               // tensor-memory lanes 32*quad .. 32*quad+31
    const int half_cols = p.bn >> 1;
    const int col_base = ((warp - 2) >> 2) * half_cols;
    uint32_t acc = 0, acc_phase = 0;
    bool ok = true;
    ROLE_TIMER(w_tfull);
    ROLE_TIMER(c_final);
    ROLE_TIMER(sec_t0);
    ROLE_TIMER(t_begin);
#ifdef SB200_ROLE_TIMERS
    t_begin = clock64();
#endif
    for (long long t = blockIdx.x; t < p.num_tiles && ok; t += gridDim.x) {
      const int b = (int)(t / tiles_per_batch);
      const int r = (int)(t % tiles_per_batch);
      int tm, tn;
      tile_mn(p, r, tm, tn);
      const int m0 = tm * UMMA_BM;
      const int n0 = tn * p.bn;
      float sum[PROMOTE_HALF_MAX];
#pragma unroll
      for (int c = 0; c < PROMOTE_HALF_MAX; ++c) sum[c] = 0.f;
      for (int ch = 0; ch < num_chunks; ++ch) {
        if (!ROLE_WAIT(w_tfull, mbar_wait(bar_tfull + 8 * acc, acc_phase, abort_flag))) {
          raise_abort(abort_flag, p.status, DEV_WAIT_TMEM_FULL);
          ok = false;
          break;
        }
        tc_fence_after();
        const uint32_t taddr = tmem_base + ((uint32_t)(quad * 32) << 16) + acc * p.bn + col_base;
#pragma unroll
        for (int c = 0; c < PROMOTE_HALF_MAX; c += 32) {
          if (c < half_cols) {
            uint32_t raw[32];
            tmem_ld_x32(taddr + c, raw);
            tmem_ld_wait();
#pragma unroll
            for (int u = 0; u < 32; ++u) sum[c + u] = __fadd_rn(sum[c + u], __uint_as_float(raw[u]));
          }
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(bar_tempty + 8 * acc);
        if (++acc == 2) { acc = 0; acc_phase ^= 1u; }
      }
      if (!ok) break;
      ROLE_SECTION_BEGIN();
      // The sums go through local memory to a function of its own: it runs once per tile, and kept inline its registers
      // (epilogue operands, staging) pushed part of `sum` out of the register file in the chunk loop above, which runs
      // once per 8 K blocks.
      float out[PROMOTE_HALF_MAX];
#pragma unroll
      for (int c = 0; c < PROMOTE_HALF_MAX; ++c) out[c] = sum[c];
      promote_finish(p, &tm_y, out, b, m0 + quad * 32 + lane, n0 + col_base, half_cols, epi_stage + (uint32_t)(warp - 2) * 4096u);
      ROLE_SECTION_END(c_final);
    }
    if (threadIdx.x == 64) { ROLE_REPORT("[cta %d] promote epilogue: total %lld, waiting for a chunk %lld, final epilogue + stores %lld\n", blockIdx.x, clock64() - t_begin, w_tfull, c_final); }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, p.tmem_cols);
  }
}

int umma_promote_set_smem(size_t smem_bytes) {
  cudaError_t e = cudaFuncSetAttribute(umma_tf32_promote_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, UMMA_MAX_DYN_SMEM);
  if (e != cudaSuccess) return fail(SOFIE_B200_ERR_CUDA, "cudaFuncSetAttribute(promote kernel, smem=%zu): %s", smem_bytes, cudaGetErrorString(e));
  return 0;
}

int umma_promote_launch(sofie_b200_gemm_plan *plan, const UmmaParams &u) {
  umma_tf32_promote_kernel<<<dim3(plan->grid), dim3(PROMOTE_THREADS), plan->smem_bytes, plan->ctx->stream>>>(plan->tm_a, plan->tm_b, plan->tm_y, u);
  SB_CUDA(cudaGetLastError());
  plan->ctx->launches++;
  return 0;
}

}  // namespace sb200
