// Contraction kernel for sm_100a: tcgen05.mma with the accumulator in tensor memory, operands
// staged in 128B-swizzled shared memory by TMA, one persistent CTA per SM.
//
// Roles inside a CTA of 640 threads (20 warps, 96 registers per thread)
//   warp 0, lane 0 : TMA producer of operand A.  Fills a ring of `stages` shared-memory stages; each
//                    stage holds a 128 x (128 bytes of K) slice of op(A) and a bn x (128 bytes of K)
//                    slice of op(B).
//   warp 2, lane 0 : TMA producer of operand B (a thread is held by every TMA instruction until the
//                    unit has taken it -- 110 to 400 cycles -- and one thread issuing both operands'
//                    loads fell behind 8-bit MMAs, which need a stage every 512 cycles).
//   warp 1, lane 0 : MMA issuer.  Four tcgen05.mma (K = 32 bytes each) per stage into one of two or four
//                    TMEM accumulators (128 lanes x bn columns each); tcgen05.commit releases
//                    the stage to the producer and, after the last K block, hands the accumulator
//                    to the epilogue.
//   warp 3         : idle (keeps the epilogue warps' index congruent to their tensor-memory lane quarter).
//   warps 4-19     : epilogue, four warps per tensor-memory lane quarter, in one, two or four teams that
//                    drain different tiles at the same time (umma_epi16.cuh).  A warp takes 64-byte row
//                    segments of its 32 rows in steps of 16 columns: tcgen05.ld of the next step is in
//                    flight while the current one goes through the fused epilogue into a swizzled staging
//                    buffer, and a complete segment leaves as one bulk tensor store.  The epilogue is bound
//                    by instruction issue, which is why it has sixteen warps and counts instructions.
//
// Tall tiles (UmmaParams::mh = 2): a 256 x 256 tile as two 128-row halves that share every B slice -- 64 KB of operands per
// K block for twice the MMA work of a 128 x 256 tile's 48 KB.  The large contractions are bound by the bytes an SM can pull
// from L2 per tensor-pipe cycle, not by the pipe; a tall tile needs a third fewer.  Both halves' accumulators fill tensor
// memory, so there is no second accumulator and the epilogue of a tile does not overlap the next tile's MMAs: the plan
// takes tall tiles only where K is long enough for that to be small change.
//
// Data layout: a K-major operand (row-major [rows, K]) is one TMA box of rows x 128 bytes per
// stage; an MN-major operand (row-major [K, cols]) is cols*es/128 boxes of (128 bytes x K-rows).
// Both land in the canonical 128B-swizzle layouts that the shared-memory matrix descriptors
// name, so no operand is transposed or re-laid in global memory.
//
// Every wait is bounded (ptx::mbar_wait).  A wait that runs out raises an abort flag in shared
// memory, writes a DeviceStatus code to the ctx status word, and all roles fall through to the
// common exit where tensor memory is freed.
#include <cudaTypedefs.h>
#include <cstdlib>
#include <mutex>

#include "gemm.cuh"
#include "ptx.cuh"
#include "umma_epi16.cuh"

namespace sb200 {
using namespace ptx;

// Work items: whole tiles first; the tiles of a short last wave are split into two N halves so that
// twice as many SMs share them (each half is an MMA of N = bn/2 into the same accumulator columns).
__device__ __forceinline__ void decode_item(const UmmaParams &p, uint32_t w, uint32_t &tile, int &n_off, int &n_len,
                                            uint32_t &idesc) {
  const uint32_t split_from = (uint32_t)p.split_from;
  if (w < split_from) {
    tile = w; n_off = 0; n_len = p.bn; idesc = p.idesc;
  } else {
    const uint32_t x = w - split_from;
    tile = split_from + (x >> 1);
    n_len = p.bn >> 1;
    n_off = (int)(x & 1u) * n_len;
    idesc = p.idesc_half;
  }
}

// Tile t of the whole problem -> batch and (M tile, N tile).  32-bit arithmetic (the host refuses plans with 2^31 items or
// more): every epilogue warp does this once per tile, and 64-bit divisions were a third of a narrow tile's instructions.
__device__ __forceinline__ void tile_coords(const UmmaParams &p, uint32_t t, uint32_t tiles_per_batch, int &b, int &tm, int &tn) {
  uint32_t r = t;
  b = 0;
  if (p.batch > 1) { b = (int)(t / tiles_per_batch); r = t - (uint32_t)b * tiles_per_batch; }
  if (p.rgroup > 0) {
    // bands of rgroup N tiles, N index fastest inside a band: the tiles in flight (one per SM) then share about sqrt(SMs)
    // slices of each operand, which fit L2 together, and a band's B slices stay there while the band's M tiles go by
    const uint32_t per = (uint32_t)p.tiles_m * (uint32_t)p.rgroup, band = r / per, rr = r - band * per;
    const uint32_t left = (uint32_t)p.tiles_n - band * (uint32_t)p.rgroup, w = left < (uint32_t)p.rgroup ? left : (uint32_t)p.rgroup;
    const uint32_t q = rr / w;
    tm = (int)q; tn = (int)(band * (uint32_t)p.rgroup + (rr - q * w));
  }
  else if (p.raster_n) { const uint32_t q = r / (uint32_t)p.tiles_n; tm = (int)q; tn = (int)(r - q * (uint32_t)p.tiles_n); }
  else { const uint32_t q = r / (uint32_t)p.tiles_m; tn = (int)q; tm = (int)(r - q * (uint32_t)p.tiles_m); }
}

// MH: M halves per tile (UmmaParams::mh), a template argument so that the one-half kernel pays nothing for the other.
// WIDE: 128-byte row segments in the epilogue (UmmaParams::wide), a template argument for the same reason.
template <int KIND, int MH, bool WIDE = false>
__global__ void __launch_bounds__(UMMA_THREADS, 1)   // 20 warps: 96 registers per thread
umma_gemm_kernel(const __grid_constant__ CUtensorMap tm_a, const __grid_constant__ CUtensorMap tm_b,
                 const __grid_constant__ CUtensorMap tm_y, const __grid_constant__ UmmaParams p, const __grid_constant__ UmmaPeerMaps peers) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw_addr = smem_u32(smem_raw);
  const uint32_t pad = (1024u - (raw_addr & 1023u)) & 1023u;  // swizzle atoms are 1024-byte aligned
  uint8_t *smem = smem_raw + pad;

  const int stages = p.stages;
  const uint32_t smem_a = smem_u32(smem);
  const uint32_t smem_b = smem_a + stages * p.a_stage_bytes;
  // operand B: a ring like A's, or -- resident -- all its K blocks, loaded once (tiles_n == 1: every tile uses the same B)
  const int b_slots = p.b_resident ? p.num_kb : stages;
  uint8_t *tail = smem + stages * p.a_stage_bytes + b_slots * p.b_stage_bytes;
  const uint32_t bar_full = smem_u32(tail);             // [stages]
  const uint32_t bar_empty = bar_full + 8 * stages;     // [stages]
  const uint32_t bar_tfull = bar_empty + 8 * stages;    // [UMMA_MAX_ACCS]
  const uint32_t bar_tempty = bar_tfull + 8 * UMMA_MAX_ACCS;   // [UMMA_MAX_ACCS]
  const uint32_t bar_bres = bar_tempty + 8 * UMMA_MAX_ACCS;    // resident operand B has landed
  uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(tail + 16 * stages + 16 * UMMA_MAX_ACCS + 8);
  volatile int *abort_flag = reinterpret_cast<volatile int *>(tmem_slot + 1);
  const uint32_t epi_stage = smem_u32(tail) + UMMA_TAIL_BYTES;   // UMMA_EPI_STAGE_BYTES per epilogue warp

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < stages; ++s) {
      mbar_init(bar_full + 8 * s, p.b_resident ? 1 : 2);   // one arrival (with its byte count) per operand that is loaded into the ring
      mbar_init(bar_empty + 8 * s, 1);
    }
    for (int i = 0; i < p.accs; ++i) {
      mbar_init(bar_tfull + 8 * i, 1);
      mbar_init(bar_tempty + 8 * i, UMMA_EPI_WARPS / p.teams);  // one arrival per epilogue warp of the team that drains it
    }
    mbar_init(bar_bres, 1);
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

  const uint32_t tiles_per_batch = (uint32_t)p.tiles_m * (uint32_t)p.tiles_n;
  const uint32_t num_items = (uint32_t)p.num_items;

  if (warp == 0 || warp == UMMA_B_PRODUCER_WARP) {
    // ------------------------------ TMA producers -----------------------------------
    // Warp 0 loads operand A; warp UMMA_B_PRODUCER_WARP loads operand B, or -- B resident -- loads it once and then takes
    // a share of A.  The K blocks of all of this CTA's tiles form one sequence, and an operand's `PT` producer lanes (the
    // first p.prod_lanes lanes of its one or two warps) take every PT-th block of it, in lockstep: what a thread does between
    // two TMA instructions (barrier wait, byte count, coordinates: a few hundred cycles for one thread) is time the TMA unit
    // idles, so one thread per operand capped a convolution with 64-byte K blocks at 60 % of the unit's rate.
    const bool b_warp = warp != 0;
    if (lane == 0 && p.b_resident && b_warp) {
      // resident operand B: every K block once, one barrier for all of them
      mbar_arrive_expect_tx(bar_bres, (uint32_t)p.num_kb * p.b_stage_bytes);
      for (int kb = 0; kb < p.num_kb; ++kb) {
        const uint32_t sb = smem_b + kb * p.b_stage_bytes;
        const int k0 = kb * p.kb_elems;
        if (!p.b_mn) {
          tma_load_3d(sb, &tm_b, bar_bres, k0, 0, 0);
        } else {
          for (int x = 0; x < p.b_boxes; ++x) tma_load_3d(sb + x * p.b_box_bytes, &tm_b, bar_bres, x * p.b_box_mn, k0, 0);
        }
      }
    }
    __syncwarp();
    const bool load_b = b_warp && !p.b_resident;     // this warp's operand
    const int PL = p.prod_lanes;
    const int PT = (!load_b && p.b_resident) ? 2 * PL : PL;   // producer lanes of this warp's operand, over all its warps
    const int pi = lane + ((b_warp && p.b_resident) ? PL : 0);
    if (lane < PL) {
      // this lane's position in the sequence of K blocks: work item w, K block kbi of it, ring stage and its phase
      uint32_t w = blockIdx.x, stage = (uint32_t)pi, phase = 0;
      int kbi = pi;
      bool ok = true, fresh = true;
      int m0 = 0, n0 = 0, ba = 0, bb = 0, ic_n = 0, ic_w = 0, ic_h = 0;
      while (true) {
        while (kbi >= p.num_kb) { kbi -= p.num_kb; w += gridDim.x; fresh = true; }
        if (w >= num_items) break;
        if (fresh) {
          fresh = false;
          uint32_t t; int n_off, n_len; uint32_t idesc;
          decode_item(p, w, t, n_off, n_len, idesc);
          int b, tm, tn;
          tile_coords(p, t, tiles_per_batch, b, tm, tn);
          m0 = tm * UMMA_BM * MH;
          n0 = tn * p.bn + n_off;  // a half item still loads a full-width B slice
          ba = p.a_bcast ? 0 : b; bb = p.b_bcast ? 0 : b;
          if (p.im2col) {
            // implicit convolution: the tile's first output pixel -> image and base pixel (tap (0, 0)) of its filter window
            ic_n = m0 / p.ic_pix;
            const int rem = m0 - ic_n * p.ic_pix, oh = rem / p.ic_wo;
            ic_h = oh * p.ic_sh - p.ic_pt;
            ic_w = (rem - oh * p.ic_wo) * p.ic_sw - p.ic_pl;
          }
        }
        if (!mbar_wait_relaxed(bar_empty + 8 * stage, phase ^ 1u, abort_flag)) {
          raise_abort(abort_flag, p.status, DEV_WAIT_SMEM_EMPTY);
          ok = false;
          break;
        }
        const uint32_t full = bar_full + 8 * stage;
        const int k0 = kbi * p.kb_elems;
        if (!load_b) {
          mbar_arrive_expect_tx(full, p.a_stage_bytes);
          const uint32_t sa = smem_a + stage * p.a_stage_bytes;
          if (p.im2col) {
            const int tap = kbi / p.ic_cblocks, cb = kbi - tap * p.ic_cblocks, tap_r = tap / p.ic_s, tap_s = tap - tap_r * p.ic_s;
            tma_load_im2col_4d(sa, &tm_a, full, cb * p.kb_elems, ic_w, ic_h, ic_n, (uint16_t)(tap_s * p.ic_dw), (uint16_t)(tap_r * p.ic_dh));
          } else if (!p.a_mn) {
            tma_load_3d(sa, &tm_a, full, k0, m0, ba);
          } else {
            for (int x = 0; x < p.a_boxes; ++x)
              tma_load_3d(sa + x * p.a_box_bytes, &tm_a, full, m0 + x * p.a_box_mn, k0, ba);
          }
        } else {
          mbar_arrive_expect_tx(full, p.b_stage_bytes);
          const uint32_t sb = smem_b + stage * p.b_stage_bytes;
          if (!p.b_mn) {
            tma_load_3d(sb, &tm_b, full, k0, n0, bb);
          } else {
            for (int x = 0; x < p.b_boxes; ++x)
              tma_load_3d(sb + x * p.b_box_bytes, &tm_b, full, n0 + x * p.b_box_mn, k0, bb);
          }
        }
        kbi += PT;
        stage += (uint32_t)PT;
        if (stage >= (uint32_t)stages) { stage -= (uint32_t)stages; phase ^= 1u; }
      }
      if (!ok) {
        // give copies that may still be in flight time to land before the CTA exits
        const uint64_t t0 = globaltimer();
        while (globaltimer() - t0 < 200000ull) {}
      }
    }
  } else if (warp == 1) {
    // ------------------------------ MMA issuer --------------------------------------
    if (lane == 0) {
      uint32_t stage = 0, phase = 0;
      uint32_t acc = 0, acc_phase = 0;
      bool ok = true;
      // descriptor words that do not change inside the loop, kept in registers (stage bases are multiples of 1024
      // bytes inside a 227 KB window, so adding the stage offset never carries out of the 14-bit address field)
      const uint64_t a_hi = (uint64_t)p.a_desc_hi << 32, b_hi = (uint64_t)p.b_desc_hi << 32;
      const uint32_t a_lo0 = p.a_desc_lo | ((smem_a >> 4) & 0x3fffu), b_lo0 = p.b_desc_lo | ((smem_b >> 4) & 0x3fffu);
      const uint32_t a_step = p.a_stage_bytes >> 4, b_step = p.b_stage_bytes >> 4;
      const uint32_t a_kadv = p.a_kadv, b_kadv = p.b_kadv;
      const uint64_t a_half = (uint64_t)(p.a_stage_bytes >> 5);   // half an A stage, in 16-byte units
      const int num_kb = p.num_kb, kb_mmas = p.kb_mmas;
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
      if (p.b_resident && !mbar_wait(bar_bres, 0u, abort_flag)) {
        raise_abort(abort_flag, p.status, DEV_WAIT_SMEM_FULL);
        ok = false;
      }
      for (uint32_t w = blockIdx.x; w < num_items && ok; w += gridDim.x) {
        uint32_t t; int n_off, n_len; uint32_t idesc;
        decode_item(p, w, t, n_off, n_len, idesc);
        if (!ROLE_WAIT(w_tempty, mbar_wait_relaxed(bar_tempty + 8 * acc, acc_phase ^ 1u, abort_flag))) {
          raise_abort(abort_flag, p.status, DEV_WAIT_TMEM_EMPTY);
          break;
        }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * (p.bn * MH);
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
          const uint32_t b_lo = b_lo0 + (p.b_resident ? (uint32_t)kb : stage) * b_step;
          ROLE_SECTION_BEGIN();
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            if (k >= kb_mmas) break;
            const uint64_t ad = a_hi | (uint64_t)(a_lo + k * a_kadv);
            const uint64_t bd = b_hi | (uint64_t)(b_lo + k * b_kadv);
#ifndef SB200_SKIP_MMA
            umma<KIND>(d_tmem, ad, bd, idesc, (kb | k) != 0 ? 1u : 0u);
            // tall tile: rows 128..255 of the A slice (the next 128 rows of the same box) against the same B slice
            if (MH == 2) umma<KIND>(d_tmem + p.bn, ad + a_half, bd, idesc, (kb | k) != 0 ? 1u : 0u);
#endif
          }
          ROLE_SECTION_END(c_mma);
          ROLE_SECTION_BEGIN();
          tc_commit(bar_empty + 8 * stage);  // stage may be refilled once these MMAs have read it
          ROLE_SECTION_END(c_commit);
          if (++stage == (uint32_t)stages) { stage = 0; phase ^= 1u; }
        }
        if (!ok) break;
        tc_commit(bar_tfull + 8 * acc);      // accumulator complete
        if (++acc == (uint32_t)p.accs) { acc = 0; acc_phase ^= 1u; }
      }
      ROLE_REPORT("[cta %d] mma issuer: total %lld, waiting for operands %lld, for a drained accumulator %lld\n", blockIdx.x,
                  clock64() - t_begin, w_full, w_tempty);
      ROLE_REPORT("[cta %d] mma issuer sections: fence %lld, issuing MMAs %lld, commits %lld\n", blockIdx.x, c_fence, c_mma, c_commit);
    }
  } else if (warp >= UMMA_FIRST_EPI_WARP) {
    // ------------------------------ epilogue -----------------------------------------
    const int quad = warp & 3;  // TMEM lanes 32*quad .. 32*quad+31 belong to this warp
    const int epi_warp = warp - UMMA_FIRST_EPI_WARP;
    // The four groups of four warps (one warp per lane quarter) form p.teams teams; a team drains every p.teams-th tile
    // of this CTA, its groups taking alternate row segments.  More teams = more tiles in the epilogue at once and fewer
    // warps paying each tile's fixed costs (what a narrow or short-K tile needs); fewer teams = an accumulator is free
    // again sooner (what a tile needs whose MMAs take as long as its epilogue).  umma_plan_init() picks.
    const int group = epi_warp >> 2;
    const int groups_per_team = (UMMA_EPI_WARPS / 4) / p.teams;
    const uint32_t team = (uint32_t)(group / groups_per_team);
    const int seg_first = group % groups_per_team;
    const uint32_t acc_mask = (uint32_t)p.accs - 1u, acc_shift = (uint32_t)p.accs >> 1;   // accs is 1, 2 or 4
    const Epi16Warp ew = epi16_warp_init<WIDE>(p.ep, epi_stage + (uint32_t)epi_warp * (WIDE ? 2 * UMMA_EPI_STAGE_BYTES : UMMA_EPI_STAGE_BYTES));
    const CUtensorMap *y_map = p.y_tma ? &tm_y : nullptr;
    const uint32_t taddr0 = tmem_base + ((uint32_t)(quad * 32) << 16);
    ROLE_TIMER(w_tfull);
    ROLE_TIMER(c_ld);
    ROLE_TIMER(c_st);
    ROLE_TIMER(sec_t0);
    ROLE_TIMER(t_begin);
#ifdef SB200_ROLE_TIMERS
    t_begin = clock64();
#endif
    // One trip per 128-row half of a tile (h: 0, and 1 for the lower half of a tall tile -- the next bn columns of tensor
    // memory, rows 128 further): the accumulator is waited for before its first half and handed back after its last.
    uint32_t i = team, w = blockIdx.x + team * gridDim.x;
    int h = 0;
    while (w < num_items) {
      const uint32_t acc = i & acc_mask, acc_phase = (i >> acc_shift) & 1u;   // tile i of this CTA: accumulator and its phase
      const uint32_t taddr = taddr0 + acc * (p.bn * MH) + h * p.bn;
      uint32_t t; int n_off, n_len; uint32_t idesc;
      decode_item(p, w, t, n_off, n_len, idesc);
      int b, tm, tn;
      tile_coords(p, t, tiles_per_batch, b, tm, tn);
      const int m0 = (tm * MH + h) * UMMA_BM;
      const int n0 = tn * p.bn + n_off;
      if (h == 0) {
        if (!ROLE_WAIT(w_tfull, mbar_wait_relaxed(bar_tfull + 8 * acc, acc_phase, abort_flag))) {
          raise_abort(abort_flag, p.status, DEV_WAIT_TMEM_FULL);
          break;
        }
        tc_fence_after();
      }
      const int row = m0 + quad * 32 + lane;
      const int c_end = min(n_len, p.N - n0);          // columns of this item that exist (warp-uniform)
      ROLE_SECTION_BEGIN();
#ifndef SB200_SKIP_EPI
      if (m0 < p.M) drain16_any<KIND == KIND_I8>(p.ep, ew, taddr, c_end, seg_first, groups_per_team, b, row, n0, p.vec_ok != 0, p.M, y_map, peers.tm);
#endif
      ROLE_SECTION_END(c_st);
      if (++h == MH) {
        h = 0;
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(bar_tempty + 8 * acc);
        i += (uint32_t)p.teams;
        w += gridDim.x * (uint32_t)p.teams;
      }
    }
    if (threadIdx.x == 32 * UMMA_FIRST_EPI_WARP) { ROLE_REPORT("[cta %d] epilogue: total %lld, waiting for an accumulator %lld, tensor-memory loads %lld, epilogue math + stores %lld\n", blockIdx.x, clock64() - t_begin, w_tfull, c_ld, c_st); }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, p.tmem_cols);
  }
}

// ------------------------------------ host side ------------------------------------------

static PFN_cuTensorMapEncodeTiled_v12000 get_encode() {
  static PFN_cuTensorMapEncodeTiled_v12000 fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void *sym = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<PFN_cuTensorMapEncodeTiled_v12000>(sym);
  });
  return fn;
}

static CUtensorMapDataType map_dtype(int dtype) {
  if (dtype == SOFIE_B200_BF16) return CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
  if (dtype == SOFIE_B200_F32) return CU_TENSOR_MAP_DATA_TYPE_FLOAT32;
  if (dtype == SOFIE_B200_I32) return CU_TENSOR_MAP_DATA_TYPE_INT32;
  return CU_TENSOR_MAP_DATA_TYPE_UINT8;
}

// im2col-mode map of a channels-last [N, H, W, C] tensor for one convolution: the bounding box holds the base pixels
// (top-left taps) of all filter windows, traversed with the convolution's strides; one load fetches `kb_elems` channels of
// 128 consecutive windows.
static int encode_im2col(CUtensorMap *tm, int dtype, const void *base, const Im2colDesc &ic, uint32_t kb_elems, bool swizzle64) {
  static PFN_cuTensorMapEncodeIm2col_v12000 enc = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void *sym = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeIm2col", &sym, cudaEnableDefault, &q) == cudaSuccess && q == cudaDriverEntryPointSuccess)
      enc = reinterpret_cast<PFN_cuTensorMapEncodeIm2col_v12000>(sym);
  });
  if (!enc) return fail(SOFIE_B200_ERR_NO_DEVICE, "cuTensorMapEncodeIm2col entry point not available");
  const uint64_t es = (uint64_t)dtype_size(dtype);
  const cuuint64_t cs = (cuuint64_t)(ic.Cs ? ic.Cs : ic.C);   // channels per pixel as stored
  cuuint64_t dims[4] = {cs, (cuuint64_t)ic.W, (cuuint64_t)ic.H, (cuuint64_t)ic.N};
  cuuint64_t strides[3] = {cs * es, (cuuint64_t)ic.W * cs * es, (cuuint64_t)ic.H * ic.W * cs * es};
  int lower[2] = {-ic.pl, -ic.pt};                                             // {W, H}: first base pixel
  int upper[2] = {ic.pr - (ic.S - 1) * ic.dw, ic.pb - (ic.R - 1) * ic.dh};    // last base pixel, from (W-1, H-1)
  cuuint32_t estr[4] = {1, (cuuint32_t)ic.sw, (cuuint32_t)ic.sh, 1};
  CUresult r = enc(tm, map_dtype(dtype), 4, const_cast<void *>(base), dims, strides, lower, upper, kb_elems, UMMA_BM, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle64 ? CU_TENSOR_MAP_SWIZZLE_64B : CU_TENSOR_MAP_SWIZZLE_128B,
                   CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS)
    return fail(SOFIE_B200_ERR_CUDA, "cuTensorMapEncodeIm2col failed (%d): image %lldx%lldx%lldx%lld, box corners (%d,%d)/(%d,%d), strides %d,%d",
                (int)r, ic.N, ic.H, ic.W, ic.C, lower[0], lower[1], upper[0], upper[1], ic.sw, ic.sh);
  return 0;
}

static CUtensorMapSwizzle swizzle_mode(int bytes) {
  return bytes == 16 ? CU_TENSOR_MAP_SWIZZLE_NONE : (bytes == 32 ? CU_TENSOR_MAP_SWIZZLE_32B : (bytes == 64 ? CU_TENSOR_MAP_SWIZZLE_64B : CU_TENSOR_MAP_SWIZZLE_128B));
}

static int encode_map(CUtensorMap *tm, int dtype, const void *base, uint64_t d0, uint64_t d1, uint64_t d2,
                      uint64_t stride1_bytes, uint64_t stride2_bytes, uint32_t b0, uint32_t b1, int swizzle_bytes = 128) {
  auto enc = get_encode();
  if (!enc) return fail(SOFIE_B200_ERR_NO_DEVICE, "cuTensorMapEncodeTiled entry point not available");
  const CUtensorMapDataType dt = map_dtype(dtype);
  cuuint64_t dims[3] = {d0, d1, d2};
  cuuint64_t strides[2] = {stride1_bytes, stride2_bytes};
  cuuint32_t box[3] = {b0, b1, 1};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = enc(tm, dt, 3, const_cast<void *>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                   swizzle_mode(swizzle_bytes), CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS)
    return fail(SOFIE_B200_ERR_CUDA,
                "cuTensorMapEncodeTiled failed (%d): dims %llu,%llu,%llu strides %llu,%llu box %u,%u", (int)r,
                (unsigned long long)d0, (unsigned long long)d1, (unsigned long long)d2,
                (unsigned long long)stride1_bytes, (unsigned long long)stride2_bytes, b0, b1);
  return 0;
}

static int pick_bn(long long N, long long tiles_m, long long batch, int sms, int min_bn, int max_bn = 256) {
  // Per-tile time model: MMA time grows with bn, shared-memory operand traffic with 128 + bn.
  // (`sms` is the number of concurrent tiles: SMs, or SM pairs in pair mode.)
  const int cand[4] = {256, 128, 64, 32};
  int best = max_bn >= min_bn ? max_bn : 256;
  double best_cost = 1e300;
  for (int bn : cand) {
    if (bn < min_bn || (bn > max_bn && max_bn >= min_bn)) continue;
    long long tiles = tiles_m * ((N + bn - 1) / bn) * batch;
    long long waves = (tiles + sms - 1) / sms;
    double per_tile = bn > 0.67 * (128 + bn) ? (double)bn : 0.67 * (128 + bn);
    double cost = waves * (per_tile + 8.0);
    if (cost < best_cost - 1e-9) { best_cost = cost; best = bn; }
  }
  return best;
}

int umma_plan_init(sofie_b200_gemm_plan *plan) {
  const sofie_b200_gemm_desc &d = plan->desc;
  UmmaParams &u = plan->up;
  int kind, es;
  switch (d.ab_dtype) {
    case SOFIE_B200_I8: kind = KIND_I8; es = 1; break;
    case SOFIE_B200_F8E4M3: kind = KIND_F8; es = 1; break;
    case SOFIE_B200_BF16: kind = KIND_F16; es = 2; break;
    case SOFIE_B200_F32: kind = KIND_TF32; es = 4; break;
    default: return 1;
  }
  // TMA needs 16-byte multiples for every global stride.
  const Im2colDesc &ic = plan->ic;
  if (((d.lda * es) % 16 && !ic.on) || (d.ldb * es) % 16) return 1;
  const int kb_bytes = plan->kb_bytes;   // 64: the 64-byte swizzle, for implicit convolutions over 64 bytes of channels
  if (kb_bytes != 128 && !(kb_bytes == 64 && ic.on)) return 1;
  if (ic.on) {
    // K runs over (filter row, filter column, channel); a K block never straddles two taps; B (the filters) is K-major
    // (the chunk-promotion kernel runs the three TF32 products over a tensor of pairs: K = 3 * R*S*C)
    if (d.trans_a || !d.trans_b || d.batch != 1 || (ic.C * es) % kb_bytes || d.K != (plan->promote ? 3 : 1) * ic.R * ic.S * ic.C ||
        d.M != ic.N * ic.Ho * ic.Wo || (plan->promote && ic.Cs != 2 * ic.C))
      return 1;
    const int up_w = ic.pr - (ic.S - 1) * ic.dw, up_h = ic.pb - (ic.R - 1) * ic.dh;
    if (ic.pl > 128 || ic.pt > 128 || up_w < -128 || up_w > 127 || up_h < -128 || up_h > 127 || ic.sw > 8 || ic.sh > 8 ||
        (ic.S - 1) * ic.dw > 65535 || (ic.R - 1) * ic.dh > 65535)
      return 1;
  }
  if (d.batch > 1 && (((d.stride_a * es) % 16) || ((d.stride_b * es) % 16))) return 1;
  if (d.M <= 0 || d.N <= 0 || d.K <= 0) return 1;
  // TF32 operands are taken K-major only (an MN-major fp32 operand goes to the CUDA-core kernel)
  if (d.ab_dtype == SOFIE_B200_F32 && (d.trans_a || !d.trans_b)) return 1;
  if (d.M > 0x7fffffffLL || d.N > 0x7fffffffLL || d.K > 0x7fffffffLL) return 1;

  plan->kind = kind;
  u.M = (int)d.M; u.N = (int)d.N; u.K = (int)d.K; u.batch = (int)d.batch;
  const int sms = plan->ctx->sm_count;
  const int tile_m = UMMA_BM;
  u.tiles_m = (int)((d.M + tile_m - 1) / tile_m);
  // an MN-major B slice is made of 128-byte-wide TMA boxes, so the slice one CTA stages must reach 128 bytes
  const int min_bn = d.trans_b ? 32 : 128 / es;
  u.bn = pick_bn(d.N, u.tiles_m, d.batch, sms, min_bn < 64 && plan->promote ? 64 : min_bn);
  // Tall tiles (two 128-row halves per tile, see the top of this file) where a model of the kernel's time says they win:
  // per tile the slower of the MMAs (128 cycles per 128 x 256 x 32-byte step) and the operand bytes at the 48 bytes per
  // cycle an SM measured pulling from L2, times the waves of tiles; a tall tile adds its exposed epilogue (8 outputs a cycle).
  u.mh = 1;
  const bool want_wide = !plan->promote && (d.flags & SOFIE_B200_GEMM_WIDE_STORES) != 0 && d.ab_dtype != SOFIE_B200_I8 && d.ab_dtype != SOFIE_B200_U8;
  if (!plan->promote && !ic.on && !d.trans_a && u.bn == 256 && es <= 2 && d.M > UMMA_BM && !want_wide) {
    const double nkb = (double)((d.K * es + kb_bytes - 1) / kb_bytes), tn = (double)((d.N + 255) / 256);
    double t[3] = {0, 0, 0};
    for (int mh = 1; mh <= 2; ++mh) {
      const double tiles = (double)((d.M + 128 * mh - 1) / (128 * mh)) * tn * (double)d.batch;
      const double waves = (double)(((long long)tiles + sms - 1) / sms);
      const double t_mma = nkb * 4.0 * mh * 128.0, t_bw = nkb * (128.0 * mh + 256.0) * kb_bytes / 48.0;
      t[mh] = waves * ((t_mma > t_bw ? t_mma : t_bw) + (mh == 2 ? 256.0 * 256.0 / 8.0 : 0.0));
    }
#ifndef SB200_TALL_RATIO
#define SB200_TALL_RATIO 0.85
#endif
    if (t[2] < SB200_TALL_RATIO * t[1]) u.mh = 2;
  }
  if (u.mh == 2) u.tiles_m = (int)((d.M + 2 * tile_m - 1) / (2 * tile_m));
  // Tile order.  With the M index fastest the tiles in flight share one B slice and sweep A, so A is re-read from DRAM
  // once per N tile unless it stays in L2; with the N index fastest it is B that is swept.  Take the cheaper one.
  {
    const double a_bytes = (double)d.M * d.K * es, b_bytes = (double)d.N * d.K * es, l2_fit = 48e6;
    const double tiles_n = (double)((d.N + u.bn - 1) / u.bn);
    const double cost_m = b_bytes + (a_bytes <= l2_fit ? a_bytes : tiles_n * a_bytes);
    const double cost_n = a_bytes + (b_bytes <= l2_fit ? b_bytes : (double)u.tiles_m * b_bytes);
    u.raster_n = cost_n < cost_m ? 1 : 0;
    // Neither operand fits: either order re-reads one operand from DRAM once per wave of tiles (ncu on FP8 8192^3: 540 MB
    // read for 134 MB of operands).  Bands of about sqrt(SMs) N tiles keep a wave's slices of both operands in L2.
    u.rgroup = 0;
    if (a_bytes > l2_fit && b_bytes > l2_fit && tiles_n >= 4 && u.tiles_m >= 4 && !ic.on) {
      int g = 1;
      while ((g + 1) * (g + 1) <= sms) ++g;
      u.rgroup = g < (int)tiles_n ? g : (int)tiles_n;
    }
  }
  if (plan->promote) {
    u.seg_kb = (int)(d.K / 3 / SPLIT_K_ALIGN);
    u.a_seg_kb[0] = 0; u.a_seg_kb[1] = u.seg_kb; u.a_seg_kb[2] = 0;         // A: hi, lo, hi
    u.b_seg_kb[0] = 0; u.b_seg_kb[1] = 0; u.b_seg_kb[2] = u.seg_kb;         // B: hi, hi, lo
  }
  u.promote_chunk = 8;   // 32 MMA steps per accumulation: truncation bias below 2e-6 relative even for same-sign data
  u.b_rows = u.bn;
  u.tiles_n = (int)((d.N + u.bn - 1) / u.bn);
  u.num_tiles = (long long)u.tiles_m * u.tiles_n * d.batch;
  u.kb_elems = kb_bytes / es;
  u.kb_mmas = kb_bytes / 32;
  u.num_kb = (int)((d.K + u.kb_elems - 1) / u.kb_elems);
  u.a_stage_bytes = UMMA_BM * u.mh * kb_bytes;
  u.b_stage_bytes = u.b_rows * kb_bytes;
  // Chunk-promotion kernel: hi and lo of both operands share a stage (64 KB for a 128-column tile: three stages; 96 KB
  // for 256 columns: two), so each operand block is loaded once for its two products: 4 loads per 12 MMAs instead of 6.
  // Measured faster in every shape, two-stage ring included (8192^3: 6.6 -> 6.05 ms).
  u.fused3 = plan->promote ? 1 : 0;
  if (u.fused3) { u.a_stage_bytes *= 2; u.b_stage_bytes *= 2; }
  u.im2col = ic.on;
  if (ic.on) {
    u.ic_wo = (int)ic.Wo; u.ic_pix = (int)(ic.Ho * ic.Wo);
    u.ic_sw = ic.sw; u.ic_sh = ic.sh; u.ic_pl = ic.pl; u.ic_pt = ic.pt;
    u.ic_dw = ic.dw; u.ic_dh = ic.dh; u.ic_s = ic.S;
    u.ic_cblocks = (int)(ic.C / u.kb_elems);
    u.ic_c = (int)ic.C;
  }
  // Accumulators in tensor memory (512 columns): four where the tile is at most 128 columns wide, else two.  Teams of
  // epilogue warps (see the kernel): the count that minimises a model of the time per tile -- the slowest of the MMAs,
  // the epilogue (a fixed latency per tile and team on top of the issue-bound part), and the accumulators' turnaround.
  // The constants are measurements: 6 output elements per cycle and SM through the epilogue, 1500 cycles per tile.
  u.accs = u.bn <= 128 ? 4 : 2;
  u.teams = 1;
  if (plan->promote) {
    u.accs = 2;
  } else if (u.mh == 2) {
    u.accs = 1;   // both halves' accumulators: all 512 columns
  } else {
    const double macs_per_clk = es == 1 ? 8192.0 : (es == 2 ? 4096.0 : 2048.0);
    const double t_mma = 128.0 * u.bn * (double)u.num_kb * u.kb_elems / macs_per_clk;
    const double t_epi = 128.0 * u.bn / 6.0, fixed = 1500.0;
    double best = 0;
    for (int t = 1; t <= u.accs; t *= 2) {
      double period = t_mma;
      if (t_epi + fixed / t > period) period = t_epi + fixed / t;
      const double turn = (t_mma + t * t_epi + fixed) / u.accs;
      if (turn > period) period = turn;
      if (t == 1 || period < 0.97 * best) { best = period; u.teams = t; }
    }
  }
  u.tmem_cols = 32;
  while (u.tmem_cols < (uint32_t)(u.accs * u.bn * u.mh)) u.tmem_cols <<= 1;

  // Wide stores: only where every group of a team still gets a whole 128-byte segment of the tile (else the plan stays narrow).
  u.wide = want_wide && (u.bn / 16) / (8 / dtype_size(d.y_dtype)) >= (UMMA_EPI_WARPS / 4) / u.teams ? 1 : 0;
  // staging buffers of the epilogue warps: 16 x 2 KB (the promotion kernel's 8 x 4 KB), 16 x 4 KB with wide stores
  const size_t epi_bytes = u.wide ? 64 * 1024 : 32 * 1024;
  const size_t budget = 227 * 1024 - 1024 /*alignment*/ - UMMA_TAIL_BYTES /*barriers*/ - epi_bytes;
  // Resident operand B: where one tile spans all of N and every batch uses the same B (the filters of a convolution with
  // few output channels, a narrow weight matrix), all K blocks of B stay in shared memory for the whole kernel and the
  // ring holds operand A only.  The TMA unit takes about two cycles per 64- or 128-byte row it moves, so with short K
  // rows a tile's operand loads, not its MMAs, set the pace, and B's rows are a third to a half of them.
  u.b_resident = 0;
  const size_t b_all = (size_t)u.num_kb * u.b_stage_bytes;
  if (!plan->promote && u.mh == 1 && u.tiles_n == 1 && (d.batch == 1 || (d.batch > 1 && d.stride_b == 0)) && b_all + 6 * (size_t)u.a_stage_bytes <= budget &&
      b_all < (1u << 20))
    u.b_resident = 1;
  int stages = u.b_resident ? (int)((budget - b_all) / u.a_stage_bytes) : (int)(budget / (u.a_stage_bytes + u.b_stage_bytes));
  if (stages > (kb_bytes == 64 ? 12 : 8)) stages = kb_bytes == 64 ? 12 : 8;
  if (stages < 2) return 1;
  u.stages = stages;
  // producer lanes per warp: an operand's lanes together hold at most half the ring, so that the MMAs never wait for a
  // lane that is itself waiting for a stage
  u.prod_lanes = stages / (u.b_resident ? 4 : 2);
  if (u.prod_lanes > 4) u.prod_lanes = 4;
  if (u.prod_lanes < 1) u.prod_lanes = 1;
  plan->smem_bytes = (size_t)stages * u.a_stage_bytes + (u.b_resident ? b_all : (size_t)stages * u.b_stage_bytes) + 1024 + UMMA_TAIL_BYTES + epi_bytes;

  u.a_mn = d.trans_a ? 1 : 0;   // stored [K,M]: M contiguous
  u.b_mn = d.trans_b ? 0 : 1;   // stored [K,N]: N contiguous
  u.a_bcast = (d.batch > 1 && d.stride_a == 0);
  u.b_bcast = (d.batch > 1 && d.stride_b == 0);

  // Shared-memory matrix descriptors: stride byte offset = one 8-row swizzle atom (1024 bytes with the 128-byte swizzle,
  // 512 with the 64-byte one), descriptor version 1, layout type 2 (SWIZZLE_128B) or 4 (SWIZZLE_64B).
  const uint32_t hi = ((8u * kb_bytes) >> 4) | (1u << 14) | ((kb_bytes == 64 ? 4u : 2u) << 29);
  u.a_desc_hi = hi;
  u.b_desc_hi = hi;
  const uint32_t panel_bytes = (uint32_t)u.kb_elems * 128u;  // one MN-major box: 128 bytes x K rows
  const uint32_t k_rows_per_mma = 32u / es;
  if (!u.a_mn) { u.a_desc_lo = 1u << 16; u.a_kadv = 32u >> 4; u.a_boxes = 1; u.a_box_bytes = u.a_stage_bytes; u.a_box_mn = 0; }
  else { u.a_desc_lo = ((panel_bytes >> 4) & 0x3fffu) << 16; u.a_kadv = (k_rows_per_mma * 128u) >> 4;
         u.a_boxes = (UMMA_BM * es) / 128; u.a_box_bytes = panel_bytes; u.a_box_mn = 128 / es; }
  if (!u.b_mn) { u.b_desc_lo = 1u << 16; u.b_kadv = 32u >> 4; u.b_boxes = 1; u.b_box_bytes = u.b_stage_bytes; u.b_box_mn = 0; }
  else { u.b_desc_lo = ((panel_bytes >> 4) & 0x3fffu) << 16; u.b_kadv = (k_rows_per_mma * 128u) >> 4;
         u.b_boxes = (u.b_rows * es) / 128; u.b_box_bytes = panel_bytes; u.b_box_mn = 128 / es;
         if (u.b_boxes < 1) return 1; }

  // Instruction descriptor: D format [4,6), A format [7,10), B format [10,13), A major bit 15,
  // B major bit 16, N>>3 at [17,23), M>>4 at [24,29).
  uint32_t cfmt, abfmt;
  switch (kind) {
    case KIND_I8: cfmt = 2; abfmt = 1; break;    // S32 accumulate, signed 8-bit operands
    case KIND_F8: cfmt = 1; abfmt = 0; break;    // F32 accumulate, E4M3
    case KIND_F16: cfmt = 1; abfmt = 1; break;   // F32 accumulate, BF16
    default: cfmt = 1; abfmt = 2; break;         // F32 accumulate, TF32
  }
  u.idesc = (cfmt << 4) | (abfmt << 7) | (abfmt << 10) | ((uint32_t)u.a_mn << 15) | ((uint32_t)u.b_mn << 16) |
            ((uint32_t)(u.bn >> 3) << 17) | ((uint32_t)(tile_m >> 4) << 24);

  const int ys = dtype_size(d.y_dtype);
  u.vec_ok = ((d.ldy * ys) % 16 == 0) && ((d.stride_y * ys) % 16 == 0);
  if (plan->split_out && ((d.N * ys) % 16 != 0 || d.ldy != 2 * d.N || d.y_dtype != SOFIE_B200_F32 || !plan->promote)) return 1;
  u.status = plan->ctx->d_status;

  // Short last wave: split its tiles in two N halves (see decode_item).  Only when at least one full wave
  // precedes it and the halves still fit one wave.
  u.split_from = u.num_tiles;
  u.num_items = u.num_tiles;
  u.idesc_half = (u.idesc & ~(0x3fu << 17)) | ((uint32_t)(u.bn >> 4) << 17);
  if (!plan->promote && !u.b_resident && u.mh == 1 && u.bn >= 64 && u.num_tiles > sms) {
    const long long tail = u.num_tiles % sms;
    if (tail > 0 && 2 * tail <= sms) {
      u.split_from = u.num_tiles - tail;
      u.num_items = u.num_tiles + tail;
    }
  }
  if (u.num_items >= (1ll << 31)) return 1;   // the kernel counts work items in 32 bits
  long long grid = u.num_tiles < plan->ctx->sm_count ? u.num_tiles : plan->ctx->sm_count;
  plan->grid = (int)grid;
  if (plan->promote) return umma_promote_set_smem(plan->smem_bytes);

  cudaError_t e = cudaSuccess;
#define SB200_UMMA_ATTR(K) \
  e = u.mh == 2 ? cudaFuncSetAttribute(umma_gemm_kernel<K, 2>, cudaFuncAttributeMaxDynamicSharedMemorySize, UMMA_MAX_DYN_SMEM) \
      : u.wide  ? cudaFuncSetAttribute(umma_gemm_kernel<K, 1, (K) != KIND_I8>, cudaFuncAttributeMaxDynamicSharedMemorySize, UMMA_MAX_DYN_SMEM) \
                : cudaFuncSetAttribute(umma_gemm_kernel<K, 1>, cudaFuncAttributeMaxDynamicSharedMemorySize, UMMA_MAX_DYN_SMEM)
  switch (kind) {
    case KIND_I8: SB200_UMMA_ATTR(KIND_I8); break;
    case KIND_F8: SB200_UMMA_ATTR(KIND_F8); break;
    case KIND_F16: SB200_UMMA_ATTR(KIND_F16); break;
    default: SB200_UMMA_ATTR(KIND_TF32); break;
  }
#undef SB200_UMMA_ATTR
  if (e != cudaSuccess) return fail(SOFIE_B200_ERR_CUDA, "cudaFuncSetAttribute(smem=%zu): %s", plan->smem_bytes, cudaGetErrorString(e));
  return 0;
}

static int build_maps(sofie_b200_gemm_plan *plan, const void *A, const void *B) {
  const sofie_b200_gemm_desc &d = plan->desc;
  const uint64_t kext = (uint64_t)(plan->k_store ? plan->k_store : d.K);   // K extent of the operands as stored
  const UmmaParams &u = plan->up;
  const int es = dtype_size(d.ab_dtype);
  if (A != plan->cached_a) {
    if ((uintptr_t)A % 16) return fail(SOFIE_B200_ERR_INVALID, "A must be 16-byte aligned for the tcgen05 path");
    const uint64_t nb = u.a_bcast ? 1 : (uint64_t)d.batch;
    int rc;
    if (plan->ic.on) {
      rc = encode_im2col(&plan->tm_a, d.ab_dtype, A, plan->ic, (uint32_t)u.kb_elems, plan->kb_bytes == 64);
    } else if (!u.a_mn) {
      uint64_t s2 = d.batch > 1 && !u.a_bcast ? (uint64_t)d.stride_a * es : (uint64_t)d.M * d.lda * es;
      rc = encode_map(&plan->tm_a, d.ab_dtype, A, kext, (uint64_t)d.M, nb, (uint64_t)d.lda * es, s2,
                      (uint32_t)u.kb_elems, (uint32_t)(UMMA_BM * u.mh));
    } else {
      uint64_t s2 = d.batch > 1 && !u.a_bcast ? (uint64_t)d.stride_a * es : (uint64_t)d.K * d.lda * es;
      rc = encode_map(&plan->tm_a, d.ab_dtype, A, (uint64_t)d.M, (uint64_t)d.K, nb, (uint64_t)d.lda * es, s2,
                      (uint32_t)u.a_box_mn, (uint32_t)u.kb_elems);
    }
    if (rc) return rc;
    plan->cached_a = A;
  }
  if (B != plan->cached_b) {
    if ((uintptr_t)B % 16) return fail(SOFIE_B200_ERR_INVALID, "B must be 16-byte aligned for the tcgen05 path");
    const uint64_t nb = u.b_bcast ? 1 : (uint64_t)d.batch;
    int rc;
    if (!u.b_mn) {
      uint64_t s2 = d.batch > 1 && !u.b_bcast ? (uint64_t)d.stride_b * es : (uint64_t)d.N * d.ldb * es;
      rc = encode_map(&plan->tm_b, d.ab_dtype, B, kext, (uint64_t)d.N, nb, (uint64_t)d.ldb * es, s2,
                      (uint32_t)u.kb_elems, (uint32_t)u.b_rows, plan->kb_bytes);
    } else {
      uint64_t s2 = d.batch > 1 && !u.b_bcast ? (uint64_t)d.stride_b * es : (uint64_t)d.K * d.ldb * es;
      rc = encode_map(&plan->tm_b, d.ab_dtype, B, (uint64_t)d.N, (uint64_t)d.K, nb, (uint64_t)d.ldb * es, s2,
                      (uint32_t)u.b_box_mn, (uint32_t)u.kb_elems);
    }
    if (rc) return rc;
    plan->cached_b = B;
  }
  return 0;
}

int umma_enqueue(sofie_b200_gemm_plan *plan, const void *A, const void *B, const EpiParams &ep, void *const *peer_y, int n_peers) {
  int rc = build_maps(plan, A, B);
  if (rc) return rc;
  UmmaParams u = plan->up;
  u.y_peers = 0;
  u.ep = ep;
  u.ep.split_out = plan->split_out;
  if (((uintptr_t)ep.Y % 16) != 0) u.vec_ok = 0;
  // Tensor map of Y for the epilogue's bulk stores: box = one row segment x the 32 rows of an epilogue warp.  A segment is
  // 64 bytes (128 in the promotion kernel): 4 steps of 16 columns of 1-byte outputs, 2 of 2-byte, 1 of 4-byte outputs.  A
  // narrow tile then has fewer segments than the lane quarter has warps, so the segment is halved until every warp has one.
  u.y_tma = 0;
  const int seg_bytes = plan->promote || u.wide ? 128 : 64;
  int seg_div = 1;
  if (!plan->promote && !u.wide) {
    const int full = 4 / dtype_size(plan->desc.y_dtype);   // steps per segment
    int g = full;
    while (g > 1 && (u.bn / 16) / g < (UMMA_EPI_WARPS / 4) / u.teams) g >>= 1;   // at least one segment per group of a team
    if (g < full) { u.ep.seg_chunks = g; seg_div = full / g; }
  }
  if (u.vec_ok) {
    const sofie_b200_gemm_desc &d = plan->desc;
    const int ys = dtype_size(d.y_dtype);
    if (ep.Y != plan->cached_y || seg_div != plan->cached_seg_div) {
      const uint64_t s2 = d.batch > 1 ? (uint64_t)d.stride_y * ys : (uint64_t)d.M * d.ldy * ys;
      // (a TF32-pair output is 2 N columns wide: the lo halves follow the hi halves)
      rc = encode_map(&plan->tm_y, d.y_dtype, ep.Y, (uint64_t)(plan->split_out ? 2 * d.N : d.N), (uint64_t)d.M, (uint64_t)d.batch, (uint64_t)d.ldy * ys, s2,
                      (uint32_t)(seg_bytes / ys / seg_div), 32, seg_bytes / seg_div);
      if (rc) return rc;
      plan->cached_y = ep.Y;
      plan->cached_seg_div = seg_div;
    }
    u.y_tma = 1;
    if (n_peers > 0) {
      const sofie_b200_gemm_desc &d = plan->desc;
      const int ys = dtype_size(d.y_dtype);
      const int seg_cols = seg_bytes / seg_div / ys;   // only whole segments leave through the bulk stores that are repeated per peer
      const bool halves = u.split_from < u.num_tiles;   // tiles of a short last wave are drained as two N halves
      if (u.bn % seg_cols != 0 || d.N % seg_cols != 0 || (halves && (u.bn / 2) % seg_cols != 0))
        return fail(SOFIE_B200_ERR_INVALID, "gemm_enqueue_peers: N (%lld) and the tile width (%d) must be whole row segments of %d columns", (long long)d.N, u.bn, seg_cols);
      const uint64_t s2 = d.batch > 1 ? (uint64_t)d.stride_y * ys : (uint64_t)d.M * d.ldy * ys;
      for (int q = 0; q < n_peers; ++q) {
        if (!peer_y[q] || (uintptr_t)peer_y[q] % 16) return fail(SOFIE_B200_ERR_INVALID, "gemm_enqueue_peers: output %d is NULL or not 16-byte aligned", q);
        rc = encode_map(&plan->peer_maps.tm[q], d.y_dtype, peer_y[q], (uint64_t)d.N, (uint64_t)d.M, (uint64_t)d.batch, (uint64_t)d.ldy * ys, s2,
                        (uint32_t)(seg_bytes / ys / seg_div), 32, seg_bytes / seg_div);
        if (rc) return rc;
      }
      u.y_peers = n_peers;
      u.ep.y_peers = n_peers;
    }
  }
  if (n_peers > 0 && (u.y_peers != n_peers || plan->promote))
    return fail(SOFIE_B200_ERR_INVALID, "gemm_enqueue_peers: needs the tensor-core kernel with 16-byte aligned outputs and pitches");
  if (plan->promote) return umma_promote_launch(plan, u);
  cudaStream_t st = plan->ctx->stream;
  dim3 grid(plan->grid), block(UMMA_THREADS);
#define SB200_UMMA_LAUNCH(K)                                                                             \
  if (u.mh == 2) umma_gemm_kernel<K, 2><<<grid, block, plan->smem_bytes, st>>>(plan->tm_a, plan->tm_b, plan->tm_y, u, plan->peer_maps); \
  else if (u.wide) umma_gemm_kernel<K, 1, (K) != KIND_I8><<<grid, block, plan->smem_bytes, st>>>(plan->tm_a, plan->tm_b, plan->tm_y, u, plan->peer_maps); \
  else umma_gemm_kernel<K, 1><<<grid, block, plan->smem_bytes, st>>>(plan->tm_a, plan->tm_b, plan->tm_y, u, plan->peer_maps)
  switch (plan->kind) {
    case KIND_I8: SB200_UMMA_LAUNCH(KIND_I8); break;
    case KIND_F8: SB200_UMMA_LAUNCH(KIND_F8); break;
    case KIND_F16: SB200_UMMA_LAUNCH(KIND_F16); break;
    default: SB200_UMMA_LAUNCH(KIND_TF32); break;
  }
#undef SB200_UMMA_LAUNCH
  SB_CUDA(cudaGetLastError());
  plan->ctx->launches++;
  return 0;
}

}  // namespace sb200
