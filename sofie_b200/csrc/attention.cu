// Fused scaled-dot-product attention for sequences of up to 128 tokens and a head size of 64:
//     out[b, :, h, :] = Softmax(scale * Q K^T) V      for every (batch b, head h) pair,
// reading Q, K and V as [batch, seq, heads * 64] tensors with a row pitch of their own -- three tensors, or the three column
// blocks of the QKV projection's output [batch, seq, 3, heads, 64], read in place -- and writing the layout the output
// projection reads, [batch, seq, heads * 64] (the folded form of ROperator_SDPA, ROperator_SDPA.hxx:103-129).  The scores never leave the SM: the chain
// of two batched contractions, a Softmax and two transposes (the graph the reference emits for an attention
// block: stacked MatMul, ROperator_Gemm.hxx:991-1065; Softmax, ROperator_Softmax.hxx:204-342; Transpose) moved
// 10x the bytes through HBM that Q, K, V and the output occupy.
//
// One persistent CTA per SM walks over (b, h) pairs.  Roles (320 threads):
//   warp 0, lane 0 : TMA producer.  Q, K, V tiles (128 rows x 128 bytes each, 128B swizzle) into a ring of stages;
//                    rows past `seq` are zero-filled by the TMA unit.
//   warp 1, lane 0 : MMA issuer.  S = Q K^T (tcgen05.mma, bf16, M = 128, N = 128, K = 64) into tensor memory, and,
//                    once the Softmax group has written P, O = P V (M = 128, N = 64, K = 128).  The S of the next
//                    pair is issued before the O of the current one, so the tensor core works during the Softmax.
//   warps 2-5 / 6-9: two Softmax groups taking alternate pairs.  A thread owns one query row (one tensor-memory
//                    lane): pass 1 finds the row maximum, pass 2 writes exp2(s * scale * log2 e - max) as bf16
//                    into shared memory in the K-major swizzled layout the second MMA reads, summing in fp32;
//                    the division by the row sum is applied to O (64 values) instead of P (128 values).  O goes
//                    to shared memory (the buffer P occupied) and leaves as one bulk tensor store per warp.
// Every wait is bounded (ptx::mbar_wait); a wait that runs out raises the abort flag and a status code.
#include <cudaTypedefs.h>
#include <math.h>
#include <algorithm>
#include <mutex>

#include "gemm.cuh"
#include "ptx.cuh"
#include "umma_store.cuh"

namespace sb200 {
using namespace ptx;

constexpr int ATT_THREADS = 320;
constexpr int ATT_STAGES = 3;                 // Q/K/V stages in flight
constexpr int ATT_TILE = 128 * 128;           // bytes of one 128-row x 64-element bf16 tile
constexpr int ATT_STAGE_BYTES = 3 * ATT_TILE; // Q, K, V
constexpr int ATT_P_BYTES = 2 * ATT_TILE;     // P: 128 rows x 128 keys bf16 = two K blocks of 64 keys
constexpr int ATT_SMEM = ATT_STAGES * ATT_STAGE_BYTES + 2 * ATT_P_BYTES + 1024 /*barriers*/ + 1024 /*alignment*/;

struct AttnParams {
  int batch, seq, heads;
  long long pairs;        // batch * heads
  float scale_log2e;      // scale * log2(e)
  int *status;
};

__device__ __forceinline__ float ex2_approx(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

__global__ void __launch_bounds__(ATT_THREADS, 1)
attention_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k, const __grid_constant__ CUtensorMap tm_v,
                 const __grid_constant__ CUtensorMap tm_out, const __grid_constant__ AttnParams p) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw_addr = smem_u32(smem_raw);
  const uint32_t pad = (1024u - (raw_addr & 1023u)) & 1023u;
  const uint32_t base = raw_addr + pad;
  uint8_t *gen = smem_raw + pad;
  const uint32_t sm_stage = base;                                          // [ATT_STAGES][Q | K | V]
  const uint32_t sm_p = base + ATT_STAGES * ATT_STAGE_BYTES;               // [2][ATT_P_BYTES]
  uint8_t *tail = gen + ATT_STAGES * ATT_STAGE_BYTES + 2 * ATT_P_BYTES;
  const uint32_t bar_full = smem_u32(tail);                 // [ATT_STAGES] Q, K, V landed
  const uint32_t bar_empty = bar_full + 8 * ATT_STAGES;     // [ATT_STAGES] both MMAs of the pair have read the stage
  const uint32_t bar_s = bar_empty + 8 * ATT_STAGES;        // [2] S complete in tensor memory
  const uint32_t bar_p = bar_s + 16;                        // [2] P written to shared memory
  const uint32_t bar_o = bar_p + 16;                        // [2] O complete in tensor memory
  const uint32_t bar_acc = bar_o + 16;                      // [2] S and O of the set have been read: the set is free
  uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(tail + 8 * (2 * ATT_STAGES + 8));
  volatile int *abort_flag = reinterpret_cast<volatile int *>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < ATT_STAGES; ++s) {
      mbar_init(bar_full + 8 * s, 1);
      mbar_init(bar_empty + 8 * s, 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(bar_s + 8 * i, 1);
      mbar_init(bar_p + 8 * i, 4);     // one arrival per warp of the Softmax group
      mbar_init(bar_o + 8 * i, 1);
      mbar_init(bar_acc + 8 * i, 4);
    }
    *abort_flag = 0;
    fence_barrier_init();
    prefetch_tensormap(&tm_q);
    prefetch_tensormap(&tm_k);
    prefetch_tensormap(&tm_v);
    prefetch_tensormap(&tm_out);
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(tmem_slot), 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  // tensor-memory columns of set s: S at 256 s (128 columns), O at 256 s + 128 (64 columns)

  // pairs of this CTA: blockIdx.x, blockIdx.x + gridDim.x, ...; the i-th of them uses stage i % ATT_STAGES and set i & 1
  const long long first = blockIdx.x, step = gridDim.x;
  const long long mine = first < p.pairs ? (p.pairs - first + step - 1) / step : 0;

  if (warp == 0) {
    if (lane == 0) {
      bool ok = true;
      for (long long i = 0; i < mine && ok; ++i) {
        const long long pr = first + i * step;
        const int b = (int)(pr / p.heads), h = (int)(pr % p.heads);
        const uint32_t st = (uint32_t)(i % ATT_STAGES), ph = (uint32_t)((i / ATT_STAGES) & 1);
        if (!mbar_wait(bar_empty + 8 * st, ph ^ 1u, abort_flag)) {
          raise_abort(abort_flag, p.status, DEV_WAIT_SMEM_EMPTY);
          ok = false;
          break;
        }
        const uint32_t full = bar_full + 8 * st;
        mbar_arrive_expect_tx(full, ATT_STAGE_BYTES);
        const uint32_t dst = sm_stage + st * ATT_STAGE_BYTES;
        tma_load_4d(dst, &tm_q, full, 0, h, 0, b);
        tma_load_4d(dst + ATT_TILE, &tm_k, full, 0, h, 0, b);
        tma_load_4d(dst + 2 * ATT_TILE, &tm_v, full, 0, h, 0, b);
      }
      if (!ok) {
        const uint64_t t0 = globaltimer();
        while (globaltimer() - t0 < 200000ull) {}
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      // descriptors: 128B swizzle, stride between 8-row groups 1024 bytes, version 1
      const uint64_t desc_hi = (uint64_t)((1024u >> 4) | (1u << 14) | (2u << 29)) << 32;
      const uint32_t kmajor_lo = 1u << 16;
      const uint32_t v_lo = (((uint32_t)ATT_TILE >> 4) & 0x3fffu) << 16;   // MN-major operand: leading offset = one 128-byte panel
      // instruction descriptors: fp32 accumulate, bf16 operands, M = 128; S: N = 128, both K-major; O: N = 64, B MN-major
      const uint32_t idesc_s = (1u << 4) | (1u << 7) | (1u << 10) | ((128u >> 3) << 17) | ((128u >> 4) << 24);
      const uint32_t idesc_o = (1u << 4) | (1u << 7) | (1u << 10) | (1u << 16) | ((64u >> 3) << 17) | ((128u >> 4) << 24);
      bool ok = true;
      auto issue_s = [&](long long i) -> bool {   // S of the i-th pair
        const uint32_t st = (uint32_t)(i % ATT_STAGES), ph = (uint32_t)((i / ATT_STAGES) & 1);
        const uint32_t set = (uint32_t)(i & 1), sph = (uint32_t)((i >> 1) & 1);
        if (!mbar_wait(bar_acc + 8 * set, sph ^ 1u, abort_flag)) { raise_abort(abort_flag, p.status, DEV_WAIT_TMEM_EMPTY); return false; }
        if (!mbar_wait(bar_full + 8 * st, ph, abort_flag)) { raise_abort(abort_flag, p.status, DEV_WAIT_SMEM_FULL); return false; }
        tc_fence_after();
        const uint32_t q = sm_stage + st * ATT_STAGE_BYTES, k = q + ATT_TILE;
#pragma unroll
        for (int kk = 0; kk < 4; ++kk) {   // K = 64 = 4 x 16
          const uint64_t ad = desc_hi | (uint64_t)(kmajor_lo | (((q >> 4) + 2 * kk) & 0x3fffu));
          const uint64_t bd = desc_hi | (uint64_t)(kmajor_lo | (((k >> 4) + 2 * kk) & 0x3fffu));
          umma<KIND_F16>(tmem_base + 256 * set, ad, bd, idesc_s, kk != 0 ? 1u : 0u);
        }
        tc_commit(bar_s + 8 * set);
        return true;
      };
      if (mine > 0) ok = issue_s(0);
      for (long long i = 0; i < mine && ok; ++i) {
        if (i + 1 < mine && !(ok = issue_s(i + 1))) break;
        const uint32_t st = (uint32_t)(i % ATT_STAGES);
        const uint32_t set = (uint32_t)(i & 1), sph = (uint32_t)((i >> 1) & 1);
        if (!mbar_wait(bar_p + 8 * set, sph, abort_flag)) {
          raise_abort(abort_flag, p.status, DEV_WAIT_SMEM_FULL);
          ok = false;
          break;
        }
        tc_fence_after();
        const uint32_t pa = sm_p + set * ATT_P_BYTES;
        const uint32_t v = sm_stage + st * ATT_STAGE_BYTES + 2 * ATT_TILE;
#pragma unroll
        for (int kk = 0; kk < 8; ++kk) {   // K = 128 keys = 8 x 16
          const uint32_t pt = pa + (kk >> 2) * ATT_TILE;   // P tile of keys [64 (kk / 4), +64)
          const uint64_t ad = desc_hi | (uint64_t)(kmajor_lo | (((pt >> 4) + 2 * (kk & 3)) & 0x3fffu));
          const uint64_t bd = desc_hi | (uint64_t)(v_lo | (((v >> 4) + 128 * kk) & 0x3fffu));   // 16 key rows x 128 bytes further
          umma<KIND_F16>(tmem_base + 256 * set + 128, ad, bd, idesc_o, kk != 0 ? 1u : 0u);
        }
        tc_commit(bar_o + 8 * set);
        tc_commit(bar_empty + 8 * st);
      }
    }
  } else {
    // ------------------------------ Softmax + output, one group per set ------------------------------
    const uint32_t set = (uint32_t)((warp - 2) >> 2);
    const int quad = warp & 3;                       // tensor-memory lanes 32 quad .. 32 quad + 31
    const int row = quad * 32 + lane;                // query row of this thread
    const uint32_t t_s = tmem_base + ((uint32_t)(quad * 32) << 16) + 256 * set;
    const uint32_t t_o = t_s + 128;
    const uint32_t pa = sm_p + set * ATT_P_BYTES;
    const uint32_t my_p = pa + row * 128;            // this row inside a 128-byte-row tile
    const int swz = row & 7;
    bool store_pending = false;
    for (long long i = set; i < mine; i += 2) {
      const long long pr = first + i * step;
      const int b = (int)(pr / p.heads), h = (int)(pr % p.heads);
      const uint32_t sph = (uint32_t)((i >> 1) & 1);
      if (!mbar_wait(bar_s + 8 * set, sph, abort_flag)) {
        raise_abort(abort_flag, p.status, DEV_WAIT_TMEM_FULL);
        break;
      }
      tc_fence_after();
      // Two register buffers: the tcgen05.ld of the next 32 columns is in flight while the current ones are processed,
      // and pass 2 starts loading before pass 1 has finished its arithmetic.
      uint32_t ra[32], rb[32];
      // The Softmax chain is bound by instruction issue, so it counts instructions: the row maximum is taken over the RAW
      // scores and scaled once (a positive scale keeps the order; a negative one takes the minimum), and only the 32-column
      // chunk that holds the end of a short sequence pays for masking.
      const bool pos = p.scale_log2e >= 0.f;
      float mx = -3.0e38f, mn = 3.0e38f;
      auto max_of = [&](const uint32_t (&r)[32], int c) {
        if (c + 32 <= p.seq) {
          if (pos) {
#pragma unroll
            for (int u = 0; u < 32; ++u) mx = fmaxf(mx, __uint_as_float(r[u]));
          } else {
#pragma unroll
            for (int u = 0; u < 32; ++u) mn = fminf(mn, __uint_as_float(r[u]));
          }
        } else {
#pragma unroll
          for (int u = 0; u < 32; ++u) {
            if (c + u < p.seq) { mx = fmaxf(mx, __uint_as_float(r[u])); mn = fminf(mn, __uint_as_float(r[u])); }
          }
        }
      };
      // pass 1: row maximum over the keys that exist
      tmem_ld_x32(t_s, ra);
      tmem_ld_wait(); tmem_ld_x32(t_s + 32, rb); max_of(ra, 0);
      tmem_ld_wait(); tmem_ld_x32(t_s + 64, ra); max_of(rb, 32);
      tmem_ld_wait(); tmem_ld_x32(t_s + 96, rb); max_of(ra, 64);
      tmem_ld_wait(); tmem_ld_x32(t_s, ra);      max_of(rb, 96);     // first chunk of pass 2 already on its way
      if (store_pending) {   // the previous output store of this warp must have read the buffer P is written to
        if (lane == 0) bulk_wait_read_all();
        __syncwarp();
        store_pending = false;
      }
      // pass 2: unnormalised probabilities as bf16 into shared memory, fp32 row sum
      const float off = (pos ? mx : mn) * p.scale_log2e;   // maximum of the scaled scores
      float2 sum2 = make_float2(0.f, 0.f);
      auto exp_store = [&](const uint32_t (&r)[32], int c) {
        uint32_t w[16];
        const bool full = c + 32 <= p.seq;
#pragma unroll
        for (int u = 0; u < 32; u += 2) {
          float e0 = ex2_approx(__fmaf_rn(__uint_as_float(r[u]), p.scale_log2e, -off));
          float e1 = ex2_approx(__fmaf_rn(__uint_as_float(r[u + 1]), p.scale_log2e, -off));
          if (!full) {
            if (c + u >= p.seq) e0 = 0.f;
            if (c + u + 1 >= p.seq) e1 = 0.f;
          }
          __nv_bfloat162 h2 = __floats2bfloat162_rn(e0, e1);
          const uint32_t hw = *reinterpret_cast<uint32_t *>(&h2);
          // the sum of what the second MMA will actually read: both bf16 halves back as fp32, one packed add
          sum2 = __fadd2_rn(sum2, make_float2(__uint_as_float(hw << 16), __uint_as_float(hw & 0xffff0000u)));
          w[u >> 1] = hw;
        }
        const uint32_t tile = my_p + (c >> 6) * ATT_TILE;   // keys [0, 64) -> tile 0, [64, 128) -> tile 1
        const int u0 = (c & 32) >> 3;                       // first 16-byte unit of this chunk inside the 128-byte row
#pragma unroll
        for (int u = 0; u < 4; ++u)
          asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(tile + (((u0 + u) ^ swz) << 4)), "r"(w[4 * u]), "r"(w[4 * u + 1]),
                       "r"(w[4 * u + 2]), "r"(w[4 * u + 3])
                       : "memory");
      };
      tmem_ld_wait(); tmem_ld_x32(t_s + 32, rb); exp_store(ra, 0);
      tmem_ld_wait(); tmem_ld_x32(t_s + 64, ra); exp_store(rb, 32);
      tmem_ld_wait(); tmem_ld_x32(t_s + 96, rb); exp_store(ra, 64);
      tmem_ld_wait();                            exp_store(rb, 96);
      const float sum = sum2.x + sum2.y;
      fence_proxy_async();   // generic-proxy writes of P become visible to the tensor core
      __syncwarp();
      if (lane == 0) mbar_arrive(bar_p + 8 * set);
      // O = P V is on its way; normalise, convert, store
      if (!mbar_wait(bar_o + 8 * set, sph, abort_flag)) {
        raise_abort(abort_flag, p.status, DEV_WAIT_TMEM_FULL);
        break;
      }
      tc_fence_after();
      const float inv = 1.f / sum;
      uint32_t w[32];
      tmem_ld_x32(t_o, ra);
      tmem_ld_x32(t_o + 32, rb);
      tmem_ld_wait();
#pragma unroll
      for (int u = 0; u < 32; u += 2) {
        __nv_bfloat162 h0 = __floats2bfloat162_rn(__uint_as_float(ra[u]) * inv, __uint_as_float(ra[u + 1]) * inv);
        __nv_bfloat162 h1 = __floats2bfloat162_rn(__uint_as_float(rb[u]) * inv, __uint_as_float(rb[u + 1]) * inv);
        w[u >> 1] = *reinterpret_cast<uint32_t *>(&h0);
        w[16 + (u >> 1)] = *reinterpret_cast<uint32_t *>(&h1);
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar_acc + 8 * set);   // S and O of this set may be overwritten
      // the second MMA has finished (bar_o), so tile 0 of P is free: it stages the 128 x 64 output tile
#pragma unroll
      for (int u = 0; u < 8; ++u)
        asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(my_p + ((u ^ swz) << 4)), "r"(w[4 * u]), "r"(w[4 * u + 1]),
                     "r"(w[4 * u + 2]), "r"(w[4 * u + 3])
                     : "memory");
      fence_proxy_async();
      __syncwarp();
      if (lane == 0) {
        tma_store_4d(&tm_out, pa + quad * 32 * 128, 0, h, quad * 32, b);   // this warp's 32 rows; rows past seq are clipped
        bulk_commit_group();
      }
      store_pending = true;
    }
    if (store_pending) {
      if (lane == 0) bulk_wait_read_all();
      __syncwarp();
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}

static PFN_cuTensorMapEncodeTiled_v12000 get_encode_att() {
  static PFN_cuTensorMapEncodeTiled_v12000 fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void *sym = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &q) == cudaSuccess && q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<PFN_cuTensorMapEncodeTiled_v12000>(sym);
  });
  return fn;
}

// 4-D bf16 tensor (d0 innermost) with a box of 64 x 1 x rows x 1 elements and the 128B swizzle.
static int encode_4d(CUtensorMap *tm, const void *base, uint64_t d0, uint64_t d1, uint64_t d2, uint64_t d3, uint64_t s1, uint64_t s2,
                     uint64_t s3, uint32_t box_rows) {
  auto enc = get_encode_att();
  if (!enc) return fail(SOFIE_B200_ERR_NO_DEVICE, "cuTensorMapEncodeTiled entry point not available");
  cuuint64_t dims[4] = {d0, d1, d2, d3};
  cuuint64_t strides[3] = {s1, s2, s3};
  cuuint32_t box[4] = {64, 1, box_rows, 1};
  cuuint32_t estr[4] = {1, 1, 1, 1};
  CUresult r = enc(tm, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<void *>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                   CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(SOFIE_B200_ERR_CUDA, "attention: cuTensorMapEncodeTiled failed (%d)", (int)r);
  return 0;
}

}  // namespace sb200

using namespace sb200;

namespace sb200 {
// Q, K, V: [batch, seq, heads, 64] bf16 with row pitches ldq / ldk / ldv elements (a row = one token); out: [batch, seq, heads * 64].
static int attention_launch(sofie_b200_ctx *ctx, const void *q, const void *k, const void *v, int64_t ldq, int64_t ldk, int64_t ldv, void *out,
                            int64_t batch, int64_t seq, int32_t heads, float scale) {
  const uint64_t dh = 64, es = 2, H = (uint64_t)heads, S = (uint64_t)seq, B = (uint64_t)batch;
  CUtensorMap tm_q, tm_k, tm_v, tm_out;
  // one box = the (up to) 128 token rows of one head
  int rc;
  if ((rc = encode_4d(&tm_q, q, dh, H, S, B, dh * es, (uint64_t)ldq * es, S * (uint64_t)ldq * es, 128))) return rc;
  if ((rc = encode_4d(&tm_k, k, dh, H, S, B, dh * es, (uint64_t)ldk * es, S * (uint64_t)ldk * es, 128))) return rc;
  if ((rc = encode_4d(&tm_v, v, dh, H, S, B, dh * es, (uint64_t)ldv * es, S * (uint64_t)ldv * es, 128))) return rc;
  // out [batch, seq, heads, 64]: one box = 32 token rows of one head (one epilogue warp)
  if ((rc = encode_4d(&tm_out, out, dh, H, S, B, dh * es, H * dh * es, S * H * dh * es, 32))) return rc;
  SB_CUDA(cudaFuncSetAttribute(attention_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, ATT_SMEM));   // per device
  AttnParams p{};
  p.batch = (int)batch; p.seq = (int)seq; p.heads = heads;
  p.pairs = (long long)batch * heads;
  p.scale_log2e = scale * 1.4426950408889634f;
  p.status = ctx->d_status;
  const long long grid = p.pairs < ctx->sm_count ? p.pairs : ctx->sm_count;
  attention_kernel<<<dim3((unsigned)grid), dim3(ATT_THREADS), ATT_SMEM, ctx->stream>>>(tm_q, tm_k, tm_v, tm_out, p);
  SB_CUDA(cudaGetLastError());
  ctx->launches++;
  return 0;
}

// [B, S, ld] rows holding [H, D] -> [B, H, S, D] (gather = true) or back (gather = false, ld = H * D)
template <class T>
__global__ void __launch_bounds__(256) heads_layout_kernel(const T *__restrict__ src, T *__restrict__ dst, long long B, long long H, long long S,
                                                           long long D, long long ld, bool gather) {
  const long long total = B * H * S * D;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const long long d = i % D, s = (i / D) % S, h = (i / (D * S)) % H, b = i / (D * S * H);
    const long long folded = (b * S + s) * ld + h * D + d;
    if (gather) dst[i] = src[folded];
    else dst[folded] = src[i];
  }
}
static int heads_layout(sofie_b200_ctx *ctx, const void *src, void *dst, int es, long long B, long long H, long long S, long long D, long long ld,
                        bool gather) {
  const long long total = B * H * S * D;
  const unsigned grid = (unsigned)std::min<long long>((total + 255) / 256, (long long)ctx->sm_count * 16);
  if (es == 4) heads_layout_kernel<uint32_t><<<grid, 256, 0, ctx->stream>>>((const uint32_t *)src, (uint32_t *)dst, B, H, S, D, ld, gather);
  else heads_layout_kernel<uint16_t><<<grid, 256, 0, ctx->stream>>>((const uint16_t *)src, (uint16_t *)dst, B, H, S, D, ld, gather);
  SB_CUDA(cudaGetLastError());
  ctx->launches++;
  return 0;
}
}  // namespace sb200

struct sofie_b200_sdpa_plan {
  sofie_b200_ctx *ctx = nullptr;
  sofie_b200_sdpa_desc d{};
  float scale = 0.f;
  int fused = 0;                                   // the tcgen05 attention kernel applies
  sofie_b200_gemm_plan *qk = nullptr, *pv = nullptr;   // chain: scores and weighted sum, batched over (batch, head)
  int64_t off_q = 0, off_k = 0, off_v = 0, off_s = 0, off_o = 0, bytes = 0;   // workspace regions
};

extern "C" {

int sofie_b200_sdpa_plan_create(sofie_b200_ctx *ctx, const sofie_b200_sdpa_desc *desc, sofie_b200_sdpa_plan **out) {
  if (!ctx || !desc || !out) return fail(SOFIE_B200_ERR_INVALID, "sdpa_plan_create: NULL argument");
  *out = nullptr;
  sofie_b200_sdpa_desc d = *desc;
  if (d.batch < 0 || d.heads < 1 || d.seq < 0 || d.head_dim < 1) return fail(SOFIE_B200_ERR_INVALID, "sdpa_plan_create: bad extent");
  if (d.v_head_dim == 0) d.v_head_dim = d.head_dim;
  if (d.dtype != SOFIE_B200_F32 && d.dtype != SOFIE_B200_BF16) return fail(SOFIE_B200_ERR_INVALID, "sdpa_plan_create: type %d not supported (F32, BF16)", d.dtype);
  if (!d.folded && (d.ldq || d.ldk || d.ldv)) return fail(SOFIE_B200_ERR_INVALID, "sdpa_plan_create: row pitches belong to the folded layout");
  if (d.ldq == 0) d.ldq = d.heads * d.head_dim;
  if (d.ldk == 0) d.ldk = d.heads * d.head_dim;
  if (d.ldv == 0) d.ldv = d.heads * d.v_head_dim;
  if (d.ldq < d.heads * d.head_dim || d.ldk < d.heads * d.head_dim || d.ldv < d.heads * d.v_head_dim)
    return fail(SOFIE_B200_ERR_INVALID, "sdpa_plan_create: a row pitch is smaller than heads * head size");
  sofie_b200_sdpa_plan *p = new sofie_b200_sdpa_plan();
  p->ctx = ctx; p->d = d;
  p->scale = d.scale != 0.f ? d.scale : 1.f / sqrtf((float)d.head_dim);
  const int es = dtype_size(d.dtype);
  p->fused = d.dtype == SOFIE_B200_BF16 && d.folded && !d.has_mask && d.head_dim == 64 && d.v_head_dim == 64 && d.seq <= 128 &&
             (d.ldq * es) % 16 == 0 && (d.ldk * es) % 16 == 0 && (d.ldv * es) % 16 == 0 && d.batch * d.heads < 0x7fffffffLL;
  if (p->fused || d.batch == 0 || d.seq == 0) { *out = p; return 0; }
  // chain: [B,H,S,D] operands (gathered from the folded layout into the workspace), scores [B*H, S, S], output
  const int64_t bh = d.batch * d.heads;
  auto region = [&](int64_t elems) { const int64_t o = p->bytes; p->bytes += (elems * es + 255) / 256 * 256; return o; };
  if (d.folded) { p->off_q = region(bh * d.seq * d.head_dim); p->off_k = region(bh * d.seq * d.head_dim); p->off_v = region(bh * d.seq * d.v_head_dim);
                  p->off_o = region(bh * d.seq * d.v_head_dim); }
  p->off_s = region(bh * d.seq * d.seq);
  sofie_b200_gemm_desc g{};
  g.M = d.seq; g.N = d.seq; g.K = d.head_dim; g.batch = bh; g.trans_b = 1; g.ab_dtype = g.y_dtype = d.dtype;
  g.stride_a = g.stride_b = d.seq * d.head_dim; g.stride_y = g.stride_c = d.seq * d.seq; g.precise = 1;
  int rc = sofie_b200_gemm_plan_create(ctx, &g, &p->qk);
  if (rc) { delete p; return rc; }
  g.N = d.v_head_dim; g.K = d.seq; g.trans_b = 0;
  g.stride_a = d.seq * d.seq; g.stride_b = g.stride_y = d.seq * d.v_head_dim; g.stride_c = 0;
  rc = sofie_b200_gemm_plan_create(ctx, &g, &p->pv);
  if (rc) { sofie_b200_gemm_plan_destroy(p->qk); delete p; return rc; }
  *out = p;
  return 0;
}

int sofie_b200_sdpa_plan_destroy(sofie_b200_sdpa_plan *plan) {
  if (!plan) return 0;
  if (plan->qk) sofie_b200_gemm_plan_destroy(plan->qk);
  if (plan->pv) sofie_b200_gemm_plan_destroy(plan->pv);
  delete plan;
  return 0;
}

const char *sofie_b200_sdpa_plan_kernel(const sofie_b200_sdpa_plan *plan) { return !plan ? "" : (plan->fused ? "attention" : "chain"); }

int64_t sofie_b200_sdpa_workspace_bytes(const sofie_b200_sdpa_plan *plan) { return plan ? plan->bytes : 0; }

int sofie_b200_sdpa_enqueue(sofie_b200_sdpa_plan *plan, const void *q, const void *k, const void *v, const void *mask, void *y, void *workspace) {
  if (!plan) return fail(SOFIE_B200_ERR_INVALID, "sdpa_enqueue: plan is NULL");
  const sofie_b200_sdpa_desc &d = plan->d;
  if (d.batch == 0 || d.seq == 0) return 0;
  if (!q || !k || !v || !y) return fail(SOFIE_B200_ERR_INVALID, "sdpa_enqueue: NULL tensor pointer");
  if ((d.has_mask != 0) != (mask != nullptr)) return fail(SOFIE_B200_ERR_INVALID, "sdpa_enqueue: the mask pointer does not match the plan");
  sofie_b200_ctx *ctx = plan->ctx;
  SB_CUDA(cudaSetDevice(ctx->device));
  if (plan->fused) {
    if (((uintptr_t)q % 16) || ((uintptr_t)k % 16) || ((uintptr_t)v % 16) || ((uintptr_t)y % 16))
      return fail(SOFIE_B200_ERR_INVALID, "sdpa_enqueue: tensors must be 16-byte aligned");
    return attention_launch(ctx, q, k, v, d.ldq, d.ldk, d.ldv, y, d.batch, d.seq, (int32_t)d.heads, plan->scale);
  }
  if (!workspace || ((uintptr_t)workspace % 256)) return fail(SOFIE_B200_ERR_INVALID, "sdpa_enqueue: this plan needs a 256-byte aligned workspace");
  const int es = dtype_size(d.dtype);
  char *ws = static_cast<char *>(workspace);
  const void *q4 = q, *k4 = k, *v4 = v;
  void *o4 = y;
  int rc;
  if (d.folded) {
    if ((rc = heads_layout(ctx, q, ws + plan->off_q, es, d.batch, d.heads, d.seq, d.head_dim, d.ldq, true))) return rc;
    if ((rc = heads_layout(ctx, k, ws + plan->off_k, es, d.batch, d.heads, d.seq, d.head_dim, d.ldk, true))) return rc;
    if ((rc = heads_layout(ctx, v, ws + plan->off_v, es, d.batch, d.heads, d.seq, d.v_head_dim, d.ldv, true))) return rc;
    q4 = ws + plan->off_q; k4 = ws + plan->off_k; v4 = ws + plan->off_v; o4 = ws + plan->off_o;
  }
  void *sc = ws + plan->off_s;
  // scores = scale * Q K^T (+ mask), rounded as the reference's CPU code rounds them (dot * scale, then + mask: ROperator_SDPA.hxx:163-170)
  sofie_b200_epilogue e{};
  e.alpha = plan->scale; e.beta = 1.f; e.out_scale = 1.f;
  if (mask) {
    if (d.dtype != SOFIE_B200_F32) return fail(SOFIE_B200_ERR_INVALID, "sdpa_enqueue: a mask is supported for F32 tensors");
    e.bias_mode = SOFIE_B200_BIAS_FULL_F32; e.bias = mask; e.ldc = d.seq;
  }
  if ((rc = sofie_b200_gemm_enqueue(plan->qk, q4, k4, sc, &e))) return rc;
  if ((rc = sofie_b200_softmax_enqueue(ctx, sc, sc, d.dtype, d.dtype, d.batch * d.heads * d.seq, d.seq, 0))) return rc;
  if ((rc = sofie_b200_gemm_enqueue(plan->pv, sc, v4, o4, nullptr))) return rc;
  if (d.folded) return heads_layout(ctx, o4, y, es, d.batch, d.heads, d.seq, d.v_head_dim, d.heads * d.v_head_dim, false);
  return 0;
}

}  // extern "C"

extern "C" int sofie_b200_attention_enqueue(sofie_b200_ctx *ctx, const void *qkv, void *out, int32_t dtype, int64_t batch, int64_t seq,
                                            int32_t heads, int32_t head_dim, float scale) {
  if (!ctx) return fail(SOFIE_B200_ERR_INVALID, "attention_enqueue: ctx is NULL");
  if (batch == 0 || seq == 0) return 0;
  if (!qkv || !out) return fail(SOFIE_B200_ERR_INVALID, "attention_enqueue: NULL tensor pointer");
  if (dtype != SOFIE_B200_BF16) return fail(SOFIE_B200_ERR_INVALID, "attention_enqueue: only bf16 tensors are supported");
  if (head_dim != 64) return fail(SOFIE_B200_ERR_INVALID, "attention_enqueue: head size %d not supported (64)", head_dim);
  if (seq < 0 || seq > 128) return fail(SOFIE_B200_ERR_INVALID, "attention_enqueue: sequence length %lld not supported (1..128)", (long long)seq);
  if (batch < 0 || heads < 1 || batch > 0x7fffffffLL / heads) return fail(SOFIE_B200_ERR_INVALID, "attention_enqueue: bad batch / heads");
  if (((uintptr_t)qkv % 16) || ((uintptr_t)out % 16)) return fail(SOFIE_B200_ERR_INVALID, "attention_enqueue: tensors must be 16-byte aligned");
  SB_CUDA(cudaSetDevice(ctx->device));
  // qkv [batch, seq, 3, heads, 64]: Q, K and V are the three column blocks of a row of 3 * heads * 64 elements
  const int64_t hd = (int64_t)heads * 64;
  const char *base = static_cast<const char *>(qkv);
  return attention_launch(ctx, base, base + hd * 2, base + 2 * hd * 2, 3 * hd, 3 * hd, 3 * hd, out, batch, seq, heads, scale);
}
