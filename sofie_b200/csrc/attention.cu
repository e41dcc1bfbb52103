// Fused scaled-dot-product attention for sequences of up to 128 tokens and a head size of 64:
//     out[b, :, h, :] = Softmax(scale * Q K^T) V      for every (batch b, head h) pair,
// reading Q, K and V straight out of the QKV projection's output [batch, seq, 3, heads, 64] and writing the
// layout the output projection reads, [batch, seq, heads * 64].  The scores never leave the SM: the chain
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
attention_kernel(const __grid_constant__ CUtensorMap tm_qkv, const __grid_constant__ CUtensorMap tm_out, const __grid_constant__ AttnParams p) {
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
    prefetch_tensormap(&tm_qkv);
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
        tma_load_4d(dst, &tm_qkv, full, 0, h, 0, b);                               // Q
        tma_load_4d(dst + ATT_TILE, &tm_qkv, full, 0, p.heads + h, 0, b);          // K
        tma_load_4d(dst + 2 * ATT_TILE, &tm_qkv, full, 0, 2 * p.heads + h, 0, b);  // V
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
      float mx = -3.0e38f;
      auto max_of = [&](const uint32_t (&r)[32], int c) {
#pragma unroll
        for (int u = 0; u < 32; ++u) mx = fmaxf(mx, (c + u < p.seq) ? __uint_as_float(r[u]) * p.scale_log2e : -3.0e38f);
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
      const float off = mx;   // maximum of the scaled scores (any sign of the scale)
      float sum = 0.f;
      auto exp_store = [&](const uint32_t (&r)[32], int c) {
        uint32_t w[16];
#pragma unroll
        for (int u = 0; u < 32; u += 2) {
          float e0 = ex2_approx(__fmaf_rn(__uint_as_float(r[u]), p.scale_log2e, -off));
          float e1 = ex2_approx(__fmaf_rn(__uint_as_float(r[u + 1]), p.scale_log2e, -off));
          if (c + u >= p.seq) e0 = 0.f;
          if (c + u + 1 >= p.seq) e1 = 0.f;
          __nv_bfloat162 h2 = __floats2bfloat162_rn(e0, e1);
          sum += __bfloat162float(h2.x) + __bfloat162float(h2.y);   // the sum of what the second MMA will actually read
          w[u >> 1] = *reinterpret_cast<uint32_t *>(&h2);
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
  const uint64_t dh = 64, es = 2, H = (uint64_t)heads, S = (uint64_t)seq, B = (uint64_t)batch;
  CUtensorMap tm_qkv, tm_out;
  // qkv [batch, seq, 3 * heads, 64]: one box = the 128 token rows of one of Q / K / V of one head
  int rc = encode_4d(&tm_qkv, qkv, dh, 3 * H, S, B, dh * es, 3 * H * dh * es, S * 3 * H * dh * es, 128);
  if (rc) return rc;
  // out [batch, seq, heads, 64]: one box = 32 token rows of one head (one epilogue warp)
  rc = encode_4d(&tm_out, out, dh, H, S, B, dh * es, H * dh * es, S * H * dh * es, 32);
  if (rc) return rc;
  SB_CUDA(cudaFuncSetAttribute(attention_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, ATT_SMEM));   // per device
  AttnParams p{};
  p.batch = (int)batch; p.seq = (int)seq; p.heads = heads;
  p.pairs = (long long)batch * heads;
  p.scale_log2e = scale * 1.4426950408889634f;
  p.status = ctx->d_status;
  const long long grid = p.pairs < ctx->sm_count ? p.pairs : ctx->sm_count;
  attention_kernel<<<dim3((unsigned)grid), dim3(ATT_THREADS), ATT_SMEM, ctx->stream>>>(tm_qkv, tm_out, p);
  SB_CUDA(cudaGetLastError());
  ctx->launches++;
  return 0;
}
