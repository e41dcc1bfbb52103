// C ABI: context, error reporting and the contraction plan / enqueue entry points.
#include <stdarg.h>
#include <stdlib.h>
#include <string.h>

#include "gemm.cuh"

namespace sb200 {

static thread_local char g_err[512] = "";

void set_error(const char *fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
}

int fail(int status, const char *fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
  return status;
}

int ensure_stage(sofie_b200_ctx *ctx, int idx, size_t bytes) {
  if (ctx->stage_bytes[idx] >= bytes) return 0;
  if (ctx->stage[idx]) SB_CUDA(cudaFree(ctx->stage[idx]));
  ctx->stage[idx] = nullptr;
  ctx->stage_bytes[idx] = 0;
  SB_CUDA(cudaMalloc(&ctx->stage[idx], bytes));
  ctx->stage_bytes[idx] = bytes;
  return 0;
}

static const char *kDeviceWait[] = {"ok", "TMA producer: no free shared-memory stage", "MMA issuer: stage never filled",
                                    "MMA issuer: accumulator never drained", "epilogue: accumulator never completed"};

}  // namespace sb200

using namespace sb200;

namespace sb200 {
// A TF32 plan over already split K-major operands (desc.K = 3*ks products; operands stored [hi | lo], lda = ldb = 2*ks)
// that runs the chunk-promotion kernel.
// Returns 1 when the tensor path does not apply to the shape.
int gemm_plan_create_promote(sofie_b200_ctx *ctx, const sofie_b200_gemm_desc &g, sofie_b200_gemm_plan **out) {
  *out = nullptr;
  sofie_b200_gemm_plan *in = new sofie_b200_gemm_plan();
  in->ctx = ctx;
  in->desc = g;
  in->promote = 1;   // sum short K chunks in registers: the tensor core's own fp32 adds truncate
  in->k_store = g.K / 3 * 2;
  const int rc = umma_plan_init(in);
  if (rc) { delete in; return rc; }
  in->use_umma = 1;
  *out = in;
  return 0;
}
// An implicit convolution as a contraction: A is the channels-last input read in im2col mode (g.M = output pixels of the
// batch, g.K = R*S*C, g.lda unused), B the filters [g.N, g.K] with K ordered (filter row, filter column, channel).
// Returns 1 when the tensor path does not apply.
int gemm_plan_create_im2col(sofie_b200_ctx *ctx, const sofie_b200_gemm_desc &g, const Im2colDesc &ic, sofie_b200_gemm_plan **out) {
  *out = nullptr;
  sofie_b200_gemm_plan *in = new sofie_b200_gemm_plan();
  in->ctx = ctx;
  in->desc = g;
  in->ic = ic;
  in->kb_bytes = (ic.C * dtype_size(g.ab_dtype)) % 128 == 0 ? 128 : 64;
  const int rc = umma_plan_init(in);
  if (rc) { delete in; return rc; }
  in->use_umma = 1;
  *out = in;
  return 0;
}
// The fp32-accurate implicit convolution: A is a channels-last tensor of TF32 pairs ([N, H, W, 2C]: hi channels, then lo
// channels) read in im2col mode, B the filters [g.N, 2 * R*S*C] as hi | lo with K ordered (filter row, filter column,
// channel), g.K = 3 * R*S*C products.  split_out: Y is written as TF32 pairs too (g.ldy = 2 * g.N).
int gemm_plan_create_promote_im2col(sofie_b200_ctx *ctx, const sofie_b200_gemm_desc &g, const Im2colDesc &ic, int split_out,
                                    sofie_b200_gemm_plan **out) {
  *out = nullptr;
  sofie_b200_gemm_plan *in = new sofie_b200_gemm_plan();
  in->ctx = ctx;
  in->desc = g;
  in->promote = 1;
  in->k_store = g.K / 3 * 2;
  in->ic = ic;
  in->split_out = split_out;
  const int rc = umma_plan_init(in);
  if (rc) { delete in; return rc; }
  in->use_umma = 1;
  *out = in;
  return 0;
}
// Epilogue parameters of a contraction described by `d` writing to Y (for kernels outside this file that apply the
// same fused epilogue: the direct convolution).
int gemm_make_epi(const sofie_b200_gemm_desc &d, void *Y, const sofie_b200_epilogue *ep, EpiParams *o);
}  // namespace sb200

extern "C" {

int sofie_b200_abi_version(void) { return SOFIE_B200_ABI_VERSION; }

const char *sofie_b200_status_string(int status) {
  switch (status) {
    case SOFIE_B200_OK: return "ok";
    case SOFIE_B200_ERR_INVALID: return "invalid argument or unsupported combination";
    case SOFIE_B200_ERR_CUDA: return "CUDA call failed";
    case SOFIE_B200_ERR_DEVICE_WAIT: return "a bounded wait inside a kernel gave up";
    case SOFIE_B200_ERR_NO_DEVICE: return "no usable sm_100 device";
    case SOFIE_B200_ERR_TOO_LARGE: return "size beyond a static limit";
  }
  return "unknown status";
}

const char *sofie_b200_last_error(void) { return g_err; }

int sofie_b200_ctx_create(sofie_b200_ctx **out, int device, void *stream) {
  if (!out) return fail(SOFIE_B200_ERR_INVALID, "ctx_create: out is NULL");
  *out = nullptr;
  int ndev = 0;
  if (cudaGetDeviceCount(&ndev) != cudaSuccess || ndev <= 0) {
    cudaGetLastError();
    return fail(SOFIE_B200_ERR_NO_DEVICE, "ctx_create: no CUDA device visible");
  }
  if (device < 0 || device >= ndev) return fail(SOFIE_B200_ERR_INVALID, "ctx_create: device %d of %d", device, ndev);
  cudaDeviceProp prop;
  SB_CUDA(cudaGetDeviceProperties(&prop, device));
  if (prop.major != 10)
    return fail(SOFIE_B200_ERR_NO_DEVICE, "ctx_create: device %d is sm_%d%d; this library is built for sm_100a only",
                device, prop.major, prop.minor);
  SB_CUDA(cudaSetDevice(device));
  sofie_b200_ctx *ctx = new sofie_b200_ctx();
  ctx->device = device;
  ctx->stream = (cudaStream_t)stream;
  ctx->sm_count = prop.multiProcessorCount;
  if (cudaMalloc(&ctx->d_status, sizeof(int)) != cudaSuccess || cudaMallocHost(&ctx->h_status, sizeof(int)) != cudaSuccess) {
    delete ctx;
    return fail(SOFIE_B200_ERR_CUDA, "ctx_create: allocating the status word failed: %s", cudaGetErrorString(cudaGetLastError()));
  }
  SB_CUDA(cudaMemsetAsync(ctx->d_status, 0, sizeof(int), ctx->stream));
  SB_CUDA(cudaStreamSynchronize(ctx->stream));
  *out = ctx;
  return 0;
}

int sofie_b200_ctx_destroy(sofie_b200_ctx *ctx) {
  if (!ctx) return 0;
  cudaSetDevice(ctx->device);
  for (int i = 0; i < 3; ++i) {
    if (ctx->stage[i]) cudaFree(ctx->stage[i]);
    if (ctx->stage2[i]) cudaFree(ctx->stage2[i]);
  }
  if (ctx->copy_in) cudaStreamDestroy(ctx->copy_in);
  if (ctx->copy_out) cudaStreamDestroy(ctx->copy_out);
  for (int i = 0; i < 2; ++i) {
    if (ctx->ev_in[i]) cudaEventDestroy(ctx->ev_in[i]);
    if (ctx->ev_done[i]) cudaEventDestroy(ctx->ev_done[i]);
    if (ctx->ev_out[i]) cudaEventDestroy(ctx->ev_out[i]);
  }
  for (auto &m : ctx->peer_mappings) cudaIpcCloseMemHandle(m.base);
  if (ctx->d_status) cudaFree(ctx->d_status);
  if (ctx->h_status) cudaFreeHost(ctx->h_status);
  delete ctx;
  return 0;
}

int sofie_b200_ctx_sync(sofie_b200_ctx *ctx) {
  if (!ctx) return fail(SOFIE_B200_ERR_INVALID, "ctx_sync: ctx is NULL");
  SB_CUDA(cudaMemcpyAsync(ctx->h_status, ctx->d_status, sizeof(int), cudaMemcpyDeviceToHost, ctx->stream));
  SB_CUDA(cudaStreamSynchronize(ctx->stream));
  int s = *ctx->h_status;
  if (s != 0) {
    cudaMemsetAsync(ctx->d_status, 0, sizeof(int), ctx->stream);
    cudaStreamSynchronize(ctx->stream);
    return fail(SOFIE_B200_ERR_DEVICE_WAIT, "device status %d: %s", s, (s > 0 && s < 5) ? kDeviceWait[s] : "unknown");
  }
  return 0;
}

int64_t sofie_b200_ctx_launch_count(const sofie_b200_ctx *ctx) { return ctx ? ctx->launches : 0; }

// ---------------------------------------------------------------------------------------

int sofie_b200_gemm_plan_create(sofie_b200_ctx *ctx, const sofie_b200_gemm_desc *desc, sofie_b200_gemm_plan **out) {
  if (!ctx || !desc || !out) return fail(SOFIE_B200_ERR_INVALID, "gemm_plan_create: NULL argument");
  *out = nullptr;
  sofie_b200_gemm_desc d = *desc;
  if (d.M < 0 || d.N < 0 || d.K < 0) return fail(SOFIE_B200_ERR_INVALID, "gemm_plan_create: negative extent");
  if (d.batch < 1) d.batch = 1;
  if (d.lda == 0) d.lda = d.trans_a ? d.M : d.K;
  if (d.ldb == 0) d.ldb = d.trans_b ? d.K : d.N;
  if (d.ldy == 0) d.ldy = d.N;
  if (d.lda < (d.trans_a ? d.M : d.K) || d.ldb < (d.trans_b ? d.K : d.N) || d.ldy < d.N)
    return fail(SOFIE_B200_ERR_INVALID, "gemm_plan_create: a row pitch is smaller than the row (lda %lld ldb %lld ldy %lld)",
                (long long)d.lda, (long long)d.ldb, (long long)d.ldy);
  switch (d.ab_dtype) {
    case SOFIE_B200_F32: case SOFIE_B200_BF16: case SOFIE_B200_I8: case SOFIE_B200_F8E4M3: break;
    default: return fail(SOFIE_B200_ERR_INVALID, "gemm_plan_create: operand type %d not supported", d.ab_dtype);
  }
  const bool int_acc = d.ab_dtype == SOFIE_B200_I8;
  switch (d.y_dtype) {
    case SOFIE_B200_F32: case SOFIE_B200_BF16: case SOFIE_B200_I8: case SOFIE_B200_U8: break;
    case SOFIE_B200_I32:
      if (!int_acc) return fail(SOFIE_B200_ERR_INVALID, "gemm_plan_create: I32 output needs I8 operands");
      break;
    default: return fail(SOFIE_B200_ERR_INVALID, "gemm_plan_create: output type %d not supported", d.y_dtype);
  }
  SB_CUDA(cudaSetDevice(ctx->device));
  sofie_b200_gemm_plan *plan = new sofie_b200_gemm_plan();
  plan->ctx = ctx;
  plan->use_umma = 0;
  // fp32 operands: the single-pass TF32 tensor path only on request; otherwise fp32 FMA.
  const bool want_umma = !(d.ab_dtype == SOFIE_B200_F32 && d.precise != 0);
  // A constant B stored [K,N] becomes a K-major copy when the tensor-core kernel can take it (K rows of 16-byte multiples,
  // dense source): one TMA box per K block instead of one per 128 bytes of columns.
  const int es_ab = dtype_size(d.ab_dtype);
  if ((d.flags & SOFIE_B200_GEMM_B_CONSTANT) && want_umma && !d.trans_b && d.M > 0 && d.N > 0 && d.K > 0 && (d.K * es_ab) % 16 == 0 &&
      d.ldb == d.N && (d.batch == 1 || d.stride_b == 0 || d.stride_b == d.K * d.N)) {
    const bool bcast = d.batch > 1 && d.stride_b == 0;
    const size_t bytes = (size_t)(bcast ? 1 : d.batch) * d.N * d.K * es_ab;
    if (cudaMalloc(&plan->b_kmajor, bytes) == cudaSuccess) {
      plan->b_src_ld = d.ldb; plan->b_src_stride = d.stride_b;
      d.trans_b = 1; d.ldb = d.K;
    } else {
      cudaGetLastError();   // no room for the copy: B is read as it is stored
      plan->b_kmajor = nullptr;
    }
  }
  plan->desc = d;
  if (want_umma && d.M > 0 && d.N > 0 && d.K > 0) {
    int rc = umma_plan_init(plan);
    if (rc < 0) { if (plan->b_kmajor) cudaFree(plan->b_kmajor); delete plan; return rc; }
    plan->use_umma = (rc == 0);
  }
  // fp32 at fp32 accuracy: large problems go to the tensor cores as 3xTF32 (gemm_split.cu), the rest to fp32 FMA
  if (d.ab_dtype == SOFIE_B200_F32 && d.precise != 0 && d.M > 0 && d.N > 0 && d.K > 0 && d.batch <= 65535 &&
      2.0 * (double)d.M * (double)d.N * (double)d.K * (double)d.batch >= SPLIT_MIN_FLOPS) {
    const long long ks = split_ks(d.K);
    sofie_b200_gemm_desc g = d;
    const bool a_bcast = d.batch > 1 && d.stride_a == 0, b_bcast = d.batch > 1 && d.stride_b == 0;
    g.K = 3 * ks; g.trans_a = 0; g.trans_b = 1; g.lda = 2 * ks; g.ldb = 2 * ks; g.precise = 0;
    g.stride_a = a_bcast ? 0 : d.M * 2 * ks;
    g.stride_b = b_bcast ? 0 : d.N * 2 * ks;
    sofie_b200_gemm_plan *in = nullptr;
    int rc = gemm_plan_create_promote(ctx, g, &in);
    if (rc < 0) { delete plan; return rc; }
    if (rc == 0) {
      const size_t abytes = (size_t)(a_bcast ? 1 : d.batch) * d.M * 2 * ks * sizeof(float);
      const size_t bbytes = (size_t)(b_bcast ? 1 : d.batch) * d.N * 2 * ks * sizeof(float);
      if (cudaMalloc(&plan->split_a, abytes) != cudaSuccess || cudaMalloc(&plan->split_b, bbytes) != cudaSuccess) {
        cudaGetLastError();
        if (plan->split_a) cudaFree(plan->split_a);
        plan->split_a = nullptr;
        delete in;   // not enough memory for the split operands: stay on the fp32 FMA kernel
      } else {
        plan->inner = in;
        plan->ks = ks;
      }
    }
  }
  *out = plan;
  return 0;
}

int sofie_b200_gemm_plan_destroy(sofie_b200_gemm_plan *plan) {
  if (!plan) return 0;
  // the plan holds no reference into the ctx that needs undoing: a plan may be destroyed after its ctx
  if (plan->split_a) cudaFree(plan->split_a);
  if (plan->split_b) cudaFree(plan->split_b);
  if (plan->b_kmajor) cudaFree(plan->b_kmajor);
  delete plan->inner;
  delete plan;
  return 0;
}

const char *sofie_b200_gemm_plan_kernel(const sofie_b200_gemm_plan *plan) {
  if (!plan) return "";
  if (plan->ic.on && plan->promote) return "umma3x_im2col";
  if (plan->inner || (plan->promote && plan->use_umma)) return "umma3x";
  if (plan->ic.on) return "umma_im2col";
  return plan->use_umma ? "umma" : "simt";
}

static int make_epi(const sofie_b200_gemm_desc &d, void *Y, const sofie_b200_epilogue *ep, EpiParams *o) {
  memset(o, 0, sizeof(*o));
  o->Y = Y;
  o->ldy = d.ldy;
  o->stride_y = d.stride_y;
  o->stride_c = d.stride_c;
  o->stride_r = d.stride_r;
  o->alpha = 1.f; o->beta = 1.f; o->out_scale = 1.f;
  o->y_dtype = d.y_dtype;
  o->acc_is_int = d.ab_dtype == SOFIE_B200_I8;
  o->params_aligned = 1; o->residual_aligned = 1; o->fast = 1;
  if (ep) {
    o->row_scale = ep->row_scale;
    o->col_scale = ep->col_scale;
    o->alpha = ep->alpha;
    o->beta = ep->beta;
    o->bias_mode = ep->bias_mode;
    o->bias = ep->bias;
    o->ldc = ep->ldc ? ep->ldc : d.N;
    o->residual = ep->residual;
    o->residual_dtype = ep->residual_dtype;
    o->ldr = ep->ldr ? ep->ldr : d.N;
    o->act = ep->act;
    o->act_alpha = ep->act_alpha;
    o->out_scale = ep->out_scale == 0.f ? 1.f : ep->out_scale;
    o->out_zp = ep->out_zero_point;
    o->params_aligned = ((uintptr_t)ep->col_scale % 16 == 0) && ((uintptr_t)ep->bias % 16 == 0);
    const int rs_ = dtype_size(ep->residual_dtype);
    // 0: no alignment known, 1: base, pitch and batch stride are multiples of 16 bytes, 2: of 32 bytes
    o->residual_aligned = 0;
    for (int a = 16; a <= 32; a *= 2)
      if (((uintptr_t)ep->residual % a == 0) && ((o->ldr * rs_) % a == 0) && ((o->stride_r * rs_) % a == 0)) o->residual_aligned = a / 16;
    o->fast = o->params_aligned && ep->bias_mode != SOFIE_B200_BIAS_FULL_F32;
    if (ep->bias_mode != SOFIE_B200_BIAS_NONE && !ep->bias)
      return fail(SOFIE_B200_ERR_INVALID, "gemm_enqueue: bias_mode %d with a NULL bias", ep->bias_mode);
    if ((ep->bias_mode == SOFIE_B200_BIAS_COL_I32 || ep->bias_mode == SOFIE_B200_BIAS_ROW_I32) && !o->acc_is_int)
      return fail(SOFIE_B200_ERR_INVALID, "gemm_enqueue: an int32 bias needs int8 operands");
    if (ep->bias_mode < 0 || ep->bias_mode > SOFIE_B200_BIAS_ROW_I32)
      return fail(SOFIE_B200_ERR_INVALID, "gemm_enqueue: bias_mode %d unknown", ep->bias_mode);
    if (ep->act < 0 || ep->act > SOFIE_B200_ACT_SIGMOID)
      return fail(SOFIE_B200_ERR_INVALID, "gemm_enqueue: activation %d unknown", ep->act);
  }
  return 0;
}

}  // extern "C"
namespace sb200 {
int gemm_make_epi(const sofie_b200_gemm_desc &d, void *Y, const sofie_b200_epilogue *ep, EpiParams *o) { return make_epi(d, Y, ep, o); }
}
extern "C" {

int sofie_b200_gemm_enqueue(sofie_b200_gemm_plan *plan, const void *A, const void *B, void *Y,
                            const sofie_b200_epilogue *ep) {
  if (!plan) return fail(SOFIE_B200_ERR_INVALID, "gemm_enqueue: plan is NULL");
  const sofie_b200_gemm_desc &d = plan->desc;
  if (d.M == 0 || d.N == 0) return 0;  // empty output: nothing to enqueue
  if (!A || !B || !Y) return fail(SOFIE_B200_ERR_INVALID, "gemm_enqueue: NULL tensor pointer");
  EpiParams e;
  int rc = make_epi(plan->desc, Y, ep, &e);
  if (rc) return rc;
  SB_CUDA(cudaSetDevice(plan->ctx->device));
  if (plan->inner) {
    sofie_b200_ctx *ctx = plan->ctx;
    const bool a_bcast = d.batch > 1 && d.stride_a == 0, b_bcast = d.batch > 1 && d.stride_b == 0;
    if ((rc = split2_enqueue(ctx, (const float *)A, plan->split_a, d.M, d.K, plan->ks, d.lda, a_bcast ? 1 : d.batch, d.stride_a, d.trans_a ? 1 : 0))) return rc;
    // a constant B is split once per address
    if (!((d.flags & SOFIE_B200_GEMM_B_CONSTANT) && plan->split_b_src == B)) {
      if ((rc = split2_enqueue(ctx, (const float *)B, plan->split_b, d.N, d.K, plan->ks, d.ldb, b_bcast ? 1 : d.batch, d.stride_b, d.trans_b ? 0 : 1))) return rc;
      plan->split_b_src = (d.flags & SOFIE_B200_GEMM_B_CONSTANT) ? B : nullptr;
    }
    return umma_enqueue(plan->inner, plan->split_a, plan->split_b, e);
  }
  if (plan->b_kmajor) {
    if (plan->b_kmajor_src != B) {   // first enqueue, or the weight moved: [batch][K,N] -> [batch][N,K]
      const bool bcast = d.batch > 1 && d.stride_b == 0;
      const int64_t shape[3] = {bcast ? 1 : d.batch, d.K, d.N};
      const int32_t perm[3] = {0, 2, 1};
      if ((rc = sofie_b200_transpose_enqueue(plan->ctx, B, plan->b_kmajor, d.ab_dtype, 3, shape, perm))) return rc;
      plan->b_kmajor_src = B;
    }
    if (plan->use_umma) return umma_enqueue(plan, A, plan->b_kmajor, e);
    return simt_enqueue(plan, A, plan->b_kmajor, e);
  }
  if (plan->use_umma && d.K > 0) return umma_enqueue(plan, A, B, e);
  return simt_enqueue(plan, A, B, e);
}

int sofie_b200_gemm_enqueue_peers(sofie_b200_gemm_plan *plan, const void *A, const void *B, void *Y, void *const *peer_Y, int32_t n_peers,
                                  const sofie_b200_epilogue *ep) {
  if (n_peers == 0) return sofie_b200_gemm_enqueue(plan, A, B, Y, ep);
  if (!plan) return fail(SOFIE_B200_ERR_INVALID, "gemm_enqueue_peers: plan is NULL");
  const sofie_b200_gemm_desc &d = plan->desc;
  if (n_peers < 0 || n_peers > sb200::UMMA_MAX_PEERS || !peer_Y) return fail(SOFIE_B200_ERR_INVALID, "gemm_enqueue_peers: 0 to %d peer outputs", sb200::UMMA_MAX_PEERS);
  if (d.M == 0 || d.N == 0) return 0;
  if (!A || !B || !Y) return fail(SOFIE_B200_ERR_INVALID, "gemm_enqueue_peers: NULL tensor pointer");
  // every element must leave through a bulk store of a complete row segment (the only store that is repeated per peer):
  // the tensor-core kernel on whole 64-column groups, with the epilogue's fast path
  if (!plan->use_umma || plan->inner || plan->b_kmajor || plan->split_out || d.N % 64 != 0 || d.K <= 0)
    return fail(SOFIE_B200_ERR_INVALID, "gemm_enqueue_peers: needs a plan on the tensor-core kernel with B as stored and N a multiple of 64");
  if (d.ab_dtype == SOFIE_B200_I8 || d.ab_dtype == SOFIE_B200_U8)
    return fail(SOFIE_B200_ERR_INVALID, "gemm_enqueue_peers: floating-point operands only (bf16, f16, FP8, fp32)");
  EpiParams e;
  int rc = make_epi(plan->desc, Y, ep, &e);
  if (rc) return rc;
  if (!e.fast) return fail(SOFIE_B200_ERR_INVALID, "gemm_enqueue_peers: epilogue vectors must be 16-byte aligned and the bias not a full matrix");
  SB_CUDA(cudaSetDevice(plan->ctx->device));
  return umma_enqueue(plan, A, B, e, peer_Y, n_peers);
}

int sofie_b200_gemm_run_host(sofie_b200_gemm_plan *plan, const void *hostA, const void *hostB, void *hostY,
                             const sofie_b200_epilogue *ep) {
  if (!plan || !hostA || !hostB || !hostY) return fail(SOFIE_B200_ERR_INVALID, "gemm_run_host: NULL argument");
  const sofie_b200_gemm_desc &d = plan->desc;
  sofie_b200_ctx *ctx = plan->ctx;
  const size_t es = dtype_size(d.ab_dtype), ys = dtype_size(d.y_dtype);
  auto extent = [](int64_t rows, int64_t ld, int64_t batch, int64_t stride) -> size_t {
    if (batch > 1 && stride != 0) return (size_t)((batch - 1) * stride + rows * ld);
    return (size_t)(rows * ld);
  };
  const size_t a_bytes = extent(d.trans_a ? d.K : d.M, d.lda, d.batch, d.stride_a) * es;
  const size_t b_bytes = extent(d.trans_b ? d.N : d.K, d.ldb, d.batch, d.stride_b) * es;
  const size_t y_bytes = extent(d.M, d.ldy, d.batch, d.stride_y) * ys;
  SB_CUDA(cudaSetDevice(ctx->device));
  int rc;
  if ((rc = ensure_stage(ctx, 0, a_bytes)) || (rc = ensure_stage(ctx, 1, b_bytes)) || (rc = ensure_stage(ctx, 2, y_bytes)))
    return rc;
  SB_CUDA(cudaMemcpyAsync(ctx->stage[0], hostA, a_bytes, cudaMemcpyHostToDevice, ctx->stream));
  SB_CUDA(cudaMemcpyAsync(ctx->stage[1], hostB, b_bytes, cudaMemcpyHostToDevice, ctx->stream));
  rc = sofie_b200_gemm_enqueue(plan, ctx->stage[0], ctx->stage[1], ctx->stage[2], ep);
  if (rc) return rc;
  SB_CUDA(cudaMemcpyAsync(hostY, ctx->stage[2], y_bytes, cudaMemcpyDeviceToHost, ctx->stream));
  return sofie_b200_ctx_sync(ctx);
}

int sofie_b200_gemm_run_host_many(sofie_b200_gemm_plan *plan, int64_t count, const void *const *hostA, const void *const *hostB,
                                  void *const *hostY, const sofie_b200_epilogue *ep) {
  if (!plan || count < 0 || (count > 0 && (!hostA || !hostB || !hostY))) return fail(SOFIE_B200_ERR_INVALID, "gemm_run_host_many: NULL argument");
  if (count == 0) return 0;
  const sofie_b200_gemm_desc &d = plan->desc;
  sofie_b200_ctx *ctx = plan->ctx;
  const size_t es = dtype_size(d.ab_dtype), ys = dtype_size(d.y_dtype);
  auto extent = [](int64_t rows, int64_t ld, int64_t batch, int64_t stride) -> size_t {
    if (batch > 1 && stride != 0) return (size_t)((batch - 1) * stride + rows * ld);
    return (size_t)(rows * ld);
  };
  const size_t bytes[3] = {extent(d.trans_a ? d.K : d.M, d.lda, d.batch, d.stride_a) * es,
                           extent(d.trans_b ? d.N : d.K, d.ldb, d.batch, d.stride_b) * es, extent(d.M, d.ldy, d.batch, d.stride_y) * ys};
  SB_CUDA(cudaSetDevice(ctx->device));
  int rc;
  for (int i = 0; i < 3; ++i) {
    if ((rc = ensure_stage(ctx, i, bytes[i]))) return rc;
    if (ctx->stage2_bytes[i] < bytes[i]) {
      if (ctx->stage2[i]) SB_CUDA(cudaFree(ctx->stage2[i]));
      ctx->stage2[i] = nullptr; ctx->stage2_bytes[i] = 0;
      SB_CUDA(cudaMalloc(&ctx->stage2[i], bytes[i]));
      ctx->stage2_bytes[i] = bytes[i];
    }
  }
  if (!ctx->copy_in) {
    SB_CUDA(cudaStreamCreateWithFlags(&ctx->copy_in, cudaStreamNonBlocking));
    SB_CUDA(cudaStreamCreateWithFlags(&ctx->copy_out, cudaStreamNonBlocking));
    for (int i = 0; i < 2; ++i) {
      SB_CUDA(cudaEventCreateWithFlags(&ctx->ev_in[i], cudaEventDisableTiming));
      SB_CUDA(cudaEventCreateWithFlags(&ctx->ev_done[i], cudaEventDisableTiming));
      SB_CUDA(cudaEventCreateWithFlags(&ctx->ev_out[i], cudaEventDisableTiming));
    }
  }
  // the copy streams start after whatever the compute stream has queued so far (earlier users of the staging buffers)
  SB_CUDA(cudaEventRecord(ctx->ev_done[0], ctx->stream));
  SB_CUDA(cudaStreamWaitEvent(ctx->copy_in, ctx->ev_done[0], 0));
  SB_CUDA(cudaStreamWaitEvent(ctx->copy_out, ctx->ev_done[0], 0));
  for (int64_t i = 0; i < count; ++i) {
    if (!hostA[i] || !hostB[i] || !hostY[i]) return fail(SOFIE_B200_ERR_INVALID, "gemm_run_host_many: NULL operand %lld", (long long)i);
    const int s = (int)(i & 1);
    void *dA = s ? ctx->stage2[0] : ctx->stage[0], *dB = s ? ctx->stage2[1] : ctx->stage[1], *dY = s ? ctx->stage2[2] : ctx->stage[2];
    if (i >= 2) SB_CUDA(cudaStreamWaitEvent(ctx->copy_in, ctx->ev_done[s], 0));   // the contraction two back has read this set
    SB_CUDA(cudaMemcpyAsync(dA, hostA[i], bytes[0], cudaMemcpyHostToDevice, ctx->copy_in));
    SB_CUDA(cudaMemcpyAsync(dB, hostB[i], bytes[1], cudaMemcpyHostToDevice, ctx->copy_in));
    SB_CUDA(cudaEventRecord(ctx->ev_in[s], ctx->copy_in));
    SB_CUDA(cudaStreamWaitEvent(ctx->stream, ctx->ev_in[s], 0));
    if (i >= 2) SB_CUDA(cudaStreamWaitEvent(ctx->stream, ctx->ev_out[s], 0));    // its Y has left for the host
    if ((rc = sofie_b200_gemm_enqueue(plan, dA, dB, dY, ep))) return rc;
    SB_CUDA(cudaEventRecord(ctx->ev_done[s], ctx->stream));
    SB_CUDA(cudaStreamWaitEvent(ctx->copy_out, ctx->ev_done[s], 0));
    SB_CUDA(cudaMemcpyAsync(hostY[i], dY, bytes[2], cudaMemcpyDeviceToHost, ctx->copy_out));
    SB_CUDA(cudaEventRecord(ctx->ev_out[s], ctx->copy_out));
  }
  SB_CUDA(cudaStreamSynchronize(ctx->copy_out));
  SB_CUDA(cudaStreamSynchronize(ctx->copy_in));
  return sofie_b200_ctx_sync(ctx);
}

}  // extern "C"
