/*
 * libsofie_b200 -- C ABI of the B200 (sm_100a) runtime that SOFIE-emitted Session code calls.
 *
 * The reference emits, per Session, an object `sofieBLAS<tagAcc> blas{queue}`
 * (core/src/RModel_ALPAKA.cxx:1138-1141), registers one configuration per contraction at
 * Session construction (`blas.addOperationConfig(m,n,k,lda,ldb,ldc,ta,tb,Epilogue)`,
 * core/src/RModel_ALPAKA.cxx:1334-1341) and then enqueues `blas.gemm / gemmrelu / matmul /
 * gemmStridedBatched` (core/inc/SOFIE/operators/ROperator_Gemm.hxx:931-1098,
 * core/inc/SOFIE/operators/ROperator_Conv.hxx:1039-1094) plus one alpaka kernel per
 * memory-bound operator.  This header is the seam that replaces those calls:
 *
 *   sofie_b200_ctx      <->  the Session's queue + blas object   (one per Session / GPU / stream)
 *   sofie_b200_*_plan   <->  one addOperationConfig entry        (created at Session init)
 *   sofie_b200_*_enqueue<->  one blas.* call or alpaka enqueue   (records work on the stream only)
 *
 * Conventions
 *  - plain pointers and sizes only; all tensors are row-major as ONNX defines them (no
 *    column-major operand swap as in ROperator_Gemm.hxx:997-1016);
 *  - every function returns 0 on success and a negative sofie_b200_status otherwise; nothing
 *    throws across this boundary.  The emitted wrapper turns non-zero into std::runtime_error,
 *    which is the reference's own error convention (core/src/RModel_ALPAKA.cxx:749-752);
 *  - the ctx borrows the CUDA stream and every tensor pointer; it owns only plans, TMA
 *    descriptors, a small status word and (for the *_host helpers) staging buffers;
 *  - enqueue functions never synchronise.  Device-side problems (a bounded wait inside a
 *    kernel that ran out) are written to a status word that sofie_b200_ctx_sync() reads;
 *  - a ctx is thread-compatible, not thread-safe: one ctx per (thread, GPU), as a reference
 *    Session is (core/src/RModel_ALPAKA.cxx:1283-1285).
 */
#ifndef SOFIE_B200_H
#define SOFIE_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define SOFIE_B200_ABI_VERSION 2

typedef enum sofie_b200_status {
  SOFIE_B200_OK = 0,
  SOFIE_B200_ERR_INVALID = -1,     /* bad argument / unsupported combination            */
  SOFIE_B200_ERR_CUDA = -2,        /* a CUDA runtime or driver call failed               */
  SOFIE_B200_ERR_DEVICE_WAIT = -3, /* a bounded wait inside a kernel gave up             */
  SOFIE_B200_ERR_NO_DEVICE = -4,   /* no sm_100 device / driver entry point unavailable  */
  SOFIE_B200_ERR_TOO_LARGE = -5    /* size beyond a documented static limit              */
} sofie_b200_status;

/* Element types.  The reference's ETensorType (core/inc/SOFIE/utils/SOFIE_common.hxx:29-32)
 * names FLOAT, INT8, UINT8, INT32, BFLOAT16; F8E4M3 is the ONNX FLOAT8E4M3FN type (17). */
typedef enum sofie_b200_dtype {
  SOFIE_B200_F32 = 0,
  SOFIE_B200_BF16 = 1,
  SOFIE_B200_I8 = 2,
  SOFIE_B200_F8E4M3 = 3,
  SOFIE_B200_I32 = 4,
  SOFIE_B200_U8 = 5
} sofie_b200_dtype;

/* Activations the reference can attach to a contraction or emits as its own operator:
 * Relu (ROperator_Relu.hxx:47-114), LeakyRelu (ROperator_LeakyRelu.hxx), Gelu erf / tanh
 * forms (ROperator_Gelu.hxx:62-98), Sigmoid (fused after Gemm in LinearWithSigmoid). */
typedef enum sofie_b200_act {
  SOFIE_B200_ACT_NONE = 0,
  SOFIE_B200_ACT_RELU = 1,
  SOFIE_B200_ACT_GELU_ERF = 2,
  SOFIE_B200_ACT_GELU_TANH = 3,
  SOFIE_B200_ACT_LEAKY_RELU = 4,
  SOFIE_B200_ACT_SIGMOID = 5
} sofie_b200_act;

/* How the additive operand C of Gemm is broadcast (ROperator_Gemm.hxx:270-301,578-617). */
typedef enum sofie_b200_bias_mode {
  SOFIE_B200_BIAS_NONE = 0,
  SOFIE_B200_BIAS_COL_F32 = 1,   /* C has shape [N]: one value per output column / channel   */
  SOFIE_B200_BIAS_ROW_F32 = 2,   /* C has shape [M,1]                                         */
  SOFIE_B200_BIAS_SCALAR_F32 = 3,/* C is a scalar                                             */
  SOFIE_B200_BIAS_COL_I32 = 4,   /* int32 bias added to the int32 accumulator (QLinearConv)   */
  SOFIE_B200_BIAS_FULL_F32 = 5,  /* C has shape [M,N] with row pitch ldc, multiplied by beta  */
  SOFIE_B200_BIAS_ROW_I32 = 6    /* int32 bias per output row, added to the int32 accumulator */
} sofie_b200_bias_mode;

/*
 * Fused epilogue of a contraction.  For accumulator value acc at (row i, column j) the
 * kernels evaluate, with every step a separately rounded fp32 operation (no FMA contraction):
 *
 *   a = acc (+ bias_i32[j] / bias_i32[i] as an integer add when bias_mode == COL_I32 / ROW_I32)
 *   v = (float)a
 *   v = v * row_scale[i]          if row_scale
 *   v = v * col_scale[j]          if col_scale
 *   v = v * alpha                 if alpha != 1
 *   v = v + bias                  (COL/ROW/SCALAR) or v + beta * C[i,j]   (FULL)
 *   v = v + residual[i,j]         if residual
 *   v = act(v)
 *   out dtype F32: v;  BF16: round-to-nearest-even;  I32: a (integer accumulators only);
 *   I8/U8: q = rintf(out_scale == 1 ? v : v / out_scale) + out_zero_point, saturated
 *          (ONNX QuantizeLinear / QLinearMatMul rounding: half to even, then saturate).
 *
 * BatchNorm folded into a contraction is expressed as col_scale = gamma/sqrt(var+eps) and
 * a COL_F32 bias = beta_bn - mean*col_scale (+ conv bias * col_scale); the reference computes
 * the same scale at code-generation time (ROperator_BatchNormalization.hxx:100-109).
 */
typedef struct sofie_b200_epilogue {
  const float *row_scale;   /* [M] or NULL                                   */
  const float *col_scale;   /* [N] or NULL                                   */
  float alpha;              /* Gemm alpha; 1 = skip                          */
  float beta;               /* multiplies C when bias_mode == FULL_F32       */
  int32_t bias_mode;        /* sofie_b200_bias_mode                          */
  const void *bias;         /* see bias_mode                                 */
  int64_t ldc;              /* row pitch (elements) of C for FULL_F32        */
  const void *residual;     /* [M,N] added before the activation, or NULL    */
  int32_t residual_dtype;   /* F32 or BF16                                   */
  int64_t ldr;              /* row pitch (elements) of residual              */
  int32_t act;              /* sofie_b200_act                                */
  float act_alpha;          /* LeakyRelu slope                               */
  float out_scale;          /* quantised outputs: divide by this; 1 = skip   */
  int32_t out_zero_point;   /* quantised outputs                             */
} sofie_b200_epilogue;

/*
 * One contraction  Y[b] = epilogue( op(A[b]) * op(B[b]) ),  b = 0..batch-1.
 * Replaces one blas.addOperationConfig registration (RModel_ALPAKA.cxx:1334-1341) and the
 * shape half of blas.gemmStridedBatched (ROperator_Gemm.hxx:991-1065).
 *   op(A) is [M,K]: A is stored [M,K] with row pitch lda, or [K,M] when trans_a.
 *   op(B) is [K,N]: B is stored [K,N] with row pitch ldb, or [N,K] when trans_b
 *   (ONNX Gemm transB; SOFIE's parser also turns a Transpose feeding a MatMul into this flag,
 *   parsers/src/RModelParser_ONNX.cxx:1186-1197).
 * A and B share one element type: F32 (computed as error-compensated 3xTF32 or fp32 FMA, see
 * `precise`), BF16, F8E4M3 (fp32 accumulate) or I8 (int32 accumulate).  A batch stride of 0
 * broadcasts that operand over the batch (a shared weight, ROperator_Gemm.hxx:854-859).
 */
typedef struct sofie_b200_gemm_desc {
  int64_t M, N, K;
  int64_t batch;                 /* >= 1 */
  int32_t trans_a, trans_b;
  int32_t ab_dtype;              /* sofie_b200_dtype of A and B   */
  int32_t y_dtype;               /* sofie_b200_dtype of Y         */
  int64_t lda, ldb, ldy;         /* row pitches in elements       */
  int64_t stride_a, stride_b, stride_y; /* batch strides in elements */
  int64_t stride_c, stride_r;    /* batch strides of FULL_F32 C and of residual */
  int32_t precise;               /* F32 inputs: 1 = fp32-accurate path (default), 0 = single-pass TF32 */
  int32_t flags;                 /* sofie_b200_gemm_flags, 0 = none */
} sofie_b200_gemm_desc;

/* Flags of sofie_b200_gemm_desc.
 *   B_CONSTANT  B is a weight (an ONNX initializer): its contents do not change while its address does not.  The
 *               reference uploads weights once at Session construction (RModel_ALPAKA.cxx:1695-1707) and re-lays
 *               convolution filters in a kernel of their own (ROperator_Conv.hxx:985-997); with this flag a plan
 *               whose B is stored [K,N] keeps a K-major copy ([N,K], allocated at plan creation) that it fills on
 *               the first enqueue and again whenever B's address changes.  The tensor-core kernel then stages every
 *               B slice with one TMA box per K block instead of one per 128 bytes of columns.  Results are identical. */
typedef enum sofie_b200_gemm_flags {
  SOFIE_B200_GEMM_B_CONSTANT = 1,
  /* The plan is meant for sofie_b200_gemm_enqueue_peers: its epilogue stages and stores 128-byte row segments instead of
   * 64-byte ones (twice the staging memory, one pipeline stage less for some shapes).  NVLink carried 128-byte rows at
   * 700 GB/s and scattered 64-byte rows at about 410 GB/s here.  Results are identical. */
  SOFIE_B200_GEMM_WIDE_STORES = 2
} sofie_b200_gemm_flags;

/*
 * Convolution over a whole NCHW batch as one implicit GEMM; replaces the reference's per-image
 * loop of Im2ColKernel + blas.matmul (ROperator_Conv.hxx:985-1103) and its per-call weight
 * re-layout (ROperator_Conv.hxx:985-997).  Shape rules follow ROperator_Conv.hxx:123-262.
 * X is [N,C,H,W]; W is [K, C/groups, R, S]; Y is [N,K,Ho,Wo].
 */
typedef struct sofie_b200_conv_desc {
  int64_t N, C, H, W;
  int64_t K, R, S;
  int32_t pad_top, pad_left, pad_bottom, pad_right;
  int32_t stride_h, stride_w;
  int32_t dil_h, dil_w;
  int32_t groups;
  int32_t x_dtype;               /* F32 or I8 (QLinearConv)   */
  int32_t y_dtype;               /* F32, BF16 or I8           */
  int32_t x_zero_point;          /* I8 input zero point: padding is filled with it */
  int32_t precise;               /* as in sofie_b200_gemm_desc */
  int32_t x_layout;              /* 0: X is [N,C,H,W] (the reference's layout); 1: X is channels-last, [N,H,W,C]      */
  int32_t y_layout;              /* the same for Y (and for a residual in the epilogue).  Channels-last is for       */
                                 /* conv -> conv chains: a generator keeps the chain channels-last and converts at   */
                                 /* its ends; the unfold then needs no layout copy and output pixels, not channels,  */
                                 /* fill the 128 accumulator rows.  x_layout = 1 needs C/groups to be a whole number */
                                 /* of 16-byte vectors.  Both = 1 selects the implicit convolution where it applies  */
                                 /* (sofie_b200_conv_plan_kernel).                                                  */
                                 /* 2: channels-last TF32 pairs, [N,H,W,2C] fp32: for every pixel the C values       */
                                 /* hi = tf32(x) and then the C values lo = tf32(x - hi) (tf32: rounded to a 10-bit  */
                                 /* mantissa).  For chains of F32 convolutions at precise = 1: the 3xTF32 contraction */
                                 /* reads such a tensor in place and writes one for the next layer.  x_layout = 2:   */
                                 /* one group, C a multiple of 32, y_layout 1 or 2.  y_layout = 2: K a multiple of   */
                                 /* 4, and x_layout = 2 or the 3-channel first layer.                                */
  int32_t flags;                 /* sofie_b200_conv_flags, 0 = none */
} sofie_b200_conv_desc;

/* Flags of sofie_b200_conv_desc.
 *   UNFOLD      take the unfold + contraction path even where the implicit convolution applies (the two paths share
 *               nothing up to the accumulator, which is what the parity tests use this for). */
typedef enum sofie_b200_conv_flags {
  SOFIE_B200_CONV_UNFOLD = 1
} sofie_b200_conv_flags;


typedef struct sofie_b200_ctx sofie_b200_ctx;
typedef struct sofie_b200_gemm_plan sofie_b200_gemm_plan;
typedef struct sofie_b200_conv_plan sofie_b200_conv_plan;

/* ---- library / context -------------------------------------------------------------- */

/* ABI version of the loaded library (compare with SOFIE_B200_ABI_VERSION). */
int sofie_b200_abi_version(void);

/* Message for a status code; never NULL. */
const char *sofie_b200_status_string(int status);

/* Text of the last error raised on this thread by any entry point ("" if none).  The emitted
 * Session wrapper puts it into the std::runtime_error it throws. */
const char *sofie_b200_last_error(void);

/* Creates the per-Session context on `device`, enqueuing on `stream` (a cudaStream_t passed as
 * void*, NULL = the legacy default stream).  Mirrors the Session constructors that take a queue
 * or, with Options::kExternalStream, a cudaStream_t (RModel_ALPAKA.cxx:1450-1477): the stream
 * is borrowed, never destroyed. */
int sofie_b200_ctx_create(sofie_b200_ctx **out, int device, void *stream);

/* Destroys plans' shared state; call after the stream is idle (RModel_ALPAKA.cxx:1479-1485). */
int sofie_b200_ctx_destroy(sofie_b200_ctx *ctx);

/* Waits for the stream (the alpaka::wait(queue) at the end of Session::infer,
 * RModel_ALPAKA.cxx:857-909) and returns SOFIE_B200_ERR_DEVICE_WAIT if a kernel reported a
 * bounded wait that ran out since the last call. */
int sofie_b200_ctx_sync(sofie_b200_ctx *ctx);

/* Number of kernels this ctx has launched so far (for launch accounting in benchmarks). */
int64_t sofie_b200_ctx_launch_count(const sofie_b200_ctx *ctx);

/* Self-test of the device-side error path (the reference has no counterpart: its kernels have no waits;
 * the status word plays the role of the exceptions alpaka raises, RModel_ALPAKA.cxx:749-752).  Enqueues a
 * one-thread kernel that waits, with the contraction kernels' own bounded wait, on a barrier nothing ever
 * signals; after `limit_us` microseconds (1 .. 100000) it gives up, records its code in the status word and
 * returns normally.  The next sofie_b200_ctx_sync() then returns SOFIE_B200_ERR_DEVICE_WAIT once, clears the
 * word, and the context stays usable. */
int sofie_b200_selftest_wait_timeout(sofie_b200_ctx *ctx, int64_t limit_us);

/* ---- contractions -------------------------------------------------------------------- */

/* Registers one contraction (blas.addOperationConfig, RModel_ALPAKA.cxx:1334-1341). */
int sofie_b200_gemm_plan_create(sofie_b200_ctx *ctx, const sofie_b200_gemm_desc *desc,
                                sofie_b200_gemm_plan **out);
int sofie_b200_gemm_plan_destroy(sofie_b200_gemm_plan *plan);

/* Name of the kernel family the plan selected: "umma" (tcgen05 + TMEM + TMA), "umma3x" (fp32 operands as
 * error-compensated 3xTF32: split operands, a tcgen05 kernel that sums short K chunks in registers because the
 * tensor core's fp32 accumulation truncates; chosen for F32 at precise = 1 from SOFIE_B200_SPLIT_MIN_FLOPS up)
 * or "simt" (CUDA cores). */
const char *sofie_b200_gemm_plan_kernel(const sofie_b200_gemm_plan *plan);

/* Enqueues the contraction with its fused epilogue on the ctx's stream: the replacement of
 * blas.gemm / gemmrelu / matmul / gemmStridedBatched (ROperator_Gemm.hxx:931-1098) and of
 * GemmBiasAddKernel (ROperator_Gemm.hxx:743-764).  `ep` may be NULL (plain product). */
int sofie_b200_gemm_enqueue(sofie_b200_gemm_plan *plan, const void *A, const void *B, void *Y,
                            const sofie_b200_epilogue *ep);

/* Another GPU's memory for sofie_b200_gemm_enqueue_peers (the reference has no counterpart: one device per Session,
 * core/src/RModel_ALPAKA.cxx:1123-1132).  Two ways to a pointer this ctx's kernels may store to:
 *  - one process driving several GPUs: sofie_b200_ctx_enable_peer(ctx, other_device) once, after which any device pointer
 *    of `other_device` is valid in this ctx's kernels;
 *  - one process per GPU: the owner exports a device pointer (anywhere inside a cudaMalloc'ed allocation) to a 72-byte handle,
 *    sends the bytes to the other process by any means, which opens it and receives a device pointer to the same byte.
 *    Close every opened pointer before the owner frees the allocation.  A handle is opened once per process; opening the
 *    same allocation again returns the mapping that is already there. */
typedef struct sofie_b200_peer_handle {
  unsigned char ipc[64]; /* the CUDA IPC handle of the allocation */
  uint64_t offset;       /* of the exported pointer inside it     */
} sofie_b200_peer_handle;
int sofie_b200_ctx_enable_peer(sofie_b200_ctx *ctx, int32_t peer_device);
int sofie_b200_peer_export(sofie_b200_ctx *ctx, const void *dev_ptr, sofie_b200_peer_handle *out);
int sofie_b200_peer_open(sofie_b200_ctx *ctx, const sofie_b200_peer_handle *handle, void **dev_ptr);
int sofie_b200_peer_close(sofie_b200_ctx *ctx, void *dev_ptr);

/* The same contraction with its result written to further buffers as well: the tensor-parallel column split of a large
 * Gemm.  The reference runs one Session per device and has no such split (core/src/RModel_ALPAKA.cxx:1123-1132: one device per
 * Session); the call replaces what a split would otherwise need after blas.gemm (ROperator_Gemm.hxx:1066-1088) -- an
 * all-gather of the column shards.  Each rank holds the columns [n0, n0 + N) of the weight, enqueues its [M, N] contraction
 * with Y pointing at column n0 of its own full-width result (ldy = the full width) and peer_Y[i] at the same column of every
 * other rank's result, mapped into this process (CUDA IPC or symmetric memory); the epilogue stores every finished row
 * segment to Y and to each peer_Y[i] with one bulk tensor store each (plain peer stores over NVLink; no multicast), so when
 * all ranks' kernels have finished every rank holds the whole [M, full width] result.  The ranks still have to meet before
 * reading it (a barrier or any collective on the stream).  n_peers 0..7.  Needs a plan on the tensor-core kernel with B as
 * it is stored (no B_CONSTANT re-layout), N a multiple of 64, 16-byte aligned outputs, pitches and epilogue vectors, and floating-point operands (bf16, f16, FP8
 * or fp32; the int8 kernels have no register left for it and return SOFIE_B200_ERR_INVALID). */
int sofie_b200_gemm_enqueue_peers(sofie_b200_gemm_plan *plan, const void *A, const void *B, void *Y, void *const *peer_Y, int32_t n_peers,
                                  const sofie_b200_epilogue *ep);

/* Same contraction with HOST operands: copies A and B to ctx-owned device staging buffers,
 * runs the plan, copies Y back and waits.  This is the shape of Session::infer on host data
 * (the CPU Session's infer(const float*), core/src/RModel.cxx:1303-1419).  Epilogue vectors
 * (scales, bias) are device pointers as in sofie_b200_gemm_enqueue. */
int sofie_b200_gemm_run_host(sofie_b200_gemm_plan *plan, const void *hostA, const void *hostB,
                             void *hostY, const sofie_b200_epilogue *ep);

/* `count` independent contractions of the plan with HOST operands (a queue of inferences, the loop a caller of
 * Session::infer, core/src/RModel.cxx:1303-1419, runs over its events): hostA[i], hostB[i] -> hostY[i].  The copies travel on two streams of the
 * context next to its compute stream, with two sets of device staging buffers: the host-to-device copy of inference
 * i+1 and the device-to-host copy of inference i-1 overlap the contraction of inference i (PCIe is full duplex).
 * Returns when every hostY[i] is written.  Pinned host memory is needed for the overlap (pageable memory works, serially).
 * The same pointer may appear several times in hostA / hostB (a shared weight matrix is still copied every time). */
int sofie_b200_gemm_run_host_many(sofie_b200_gemm_plan *plan, int64_t count, const void *const *hostA,
                                  const void *const *hostB, void *const *hostY, const sofie_b200_epilogue *ep);

/* ---- convolution ---------------------------------------------------------------------- */

/* Registers a convolution and re-lays the weights once (the reference redoes its weight
 * re-layout on every inference, ROperator_Conv.hxx:985-997).  `W` is the device pointer of the
 * [K, C/groups, R, S] weights in x_dtype (F32 or I8). */
int sofie_b200_conv_plan_create(sofie_b200_ctx *ctx, const sofie_b200_conv_desc *desc, const void *W,
                                sofie_b200_conv_plan **out);
int sofie_b200_conv_plan_destroy(sofie_b200_conv_plan *plan);
/* Output extent per ROperator_Conv.hxx:123-262. */
int sofie_b200_conv_out_shape(const sofie_b200_conv_desc *desc, int64_t *Ho, int64_t *Wo);
/* Bytes of caller-provided scratch the plan needs per enqueue (0 if none): the unfolded input,
 * [groups][N][Ho*Wo][kpad] elements with kpad = C/groups*R*S rounded up to 16 bytes -- or, for an F32
 * convolution at precise = 1 of at least SOFIE_B200_SPLIT_MIN_FLOPS (2 * K/groups * Ho*Wo * kpad * N), which runs
 * as error-compensated 3xTF32 on the tensor cores, two segments (hi | lo) of C/groups*R*S rounded up to 32; plus a channels-last
 * copy of the input (N*C*H*W elements, 256-byte aligned behind the unfolded matrix) when C/groups is a whole number
 * of 16-byte vectors, from which the unfold is plain vector copies.  The Im2Col
 * scratch of the reference is per image (ROperator_Conv.hxx:1002-1103); this one covers the batch. */
#define SOFIE_B200_SPLIT_MIN_FLOPS 4e8
int64_t sofie_b200_conv_workspace_bytes(const sofie_b200_conv_plan *plan);
/* Kernel family of the plan's contraction, as sofie_b200_gemm_plan_kernel reports it, or one of the two forms that need no
 * unfold and no workspace (workspace_bytes = 0, `workspace` may be NULL):
 *   "direct"       the 3-channel 3x3 first layer (NCHW input, one group) on the CUDA cores;
 *   "umma_im2col"  implicit convolution: x_layout = y_layout = 1, one group, I8 input (zero point 0, or no padding) or
 *                  F32 at precise = 0, C * element size a multiple of 64 bytes -- the tensor-core contraction reads X
 *                  itself through im2col-mode TMA loads;
 *   "umma3x_im2col" the same for F32 at fp32 accuracy: x_layout = 2 (TF32 pairs), three TF32 products summed in fp32. */
const char *sofie_b200_conv_plan_kernel(const sofie_b200_conv_plan *plan);
/* Enqueues Y = epilogue(conv(X, W)); columns of the epilogue are output channels. */
int sofie_b200_conv_enqueue(sofie_b200_conv_plan *plan, const void *X, void *Y, void *workspace,
                            const sofie_b200_epilogue *ep);

/* (No counterpart in the reference.)  The same convolution for hosts that forbid device allocation
 * once they are configured -- fixed-memory-budget services such as online event filters, which carve up
 * GPU memory at start-up and must not see a cudaMalloc (device-wide serialisation, late out-of-memory
 * failures) from inside their event loop.  No plan, no workspace argument: the padded weights and the
 * unfolded input go to a 16 MiB array that is part of the library image, so nothing is allocated or
 * freed, on the device or by any library, in this call.
 *   - Every GPU that uses the library holds those 16 MiB until the process exits.  CUDA loads a module's code and
 *     static arrays lazily, on first use: the 16 MiB are reserved by the first call of this function on a device,
 *     and the first launch of each kernel it uses (int8 and fp32 paths have different ones) loads that kernel's
 *     code.  So a host that forbids allocation after configuration makes one warm-up call per device for each
 *     input type it will use, AT configuration time; from the second call on, device memory does not move.
 *   - A convolution whose padded weights plus unfolded input ([groups][N][Ho*Wo][C/groups*R*S rounded
 *     up to 16 bytes] elements) exceed 16 MiB returns SOFIE_B200_ERR_TOO_LARGE.
 *   - The first call on each device looks the array's address up (cudaGetSymbolAddress, with that device
 *     current) and caches it; make that first call before any stream capture begins.
 *   - Every argument is checked before anything is enqueued: a refused call launches nothing and leaves the
 *     array untouched.
 *   - The array is shared by every call on the device and keeps the last call's bytes; a call writes all
 *     it reads, so no clearing is needed, but calls that may overlap on the GPU (other streams, other
 *     contexts) race on it.  Calls on one stream are safe.
 * X, W ([K, C/groups, R, S] in x_dtype), Y and the epilogue vectors are device pointers as in
 * sofie_b200_conv_enqueue; integer results are identical to the plan-based call, F32 ones agree within the 1e-5
 * bar (this call always uses the fp32 FMA kernel for F32 at precise = 1). */
int sofie_b200_conv_enqueue_noalloc(sofie_b200_ctx *ctx, const sofie_b200_conv_desc *desc, const void *X,
                                    const void *W, void *Y, const sofie_b200_epilogue *ep);

/* ---- attention ------------------------------------------------------------------------- */

/* Fused scaled-dot-product attention: out[b, :, h, :] = Softmax(scale * Q K^T) V for every batch b and head h, with
 * Q, K, V read in place from the QKV projection's output, qkv [batch, seq, 3, heads, head_dim] (Q of all heads, then
 * K, then V, per token), and out written as [batch, seq, heads * head_dim], the layout the output projection reads.
 * One kernel replaces the graph the reference emits for an attention block -- Transpose, stacked MatMul
 * (blas.gemmStridedBatched, ROperator_Gemm.hxx:991-1065), Softmax (ROperator_Softmax.hxx:204-342), stacked MatMul,
 * Transpose -- whose scores and probabilities make five round trips through HBM.  Scores are kept in fp32, the
 * probabilities are rounded to bf16 before the second contraction (as the unfused graph on bf16 tensors does).
 * Supported: dtype SOFIE_B200_BF16, head_dim 64, 1 <= seq <= 128; anything else returns SOFIE_B200_ERR_INVALID and
 * the caller emits the unfused operators. */
int sofie_b200_attention_enqueue(sofie_b200_ctx *ctx, const void *qkv, void *out, int32_t dtype, int64_t batch,
                                 int64_t seq, int32_t heads, int32_t head_dim, float scale);

/*
 * Scaled dot-product attention, Y = Softmax(scale * Q K^T + mask) V per (batch, head): the reference's
 * ROperator_SDPA (core/inc/SOFIE/operators/ROperator_SDPA.hxx:38-57 constructor, :81-139 shapes, :141-200 the CPU
 * arithmetic this follows: dot * scale, + mask, max, exp, / sum, weighted sum; GPU form :203-330).
 *   folded = 0   Q, K [batch, heads, seq, head_dim], V [.., v_head_dim], Y [batch, heads, seq, v_head_dim]
 *   folded = 1   Q, K, V, Y are [batch, seq, heads * dim] (ROperator_SDPA's rank-3 form with num_heads); ldq / ldk / ldv are
 *                the row pitches in elements of Q, K, V (0 = dense), so the three column blocks of one QKV projection
 *                output are read in place; Y is dense.
 *   mask         additive, [batch, heads, seq, seq] F32, or absent.  scale = 0 selects 1 / sqrt(head_dim).
 * A plan selects the fused tcgen05 kernel ("attention": BF16, folded, no mask, head sizes 64, seq <= 128; no
 * workspace) or the operator chain the reference emits for an attention block ("chain": batched contraction, Softmax,
 * batched contraction, with the operands gathered per head in the caller's workspace).
 */
typedef struct sofie_b200_sdpa_desc {
  int64_t batch, heads, seq, head_dim, v_head_dim;   /* v_head_dim 0 = head_dim */
  int32_t dtype;                                     /* F32 or BF16 */
  int32_t folded;
  int32_t has_mask;
  float scale;
  int64_t ldq, ldk, ldv;
} sofie_b200_sdpa_desc;
typedef struct sofie_b200_sdpa_plan sofie_b200_sdpa_plan;
int sofie_b200_sdpa_plan_create(sofie_b200_ctx *ctx, const sofie_b200_sdpa_desc *desc, sofie_b200_sdpa_plan **out);
int sofie_b200_sdpa_plan_destroy(sofie_b200_sdpa_plan *plan);
/* "attention" or "chain". */
const char *sofie_b200_sdpa_plan_kernel(const sofie_b200_sdpa_plan *plan);
/* Bytes of 256-byte aligned caller scratch an enqueue needs (0 for the fused kernel). */
int64_t sofie_b200_sdpa_workspace_bytes(const sofie_b200_sdpa_plan *plan);
int sofie_b200_sdpa_enqueue(sofie_b200_sdpa_plan *plan, const void *q, const void *k, const void *v, const void *mask, void *y,
                            void *workspace);

/* ---- memory-bound operators the fusion pass leaves ----------------------------------- */

/* LayerNormalization over the last `cols` elements of each of `rows` rows
 * (ROperator_LayerNormalization.hxx:249-321): mean, biased variance, invStd = 1/sqrt(var+eps),
 * y = scale*invStd*(x-mean)+bias.  scale/bias are F32 [cols] or NULL; mean_out/invstd_out are
 * optional F32 [rows].  x and y are F32 or BF16. */
int sofie_b200_layernorm_enqueue(sofie_b200_ctx *ctx, const void *x, void *y, int32_t x_dtype,
                                 int32_t y_dtype, int64_t rows, int64_t cols, const float *scale,
                                 const float *bias, float eps, float *mean_out, float *invstd_out);

/* Softmax / LogSoftmax along the last axis (ROperator_Softmax.hxx:82-119). */
int sofie_b200_softmax_enqueue(sofie_b200_ctx *ctx, const void *x, void *y, int32_t x_dtype,
                               int32_t y_dtype, int64_t rows, int64_t cols, int32_t log_softmax);
/* The same along any axis: x viewed as [outer, n, inner] and normalised over n (ROperator_Softmax.hxx:120-200, the
 * generic-axis path, which divides by the sum).  F32 or BF16, x and y of one type. */
int sofie_b200_softmax_axis_enqueue(sofie_b200_ctx *ctx, const void *x, void *y, int32_t dtype, int64_t outer, int64_t n,
                                    int64_t inner, int32_t log_softmax);

/* Unary elementwise y = act(x) (ROperator_Relu.hxx:47-114, ROperator_Gelu.hxx:42-123,
 * ROperator_LeakyRelu.hxx).  F32 or BF16. */
int sofie_b200_unary_enqueue(sofie_b200_ctx *ctx, const void *x, void *y, int32_t dtype, int64_t n,
                             int32_t act, float act_alpha);

/* Binary elementwise with trailing-dimension broadcast of b (ROperator_BasicBinary.hxx:380,
 * 520-636): y[i] = a[i] op b[i % nb], op: 0 Add, 1 Sub, 2 Mul, 3 Div; optional activation. */
int sofie_b200_binary_enqueue(sofie_b200_ctx *ctx, const void *a, const void *b, void *y, int32_t dtype,
                              int64_t n, int64_t nb, int32_t op, int32_t act);

/* Inference BatchNormalization on NCHW-like data (ROperator_BatchNormalization.hxx:100-153):
 * y = (x - mean[c]) * fused_scale[c] + bias[c], c = (i / inner) % channels; optional Relu. */
int sofie_b200_batchnorm_enqueue(sofie_b200_ctx *ctx, const float *x, float *y, int64_t outer,
                                 int64_t channels, int64_t inner, const float *fused_scale,
                                 const float *bias, const float *mean, int32_t act);

/* GlobalAveragePool: y[n,c] = sum(x[n,c,:]) / inner (ROperator_Pool.hxx:225-237,531-536).
 * x is F32, BF16 or I8; y is F32. */
int sofie_b200_global_avgpool_enqueue(sofie_b200_ctx *ctx, const void *x, float *y, int32_t x_dtype,
                                      int64_t nc, int64_t inner);

/* The same GlobalAveragePool (ROperator_Pool.hxx:225-237,531-536) on a channels-last tensor [n, pixels, channels]
 * (what a convolution with y_layout = 1 writes): y[n,c] = sum(x[n,:,c]) / pixels, summed in pixel order. */
int sofie_b200_global_avgpool_nhwc_enqueue(sofie_b200_ctx *ctx, const void *x, float *y, int32_t x_dtype,
                                           int64_t n, int64_t pixels, int64_t channels);

/* QuantizeLinear / DequantizeLinear (ONNX): q = sat(rint(x/scale)+zp);  x = (q-zp)*scale.
 * Per-tensor when channels == 1, else per-channel with c = (i / inner) % channels. */
int sofie_b200_quantize_enqueue(sofie_b200_ctx *ctx, const float *x, void *q, int32_t q_dtype, int64_t n,
                                const float *scale, const int32_t *zero_point, int64_t channels,
                                int64_t inner);
int sofie_b200_dequantize_enqueue(sofie_b200_ctx *ctx, const void *q, float *x, int32_t q_dtype, int64_t n,
                                  const float *scale, const int32_t *zero_point, int64_t channels,
                                  int64_t inner);

/* Transpose (ROperator_Transpose, core/inc/SOFIE/operators/ROperator_Transpose.hxx:32-36): output dimension d
 * is input dimension perm[d]; rank 1..4, any element type (moved as opaque words).  The head split / merge
 * of attention ([B,S,H,D] <-> [B,H,S,D]) keeps the innermost dimension and runs on 16-byte vectors. */
int sofie_b200_transpose_enqueue(sofie_b200_ctx *ctx, const void *x, void *y, int32_t dtype, int32_t rank,
                                 const int64_t *in_shape, const int32_t *perm);

/* The depth taps of a 3-D convolution as channels (the reference's Conv takes rank-5 inputs through the same im2col + matmul
 * loop as rank-4 ones, ROperator_Conv.hxx:123-262 shapes, :406-642 code): x [n, c, d, hw] -> y [n * d_out, c * taps, hw] with
 * y[(n, od), (c, t), :] = x[n, c, od * stride_d - pad_front + t * dil_d, :], zero outside the depth range.  A 3-D convolution is
 * then this call, a 2-D convolution over n * d_out slices of c * taps channels (the weights [K, C, T, R, S] are [K, C * T, R, S]
 * as stored) and a transpose of [n, d_out, K, Ho * Wo] to [n, K, d_out, Ho * Wo].  F32 or 8-bit elements. */
int sofie_b200_depth_unfold_enqueue(sofie_b200_ctx *ctx, const void *x, void *y, int32_t dtype, int64_t n, int64_t c, int64_t d, int64_t hw,
                                    int64_t taps, int64_t d_out, int64_t stride_d, int64_t pad_front, int64_t dil_d);

/* Type conversion between F32, BF16 and F8E4M3 (saturating round-to-nearest-even; I8 as a source too), with an
 * optional per-row scale: y[r,c] = cvt(x[r,c] / row_scale[r]) (row_scale may be NULL). */
int sofie_b200_convert_enqueue(sofie_b200_ctx *ctx, const void *x, void *y, int32_t x_dtype, int32_t y_dtype,
                               int64_t rows, int64_t cols, const float *row_scale);

/* ---- device arena (Options::kCustomMemory) -------------------------------------------- */

/* Lifetime of one pooled tensor: alive on operator steps [begin, end), `size` bytes
 * (TensorLifeInfo, core/inc/SOFIE/utils/shared/MemoryPlanner.inc:33-45). */
typedef struct sofie_b200_tensor_life {
  int64_t begin, end, size;
} sofie_b200_tensor_life;

/* Plans one arena for `n` tensors: best fit with coalescing of freed neighbours and 256-byte
 * alignment, the policy of OrganizeMemory (MemoryPlanner.inc:47-132, alignment
 * RModel_ALPAKA.cxx:25).  Writes n offsets and the arena size in bytes. */
int sofie_b200_plan_arena(const sofie_b200_tensor_life *lives, int64_t n, int64_t *offsets,
                          int64_t *total_bytes);

#ifdef __cplusplus
}
#endif
#endif /* SOFIE_B200_H */
