// Plan object behind sofie_b200_gemm_plan and the two kernel families it can select.
#pragma once
#include <cuda.h>
#include "epilogue.cuh"

// Built with -DSB200_ROLE_TIMERS, the first and last CTA print how many cycles each role spent waiting
// (a debugging aid for the pipeline; never defined in the shipped library).
#ifdef SB200_ROLE_TIMERS
#define ROLE_TIMER(name) long long name = 0
#define ROLE_WAIT(name, expr) [&] { const long long t0__ = clock64(); const bool r__ = (expr); name += clock64() - t0__; return r__; }()
#define ROLE_SECTION_BEGIN() sec_t0 = clock64()
#define ROLE_SECTION_END(name) name += clock64() - sec_t0
#define ROLE_REPORT(...) if (blockIdx.x <= 1 || blockIdx.x >= gridDim.x - 2) printf(__VA_ARGS__)
#else
#define ROLE_TIMER(name)
#define ROLE_WAIT(name, expr) (expr)
#define ROLE_REPORT(...)
#define ROLE_SECTION_BEGIN()
#define ROLE_SECTION_END(name)
#endif

namespace sb200 {

constexpr int UMMA_BM = 128;          // rows of one accumulator tile (TMEM lanes)
constexpr int UMMA_STAGE_K_BYTES = 128;  // K extent of one shared-memory stage, in bytes (one 128B swizzle row)
// The opt-in limit is a property of the FUNCTION, shared by every plan that launches it: it is always set to the
// device maximum, never to one plan's size (a later, smaller plan would otherwise make an earlier one unlaunchable).
constexpr int UMMA_MAX_DYN_SMEM = 227 * 1024;
constexpr int UMMA_TAIL_BYTES = 1024;  // barriers, TMEM slot and abort flag behind the stage ring; the epilogue staging follows
// Warp roles of the tcgen05 kernel: warp 0 TMA producer of operand A, warp 1 MMA issuer, warp 2 TMA producer of operand B,
// warp 3 idle (it keeps the epilogue warps' index congruent to their tensor-memory lane quarter), then the epilogue warps.
constexpr int UMMA_EPI_WARPS = 16;    // four epilogue warps per tensor-memory lane quarter, taking 64-byte row segments in turn
constexpr int UMMA_B_PRODUCER_WARP = 2;
constexpr int UMMA_FIRST_EPI_WARP = 4;
constexpr int UMMA_THREADS = 32 * (UMMA_FIRST_EPI_WARP + UMMA_EPI_WARPS);
constexpr int UMMA_MAX_ACCS = 4;      // accumulators in tensor memory (UmmaParams::accs: 2 or 4)
constexpr int UMMA_EPI_STAGE_BYTES = 2048;   // staging buffer of one epilogue warp: 32 rows x 64 bytes

// Tensor maps of further outputs (sofie_b200_gemm_enqueue_peers): peers' copies of Y, written by the epilogue's bulk stores.
constexpr int UMMA_MAX_PEERS = 7;
struct UmmaPeerMaps {
  CUtensorMap tm[UMMA_MAX_PEERS];
};

// Everything the tcgen05 kernel needs besides the two tensor maps.
struct UmmaParams {
  int M, N, K, batch;
  int tiles_m, tiles_n;
  long long num_tiles;
  long long split_from, num_items;  // work items: tiles below split_from whole, the rest as two N halves each
  uint32_t idesc_half;              // instruction descriptor with N = bn/2
  int num_kb;          // K blocks of kb_elems elements
  int kb_elems;        // K elements per stage (128 bytes / element size)
  int bn;              // N extent of the tile and of each MMA (32, 64, 128 or 256)
  int stages;
  uint32_t tmem_cols;  // allocated TMEM columns: power of two >= 2*bn
  uint32_t a_stage_bytes, b_stage_bytes;
  uint32_t idesc;      // tcgen05 instruction descriptor
  uint32_t a_desc_hi, b_desc_hi;   // upper words of the shared-memory matrix descriptors
  uint32_t a_desc_lo, b_desc_lo;   // constant part of the lower words (leading byte offset field)
  uint32_t a_kadv, b_kadv;         // start-address advance per MMA K step, in 16-byte units
  int a_mn, b_mn;                  // operand is MN-major (its M or N index is contiguous) in global memory
  int a_boxes, b_boxes;            // TMA boxes per stage
  uint32_t a_box_bytes, b_box_bytes;
  int a_box_mn, b_box_mn;          // MN elements covered by one box of an MN-major operand
  int a_bcast, b_bcast;            // operand shared by the whole batch
  int vec_ok;                      // 16-byte vector stores of 32-column chunks are aligned
  int raster_n;                    // tile order inside a batch: 0 = M index fastest, 1 = N index fastest
  int y_peers;                     // further outputs of the same shape and pitch (other GPUs' copies of Y): every finished row segment
                                   // is stored to each of them as well (UmmaPeerMaps)
  int rgroup;                      // > 0: tiles go in bands of this many N tiles, N index fastest inside a band (neither operand fits L2)
  int y_tma;                       // the epilogue may store complete row segments through the tensor map of Y
  int seg_kb;                      // chunk-promotion kernel: K blocks per split segment (ks / 32)
  int a_seg_kb[3], b_seg_kb[3];    // K block at which each of the three product segments starts in the stored A / B (hi | lo)
  int promote_chunk;               // chunk-promotion kernel: K blocks per tensor-memory accumulation
  int fused3;                      // chunk-promotion kernel: a stage holds A hi | A lo | B hi | B lo of one K block and feeds all three
                                   // products (4 loads per 12 MMAs instead of 6); stage byte counts are the doubled ones
  int b_rows;                      // N extent of the B slice one CTA stages (= bn)
  int kb_mmas;                     // MMAs (32 bytes of K each) per K block: 4, or 2 when a K block is 64 bytes
  int wide;                        // 128-byte row segments in the epilogue (4 KB of staging per warp) instead of 64-byte ones
  int prod_lanes;                  // TMA producer lanes per producer warp (1 to 4)
  int b_resident;                  // all K blocks of operand B stay in shared memory (tiles_n == 1); the ring holds A only
  int accs;                        // accumulators in tensor memory: 1 (tall tiles), 2 or 4
  int mh;                          // M halves of a tile: 1, or 2 = a tall 256 x bn tile whose two 128-row halves share every B slice
  int teams;                       // teams of epilogue warps, each draining a tile of its own: 1, 2 or 4, at most accs
  int im2col;
  int ic_wo, ic_pix;               // output width, output pixels per image
  int ic_sw, ic_sh, ic_pl, ic_pt;  // strides; left and top padding
  int ic_dw, ic_dh, ic_s;          // dilations; filter width
  int ic_cblocks;                  // K blocks per filter tap
  int ic_c;                        // channels per pixel (a tensor of TF32 pairs stores 2 * ic_c: hi channels, then lo)
  EpiParams ep;
  int *status;
};

// x rounded to the nearest TF32 value (ties away from zero); values whose rounding would overflow are truncated
__device__ __forceinline__ float tf32_rn(float x) {
  const uint32_t b = __float_as_uint(x);
  const uint32_t r = ((b & 0x7f800000u) >= 0x7f000000u) ? b : b + 0x1000u;
  return __uint_as_float(r & 0xffffe000u);
}

// Problems below this many flops stay on the fp32 FMA kernel (the split passes would dominate).
constexpr double SPLIT_MIN_FLOPS = 4e8;
// Split operands are stored as [hi | lo], each segment SPLIT_K_ALIGN-aligned in K (one K block of the TF32 kernel), so that
// the three products hi*hi, lo*hi, hi*lo are whole K blocks whose A and B coordinates are looked up per segment.
constexpr long long SPLIT_K_ALIGN = 32;
inline long long split_ks(long long K) { return (K + SPLIT_K_ALIGN - 1) / SPLIT_K_ALIGN * SPLIT_K_ALIGN; }

// Tile r of a batch -> (M tile, N tile).  Consecutive tiles run at the same time on neighbouring SMs, so the index that
// varies fastest decides which operand slice they share in L2 (see umma_plan_init for the choice).
__device__ __forceinline__ void tile_mn(const UmmaParams &p, int r, int &tm, int &tn) {
  if (p.raster_n) { tn = r % p.tiles_n; tm = r / p.tiles_n; }
  else { tm = r % p.tiles_m; tn = r / p.tiles_m; }
}

struct SimtParams {
  const void *A, *B;
  int M, N, K, batch;
  long long lda, ldb, stride_a, stride_b;
  int trans_a, trans_b;
  EpiParams ep;
};

}  // namespace sb200

namespace sb200 {
// The convolution an implicit plan stands for (sofie_b200_gemm_plan::ic): A is the [N, H, W, C] input itself.
struct Im2colDesc {
  int on = 0;
  long long N = 0, H = 0, W = 0, C = 0, Ho = 0, Wo = 0;
  long long Cs = 0;   // channels per pixel as stored, when not C: 2 * C for a tensor of TF32 pairs (hi channels, then lo channels)
  int R = 1, S = 1, pt = 0, pl = 0, pb = 0, pr = 0, sh = 1, sw = 1, dh = 1, dw = 1;
};
}  // namespace sb200

struct sofie_b200_gemm_plan {
  sofie_b200_ctx *ctx = nullptr;
  sofie_b200_gemm_desc desc{};
  int use_umma = 0;
  int kind = 0;                    // ptx::KIND_*
  sb200::UmmaParams up{};
  size_t smem_bytes = 0;
  int grid = 0;
  // tensor maps are rebuilt only when an operand pointer changes
  const void *cached_a = nullptr, *cached_b = nullptr;
  CUtensorMap tm_a{}, tm_b{}, tm_y{};
  sb200::UmmaPeerMaps peer_maps{};        // maps of the peers' outputs of the enqueue in progress
  const void *cached_y = nullptr;
  int cached_seg_div = 0;          // row-segment divisor the cached map of Y was built for
  // fp32-accurate tensor path (3xTF32): split operands [rows, 3*ks] and the TF32 plan that multiplies them
  sofie_b200_gemm_plan *inner = nullptr;
  float *split_a = nullptr, *split_b = nullptr;
  long long ks = 0;
  long long k_store = 0;           // K extent of the operands as stored (two segments) when it differs from desc.K (three products)
  int promote = 0;                 // this (inner TF32) plan runs the chunk-promotion kernel
  sb200::Im2colDesc ic{};          // set: operand A is an image tensor read in im2col mode (implicit convolution)
  int kb_bytes = 128;              // K extent of one shared-memory stage in bytes: 128 (128B swizzle) or 64 (64B swizzle)
  int split_out = 0;               // chunk-promotion kernel: write Y as TF32 pairs (EpiParams::split_out)
  // SOFIE_B200_GEMM_B_CONSTANT: a weight B stored [K,N] is kept as a K-major copy [N,K] (b_kmajor, owned by the plan) that is
  // refreshed when B's address changes; `desc` then describes the contraction on the copy (trans_b = 1, ldb = K)
  void *b_kmajor = nullptr;
  const void *b_kmajor_src = nullptr;
  long long b_src_ld = 0, b_src_stride = 0;   // pitch and batch stride of B as the caller stores it
  const void *split_b_src = nullptr;          // constant B whose hi | lo split is already in split_b
};

namespace sb200 {
// gemm_umma.cu
int umma_plan_init(sofie_b200_gemm_plan *plan);          // 0 if the tcgen05 path applies, 1 if not, <0 error
int umma_enqueue(sofie_b200_gemm_plan *plan, const void *A, const void *B, const EpiParams &ep, void *const *peer_y = nullptr, int n_peers = 0);
// gemm_umma3x.cu (TF32 kernel that sums short K chunks in registers)
int umma_promote_set_smem(size_t smem_bytes);
int umma_promote_launch(sofie_b200_gemm_plan *plan, const UmmaParams &u);
// api.cu
int gemm_make_epi(const sofie_b200_gemm_desc &d, void *Y, const sofie_b200_epilogue *ep, EpiParams *o);
int gemm_plan_create_promote(sofie_b200_ctx *ctx, const sofie_b200_gemm_desc &g, sofie_b200_gemm_plan **out);
int gemm_plan_create_im2col(sofie_b200_ctx *ctx, const sofie_b200_gemm_desc &g, const Im2colDesc &ic, sofie_b200_gemm_plan **out);
int gemm_plan_create_promote_im2col(sofie_b200_ctx *ctx, const sofie_b200_gemm_desc &g, const Im2colDesc &ic, int split_out, sofie_b200_gemm_plan **out);
// gemm_split.cu
int split2_enqueue(sofie_b200_ctx *ctx, const float *src, float *dst, long long rows, long long K, long long Ks, long long ld,
                   long long batch, long long batch_stride, int mn);
// gemm_simt.cu
int simt_enqueue(sofie_b200_gemm_plan *plan, const void *A, const void *B, const EpiParams &ep);
}  // namespace sb200
