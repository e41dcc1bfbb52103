// Internal definitions shared by the translation units of libsofie_b200.
#pragma once
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <cuda_fp8.h>
#include <stdint.h>
#include <stdio.h>
#include <string>
#include <vector>

#include "../../include/sofie_b200.h"

namespace sb200 {

// Per-thread error text behind sofie_b200_last_error().
void set_error(const char *fmt, ...);
int fail(int status, const char *fmt, ...);

#define SB_CUDA(call)                                                                         \
  do {                                                                                        \
    cudaError_t e__ = (call);                                                                 \
    if (e__ != cudaSuccess)                                                                   \
      return ::sb200::fail(SOFIE_B200_ERR_CUDA, "%s failed: %s (%s:%d)", #call,              \
                           cudaGetErrorString(e__), __FILE__, __LINE__);                      \
  } while (0)

// Codes written by kernels into the ctx status word (0 = fine).
enum DeviceStatus : int {
  DEV_OK = 0,
  DEV_WAIT_SMEM_EMPTY = 1,  // TMA producer waited for a free shared-memory stage
  DEV_WAIT_SMEM_FULL = 2,   // MMA issuer waited for a filled stage
  DEV_WAIT_TMEM_EMPTY = 3,  // MMA issuer waited for a drained accumulator
  DEV_WAIT_TMEM_FULL = 4,   // epilogue waited for a finished accumulator
};

inline int dtype_size(int dt) {
  switch (dt) {
    case SOFIE_B200_F32: return 4;
    case SOFIE_B200_BF16: return 2;
    case SOFIE_B200_I8: return 1;
    case SOFIE_B200_F8E4M3: return 1;
    case SOFIE_B200_I32: return 4;
    case SOFIE_B200_U8: return 1;
  }
  return 0;
}

}  // namespace sb200

struct sofie_b200_ctx {
  int device = 0;
  cudaStream_t stream = nullptr;
  int sm_count = 0;
  int *d_status = nullptr;   // device status word (DeviceStatus)
  int *h_status = nullptr;   // pinned mirror
  int64_t launches = 0;
  // staging for the *_host helpers (grown on demand)
  void *stage[3] = {nullptr, nullptr, nullptr};
  size_t stage_bytes[3] = {0, 0, 0};
  // sofie_b200_gemm_run_host_many: a second set of staging buffers, copy streams and events (created on first use)
  void *stage2[3] = {nullptr, nullptr, nullptr};
  size_t stage2_bytes[3] = {0, 0, 0};
  cudaStream_t copy_in = nullptr, copy_out = nullptr;
  cudaEvent_t ev_in[2] = {nullptr, nullptr}, ev_done[2] = {nullptr, nullptr}, ev_out[2] = {nullptr, nullptr};
  // sofie_b200_peer_open: the other processes' allocations mapped here (IPC handle bytes -> base pointer, users)
  struct PeerMapping { unsigned char ipc[64]; void *base; int users; };
  std::vector<PeerMapping> peer_mappings;
};

namespace sb200 {
int ensure_stage(sofie_b200_ctx *ctx, int idx, size_t bytes);
}
