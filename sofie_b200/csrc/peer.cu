// Another GPU's memory for the contraction's peer stores (sofie_b200_gemm_enqueue_peers): peer access inside one process,
// and CUDA IPC between the processes of a one-process-per-GPU job.  The reference binds one device per Session
// (core/src/RModel_ALPAKA.cxx:1123-1132) and has nothing of the kind.
#include <cuda.h>
#include <string.h>

#include <mutex>

#include "common.cuh"

using namespace sb200;

namespace {

typedef CUresult (*AddressRangeFn)(CUdeviceptr *, size_t *, CUdeviceptr);

AddressRangeFn address_range_entry() {
  static AddressRangeFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void *sym = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuMemGetAddressRange", &sym, cudaEnableDefault, &q) == cudaSuccess && q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<AddressRangeFn>(sym);
  });
  return fn;
}

}  // namespace

extern "C" {

int sofie_b200_ctx_enable_peer(sofie_b200_ctx *ctx, int32_t peer_device) {
  if (!ctx) return fail(SOFIE_B200_ERR_INVALID, "ctx_enable_peer: ctx is NULL");
  if (peer_device == ctx->device) return 0;
  int can = 0;
  SB_CUDA(cudaDeviceCanAccessPeer(&can, ctx->device, peer_device));
  if (!can) return fail(SOFIE_B200_ERR_NO_DEVICE, "ctx_enable_peer: device %d cannot reach device %d", ctx->device, (int)peer_device);
  SB_CUDA(cudaSetDevice(ctx->device));
  cudaError_t e = cudaDeviceEnablePeerAccess(peer_device, 0);
  if (e == cudaErrorPeerAccessAlreadyEnabled) {
    cudaGetLastError();   // somebody else in the process enabled it: fine
    return 0;
  }
  SB_CUDA(e);
  return 0;
}

int sofie_b200_peer_export(sofie_b200_ctx *ctx, const void *dev_ptr, sofie_b200_peer_handle *out) {
  if (!ctx || !dev_ptr || !out) return fail(SOFIE_B200_ERR_INVALID, "peer_export: NULL argument");
  AddressRangeFn range = address_range_entry();
  if (!range) return fail(SOFIE_B200_ERR_NO_DEVICE, "peer_export: cuMemGetAddressRange entry point not available");
  SB_CUDA(cudaSetDevice(ctx->device));
  CUdeviceptr base = 0;
  size_t bytes = 0;
  if (range(&base, &bytes, (CUdeviceptr)(uintptr_t)dev_ptr) != CUDA_SUCCESS)
    return fail(SOFIE_B200_ERR_INVALID, "peer_export: %p is not inside a device allocation", dev_ptr);
  cudaIpcMemHandle_t h;
  static_assert(sizeof(h) == sizeof(out->ipc), "the IPC handle is 64 bytes");
  SB_CUDA(cudaIpcGetMemHandle(&h, (void *)(uintptr_t)base));
  memcpy(out->ipc, &h, sizeof(h));
  out->offset = (uint64_t)((uintptr_t)dev_ptr - (uintptr_t)base);
  return 0;
}

int sofie_b200_peer_open(sofie_b200_ctx *ctx, const sofie_b200_peer_handle *handle, void **dev_ptr) {
  if (!ctx || !handle || !dev_ptr) return fail(SOFIE_B200_ERR_INVALID, "peer_open: NULL argument");
  for (auto &m : ctx->peer_mappings)
    if (memcmp(m.ipc, handle->ipc, sizeof(m.ipc)) == 0) {
      m.users++;
      *dev_ptr = (char *)m.base + handle->offset;
      return 0;
    }
  SB_CUDA(cudaSetDevice(ctx->device));
  cudaIpcMemHandle_t h;
  memcpy(&h, handle->ipc, sizeof(h));
  void *base = nullptr;
  SB_CUDA(cudaIpcOpenMemHandle(&base, h, cudaIpcMemLazyEnablePeerAccess));
  sofie_b200_ctx::PeerMapping m;
  memcpy(m.ipc, handle->ipc, sizeof(m.ipc));
  m.base = base;
  m.users = 1;
  ctx->peer_mappings.push_back(m);
  *dev_ptr = (char *)base + handle->offset;
  return 0;
}

int sofie_b200_peer_close(sofie_b200_ctx *ctx, void *dev_ptr) {
  if (!ctx || !dev_ptr) return fail(SOFIE_B200_ERR_INVALID, "peer_close: NULL argument");
  AddressRangeFn range = address_range_entry();
  for (size_t i = 0; i < ctx->peer_mappings.size(); ++i) {
    auto &m = ctx->peer_mappings[i];
    CUdeviceptr base = 0;
    size_t bytes = 0;
    if (!range || range(&base, &bytes, (CUdeviceptr)(uintptr_t)m.base) != CUDA_SUCCESS) continue;
    if ((uintptr_t)dev_ptr < (uintptr_t)base || (uintptr_t)dev_ptr >= (uintptr_t)base + bytes) continue;
    if (--m.users == 0) {
      SB_CUDA(cudaSetDevice(ctx->device));
      SB_CUDA(cudaStreamSynchronize(ctx->stream));   // no store of ours may still be on its way there
      cudaError_t e = cudaIpcCloseMemHandle(m.base);
      ctx->peer_mappings.erase(ctx->peer_mappings.begin() + i);
      SB_CUDA(e);
    }
    return 0;
  }
  return fail(SOFIE_B200_ERR_INVALID, "peer_close: %p was not returned by peer_open", dev_ptr);
}

}  // extern "C"
