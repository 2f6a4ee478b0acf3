// Peer-memory plumbing for the distributed step's copy-engine exchange: export a device
// allocation as a CUDA IPC handle, map a peer's allocation on the CURRENT device (so that
// copies into it are direct NVLink transfers driven by the copy engines), and fan one source
// buffer out to several mapped destinations with asynchronous device-to-device copies.
#include "../../include/muon_b200.h"

#include "common.cuh"

#include <cuda.h>
#include <cstring>

using namespace mb;

namespace {

typedef CUresult (*GetRangeFn)(CUdeviceptr*, size_t*, CUdeviceptr);

GetRangeFn get_range_fn() {
  static GetRangeFn fn = [] {
    void* sym = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuMemGetAddressRange", &sym, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      return reinterpret_cast<GetRangeFn>(sym);
    return static_cast<GetRangeFn>(nullptr);
  }();
  return fn;
}

}  // namespace

extern "C" {

int muon_b200_ipc_export(const void* ptr, void* handle64, int64_t* offset_out,
                         int64_t* alloc_bytes_out) {
  static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handle is 64 bytes");
  if (!ptr || !handle64 || !offset_out)
    return set_error(ERR_INVALID_ARG, "ipc_export: null argument");
  GetRangeFn range = get_range_fn();
  if (!range) return set_error(ERR_CUDA, "cuMemGetAddressRange entry point not available");
  CUdeviceptr base = 0;
  size_t size = 0;
  CUresult r = range(&base, &size, reinterpret_cast<CUdeviceptr>(ptr));
  if (r != CUDA_SUCCESS)
    return set_error(ERR_CUDA, "cuMemGetAddressRange failed with CUresult %d", (int)r);
  cudaIpcMemHandle_t h;
  MB_CUDA_CHECK(cudaIpcGetMemHandle(&h, reinterpret_cast<void*>(base)));
  std::memcpy(handle64, &h, sizeof(h));
  *offset_out = (int64_t)(reinterpret_cast<CUdeviceptr>(ptr) - base);
  if (alloc_bytes_out) *alloc_bytes_out = (int64_t)size;
  return OK;
}

int muon_b200_ipc_open(const void* handle64, void** base_out) {
  if (!handle64 || !base_out) return set_error(ERR_INVALID_ARG, "ipc_open: null argument");
  cudaIpcMemHandle_t h;
  std::memcpy(&h, handle64, sizeof(h));
  MB_CUDA_CHECK(cudaIpcOpenMemHandle(base_out, h, cudaIpcMemLazyEnablePeerAccess));
  return OK;
}

int muon_b200_ipc_close(void* base) {
  if (!base) return OK;
  MB_CUDA_CHECK(cudaIpcCloseMemHandle(base));
  return OK;
}

int muon_b200_push_copies(void* const* dst, int n, const void* src, int64_t bytes,
                          muon_b200_stream_t stream) {
  if (n < 0 || (n > 0 && !dst) || !src || bytes < 0)
    return set_error(ERR_INVALID_ARG, "push_copies: bad arguments");
  for (int i = 0; i < n; ++i) {
    if (!dst[i]) return set_error(ERR_INVALID_ARG, "push_copies: destination %d is NULL", i);
    MB_CUDA_CHECK(cudaMemcpyAsync(dst[i], src, (size_t)bytes, cudaMemcpyDeviceToDevice,
                                  static_cast<cudaStream_t>(stream)));
  }
  return OK;
}

}  // extern "C"
