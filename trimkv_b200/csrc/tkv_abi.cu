// Error string, version and status read-back of the C ABI (include/trimkv_b200.h).
#include <cstdarg>
#include <cstdio>
#include <cstring>
#include "tkv_common.cuh"

namespace tkv {
static thread_local char g_err[512] = "";

int fail(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
  return code;
}

int check_launch(const char* what) {
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return fail(TKV_ERR_LAUNCH, "%s: %s", what, cudaGetErrorString(e));
  return TKV_OK;
}
}  // namespace tkv

extern "C" int tkv_version(void) { return 100; }

extern "C" const char* tkv_last_error(void) { return tkv::g_err; }

extern "C" int tkv_read_status(int32_t* status, tkv_stream_t stream) {
  if (status == nullptr) return tkv::fail(TKV_ERR_ARG, "tkv_read_status: status is NULL");
  int32_t h = 0;
  cudaError_t e = cudaMemcpyAsync(&h, status, sizeof(h), cudaMemcpyDeviceToHost, (cudaStream_t)stream);
  if (e == cudaSuccess) e = cudaStreamSynchronize((cudaStream_t)stream);
  if (e != cudaSuccess) return tkv::fail(TKV_ERR_LAUNCH, "tkv_read_status: %s", cudaGetErrorString(e));
  if (h != 0) {
    e = cudaMemsetAsync(status, 0, sizeof(h), (cudaStream_t)stream);
    if (e != cudaSuccess) return tkv::fail(TKV_ERR_LAUNCH, "tkv_read_status: %s", cudaGetErrorString(e));
  }
  return h;
}

extern "C" int tkv_enable_peer_access(int peer_device) {
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return tkv::fail(TKV_ERR_LAUNCH, "tkv_enable_peer_access: %s", cudaGetErrorString(e));
  if (dev == peer_device) return TKV_OK;
  int can = 0;
  e = cudaDeviceCanAccessPeer(&can, dev, peer_device);
  if (e != cudaSuccess) return tkv::fail(TKV_ERR_LAUNCH, "tkv_enable_peer_access: %s", cudaGetErrorString(e));
  if (!can) return tkv::fail(TKV_ERR_UNSUPPORTED, "tkv_enable_peer_access: device %d cannot access device %d", dev, peer_device);
  e = cudaDeviceEnablePeerAccess(peer_device, 0);
  if (e == cudaErrorPeerAccessAlreadyEnabled) { (void)cudaGetLastError(); return TKV_OK; }
  if (e != cudaSuccess) return tkv::fail(TKV_ERR_LAUNCH, "tkv_enable_peer_access: %s", cudaGetErrorString(e));
  return TKV_OK;
}

// ---- CUDA IPC helpers for the head-sharded exchange (host-only; no kernels) ---------------------------------
namespace tkv {
typedef int (*GetAddressRangeFn)(unsigned long long*, size_t*, unsigned long long);   // cuMemGetAddressRange
static GetAddressRangeFn address_range_fn() {
  static GetAddressRangeFn fn = nullptr;
  if (fn == nullptr) {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuMemGetAddressRange", &ptr, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<GetAddressRangeFn>(ptr);
  }
  return fn;
}
}  // namespace tkv

extern "C" int tkv_ipc_export(const void* ptr, void* handle_out, int64_t* offset_out) {
  using namespace tkv;
  if (!ptr || !handle_out || !offset_out) return fail(TKV_ERR_ARG, "tkv_ipc_export: NULL pointer argument");
  static_assert(sizeof(cudaIpcMemHandle_t) == TKV_IPC_HANDLE_BYTES, "handle size");
  GetAddressRangeFn range = address_range_fn();
  if (range == nullptr) return fail(TKV_ERR_LAUNCH, "tkv_ipc_export: cuMemGetAddressRange is not available");
  unsigned long long base = 0; size_t size = 0;
  if (range(&base, &size, (unsigned long long)(uintptr_t)ptr) != 0)
    return fail(TKV_ERR_ARG, "tkv_ipc_export: %p is not inside a device allocation", ptr);
  cudaIpcMemHandle_t h;
  cudaError_t e = cudaIpcGetMemHandle(&h, reinterpret_cast<void*>((uintptr_t)base));
  if (e != cudaSuccess) return fail(TKV_ERR_LAUNCH, "tkv_ipc_export: %s", cudaGetErrorString(e));
  memcpy(handle_out, &h, sizeof(h));
  *offset_out = (int64_t)((unsigned long long)(uintptr_t)ptr - base);
  return TKV_OK;
}

extern "C" int tkv_ipc_import(const void* handle, void** base_out) {
  using namespace tkv;
  if (!handle || !base_out) return fail(TKV_ERR_ARG, "tkv_ipc_import: NULL pointer argument");
  cudaIpcMemHandle_t h;
  memcpy(&h, handle, sizeof(h));
  void* p = nullptr;
  // Opened with the CURRENT device: if the memory lives on another GPU, peer access from the current device to it
  // is enabled as part of the mapping.
  cudaError_t e = cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess);
  if (e != cudaSuccess) return fail(TKV_ERR_LAUNCH, "tkv_ipc_import: %s", cudaGetErrorString(e));
  *base_out = p;
  return TKV_OK;
}

extern "C" int tkv_ipc_close(void* base) {
  if (base == nullptr) return TKV_OK;
  cudaError_t e = cudaIpcCloseMemHandle(base);
  if (e != cudaSuccess) return tkv::fail(TKV_ERR_LAUNCH, "tkv_ipc_close: %s", cudaGetErrorString(e));
  return TKV_OK;
}
