// Error string, version and status read-back of the C ABI (include/trimkv_b200.h).
#include <cstdarg>
#include <cstdio>
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
