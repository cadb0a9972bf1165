// Error reporting shared by every entry point of the C ABI.
#include "common.cuh"

namespace ifv2 {

char* error_buffer() {
  static thread_local char buf[512] = {0};
  return buf;
}

int set_error(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(error_buffer(), 512, fmt, ap);
  va_end(ap);
  return code;
}

int check_launch(const char* what) {
  cudaError_t e = cudaGetLastError();
  if (e == cudaSuccess) return IFV2_OK;
  set_error((int)e, "%s: launch failed: %s", what, cudaGetErrorString(e));
  return (int)e;
}

int clear_launch_status(int32_t* status, void* stream, const char* what) {
  cudaError_t e = cudaMemsetAsync(status, 0, sizeof(int32_t), (cudaStream_t)stream);
  if (e == cudaSuccess) return IFV2_OK;
  return set_error((int)e, "%s: clearing the status word failed: %s", what, cudaGetErrorString(e));
}

}  // namespace ifv2

extern "C" int ifv2_check_status(int32_t* status, void* stream) {
  IFV2_REQUIRE(status != nullptr, IFV2_ERR_INVALID_ARG, "check_status: null status block");
  int32_t host[2] = {0, 0};
  cudaStream_t st = (cudaStream_t)stream;
  cudaError_t e = cudaMemcpyAsync(host, status, sizeof(host), cudaMemcpyDeviceToHost, st);
  if (e == cudaSuccess) e = cudaStreamSynchronize(st);
  if (e != cudaSuccess)
    return ifv2::set_error((int)e, "check_status: %s", cudaGetErrorString(e));
  if (host[0] == 0 && host[1] == 0) return IFV2_OK;
  e = cudaMemsetAsync(status, 0, sizeof(host), st);
  if (e == cudaSuccess) e = cudaStreamSynchronize(st);
  if (e != cudaSuccess)
    return ifv2::set_error((int)e, "check_status: %s", cudaGetErrorString(e));
  return ifv2::set_error(IFV2_ERR_DEVICE_STATUS,
                         "a kernel abandoned a bounded wait (site %d): the outputs of that launch "
                         "are undefined", host[1] != 0 ? host[1] : host[0]);
}

extern "C" const char* ifv2_last_error(void) { return ifv2::error_buffer(); }
extern "C" int ifv2_version(void) { return 200; }
