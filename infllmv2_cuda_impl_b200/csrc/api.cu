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

}  // namespace ifv2

extern "C" const char* ifv2_last_error(void) { return ifv2::error_buffer(); }
extern "C" int ifv2_version(void) { return 100; }
