// Entry points whose kernels are not built yet: they reject every call.
#include "common.cuh"
using namespace ifv2;

extern "C" int64_t ifv2_decode_workspace_bytes(int batch, int heads_q, int head_dim, int max_blocks) {
  return (int64_t)batch * heads_q * max_blocks * (head_dim + 2) * 4;
}
extern "C" int ifv2_decode(const void*, void*, void*, const void*, const void*, void*, float*,
                           const int64_t*, int, const int32_t*, int, int, int, int, int64_t, int64_t,
                           float, void*, int64_t, void*) {
  return set_error(IFV2_ERR_UNSUPPORTED, "decode: not built yet");
}
