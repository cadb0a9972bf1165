// Host side of TMA: encodes tensor maps through the driver entry point, looked up at run time
// so that the library links against the CUDA runtime only and loads on machines without a GPU.
#include <mutex>
#include "tc05.cuh"

namespace ifv2 {
namespace {

using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                   const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                   const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                   CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
  });
  return fn;
}

}  // namespace

int make_tensor_map_bf16_3d(CUtensorMap* map, const void* base, uint64_t d0, uint64_t d1,
                            uint64_t d2, uint64_t stride1_bytes, uint64_t stride2_bytes,
                            uint32_t b0, uint32_t b1, uint32_t b2) {
  EncodeTiledFn fn = encode_fn();
  IFV2_REQUIRE(fn != nullptr, IFV2_ERR_DRIVER, "cuTensorMapEncodeTiled is not available (no driver?)");
  IFV2_REQUIRE(reinterpret_cast<uintptr_t>(base) % 16 == 0, IFV2_ERR_INVALID_ARG,
               "tensor base address must be 16-byte aligned");
  IFV2_REQUIRE(stride1_bytes % 16 == 0 && stride2_bytes % 16 == 0, IFV2_ERR_INVALID_ARG,
               "tensor strides must be multiples of 16 bytes");
  cuuint64_t dims[3] = {d0, d1 ? d1 : 1, d2 ? d2 : 1};
  cuuint64_t strides[2] = {stride1_bytes, stride2_bytes};
  cuuint32_t box[3] = {b0, b1, b2};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(base), dims, strides,
                  box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  IFV2_REQUIRE(r == CUDA_SUCCESS, IFV2_ERR_DRIVER, "cuTensorMapEncodeTiled failed with CUresult %d",
               (int)r);
  return IFV2_OK;
}

}  // namespace ifv2
