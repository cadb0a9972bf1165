// Warp-level tile helpers shared by the decode-time kernels (one query token per sequence: the
// 16 query heads of a KV head are exactly one mma.sync M tile, far too small for tcgen05):
// cp.async tiles of 32 keys x 128 features in swizzled shared memory, ldmatrix fragments,
// mma.sync m16n8k16 bf16 -> fp32.
#pragma once
#include "common.cuh"

namespace ifv2 {
namespace mmasync {

constexpr int kUnit = 32;                               // keys per shared-memory tile

__device__ __forceinline__ void cp_async16(void* smem, const void* gmem) {
  const uint32_t s = (uint32_t)__cvta_generic_to_shared(smem);
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(s), "l"(gmem) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}
__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], const void* smem) {
  const uint32_t s = (uint32_t)__cvta_generic_to_shared(smem);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(s));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], const void* smem) {
  const uint32_t s = (uint32_t)__cvta_generic_to_shared(smem);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(s));
}
__device__ __forceinline__ void mma_bf16(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, "
      "{%8, %9}, {%0, %1, %2, %3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack2(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}

// A (kUnit keys) x 128-d bf16 tile in shared memory: row = key (256 B), 16-byte chunk c of row r is
// stored at chunk (c ^ (r & 7)) so that ldmatrix reads of 8 consecutive rows hit 8 bank groups.
__device__ __forceinline__ uint8_t* tile_addr(uint8_t* tile, int row, int chunk) {
  return tile + row * 256 + ((chunk ^ (row & 7)) << 4);
}

// one warp copies the kUnit keys starting at `base` (one KV head); rows >= `rows` are not fetched
__device__ __forceinline__ void load_tile(uint8_t* tile, const __nv_bfloat16* base, int64_t row_stride,
                                          int rows, int lane) {
#pragma unroll 4
  for (int i = lane; i < kUnit * 16; i += 32) {
    const int row = i >> 4, chunk = i & 15;
    if (row < rows) cp_async16(tile_addr(tile, row, chunk), base + (int64_t)row * row_stride + chunk * 8);
  }
}

}  // namespace mmasync
}  // namespace ifv2
