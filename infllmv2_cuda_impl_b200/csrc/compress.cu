// Key compression: the step in front of the stage-1 scorer.  Compressed key j of a sequence is
// the mean of the keys of tokens [stride*j, stride*j + kernel) (only full windows), per KV head
// and feature: kernel 32 / stride 16 for the scorer, 128 / 64 for the coarse variant.  HBM-bound:
// every key row is read once from DRAM (the overlapping second read of a window comes from L2).
// One thread owns 8 features (16 bytes) of one compressed key and head and walks the window with
// 16-byte loads; consecutive threads cover the contiguous (head, feature) row of a token, so a
// warp reads 512 contiguous bytes per window step.  fp32 accumulation, one rounding to bf16.
#include "common.cuh"

namespace ifv2 {
namespace {

constexpr int kThreads = 256;
constexpr int kVecPerRow = kHeadDim / 8;      // 16-byte vectors per (token, head) row

__device__ __forceinline__ void add_bf16x8(float (&acc)[8], const uint4& raw) {
  const __nv_bfloat162* h2 = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 f = __bfloat1622float2(h2[i]);
    acc[2 * i] += f.x;
    acc[2 * i + 1] += f.y;
  }
}

__device__ __forceinline__ uint4 mean_to_bf16x8(const float (&acc)[8], float n) {
  uint4 out;
  __nv_bfloat162* o2 = reinterpret_cast<__nv_bfloat162*>(&out);
#pragma unroll
  for (int i = 0; i < 4; ++i) o2[i] = __floats2bfloat162_rn(__fdiv_rn(acc[2 * i], n), __fdiv_rn(acc[2 * i + 1], n));
  return out;
}

struct CompressParams {
  const __nv_bfloat16* k;      // (total_k, heads, 128)
  __nv_bfloat16* kc;           // (total_c, heads, 128)
  const int32_t* cu_k;         // (batch + 1) or null = one sequence starting at 0
  const int32_t* cu_c;         // (batch + 1) or null
  int batch, heads, kernel, stride;
  int64_t total_c;
};

__global__ void __launch_bounds__(kThreads) compress_keys_kernel(const CompressParams p) {
  const int64_t n_vec = p.total_c * p.heads * kVecPerRow;
  for (int64_t idx = (int64_t)blockIdx.x * kThreads + threadIdx.x; idx < n_vec;
       idx += (int64_t)gridDim.x * kThreads) {
    const int v = (int)(idx % kVecPerRow);
    const int h = (int)((idx / kVecPerRow) % p.heads);
    const int64_t j = idx / ((int64_t)kVecPerRow * p.heads);
    int64_t tok0;
    if (p.cu_c != nullptr) {
      const int b = find_sequence(p.cu_c, p.batch, (int)j);
      tok0 = (int64_t)p.cu_k[b] + (j - p.cu_c[b]) * p.stride;
    } else {
      tok0 = j * p.stride;
    }
    const __nv_bfloat16* src = p.k + (tok0 * p.heads + h) * kHeadDim + v * 8;
    const int64_t row = (int64_t)p.heads * kHeadDim;
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    int t = 0;
    for (; t + 4 <= p.kernel; t += 4) {        // four loads in flight per thread
      const uint4 a = __ldg(reinterpret_cast<const uint4*>(src + (t + 0) * row));
      const uint4 b4 = __ldg(reinterpret_cast<const uint4*>(src + (t + 1) * row));
      const uint4 c = __ldg(reinterpret_cast<const uint4*>(src + (t + 2) * row));
      const uint4 d = __ldg(reinterpret_cast<const uint4*>(src + (t + 3) * row));
      add_bf16x8(acc, a);
      add_bf16x8(acc, b4);
      add_bf16x8(acc, c);
      add_bf16x8(acc, d);
    }
    for (; t < p.kernel; ++t) add_bf16x8(acc, __ldg(reinterpret_cast<const uint4*>(src + t * row)));
    *reinterpret_cast<uint4*>(p.kc + (j * p.heads + h) * kHeadDim + v * 8) =
        mean_to_bf16x8(acc, (float)p.kernel);
  }
}

struct AppendParams {
  const __nv_bfloat16* k_cache;   // (batch, cap, heads, 128)
  __nv_bfloat16* kc_cache;        // (batch, c_cap, heads, 128)
  const int32_t* cache_seqlens;   // (batch) lengths AFTER the append
  int batch, heads, kernel, stride;
  int64_t cap, c_cap;
};

// Decode-time update: a sequence whose length just reached kernel + stride*j completes window j.
__global__ void __launch_bounds__(kThreads) compress_keys_append_kernel(const AppendParams p) {
  const int64_t n_vec = (int64_t)p.batch * p.heads * kVecPerRow;
  const int64_t idx = (int64_t)blockIdx.x * kThreads + threadIdx.x;
  if (idx >= n_vec) return;
  const int v = (int)(idx % kVecPerRow);
  const int h = (int)((idx / kVecPerRow) % p.heads);
  const int b = (int)(idx / ((int64_t)kVecPerRow * p.heads));
  const int len = p.cache_seqlens[b];
  if (len < p.kernel || len > p.cap || (len - p.kernel) % p.stride != 0) return;
  const int64_t j = (len - p.kernel) / p.stride;
  if (j >= p.c_cap) return;
  const int64_t row = (int64_t)p.heads * kHeadDim;
  const __nv_bfloat16* src =
      p.k_cache + (((int64_t)b * p.cap + (len - p.kernel)) * p.heads + h) * kHeadDim + v * 8;
  float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
  for (int t = 0; t < p.kernel; ++t)
    add_bf16x8(acc, __ldg(reinterpret_cast<const uint4*>(src + t * row)));
  *reinterpret_cast<uint4*>(p.kc_cache + (((int64_t)b * p.c_cap + j) * p.heads + h) * kHeadDim + v * 8) =
      mean_to_bf16x8(acc, (float)p.kernel);
}

}  // namespace
}  // namespace ifv2

using namespace ifv2;

extern "C" int ifv2_compress_keys(const void* k, void* kc, const int32_t* cu_seqlens_k,
                                  const int32_t* cu_seqlens_c, int batch, int64_t total_k,
                                  int64_t total_c, int heads_k, int head_dim, int kernel_size,
                                  int kernel_stride, void* stream) {
  IFV2_REQUIRE(head_dim == kHeadDim, IFV2_ERR_UNSUPPORTED,
               "compress_keys: head_dim %d not supported (only 128)", head_dim);
  IFV2_REQUIRE(batch >= 1 && heads_k >= 1 && total_k >= 0 && total_c >= 0 && kernel_size >= 1 &&
                   kernel_stride >= 1,
               IFV2_ERR_INVALID_ARG, "compress_keys: bad size");
  IFV2_REQUIRE((cu_seqlens_k == nullptr) == (cu_seqlens_c == nullptr), IFV2_ERR_INVALID_ARG,
               "compress_keys: cu_seqlens_k and cu_seqlens_c go together");
  if (total_c == 0) return IFV2_OK;
  IFV2_REQUIRE(k && kc, IFV2_ERR_INVALID_ARG, "compress_keys: null pointer");
  IFV2_REQUIRE(reinterpret_cast<uintptr_t>(k) % 16 == 0 && reinterpret_cast<uintptr_t>(kc) % 16 == 0,
               IFV2_ERR_INVALID_ARG, "compress_keys: tensors must be 16-byte aligned");
  IFV2_REQUIRE(total_k <= INT32_MAX && total_c <= INT32_MAX, IFV2_ERR_TOO_LARGE,
               "compress_keys: more than 2^31-1 rows");
  if (cu_seqlens_k == nullptr)
    IFV2_REQUIRE(batch == 1 && (total_c - 1) * kernel_stride + kernel_size <= total_k,
                 IFV2_ERR_INVALID_ARG, "compress_keys: windows reach past the %lld keys",
                 (long long)total_k);
  CompressParams p{static_cast<const __nv_bfloat16*>(k), static_cast<__nv_bfloat16*>(kc),
                   cu_seqlens_k, cu_seqlens_c, batch, heads_k, kernel_size, kernel_stride, total_c};
  const int64_t n_vec = total_c * heads_k * kVecPerRow;
  int64_t blocks = ceil_div64(n_vec, kThreads);
  const int64_t cap = (int64_t)kNumSMs * 16;
  if (blocks > cap) blocks = cap;
  compress_keys_kernel<<<(int)blocks, kThreads, 0, (cudaStream_t)stream>>>(p);
  return check_launch("compress_keys");
}

extern "C" int ifv2_compress_keys_append(const void* k_cache, void* kc_cache,
                                         const int32_t* cache_seqlens, int batch,
                                         int64_t cache_capacity, int64_t compressed_capacity,
                                         int heads_k, int head_dim, int kernel_size,
                                         int kernel_stride, void* stream) {
  IFV2_REQUIRE(head_dim == kHeadDim, IFV2_ERR_UNSUPPORTED,
               "compress_keys_append: head_dim %d not supported (only 128)", head_dim);
  IFV2_REQUIRE(batch >= 1 && heads_k >= 1 && cache_capacity >= 1 && compressed_capacity >= 0 &&
                   kernel_size >= 1 && kernel_stride >= 1,
               IFV2_ERR_INVALID_ARG, "compress_keys_append: bad size");
  IFV2_REQUIRE(k_cache && kc_cache && cache_seqlens, IFV2_ERR_INVALID_ARG,
               "compress_keys_append: null pointer");
  AppendParams p{static_cast<const __nv_bfloat16*>(k_cache), static_cast<__nv_bfloat16*>(kc_cache),
                 cache_seqlens, batch, heads_k, kernel_size, kernel_stride, cache_capacity,
                 compressed_capacity};
  const int64_t n_vec = (int64_t)batch * heads_k * kVecPerRow;
  compress_keys_append_kernel<<<(int)ceil_div64(n_vec, kThreads), kThreads, 0, (cudaStream_t)stream>>>(p);
  return check_launch("compress_keys_append");
}
