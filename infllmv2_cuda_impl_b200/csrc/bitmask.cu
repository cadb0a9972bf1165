// Bitmask kernels: top-k list -> uint64 rows, bool <-> uint64, and the row->column mask
// transpose.  All are HBM-bound byte/bit shuffles: coalesced vector access, warp ballots and
// reductions, no tensor cores.
#include "common.cuh"

namespace ifv2 {
namespace {

constexpr int kThreads = 256;
constexpr int kWarps = kThreads / 32;

// One warp per row: the row's indices are OR-ed into a per-warp word array in shared memory,
// which is then written out whole (so the output needs no pre-zeroing).
__global__ void __launch_bounds__(kThreads)
topk_to_uint64_kernel(const int32_t* __restrict__ idx, unsigned long long* __restrict__ out,
                      int64_t rows, int k, int words) {
  extern __shared__ unsigned long long smem_words[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  unsigned long long* w = smem_words + (size_t)warp * words;
  const int limit = words * 64;
  const bool vec4 = (k & 3) == 0;
  for (int64_t row = (int64_t)blockIdx.x * kWarps + warp; row < rows;
       row += (int64_t)gridDim.x * kWarps) {
    for (int i = lane; i < words; i += 32) w[i] = 0ull;
    __syncwarp();
    const int32_t* r = idx + row * k;
    if (vec4) {
      const int4* r4 = reinterpret_cast<const int4*>(r);
      for (int i = lane; i < (k >> 2); i += 32) {
        int4 v = __ldg(r4 + i);
        int e[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
        for (int j = 0; j < 4; ++j)
          if (e[j] >= 0 && e[j] < limit) atomicOr(&w[e[j] >> 6], 1ull << (e[j] & 63));
      }
    } else {
      for (int i = lane; i < k; i += 32) {
        int v = __ldg(r + i);
        if (v >= 0 && v < limit) atomicOr(&w[v >> 6], 1ull << (v & 63));
      }
    }
    __syncwarp();
    unsigned long long* o = out + row * words;
    for (int i = lane; i < words; i += 32) o[i] = w[i];
    __syncwarp();
  }
}

// V bytes of bools per lane -> V bits; 32/V lanes make one 32-bit half word.
template <int V>
__device__ __forceinline__ uint32_t bools_to_bits(const uint8_t* p);

template <>
__device__ __forceinline__ uint32_t bools_to_bits<4>(const uint8_t* p) {
  uint32_t x = __ldg(reinterpret_cast<const uint32_t*>(p));
  uint32_t m = __vcmpne4(x, 0u) & 0x01010101u;
  return (m * 0x01020408u) >> 24;   // byte j != 0 -> bit j (no carries: every product bit has one source)
}

template <>
__device__ __forceinline__ uint32_t bools_to_bits<16>(const uint8_t* p) {
  uint4 x = __ldg(reinterpret_cast<const uint4*>(p));
  uint32_t b0 = ((__vcmpne4(x.x, 0u) & 0x01010101u) * 0x01020408u) >> 24;
  uint32_t b1 = ((__vcmpne4(x.y, 0u) & 0x01010101u) * 0x01020408u) >> 24;
  uint32_t b2 = ((__vcmpne4(x.z, 0u) & 0x01010101u) * 0x01020408u) >> 24;
  uint32_t b3 = ((__vcmpne4(x.w, 0u) & 0x01010101u) * 0x01020408u) >> 24;
  return b0 | (b1 << 4) | (b2 << 8) | (b3 << 12);
}

// Vector path: last_dim % V == 0 so every lane's V-byte group is aligned and entirely inside
// or outside the row.  A warp converts 32*V consecutive elements (= V/2 words) per step.
template <int V>
__global__ void __launch_bounds__(kThreads)
blockmask_to_uint64_vec_kernel(const uint8_t* __restrict__ mask, uint32_t* __restrict__ out32,
                               int64_t rows, int64_t last_dim, int64_t words) {
  constexpr int G = 32 / V;                        // lanes per 32-bit half word
  constexpr int kElemsPerStep = 32 * V;
  const int lane = threadIdx.x & 31;
  const int64_t steps_per_row = (words * 64 + kElemsPerStep - 1) / kElemsPerStep;
  const int64_t total = rows * steps_per_row;
  const int64_t warp0 = (int64_t)blockIdx.x * kWarps + (threadIdx.x >> 5);
  const uint32_t gmask = (G == 32 ? 0xFFFFFFFFu : ((1u << G) - 1u)) << (lane - lane % G);
  for (int64_t s = warp0; s < total; s += (int64_t)gridDim.x * kWarps) {
    const int64_t row = s / steps_per_row, step = s - row * steps_per_row;
    const int64_t e = step * kElemsPerStep + (int64_t)lane * V;      // first element of this lane
    uint32_t bits = 0;
    if (e < last_dim) bits = bools_to_bits<V>(mask + row * last_dim + e);
    uint32_t half = __reduce_or_sync(gmask, bits << (V * (lane % G)));
    const int64_t half_idx = step * (kElemsPerStep / 32) + lane / G;  // 32-bit half within the row
    if (lane % G == 0 && half_idx < words * 2) out32[row * words * 2 + half_idx] = half;
  }
}

// Generic path (any last_dim): byte loads + ballots, one 64-bit word per warp step.
__global__ void __launch_bounds__(kThreads)
blockmask_to_uint64_kernel(const uint8_t* __restrict__ mask, unsigned long long* __restrict__ out,
                           int64_t rows, int64_t last_dim, int64_t words) {
  const int lane = threadIdx.x & 31;
  const int64_t total = rows * words;
  const int64_t warp0 = (int64_t)blockIdx.x * kWarps + (threadIdx.x >> 5);
  for (int64_t s = warp0; s < total; s += (int64_t)gridDim.x * kWarps) {
    const int64_t row = s / words, w = s - row * words;
    const uint8_t* p = mask + row * last_dim;
    const int64_t e0 = w * 64 + lane, e1 = e0 + 32;
    uint32_t lo = __ballot_sync(0xFFFFFFFFu, e0 < last_dim && __ldg(p + e0) != 0);
    uint32_t hi = __ballot_sync(0xFFFFFFFFu, e1 < last_dim && __ldg(p + e1) != 0);
    if (lane == 0) out[s] = (unsigned long long)lo | ((unsigned long long)hi << 32);
  }
}

__device__ __forceinline__ uint32_t nibble_to_bytes(uint32_t n) {
  return (n & 1u) | ((n & 2u) << 7) | ((n & 4u) << 14) | ((n & 8u) << 21);
}

// One thread per V output bytes (V in {16, 4, 1}); V > 1 needs last_dim % V == 0.
template <int V>
__global__ void __launch_bounds__(kThreads)
uint64_to_bool_kernel(const unsigned long long* __restrict__ in, uint8_t* __restrict__ out,
                      int64_t rows, int64_t last_dim, int64_t words) {
  const int64_t per_row = last_dim / V;
  const int64_t total = rows * per_row;
  for (int64_t i = (int64_t)blockIdx.x * kThreads + threadIdx.x; i < total;
       i += (int64_t)gridDim.x * kThreads) {
    const int64_t row = i / per_row, c = (i - row * per_row) * V;
    const unsigned long long w = __ldg(in + row * words + (c >> 6));
    const uint32_t bits = (uint32_t)(w >> (c & 63));
    uint8_t* o = out + row * last_dim + c;
    if constexpr (V == 16) {
      uint4 r;
      r.x = nibble_to_bytes(bits & 0xF);
      r.y = nibble_to_bytes((bits >> 4) & 0xF);
      r.z = nibble_to_bytes((bits >> 8) & 0xF);
      r.w = nibble_to_bytes((bits >> 12) & 0xF);
      *reinterpret_cast<uint4*>(o) = r;
    } else if constexpr (V == 4) {
      *reinterpret_cast<uint32_t*>(o) = nibble_to_bytes(bits & 0xF);
    } else {
      *o = (uint8_t)(bits & 1u);
    }
  }
}

// 64x64 bit-matrix transpose per warp.  grid = (words_k, ceil(words_t / 8), heads); warp i of
// the CTA owns token tile 8*blockIdx.y + i; the 64 result words of the eight warps are staged
// in shared memory so each output row receives 64 contiguous bytes.
__global__ void __launch_bounds__(kThreads)
transpose_blockmask_kernel(const unsigned long long* __restrict__ in,
                           unsigned long long* __restrict__ out, int64_t tokens, int k_blocks,
                           int words_k, int64_t words_t) {
  __shared__ unsigned long long tile[64][kWarps + 1];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int w = blockIdx.x, h = blockIdx.z;
  const int64_t tt = (int64_t)blockIdx.y * kWarps + warp;
  const unsigned long long* src = in + (int64_t)h * tokens * words_k;
  const int64_t t0 = tt * 64 + lane, t1 = t0 + 32;
  const unsigned long long a = (t0 < tokens) ? __ldg(src + t0 * words_k + w) : 0ull;
  const unsigned long long b = (t1 < tokens) ? __ldg(src + t1 * words_k + w) : 0ull;
  unsigned long long r0 = 0, r1 = 0;            // words for block bits `lane` and `lane + 32`
#pragma unroll
  for (int j = 0; j < 32; ++j) {
    uint32_t lo = __ballot_sync(0xFFFFFFFFu, (a >> j) & 1ull);
    uint32_t hi = __ballot_sync(0xFFFFFFFFu, (b >> j) & 1ull);
    if (lane == j) r0 = (unsigned long long)lo | ((unsigned long long)hi << 32);
    lo = __ballot_sync(0xFFFFFFFFu, (a >> (j + 32)) & 1ull);
    hi = __ballot_sync(0xFFFFFFFFu, (b >> (j + 32)) & 1ull);
    if (lane == j) r1 = (unsigned long long)lo | ((unsigned long long)hi << 32);
  }
  tile[lane][warp] = r0;
  tile[lane + 32][warp] = r1;
  __syncthreads();
  unsigned long long* dst = out + (int64_t)h * k_blocks * words_t;
#pragma unroll
  for (int r = 0; r < (64 * kWarps) / kThreads; ++r) {
    const int idx = threadIdx.x + r * kThreads;
    const int j = idx / kWarps, i = idx % kWarps;
    const int blk = w * 64 + j;
    const int64_t ot = (int64_t)blockIdx.y * kWarps + i;
    if (blk < k_blocks && ot < words_t) dst[(int64_t)blk * words_t + ot] = tile[j][i];
  }
}

inline int grid_for(int64_t work_items, int per_block) {
  int64_t blocks = ceil_div64(work_items, per_block);
  const int64_t cap = (int64_t)kNumSMs * 16;            // grid-stride beyond this
  if (blocks > cap) blocks = cap;
  if (blocks < 1) blocks = 1;
  return (int)blocks;
}

}  // namespace
}  // namespace ifv2

using namespace ifv2;

extern "C" int ifv2_topk_to_uint64(const int32_t* topk_idx, int64_t* out_words, int64_t rows, int k,
                                   int k_blocks, int words, void* stream) {
  IFV2_REQUIRE(rows >= 0 && k >= 0 && words >= 0 && k_blocks >= 0, IFV2_ERR_INVALID_ARG,
               "topk_to_uint64: negative size");
  if (rows == 0 || words == 0) return IFV2_OK;
  IFV2_REQUIRE(topk_idx != nullptr || k == 0, IFV2_ERR_INVALID_ARG, "topk_to_uint64: null input");
  IFV2_REQUIRE(out_words != nullptr, IFV2_ERR_INVALID_ARG, "topk_to_uint64: null output");
  IFV2_REQUIRE(words == (k_blocks + 63) / 64, IFV2_ERR_INVALID_ARG,
               "topk_to_uint64: words (%d) != ceil(k_blocks / 64) (k_blocks = %d)", words, k_blocks);
  const size_t smem = (size_t)kWarps * words * sizeof(unsigned long long);
  IFV2_REQUIRE(smem <= 48 * 1024, IFV2_ERR_TOO_LARGE,
               "topk_to_uint64: %d words per row exceed the 768-word limit", words);
  topk_to_uint64_kernel<<<grid_for(rows, kWarps), kThreads, smem, (cudaStream_t)stream>>>(
      topk_idx, reinterpret_cast<unsigned long long*>(out_words), rows, k, words);
  return check_launch("topk_to_uint64");
}

extern "C" int ifv2_blockmask_to_uint64(const uint8_t* mask, int64_t* out_words, int64_t rows,
                                        int64_t last_dim, int64_t words, void* stream) {
  IFV2_REQUIRE(rows >= 0 && last_dim >= 0 && words >= 0, IFV2_ERR_INVALID_ARG,
               "blockmask_to_uint64: negative size");
  if (rows == 0 || words == 0) return IFV2_OK;
  IFV2_REQUIRE(mask != nullptr && out_words != nullptr, IFV2_ERR_INVALID_ARG,
               "blockmask_to_uint64: null pointer");
  IFV2_REQUIRE(words == (last_dim + 63) / 64, IFV2_ERR_INVALID_ARG,
               "blockmask_to_uint64: words != ceil(last_dim / 64)");
  cudaStream_t st = (cudaStream_t)stream;
  const bool a16 = (last_dim % 16 == 0) && (reinterpret_cast<uintptr_t>(mask) % 16 == 0);
  const bool a4 = (last_dim % 4 == 0) && (reinterpret_cast<uintptr_t>(mask) % 4 == 0);
  if (a16) {
    const int64_t steps = rows * ceil_div64(words * 64, 512);
    blockmask_to_uint64_vec_kernel<16><<<grid_for(steps, kWarps), kThreads, 0, st>>>(
        mask, reinterpret_cast<uint32_t*>(out_words), rows, last_dim, words);
  } else if (a4) {
    const int64_t steps = rows * ceil_div64(words * 64, 128);
    blockmask_to_uint64_vec_kernel<4><<<grid_for(steps, kWarps), kThreads, 0, st>>>(
        mask, reinterpret_cast<uint32_t*>(out_words), rows, last_dim, words);
  } else {
    blockmask_to_uint64_kernel<<<grid_for(rows * words, kWarps), kThreads, 0, st>>>(
        mask, reinterpret_cast<unsigned long long*>(out_words), rows, last_dim, words);
  }
  return check_launch("blockmask_to_uint64");
}

extern "C" int ifv2_uint64_to_bool(const int64_t* in_words, uint8_t* out_mask, int64_t rows,
                                   int64_t last_dim, int64_t words, void* stream) {
  IFV2_REQUIRE(rows >= 0 && last_dim >= 0 && words >= 0, IFV2_ERR_INVALID_ARG,
               "uint64_to_bool: negative size");
  if (rows == 0 || last_dim == 0) return IFV2_OK;
  IFV2_REQUIRE(in_words != nullptr && out_mask != nullptr, IFV2_ERR_INVALID_ARG,
               "uint64_to_bool: null pointer");
  IFV2_REQUIRE(last_dim <= words * 64, IFV2_ERR_INVALID_ARG,
               "uint64_to_bool: last_dim (%lld) exceeds 64 * words (%lld)", (long long)last_dim,
               (long long)words);
  cudaStream_t st = (cudaStream_t)stream;
  const auto* in = reinterpret_cast<const unsigned long long*>(in_words);
  const uintptr_t addr = reinterpret_cast<uintptr_t>(out_mask);
  if (last_dim % 16 == 0 && addr % 16 == 0) {
    uint64_to_bool_kernel<16><<<grid_for(rows * (last_dim / 16), kThreads), kThreads, 0, st>>>(
        in, out_mask, rows, last_dim, words);
  } else if (last_dim % 4 == 0 && addr % 4 == 0) {
    uint64_to_bool_kernel<4><<<grid_for(rows * (last_dim / 4), kThreads), kThreads, 0, st>>>(
        in, out_mask, rows, last_dim, words);
  } else {
    uint64_to_bool_kernel<1><<<grid_for(rows * last_dim, kThreads), kThreads, 0, st>>>(
        in, out_mask, rows, last_dim, words);
  }
  return check_launch("uint64_to_bool");
}

extern "C" int ifv2_transpose_blockmask(const int64_t* fwd_words, int64_t* bwd_words, int heads,
                                        int64_t tokens, int k_blocks, void* stream) {
  IFV2_REQUIRE(heads >= 0 && tokens >= 0 && k_blocks >= 0, IFV2_ERR_INVALID_ARG,
               "transpose_blockmask: negative size");
  if (heads == 0 || tokens == 0 || k_blocks == 0) return IFV2_OK;
  IFV2_REQUIRE(fwd_words != nullptr && bwd_words != nullptr, IFV2_ERR_INVALID_ARG,
               "transpose_blockmask: null pointer");
  const int words_k = (k_blocks + 63) / 64;
  const int64_t words_t = (tokens + 63) / 64;
  const int64_t gy = ceil_div64(words_t, kWarps);
  IFV2_REQUIRE(gy <= 65535 && heads <= 65535, IFV2_ERR_TOO_LARGE,
               "transpose_blockmask: more than 33.5M tokens or 65535 heads");
  dim3 grid(words_k, (unsigned)gy, heads);
  transpose_blockmask_kernel<<<grid, kThreads, 0, (cudaStream_t)stream>>>(
      reinterpret_cast<const unsigned long long*>(fwd_words),
      reinterpret_cast<unsigned long long*>(bwd_words), tokens, k_blocks, words_k, words_t);
  return check_launch("transpose_blockmask");
}
