// Cache maintenance around the decode path: the bookkeeping a serving loop does between two
// sparse-attention steps, as two bandwidth-trivial kernels instead of a handful of framework ops.
//
//   fill:   packed prefill tensors (total, heads, 128) -> per-sequence caches (batch, capacity,
//           heads, 128), rows [0, len_b) of every sequence (keys, values, compressed keys).
//   append: one decode step.  The new key / value row of every sequence goes to position
//           len_b of its cache; a sequence whose new length completes a compression window
//           (len >= kernel and (len - kernel) % stride == 0) gets that window's mean written to
//           its compressed-key cache (up to two compressions: 32/16 for the scorer, 128/64 for
//           the coarse row sums); the new lengths and compressed-key counts are written out so
//           that the next kernels of the step need no host arithmetic.
// 16-byte vectors throughout; the append kernel gives a sequence to one CTA.
#include "common.cuh"

namespace ifv2 {
namespace {

constexpr int kThreads = 256;
constexpr int kVecPerRow = kHeadDim / 8;

__device__ __forceinline__ void acc_bf16x8(float (&acc)[8], const uint4& raw) {
  const __nv_bfloat162* h2 = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 f = __bfloat1622float2(h2[i]);
    acc[2 * i] += f.x;
    acc[2 * i + 1] += f.y;
  }
}

__device__ __forceinline__ uint4 mean_bf16x8(const float (&acc)[8], float n) {
  uint4 out;
  __nv_bfloat162* o2 = reinterpret_cast<__nv_bfloat162*>(&out);
#pragma unroll
  for (int i = 0; i < 4; ++i)
    o2[i] = __floats2bfloat162_rn(__fdiv_rn(acc[2 * i], n), __fdiv_rn(acc[2 * i + 1], n));
  return out;
}

__host__ __device__ inline int windows(int len, int kernel, int stride) {
  return len >= kernel ? (len - kernel) / stride + 1 : 0;
}

struct FillParams {
  const uint4* src;            // (total, heads, 128) bf16 as 16-byte vectors
  uint4* cache;                // (batch, cap, heads, 128)
  const int32_t* cu;           // (batch + 1)
  int32_t* seqlens_out;        // (batch) or null: min(len_b, cap)
  int batch, heads;
  int64_t total, cap;
};

__global__ void __launch_bounds__(kThreads) cache_fill_kernel(const FillParams p) {
  const int64_t row_vecs = (int64_t)p.heads * kVecPerRow;
  const int64_t n_vec = p.total * row_vecs;
  for (int64_t idx = (int64_t)blockIdx.x * kThreads + threadIdx.x; idx < n_vec;
       idx += (int64_t)gridDim.x * kThreads) {
    const int64_t t = idx / row_vecs, r = idx % row_vecs;
    const int b = find_sequence(p.cu, p.batch, (int)t);
    const int64_t pos = t - p.cu[b];
    if (pos < p.cap) p.cache[((int64_t)b * p.cap + pos) * row_vecs + r] = __ldg(p.src + idx);
  }
  if (p.seqlens_out != nullptr) {
    const int64_t b = (int64_t)blockIdx.x * kThreads + threadIdx.x;
    if (b < p.batch) p.seqlens_out[b] = (int32_t)min((int64_t)(p.cu[b + 1] - p.cu[b]), p.cap);
  }
}

struct AppendParams {
  const uint4* k_new;          // (batch, heads, 128)
  const uint4* v_new;
  uint4* k_cache;              // (batch, cap, heads, 128)
  uint4* v_cache;
  uint4* kc_cache;             // (batch, c_cap, heads, 128) or null
  uint4* kc2_cache;            // (batch, c2_cap, heads, 128) or null
  int32_t* seqlens;            // (batch) in: lengths before the append, out: after it
  int32_t* positions;          // (batch) out: the lengths before the append, or null
  int32_t* n_comp;             // (batch) compressed keys after the append, or null
  int32_t* n_comp2;
  int batch, heads, kernel, stride, kernel2, stride2;
  int64_t cap, c_cap, c2_cap;
};

constexpr int kRowsPerPart = 4;      // window rows a thread fetches per round

// Mean of the last `kernel` key rows of one sequence -> dst (one compressed key, all heads).
// The CTA's threads fetch the rows of a round side by side into shared memory (one trip to
// memory per round instead of one per row); the rows are then added in token order, the order of
// compress_keys_kernel, so a window completed during decode equals the one a prefill computes.
// Called by all threads of the CTA (it synchronises).
__device__ __forceinline__ void window_mean(const uint4* k_seq, uint4* dst, int len, int kernel,
                                            int row_vecs, uint4* stage /* [kRowsPerPart * kThreads] */) {
  const int tid = threadIdx.x;
  const int cols = min(row_vecs, kThreads);             // vectors of a row handled per pass
  const int parts = kThreads / cols;                    // thread groups fetching different rows
  const int part = tid / cols, c = tid % cols;
  const int rows_per_round = parts * kRowsPerPart;      // rows_per_round * cols <= 4 * kThreads
  const uint4* first = k_seq + (int64_t)(len - kernel) * row_vecs;
  for (int c0 = 0; c0 < row_vecs; c0 += cols) {
    const int r = c0 + c;
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    for (int t0 = 0; t0 < kernel; t0 += rows_per_round) {
      if (part < parts && r < row_vecs) {
        uint4 v[kRowsPerPart];
#pragma unroll
        for (int i = 0; i < kRowsPerPart; ++i) {         // all loads of the round first
          const int t = t0 + part * kRowsPerPart + i;
          if (t < kernel) v[i] = first[(int64_t)t * row_vecs + r];
        }
#pragma unroll
        for (int i = 0; i < kRowsPerPart; ++i)
          if (t0 + part * kRowsPerPart + i < kernel) stage[(part * kRowsPerPart + i) * cols + c] = v[i];
      }
      __syncthreads();
      if (part == 0 && r < row_vecs) {
        const int rows = min(rows_per_round, kernel - t0);
        for (int t = 0; t < rows; ++t) acc_bf16x8(acc, stage[t * cols + c]);
      }
      __syncthreads();
    }
    if (part == 0 && r < row_vecs) dst[r] = mean_bf16x8(acc, (float)kernel);
  }
}

// One CTA per sequence.  The lengths are updated in place: every thread that reads a sequence's
// length sits in the CTA that later writes it, and a barrier separates the two.
__global__ void __launch_bounds__(kThreads) decode_append_kernel(const AppendParams p) {
  __shared__ uint4 stage[kRowsPerPart * kThreads];        // 16 KB
  const int row_vecs = p.heads * kVecPerRow;
  const int b = blockIdx.x;
  const int old_len = p.seqlens[b];
  __syncthreads();
  const bool room = old_len >= 0 && old_len < p.cap;      // a full cache is left untouched
  const int len = room ? old_len + 1 : old_len;
  if (room) {                                             // (uniform over the CTA)
    for (int r = threadIdx.x; r < row_vecs; r += kThreads) {
      const int64_t at = ((int64_t)b * p.cap + old_len) * row_vecs + r;
      p.k_cache[at] = __ldg(p.k_new + (int64_t)b * row_vecs + r);
      p.v_cache[at] = __ldg(p.v_new + (int64_t)b * row_vecs + r);
    }
    const bool win1 = p.kc_cache != nullptr && len >= p.kernel && (len - p.kernel) % p.stride == 0 &&
                      (len - p.kernel) / p.stride < p.c_cap;
    const bool win2 = p.kc2_cache != nullptr && len >= p.kernel2 && (len - p.kernel2) % p.stride2 == 0 &&
                      (len - p.kernel2) / p.stride2 < p.c2_cap;
    if (win1 || win2) {
      __syncthreads();                                    // the new key row is among the rows read
      const uint4* k_seq = p.k_cache + (int64_t)b * p.cap * row_vecs;
      if (win1)
        window_mean(k_seq, p.kc_cache + ((int64_t)b * p.c_cap + (len - p.kernel) / p.stride) * row_vecs,
                    len, p.kernel, row_vecs, stage);
      if (win2)
        window_mean(k_seq, p.kc2_cache + ((int64_t)b * p.c2_cap + (len - p.kernel2) / p.stride2) * row_vecs,
                    len, p.kernel2, row_vecs, stage);
    }
  }
  if (threadIdx.x == 0) {
    p.seqlens[b] = len;
    if (p.positions != nullptr) p.positions[b] = old_len;
    if (p.n_comp != nullptr)
      p.n_comp[b] = (int32_t)min((int64_t)windows(len, p.kernel, p.stride), p.c_cap);
    if (p.n_comp2 != nullptr)
      p.n_comp2[b] = (int32_t)min((int64_t)windows(len, p.kernel2, p.stride2), p.c2_cap);
  }
}

}  // namespace
}  // namespace ifv2

using namespace ifv2;

extern "C" int ifv2_cache_fill(const void* src, void* cache, const int32_t* cu_seqlens,
                               int32_t* seqlens_out, int batch, int64_t total, int64_t capacity,
                               int heads_k, int head_dim, void* stream) {
  IFV2_REQUIRE(head_dim == kHeadDim, IFV2_ERR_UNSUPPORTED,
               "cache_fill: head_dim %d not supported (only 128)", head_dim);
  IFV2_REQUIRE(batch >= 1 && heads_k >= 1 && total >= 0 && capacity >= 1, IFV2_ERR_INVALID_ARG,
               "cache_fill: bad size");
  IFV2_REQUIRE(cu_seqlens != nullptr && cache != nullptr && (src != nullptr || total == 0),
               IFV2_ERR_INVALID_ARG, "cache_fill: null pointer");
  IFV2_REQUIRE(reinterpret_cast<uintptr_t>(src) % 16 == 0 && reinterpret_cast<uintptr_t>(cache) % 16 == 0,
               IFV2_ERR_INVALID_ARG, "cache_fill: tensors must be 16-byte aligned");
  IFV2_REQUIRE(total <= INT32_MAX, IFV2_ERR_TOO_LARGE, "cache_fill: more than 2^31-1 rows");
  FillParams p{static_cast<const uint4*>(src), static_cast<uint4*>(cache), cu_seqlens, seqlens_out,
               batch, heads_k, total, capacity};
  const int64_t n_vec = total * heads_k * kVecPerRow;
  int64_t blocks = ceil_div64(n_vec > batch ? n_vec : batch, kThreads);
  const int64_t min_blocks = ceil_div64(batch, kThreads);     // the threads that write seqlens_out
  const int64_t cap = (int64_t)kNumSMs * 16;
  if (blocks > cap) blocks = cap > min_blocks ? cap : min_blocks;
  cache_fill_kernel<<<(int)blocks, kThreads, 0, (cudaStream_t)stream>>>(p);
  return check_launch("cache_fill");
}

extern "C" int ifv2_decode_append(const void* k_new, const void* v_new, void* k_cache, void* v_cache,
                                  void* kc_cache, void* kc2_cache, int32_t* cache_seqlens,
                                  int32_t* positions, int32_t* n_comp, int32_t* n_comp2, int batch,
                                  int64_t capacity, int64_t c_capacity, int64_t c2_capacity,
                                  int heads_k, int head_dim, int kernel_size, int kernel_stride,
                                  int kernel2_size, int kernel2_stride, void* stream) {
  IFV2_REQUIRE(head_dim == kHeadDim, IFV2_ERR_UNSUPPORTED,
               "decode_append: head_dim %d not supported (only 128)", head_dim);
  IFV2_REQUIRE(batch >= 1 && heads_k >= 1 && capacity >= 1, IFV2_ERR_INVALID_ARG,
               "decode_append: bad size");
  IFV2_REQUIRE(k_new && v_new && k_cache && v_cache && cache_seqlens, IFV2_ERR_INVALID_ARG,
               "decode_append: null pointer");
  IFV2_REQUIRE(cache_seqlens != positions, IFV2_ERR_INVALID_ARG,
               "decode_append: positions must not alias cache_seqlens");
  IFV2_REQUIRE(kc_cache == nullptr || (c_capacity >= 1 && kernel_size >= 1 && kernel_stride >= 1),
               IFV2_ERR_INVALID_ARG, "decode_append: bad compression arguments");
  IFV2_REQUIRE(kc2_cache == nullptr || (c2_capacity >= 1 && kernel2_size >= 1 && kernel2_stride >= 1),
               IFV2_ERR_INVALID_ARG, "decode_append: bad second compression arguments");
  IFV2_REQUIRE((n_comp == nullptr || kc_cache != nullptr) && (n_comp2 == nullptr || kc2_cache != nullptr),
               IFV2_ERR_INVALID_ARG, "decode_append: a count output needs its compressed cache");
  for (const void* ptr : {k_new, v_new, (const void*)k_cache, (const void*)v_cache,
                          (const void*)kc_cache, (const void*)kc2_cache})
    IFV2_REQUIRE(reinterpret_cast<uintptr_t>(ptr) % 16 == 0, IFV2_ERR_INVALID_ARG,
                 "decode_append: tensors must be 16-byte aligned");
  IFV2_REQUIRE(batch <= 1 << 30, IFV2_ERR_TOO_LARGE, "decode_append: batch too large");
  AppendParams p{static_cast<const uint4*>(k_new), static_cast<const uint4*>(v_new),
                 static_cast<uint4*>(k_cache), static_cast<uint4*>(v_cache),
                 static_cast<uint4*>(kc_cache), static_cast<uint4*>(kc2_cache), cache_seqlens,
                 positions, n_comp, n_comp2, batch, heads_k,
                 kc_cache ? kernel_size : 1, kc_cache ? kernel_stride : 1,
                 kc2_cache ? kernel2_size : 1, kc2_cache ? kernel2_stride : 1,
                 capacity, c_capacity, c2_capacity};
  decode_append_kernel<<<batch, kThreads, 0, (cudaStream_t)stream>>>(p);
  return check_launch("decode_append");
}
