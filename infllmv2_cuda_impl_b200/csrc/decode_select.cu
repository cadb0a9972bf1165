// Block selection for decode in one launch: 64-token max-pool of a stage-1 score row, top-k of
// the block scores and the uint64 block mask the decode kernel reads -- the work of the pool,
// top-k and pack kernels (plus the layout change between them) for the few rows a decode step
// has (batch x KV heads), where those are pure launch latency.
//
// One CTA owns one (sequence, KV head) row.  The row's scores are staged in shared memory with
// 16-byte loads (one trip to HBM instead of a chain of scalar loads).  Thread t owns the
// contiguous blocks [t*per, (t+1)*per): it pools them (5-wide, stride-4 window over the compressed-key scores,
// +inf on the init and local blocks, -inf where no key exists) into 16-bit ordered keys in shared
// memory; the CTA bisects the key space for the k-th largest value (one barrier per probe); a
// block-wide scan over (above-threshold, tie) counts then gives every selected block its output
// slot, ties going to the lowest index -- the rule of the warp-per-row kernel, so the results are
// identical to pool -> top-k -> pack run one after the other.
#include "common.cuh"

namespace ifv2 {
namespace {

constexpr int kThreads = 256;
constexpr int kWarps = kThreads / 32;
constexpr int kMaxBlocks = 8192;

struct SelectParams {
  const void* score;            // (heads, batch, row_stride) bf16 / fp16
  const int32_t* seqused_c;     // (batch) compressed keys per sequence, or null = max_seqlen_c
  const int32_t* positions;     // (batch) position of the query token in its sequence
  unsigned long long* mask;     // (batch, heads, words)
  int32_t* topk_idx;            // (batch, heads, k) or null
  int64_t row_stride;
  int batch, heads, max_seqlen_c, n_blocks, words, k, local_blocks, init_blocks, block_size;
  int pool_stride;              // block_size / compression stride (4)
  int staged_elems;             // scores of a row staged in shared memory (0 = read from global)
};

__device__ __forceinline__ float to_float(__nv_bfloat16 v) { return __bfloat162float(v); }
__device__ __forceinline__ float to_float(__half v) { return __half2float(v); }
__device__ __forceinline__ uint16_t rounded_bits(float f, __nv_bfloat16) {
  return __bfloat16_as_ushort(__float2bfloat16_rn(f));
}
__device__ __forceinline__ uint16_t rounded_bits(float f, __half) {
  return __half_as_ushort(__float2half_rn(f));
}
template <typename T> struct Inf;
template <> struct Inf<__nv_bfloat16> { static constexpr uint16_t kPos = 0x7F80; };
template <> struct Inf<__half> { static constexpr uint16_t kPos = 0x7C00; };

__device__ __forceinline__ uint32_t ordered_key(uint16_t bits, uint16_t neg_zero) {
  if (bits == neg_zero) bits = 0;                               // -0 compares equal to +0
  return (bits & 0x8000u) ? (~(uint32_t)bits & 0xFFFFu) : ((uint32_t)bits | 0x8000u);
}

template <typename T>
__global__ void __launch_bounds__(kThreads) decode_select_kernel(const SelectParams p) {
  extern __shared__ __align__(16) uint8_t dyn_smem[];          // the staged score row, if it fits
  __shared__ uint16_t keys[kMaxBlocks];
  __shared__ unsigned long long words[kMaxBlocks / 64];
  __shared__ int partial[2][kWarps];
  __shared__ int scan_gt[kWarps], scan_tie[kWarps];
  const int h = blockIdx.x, b = blockIdx.y;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const T* x = static_cast<const T*>(p.score) + ((int64_t)h * p.batch + b) * p.row_stride;
  const int k_len = p.seqused_c ? max(0, min(p.seqused_c[b], p.max_seqlen_c)) : p.max_seqlen_c;
  const int bq = p.positions[b] / p.block_size;
  const int n = p.n_blocks;
  const int per = (n + kThreads - 1) / kThreads;
  const int i0 = min(tid * per, n), i1 = min(i0 + per, n);
  constexpr uint16_t kPosInf = Inf<T>::kPos, kNegInf = Inf<T>::kPos | 0x8000;

  for (int w = tid; w < p.words; w += kThreads) words[w] = 0ull;
  // ---- stage the row (only whole 16-byte vectors below k_len rounded up: the row's padding up to
  // row_stride may be read, nothing past it)
  const T* xs = x;
  if (p.staged_elems > 0) {
    const int n_vec = min((k_len + 7) / 8, p.staged_elems / 8);
    uint4* dst = reinterpret_cast<uint4*>(dyn_smem);
    for (int v = tid; v < n_vec; v += kThreads) dst[v] = __ldg(reinterpret_cast<const uint4*>(x) + v);
    __syncthreads();
    xs = reinterpret_cast<const T*>(dyn_smem);
  }
  const bool from_smem = p.staged_elems > 0;
  // ---- pool: block i <- max x[s*i - 1 .. s*i + s - 1] (kernel s + 1, stride s, padding 1)
  for (int i = i0; i < i1; ++i) {
    uint16_t bits;
    if (i < p.init_blocks || (bq >= i && bq <= i + p.local_blocks)) {
      bits = kPosInf;
    } else {
      const int s = max(i * p.pool_stride - 1, 0), e = min(i * p.pool_stride + p.pool_stride, k_len);
      float m = -INFINITY;
      if (from_smem) {
        for (int j = s; j < e; ++j) m = fmaxf(m, to_float(xs[j]));
      } else {
        for (int j = s; j < e; ++j) m = fmaxf(m, to_float(ldg16(x + j)));
      }
      bits = rounded_bits(m, T());                     // exact: m is one of the inputs or -inf
    }
    keys[i] = (uint16_t)ordered_key(bits, 0x8000);
  }
  __syncthreads();

  // ---- bisection for the k_eff-th largest key
  const int k_eff = min(p.k, n);
  uint32_t lo = ordered_key(kNegInf, 0x8000), hi = ordered_key(kPosInf, 0x8000) + 1u;
  int it = 0;
  while (hi - lo > 1u) {
    const uint32_t mid = (lo + hi) >> 1;
    int c = 0;
    for (int i = i0; i < i1; ++i) c += keys[i] >= mid;
    c = __reduce_add_sync(0xFFFFFFFFu, c);
    if (lane == 0) partial[it & 1][warp] = c;
    __syncthreads();                                   // (the other buffer is free again by now)
    int cnt = 0;
#pragma unroll
    for (int w = 0; w < kWarps; ++w) cnt += partial[it & 1][w];
    if (cnt >= k_eff) lo = mid; else hi = mid;
    ++it;
  }
  // ---- slots: everything above the threshold, then ties lowest index first
  int gt = 0, tie = 0;
  for (int i = i0; i < i1; ++i) {
    gt += keys[i] > lo;
    tie += keys[i] == lo;
  }
  int gt_scan = gt, tie_scan = tie;
#pragma unroll
  for (int d = 1; d < 32; d <<= 1) {
    const int a = __shfl_up_sync(0xFFFFFFFFu, gt_scan, d), t = __shfl_up_sync(0xFFFFFFFFu, tie_scan, d);
    if (lane >= d) { gt_scan += a; tie_scan += t; }
  }
  if (lane == 31) { scan_gt[warp] = gt_scan; scan_tie[warp] = tie_scan; }
  __syncthreads();
  int gt_before = gt_scan - gt, tie_before = tie_scan - tie, gt_total = 0;
#pragma unroll
  for (int w = 0; w < kWarps; ++w) {
    if (w < warp) { gt_before += scan_gt[w]; tie_before += scan_tie[w]; }
    gt_total += scan_gt[w];
  }
  const int need = k_eff - gt_total;                   // ties to take (>= 1 unless k_eff == 0)
  int32_t* out_idx = p.topk_idx ? p.topk_idx + ((int64_t)b * p.heads + h) * p.k : nullptr;
  for (int i = i0; i < i1; ++i) {
    const bool g = keys[i] > lo, t = keys[i] == lo;
    if (g || (t && tie_before < need)) {
      const int pos = gt_before + min(tie_before, need);
      const bool keep = i <= bq;                       // later blocks only ever come out as -1
      if (out_idx != nullptr && pos < p.k) out_idx[pos] = keep ? i : -1;
      if (keep && (i >> 6) < p.words) atomicOr(&words[i >> 6], 1ull << (i & 63));
    }
    gt_before += g;
    tie_before += t;
  }
  if (out_idx != nullptr)
    for (int i = k_eff + tid; i < p.k; i += kThreads) out_idx[i] = -1;
  __syncthreads();
  unsigned long long* mrow = p.mask + ((int64_t)b * p.heads + h) * p.words;
  for (int w = tid; w < p.words; w += kThreads) mrow[w] = words[w];
}

}  // namespace
}  // namespace ifv2

using namespace ifv2;

extern "C" int ifv2_decode_select(const void* score, int is_bf16, int64_t row_stride,
                                  const int32_t* seqused_c, const int32_t* positions, int64_t* mask,
                                  int32_t* topk_idx, int batch, int heads, int max_seqlen_c,
                                  int n_blocks, int mask_words, int k, int local_blocks,
                                  int init_blocks, int block_size, int stride, void* stream) {
  IFV2_REQUIRE(batch >= 0 && heads >= 0 && max_seqlen_c >= 0 && n_blocks >= 0 && k >= 0 &&
                   mask_words >= 0 && local_blocks >= 0 && init_blocks >= 0,
               IFV2_ERR_INVALID_ARG, "decode_select: negative size");
  IFV2_REQUIRE(block_size >= 1 && stride >= 1 && block_size % stride == 0, IFV2_ERR_INVALID_ARG,
               "decode_select: block_size must be a multiple of the compression stride");
  IFV2_REQUIRE(n_blocks <= kMaxBlocks, IFV2_ERR_TOO_LARGE,
               "decode_select: n_blocks = %d exceeds the %d-block limit", n_blocks, kMaxBlocks);
  IFV2_REQUIRE(mask_words <= kMaxBlocks / 64, IFV2_ERR_TOO_LARGE, "decode_select: more than %d mask words",
               kMaxBlocks / 64);
  IFV2_REQUIRE(row_stride >= max_seqlen_c, IFV2_ERR_INVALID_ARG, "decode_select: row_stride < max_seqlen_c");
  IFV2_REQUIRE(batch <= 65535, IFV2_ERR_TOO_LARGE, "decode_select: batch > 65535");
  if (batch == 0 || heads == 0 || mask_words == 0) return IFV2_OK;
  IFV2_REQUIRE(positions && mask && (score || max_seqlen_c == 0), IFV2_ERR_INVALID_ARG,
               "decode_select: null pointer");
  // stage the row when it is 16-byte aligned throughout and fits (rows of up to 32768 scores do)
  const int padded = ((max_seqlen_c + 7) / 8) * 8;
  const bool stage = reinterpret_cast<uintptr_t>(score) % 16 == 0 && row_stride % 8 == 0 &&
                     padded <= row_stride && padded * 2 <= 64 * 1024;
  SelectParams p{score, seqused_c, positions, reinterpret_cast<unsigned long long*>(mask), topk_idx,
                 row_stride, batch, heads, max_seqlen_c, n_blocks, mask_words, k, local_blocks,
                 init_blocks, block_size, block_size / stride, stage ? padded : 0};
  const size_t smem = stage ? (size_t)padded * 2 : 0;
  const dim3 grid(heads, batch);
  cudaError_t e = cudaSuccess;
  if (is_bf16) {
    if (smem > 24 * 1024)
      e = cudaFuncSetAttribute(decode_select_kernel<__nv_bfloat16>,
                               cudaFuncAttributeMaxDynamicSharedMemorySize, 64 * 1024);
    if (e != cudaSuccess) return set_error((int)e, "decode_select: %s", cudaGetErrorString(e));
    decode_select_kernel<__nv_bfloat16><<<grid, kThreads, smem, (cudaStream_t)stream>>>(p);
  } else {
    if (smem > 24 * 1024)
      e = cudaFuncSetAttribute(decode_select_kernel<__half>,
                               cudaFuncAttributeMaxDynamicSharedMemorySize, 64 * 1024);
    if (e != cudaSuccess) return set_error((int)e, "decode_select: %s", cudaGetErrorString(e));
    decode_select_kernel<__half><<<grid, kThreads, smem, (cudaStream_t)stream>>>(p);
  }
  return check_launch("decode_select");
}
