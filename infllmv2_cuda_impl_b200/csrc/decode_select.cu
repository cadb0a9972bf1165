// Block selection for decode in one launch: 64-token max-pool of a stage-1 score row, top-k of
// the block scores and the uint64 block mask the decode kernel reads -- the work of the pool,
// top-k and pack kernels (plus the layout change between them) for the few rows a decode step
// has (batch x KV heads), where those are pure launch latency.
//
// One CTA owns one (sequence, KV head) row.  The row's scores are staged in shared memory with
// 16-byte loads (one trip to HBM instead of a chain of scalar loads); the selection itself is
// dsel::select_row (decode_select.cuh).
#include "decode_select.cuh"
#include "mma_sync.cuh"

namespace ifv2 {
namespace {

using namespace dsel;

struct SelectParams {
  const void* score;            // (heads, batch, row_stride) bf16 / fp16
  const int32_t* seqused_c;     // (batch) compressed keys per sequence, or null = max_seqlen_c
  const int32_t* positions;     // (batch) position of the query token in its sequence
  unsigned long long* mask;     // (batch, heads, words)
  int32_t* topk_idx;            // (batch, heads, k) or null
  int64_t row_stride;
  int batch, heads, max_seqlen_c, block_size;
  int staged_elems;             // scores of a row staged in shared memory (0 = read from global)
  Args a;
};

template <typename T>
__global__ void __launch_bounds__(kThreads) decode_select_kernel(const SelectParams p) {
  extern __shared__ __align__(16) uint8_t dyn_smem[];          // the staged score row, if it fits
  __shared__ Smem sm;
  const int h = blockIdx.x, b = blockIdx.y, tid = threadIdx.x;
  const T* x = static_cast<const T*>(p.score) + ((int64_t)h * p.batch + b) * p.row_stride;
  const int k_len = p.seqused_c ? max(0, min(p.seqused_c[b], p.max_seqlen_c)) : p.max_seqlen_c;
  const int bq = p.positions[b] / p.block_size;
  // stage the row (only whole 16-byte vectors below k_len rounded up: the row's padding up to
  // row_stride may be read, nothing past it)
  const T* xs = x;
  if (p.staged_elems > 0) {
    const int n_vec = min((k_len + 7) / 8, p.staged_elems / 8);
    uint4* dst = reinterpret_cast<uint4*>(dyn_smem);
    // asynchronous copies: all of a thread's vectors are in flight at once
    for (int v = tid; v < n_vec; v += kThreads) mmasync::cp_async16(dst + v, reinterpret_cast<const uint4*>(x) + v);
    mmasync::cp_async_commit();
    mmasync::cp_async_wait<0>();
    __syncthreads();
    xs = reinterpret_cast<const T*>(dyn_smem);
  }
  select_row<T>(xs, p.staged_elems > 0, k_len, bq, p.a, sm,
                p.mask + ((int64_t)b * p.heads + h) * p.a.words,
                p.topk_idx ? p.topk_idx + ((int64_t)b * p.heads + h) * p.a.k : nullptr,
                p.positions[b] < p.a.dense_len);
}

}  // namespace
}  // namespace ifv2

using namespace ifv2;
extern "C" int ifv2_decode_select(const void* score, int is_bf16, int64_t row_stride,
                                  const int32_t* seqused_c, const int32_t* positions, int64_t* mask,
                                  int32_t* topk_idx, int batch, int heads, int max_seqlen_c,
                                  int n_blocks, int mask_words, int k, int local_blocks,
                                  int init_blocks, int block_size, int stride, int dense_len,
                                  void* stream) {
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
                 row_stride, batch, heads, max_seqlen_c, block_size, stage ? padded : 0,
                 Args{n_blocks, mask_words, k, local_blocks, init_blocks, block_size / stride,
                      dense_len > 0 ? dense_len : 0}};
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
