// Selection core shared by the decode selection kernels: from one row of stage-1 scores (one
// query token against the compressed keys of its sequence) to the packed block mask.
//
// Thread t of the CTA owns the contiguous blocks [t*per, (t+1)*per): it pools them (window
// pool_stride + 1, stride pool_stride, padding 1 over the compressed-key scores, +inf on the init
// and local blocks, -inf where no key exists) into 16-bit ordered keys in shared memory; the CTA
// bisects the key space for the k-th largest value (one barrier per probe); a block-wide scan
// over (above-threshold, tie) counts then gives every selected block its output slot, ties going
// to the lowest index -- the rule of the warp-per-row top-k kernel, so the result equals
// max-pool -> top-k -> mask pack run one after the other.
#pragma once
#include "common.cuh"

namespace ifv2 {
namespace dsel {

constexpr int kThreads = 256;
constexpr int kWarps = kThreads / 32;
constexpr int kMaxBlocks = 8192;

struct Smem {
  uint16_t keys[kMaxBlocks];
  unsigned long long words[kMaxBlocks / 64];
  int partial[2][kWarps];
  int scan_gt[kWarps], scan_tie[kWarps];
};

struct Args {
  int n_blocks, words, k, local_blocks, init_blocks, pool_stride;
  int dense_len;     // a query at a position below this attends every block it can see (0 = never)
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

__device__ __forceinline__ uint32_t ordered_key(uint16_t bits) {
  if (bits == 0x8000u) bits = 0;                                // -0 compares equal to +0
  return (bits & 0x8000u) ? (~(uint32_t)bits & 0xFFFFu) : ((uint32_t)bits | 0x8000u);
}

// xs: the row's scores (k_len of them are real), in shared memory when `in_smem`, else in global
// memory.  bq: the query token's own block.  mrow: (words) output mask words; out_idx: (k) or
// null.  Called by all kThreads threads of the CTA; sm.words need not be initialised.
template <typename T>
__device__ __forceinline__ void select_row(const T* xs, bool in_smem, int k_len, int bq, const Args& a,
                                           Smem& sm, unsigned long long* mrow, int32_t* out_idx,
                                           bool dense = false) {
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  if (dense) {
    // a short sequence: every block up to the query's own (the list, where asked for, can only
    // name the first k of them)
    for (int w = tid; w < a.words; w += kThreads) {
      const int first = w * 64;
      mrow[w] = (bq < first) ? 0ull : ((bq - first >= 63) ? ~0ull : ((2ull << (bq - first)) - 1ull));
    }
    if (out_idx != nullptr)
      for (int i = tid; i < a.k; i += kThreads) out_idx[i] = (i <= bq && i < a.n_blocks) ? i : -1;
    return;
  }
  const int n = a.n_blocks;
  const int per = (n + kThreads - 1) / kThreads;
  const int i0 = min(tid * per, n), i1 = min(i0 + per, n);
  constexpr uint16_t kPosInf = Inf<T>::kPos, kNegInf = Inf<T>::kPos | 0x8000;

  for (int w = tid; w < a.words; w += kThreads) sm.words[w] = 0ull;
  // ---- pool: block i <- max x[s*i - 1 .. s*i + s - 1] (kernel s + 1, stride s, padding 1)
  for (int i = i0; i < i1; ++i) {
    uint16_t bits;
    if (i < a.init_blocks || (bq >= i && bq <= i + a.local_blocks)) {
      bits = kPosInf;
    } else {
      const int s = max(i * a.pool_stride - 1, 0), e = min(i * a.pool_stride + a.pool_stride, k_len);
      float m = -INFINITY;
      if (in_smem) {
        for (int j = s; j < e; ++j) m = fmaxf(m, to_float(xs[j]));
      } else {
        for (int j = s; j < e; ++j) m = fmaxf(m, to_float(ldg16(xs + j)));
      }
      bits = rounded_bits(m, T());                     // exact: m is one of the inputs or -inf
    }
    sm.keys[i] = (uint16_t)ordered_key(bits);
  }
  __syncthreads();

  // ---- bisection for the k_eff-th largest key
  const int k_eff = min(a.k, n);
  uint32_t lo = ordered_key(kNegInf), hi = ordered_key(kPosInf) + 1u;
  int it = 0;
  while (hi - lo > 1u) {
    const uint32_t mid = (lo + hi) >> 1;
    int c = 0;
    for (int i = i0; i < i1; ++i) c += sm.keys[i] >= mid;
    c = __reduce_add_sync(0xFFFFFFFFu, c);
    if (lane == 0) sm.partial[it & 1][warp] = c;
    __syncthreads();                                   // (the other buffer is free again by now)
    int cnt = 0;
#pragma unroll
    for (int w = 0; w < kWarps; ++w) cnt += sm.partial[it & 1][w];
    if (cnt >= k_eff) lo = mid; else hi = mid;
    ++it;
  }
  // ---- slots: everything above the threshold, then ties lowest index first
  int gt = 0, tie = 0;
  for (int i = i0; i < i1; ++i) {
    gt += sm.keys[i] > lo;
    tie += sm.keys[i] == lo;
  }
  int gt_scan = gt, tie_scan = tie;
#pragma unroll
  for (int d = 1; d < 32; d <<= 1) {
    const int g2 = __shfl_up_sync(0xFFFFFFFFu, gt_scan, d), t2 = __shfl_up_sync(0xFFFFFFFFu, tie_scan, d);
    if (lane >= d) { gt_scan += g2; tie_scan += t2; }
  }
  if (lane == 31) { sm.scan_gt[warp] = gt_scan; sm.scan_tie[warp] = tie_scan; }
  __syncthreads();
  int gt_before = gt_scan - gt, tie_before = tie_scan - tie, gt_total = 0;
#pragma unroll
  for (int w = 0; w < kWarps; ++w) {
    if (w < warp) { gt_before += sm.scan_gt[w]; tie_before += sm.scan_tie[w]; }
    gt_total += sm.scan_gt[w];
  }
  const int need = k_eff - gt_total;                   // ties to take (>= 1 unless k_eff == 0)
  for (int i = i0; i < i1; ++i) {
    const bool g = sm.keys[i] > lo, t = sm.keys[i] == lo;
    if (g || (t && tie_before < need)) {
      const int pos = gt_before + min(tie_before, need);
      const bool keep = i <= bq;                       // later blocks only ever come out as -1
      if (out_idx != nullptr && pos < a.k) out_idx[pos] = keep ? i : -1;
      if (keep && (i >> 6) < a.words) atomicOr(&sm.words[i >> 6], 1ull << (i & 63));
    }
    gt_before += g;
    tie_before += t;
  }
  if (out_idx != nullptr)
    for (int i = k_eff + tid; i < a.k; i += kThreads) out_idx[i] = -1;
  __syncthreads();
  for (int w = tid; w < a.words; w += kThreads) mrow[w] = sm.words[w];
}

}  // namespace dsel
}  // namespace ifv2
