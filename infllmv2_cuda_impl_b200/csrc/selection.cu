// Selection kernels: 1-D max-pool of stage-1 scores to 64-token block scores, and per-query
// top-k of block scores.  Both are HBM-bound: one warp per row, 16-byte loads, warp shuffles.
#include "common.cuh"

namespace ifv2 {
namespace {

constexpr int kThreads = 256;
constexpr int kWarps = kThreads / 32;

template <typename T> struct Num;
template <> struct Num<__nv_bfloat16> {
  using T2 = __nv_bfloat162;
  static __device__ __forceinline__ float to_f(__nv_bfloat16 v) { return __bfloat162float(v); }
  static __device__ __forceinline__ __nv_bfloat16 from_f(float f) { return __float2bfloat16_rn(f); }
  static __device__ __forceinline__ __nv_bfloat16 from_bits(uint16_t b) {
    return __ushort_as_bfloat16(b);
  }
  static constexpr uint16_t kPosInf = 0x7F80, kNegInf = 0xFF80;
};
template <> struct Num<__half> {
  using T2 = __half2;
  static __device__ __forceinline__ float to_f(__half v) { return __half2float(v); }
  static __device__ __forceinline__ __half from_f(float f) { return __float2half_rn(f); }
  static __device__ __forceinline__ __half from_bits(uint16_t b) { return __ushort_as_half(b); }
  static constexpr uint16_t kPosInf = 0x7C00, kNegInf = 0xFC00;
};

struct PoolParams {
  const void* in;
  void* out;
  const int32_t* cu_q;
  const int32_t* cu_k;
  const int32_t* cache_lens;
  int batch, heads;
  int64_t total_q;        // rows per head
  int k_len;              // fixed-length: keys per row; varlen: row width (max_seqlen_k)
  int64_t in_row_stride;
  int out_len, cache_len, kernel, stride, padding, block_size, local_blocks, init_blocks;
};

template <bool kVarlen>
__device__ __forceinline__ void row_geometry(const PoolParams& p, int64_t q, int& k_len, int& bq) {
  if constexpr (kVarlen) {
    const int b = find_sequence(p.cu_q, p.batch, (int)q);
    k_len = min(p.cu_k[b + 1] - p.cu_k[b], p.k_len);
    bq = (int)((q - p.cu_q[b] + p.cache_lens[b]) / p.block_size);
  } else {
    k_len = p.k_len;
    bq = (int)((q + p.cache_len) / p.block_size);
  }
}

// Fast path: kernel 5 / stride 4 / padding 1 (block 64 over compression stride 16) and 16-byte
// aligned rows.  A lane loads 8 consecutive scores and produces the two block scores whose
// windows they cover: block 2m <- x[8m-1 .. 8m+3], block 2m+1 <- x[8m+3 .. 8m+7].
template <typename T, bool kVarlen>
__global__ void __launch_bounds__(kThreads) max_pool_k5s4_kernel(const PoolParams p) {
  using N = Num<T>;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int64_t rows = (int64_t)p.heads * p.total_q;
  const T* in = static_cast<const T*>(p.in);
  T* out = static_cast<T*>(p.out);
  const float ninf = -INFINITY;
  for (int64_t row = (int64_t)blockIdx.x * kWarps + warp; row < rows;
       row += (int64_t)gridDim.x * kWarps) {
    const int64_t q = row % p.total_q;
    int k_len, bq;
    row_geometry<kVarlen>(p, q, k_len, bq);
    const T* x = in + row * p.in_row_stride;
    T* y = out + row * p.out_len;
    for (int m0 = 0; 2 * m0 < p.out_len; m0 += 32) {     // warp-uniform trip count (shuffles inside)
      const int m = m0 + lane;
      const int e0 = 8 * m;
      float v[8];
      if (e0 < k_len) {
        const uint4 raw = __ldg(reinterpret_cast<const uint4*>(x + e0));
        const T* t = reinterpret_cast<const T*>(&raw);
#pragma unroll
        for (int j = 0; j < 8; ++j) v[j] = (e0 + j < k_len) ? N::to_f(t[j]) : ninf;
      } else {
#pragma unroll
        for (int j = 0; j < 8; ++j) v[j] = ninf;
      }
      // x[8m-1]: the neighbour lane's last element (lane 0 re-reads it; it is in L1)
      float prev = __shfl_up_sync(0xFFFFFFFFu, v[7], 1);
      if (lane == 0) prev = (e0 >= 1 && e0 - 1 < k_len) ? N::to_f(ldg16(x + e0 - 1)) : ninf;
      float r0 = fmaxf(fmaxf(prev, v[0]), fmaxf(fmaxf(v[1], v[2]), v[3]));
      float r1 = fmaxf(fmaxf(v[3], v[4]), fmaxf(fmaxf(v[5], v[6]), v[7]));
      const int b0 = 2 * m, b1 = b0 + 1;
      if (b0 >= p.out_len) continue;
      if (b0 < p.init_blocks || (bq >= b0 && bq <= b0 + p.local_blocks)) r0 = INFINITY;
      if (b1 < p.init_blocks || (bq >= b1 && bq <= b1 + p.local_blocks)) r1 = INFINITY;
      if ((p.out_len & 1) == 0) {
        typename N::T2 pr;
        pr.x = N::from_f(r0);
        pr.y = N::from_f(r1);
        *reinterpret_cast<typename N::T2*>(y + b0) = pr;
      } else {
        y[b0] = N::from_f(r0);
        if (b1 < p.out_len) y[b1] = N::from_f(r1);
      }
    }
  }
}

// Generic path: any kernel/stride/padding and any alignment; a lane per output block.
template <typename T, bool kVarlen>
__global__ void __launch_bounds__(kThreads) max_pool_generic_kernel(const PoolParams p) {
  using N = Num<T>;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int64_t rows = (int64_t)p.heads * p.total_q;
  const T* in = static_cast<const T*>(p.in);
  T* out = static_cast<T*>(p.out);
  for (int64_t row = (int64_t)blockIdx.x * kWarps + warp; row < rows;
       row += (int64_t)gridDim.x * kWarps) {
    const int64_t q = row % p.total_q;
    int k_len, bq;
    row_geometry<kVarlen>(p, q, k_len, bq);
    const T* x = in + row * p.in_row_stride;
    T* y = out + row * p.out_len;
    for (int b = lane; b < p.out_len; b += 32) {
      float r;
      if (b < p.init_blocks || (bq >= b && bq <= b + p.local_blocks)) {
        r = INFINITY;
      } else {
        const int s = max(b * p.stride - p.padding, 0);
        const int e = min(b * p.stride - p.padding + p.kernel, k_len);
        r = -INFINITY;
        for (int i = s; i < e; ++i) r = fmaxf(r, N::to_f(ldg16(x + i)));
      }
      y[b] = N::from_f(r);
    }
  }
}

template <typename T, bool kVarlen>
int launch_pool(const PoolParams& p, cudaStream_t st) {
  const int64_t rows = (int64_t)p.heads * p.total_q;
  int64_t blocks = ceil_div64(rows, kWarps);
  const int64_t cap = (int64_t)kNumSMs * 8;
  if (blocks > cap) blocks = cap;
  const bool fast = p.kernel == 5 && p.stride == 4 && p.padding == 1 &&
                    (p.in_row_stride % 8 == 0) && (reinterpret_cast<uintptr_t>(p.in) % 16 == 0) &&
                    (reinterpret_cast<uintptr_t>(p.out) % 4 == 0);
  if (fast)
    max_pool_k5s4_kernel<T, kVarlen><<<(int)blocks, kThreads, 0, st>>>(p);
  else
    max_pool_generic_kernel<T, kVarlen><<<(int)blocks, kThreads, 0, st>>>(p);
  return check_launch("max_pooling_1d");
}

// ---------------------------------------------------------------------------------------------
// Top-k: the k entries first in (value descending, index ascending) order, emitted ascending.
//
// A warp owns a row.  The row sits in registers as packed 16-bit pairs (lane-contiguous groups
// of 8 elements, so element index order is (iteration, lane, slot)).  The k-th largest value is
// found by bisection over the 16-bit ordered key space; each probe counts `x >= candidate`
// with native packed compares.  Entries above the threshold are all taken, entries equal to it
// are taken lowest index first, and output slots come from one packed warp prefix scan.

struct TopkParams {
  const void* score;
  int32_t* out;                    // (heads, total_q, k) block lists, or null
  unsigned long long* mask;        // (heads, total_q, mask_words) packed selection, or null
  int mask_words;
  const int32_t* cu_q;
  const int32_t* cache_lens;
  int batch, heads;
  int64_t total_q;
  int n_blocks;
  int64_t row_stride;
  int k, cache_len, block_size;
};

// ordered key (0..65535, monotone in the float value) -> raw 16-bit pattern
__device__ __forceinline__ uint16_t ordered_to_bits(uint32_t o) {
  return (uint16_t)((o & 0x8000u) ? (o ^ 0x8000u) : (~o & 0xFFFFu));
}
__device__ __forceinline__ uint32_t bits_to_ordered(uint16_t b) {
  return (b & 0x8000u) ? (~(uint32_t)b & 0xFFFFu) : ((uint32_t)b | 0x8000u);
}

template <typename T> struct Pack;
template <> struct Pack<__nv_bfloat16> {
  using T2 = __nv_bfloat162;
  static __device__ __forceinline__ T2 splat(uint16_t bits) {
    return __halves2bfloat162(__ushort_as_bfloat16(bits), __ushort_as_bfloat16(bits));
  }
  static __device__ __forceinline__ T2 zero() { return __float2bfloat162_rn(0.f); }
  static __device__ __forceinline__ int hsum(T2 v) {
    return (int)(__bfloat162float(v.x) + __bfloat162float(v.y));
  }
  // 0xFFFF in the half of the word whose comparison holds
  static __device__ __forceinline__ uint32_t ge_mask(T2 a, T2 b) { return __hge2_mask(a, b); }
  static __device__ __forceinline__ uint32_t gt_mask(T2 a, T2 b) { return __hgt2_mask(a, b); }
  static __device__ __forceinline__ uint32_t eq_mask(T2 a, T2 b) { return __heq2_mask(a, b); }
};
template <> struct Pack<__half> {
  using T2 = __half2;
  static __device__ __forceinline__ T2 splat(uint16_t bits) {
    return __halves2half2(__ushort_as_half(bits), __ushort_as_half(bits));
  }
  static __device__ __forceinline__ T2 zero() { return __float2half2_rn(0.f); }
  static __device__ __forceinline__ int hsum(T2 v) {
    return (int)(__half2float(v.x) + __half2float(v.y));
  }
  static __device__ __forceinline__ uint32_t ge_mask(T2 a, T2 b) { return __hge2_mask(a, b); }
  static __device__ __forceinline__ uint32_t gt_mask(T2 a, T2 b) { return __hgt2_mask(a, b); }
  static __device__ __forceinline__ uint32_t eq_mask(T2 a, T2 b) { return __heq2_mask(a, b); }
};

// Output stores are guarded by the capacity of the row: a slot outside [0, k) is never written
// (-DIFV2_TOPK_CHECK additionally reports such a slot).
#ifdef IFV2_TOPK_CHECK
#define IFV2_TOPK_STORE(pos, val)                                                               \
  do {                                                                                          \
    if (o != nullptr && (unsigned)(pos) < (unsigned)k_cap) o[(pos)] = (val);                    \
    else if (o != nullptr) printf("topk: slot %d outside [0,%d) lane %d k_sel %d need %d exact %d bq %d\n", (int)(pos), k_cap, \
                lane, k_sel, need, (int)exact, bq);                                             \
  } while (0)
#else
#define IFV2_TOPK_STORE(pos, val)                                  \
  do {                                                             \
    if (o != nullptr && (unsigned)(pos) < (unsigned)k_cap) o[(pos)] = (val);   \
  } while (0)
#endif

// Selection over the first kIts iterations (256 entries each) of a row held in registers; the
// iteration count is a template parameter so that the probe and emit loops are straight-line
// code.  Returns the number of entries emitted, or -1 when a restricted selection turns out not
// to be equivalent to the full one.
template <typename T, int kPairs, int kIts>
__device__ __forceinline__ int topk_row(const typename Pack<T>::T2 (&v)[kPairs],
                                        typename Pack<T>::T2 tail2, bool restricted, int k_sel,
                                        int bq, int lane, int32_t* o, int k_cap,
                                        unsigned long long* mw, int mask_words) {
  using N = Num<T>;
  using P = Pack<T>;
  using T2 = typename P::T2;
  // ---- bisection for the k_sel-th largest value over ordered keys [-inf, +inf]
  uint32_t lo = bits_to_ordered(N::kNegInf), hi = bits_to_ordered(N::kPosInf) + 1u;
  bool exact = false;                     // count(x >= val(lo)) == k_sel: no tie handling needed
  while (hi - lo > 1u) {
    const uint32_t mid = (lo + hi) >> 1;
    const T2 c = P::splat(ordered_to_bits(mid));
    T2 acc = P::zero();
#pragma unroll
    for (int it = 0; it < kIts; ++it) {
      if (it < kIts) {
#pragma unroll
        for (int j = 0; j < 4; ++j) acc = __hadd2(acc, __hge2(v[it * 4 + j], c));
      }
    }
    const int cnt = __reduce_add_sync(0xFFFFFFFFu, P::hsum(acc));
    if (cnt >= k_sel) {
      lo = mid;
      if (cnt == k_sel) { exact = true; break; }
    } else {
      hi = mid;
    }
  }
  const T2 thr = P::splat(ordered_to_bits(lo));
  if (restricted) {
    // a later entry above the threshold would have displaced one of the selected ones
    const float tm = fmaxf(N::to_f(tail2.x), N::to_f(tail2.y));
    const bool bad = tm > N::to_f(thr.x);
    if (__any_sync(0xFFFFFFFFu, bad)) return -1;        // redo over the full width
  }
  int need = 0;                           // how many entries equal to the threshold to take
  if (!exact) {
    T2 acc = P::zero();
#pragma unroll
    for (int it = 0; it < kIts; ++it) {
      if (it < kIts) {
#pragma unroll
        for (int j = 0; j < 4; ++j) acc = __hadd2(acc, __hgt2(v[it * 4 + j], thr));
      }
    }
    need = k_sel - __reduce_add_sync(0xFFFFFFFFu, P::hsum(acc));
  }

  // ---- emit in index order
  int base_gt = 0, base_tie = 0;          // counts over all earlier iterations
#pragma unroll
  for (int it = 0; it < kIts; ++it) {
    if (it < kIts) {
      uint32_t gt_bits = 0, tie_bits = 0;   // bit s: slot s of this lane's 8 elements
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const T2 pr = v[it * 4 + j];
        const uint32_t mg = exact ? P::ge_mask(pr, thr) : P::gt_mask(pr, thr);
        gt_bits |= ((mg & 1u) | ((mg >> 15) & 2u)) << (2 * j);
        if (!exact) {
          const uint32_t me = P::eq_mask(pr, thr);
          tie_bits |= ((me & 1u) | ((me >> 15) & 2u)) << (2 * j);
        }
      }
      // packed inclusive scan over lanes: low 16 bits = taken-for-sure, high 16 = ties
      const uint32_t mine = (uint32_t)__popc(gt_bits) | ((uint32_t)__popc(tie_bits) << 16);
      uint32_t scan = mine;
#pragma unroll
      for (int d = 1; d < 32; d <<= 1) {
        const uint32_t up = __shfl_up_sync(0xFFFFFFFFu, scan, d);
        if (lane >= d) scan += up;
      }
      const uint32_t total = __shfl_sync(0xFFFFFFFFu, scan, 31);
      const uint32_t excl = scan - mine;
      int gt_before = base_gt + (int)(excl & 0xFFFFu);
      int tie_before = base_tie + (int)(excl >> 16);
      const int e0 = (it * 32 + lane) * 8;
      // slots of this lane that the query may see (index <= bq): only those reach the mask
      const uint32_t vis_bits = (bq >= e0 + 7) ? 0xFFu : ((bq < e0) ? 0u : ((2u << (bq - e0)) - 1u));
      uint32_t taken = gt_bits;           // slots selected in this iteration
      if (tie_bits == 0u) {               // the common case: walk the few set bits
        int pos = gt_before + min(tie_before, need);
        uint32_t sel = gt_bits;
        while (sel) {
          const int s = __ffs(sel) - 1;
          sel &= sel - 1u;
          const int idx = e0 + s;
          IFV2_TOPK_STORE(pos, (idx <= bq) ? idx : -1);
          ++pos;
        }
      } else {
#pragma unroll
        for (int s = 0; s < 8; ++s) {
          const bool g = (gt_bits >> s) & 1u, t = (tie_bits >> s) & 1u;
          if (g || (t && tie_before < need)) {
            const int pos = gt_before + min(tie_before, need);
            const int idx = e0 + s;
            IFV2_TOPK_STORE(pos, (idx <= bq) ? idx : -1);
            taken |= 1u << s;
          }
          gt_before += g;
          tie_before += t;
        }
      }
      if (mw != nullptr) {
        // eight lanes own the 64 consecutive entries of one mask word: OR their bytes together
        unsigned long long wv = (unsigned long long)(taken & vis_bits) << (8 * (lane & 7));
        wv |= __shfl_xor_sync(0xFFFFFFFFu, wv, 1);
        wv |= __shfl_xor_sync(0xFFFFFFFFu, wv, 2);
        wv |= __shfl_xor_sync(0xFFFFFFFFu, wv, 4);
        const int w = it * 4 + (lane >> 3);
        if ((lane & 7) == 0 && w < mask_words) mw[w] = wv;
      }
      base_gt += (int)(total & 0xFFFFu);
      base_tie += (int)(total >> 16);
    }
  }
  return base_gt + min(base_tie, need);
}

template <typename T, int kIters>
__global__ void __launch_bounds__(kThreads, (kIters <= 8) ? 2 : 1) topk_select_kernel(const TopkParams p) {
  using N = Num<T>;
  using P = Pack<T>;
  using T2 = typename P::T2;
  constexpr int kPairs = kIters * 4;          // packed registers per lane
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int64_t rows = (int64_t)p.heads * p.total_q;
  const T* score = static_cast<const T*>(p.score);
  const int n = p.n_blocks;
  const int k_eff = min(p.k, n);
  const bool aligned = (p.row_stride % 8 == 0) && (reinterpret_cast<uintptr_t>(p.score) % 16 == 0);
  const T2 pad2 = P::splat(N::kNegInf);
  const T ninf = N::from_bits(N::kNegInf);

  for (int64_t row = (int64_t)blockIdx.x * kWarps + warp; row < rows;
       row += (int64_t)gridDim.x * kWarps) {
    const int64_t q = row % p.total_q;
    int bq;
    if (p.cu_q != nullptr) {
      const int b = find_sequence(p.cu_q, p.batch, (int)q);
      const int cl = p.cache_lens ? p.cache_lens[b] : p.cache_len;
      bq = (int)((q - p.cu_q[b] + cl) / p.block_size);
    } else {
      bq = (int)((q + p.cache_len) / p.block_size);
    }
    const T* x = score + row * p.row_stride;
    int32_t* o = p.out ? p.out + row * p.k : nullptr;
    unsigned long long* mw = p.mask ? p.mask + row * p.mask_words : nullptr;

    // Entries past the query's own block only ever come out as -1.  When none of them beats the
    // k-th best earlier entry (always the case for stage-1 block scores: later blocks hold 0 or
    // -inf and ties go to the lower index) the selection can run over the earlier entries alone;
    // that is checked after the fact, and a row that fails it is redone over the full width.
    const int head = min(n, bq + 1);
    int emitted = 0;
    for (int attempt = 0; attempt < 2; ++attempt) {
      const bool restricted = (attempt == 0) && head < n;
      const int width = restricted ? head : n;              // entries that take part
      const int its = (width + 255) >> 8;                   // 256 entries per iteration
      const int k_sel = min(k_eff, width);

      // ---- load: element index of (it, lane, slot) is (it*32 + lane)*8 + slot
      T2 v[kPairs];
#pragma unroll
      for (int it = 0; it < kIters; ++it) {
        const int e0 = (it * 32 + lane) * 8;
        if (aligned && e0 + 8 <= n) {
          const uint4 raw = __ldg(reinterpret_cast<const uint4*>(x + e0));
          const T2* t = reinterpret_cast<const T2*>(&raw);
#pragma unroll
          for (int j = 0; j < 4; ++j) v[it * 4 + j] = t[j];
        } else {
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            T2 pr = pad2;
            if (e0 + 2 * j < n) pr.x = ldg16(x + e0 + 2 * j);
            if (e0 + 2 * j + 1 < n) pr.y = ldg16(x + e0 + 2 * j + 1);
            v[it * 4 + j] = pr;
          }
        }
      }
      // ---- split off the entries past `width`: their maximum is kept, their slots become -inf
      T2 tail2 = pad2;
      if (restricted) {
#pragma unroll
        for (int it = 0; it < kIters; ++it) {
          const int nh = width - (it * 32 + lane) * 8;      // entries of this lane that take part
          if (nh < 8) {
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              T2 pr = v[it * 4 + j], tl = pad2;
              if (2 * j >= nh) { tl.x = pr.x; pr.x = ninf; }
              if (2 * j + 1 >= nh) { tl.y = pr.y; pr.y = ninf; }
              tail2 = __hmax2(tail2, tl);
              v[it * 4 + j] = pr;
            }
          }
        }
      }

      // ---- bisection + emission over the `its` iterations that take part
      // (an even iteration count keeps the number of instantiated bodies, and with it the
      //  instruction-cache footprint, small; the extra iteration only holds -inf slots)
      int got = -1;
      const int its_used = min(kIters, (its + 1) & ~1);
      switch (its_used) {
#define IFV2_TOPK_CASE(I)                                                                \
        case I:                                                                          \
          if constexpr (I <= kIters)                                                     \
            got = topk_row<T, kPairs, I>(v, tail2, restricted, k_sel, bq, lane, o, p.k,  \
                                         mw, p.mask_words);                              \
          break;
        IFV2_TOPK_CASE(2) IFV2_TOPK_CASE(4) IFV2_TOPK_CASE(6)
#undef IFV2_TOPK_CASE
        default:
          got = topk_row<T, kPairs, kIters>(v, tail2, restricted, k_sel, bq, lane, o, p.k, mw,
                                            p.mask_words);
          break;
      }
      if (got < 0) continue;
      emitted = got;
      // mask words past the iterations that took part hold no selected block
      if (mw != nullptr) {
        const int covered = (its_used == 2 || its_used == 4 || its_used == 6 ? its_used : kIters) * 4;
        for (int w = covered + lane; w < p.mask_words; w += 32) mw[w] = 0ull;
      }
      break;
    }
    // unused tail (k > entries that took part, or NaN scores that no probe counts)
    if (o != nullptr)
      for (int i = emitted + lane; i < p.k; i += 32) o[i] = -1;
  }
}

template <typename T>
int launch_topk(const TopkParams& p, cudaStream_t st) {
  const int64_t rows = (int64_t)p.heads * p.total_q;
  int64_t blocks = ceil_div64(rows, kWarps);
  const int64_t cap = (int64_t)kNumSMs * 8;
  if (blocks > cap) blocks = cap;
  if (p.n_blocks <= 256)
    topk_select_kernel<T, 1><<<(int)blocks, kThreads, 0, st>>>(p);
  else if (p.n_blocks <= 512)
    topk_select_kernel<T, 2><<<(int)blocks, kThreads, 0, st>>>(p);
  else if (p.n_blocks <= 1024)
    topk_select_kernel<T, 4><<<(int)blocks, kThreads, 0, st>>>(p);
  else if (p.n_blocks <= 2048)
    topk_select_kernel<T, 8><<<(int)blocks, kThreads, 0, st>>>(p);
  else if (p.n_blocks <= 4096)
    topk_select_kernel<T, 16><<<(int)blocks, kThreads, 0, st>>>(p);
  else
    topk_select_kernel<T, 32><<<(int)blocks, kThreads, 0, st>>>(p);
  return check_launch("topk_select");
}

}  // namespace
}  // namespace ifv2

using namespace ifv2;

static int check_pool_args(const void* in, const void* out, int heads, int64_t total_q, int k_len,
                           int64_t in_row_stride, int out_len, int kernel, int stride, int padding,
                           int block_size, int local_blocks, int init_blocks) {
  IFV2_REQUIRE(heads >= 0 && total_q >= 0 && k_len >= 0 && out_len >= 0, IFV2_ERR_INVALID_ARG,
               "max_pooling_1d: negative size");
  IFV2_REQUIRE(kernel >= 1 && stride >= 1 && padding >= 0 && block_size >= 1, IFV2_ERR_INVALID_ARG,
               "max_pooling_1d: kernel/stride/block_size must be >= 1 and padding >= 0");
  IFV2_REQUIRE(local_blocks >= 0 && init_blocks >= 0, IFV2_ERR_INVALID_ARG,
               "max_pooling_1d: local_blocks / init_blocks must be >= 0");
  IFV2_REQUIRE(in_row_stride >= k_len, IFV2_ERR_INVALID_ARG,
               "max_pooling_1d: in_row_stride (%lld) < k_len (%d)", (long long)in_row_stride, k_len);
  if (heads == 0 || total_q == 0 || out_len == 0) return 1;   // nothing to do
  IFV2_REQUIRE(in != nullptr || k_len == 0, IFV2_ERR_INVALID_ARG, "max_pooling_1d: null input");
  IFV2_REQUIRE(out != nullptr, IFV2_ERR_INVALID_ARG, "max_pooling_1d: null output");
  return 0;
}

extern "C" int ifv2_max_pooling_1d(const void* in, void* out, int is_bf16, int heads, int q_len,
                                   int k_len, int64_t in_row_stride, int out_len, int cache_len,
                                   int kernel_size, int stride, int padding, int block_size,
                                   int local_blocks, int init_blocks, void* stream) {
  int rc = check_pool_args(in, out, heads, q_len, k_len, in_row_stride, out_len, kernel_size, stride,
                           padding, block_size, local_blocks, init_blocks);
  if (rc != 0) return rc > 0 ? IFV2_OK : rc;
  IFV2_REQUIRE(cache_len >= 0, IFV2_ERR_INVALID_ARG, "max_pooling_1d: cache_len < 0");
  PoolParams p{in, out, nullptr, nullptr, nullptr, 1, heads, q_len, k_len, in_row_stride, out_len,
               cache_len, kernel_size, stride, padding, block_size, local_blocks, init_blocks};
  return is_bf16 ? launch_pool<__nv_bfloat16, false>(p, (cudaStream_t)stream)
                 : launch_pool<__half, false>(p, (cudaStream_t)stream);
}

extern "C" int ifv2_max_pooling_1d_varlen(const void* in, void* out, const int32_t* cu_seqlens_q,
                                          const int32_t* cu_seqlens_k, const int32_t* cache_lens,
                                          int is_bf16, int batch, int heads, int64_t total_q,
                                          int max_seqlen_k, int64_t in_row_stride, int out_len,
                                          int kernel_size, int stride, int padding, int block_size,
                                          int local_blocks, int init_blocks, void* stream) {
  int rc = check_pool_args(in, out, heads, total_q, max_seqlen_k, in_row_stride, out_len, kernel_size,
                           stride, padding, block_size, local_blocks, init_blocks);
  if (rc != 0) return rc > 0 ? IFV2_OK : rc;
  IFV2_REQUIRE(batch >= 1 && cu_seqlens_q && cu_seqlens_k && cache_lens, IFV2_ERR_INVALID_ARG,
               "max_pooling_1d_varlen: batch >= 1 and cu_seqlens_q/cu_seqlens_k/cache_lens required");
  IFV2_REQUIRE(total_q <= INT32_MAX, IFV2_ERR_TOO_LARGE, "max_pooling_1d_varlen: total_q > 2^31-1");
  PoolParams p{in, out, cu_seqlens_q, cu_seqlens_k, cache_lens, batch, heads, total_q, max_seqlen_k,
               in_row_stride, out_len, 0, kernel_size, stride, padding, block_size, local_blocks,
               init_blocks};
  return is_bf16 ? launch_pool<__nv_bfloat16, true>(p, (cudaStream_t)stream)
                 : launch_pool<__half, true>(p, (cudaStream_t)stream);
}

extern "C" int ifv2_topk_select(const void* score, int32_t* out_idx, int is_bf16, int heads,
                                int64_t total_q, int n_blocks, int64_t row_stride, int k,
                                const int32_t* cu_seqlens_q, const int32_t* cache_lens, int batch,
                                int cache_len, int block_size, void* stream) {
  IFV2_REQUIRE(heads >= 0 && total_q >= 0 && n_blocks >= 0 && k >= 0, IFV2_ERR_INVALID_ARG,
               "topk_select: negative size");
  IFV2_REQUIRE(block_size >= 1 && cache_len >= 0, IFV2_ERR_INVALID_ARG,
               "topk_select: block_size must be >= 1 and cache_len >= 0");
  IFV2_REQUIRE(row_stride >= n_blocks, IFV2_ERR_INVALID_ARG, "topk_select: row_stride < n_blocks");
  IFV2_REQUIRE(n_blocks <= 8192, IFV2_ERR_TOO_LARGE,
               "topk_select: n_blocks = %d exceeds the 8192-block limit", n_blocks);
  IFV2_REQUIRE(cache_lens == nullptr || cu_seqlens_q != nullptr, IFV2_ERR_INVALID_ARG,
               "topk_select: cache_lens needs cu_seqlens_q");
  IFV2_REQUIRE(cu_seqlens_q == nullptr || batch >= 1, IFV2_ERR_INVALID_ARG,
               "topk_select: batch must be >= 1 with cu_seqlens_q");
  if (heads == 0 || total_q == 0 || k == 0) return IFV2_OK;
  IFV2_REQUIRE(out_idx != nullptr && (score != nullptr || n_blocks == 0), IFV2_ERR_INVALID_ARG,
               "topk_select: null pointer");
  IFV2_REQUIRE(total_q <= INT32_MAX, IFV2_ERR_TOO_LARGE, "topk_select: total_q > 2^31-1");
  TopkParams p{score, out_idx, nullptr, 0, cu_seqlens_q, cache_lens, batch, heads, total_q, n_blocks,
               row_stride, k, cache_len, block_size};
  return is_bf16 ? launch_topk<__nv_bfloat16>(p, (cudaStream_t)stream)
                 : launch_topk<__half>(p, (cudaStream_t)stream);
}

extern "C" int ifv2_topk_select_mask(const void* score, int32_t* out_idx, int64_t* row_mask,
                                     int64_t* col_mask, int is_bf16, int heads, int64_t total_q,
                                     int n_blocks, int64_t row_stride, int k, int k_blocks,
                                     const int32_t* cu_seqlens_q, const int32_t* cache_lens, int batch,
                                     int cache_len, int block_size, void* stream) {
  IFV2_REQUIRE(heads >= 0 && total_q >= 0 && n_blocks >= 0 && k >= 0 && k_blocks >= 0,
               IFV2_ERR_INVALID_ARG, "topk_select_mask: negative size");
  IFV2_REQUIRE(block_size >= 1 && cache_len >= 0, IFV2_ERR_INVALID_ARG,
               "topk_select_mask: block_size must be >= 1 and cache_len >= 0");
  IFV2_REQUIRE(row_stride >= n_blocks, IFV2_ERR_INVALID_ARG, "topk_select_mask: row_stride < n_blocks");
  IFV2_REQUIRE(n_blocks <= 8192 && k_blocks <= 8192, IFV2_ERR_TOO_LARGE,
               "topk_select_mask: n_blocks = %d / k_blocks = %d exceed the 8192-block limit", n_blocks,
               k_blocks);
  IFV2_REQUIRE(cache_lens == nullptr || cu_seqlens_q != nullptr, IFV2_ERR_INVALID_ARG,
               "topk_select_mask: cache_lens needs cu_seqlens_q");
  IFV2_REQUIRE(cu_seqlens_q == nullptr || batch >= 1, IFV2_ERR_INVALID_ARG,
               "topk_select_mask: batch must be >= 1 with cu_seqlens_q");
  if (heads == 0 || total_q == 0 || k_blocks == 0) return IFV2_OK;
  IFV2_REQUIRE(row_mask != nullptr && (score != nullptr || n_blocks == 0), IFV2_ERR_INVALID_ARG,
               "topk_select_mask: null pointer");
  IFV2_REQUIRE(total_q <= INT32_MAX, IFV2_ERR_TOO_LARGE, "topk_select_mask: total_q > 2^31-1");
  const int words = (k_blocks + 63) / 64;
  TopkParams p{score, out_idx, reinterpret_cast<unsigned long long*>(row_mask), words, cu_seqlens_q,
               cache_lens, batch, heads, total_q, n_blocks, row_stride, k, cache_len, block_size};
  int rc = is_bf16 ? launch_topk<__nv_bfloat16>(p, (cudaStream_t)stream)
                   : launch_topk<__half>(p, (cudaStream_t)stream);
  if (rc != IFV2_OK || col_mask == nullptr) return rc;
  return ifv2_transpose_blockmask(row_mask, col_mask, heads, total_q, k_blocks, stream);
}
