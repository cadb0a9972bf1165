// Sparse decode over a KV cache: one new query token per sequence, 16 query heads per KV head.
//
// With a single token the query tile is 16 rows, far too small for a tcgen05 tile, and the work
// is HBM-bound: every selected 64-key block is read once (K and V, 32 KB) and used by 16 rows.
// So this kernel is built around bandwidth: the selected blocks of one (sequence, KV head) are
// split over several CTAs (as many as fill the SMs in ONE wave, three CTAs per SM), each warp
// streams its blocks as 32-key units into swizzled shared memory (K and V of the next unit are
// fetched as soon as the current product has consumed its tile), the 16 x 32 products run on
// mma.sync m16n8k16 (exactly one M tile), and the per-split (max, sum, O) partials are merged by
// a small second kernel.
//
// Launches: [append new K/V in place] -> split kernel -> combine kernel.
//
// Tile loads: when the cache rows can be described by one tensor map (16-byte aligned base, batch
// stride a whole number of rows) a warp's K and V tiles arrive as two TMA boxes each ({64 d, 1 head,
// 32 keys}, 128-byte swizzle) on a per-warp mbarrier, issued by one lane, instead of 512 sixteen-byte
// cp.async requests per tile; other layouts use cp.async.  Both forms run at the same speed: what
// held the step at half the HBM bandwidth was a launch of 1.15 waves, see the split count below.
#include <string.h>
#include "mma_sync.cuh"
#include "tc05.cuh"

namespace ifv2 {
namespace {

using namespace mmasync;

constexpr int kMaxSplits = 16;                          // CTAs per (sequence, KV head), chosen per launch
constexpr int kWarps = 4;
constexpr int kWarpSmem = 2 * kUnit * 256;              // one K tile + one V tile per warp
constexpr int kThreads = kWarps * 32;
// resident CTAs per SM the split kernel is compiled for: 3 (168 registers, 12 warps) measured 4 %
// faster than 2 (212 registers) on the batch-64 decode step -- more copies in flight per SM
#ifndef IFV2_DECODE_CTAS_PER_SM
#define IFV2_DECODE_CTAS_PER_SM 3
#endif
constexpr int kPartialFloats = kHeadDim + 4;            // O row, running max (log2 units), sum, pad (16-byte rows)
constexpr float kLog2e = 1.4426950408889634f;
constexpr float kLn2 = 0.6931471805599453f;

struct DecodeParams {
  const __nv_bfloat16* q;         // (batch, heads_q, 128)
  const __nv_bfloat16* k_cache;   // (batch, capacity, heads_k, 128), batch stride given
  const __nv_bfloat16* v_cache;
  const unsigned long long* mask; // (batch, heads_k, mask_words) or null
  int mask_words;
  const int32_t* cache_seqlens;
  int new_tokens;                 // 1 when k_new / v_new were appended, else 0
  int64_t capacity;               // positions a sequence may use; lengths are clamped to it
  int heads_q, heads_k;
  int64_t batch_stride;           // elements between sequences in the caches
  const int32_t* block_table;     // (batch, bt_stride) page of every page_size positions, or null
  int bt_stride, page_size;
  const int32_t* cache_batch_idx; // (batch) row of the caches each sequence uses, or null
  const int32_t* leftpad;         // (batch) position of a sequence's first key, or null
  float scale_log2;
  int splits;                     // CTAs sharing one (sequence, KV head), 1 .. kMaxSplits
  float* partial;                 // (batch, heads_k, splits, 16, kPartialFloats)
  __nv_bfloat16* out;             // (batch, heads_q, 128)
  float* lse;                     // (batch, heads_q) or null
  int use_tma;                    // tiles come through the tensor maps given to the kernel
  int64_t rows_per_slot;          // cache rows between two sequence slots (TMA path, unpaged)
};

// Row of position `pos` of sequence b in the (rows, heads_k, 128) view of a cache.
__device__ __forceinline__ int cache_row(const DecodeParams& p, int b, int slot, int64_t pos) {
  if (p.block_table != nullptr) {
    const int page = __ldg(p.block_table + (int64_t)b * p.bt_stride + pos / p.page_size);
    return page * p.page_size + (int)(pos % p.page_size);
  }
  return (int)(slot * p.rows_per_slot + pos);
}

// Tile layout of the TMA path: two 4 KB halves (d 0..63, d 64..127) of 32 rows x 128 bytes, 16-byte
// chunk c of row r stored at chunk (c ^ (r & 7)) -- the 128-byte swizzle the copy engine applies.
__device__ __forceinline__ uint8_t* tile_addr_tma(uint8_t* tile, int row, int chunk) {
  return tile + (chunk >> 3) * 4096 + row * 128 + (((chunk & 7) ^ (row & 7)) << 4);
}

constexpr long long kDecodeWaitLimit = 1ll << 28;       // clocks; a copy takes microseconds

// Element offset of position `pos` of sequence b (head 0) in a cache: contiguous rows, rows of
// another sequence slot (cache_batch_idx), or pages of a block table.
__device__ __forceinline__ int64_t cache_row_offset(const int32_t* block_table, int bt_stride,
                                                    int page_size, int64_t batch_stride,
                                                    int64_t row_stride, int b, int slot, int64_t pos) {
  if (block_table != nullptr) {
    const int page = __ldg(block_table + (int64_t)b * bt_stride + pos / page_size);
    return ((int64_t)page * page_size + pos % page_size) * row_stride;
  }
  return slot * batch_stride + pos * row_stride;
}

__global__ void decode_append_kernel(__nv_bfloat16* k_cache, __nv_bfloat16* v_cache,
                                     const __nv_bfloat16* k_new, const __nv_bfloat16* v_new,
                                     const int32_t* cache_seqlens, int heads_k, int64_t capacity,
                                     int64_t batch_stride, const int32_t* block_table, int bt_stride,
                                     int page_size, const int32_t* cache_batch_idx) {
  const int b = blockIdx.x;
  const int64_t pos = cache_seqlens[b];
  if (pos < 0 || pos >= capacity) return;           // no room: the host documents this as an error
  const int n = heads_k * kHeadDim / 8;             // 16-byte vectors per token
  const int64_t row_stride = (int64_t)heads_k * kHeadDim;
  const int slot = cache_batch_idx ? cache_batch_idx[b] : b;
  const int64_t off = cache_row_offset(block_table, bt_stride, page_size, batch_stride, row_stride, b,
                                       slot, pos);
  const uint4* ks = reinterpret_cast<const uint4*>(k_new + (int64_t)b * heads_k * kHeadDim);
  const uint4* vs = reinterpret_cast<const uint4*>(v_new + (int64_t)b * heads_k * kHeadDim);
  uint4* kd = reinterpret_cast<uint4*>(k_cache + off);
  uint4* vd = reinterpret_cast<uint4*>(v_cache + off);
  for (int i = threadIdx.x; i < n; i += blockDim.x) {
    kd[i] = ks[i];
    vd[i] = vs[i];
  }
}

// index of the j-th (0-based) block of the selection, scanning the mask words upward
struct BlockList {
  const unsigned long long* words;   // null = every block below nblk
  int nwords, nblk;
  __device__ unsigned long long word(int w) const {
    unsigned long long x = __ldg(words + w);
    const int first = w * 64;
    if (nblk - first < 64) x &= (nblk > first) ? ((1ull << (nblk - first)) - 1ull) : 0ull;
    return x;
  }
  __device__ int count() const {
    if (words == nullptr) return nblk;
    int n = 0;
    for (int w = 0; w < nwords; ++w) n += __popcll(word(w));
    return n;
  }
  __device__ int nth(int j) const {
    if (words == nullptr) return j;
    for (int w = 0; w < nwords; ++w) {
      unsigned long long x = word(w);
      const int c = __popcll(x);
      if (j < c) {
        for (int i = 0; i < j; ++i) x &= x - 1;      // drop the j lowest set bits
        return w * 64 + __ffsll((long long)x) - 1;
      }
      j -= c;
    }
    return -1;
  }
};

template <bool kTma>
__global__ void __launch_bounds__(kThreads, IFV2_DECODE_CTAS_PER_SM)
decode_split_kernel(const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v,
                    const DecodeParams p) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  __shared__ uint64_t tile_bar[kWarps][2];              // per warp: K tile, V tile landed
  const int split = blockIdx.x, h = blockIdx.y, b = blockIdx.z;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t = lane & 3;
  uint8_t* k_tile = smem + warp * kWarpSmem;
  uint8_t* v_tile = k_tile + kUnit * 256;
  if (kTma) {
    if (lane == 0) {
      tc::mbar_init(&tile_bar[warp][0], 1);
      tc::mbar_init(&tile_bar[warp][1], 1);
      tc::fence_barrier_init();
    }
    __syncwarp();
  }
  uint32_t k_phase = 0, v_phase = 0;                    // parity of the next completion of each barrier
  bool expired = false;                                 // a bounded wait ran out: the partial is poisoned

  const int pad = p.leftpad ? p.leftpad[b] : 0;                 // keys are positions pad .. end-1
  // a length beyond the capacity is a caller error with a defined result: the keys are the
  // positions that exist, and the new token counts only if the append had room for it
  const int64_t end = min(max((int64_t)p.cache_seqlens[b], (int64_t)0) + p.new_tokens, p.capacity);
  const int len = (int)max(end - pad, (int64_t)0);
  const int slot = p.cache_batch_idx ? p.cache_batch_idx[b] : b;
  BlockList list{p.mask ? p.mask + ((int64_t)b * p.heads_k + h) * p.mask_words : nullptr, p.mask_words,
                 (len + kBlockN - 1) / kBlockN};
  const int n = list.count();
  const int per_split = (n + p.splits - 1) / p.splits;
  const int j_begin = split * per_split, j_end = min(n, j_begin + per_split);

  const int64_t row_stride = (int64_t)p.heads_k * kHeadDim;
  // first row of the 32-key unit that starts at key `k0` (a unit never straddles a page: pages
  // are multiples of 64 positions and a paged cache has no left padding)
  auto unit = [&](const __nv_bfloat16* cache, int k0) -> const __nv_bfloat16* {
    return cache + cache_row_offset(p.block_table, p.bt_stride, p.page_size, p.batch_stride, row_stride,
                                    b, slot, (int64_t)k0 + pad) + (int64_t)h * kHeadDim;
  };

  // one tile (32 keys x 128 d of this KV head, first key `k0`): TMA boxes on the warp's barrier, or
  // 16-byte cp.async copies
  auto fetch = [&](bool is_v, uint8_t* tile, int k0) {
    if (kTma) {
      __syncwarp();                              // every lane is done reading the tile being replaced
      if (lane == 0) {
        // the tile was read through ldmatrix / written by plain stores: order those before the copy
        tc::fence_proxy_async_smem();
        uint64_t* bar = &tile_bar[warp][is_v ? 1 : 0];
        const int row = cache_row(p, b, slot, (int64_t)k0 + pad);
        tc::mbar_expect_tx(bar, kUnit * 256);
        tc::tma_load_3d(tile, is_v ? &map_v : &map_k, bar, 0, h, row);
        tc::tma_load_3d(tile + 4096, is_v ? &map_v : &map_k, bar, 64, h, row);
      }
    } else {
      load_tile(tile, unit(is_v ? p.v_cache : p.k_cache, k0), row_stride, len - k0, lane);
      cp_async_commit();
    }
  };
  // wait for the warp's K (or V) tile; cp.async path: `pending` younger groups may stay in flight
  auto arrived = [&](bool is_v) {
    if (kTma) {
      uint64_t* bar = &tile_bar[warp][is_v ? 1 : 0];
      const uint32_t par = is_v ? v_phase : k_phase;
      if (!tc::mbar_try_wait(bar, par)) {
        const long long t0 = clock64();
        while (!tc::mbar_try_wait_hint(bar, par, 1000)) {
          if (clock64() - t0 > kDecodeWaitLimit) {     // give up: the result of this warp becomes NaN
            expired = true;
            break;
          }
        }
      }
      if (is_v) v_phase ^= 1u; else k_phase ^= 1u;
    } else {
      cp_async_wait<1>();
    }
    __syncwarp();
  };
  auto kt = [&](int row, int chunk) { return kTma ? tile_addr_tma(k_tile, row, chunk) : tile_addr(k_tile, row, chunk); };
  auto vt = [&](int row, int chunk) { return kTma ? tile_addr_tma(v_tile, row, chunk) : tile_addr(v_tile, row, chunk); };

  // Q fragments of the 16 heads (rows g and g + 8), all 8 k-steps
  uint32_t qf[8][4];
  {
    const __nv_bfloat16* q0 = p.q + ((int64_t)b * p.heads_q + h * kGroup + g) * kHeadDim;
    const __nv_bfloat16* q1 = q0 + 8 * kHeadDim;
#pragma unroll
    for (int ks = 0; ks < 8; ++ks) {
      qf[ks][0] = *reinterpret_cast<const uint32_t*>(q0 + ks * 16 + 2 * t);
      qf[ks][1] = *reinterpret_cast<const uint32_t*>(q1 + ks * 16 + 2 * t);
      qf[ks][2] = *reinterpret_cast<const uint32_t*>(q0 + ks * 16 + 8 + 2 * t);
      qf[ks][3] = *reinterpret_cast<const uint32_t*>(q1 + ks * 16 + 8 + 2 * t);
    }
  }

  float o[16][4];
#pragma unroll
  for (int i = 0; i < 16; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
  float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;    // rows g and g + 8 (log2 units)

  // The warp streams its blocks as 32-key units (two per block), so that the K tile of the next
  // unit is already in flight while this unit's softmax and P.V run.
  int j = j_begin + warp, half = 0;
  int blk = (j < j_end) ? list.nth(j) : -1;
  int key0 = blk * kBlockN;
  auto advance = [&](int& jj, int& hh, int& bb) -> int {          // next unit; returns its first key or -1
    if (hh == 0 && bb * kBlockN + kUnit < len) {
      hh = 1;
      return bb * kBlockN + kUnit;
    }
    jj += kWarps;
    hh = 0;
    bb = (jj < j_end) ? list.nth(jj) : -1;
    return bb >= 0 ? bb * kBlockN : -1;
  };
  if (blk >= 0) {
    fetch(false, k_tile, key0);
    fetch(true, v_tile, key0);
  } else {
    key0 = -1;
  }
  while (key0 >= 0) {
    int jn = j, hn = half, bn = blk;
    const int key_next = advance(jn, hn, bn);
    arrived(false);                     // K of this unit has landed (V may still be in flight)

    // ---- S = Q . K^T   (16 x 32)
    float s[kUnit / 8][4];
#pragma unroll
    for (int nt = 0; nt < kUnit / 8; ++nt) s[nt][0] = s[nt][1] = s[nt][2] = s[nt][3] = 0.f;
#pragma unroll
    for (int nt = 0; nt < kUnit / 8; ++nt) {
#pragma unroll
      for (int kp = 0; kp < 4; ++kp) {        // two k-steps (32 d) per ldmatrix.x4
        uint32_t bf[4];
        ldmatrix_x4(bf, kt(nt * 8 + (lane & 7), kp * 4 + (lane >> 3)));
        mma_bf16(s[nt], qf[2 * kp], bf[0], bf[1]);
        mma_bf16(s[nt], qf[2 * kp + 1], bf[2], bf[3]);
      }
    }
    __syncwarp();
    if (key_next >= 0) fetch(false, k_tile, key_next);
    else if (!kTma) cp_async_commit();        // (keeps the group count of the waits uniform)

    // ---- online softmax (rows g and g + 8; a row's scores live in the 4 lanes of a quad)
    float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
    for (int nt = 0; nt < kUnit / 8; ++nt) {
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        const bool vis = key0 + nt * 8 + 2 * t + e < len;
        s[nt][e] = vis ? s[nt][e] * p.scale_log2 : -INFINITY;
        s[nt][2 + e] = vis ? s[nt][2 + e] * p.scale_log2 : -INFINITY;
        mx0 = fmaxf(mx0, s[nt][e]);
        mx1 = fmaxf(mx1, s[nt][2 + e]);
      }
    }
    mx0 = fmaxf(mx0, __shfl_xor_sync(0xFFFFFFFFu, mx0, 1));
    mx0 = fmaxf(mx0, __shfl_xor_sync(0xFFFFFFFFu, mx0, 2));
    mx1 = fmaxf(mx1, __shfl_xor_sync(0xFFFFFFFFu, mx1, 1));
    mx1 = fmaxf(mx1, __shfl_xor_sync(0xFFFFFFFFu, mx1, 2));
    const float mn0 = fmaxf(m0, mx0), mn1 = fmaxf(m1, mx1);
    const float f0 = (mn0 == -INFINITY) ? 1.f : exp2f(m0 - mn0);
    const float f1 = (mn1 == -INFINITY) ? 1.f : exp2f(m1 - mn1);
    const float sub0 = (mn0 == -INFINITY) ? 0.f : mn0, sub1 = (mn1 == -INFINITY) ? 0.f : mn1;
    m0 = mn0;
    m1 = mn1;
    float sum0 = 0.f, sum1 = 0.f;
    uint32_t pf[kUnit / 16][4];               // P as A fragments for the k-steps of P . V
#pragma unroll
    for (int nt = 0; nt < kUnit / 8; ++nt) {
      const float p00 = exp2f(s[nt][0] - sub0), p01 = exp2f(s[nt][1] - sub0);
      const float p10 = exp2f(s[nt][2] - sub1), p11 = exp2f(s[nt][3] - sub1);
      sum0 += p00 + p01;
      sum1 += p10 + p11;
      pf[nt >> 1][(nt & 1) * 2 + 0] = pack2(p00, p01);
      pf[nt >> 1][(nt & 1) * 2 + 1] = pack2(p10, p11);
    }
    l0 = l0 * f0 + sum0;                      // per-lane partial sums; reduced over the quad at the end
    l1 = l1 * f1 + sum1;
    if (__any_sync(0xFFFFFFFFu, f0 != 1.f || f1 != 1.f)) {
#pragma unroll
      for (int i = 0; i < 16; ++i) {
        o[i][0] *= f0;
        o[i][1] *= f0;
        o[i][2] *= f1;
        o[i][3] *= f1;
      }
    }

    // ---- O += P . V   (16 x 128), V rows past `len` were never fetched: their P is 0, but the
    //      stale shared-memory bytes could be NaN, so those rows are zeroed first
    arrived(true);                            // V of this unit has landed
    if (key0 + kUnit > len) {
      for (int i = lane; i < kUnit * 16; i += 32) {
        const int row = i >> 4;
        if (key0 + row >= len)
          *reinterpret_cast<uint4*>(vt(row, i & 15)) = make_uint4(0u, 0u, 0u, 0u);
      }
      __syncwarp();
    }
#pragma unroll
    for (int kk = 0; kk < kUnit / 16; ++kk) {
#pragma unroll
      for (int np = 0; np < 8; ++np) {        // two 8-wide d tiles per ldmatrix.x4.trans
        uint32_t bf[4];
        ldmatrix_x4_trans(bf, vt(kk * 16 + (lane & 7) + ((lane >> 3) & 1) * 8, np * 2 + (lane >> 4)));
        mma_bf16(o[2 * np], pf[kk], bf[0], bf[1]);
        mma_bf16(o[2 * np + 1], pf[kk], bf[2], bf[3]);
      }
    }
    __syncwarp();
    if (key_next >= 0) fetch(true, v_tile, key_next);
    else if (!kTma) cp_async_commit();
    j = jn;
    half = hn;
    blk = bn;
    key0 = key_next;
  }
  if (!kTma) cp_async_wait<0>();
  if (__any_sync(0xFFFFFFFFu, expired)) l0 = l1 = __int_as_float(0x7FC00000);   // NaN: visible, not silent
  l0 += __shfl_xor_sync(0xFFFFFFFFu, l0, 1);
  l0 += __shfl_xor_sync(0xFFFFFFFFu, l0, 2);
  l1 += __shfl_xor_sync(0xFFFFFFFFu, l1, 1);
  l1 += __shfl_xor_sync(0xFFFFFFFFu, l1, 2);

  // ---- merge the 4 warps of the CTA through shared memory (reusing the tile space)
  __syncthreads();
  float* stage = reinterpret_cast<float*>(smem);             // [warp][16 rows][kPartialFloats]
  {
    float* w0 = stage + ((size_t)warp * 16 + g) * kPartialFloats;
    float* w1 = w0 + 8 * kPartialFloats;
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      w0[i * 8 + 2 * t] = o[i][0];
      w0[i * 8 + 2 * t + 1] = o[i][1];
      w1[i * 8 + 2 * t] = o[i][2];
      w1[i * 8 + 2 * t + 1] = o[i][3];
    }
    if (t == 0) {
      w0[kHeadDim] = m0;
      w0[kHeadDim + 1] = l0;
      w1[kHeadDim] = m1;
      w1[kHeadDim + 1] = l1;
    }
  }
  __syncthreads();
  float* dst = p.partial + ((((int64_t)b * p.heads_k + h) * p.splits + split) * 16) * kPartialFloats;
  for (int i = threadIdx.x; i < 16 * kPartialFloats; i += kThreads) {
    const int row = i / kPartialFloats, c = i - row * kPartialFloats;
    float mw[kWarps], mmax = -INFINITY;
#pragma unroll
    for (int w = 0; w < kWarps; ++w) {
      mw[w] = stage[((size_t)w * 16 + row) * kPartialFloats + kHeadDim];
      mmax = fmaxf(mmax, mw[w]);
    }
    float acc = 0.f;
    if (c == kHeadDim) {
      acc = mmax;
    } else if (c < kHeadDim + 2) {
#pragma unroll
      for (int w = 0; w < kWarps; ++w) {
        const float f = (mw[w] == -INFINITY) ? 0.f : exp2f(mw[w] - mmax);
        acc += f * stage[((size_t)w * 16 + row) * kPartialFloats + c];    // O columns and the sum
      }
    }
    dst[i] = acc;
  }
}

// one CTA per (sequence, KV head): merge the per-split partials, normalise, write bf16 + lse
__global__ void __launch_bounds__(256) decode_combine_kernel(const DecodeParams p) {
  const int h = blockIdx.x, b = blockIdx.y;
  const int row = threadIdx.x >> 4, c0 = (threadIdx.x & 15) * 8;
  const float* src = p.partial + (((int64_t)b * p.heads_k + h) * p.splits * 16 + row) * kPartialFloats;
  float ms[kMaxSplits], mmax = -INFINITY;
#pragma unroll
  for (int s = 0; s < kMaxSplits; ++s) {
    ms[s] = (s < p.splits) ? src[(size_t)s * 16 * kPartialFloats + kHeadDim] : -INFINITY;
    mmax = fmaxf(mmax, ms[s]);
  }
  float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f}, lsum = 0.f;
#pragma unroll
  for (int s = 0; s < kMaxSplits; ++s) {
    if (s >= p.splits) break;
    const float f = (ms[s] == -INFINITY) ? 0.f : exp2f(ms[s] - mmax);
    const float* ps = src + (size_t)s * 16 * kPartialFloats;
    lsum += f * ps[kHeadDim + 1];
    const float4 a = *reinterpret_cast<const float4*>(ps + c0);
    const float4 bq = *reinterpret_cast<const float4*>(ps + c0 + 4);
    acc[0] += f * a.x; acc[1] += f * a.y; acc[2] += f * a.z; acc[3] += f * a.w;
    acc[4] += f * bq.x; acc[5] += f * bq.y; acc[6] += f * bq.z; acc[7] += f * bq.w;
  }
  const float inv = (lsum > 0.f) ? 1.f / lsum : 0.f;
  const int64_t qrow = (int64_t)b * p.heads_q + h * kGroup + row;
  uint4 v4;
  v4.x = pack2(acc[0] * inv, acc[1] * inv);
  v4.y = pack2(acc[2] * inv, acc[3] * inv);
  v4.z = pack2(acc[4] * inv, acc[5] * inv);
  v4.w = pack2(acc[6] * inv, acc[7] * inv);
  *reinterpret_cast<uint4*>(p.out + qrow * kHeadDim + c0) = v4;
  if (p.lse != nullptr && (threadIdx.x & 15) == 0)
    p.lse[qrow] = (lsum > 0.f) ? (mmax + log2f(lsum)) * kLn2 : INFINITY;
}

}  // namespace
}  // namespace ifv2

using namespace ifv2;

extern "C" int64_t ifv2_decode_workspace_bytes(int batch, int heads_q, int head_dim, int max_blocks) {
  (void)max_blocks;
  if (batch < 0 || heads_q < 0 || head_dim != kHeadDim) return 0;
  return (int64_t)batch * heads_q * kMaxSplits * kPartialFloats * 4 + 256;
}

// Rotary embedding of the decode step's new key and of its query, both at the position the key is
// appended at (the reference rotates them while it copies them, flash_fwd_kernel.h:787-930 with
// rotary.h): interleaved pairs (2i, 2i+1) or halves (i, i + rotary_dim/2); features past rotary_dim
// pass through; fp32 arithmetic, one rounding.  One thread per (row, pair).
__global__ void decode_rotary_kernel(const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ k_new,
                                     __nv_bfloat16* __restrict__ q_out, __nv_bfloat16* __restrict__ k_out,
                                     const __nv_bfloat16* __restrict__ cos_t, const __nv_bfloat16* __restrict__ sin_t,
                                     const int32_t* __restrict__ cache_seqlens, int batch, int heads_q,
                                     int heads_k, int rotary_dim, int seqlen_ro, int interleaved) {
  const int rows = heads_q + heads_k;                  // per sequence: query heads, then key heads
  const int64_t n = (int64_t)batch * rows * (kHeadDim / 2);
  for (int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; idx < n;
       idx += (int64_t)gridDim.x * blockDim.x) {
    const int i = (int)(idx % (kHeadDim / 2));
    const int r = (int)((idx / (kHeadDim / 2)) % rows);
    const int b = (int)(idx / ((int64_t)(kHeadDim / 2) * rows));
    const bool is_q = r < heads_q;
    const __nv_bfloat16* src = is_q ? q + ((int64_t)b * heads_q + r) * kHeadDim
                                    : k_new + ((int64_t)b * heads_k + (r - heads_q)) * kHeadDim;
    __nv_bfloat16* dst = is_q ? q_out + ((int64_t)b * heads_q + r) * kHeadDim
                              : k_out + ((int64_t)b * heads_k + (r - heads_q)) * kHeadDim;
    const int half = rotary_dim / 2;
    // the two features this thread owns
    int i0, i1;
    if (i < half) {
      i0 = interleaved ? 2 * i : i;
      i1 = interleaved ? 2 * i + 1 : i + half;
    } else {                                            // pass-through part, two features per thread
      i0 = rotary_dim + 2 * (i - half);
      i1 = i0 + 1;
    }
    float x0 = __bfloat162float(src[i0]), x1 = __bfloat162float(src[i1]);
    if (i < half) {
      const int pos = min(max(cache_seqlens[b], 0), seqlen_ro - 1);
      const float c = __bfloat162float(cos_t[(int64_t)pos * half + i]);
      const float sn = __bfloat162float(sin_t[(int64_t)pos * half + i]);
      const float re = x0 * c - x1 * sn, im = x0 * sn + x1 * c;
      x0 = re;
      x1 = im;
    }
    dst[i0] = __float2bfloat16_rn(x0);
    dst[i1] = __float2bfloat16_rn(x1);
  }
}

static int decode_impl(const void* q, void* k_cache, void* v_cache, const void* k_new,
                       const void* v_new, void* out, float* lse, const int64_t* mask,
                       int mask_words, const int32_t* cache_seqlens, int batch, int heads_q,
                       int heads_k, int head_dim, int64_t cache_capacity,
                       int64_t cache_batch_stride, const int32_t* block_table,
                       int block_table_stride, int page_size, const int32_t* cache_batch_idx,
                       const int32_t* cache_leftpad, float softmax_scale, void* workspace,
                       int64_t workspace_bytes, void* stream) {
  IFV2_REQUIRE(head_dim == kHeadDim, IFV2_ERR_UNSUPPORTED, "decode: head_dim %d not supported (only 128)",
               head_dim);
  IFV2_REQUIRE(heads_k >= 1 && heads_q == heads_k * kGroup, IFV2_ERR_UNSUPPORTED,
               "decode: heads_q (%d) must be 16 x heads_k (%d)", heads_q, heads_k);
  IFV2_REQUIRE(batch >= 0 && cache_capacity >= 1, IFV2_ERR_INVALID_ARG, "decode: bad batch or capacity");
  if (batch == 0) return IFV2_OK;
  IFV2_REQUIRE(q && k_cache && v_cache && out && cache_seqlens && workspace, IFV2_ERR_INVALID_ARG,
               "decode: null pointer");
  IFV2_REQUIRE((k_new == nullptr) == (v_new == nullptr), IFV2_ERR_INVALID_ARG,
               "decode: pass both k_new and v_new, or neither");
  if (block_table != nullptr) {
    IFV2_REQUIRE(page_size >= kBlockN && page_size % kBlockN == 0 && block_table_stride >= 1,
                 IFV2_ERR_INVALID_ARG, "decode: page size must be a positive multiple of 64");
    IFV2_REQUIRE(cache_leftpad == nullptr && cache_batch_idx == nullptr, IFV2_ERR_UNSUPPORTED,
                 "decode: a paged cache takes neither cache_leftpad nor cache_batch_idx");
    IFV2_REQUIRE(cache_capacity <= (int64_t)block_table_stride * page_size, IFV2_ERR_INVALID_ARG,
                 "decode: cache_capacity exceeds the block table");
  } else {
    IFV2_REQUIRE(cache_batch_stride >= cache_capacity * heads_k * kHeadDim, IFV2_ERR_INVALID_ARG,
                 "decode: cache_batch_stride smaller than one sequence");
  }
  IFV2_REQUIRE(mask == nullptr || mask_words >= 1, IFV2_ERR_INVALID_ARG, "decode: mask_words < 1");
  IFV2_REQUIRE(workspace_bytes >= ifv2_decode_workspace_bytes(batch, heads_q, head_dim, 0),
               IFV2_ERR_INVALID_ARG, "decode: workspace too small");
  IFV2_REQUIRE(reinterpret_cast<uintptr_t>(workspace) % 16 == 0, IFV2_ERR_INVALID_ARG,
               "decode: workspace must be 16-byte aligned");
  IFV2_REQUIRE(batch <= 65535 && heads_k <= 65535, IFV2_ERR_TOO_LARGE, "decode: batch or heads_k > 65535");
  cudaStream_t st = (cudaStream_t)stream;
  if (k_new != nullptr) {
    decode_append_kernel<<<batch, 128, 0, st>>>(
        static_cast<__nv_bfloat16*>(k_cache), static_cast<__nv_bfloat16*>(v_cache),
        static_cast<const __nv_bfloat16*>(k_new), static_cast<const __nv_bfloat16*>(v_new),
        cache_seqlens, heads_k, cache_capacity, cache_batch_stride, block_table, block_table_stride,
        page_size, cache_batch_idx);
    int rc = check_launch("decode_append");
    if (rc) return rc;
  }
  DecodeParams p;
  p.q = static_cast<const __nv_bfloat16*>(q);
  p.k_cache = static_cast<const __nv_bfloat16*>(k_cache);
  p.v_cache = static_cast<const __nv_bfloat16*>(v_cache);
  p.mask = reinterpret_cast<const unsigned long long*>(mask);
  p.mask_words = mask_words;
  p.cache_seqlens = cache_seqlens;
  p.new_tokens = k_new != nullptr ? 1 : 0;
  p.capacity = cache_capacity;
  p.heads_q = heads_q;
  p.heads_k = heads_k;
  p.batch_stride = cache_batch_stride;
  p.block_table = block_table;
  p.bt_stride = block_table_stride;
  p.page_size = page_size > 0 ? page_size : 1;
  p.cache_batch_idx = cache_batch_idx;
  p.leftpad = cache_leftpad;
  p.scale_log2 = softmax_scale * kLog2e;
  // One wave: as many CTAs per (sequence, KV head) as still fit the SMs all at once.  A launch
  // that spills into a second, mostly empty wave takes twice as long (measured at batch 64 x 2 KV
  // heads, top-64: 3 splits = 384 CTAs on 444 slots 62 us, 4 splits = 512 CTAs 78 us, 8 splits 79 us).
  const int64_t slots = (int64_t)kNumSMs * IFV2_DECODE_CTAS_PER_SM;
  const int64_t pairs = (int64_t)batch * heads_k;
  int splits = (int)(slots / pairs);
  if (splits < 1) splits = 1;
  if (splits > kMaxSplits) splits = kMaxSplits;
  p.splits = splits;
  p.partial = static_cast<float*>(workspace);
  p.out = static_cast<__nv_bfloat16*>(out);
  p.lse = lse;
  const size_t smem = ((size_t)kWarps * kWarpSmem > (size_t)kWarps * 16 * kPartialFloats * 4
                           ? (size_t)kWarps * kWarpSmem : (size_t)kWarps * 16 * kPartialFloats * 4) + 1024;
  // TMA needs the caches as (rows, heads_k, 128) views: 16-byte aligned bases and, without a block
  // table, a batch stride of whole rows.  The row extent of the maps is only a clipping bound; the
  // kernel never asks for a row outside the sequences' own positions.
  const int64_t row_elems = (int64_t)heads_k * kHeadDim;
  const bool tma_ok = reinterpret_cast<uintptr_t>(k_cache) % 16 == 0 && reinterpret_cast<uintptr_t>(v_cache) % 16 == 0 &&
                      (block_table != nullptr || cache_batch_stride % row_elems == 0);
  p.use_tma = tma_ok ? 1 : 0;
  p.rows_per_slot = tma_ok && block_table == nullptr ? cache_batch_stride / row_elems : 0;
  CUtensorMap map_k, map_v;
  if (tma_ok) {
    const uint64_t rows = 0x7FFFFFFFull;
    int rc2 = make_tensor_map_bf16_3d(&map_k, k_cache, kHeadDim, heads_k, rows, kHeadDim * 2,
                                      (uint64_t)row_elems * 2, 64, 1, kUnit);
    if (rc2) return rc2;
    rc2 = make_tensor_map_bf16_3d(&map_v, v_cache, kHeadDim, heads_k, rows, kHeadDim * 2,
                                  (uint64_t)row_elems * 2, 64, 1, kUnit);
    if (rc2) return rc2;
  } else {
    memset(&map_k, 0, sizeof(map_k));
    memset(&map_v, 0, sizeof(map_v));
  }
  cudaError_t e = cudaFuncSetAttribute(tma_ok ? decode_split_kernel<true> : decode_split_kernel<false>,
                                       cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return set_error((int)e, "decode: %s", cudaGetErrorString(e));
  if (tma_ok)
    decode_split_kernel<true><<<dim3(p.splits, heads_k, batch), kThreads, smem, st>>>(map_k, map_v, p);
  else
    decode_split_kernel<false><<<dim3(p.splits, heads_k, batch), kThreads, smem, st>>>(map_k, map_v, p);
  int rc = check_launch("decode_split");
  if (rc) return rc;
  decode_combine_kernel<<<dim3(heads_k, batch), 256, 0, st>>>(p);
  return check_launch("decode_combine");
}

extern "C" int ifv2_decode(const void* q, void* k_cache, void* v_cache, const void* k_new,
                           const void* v_new, void* out, float* lse, const int64_t* mask,
                           int mask_words, const int32_t* cache_seqlens, int batch, int heads_q,
                           int heads_k, int head_dim, int64_t cache_capacity,
                           int64_t cache_batch_stride, float softmax_scale, void* workspace,
                           int64_t workspace_bytes, void* stream) {
  return decode_impl(q, k_cache, v_cache, k_new, v_new, out, lse, mask, mask_words, cache_seqlens,
                     batch, heads_q, heads_k, head_dim, cache_capacity, cache_batch_stride, nullptr, 0,
                     0, nullptr, nullptr, softmax_scale, workspace, workspace_bytes, stream);
}

extern "C" int ifv2_decode_paged(const void* q, void* k_cache, void* v_cache, const void* k_new,
                                 const void* v_new, void* out, float* lse, const int64_t* mask,
                                 int mask_words, const int32_t* cache_seqlens, int batch,
                                 int heads_q, int heads_k, int head_dim, int64_t cache_capacity,
                                 int64_t cache_batch_stride, const int32_t* block_table,
                                 int block_table_stride, int page_size,
                                 const int32_t* cache_batch_idx, const int32_t* cache_leftpad,
                                 float softmax_scale, void* workspace, int64_t workspace_bytes,
                                 void* stream) {
  return decode_impl(q, k_cache, v_cache, k_new, v_new, out, lse, mask, mask_words, cache_seqlens,
                     batch, heads_q, heads_k, head_dim, cache_capacity, cache_batch_stride, block_table,
                     block_table_stride, page_size, cache_batch_idx, cache_leftpad, softmax_scale,
                     workspace, workspace_bytes, stream);
}

extern "C" int ifv2_decode_rotary(const void* q, const void* k_new, void* q_out, void* k_out,
                                  const void* rotary_cos, const void* rotary_sin,
                                  const int32_t* cache_seqlens, int batch, int heads_q, int heads_k,
                                  int head_dim, int rotary_dim, int seqlen_ro, int interleaved,
                                  void* stream) {
  IFV2_REQUIRE(head_dim == kHeadDim, IFV2_ERR_UNSUPPORTED, "decode_rotary: head_dim %d not supported (only 128)",
               head_dim);
  IFV2_REQUIRE(batch >= 0 && heads_q >= 1 && heads_k >= 1 && seqlen_ro >= 1, IFV2_ERR_INVALID_ARG,
               "decode_rotary: bad size");
  IFV2_REQUIRE(rotary_dim >= 0 && rotary_dim <= kHeadDim && rotary_dim % 16 == 0, IFV2_ERR_INVALID_ARG,
               "decode_rotary: rotary_dim must be a multiple of 16 and <= head_dim");
  if (batch == 0) return IFV2_OK;
  IFV2_REQUIRE(q && k_new && q_out && k_out && cache_seqlens && (rotary_dim == 0 || (rotary_cos && rotary_sin)),
               IFV2_ERR_INVALID_ARG, "decode_rotary: null pointer");
  const int64_t n = (int64_t)batch * (heads_q + heads_k) * (kHeadDim / 2);
  int64_t blocks = ceil_div64(n, 256);
  if (blocks > (int64_t)kNumSMs * 8) blocks = (int64_t)kNumSMs * 8;
  decode_rotary_kernel<<<(int)blocks, 256, 0, (cudaStream_t)stream>>>(
      static_cast<const __nv_bfloat16*>(q), static_cast<const __nv_bfloat16*>(k_new),
      static_cast<__nv_bfloat16*>(q_out), static_cast<__nv_bfloat16*>(k_out),
      static_cast<const __nv_bfloat16*>(rotary_cos), static_cast<const __nv_bfloat16*>(rotary_sin),
      cache_seqlens, batch, heads_q, heads_k, rotary_dim, seqlen_ro, interleaved ? 1 : 0);
  return check_launch("decode_rotary");
}
