// Stage-1 scorer: group-summed softmax probabilities of the queries against the compressed keys,
// optionally max-pooled to 64-token block scores in the same kernel.
//
// One CTA (one per SM) owns 16 consecutive tokens x the 16 query heads of one KV head: two 128-row
// query tiles A and B, each fetched by 3-D TMA boxes from the caller's (token, head, d) layout, and
// streams 128-key tiles of the compressed keys twice through a 4-slot ring.  Every key tile serves
// both query tiles, which halves the L2 -> SM key traffic per score against an 8-token CTA:
//   pass 1:  S = Q_t . Kc^T  (rows = query rows of tile t in TMEM lanes) -> reference point m
//            and sum l per row
//   pass 2:  S^T = Kc . Q_t^T  (rows = keys in TMEM lanes)
//            -> p = exp2(c*s - c*m - log2 l); because the 16 heads of a token are now 16 adjacent
//            COLUMNS of one thread's row, the GQA group sum is an in-register sum.
// Both passes use the same swizzled shared-memory tiles with the operand roles swapped.
// In pass 2 the per-row constant -(c*m + log2 l)/c rides along inside the tensor-core product as
// one extra 16-wide K step (a tile of ones against a tile holding the constant split into three
// bf16 terms), so the softmax warps do one multiply and one ex2 per score and nothing else.
// Pass 1 does not track the running maximum: m is the maximum of the row's first visible 32-key
// chunk and stays fixed, so a score costs one FMA, one ex2 and one add; the sum is exact for any
// reference point as long as it stays finite, and a chunk whose sum leaves the fp32 range (a score
// more than ~100 log2 units above m) is redone with a fresh maximum.
// The bf16 result row (Hk, token, key) is written straight from registers, columns past the last
// visible key are zero-filled (no pre-zeroing, slice or NaN scrub).  With pooling enabled each
// tile's 128 x 16 scores also go through a small shared-memory window and leave as 32 x 16 block
// scores (5-wide / stride-4 max, +inf on the init and causal-local blocks), bit-identical to
// running the max-pool kernel on the score tensor.
// The two query tiles are two independent pipelines that share nothing but the key ring: each has
// its own MMA-issuing warp, its own pair of 128-column accumulator buffers in TMEM, its own eight
// softmax warps and its own barriers, so the tiles drift out of phase and one tile's exponentials
// fill the special-function unit while the other waits, loads or pools (a single lock-stepped
// pipeline leaves the unit idle in those phases).
// Warp roles: warp 0 = TMA producer, warps 1-2 = MMA issuers (tile A, tile B), warps 3-18 =
// softmax: per tile two groups of four warps; both groups cover all 128 TMEM lanes and each takes
// half of every accumulator's 128 columns (pass 1: 64 of the keys, merged once at the end;
// pass 2: 4 of the tile's 8 tokens).
#include "tc05.cuh"

namespace ifv2 {
namespace {

using namespace tc;

constexpr int kTokPerCta = 16;
constexpr int kTokPerBox = 8;                 // tokens of one 128-row query tile
constexpr int kHalfThreads = 256;              // softmax threads of one query tile
constexpr int kSoftmaxThreads = 2 * kHalfThreads;
constexpr int kThreads = 96 + kSoftmaxThreads; // + TMA warp + two MMA warps
constexpr int kKeysPerTile = 128;
constexpr int kStages = 4;                    // key-tile ring
constexpr uint32_t kHalfBytes = 128 * 128;    // 128 rows x 64 bf16
constexpr uint32_t kTmemCols = 512;
constexpr int kPoolSlots = 136;               // 1 halo + 128 keys, padded
#ifndef IFV2_STAGE1_POLY_STRIDE
#define IFV2_STAGE1_POLY_STRIDE 0
#endif
// every kPolyStride-th exponential of a row runs as a polynomial on the FMA pipe (0: none).  Measured at
// 131072 tokens: strides 0, 6 and 8 run within 1 % of each other and 4 is 5 % slower -- the kernel is
// bound by the per-step chain of its softmax warps, not by the throughput of the exponential unit.
constexpr int kPolyStride = IFV2_STAGE1_POLY_STRIDE;
__device__ __forceinline__ float exp2_mixed(float x, int c) {
  return (kPolyStride > 0 && c % (kPolyStride > 0 ? kPolyStride : 1) == (kPolyStride - 1))
             ? exp2_fma(x) : exp2f(x);
}
// the same for pass 1, whose argument is not bounded above: past 2^128 the polynomial form must
// produce inf / NaN (which the overflow check catches), not wrap into the sign bit
__device__ __forceinline__ float exp2_mixed_unbounded(float x, int c) {
  return (kPolyStride > 0 && c % (kPolyStride > 0 ? kPolyStride : 1) == (kPolyStride - 1))
             ? exp2_fma(fminf(x, 128.f)) : exp2f(x);
}
constexpr float kSumLimit = 1e30f;            // a chunk sum at or above this is redone with a fresh maximum

struct Stage1Params {
  __nv_bfloat16* out;             // scores, may be null when only block scores are wanted
  __nv_bfloat16* pooled;          // block scores, may be null
  const int32_t* cu_q;
  const int32_t* cu_k;
  const int32_t* cu_v;            // keys of the row sums (pass 1); null = the keys of pass 2
  const int32_t* seqused_k;       // keys in use per sequence (<= its cu_k extent), may be null
  const int32_t* seqused_v;       // the same for the row-sum keys (needs cu_v), may be null
  const int32_t* cache_lens;      // per sequence, may be null
  const int32_t* leftpad_k;       // scored keys start this many rows into the sequence's extent, or null
  const int32_t* block_table;     // (batch, bt_stride) page of every page_size scored keys, or null
  int bt_stride, page_size;
  int64_t total_q;
  int heads_q, heads_k;
  int max_seqlen_k;
  int64_t out_row_stride;
  int pooled_len, cache_len, local_blocks, init_blocks;
  float scale_log2, inv_scale_log2;
  int causal;
  int32_t* status;
};

struct Smem {
  uint8_t q[2][2][kHalfBytes];         // [query tile][d half]
  uint8_t kc[kStages][2][kHalfBytes];  // [stage][d half]
  uint8_t ones[4096];                  // 128 x 16 bf16, no swizzle: columns 0..2 = 1
  uint8_t rowc[2][4096];               // per query tile, 128 x 16 bf16, no swizzle: columns 0..2 = row constant (3 terms)
  __nv_bfloat16 pool[2][3][kTokPerBox][kPoolSlots];   // per query tile: scores of the last three key tiles
  __nv_bfloat16 carry[2][4][kTokPerBox];              // (pooling is deferred by one tile), and each tile's last key
  float2 stat[2][128];                 // pass-1 (reference point, sum) of the second column half, per row
  // kc_free[s]: the products of BOTH query tiles that read key slot s are complete (2 arrivals);
  // per query tile: acc_full[b]: accumulator buffer b holds a step's scores; acc_empty[b]: its 8
  // softmax warps have read it
  uint64_t q_full, kc_full[kStages], kc_free[kStages], acc_full[2][2], acc_empty[2][2], rowc_ready[2],
      pool_full[2][3];
  uint32_t tmem_base;
  int abort_flag;
};

// Number of leading compressed keys visible to local token i (C integer division, as the
// reference's device code): with compression stride st, key j covers tokens [st*j, st*j + 2*st)
// and the pattern is aligned to the END of the keys when the query segment is shorter than the
// keys cover.  st = 16 for the scored keys; the coarse keys of the row sums use 64.
__device__ __forceinline__ int visible_limit(int i, int lq, int lc, int causal, int st = 16) {
  if (!causal) return lc;
  const int off = lc - (lq - st + 1) / st;
  return min(lc, max(0, (i + 1) / st - 1 + off));
}

__device__ __forceinline__ float bf16_round(float x) {
  return __bfloat162float(__float2bfloat16_rn(x));
}

template <bool kPooled>
__global__ void __launch_bounds__(kThreads, 1)      // 19 warps: at most 96 registers per thread
stage1_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_kc,
              const __grid_constant__ CUtensorMap map_kv, const Stage1Params p) {
  extern __shared__ uint8_t smem_raw[];
  Smem& sm = *reinterpret_cast<Smem*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                      ~(uintptr_t)1023);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int b = blockIdx.y, h = blockIdx.z;
  const int q0 = p.cu_q[b], lq = p.cu_q[b + 1] - q0;
  // scored keys of the sequence: rows [k0, k0 + lc) of a packed tensor (optionally starting
  // `leftpad_k` rows into the sequence's extent), or positions [0, lc) of a paged cache
  int k0, lc;
  {
    const int pad = p.leftpad_k ? p.leftpad_k[b] : 0;
    const int extent = p.cu_k[b + 1] - p.cu_k[b];
    k0 = p.block_table ? 0 : p.cu_k[b] + pad;
    lc = max(0, (p.seqused_k ? min(p.seqused_k[b], extent) : extent) - pad);
  }
  const int tok0 = ((int)gridDim.x - 1 - (int)blockIdx.x) * kTokPerCta;   // long tiles first
  if (tok0 >= lq) return;
  // an earlier CTA of this launch gave up on a wait: do not pile up more waits
  if (*reinterpret_cast<volatile int32_t*>(p.status) != 0) return;
  const int ntok = min(kTokPerCta, lq - tok0);
  const int lim_max = visible_limit(tok0 + ntok - 1, lq, lc, p.causal);    // limits grow with i
  // Pass 1 (row sums) runs over the keys given as `v`: the same compressed keys, or a coarser
  // compression (kernel 128 / stride 64) whose log-sum-exp then normalises the scores of
  // pass 2 -- the reference switches on the key counts (flash_fwd_kernel.h:1236-1240)
  const int v0 = p.cu_v ? p.cu_v[b] : k0;
  const int lcv = !p.cu_v ? lc
                  : p.seqused_v ? max(0, min(p.seqused_v[b], p.cu_v[b + 1] - v0)) : p.cu_v[b + 1] - v0;
  const int st1 = (lcv == lc) ? 16 : 64;
  const int lim_max1 = visible_limit(tok0 + ntok - 1, lq, lcv, p.causal, st1);
  // (read through a warp broadcast: it tells the compiler that the value is warp-uniform, so the
  //  MMA issuer's descriptor arithmetic stays in uniform registers instead of being moved there
  //  operand by operand for every MMA)
  const int n_tiles = __shfl_sync(0xFFFFFFFFu, (lim_max + kKeysPerTile - 1) / kKeysPerTile, 0);
  const int n_tiles1 = __shfl_sync(0xFFFFFFFFu, (lim_max1 + kKeysPerTile - 1) / kKeysPerTile, 0);
  const int n_steps = n_tiles1 + n_tiles;      // pass-1 tiles, then pass-2 tiles

  if (threadIdx.x == 0) {
    sm.abort_flag = 0;
    mbar_init(&sm.q_full, 1);
    for (int s = 0; s < kStages; ++s) {
      mbar_init(&sm.kc_full[s], 1);
      mbar_init(&sm.kc_free[s], 2);               // one commit per MMA warp
    }
    for (int hq = 0; hq < 2; ++hq) {
      for (int s = 0; s < 2; ++s) {
        mbar_init(&sm.acc_full[hq][s], 1);
        mbar_init(&sm.acc_empty[hq][s], 8);       // one arrival per softmax warp of the tile
      }
      mbar_init(&sm.rowc_ready[hq], 4);
      for (int s = 0; s < 3; ++s) mbar_init(&sm.pool_full[hq][s], 8);
    }
    fence_barrier_init();
    prefetch_tensormap(&map_q);
    prefetch_tensormap(&map_kc);
    prefetch_tensormap(&map_kv);
  }
  if (warp == 1) {
    tmem_alloc(&sm.tmem_base, kTmemCols);
    tmem_relinquish();
  }
  // the tile of ones (columns 0..2) and the zero part of the row-constant tiles
  for (int i = threadIdx.x; i < 4096 / 4; i += kThreads) reinterpret_cast<uint32_t*>(sm.ones)[i] = 0u;
  for (int i = threadIdx.x; i < 8192 / 4; i += kThreads) reinterpret_cast<uint32_t*>(sm.rowc)[i] = 0u;
  __syncthreads();
  if (threadIdx.x < 128) {
    const __nv_bfloat16 one = __float2bfloat16_rn(1.f);
    for (int c = 0; c < 3; ++c)
      *reinterpret_cast<__nv_bfloat16*>(sm.ones + umma_noswz16_off(threadIdx.x, c)) = one;
  }
  fence_proxy_async_smem();
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = __shfl_sync(0xFFFFFFFFu, sm.tmem_base, 0);
  volatile int* abort_flag = &sm.abort_flag;

  if (warp == 0) {
    // ================================================================ TMA producer
    if (lane == 0 && n_steps > 0) {
      mbar_expect_tx(&sm.q_full, 4 * kHalfBytes);
      for (int tile = 0; tile < 2; ++tile)       // rows past the last token come back as zeros or as
        for (int dh = 0; dh < 2; ++dh)           // the next sequence's rows; they are never stored
          tma_load_3d(sm.q[tile][dh], &map_q, &sm.q_full, dh * 64, h * kGroup, q0 + tok0 + tile * kTokPerBox);
      int issued = 0;
      for (int t = 0; t < n_steps; ++t) {
        const int s = t % kStages;
        if (t >= kStages && !mbar_wait(&sm.kc_free[s], (uint32_t)((t / kStages - 1) & 1), abort_flag,
                                       p.status, 41))
          break;
        mbar_expect_tx(&sm.kc_full[s], 2 * kHalfBytes);
        if (t < n_tiles1) {
          int row = v0 + t * kKeysPerTile;
          if (p.block_table != nullptr)          // (the row sums then run over the scored keys themselves)
            row = __ldg(p.block_table + (int64_t)b * p.bt_stride + (t * kKeysPerTile) / p.page_size) * p.page_size +
                  (t * kKeysPerTile) % p.page_size;
          tma_load_3d(sm.kc[s][0], &map_kv, &sm.kc_full[s], 0, h, row);
          tma_load_3d(sm.kc[s][1], &map_kv, &sm.kc_full[s], 64, h, row);
        } else {
          const int pos = (t - n_tiles1) * kKeysPerTile;
          int row = k0 + pos;
          if (p.block_table != nullptr)          // a 128-key tile never straddles a page
            row = __ldg(p.block_table + (int64_t)b * p.bt_stride + pos / p.page_size) * p.page_size +
                  pos % p.page_size;
          tma_load_3d(sm.kc[s][0], &map_kc, &sm.kc_full[s], 0, h, row);
          tma_load_3d(sm.kc[s][1], &map_kc, &sm.kc_full[s], 64, h, row);
        }
        issued = t + 1;
      }
      if (*abort_flag) {
        mbar_wait_drain(&sm.q_full, 0);
        for (int j = max(0, issued - kStages); j < issued; ++j)
          mbar_wait_drain(&sm.kc_full[j % kStages], (uint32_t)((j / kStages) & 1));
      }
    }
  } else if (warp <= 2) {
    // ================================================================ MMA issuer of query tile hq
    // All 32 lanes run the same issue code (descriptors stay in uniform registers); `leader`
    // enables the MMA / commit instructions in one lane only.
    if (n_steps > 0) {
      const int hq = __shfl_sync(0xFFFFFFFFu, warp - 1, 0);
      const uint32_t leader = (lane == 0) ? 1u : 0u;
      constexpr uint32_t idesc = umma_idesc_bf16(128, 128, false);
      const uint64_t q_desc = umma_desc_sw128(smem_u32(sm.q[0][0]), 16, 1024) + (uint32_t)hq * ((2 * kHalfBytes) >> 4);
      const uint64_t kc_desc0 = umma_desc_sw128(smem_u32(sm.kc[0][0]), 16, 1024);
      constexpr uint32_t kStage = (2 * kHalfBytes) >> 4;      // descriptor address units per ring stage
      const uint64_t d_ones = umma_desc_noswz16(smem_u32(sm.ones));
      const uint64_t d_rowc = umma_desc_noswz16(smem_u32(sm.rowc[0])) + (uint32_t)hq * (4096u >> 4);
      const uint32_t acc0 = tmem + (uint32_t)hq * 256u;
      bool ok = __all_sync(0xFFFFFFFFu, mbar_wait(&sm.q_full, 0, abort_flag, p.status, 51));
      for (int t = 0; t < n_steps && ok; ++t) {
        const int s = t % kStages, ab = t & 1;
        const bool pass2 = t >= n_tiles1;
        bool w = mbar_wait(&sm.kc_full[s], (uint32_t)((t / kStages) & 1), abort_flag, p.status, 52);
        if (w && t >= 2)
          w = mbar_wait(&sm.acc_empty[hq][ab], (uint32_t)(((t >> 1) & 1) ^ 1), abort_flag, p.status, 53);
        if (w && t == n_tiles1) w = mbar_wait(&sm.rowc_ready[hq], 0, abort_flag, p.status, 54);
        ok = __all_sync(0xFFFFFFFFu, w);
        if (!ok) break;
        tc_fence_after();
        const uint64_t kc_desc = kc_desc0 + (uint32_t)s * kStage;
        const uint32_t acc = acc0 + (uint32_t)ab * 128u;
        if (!pass2) {
#pragma unroll
          for (int kk = 0; kk < 8; ++kk) {
            const uint32_t off = ((kk >> 2) * kHalfBytes + (kk & 3) * 32) >> 4;
            umma_ss_pred(acc, q_desc + off, kc_desc + off, idesc, kk > 0, leader);
          }
        } else {
#pragma unroll
          for (int kk = 0; kk < 8; ++kk) {
            const uint32_t off = ((kk >> 2) * kHalfBytes + (kk & 3) * 32) >> 4;
            umma_ss_pred(acc, kc_desc + off, q_desc + off, idesc, kk > 0, leader);
          }
          umma_ss_pred(acc, d_ones, d_rowc, idesc, true, leader);   // + row constant
        }
        umma_commit_pred(&sm.kc_free[s], leader);
        umma_commit_pred(&sm.acc_full[hq][ab], leader);
      }
    }
  } else {
    // ================================================================ softmax warps
    const int hq = (warp - 3) >> 3;                  // query tile
    const int quad = warp & 3;
    const int grp = ((warp - 3) >> 2) & 1;           // which half of the accumulator's columns
    const int r = quad * 32 + lane;                  // TMEM lane: pass 1 = query row, pass 2 = key
    const uint32_t lane_off = ((uint32_t)(quad * 32) << 16) + (uint32_t)(hq * 256 + grp * 64);
    const int st = threadIdx.x - 96 - hq * kHalfThreads;   // 0..255 among the tile's softmax threads
    const int tokh = tok0 + hq * kTokPerBox;         // first token of this tile
    const int ntokh = min(max(ntok - hq * kTokPerBox, 0), kTokPerBox);
    uint64_t* acc_full = sm.acc_full[hq];
    uint64_t* acc_empty = sm.acc_empty[hq];
    uint64_t* pool_full = sm.pool_full[hq];
    bool ok = true;

    // ---------------- pass 1: sum of this thread's query row over its half of every key tile
    {
      const int tl = r >> 4;
      const int lim_row = (tl < ntokh) ? visible_limit(tokh + tl, lq, lcv, p.causal, st1) : 0;
      float m = -INFINITY, l = 0.f;
      for (int t = 0; t < n_tiles1; ++t) {
        const int ab = t & 1;
        ok = mbar_wait_warp(&acc_full[ab], (uint32_t)((t >> 1) & 1), abort_flag, p.status, 61);
        if (!ok) break;
        tc_fence_after();
        // visible columns among this group's 64
        const int lim = min(max(lim_row - t * kKeysPerTile - grp * 64, 0), 64);
        const bool full = __all_sync(0xFFFFFFFFu, lim == 64);
        uint32_t x[64];
        tmem_ld64_wait(tmem + lane_off + ab * 128, x);
        // the scores are in registers: the accumulator goes back to the MMA warp at once
        tc_fence_before();
        mbar_arrive_warp(&acc_empty[ab]);
        if (!full) {
#pragma unroll
          for (int c = 0; c < 64; ++c)
            if (c >= lim) x[c] = 0xFF800000u;                             // -inf
        }
        if (m == -INFINITY) {            // no visible score yet: the first one fixes the reference point
          float mx = -INFINITY;
#pragma unroll
          for (int c = 0; c < 64; ++c) mx = fmaxf(mx, __uint_as_float(x[c]));
          m = mx;
        }
        if (m > -INFINITY) {
          float neg = -m * p.scale_log2;
          const uint64_t c2 = pack_f32x2(p.scale_log2, p.scale_log2), n2 = pack_f32x2(neg, neg);
          uint64_t s2[4];
#pragma unroll
          for (int i = 0; i < 4; ++i) s2[i] = pack_f32x2(0.f, 0.f);
#pragma unroll
          for (int c = 0; c < 64; c += 2) {
            float a0, a1;
            unpack_f32x2(fma_f32x2(pack_f32x2(x[c], x[c + 1]), c2, n2), a0, a1);
            s2[(c >> 1) & 3] = add_f32x2(s2[(c >> 1) & 3], pack_f32x2(exp2_mixed_unbounded(a0, c),
                                                                      exp2_mixed_unbounded(a1, c + 1)));
          }
          float lo, hi;
          unpack_f32x2(add_f32x2(add_f32x2(s2[0], s2[1]), add_f32x2(s2[2], s2[3])), lo, hi);
          float cs = lo + hi;
          if (!(cs < kSumLimit)) {       // a score far above the reference point: move the point to the maximum
            float mx = m;
#pragma unroll
            for (int c = 0; c < 64; ++c) mx = fmaxf(mx, __uint_as_float(x[c]));
            l *= exp2f((m - mx) * p.scale_log2);
            m = mx;
            neg = -m * p.scale_log2;
            cs = 0.f;
#pragma unroll
            for (int c = 0; c < 64; ++c) cs += exp2f(fmaf(__uint_as_float(x[c]), p.scale_log2, neg));
          }
          l += cs;
        }
      }
      // merge the two key halves of every row, then publish the row constant for pass 2, in
      // units of the raw score: -(m + log2(l) / c), as three bf16 terms
      if (grp == 1) sm.stat[hq][r] = make_float2(m, l);
      if (hq == 0) asm volatile("bar.sync 1, 256;" ::: "memory");
      else asm volatile("bar.sync 2, 256;" ::: "memory");
      if (grp == 0) {
        const float2 o = sm.stat[hq][r];
        const float mm = fmaxf(m, o.x);
        if (mm > -INFINITY)
          l = l * ((m > -INFINITY) ? exp2f((m - mm) * p.scale_log2) : 0.f) +
              o.y * ((o.x > -INFINITY) ? exp2f((o.x - mm) * p.scale_log2) : 0.f);
        m = mm;
        // a row without any visible pass-1 key scores 0 everywhere, as in the reference's oracle
        // (tests/stage1/complse_online_softmax.py: its NaN row sum is scrubbed to 0)
        const float rc = (l > 0.f) ? -(m + log2f(l) * p.inv_scale_log2) : -30000.f;
        const float t0 = bf16_round(rc), t1 = bf16_round(rc - t0), t2 = bf16_round(rc - t0 - t1);
        uint8_t* rowc = sm.rowc[hq];
        *reinterpret_cast<__nv_bfloat16*>(rowc + umma_noswz16_off(r, 0)) = __float2bfloat16_rn(t0);
        *reinterpret_cast<__nv_bfloat16*>(rowc + umma_noswz16_off(r, 1)) = __float2bfloat16_rn(t1);
        *reinterpret_cast<__nv_bfloat16*>(rowc + umma_noswz16_off(r, 2)) = __float2bfloat16_rn(t2);
        fence_proxy_async_smem();
        mbar_arrive_warp(&sm.rowc_ready[hq]);
      }
    }

    // ---------------- pass 2: this thread's key against 4 tokens x 16 heads
    constexpr int kTokPerThread = kTokPerBox / 2;            // tokens grp*4 .. grp*4+3 of the tile
    int lim_tok[kTokPerThread];
    const int cache_len = p.cache_lens ? p.cache_lens[b] : p.cache_len;
#pragma unroll
    for (int j = 0; j < kTokPerThread; ++j) {
      // a token without any visible row-sum key scores exactly 0 (the huge negative row constant
      // alone leaves 2^-125 per polynomial exponential)
      const int tk = tokh + grp * kTokPerThread + j;
      lim_tok[j] = (grp * kTokPerThread + j < ntokh && visible_limit(tk, lq, lcv, p.causal, st1) > 0)
                       ? visible_limit(tk, lq, lc, p.causal) : 0;
    }
    __nv_bfloat16* out_base =
        p.out ? p.out + ((int64_t)h * p.total_q + q0 + tokh) * p.out_row_stride : nullptr;
    __nv_bfloat16* pool_base =
        kPooled ? p.pooled + ((int64_t)h * p.total_q + q0 + tokh) * p.pooled_len : nullptr;
    const __nv_bfloat16 ninf_b = __float2bfloat16_rn(-INFINITY);
    __nv_bfloat16 (*pool)[kTokPerBox][kPoolSlots] = sm.pool[hq];
    __nv_bfloat16 (*carry)[kTokPerBox] = sm.carry[hq];

    // Max-pool of one finished key tile: 32 blocks x 8 tokens, one per thread.  It runs one tile
    // late, after the next tile's exponentials, so that no warp waits for the others here.
    auto pool_tile = [&](int tile) -> bool {
      if (!mbar_wait_warp(&pool_full[tile % 3], (uint32_t)((tile / 3) & 1), abort_flag, p.status, 63))
        return false;
      {
        const int t8 = st >> 5, bl = st & 31;
        const int blk = tile * 32 + bl;
        const __nv_bfloat16* w = &pool[tile % 3][t8][4 * bl];             // slots 4bl .. 4bl+4
        float mxv = fmaxf(fmaxf(__bfloat162float(w[1]), __bfloat162float(w[2])),
                          fmaxf(__bfloat162float(w[3]), __bfloat162float(w[4])));
        float first = -INFINITY;                                          // key 4*blk - 1
        if (bl > 0) first = __bfloat162float(w[0]);
        else if (tile > 0) first = __bfloat162float(carry[(tile - 1) & 3][t8]);
        mxv = fmaxf(mxv, first);
        const int bq = (tokh + t8 + cache_len) / kBlockN;
        if (blk < p.init_blocks || (bq >= blk && bq <= blk + p.local_blocks)) mxv = INFINITY;
        if (t8 < ntokh && blk < p.pooled_len)
          pool_base[(int64_t)t8 * p.pooled_len + blk] = __float2bfloat16_rn(mxv);
      }
      return true;
    };

    if (ok) {
      for (int t = n_tiles1; t < n_steps; ++t) {
        const int ab = t & 1, tile = t - n_tiles1;
        ok = mbar_wait_warp(&acc_full[ab], (uint32_t)((t >> 1) & 1), abort_flag, p.status, 62);
        if (!ok) break;
        tc_fence_after();
        const int key = tile * kKeysPerTile + r;
        float val[kTokPerThread];
        uint32_t x[64];                                   // 4 tokens x 16 heads
        tmem_ld64_wait(tmem + lane_off + ab * 128, x);
        // the accumulator is in registers now: hand it back before the arithmetic
        tc_fence_before();
        mbar_arrive_warp(&acc_empty[ab]);
        {
          const uint64_t c2 = pack_f32x2(p.scale_log2, p.scale_log2);
#pragma unroll
          for (int j = 0; j < kTokPerThread; ++j) {
            uint64_t a2[2] = {pack_f32x2(0.f, 0.f), pack_f32x2(0.f, 0.f)};
#pragma unroll
            for (int g = 0; g < 16; g += 2) {
              float y0, y1;
              unpack_f32x2(mul_f32x2(pack_f32x2(x[j * 16 + g], x[j * 16 + g + 1]), c2), y0, y1);
              a2[(g >> 1) & 1] = add_f32x2(a2[(g >> 1) & 1], pack_f32x2(exp2_mixed(y0, g), exp2_mixed(y1, g + 1)));
            }
            float lo, hi;
            unpack_f32x2(add_f32x2(a2[0], a2[1]), lo, hi);
            val[j] = lo + hi;
          }
        }
        if (kPooled && tile > 0) {
          ok = pool_tile(tile - 1);
          if (!ok) break;
        }
#pragma unroll
        for (int j = 0; j < kTokPerThread; ++j) {
          const int t8 = grp * kTokPerThread + j;
          // existing but invisible keys score 0; keys past the sequence do not exist (-inf in the pool)
          const __nv_bfloat16 vb = __float2bfloat16_rn((key < lim_tok[j]) ? val[j] : 0.f);
          if (out_base != nullptr && t8 < ntokh && key < p.max_seqlen_k)
            out_base[(int64_t)t8 * p.out_row_stride + key] = vb;
          if (kPooled) {
            const __nv_bfloat16 pv = (key < lc) ? vb : ninf_b;
            pool[tile % 3][t8][1 + r] = pv;
            if (r == 127) carry[tile & 3][t8] = pv;
          }
        }
        // (after the deferred pooling reads: this arrival is what lets a later tile reuse them)
        if (kPooled) mbar_arrive_warp(&pool_full[tile % 3]);
      }
      if (ok && kPooled && n_tiles > 0) ok = pool_tile(n_tiles - 1);
      // columns past the last tile are zero (rows are 16-byte aligned: stride % 8 == 0)
      const int first = n_tiles * kKeysPerTile;
      if (ok && out_base != nullptr && first < p.max_seqlen_k) {
        const int vec_per_row = (p.max_seqlen_k - first + 7) / 8;   // may spill into row padding
        const uint4 z = make_uint4(0u, 0u, 0u, 0u);
        for (int t8 = 0; t8 < ntokh; ++t8) {
          uint4* dst = reinterpret_cast<uint4*>(out_base + (int64_t)t8 * p.out_row_stride + first);
          for (int i = st; i < vec_per_row; i += kHalfThreads) dst[i] = z;
        }
      }
      // block scores past the last tile: their keys are invisible (0) or do not exist (-inf);
      // the first such block still sees the last key of the last tile
      if (ok && kPooled) {
        const int first_blk = n_tiles * 32;
        for (int t8 = 0; t8 < ntokh; ++t8) {
          const int bq = (tokh + t8 + cache_len) / kBlockN;
          for (int blk = first_blk + st; blk < p.pooled_len; blk += kHalfThreads) {
            float v = (4 * blk < lc) ? 0.f : -INFINITY;                   // keys 4blk .. 4blk+3
            if (blk > 0 && 4 * blk - 1 < lc)                              // key 4blk - 1
              v = fmaxf(v, (blk == first_blk && n_tiles > 0)
                               ? __bfloat162float(carry[(n_tiles - 1) & 3][t8]) : 0.f);
            if (blk < p.init_blocks || (bq >= blk && bq <= blk + p.local_blocks)) v = INFINITY;
            pool_base[(int64_t)t8 * p.pooled_len + blk] = __float2bfloat16_rn(v);
          }
        }
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem, kTmemCols);
}

int launch_stage1(const void* q, const void* kc, const void* kv, void* out, void* pooled,
                  const int32_t* cu_seqlens_q, const int32_t* cu_seqlens_k,
                  const int32_t* cu_seqlens_v, int64_t total_v, const int32_t* seqused_k,
                  const int32_t* seqused_v, const int32_t* cache_lens, int batch, int64_t total_q, int64_t total_c,
                  int heads_q, int heads_k, int head_dim, int max_seqlen_q, int max_seqlen_k,
                  int64_t out_row_stride, int pooled_len, int cache_len, int local_blocks,
                  int init_blocks, float softmax_scale, int causal, int32_t* status, void* stream,
                  const char* what, const int32_t* leftpad_k = nullptr,
                  const int32_t* block_table = nullptr, int block_table_stride = 0, int page_size = 0) {
  IFV2_REQUIRE(head_dim == kHeadDim, IFV2_ERR_UNSUPPORTED,
               "%s: head_dim %d not supported (only 128, as in the reference build)", what, head_dim);
  IFV2_REQUIRE(heads_k >= 1 && heads_q == heads_k * kGroup, IFV2_ERR_UNSUPPORTED,
               "%s: heads_q (%d) must be 16 x heads_k (%d)", what, heads_q, heads_k);
  IFV2_REQUIRE(batch >= 1 && total_q >= 0 && total_c >= 0 && max_seqlen_q >= 0 && max_seqlen_k >= 0,
               IFV2_ERR_INVALID_ARG, "%s: negative size or batch < 1", what);
  if (total_q == 0 || max_seqlen_q == 0) return IFV2_OK;
  if (max_seqlen_k == 0 && pooled == nullptr) return IFV2_OK;
  IFV2_REQUIRE(softmax_scale > 0.f, IFV2_ERR_INVALID_ARG, "%s: softmax_scale must be > 0", what);
  IFV2_REQUIRE(q && cu_seqlens_q && cu_seqlens_k && status && (kc || total_c == 0) && (out || pooled),
               IFV2_ERR_INVALID_ARG, "%s: null pointer", what);
  if (out != nullptr) {
    IFV2_REQUIRE(out_row_stride >= ((max_seqlen_k + 7) / 8) * 8 && out_row_stride % 8 == 0,
                 IFV2_ERR_INVALID_ARG,
                 "%s: out_row_stride (%lld) must be a multiple of 8 and >= max_seqlen_k rounded up to 8",
                 what, (long long)out_row_stride);
    IFV2_REQUIRE(reinterpret_cast<uintptr_t>(out) % 16 == 0, IFV2_ERR_INVALID_ARG,
                 "%s: out must be 16-byte aligned", what);
  }
  IFV2_REQUIRE(pooled == nullptr ||
                   (pooled_len >= 1 && cache_len >= 0 && local_blocks >= 0 && init_blocks >= 0),
               IFV2_ERR_INVALID_ARG, "%s: bad pooling arguments", what);
  IFV2_REQUIRE(total_q <= INT32_MAX && total_c <= INT32_MAX, IFV2_ERR_TOO_LARGE,
               "%s: more than 2^31-1 rows", what);
  IFV2_REQUIRE(batch <= 65535 && heads_k <= 65535, IFV2_ERR_TOO_LARGE, "%s: batch or heads_k > 65535",
               what);

  // separate row-sum keys are announced by their cu_seqlens; the tensor itself may be empty
  IFV2_REQUIRE(cu_seqlens_v != nullptr || kv == nullptr, IFV2_ERR_INVALID_ARG,
               "%s: row-sum keys need their cu_seqlens", what);
  IFV2_REQUIRE(seqused_v == nullptr || cu_seqlens_v != nullptr, IFV2_ERR_INVALID_ARG,
               "%s: seqused_v needs cu_seqlens_v", what);
  IFV2_REQUIRE(cu_seqlens_v == nullptr || (total_v >= 0 && total_v <= INT32_MAX && (kv || total_v == 0)),
               IFV2_ERR_INVALID_ARG, "%s: bad row-sum keys", what);
  if (block_table != nullptr) {
    IFV2_REQUIRE(page_size >= kKeysPerTile && page_size % kKeysPerTile == 0 && block_table_stride >= 1,
                 IFV2_ERR_INVALID_ARG, "%s: page size must be a positive multiple of 128 compressed keys", what);
    IFV2_REQUIRE(leftpad_k == nullptr, IFV2_ERR_UNSUPPORTED,
                 "%s: a paged cache takes no leftpad_k (as in the reference)", what);
    IFV2_REQUIRE(cu_seqlens_v == nullptr, IFV2_ERR_UNSUPPORTED,
                 "%s: separate row-sum keys are not supported with a paged cache", what);
    IFV2_REQUIRE((int64_t)block_table_stride * page_size >= max_seqlen_k, IFV2_ERR_INVALID_ARG,
                 "%s: the block table covers fewer than max_seqlen_k keys", what);
  }
  IFV2_REQUIRE(leftpad_k == nullptr || cu_seqlens_v == nullptr, IFV2_ERR_UNSUPPORTED,
               "%s: leftpad_k is not supported together with separate row-sum keys", what);
  CUtensorMap map_q, map_kc, map_kv;
  int rc = make_tensor_map_bf16_3d(&map_q, q, kHeadDim, heads_q, total_q, kHeadDim * 2,
                                   (uint64_t)heads_q * kHeadDim * 2, 64, kGroup, kTokPerBox);
  if (rc) return rc;
  // an empty key tensor still needs a valid map: point it at q, no tile is ever fetched
  rc = make_tensor_map_bf16_3d(&map_kc, total_c > 0 ? kc : q, kHeadDim, heads_k,
                               total_c > 0 ? total_c : 1, kHeadDim * 2,
                               (uint64_t)heads_k * kHeadDim * 2, 64, 1, kKeysPerTile);
  if (rc) return rc;
  const bool own_v = kv != nullptr && total_v > 0;
  rc = make_tensor_map_bf16_3d(&map_kv, own_v ? kv : (total_c > 0 ? kc : q), kHeadDim, heads_k,
                               own_v ? total_v : (total_c > 0 ? total_c : 1), kHeadDim * 2,
                               (uint64_t)heads_k * kHeadDim * 2, 64, 1, kKeysPerTile);
  if (rc) return rc;

  Stage1Params p;
  p.out = static_cast<__nv_bfloat16*>(out);
  p.pooled = static_cast<__nv_bfloat16*>(pooled);
  p.cu_q = cu_seqlens_q;
  p.cu_k = cu_seqlens_k;
  p.cu_v = cu_seqlens_v;
  p.seqused_k = seqused_k;
  p.seqused_v = seqused_v;
  p.cache_lens = cache_lens;
  p.leftpad_k = leftpad_k;
  p.block_table = block_table;
  p.bt_stride = block_table_stride;
  p.page_size = page_size > 0 ? page_size : 1;
  p.total_q = total_q;
  p.heads_q = heads_q;
  p.heads_k = heads_k;
  p.max_seqlen_k = max_seqlen_k;
  p.out_row_stride = out_row_stride;
  p.pooled_len = pooled_len;
  p.cache_len = cache_len;
  p.local_blocks = local_blocks;
  p.init_blocks = init_blocks;
  p.scale_log2 = softmax_scale * 1.4426950408889634f;
  p.inv_scale_log2 = 1.f / p.scale_log2;
  p.causal = causal ? 1 : 0;
  p.status = status;

  const size_t smem = sizeof(Smem) + 1024;
  dim3 grid((max_seqlen_q + kTokPerCta - 1) / kTokPerCta, batch, heads_k);
  rc = clear_launch_status(status, stream, what);
  if (rc) return rc;
  cudaError_t e;
  if (pooled != nullptr) {
    e = cudaFuncSetAttribute(stage1_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             (int)smem);
    if (e != cudaSuccess) return set_error((int)e, "%s: %s", what, cudaGetErrorString(e));
    stage1_kernel<true><<<grid, kThreads, smem, (cudaStream_t)stream>>>(map_q, map_kc, map_kv, p);
  } else {
    e = cudaFuncSetAttribute(stage1_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             (int)smem);
    if (e != cudaSuccess) return set_error((int)e, "%s: %s", what, cudaGetErrorString(e));
    stage1_kernel<false><<<grid, kThreads, smem, (cudaStream_t)stream>>>(map_q, map_kc, map_kv, p);
  }
  return check_launch(what);
}

}  // namespace
}  // namespace ifv2

using namespace ifv2;

extern "C" int ifv2_stage1_scores(const void* q, const void* kc, const void* lse_keys, void* out,
                                  const int32_t* cu_seqlens_q, const int32_t* cu_seqlens_k,
                                  const int32_t* cu_seqlens_v, int64_t total_v,
                                  const int32_t* seqused_k, const int32_t* seqused_v, int batch,
                                  int64_t total_q, int64_t total_c, int heads_q, int heads_k, int head_dim,
                                  int max_seqlen_q, int max_seqlen_k,
                                  int64_t out_row_stride, float softmax_scale, int causal,
                                  int32_t* status, void* stream) {
  IFV2_REQUIRE(out != nullptr || total_q == 0 || max_seqlen_k == 0 || max_seqlen_q == 0,
               IFV2_ERR_INVALID_ARG, "stage1_scores: null pointer");
  return launch_stage1(q, kc, lse_keys, out, nullptr, cu_seqlens_q, cu_seqlens_k, cu_seqlens_v,
                       total_v, seqused_k, seqused_v, nullptr, batch, total_q,
                       total_c, heads_q, heads_k, head_dim, max_seqlen_q, max_seqlen_k,
                       out_row_stride, 0, 0, 0, 0, softmax_scale, causal, status, stream,
                       "stage1_scores");
}

extern "C" int ifv2_stage1_block_scores(const void* q, const void* kc, const void* lse_keys,
                                        void* scores_or_null, void* block_scores,
                                        const int32_t* cu_seqlens_q, const int32_t* cu_seqlens_k,
                                        const int32_t* cu_seqlens_v, int64_t total_v,
                                        const int32_t* seqused_k, const int32_t* seqused_v,
                                        const int32_t* cache_lens, int batch, int64_t total_q, int64_t total_c, int heads_q,
                                        int heads_k, int head_dim, int max_seqlen_q,
                                        int max_seqlen_k, int64_t scores_row_stride, int n_blocks,
                                        int cache_len, int local_blocks, int init_blocks,
                                        float softmax_scale, int causal, int32_t* status,
                                        void* stream) {
  IFV2_REQUIRE(block_scores != nullptr || total_q == 0 || max_seqlen_q == 0, IFV2_ERR_INVALID_ARG,
               "stage1_block_scores: null block_scores");
  return launch_stage1(q, kc, lse_keys, scores_or_null, block_scores, cu_seqlens_q, cu_seqlens_k,
                       cu_seqlens_v, total_v, seqused_k, seqused_v, cache_lens,
                       batch, total_q, total_c, heads_q, heads_k, head_dim, max_seqlen_q,
                       max_seqlen_k, scores_row_stride, n_blocks, cache_len, local_blocks,
                       init_blocks, softmax_scale, causal, status, stream, "stage1_block_scores");
}

extern "C" int ifv2_stage1_paged(const void* q, const void* kc, void* scores_or_null,
                                 void* block_scores_or_null, const int32_t* cu_seqlens_q,
                                 const int32_t* cu_seqlens_k, const int32_t* seqused_k,
                                 const int32_t* leftpad_k, const int32_t* block_table,
                                 int block_table_stride, int page_size, const int32_t* cache_lens,
                                 int batch, int64_t total_q, int64_t total_c, int heads_q, int heads_k,
                                 int head_dim, int max_seqlen_q, int max_seqlen_k,
                                 int64_t scores_row_stride, int n_blocks, int cache_len,
                                 int local_blocks, int init_blocks, float softmax_scale, int causal,
                                 int32_t* status, void* stream) {
  IFV2_REQUIRE(scores_or_null != nullptr || block_scores_or_null != nullptr || total_q == 0 ||
                   max_seqlen_q == 0,
               IFV2_ERR_INVALID_ARG, "stage1_paged: no output given");
  return launch_stage1(q, kc, nullptr, scores_or_null, block_scores_or_null, cu_seqlens_q, cu_seqlens_k,
                       nullptr, 0, seqused_k, nullptr, cache_lens, batch, total_q, total_c, heads_q,
                       heads_k, head_dim, max_seqlen_q, max_seqlen_k, scores_row_stride, n_blocks,
                       cache_len, local_blocks, init_blocks, softmax_scale, causal, status, stream,
                       "stage1_paged", leftpad_k, block_table, block_table_stride, page_size);
}
