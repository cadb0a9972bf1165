// Stage-2 backward on tcgen05 tensor cores, without atomics and without an fp32 dQ accumulator
// in HBM.  Three launches:
//   1. dot_do_o      D[row] = sum_c dO[row,c] * O[row,c]                       (HBM-bound)
//   2. dq kernel     one CTA per 128-row query tile (8 tokens x 16 heads), walking the union of
//                    its tokens' selected blocks exactly like the forward:
//                      S = Q.K^T, dP = dO.V^T, dS = exp2(S*c - lse) * (dP - D), dQ += dS.K
//                    dQ stays in TMEM for the whole walk and is written once, as bf16.
//   3. dkv kernel    one CTA per (64-key block, sequence, KV head), walking the token octets
//                    that selected the block (from the transposed bitmask):
//                      S, dP as above, P and dS go to swizzled shared memory, then
//                      dV^T += dO^T.P, dK^T += Q^T.dS with both operands MN-major.
//                    dK / dV of a block are written once; the sum over the 16 query heads of
//                    the group is implicit because those heads are rows of the same tile.
// Recomputing S and dP in both kernels costs 7 tile products instead of 5, but removes the
// scatter of 16x128 fp32 tiles per (token, block) pair that bounds an atomics-based design.
#include "tc05.cuh"

namespace ifv2 {
namespace {

using namespace tc;

constexpr int kTokPerTile = 8;
// Both gradient kernels: warp 0 TMA, warps 1 and 2 MMA issuers, warp 3 owns the TMEM allocation (and
// in the dQ kernel issues a product of its own), warps 4-11 do the softmax work of the even steps
// and 12-19 of the odd ones.  Within a turn a warp
// takes 32 of a block's 64 key columns for the 32 rows of its TMEM lane quadrant (no row reductions
// are needed in the backward, so the column halves are independent).
constexpr int kDkvThreads = 640;
constexpr int kDqThreads = 640;
constexpr int kMaxMaskWords = 128;
constexpr uint32_t kTileHalfBytes = 128 * 128;   // 128 rows x 64 bf16
constexpr uint32_t kKVHalfBytes = 64 * 128;      // 64 keys x 64 bf16
constexpr float kLog2e = 1.4426950408889634f;

struct BwdParams {
  const float* lse;           // (heads_k, total_q * 16)
  float* dvec;                // (heads_k, total_q * 16)   D = rowsum(dO * O)
  __nv_bfloat16* dq;
  __nv_bfloat16* dk;
  __nv_bfloat16* dv;
  const unsigned long long* fwd_mask;   // (heads_k, total_q, fwd_words) or null
  int fwd_words;
  const unsigned long long* bwd_mask;   // (heads_k, k_blocks, bwd_words) or null
  int64_t bwd_words;
  int k_blocks;
  const int32_t* cu_q;
  const int32_t* cu_k;
  int64_t total_q;
  int heads_q, heads_k;
  float scale, scale_log2;
  int causal;
  int32_t* status;
};

// ------------------------------------------------------------------ 1. D = rowsum(dO * O) ----
__global__ void __launch_bounds__(256)
dot_do_o_kernel(const __nv_bfloat16* __restrict__ dout, const __nv_bfloat16* __restrict__ out,
                float* __restrict__ dvec, int64_t total_q, int heads_q) {
  const int lane = threadIdx.x & 31, sub = lane >> 4, l16 = lane & 15;
  const int64_t rows = total_q * heads_q;
  const int64_t warp0 = ((int64_t)blockIdx.x * 256 + threadIdx.x) >> 5;
  const int64_t nwarps = ((int64_t)gridDim.x * 256) >> 5;
  for (int64_t r2 = warp0; r2 * 2 < rows; r2 += nwarps) {
    const int64_t row = r2 * 2 + sub;
    float acc = 0.f;
    if (row < rows) {
      const uint4 a = __ldg(reinterpret_cast<const uint4*>(dout + row * kHeadDim) + l16);
      const uint4 b = __ldg(reinterpret_cast<const uint4*>(out + row * kHeadDim) + l16);
      const __nv_bfloat162* pa = reinterpret_cast<const __nv_bfloat162*>(&a);
      const __nv_bfloat162* pb = reinterpret_cast<const __nv_bfloat162*>(&b);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 x = __bfloat1622float2(pa[j]), y = __bfloat1622float2(pb[j]);
        acc = fmaf(x.x, y.x, acc);
        acc = fmaf(x.y, y.y, acc);
      }
    }
#pragma unroll
    for (int d = 8; d >= 1; d >>= 1) acc += __shfl_xor_sync(0xFFFFFFFFu, acc, d);
    if (l16 == 0 && row < rows) {
      const int64_t tok = row / heads_q;
      const int hq = (int)(row - tok * heads_q);
      dvec[(int64_t)(hq / kGroup) * total_q * kGroup + tok * kGroup + (hq % kGroup)] = acc;
    }
  }
}

// One thread's mask row, read in the order the tile's blocks are walked (highest first): the word
// of the current 64 blocks stays in a register and the word below it is fetched ahead, so that a
// step does not start with a round trip to global memory.
struct MaskRowReader {
  const unsigned long long* row;   // null: every block counts as selected
  int wi;                          // index of the word in `cur`, -1 before the first read
  unsigned long long cur, below;
  __device__ explicit MaskRowReader(const unsigned long long* r) : row(r), wi(-1), cur(0ull), below(0ull) {}
  __device__ bool selected(int blk) {
    if (row == nullptr) return true;
    const int j = blk >> 6;
    if (j != wi) {
      cur = (wi >= 0 && j == wi - 1) ? below : __ldg(row + j);
      wi = j;
      below = j > 0 ? __ldg(row + j - 1) : 0ull;
    }
    return (cur >> (blk & 63)) & 1ull;
  }
};

// Highest-to-lowest walk over the set bits of a tile's union mask.
struct BlockWalk {
  const unsigned long long* words;
  int w;
  unsigned long long cur;
  __device__ BlockWalk(const unsigned long long* u, int nwords) : words(u), w(nwords), cur(0) {}
  __device__ int next() {
    while (cur == 0ull) {
      if (w == 0) return -1;
      cur = words[--w];
    }
    const int b = 63 - __clzll(cur);
    cur &= ~(1ull << b);
    return w * 64 + b;
  }
};

// ------------------------------------------------------------------ 2. dQ kernel -------------
struct DqSmem {
  uint8_t q[2][kTileHalfBytes];
  uint8_t dout[2][kTileHalfBytes];
  uint8_t k[3][2][kKVHalfBytes];      // [stage][d half]; K lives until dS.K of its block is done,
  uint8_t v[2][2][kKVHalfBytes];      // so it needs one more stage than V to be prefetched in time
  unsigned long long umask[kMaxMaskWords];
  // s_full[s] / dp_full[s]: S (dP) of TMEM buffer s is complete; dp_full also releases the V tile of
  // slot s; dq_done[k] releases the K tile of ring slot k and the TMEM buffer of that step and,
  // for the last block, tells the epilogue that dQ is complete.
  // s_empty[s]: the softmax warps have read S of buffer s (dS goes over the dP columns, so the next S
  // for the buffer need not wait for the dQ product that reads dS).
  uint64_t qdo_full, k_full[3], dq_done[3], v_full[2], s_full[2], dp_full[2], ds_ready[2], s_empty[2];
  uint64_t qdo_tmem;   // 8 arrivals: Q and dO have been copied from shared memory into TMEM
  uint32_t tmem_base;
  int n_blocks;
  int abort_flag;
};

// Roles: warp 0 copies; warp 1 issues S = Q K^T, warp 3 (which also owns the TMEM allocation)
// dP = dO V^T, both with the A operand in TMEM, warp 2 dQ += dS K: one issuing warp per product,
// because a warp that shares its scheduler with four softmax warps needs 600-700 clocks to issue
// eight MMAs; warps 4-11 do the softmax work of the even steps and 12-19 of the odd ones (each
// turn has the TMEM buffer of its parity).  A step's P is computed as
// soon as its S is there, while its dP product runs.
__global__ void __launch_bounds__(kDqThreads, 1)
sparse_attn_bwd_dq_kernel(const __grid_constant__ CUtensorMap map_q,
                          const __grid_constant__ CUtensorMap map_do,
                          const __grid_constant__ CUtensorMap map_k,
                          const __grid_constant__ CUtensorMap map_v, const BwdParams p) {
  extern __shared__ uint8_t smem_raw[];
  DqSmem& sm = *reinterpret_cast<DqSmem*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                          ~(uintptr_t)1023);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int b = blockIdx.y, h = blockIdx.z;
  const int q0 = p.cu_q[b], lq = p.cu_q[b + 1] - q0;
  const int k0 = p.cu_k[b], lk = p.cu_k[b + 1] - k0;
  const int tok0 = ((int)gridDim.x - 1 - (int)blockIdx.x) * kTokPerTile;
  if (tok0 >= lq) return;
  if (*reinterpret_cast<volatile int32_t*>(p.status) != 0) return;
  const int ntok = min(kTokPerTile, lq - tok0);
  const int shift = lk - lq;
  const int nblk_k = (lk + kBlockN - 1) / kBlockN;
  const int words =
      (p.fwd_mask != nullptr) ? p.fwd_words : min(kMaxMaskWords, (nblk_k + 63) / 64);
  {
    int last_blk = nblk_k - 1;
    if (p.causal) last_blk = min(last_blk, (tok0 + ntok - 1 + shift) >= 0
                                               ? (tok0 + ntok - 1 + shift) / kBlockN : -1);
    for (int w = threadIdx.x; w < words; w += kDqThreads) {
      unsigned long long u = 0ull;
      if (p.fwd_mask != nullptr) {
        const unsigned long long* row =
            p.fwd_mask + ((int64_t)h * p.total_q + q0 + tok0) * p.fwd_words + w;
        for (int t = 0; t < ntok; ++t) u |= __ldg(row + (int64_t)t * p.fwd_words);
      } else {
        u = ~0ull;
      }
      const int first = w * 64;
      if (last_blk < first) u = 0ull;
      else if (last_blk - first < 63) u &= (2ull << (last_blk - first)) - 1ull;
      sm.umask[w] = u;
    }
  }
  if (threadIdx.x == 0) {
    sm.abort_flag = 0;
    mbar_init(&sm.qdo_full, 1);
    for (int s = 0; s < 3; ++s) {
      mbar_init(&sm.k_full[s], 1);
      mbar_init(&sm.dq_done[s], 1);
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(&sm.v_full[s], 1);
      mbar_init(&sm.s_full[s], 1);
      mbar_init(&sm.dp_full[s], 1);
      mbar_init(&sm.ds_ready[s], 8);         // one arrival per softmax warp of the buffer's turn
      mbar_init(&sm.s_empty[s], 8);
    }
    mbar_init(&sm.qdo_tmem, 8);
    fence_barrier_init();
  }
  if (warp == 3) {
    tmem_alloc(&sm.tmem_base, 512);
    tmem_relinquish();
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    int n = 0;
    for (int w = 0; w < words; ++w) n += __popcll(sm.umask[w]);
    sm.n_blocks = n;
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  // (read through a warp broadcast: it tells the compiler that the value is warp-uniform, so the
  //  MMA issuer's descriptor arithmetic stays in uniform registers instead of being moved there
  //  operand by operand for every MMA)
  const int n_blocks = __shfl_sync(0xFFFFFFFFu, sm.n_blocks, 0);
  const uint32_t tmem = __shfl_sync(0xFFFFFFFFu, sm.tmem_base, 0);
  const uint32_t tmem_dq = tmem + 256;             // [0,128) buffer 0: S | dP, [128,256) buffer 1
  const uint32_t tmem_q = tmem + 384, tmem_do = tmem + 448;   // A operands: 128 rows x 128 d as bf16 pairs
  volatile int* abort_flag = &sm.abort_flag;

  if (warp == 0) {
    if (lane == 0 && n_blocks > 0) {
      mbar_expect_tx(&sm.qdo_full, 4 * kTileHalfBytes);
      tma_load_3d(sm.q[0], &map_q, &sm.qdo_full, 0, h * kGroup, q0 + tok0);
      tma_load_3d(sm.q[1], &map_q, &sm.qdo_full, 64, h * kGroup, q0 + tok0);
      tma_load_3d(sm.dout[0], &map_do, &sm.qdo_full, 0, h * kGroup, q0 + tok0);
      tma_load_3d(sm.dout[1], &map_do, &sm.qdo_full, 64, h * kGroup, q0 + tok0);
      BlockWalk walk(sm.umask, words);
      int issued = 0;
      for (int i = 0; i < n_blocks; ++i) {
        const int blk = walk.next();
        const int s = i & 1, sk = i % 3, key = k0 + blk * kBlockN;
        const uint32_t par = (uint32_t)((i >> 1) & 1), park = (uint32_t)((i / 3) & 1);
        if (i >= 3 && !mbar_wait(&sm.dq_done[sk], park ^ 1u, abort_flag, p.status, 71)) break;
        mbar_expect_tx(&sm.k_full[sk], 2 * kKVHalfBytes);
        tma_load_3d(sm.k[sk][0], &map_k, &sm.k_full[sk], 0, h, key);
        tma_load_3d(sm.k[sk][1], &map_k, &sm.k_full[sk], 64, h, key);
        if (i >= 2 && !mbar_wait(&sm.dp_full[s], par ^ 1u, abort_flag, p.status, 72)) {
          issued = i + 1;
          break;
        }
        mbar_expect_tx(&sm.v_full[s], 2 * kKVHalfBytes);
        tma_load_3d(sm.v[s][0], &map_v, &sm.v_full[s], 0, h, key);
        tma_load_3d(sm.v[s][1], &map_v, &sm.v_full[s], 64, h, key);
        issued = i + 1;
      }
      if (*abort_flag) {
        mbar_wait_drain(&sm.qdo_full, 0);
        for (int j = max(0, issued - 2); j < issued; ++j) {
          mbar_wait_drain(&sm.k_full[j % 3], (uint32_t)((j / 3) & 1));
          mbar_wait_drain(&sm.v_full[j & 1], (uint32_t)((j >> 1) & 1));
        }
      }
    }
  } else if (warp == 1) {
    // S = Q K^T.  All 32 lanes run the same issue code (descriptors stay in uniform registers);
    // `leader` enables the MMA / commit instructions in one lane only.
    if (n_blocks > 0) {
      const uint32_t leader = (lane == 0) ? 1u : 0u;
      constexpr uint32_t idesc_s = umma_idesc_bf16(128, 64, false);
      const uint64_t k_desc0 = umma_desc_sw128(smem_u32(sm.k[0][0]), 16, 1024);
      constexpr uint32_t kStage = (2 * kKVHalfBytes) >> 4;     // descriptor address units per ring stage
      // Q and dO are A operands read from TMEM: the Q.K^T and dO.V^T products then fetch only
      // their 2 KB key tiles from shared memory per step instead of 6 KB
      bool ok = __all_sync(0xFFFFFFFFu, mbar_wait(&sm.qdo_tmem, 0, abort_flag, p.status, 73));
      tc_fence_after();
      int sk = 0, kround = 0;                       // j % 3, j / 3
      for (int j = 0; j < n_blocks && ok; ++j) {
        const int s = j & 1;
        const uint32_t par = (uint32_t)((j >> 1) & 1);
        bool w = mbar_wait(&sm.k_full[sk], (uint32_t)(kround & 1), abort_flag, p.status, 74);
        // the S columns were last read by the softmax warps of step j - 2
        if (w && j >= 2) w = mbar_wait(&sm.s_empty[s], par ^ 1u, abort_flag, p.status, 80);
        if (!__all_sync(0xFFFFFFFFu, w)) break;
        tc_fence_after();
        const uint64_t k_desc = k_desc0 + (uint32_t)sk * kStage;
#pragma unroll
        for (int kk = 0; kk < 8; ++kk) {
          const uint32_t boff = ((kk >> 2) * kKVHalfBytes + (kk & 3) * 32) >> 4;
          umma_ts_pred(tmem + s * 128, tmem_q + kk * 8, k_desc + boff, idesc_s, kk > 0, leader);
        }
        umma_commit_pred(&sm.s_full[s], leader);
        if (++sk == 3) { sk = 0; ++kround; }
      }
    }
  } else if (warp == 3) {
    // dP = dO V^T, on a warp of its own: one warp issuing S and dP was busy four fifths of a step
    if (n_blocks > 0) {
      const uint32_t leader = (lane == 0) ? 1u : 0u;
      constexpr uint32_t idesc_s = umma_idesc_bf16(128, 64, false);
      const uint64_t v_desc0 = umma_desc_sw128(smem_u32(sm.v[0][0]), 16, 1024);
      constexpr uint32_t kStage = (2 * kKVHalfBytes) >> 4;
      bool ok = __all_sync(0xFFFFFFFFu, mbar_wait(&sm.qdo_tmem, 0, abort_flag, p.status, 67));
      tc_fence_after();
      int sk2 = 1, kround2 = -1;                    // (j - 2) % 3, (j - 2) / 3 (used from j = 2 on)
      for (int j = 0; j < n_blocks && ok; ++j) {
        const int s = j & 1;
        const uint32_t par = (uint32_t)((j >> 1) & 1);
        // the dP columns hold dS of step j - 2 until its dQ product is complete
        bool w = mbar_wait(&sm.v_full[s], par, abort_flag, p.status, 75);
        if (w && j >= 2) w = mbar_wait(&sm.dq_done[sk2], (uint32_t)(kround2 & 1), abort_flag, p.status, 68);
        if (!__all_sync(0xFFFFFFFFu, w)) break;
        tc_fence_after();
        const uint64_t v_desc = v_desc0 + (uint32_t)s * kStage;
#pragma unroll
        for (int kk = 0; kk < 8; ++kk) {
          const uint32_t boff = ((kk >> 2) * kKVHalfBytes + (kk & 3) * 32) >> 4;
          umma_ts_pred(tmem + s * 128 + 64, tmem_do + kk * 8, v_desc + boff, idesc_s, kk > 0, leader);
        }
        umma_commit_pred(&sm.dp_full[s], leader);
        if (++sk2 == 3) { sk2 = 0; ++kround2; }
      }
    }
  } else if (warp == 2) {
    // dQ += dS K (dS as bf16 pairs in the step's TMEM buffer, K read along the keys)
    if (n_blocks > 0) {
      const uint32_t leader = (lane == 0) ? 1u : 0u;
      constexpr uint32_t idesc_dq = umma_idesc_bf16(128, 128, true);
      const uint64_t k_desc0_mn = umma_desc_sw128(smem_u32(sm.k[0][0]), kKVHalfBytes, 1024);
      constexpr uint32_t kStage = (2 * kKVHalfBytes) >> 4;
      int sk = 0, kround = 0;
      for (int i = 0; i < n_blocks; ++i) {
        const int s = i & 1;
        bool w = mbar_wait(&sm.k_full[sk], (uint32_t)(kround & 1), abort_flag, p.status, 70);
        if (w) w = mbar_wait(&sm.ds_ready[s], (uint32_t)((i >> 1) & 1), abort_flag, p.status, 76);
        if (!__all_sync(0xFFFFFFFFu, w)) break;
        tc_fence_after();
        const uint64_t k_mn = k_desc0_mn + (uint32_t)sk * kStage;
#pragma unroll
        for (int kk = 0; kk < 4; ++kk)      // dS of keys 0-31 sits at columns [64, 80), of keys 32-63 at [96, 112)
          umma_ts_pred(tmem_dq, tmem + s * 128 + 64 + (kk >> 1) * 32 + (kk & 1) * 8, k_mn + ((kk * 2048) >> 4), idesc_dq,
                       (i > 0) || (kk > 0), leader);
        umma_commit_pred(&sm.dq_done[sk], leader);
        if (++sk == 3) { sk = 0; ++kround; }
      }
    }
  } else if (warp >= 4) {
    const int quad = warp & 3;
    const int turn = (warp - 4) >> 3;                // this warp takes the steps with i & 1 == turn
    const int grp = ((warp - 4) & 7) >> 2;           // which 32 key columns
    const int r = quad * 32 + lane;
    const int tl = r >> 4, g = r & 15;
    const int tok = tok0 + tl;
    const bool valid = tl < ntok;
    const uint32_t lane_off = (uint32_t)(quad * 32) << 16;
    const unsigned long long* mrow =
        (p.fwd_mask != nullptr && valid)
            ? p.fwd_mask + ((int64_t)h * p.total_q + q0 + tok) * p.fwd_words : nullptr;
    const int row_limit = valid ? min(lk, p.causal ? tok + shift + 1 : lk) : 0;
    const int64_t stat_idx = (int64_t)h * p.total_q * kGroup + (int64_t)(q0 + tok) * kGroup + g;
    const float neg_lse = valid ? -p.lse[stat_idx] * kLog2e : -INFINITY;   // +inf lse -> P = 0
    const float dsum = valid ? p.dvec[stat_idx] : 0.f;
    bool ok = true;
    if (n_blocks > 0 && turn == 0) {
      // the warps of the first turn move Q and dO into TMEM: column group 0 this thread's Q row,
      // group 1 its dO row, from the swizzled tiles
      // (row r of a d half: 16-byte chunk c sits at chunk c ^ (r & 7); TMEM column j = d 2j, 2j+1)
      ok = __all_sync(0xFFFFFFFFu, mbar_wait(&sm.qdo_full, 0, abort_flag, p.status, 79));
      if (ok) {
        const uint8_t* tile = (grp == 0) ? sm.q[0] : sm.dout[0];
        const uint32_t dst = ((grp == 0) ? tmem_q : tmem_do) + lane_off;
#pragma unroll
        for (int hh = 0; hh < 2; ++hh) {
          uint32_t regs[32];
          const uint8_t* rowp = tile + hh * kTileHalfBytes + r * 128;
#pragma unroll
          for (int c = 0; c < 8; ++c) {
            const uint4 w = *reinterpret_cast<const uint4*>(rowp + ((c ^ (r & 7)) << 4));
            regs[4 * c] = w.x; regs[4 * c + 1] = w.y; regs[4 * c + 2] = w.z; regs[4 * c + 3] = w.w;
          }
          tmem_st32(dst + hh * 32, regs);
        }
        tmem_wait_st();
        tc_fence_before();
        mbar_arrive_warp(&sm.qdo_tmem);
      }
    }
    BlockWalk walk(sm.umask, words);
    MaskRowReader mask_reader(mrow);
    if (turn == 1 && n_blocks > 0) walk.next();
    for (int i = turn; i < n_blocks && ok; i += 2) {
      const int blk = walk.next();
      walk.next();                                   // the other turn's block
      const int s = i & 1;
      const uint32_t par = (uint32_t)((i >> 1) & 1);
      const bool selected = valid && mask_reader.selected(blk);
      const int lim = (selected ? min(max(row_limit - blk * kBlockN, 0), kBlockN) : 0) - grp * 32;
      // ---- P = exp2(S * scale - lse): needs S only, runs while the dP product does
      ok = __all_sync(0xFFFFFFFFu, mbar_wait(&sm.s_full[s], par, abort_flag, p.status, 77));
      if (!ok) break;
      tc_fence_after();
      uint32_t x[32];
      tmem_ld32(tmem + lane_off + s * 128 + grp * 32, x);
      tmem_wait_ld_dep(x);
      tc_fence_before();
      mbar_arrive_warp(&sm.s_empty[s]);
      {
        const uint64_t c2 = pack_f32x2(p.scale_log2, p.scale_log2), n2 = pack_f32x2(neg_lse, neg_lse);
#pragma unroll
        for (int c = 0; c < 32; c += 2) {
          float y0, y1;
          unpack_f32x2(fma_f32x2(pack_f32x2(x[c], x[c + 1]), c2, n2), y0, y1);
          x[c] = __float_as_uint(c < lim ? exp2f(y0) : 0.f);
          x[c + 1] = __float_as_uint(c + 1 < lim ? exp2f(y1) : 0.f);
        }
      }
      // ---- dS = P * (dP - D), written over the first half of this thread's dP columns as bf16 pairs
      ok = __all_sync(0xFFFFFFFFu, mbar_wait(&sm.dp_full[s], par, abort_flag, p.status, 69));
      if (!ok) break;
      tc_fence_after();
      uint32_t packed[16];
      {
        uint32_t dpv[32];
        tmem_ld32(tmem + lane_off + s * 128 + 64 + grp * 32, dpv);
        tmem_wait_ld_dep(dpv);
        const uint64_t md2 = pack_f32x2(-dsum, -dsum);
#pragma unroll
        for (int c = 0; c < 32; c += 2) {
          float d0, d1;
          unpack_f32x2(mul_f32x2(pack_f32x2(x[c], x[c + 1]), add_f32x2(pack_f32x2(dpv[c], dpv[c + 1]), md2)), d0, d1);
          packed[c >> 1] = pack_bf16(d0, d1);
        }
      }
      // (each column group writes inside the dP columns it read itself: no warp's dS can land on
      //  values that another warp has yet to load)
      tmem_st16(tmem + lane_off + s * 128 + 64 + grp * 32, packed);
      tmem_wait_st();
      tc_fence_before();
      mbar_arrive_warp(&sm.ds_ready[s]);
    }
    // the warps of the first turn write the tile's dQ
    if (turn != 0) ok = false;
    if (ok && n_blocks > 0) {
      // the last block's product: S / dP of that block is complete, hence every dQ product up to
      // block n-3 is too, so this barrier is at most one phase behind and the parity is unambiguous
      ok = __all_sync(0xFFFFFFFFu, mbar_wait(&sm.dq_done[(n_blocks - 1) % 3],
                                             (uint32_t)(((n_blocks - 1) / 3) & 1), abort_flag, p.status, 78));
      tc_fence_after();
    }
    if (ok) {
      __nv_bfloat16* orow = p.dq + ((int64_t)(q0 + tok) * p.heads_q + h * kGroup + g) * kHeadDim;
#pragma unroll 1
      for (int c = grp * 64; c < grp * 64 + 64; c += 32) {
        uint32_t o[32];
        if (n_blocks > 0) {
          tmem_ld32(tmem_dq + lane_off + c, o);
          tmem_wait_ld();
        } else {
#pragma unroll
          for (int j = 0; j < 32; ++j) o[j] = 0u;
        }
        if (valid) {
          uint4* dst = reinterpret_cast<uint4*>(orow + c);
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            uint4 v4;
            v4.x = pack_bf16(__uint_as_float(o[8 * j + 0]) * p.scale, __uint_as_float(o[8 * j + 1]) * p.scale);
            v4.y = pack_bf16(__uint_as_float(o[8 * j + 2]) * p.scale, __uint_as_float(o[8 * j + 3]) * p.scale);
            v4.z = pack_bf16(__uint_as_float(o[8 * j + 4]) * p.scale, __uint_as_float(o[8 * j + 5]) * p.scale);
            v4.w = pack_bf16(__uint_as_float(o[8 * j + 6]) * p.scale, __uint_as_float(o[8 * j + 7]) * p.scale);
            dst[j] = v4;
          }
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 3) tmem_dealloc(tmem, 512);
}

// ------------------------------------------------------------------ 3. dK / dV kernel --------
struct DkvSmem {
  uint8_t k[2][kKVHalfBytes];          // resident K block, [d half]
  uint8_t v[2][kKVHalfBytes];
  uint8_t q[3][2][kTileHalfBytes];     // [ring slot][d half]: three Q tiles in flight,
  uint8_t dout[2][2][kTileHalfBytes];  // two dO tiles
  uint8_t pmat[kTileHalfBytes];        // P  (128 rows x 64 keys bf16, 128-byte swizzle)
  uint8_t dsmat[kTileHalfBytes];       // dS
  // q_full[s]: the Q tile of a step and its record (step_m, step_bits) are in slot s, or, once
  //   total_steps is set, there is no such step;  do_full[s]: the dO tile;
  // s_full / dp_full[b]: S (dP) of TMEM buffer b is complete;  sdp_empty[b]: both were read;
  // p_ready / ds_ready: the softmax warps wrote P (dS);
  // do_free[s] (two arrivals: after dP and after dV of a step): dO slot s may be refilled and P
  //   rewritten;  dk_done[s]: the dK product is complete -> dS may be rewritten, Q slot s refilled,
  //   and after the last step the accumulators are final
  uint64_t kv_full, q_full[3], do_full[2], s_full[2], dp_full[2], sdp_empty[2], p_ready, ds_ready,
      do_free[2], dk_done[3];
  int step_m[3];                       // octet index of the step in Q slot s
  uint32_t step_bits[3];               // which of its 8 tokens selected the block
  int total_steps;                     // INT_MAX until the copy warp has reached the end of its walk
  uint32_t tmem_base;
  int abort_flag;
};

// Walk over the token octets [8m, 8m+8) of a sequence in which at least one token selected the
// key block (bits of the transposed mask row, indexed by GLOBAL token), lowest octet first.
// A whole warp walks together: lane l caches words wbase + l and wbase + 32 + l of the row, so a
// step costs shuffles instead of a round trip to global memory, runs of empty words are skipped
// with one ballot, and the next 32 words are fetched while the cached ones are in use.
// Every lane must call next() (the calls are warp-collective) and every lane gets the same answer.
struct OctetWalk {
  const unsigned long long* row;   // null = dense
  int64_t words, wbase;
  unsigned long long cur, nxt;
  int q0, lq, m, m_end, lane;
  __device__ unsigned long long fetch(int64_t w) const {
    return (row != nullptr && w < words) ? __ldg(row + w) : 0ull;
  }
  __device__ OctetWalk(const unsigned long long* r, int64_t w, int q0_, int lq_, int m_lo, int lane_)
      : row(r), words(w), q0(q0_), lq(lq_), m(m_lo), m_end((lq_ + 7) / 8), lane(lane_) {
    wbase = ((int64_t)q0 + 8 * (int64_t)m_lo) >> 6;
    cur = fetch(wbase + lane);
    nxt = fetch(wbase + 32 + lane);
  }
  __device__ unsigned long long word(int64_t w) const {   // wbase <= w < wbase + 64
    const int off = (int)(w - wbase);
    const unsigned long long a = __shfl_sync(0xFFFFFFFFu, cur, off & 31);
    const unsigned long long b = __shfl_sync(0xFFFFFFFFu, nxt, off & 31);
    return off < 32 ? a : b;
  }
  // returns the octet index and the selection bits of its 8 tokens, or -1 when exhausted
  __device__ int next(uint32_t& bits) {
    while (m < m_end) {
      const int ntok = min(8, lq - 8 * m);
      const uint32_t vmask = (1u << ntok) - 1u;
      if (row == nullptr) {
        bits = vmask;
        return m++;
      }
      const int64_t t = (int64_t)q0 + 8 * (int64_t)m;
      const int64_t w = t >> 6;
      const int sh = (int)(t & 63);
      while (w >= wbase + 32) {
        cur = nxt;
        wbase += 32;
        nxt = fetch(wbase + 32 + lane);
      }
      const unsigned long long here = word(w) >> sh;
      unsigned long long lo = here;
      if (sh > 56) lo |= word(w + 1) << (64 - sh);
      bits = (uint32_t)lo & vmask;
      if (bits) return m++;
      if (here != 0ull) {          // later tokens of this word selected the block
        ++m;
        continue;
      }
      // nothing left in word w: go to the first cached word after it that has a bit
      const int off = (int)(w - wbase);
      const uint32_t ne_cur = __ballot_sync(0xFFFFFFFFu, cur != 0ull);
      const uint32_t ne_nxt = __ballot_sync(0xFFFFFFFFu, nxt != 0ull);
      const uint32_t later = off < 31 ? (ne_cur & (0xFFFFFFFFu << (off + 1))) : 0u;
      int64_t wn;
      if (later) wn = wbase + __ffs(later) - 1;
      else if (ne_nxt) wn = wbase + 32 + __ffs(ne_nxt) - 1;
      else wn = wbase + 64;
      // the first octet with a token in word wn (it may begin in the word before, which is empty)
      const int64_t mn = (wn * 64 - (int64_t)q0) >> 3;
      m = (int)max((int64_t)m + 1, min(mn, (int64_t)m_end));
    }
    return -1;
  }
};

// One step = one token octet that selected the block: S = Q K^T and dP = dO V^T into TMEM, the
// softmax warps turn S into P = exp2(S * scale - lse) and dP into dS = P * (dP - D), both stored
// to shared memory as bf16, then dV^T += dO^T P and dK^T += Q^T dS.
// Roles: the copy warp is the only one that walks the mask row; it leaves each step's octet index
// and selection bits beside the Q tile (and the step count at the end of the walk), so the other
// warps learn them from the tile's barrier.  Two warps issue the products, one S and dP, the other
// dV and dK: each waits, issues and commits on its own, so neither one's barrier round trips hold
// up the other's instructions, and the S / dP warp runs up to two steps ahead (two TMEM buffers).
// Q has three ring slots and dO two.
__global__ void __launch_bounds__(kDkvThreads, 1)
sparse_attn_bwd_dkv_kernel(const __grid_constant__ CUtensorMap map_q,
                           const __grid_constant__ CUtensorMap map_do,
                           const __grid_constant__ CUtensorMap map_k,
                           const __grid_constant__ CUtensorMap map_v, const BwdParams p) {
  extern __shared__ uint8_t smem_raw[];
  DkvSmem& sm = *reinterpret_cast<DkvSmem*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                            ~(uintptr_t)1023);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // block index slowest: the blocks every token selects (block 0 of each sequence) start first
  const int b = blockIdx.x, h = blockIdx.y, n = blockIdx.z;
  const int q0 = p.cu_q[b], lq = p.cu_q[b + 1] - q0;
  const int k0 = p.cu_k[b], lk = p.cu_k[b + 1] - k0;
  if (n * kBlockN >= lk) return;
  if (*reinterpret_cast<volatile int32_t*>(p.status) != 0) return;
  const int shift = lk - lq;
  const int nkeys = min(kBlockN, lk - n * kBlockN);
  // first token that can see key 64n (causal), as an octet index
  const int m_lo = p.causal ? max(0, n * kBlockN - shift) / kTokPerTile : 0;
  const unsigned long long* mask_row =
      (p.bwd_mask != nullptr && n < p.k_blocks)
          ? p.bwd_mask + ((int64_t)h * p.k_blocks + n) * p.bwd_words : nullptr;
  const bool never_selected = (p.bwd_mask != nullptr && n >= p.k_blocks);

  if (threadIdx.x == 0) {
    sm.abort_flag = 0;
    sm.total_steps = never_selected ? 0 : INT_MAX;
    mbar_init(&sm.kv_full, 1);
    for (int s = 0; s < 3; ++s) {
      mbar_init(&sm.q_full[s], 1);
      mbar_init(&sm.dk_done[s], 1);
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(&sm.do_full[s], 1);
      mbar_init(&sm.do_free[s], 2);
      mbar_init(&sm.s_full[s], 1);
      mbar_init(&sm.dp_full[s], 1);
      mbar_init(&sm.sdp_empty[s], 8);
    }
    mbar_init(&sm.p_ready, 8);
    mbar_init(&sm.ds_ready, 8);
    fence_barrier_init();
  }
  if (warp == 3) {
    tmem_alloc(&sm.tmem_base, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = __shfl_sync(0xFFFFFFFFu, sm.tmem_base, 0);   // warp-uniform for the compiler
  const uint32_t tmem_dv = tmem + 256, tmem_dk = tmem + 320;   // [128 d lanes x 64 key columns]
  volatile int* abort_flag = &sm.abort_flag;
  volatile int* total_steps = &sm.total_steps;

  // Step i uses Q slot i % 3, dO slot i & 1, TMEM buffer i & 1.
  if (warp == 0) {
    // the whole warp walks the octet list; lane 0 waits for ring slots and issues the copies
    if (!never_selected) {
      if (lane == 0) {
        mbar_expect_tx(&sm.kv_full, 4 * kKVHalfBytes);
        tma_load_3d(sm.k[0], &map_k, &sm.kv_full, 0, h, k0 + n * kBlockN);
        tma_load_3d(sm.k[1], &map_k, &sm.kv_full, 64, h, k0 + n * kBlockN);
        tma_load_3d(sm.v[0], &map_v, &sm.kv_full, 0, h, k0 + n * kBlockN);
        tma_load_3d(sm.v[1], &map_v, &sm.kv_full, 64, h, k0 + n * kBlockN);
      }
      OctetWalk walk(mask_row, p.bwd_words, q0, lq, m_lo, lane);
      uint32_t bits;
      int issued_q = 0, issued_do = 0;
      int qs = 0, qround = 0;                      // i % 3, i / 3
      for (int i = 0;; ++i) {
        const int m = walk.next(bits);
        const int ds = i & 1;
        const int tok = q0 + m * kTokPerTile;
        bool ok = true;
        if (lane == 0) {
          if (i >= 3) ok = mbar_wait(&sm.dk_done[qs], (uint32_t)((qround & 1) ^ 1), abort_flag, p.status, 81);
          if (ok && m < 0) {
            // end of the walk: the barriers of the next two steps (one for each softmax turn)
            // complete without a tile, and the count says why
            *total_steps = i;
            mbar_arrive(&sm.q_full[qs]);
            const int qs1 = (i + 1) % 3;
            if (i + 1 >= 3) ok = mbar_wait(&sm.dk_done[qs1], (uint32_t)((((i + 1) / 3) & 1) ^ 1), abort_flag, p.status, 97);
            if (ok) mbar_arrive(&sm.q_full[qs1]);
          } else if (ok) {
            sm.step_m[qs] = m;
            sm.step_bits[qs] = bits;
            mbar_expect_tx(&sm.q_full[qs], 2 * kTileHalfBytes);
            tma_load_3d(sm.q[qs][0], &map_q, &sm.q_full[qs], 0, h * kGroup, tok);
            tma_load_3d(sm.q[qs][1], &map_q, &sm.q_full[qs], 64, h * kGroup, tok);
            issued_q = i + 1;
            if (i >= 2) ok = mbar_wait(&sm.do_free[ds], (uint32_t)(((i >> 1) & 1) ^ 1), abort_flag, p.status, 89);
            if (ok) {
              mbar_expect_tx(&sm.do_full[ds], 2 * kTileHalfBytes);
              tma_load_3d(sm.dout[ds][0], &map_do, &sm.do_full[ds], 0, h * kGroup, tok);
              tma_load_3d(sm.dout[ds][1], &map_do, &sm.do_full[ds], 64, h * kGroup, tok);
              issued_do = i + 1;
            }
          }
        }
        if (m < 0 || !__shfl_sync(0xFFFFFFFFu, ok, 0)) break;
        if (++qs == 3) { qs = 0; ++qround; }
      }
      if (lane == 0 && *abort_flag) {
        mbar_wait_drain(&sm.kv_full, 0);
        for (int j = max(0, issued_q - 3); j < issued_q; ++j)
          mbar_wait_drain(&sm.q_full[j % 3], (uint32_t)((j / 3) & 1));
        for (int j = max(0, issued_do - 2); j < issued_do; ++j)
          mbar_wait_drain(&sm.do_full[j & 1], (uint32_t)((j >> 1) & 1));
      }
    }
  } else if (warp == 1) {
    // S and dP.  All 32 lanes run the same issue code (descriptors stay in uniform registers);
    // `leader` enables the MMA / commit instructions in one lane only.
    if (!never_selected) {
      const uint32_t leader = (lane == 0) ? 1u : 0u;
      constexpr uint32_t idesc_s = umma_idesc_bf16(128, 64, false);             // K-major x K-major
      const uint64_t k_desc = umma_desc_sw128(smem_u32(sm.k[0]), 16, 1024);
      const uint64_t v_desc = umma_desc_sw128(smem_u32(sm.v[0]), 16, 1024);
      // ring slot s = slot 0 + s * kRing (plain arithmetic keeps the descriptors in registers)
      const uint64_t q_desc0 = umma_desc_sw128(smem_u32(sm.q[0][0]), 16, 1024);
      const uint64_t do_desc0 = umma_desc_sw128(smem_u32(sm.dout[0][0]), 16, 1024);
      constexpr uint32_t kRing = (2 * kTileHalfBytes) >> 4;
      bool ok = __all_sync(0xFFFFFFFFu, mbar_wait(&sm.kv_full, 0, abort_flag, p.status, 82));
      // (issuing S(j + 1) ahead of dP(j), so that the exponentials of a step would not wait for its
      // dO tile, measured 12 % slower: dS, dK and with them the Q slots then come later)
      int qs = 0, qround = 0;
      for (int j = 0; ok; ++j) {
        const int bf = j & 1;
        const uint32_t par = (uint32_t)((j >> 1) & 1);
        bool w = mbar_wait(&sm.q_full[qs], (uint32_t)(qround & 1), abort_flag, p.status, 83);
        if (!__all_sync(0xFFFFFFFFu, w)) break;
        if (j >= *total_steps) break;
        if (j >= 2) w = mbar_wait(&sm.sdp_empty[bf], par ^ 1u, abort_flag, p.status, 84);
        if (!__all_sync(0xFFFFFFFFu, w)) break;
        tc_fence_after();
#pragma unroll
        for (int kk = 0; kk < 8; ++kk) {
          const uint32_t aoff = ((kk >> 2) * kTileHalfBytes + (kk & 3) * 32) >> 4;
          const uint32_t boff = ((kk >> 2) * kKVHalfBytes + (kk & 3) * 32) >> 4;
          umma_ss_pred(tmem + bf * 128, q_desc0 + qs * kRing + aoff, k_desc + boff, idesc_s, kk > 0, leader);
        }
        umma_commit_pred(&sm.s_full[bf], leader);
        if (!__all_sync(0xFFFFFFFFu, mbar_wait(&sm.do_full[bf], par, abort_flag, p.status, 90))) break;
        tc_fence_after();
#pragma unroll
        for (int kk = 0; kk < 8; ++kk) {
          const uint32_t aoff = ((kk >> 2) * kTileHalfBytes + (kk & 3) * 32) >> 4;
          const uint32_t boff = ((kk >> 2) * kKVHalfBytes + (kk & 3) * 32) >> 4;
          umma_ss_pred(tmem + bf * 128 + 64, do_desc0 + bf * kRing + aoff, v_desc + boff, idesc_s, kk > 0, leader);
        }
        umma_commit_pred(&sm.dp_full[bf], leader);
        umma_commit_pred(&sm.do_free[bf], leader);       // first of the two arrivals that release the dO slot
        if (++qs == 3) { qs = 0; ++qround; }
      }
    }
  } else if (warp == 2) {
    // dV^T (128 d x 64 keys) += dO^T . P ; dK^T += Q^T . dS ; K extent = the 128 tile rows
    if (!never_selected) {
      const uint32_t leader = (lane == 0) ? 1u : 0u;
      constexpr uint32_t idesc_t = umma_idesc_bf16(128, 64, true, true);        // MN-major x MN-major
      const uint64_t p_desc = umma_desc_sw128(smem_u32(sm.pmat), 16, 1024);
      const uint64_t ds_desc = umma_desc_sw128(smem_u32(sm.dsmat), 16, 1024);
      const uint64_t q_mn0 = umma_desc_sw128(smem_u32(sm.q[0][0]), kTileHalfBytes, 1024);
      const uint64_t do_mn0 = umma_desc_sw128(smem_u32(sm.dout[0][0]), kTileHalfBytes, 1024);
      constexpr uint32_t kRing = (2 * kTileHalfBytes) >> 4;
      int qs = 0, qround = 0;
      for (int i = 0;; ++i) {
        const int ds = i & 1;
        if (!__all_sync(0xFFFFFFFFu, mbar_wait(&sm.q_full[qs], (uint32_t)(qround & 1), abort_flag, p.status, 94)))
          break;
        if (i >= *total_steps) break;
        // P of step i follows S of step i, which followed the dO tile's arrival only in program
        // order of the other warp: wait for the tile here too
        bool w = mbar_wait(&sm.do_full[ds], (uint32_t)((i >> 1) & 1), abort_flag, p.status, 95);
        if (w) w = mbar_wait(&sm.p_ready, (uint32_t)(i & 1), abort_flag, p.status, 85);
        if (!__all_sync(0xFFFFFFFFu, w)) break;
        tc_fence_after();
#pragma unroll
        for (int kk = 0; kk < 8; ++kk)
          umma_ss_pred(tmem_dv, do_mn0 + ds * kRing + ((kk * 2048) >> 4), p_desc + ((kk * 2048) >> 4), idesc_t,
                       (i > 0) || (kk > 0), leader);
        umma_commit_pred(&sm.do_free[ds], leader);       // second arrival: dO slot and P are free
        if (!__all_sync(0xFFFFFFFFu, mbar_wait(&sm.ds_ready, (uint32_t)(i & 1), abort_flag, p.status, 91))) break;
        tc_fence_after();
#pragma unroll
        for (int kk = 0; kk < 8; ++kk)
          umma_ss_pred(tmem_dk, q_mn0 + qs * kRing + ((kk * 2048) >> 4), ds_desc + ((kk * 2048) >> 4), idesc_t,
                       (i > 0) || (kk > 0), leader);
        umma_commit_pred(&sm.dk_done[qs], leader);
        if (++qs == 3) { qs = 0; ++qround; }
      }
    }
  } else if (warp >= 4) {
    // One step of softmax work (two TMEM loads, 32 exponentials per thread, two rounds of shared-
    // memory stores + proxy fence + barrier, the row statistics from global memory) takes longer
    // than the four products of a step, so two groups of eight warps take the steps in turn.
    const int quad = warp & 3;
    const int turn = (warp - 4) >> 3;                // this warp takes the steps with i & 1 == turn
    const int grp = ((warp - 4) & 7) >> 2;           // which 32 key columns
    const int r = quad * 32 + lane;
    const int tl = r >> 4, g = r & 15;
    const uint32_t lane_off = (uint32_t)(quad * 32) << 16;
    bool ok = true;
    int steps = 0;
    // row r of a 128-byte-swizzled tile: 16-byte chunk c sits at chunk (c ^ (r & 7))
    uint8_t* prow = sm.pmat + r * 128;
    uint8_t* drow = sm.dsmat + r * 128;
    if (!never_selected) {
      for (int i = turn;; i += 2) {
        const int qs = i % 3, qround = i / 3;
        const int pqs = (i + 2) % 3, pround = (i - 1) / 3;         // of step i - 1 (used for i >= 1)
        // the step's record arrives with its Q tile, well before its S
        ok = __all_sync(0xFFFFFFFFu, mbar_wait(&sm.q_full[qs], (uint32_t)(qround & 1), abort_flag, p.status, 96));
        if (!ok) break;
        steps = *total_steps;
        if (i >= steps) break;
        const int m = sm.step_m[qs];
        const uint32_t bits = sm.step_bits[qs];
        const int bf = i & 1;
        const uint32_t par = (uint32_t)((i >> 1) & 1);
        const int tok = m * kTokPerTile + tl;                     // local token of this row
        const bool selected = (bits >> tl) & 1u;
        const int64_t stat_idx = (int64_t)h * p.total_q * kGroup + (int64_t)(q0 + tok) * kGroup + g;
        const float neg_lse = selected ? -__ldg(p.lse + stat_idx) * kLog2e : -INFINITY;
        const float dsum = selected ? __ldg(p.dvec + stat_idx) : 0.f;
        // keys of this block the row may see
        const int row_limit = selected ? min(lk, p.causal ? tok + shift + 1 : lk) : 0;
        const int lim = min(max(row_limit - n * kBlockN, 0), kBlockN) - grp * 32;   // within this group's columns
        // ---- P = exp2(S * scale - lse), needs S only
        ok = __all_sync(0xFFFFFFFFu, mbar_wait(&sm.s_full[bf], par, abort_flag, p.status, 86));
        if (!ok) break;
        tc_fence_after();
        uint32_t x[32];                               // P of this thread's 32 columns, fp32 bits
        {
          uint32_t pp[16];
          tmem_ld32(tmem + lane_off + bf * 128 + grp * 32, x);
          tmem_wait_ld_dep(x);
          const uint64_t c2 = pack_f32x2(p.scale_log2, p.scale_log2), n2 = pack_f32x2(neg_lse, neg_lse);
#pragma unroll
          for (int c = 0; c < 32; c += 2) {
            float y0, y1;
            unpack_f32x2(fma_f32x2(pack_f32x2(x[c], x[c + 1]), c2, n2), y0, y1);
            const float x0 = c < lim ? exp2f(y0) : 0.f, x1 = c + 1 < lim ? exp2f(y1) : 0.f;
            x[c] = __float_as_uint(x0);
            x[c + 1] = __float_as_uint(x1);
            pp[c >> 1] = pack_bf16(x0, x1);
          }
          // the dV product of the step before must have read P before it is rewritten
          if (i >= 1) {
            ok = __all_sync(0xFFFFFFFFu, mbar_wait(&sm.do_free[(i - 1) & 1], (uint32_t)(((i - 1) >> 1) & 1),
                                                   abort_flag, p.status, 87));
            if (!ok) break;
          }
#pragma unroll
          for (int c = 0; c < 4; ++c)                  // this group's four 16-byte chunks of the row
            *reinterpret_cast<uint4*>(prow + (((grp * 4 + c) ^ (r & 7)) << 4)) =
                make_uint4(pp[4 * c], pp[4 * c + 1], pp[4 * c + 2], pp[4 * c + 3]);
          fence_proxy_async_smem();
          mbar_arrive_warp(&sm.p_ready);
        }
        // ---- dS = P * (dP - D)
        ok = __all_sync(0xFFFFFFFFu, mbar_wait(&sm.dp_full[bf], par, abort_flag, p.status, 92));
        if (!ok) break;
        tc_fence_after();
        {
          uint32_t dpv[32], dd[16];
          tmem_ld32(tmem + lane_off + bf * 128 + 64 + grp * 32, dpv);
          tmem_wait_ld_dep(dpv);
          tc_fence_before();
          mbar_arrive_warp(&sm.sdp_empty[bf]);               // S / dP of this buffer may be overwritten
          const uint64_t md2 = pack_f32x2(-dsum, -dsum);
#pragma unroll
          for (int c = 0; c < 32; c += 2) {
            float d0, d1;
            unpack_f32x2(mul_f32x2(pack_f32x2(x[c], x[c + 1]), add_f32x2(pack_f32x2(dpv[c], dpv[c + 1]), md2)), d0, d1);
            dd[c >> 1] = pack_bf16(d0, d1);
          }
          // the dK product of the step before must have read dS before it is rewritten
          if (i >= 1) {
            ok = __all_sync(0xFFFFFFFFu, mbar_wait(&sm.dk_done[pqs], (uint32_t)(pround & 1), abort_flag, p.status, 93));
            if (!ok) break;
          }
#pragma unroll
          for (int c = 0; c < 4; ++c)
            *reinterpret_cast<uint4*>(drow + (((grp * 4 + c) ^ (r & 7)) << 4)) =
                make_uint4(dd[4 * c], dd[4 * c + 1], dd[4 * c + 2], dd[4 * c + 3]);
          fence_proxy_async_smem();
          mbar_arrive_warp(&sm.ds_ready);
        }
      }
    }
    // the warps of the first turn write the block's gradients
    if (turn != 0) ok = false;
    if (ok && steps > 0) {
      ok = __all_sync(0xFFFFFFFFu, mbar_wait(&sm.dk_done[(steps - 1) % 3],
                                             (uint32_t)(((steps - 1) / 3) & 1), abort_flag, p.status, 88));
      tc_fence_after();
    }
    if (ok) {
      // this thread owns feature d = r of dV^T / dK^T; 64 key columns each
      const int d = r;
      __nv_bfloat16* dv_base = p.dv + ((int64_t)(k0 + n * kBlockN) * p.heads_k + h) * kHeadDim + d;
      __nv_bfloat16* dk_base = p.dk + ((int64_t)(k0 + n * kBlockN) * p.heads_k + h) * kHeadDim + d;
      const int64_t key_stride = (int64_t)p.heads_k * kHeadDim;
      {
        const int c0 = grp * 32;
        uint32_t a[32], bb[32];
        if (steps > 0) {
          tmem_ld32x2_wait(tmem_dv + lane_off + c0, a, tmem_dk + lane_off + c0, bb);
        } else {
#pragma unroll
          for (int j = 0; j < 32; ++j) { a[j] = 0u; bb[j] = 0u; }
        }
#pragma unroll
        for (int j = 0; j < 32; ++j) {
          if (c0 + j < nkeys) {
            dv_base[(int64_t)(c0 + j) * key_stride] = __float2bfloat16_rn(__uint_as_float(a[j]));
            dk_base[(int64_t)(c0 + j) * key_stride] =
                __float2bfloat16_rn(__uint_as_float(bb[j]) * p.scale);
          }
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 3) tmem_dealloc(tmem, 512);
}

}  // namespace
}  // namespace ifv2

using namespace ifv2;

extern "C" int64_t ifv2_sparse_attn_bwd_workspace_bytes(int64_t total_q, int heads_q, int head_dim) {
  (void)head_dim;
  return total_q * heads_q * 4 + 256;       // D = rowsum(dO * O), one fp32 per (token, query head)
}

extern "C" int ifv2_sparse_attn_bwd(const void* dout, const void* q, const void* k, const void* v,
                                    const void* out, const float* lse, void* dq, void* dk, void* dv,
                                    const int64_t* fwd_mask, int fwd_mask_words,
                                    const int64_t* bwd_mask, int64_t bwd_mask_words,
                                    const int32_t* cu_seqlens_q, const int32_t* cu_seqlens_k,
                                    int batch, int64_t total_q, int64_t total_k, int heads_q,
                                    int heads_k, int head_dim, int max_seqlen_q, int max_seqlen_k,
                                    float softmax_scale, int causal, void* workspace,
                                    int64_t workspace_bytes, int32_t* status, void* stream) {
  IFV2_REQUIRE(head_dim == kHeadDim, IFV2_ERR_UNSUPPORTED,
               "sparse_attn_bwd: head_dim %d not supported (only 128)", head_dim);
  IFV2_REQUIRE(heads_k >= 1 && heads_q == heads_k * kGroup, IFV2_ERR_UNSUPPORTED,
               "sparse_attn_bwd: heads_q (%d) must be 16 x heads_k (%d)", heads_q, heads_k);
  IFV2_REQUIRE(batch >= 1 && total_q >= 0 && total_k >= 0 && max_seqlen_q >= 0 && max_seqlen_k >= 0,
               IFV2_ERR_INVALID_ARG, "sparse_attn_bwd: negative size or batch < 1");
  if (total_q == 0 && total_k == 0) return IFV2_OK;
  IFV2_REQUIRE(dout && q && k && v && out && lse && dq && dk && dv && cu_seqlens_q && cu_seqlens_k &&
                   status && workspace,
               IFV2_ERR_INVALID_ARG, "sparse_attn_bwd: null pointer");
  IFV2_REQUIRE((fwd_mask == nullptr) == (bwd_mask == nullptr), IFV2_ERR_INVALID_ARG,
               "sparse_attn_bwd: pass both the row mask and the column mask, or neither");
  IFV2_REQUIRE(workspace_bytes >= ifv2_sparse_attn_bwd_workspace_bytes(total_q, heads_q, head_dim),
               IFV2_ERR_INVALID_ARG, "sparse_attn_bwd: workspace too small");
  IFV2_REQUIRE(reinterpret_cast<uintptr_t>(workspace) % 16 == 0, IFV2_ERR_INVALID_ARG,
               "sparse_attn_bwd: workspace must be 16-byte aligned");
  IFV2_REQUIRE(total_q <= INT32_MAX && total_k <= INT32_MAX, IFV2_ERR_TOO_LARGE,
               "sparse_attn_bwd: more than 2^31-1 tokens");
  const int k_blocks = (max_seqlen_k + kBlockN - 1) / kBlockN;
  IFV2_REQUIRE((k_blocks + 63) / 64 <= kMaxMaskWords, IFV2_ERR_TOO_LARGE,
               "sparse_attn_bwd: max_seqlen_k %d exceeds %d keys", max_seqlen_k,
               kMaxMaskWords * 64 * kBlockN);
  if (fwd_mask != nullptr) {
    IFV2_REQUIRE(fwd_mask_words == (k_blocks + 63) / 64, IFV2_ERR_INVALID_ARG,
                 "sparse_attn_bwd: row mask must have ceil(ceil(max_seqlen_k/64)/64) = %d words",
                 (k_blocks + 63) / 64);
    IFV2_REQUIRE(bwd_mask_words == (total_q + 63) / 64, IFV2_ERR_INVALID_ARG,
                 "sparse_attn_bwd: column mask must have ceil(total_q/64) = %lld words",
                 (long long)((total_q + 63) / 64));
  }
  IFV2_REQUIRE(batch <= 65535 && heads_k <= 65535, IFV2_ERR_TOO_LARGE,
               "sparse_attn_bwd: batch or heads_k > 65535");
  cudaStream_t st = (cudaStream_t)stream;

  BwdParams p;
  p.lse = lse;
  p.dvec = static_cast<float*>(workspace);
  p.dq = static_cast<__nv_bfloat16*>(dq);
  p.dk = static_cast<__nv_bfloat16*>(dk);
  p.dv = static_cast<__nv_bfloat16*>(dv);
  p.fwd_mask = reinterpret_cast<const unsigned long long*>(fwd_mask);
  p.fwd_words = fwd_mask_words;
  p.bwd_mask = reinterpret_cast<const unsigned long long*>(bwd_mask);
  p.bwd_words = bwd_mask_words;
  p.k_blocks = k_blocks;
  p.cu_q = cu_seqlens_q;
  p.cu_k = cu_seqlens_k;
  p.total_q = total_q;
  p.heads_q = heads_q;
  p.heads_k = heads_k;
  p.scale = softmax_scale;
  p.scale_log2 = softmax_scale * kLog2e;
  p.causal = causal ? 1 : 0;
  p.status = status;

  {
    const int rc0 = clear_launch_status(status, stream, "sparse_attn_bwd");
    if (rc0) return rc0;
  }
  if (total_q > 0) {
    const int64_t rows = total_q * heads_q;
    int64_t blocks = ceil_div64(rows, 16);
    if (blocks > (int64_t)kNumSMs * 16) blocks = (int64_t)kNumSMs * 16;
    dot_do_o_kernel<<<(int)blocks, 256, 0, st>>>(static_cast<const __nv_bfloat16*>(dout),
                                                 static_cast<const __nv_bfloat16*>(out), p.dvec,
                                                 total_q, heads_q);
    int rc = check_launch("dot_do_o");
    if (rc) return rc;
  }

  CUtensorMap map_q, map_do, map_k, map_v;
  const uint64_t tq = total_q > 0 ? total_q : 1, tk = total_k > 0 ? total_k : 1;
  int rc = make_tensor_map_bf16_3d(&map_q, q, kHeadDim, heads_q, tq, kHeadDim * 2,
                                   (uint64_t)heads_q * kHeadDim * 2, 64, kGroup, kTokPerTile);
  if (rc) return rc;
  rc = make_tensor_map_bf16_3d(&map_do, dout, kHeadDim, heads_q, tq, kHeadDim * 2,
                               (uint64_t)heads_q * kHeadDim * 2, 64, kGroup, kTokPerTile);
  if (rc) return rc;
  rc = make_tensor_map_bf16_3d(&map_k, k, kHeadDim, heads_k, tk, kHeadDim * 2,
                               (uint64_t)heads_k * kHeadDim * 2, 64, 1, kBlockN);
  if (rc) return rc;
  rc = make_tensor_map_bf16_3d(&map_v, v, kHeadDim, heads_k, tk, kHeadDim * 2,
                               (uint64_t)heads_k * kHeadDim * 2, 64, 1, kBlockN);
  if (rc) return rc;

  if (total_q > 0 && max_seqlen_q > 0) {
    const size_t smem = sizeof(DqSmem) + 1024;
    cudaError_t e = cudaFuncSetAttribute(sparse_attn_bwd_dq_kernel,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return set_error((int)e, "sparse_attn_bwd: %s", cudaGetErrorString(e));
    dim3 grid((max_seqlen_q + kTokPerTile - 1) / kTokPerTile, batch, heads_k);
    sparse_attn_bwd_dq_kernel<<<grid, kDqThreads, smem, st>>>(map_q, map_do, map_k, map_v, p);
    rc = check_launch("sparse_attn_bwd_dq");
    if (rc) return rc;
  }
  if (total_k > 0 && max_seqlen_k > 0) {
    const size_t smem = sizeof(DkvSmem) + 1024;
    cudaError_t e = cudaFuncSetAttribute(sparse_attn_bwd_dkv_kernel,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return set_error((int)e, "sparse_attn_bwd: %s", cudaGetErrorString(e));
    dim3 grid(batch, heads_k, k_blocks);
    sparse_attn_bwd_dkv_kernel<<<grid, kDkvThreads, smem, st>>>(map_q, map_do, map_k, map_v, p);
    rc = check_launch("sparse_attn_bwd_dkv");
    if (rc) return rc;
  }
  return IFV2_OK;
}

// ------------------------------------------------------------------ allocation-free variant --
// Scratch for ifv2_sparse_attn_bwd_noalloc: the D = rowsum(dO * O) rows, one fp32 per
// (token, query head), for up to kNoAllocMaxRows rows.  Every process that loads the library
// holds these 16 MiB on each GPU it touches, until it exits.
#include <mutex>

static constexpr long long kNoAllocMaxRows = 4ll << 20;
static __device__ __align__(256) unsigned char g_bwd_noalloc_scratch[kNoAllocMaxRows * 4 + 256];

namespace {
constexpr int kMaxDevices = 64;
std::mutex g_noalloc_mutex;
void* g_noalloc_ptr[kMaxDevices] = {nullptr};   // device address of the array, per device
}  // namespace

extern "C" int ifv2_sparse_attn_bwd_noalloc(
    const void* dout, const void* q, const void* k, const void* v, const void* out,
    const float* lse, void* dq, void* dk, void* dv, const int64_t* fwd_mask, int fwd_mask_words,
    const int64_t* bwd_mask, int64_t bwd_mask_words, const int32_t* cu_seqlens_q,
    const int32_t* cu_seqlens_k, int batch, int64_t total_q, int64_t total_k, int heads_q,
    int heads_k, int head_dim, int max_seqlen_q, int max_seqlen_k, float softmax_scale, int causal,
    int32_t* status, void* stream) {
  IFV2_REQUIRE(total_q >= 0 && heads_q >= 0, IFV2_ERR_INVALID_ARG,
               "sparse_attn_bwd_noalloc: negative size");
  IFV2_REQUIRE(total_q * (int64_t)heads_q <= kNoAllocMaxRows, IFV2_ERR_TOO_LARGE,
               "sparse_attn_bwd_noalloc: total_q x heads_q = %lld query rows exceed the built-in "
               "scratch of %lld rows; use ifv2_sparse_attn_bwd with a caller workspace",
               (long long)(total_q * (int64_t)heads_q), kNoAllocMaxRows);
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess)
    return set_error((int)e, "sparse_attn_bwd_noalloc: cudaGetDevice: %s", cudaGetErrorString(e));
  IFV2_REQUIRE(dev >= 0 && dev < kMaxDevices, IFV2_ERR_TOO_LARGE,
               "sparse_attn_bwd_noalloc: device ordinal %d not supported", dev);
  void* scratch = nullptr;
  {
    // Set-up, once per device, with that device current: in host code the array's name is only a
    // stand-in, the address a kernel can use comes from the runtime.
    std::lock_guard<std::mutex> lock(g_noalloc_mutex);
    if (g_noalloc_ptr[dev] == nullptr) {
      void* ptr = nullptr;
      e = cudaGetSymbolAddress(&ptr, g_bwd_noalloc_scratch);
      if (e != cudaSuccess || ptr == nullptr)
        return set_error(e != cudaSuccess ? (int)e : IFV2_ERR_DRIVER,
                         "sparse_attn_bwd_noalloc: cudaGetSymbolAddress: %s", cudaGetErrorString(e));
      g_noalloc_ptr[dev] = ptr;
    }
    scratch = g_noalloc_ptr[dev];
  }
  // Nothing in the scratch has to start at zero: the first kernel of the backward overwrites
  // every D row that the later kernels read.
  return ifv2_sparse_attn_bwd(dout, q, k, v, out, lse, dq, dk, dv, fwd_mask, fwd_mask_words, bwd_mask,
                              bwd_mask_words, cu_seqlens_q, cu_seqlens_k, batch, total_q, total_k,
                              heads_q, heads_k, head_dim, max_seqlen_q, max_seqlen_k, softmax_scale,
                              causal, scratch, (int64_t)sizeof(g_bwd_noalloc_scratch), status, stream);
}
