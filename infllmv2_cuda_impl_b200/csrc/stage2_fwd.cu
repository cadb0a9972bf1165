// Stage-2 forward: block-sparse varlen flash attention on tcgen05 tensor cores.
//
// One CTA owns a 128-row query tile = 8 consecutive tokens x the 16 query heads of one KV head
// (in the caller's (token, head, d) layout those 16 heads are contiguous, so one 3-D TMA box
// {64 d, 16 heads, 8 tokens} fetches the tile with no host-side transpose).  The CTA walks the
// UNION of its 8 tokens' block-mask rows from the highest block down; a token that did not
// select a block sees -inf for it.  Per 64-key block:
//     S(128x64)  = Q . K^T      tcgen05.mma, operands in swizzled smem, accumulator in TMEM
//     P = exp2(S*c - m*c)       4 softmax warps, one TMEM lane (= row) per thread; P is written
//                               back over S in TMEM as packed bf16
//     O(128x128) += P . V       tcgen05.mma with the A operand read from TMEM
// Warp roles: warp 0 = TMA producer, warp 1 = MMA issuer (+ TMEM owner), warps 2-5 = softmax /
// epilogue.  K and V each have a 2-deep ring; S/P is double-buffered in TMEM so Q.K^T of the
// next block overlaps the softmax of the current one.  TMEM: 2 x 64 (S/P) + 128 (O) = 256
// columns, shared memory 96 KB, so two CTAs share an SM and fill each other's bubbles.
// The running max is only raised when it grows by more than 2^8 (the accumulator then needs a
// rescale); P stays bounded by 256 and the final 1/l normalisation makes the result exact.
// Measured with the optional timeline below: the tensor pipe is ~70 % busy and what bounds a
// CTA is the latency of the chain S ready -> P ready -> P.V -> next Q.K^T on each S buffer
// while the co-resident CTA competes for the tensor pipe and the exponential unit.  Splitting a
// row over two threads (8 softmax warps, half-row maxima exchanged through shared memory) or
// giving each S buffer its own warp group did not shorten that chain and ran 8-12 % slower;
// evaluating every 2nd, 3rd or 4th pair of exponentials on the FMA pipe (degree-3 polynomial)
// ran 8, 4 and 3 % slower: the exponential unit is not what the softmax warps wait for.
#include "tc05.cuh"

namespace ifv2 {
namespace {

using namespace tc;

constexpr int kTokPerTile = 8;
constexpr int kThreads = 192;
constexpr int kMaxMaskWords = 128;            // 8192 key blocks = 524288 keys per sequence
constexpr uint32_t kQHalfBytes = 128 * 128;   // 128 rows x 64 bf16
constexpr uint32_t kKVHalfBytes = 64 * 128;   // 64 keys x 64 bf16
constexpr uint32_t kTmemCols = 256;
constexpr float kRescaleThreshold = 8.0f;     // log2 units

struct FwdParams {
  __nv_bfloat16* out;
  float* lse;
  const unsigned long long* mask;
  int mask_words;
  const int32_t* cu_q;
  const int32_t* cu_k;
  const int32_t* seqused_k;       // keys in use per sequence, or null (then the cu_k extent)
  const int32_t* leftpad_k;       // keys of a sequence start this many rows into its cu_k extent, or null
  const int32_t* block_table;     // (batch, bt_stride) page of every page_size key positions, or null
  int bt_stride, page_size;
  int64_t total_q;
  int heads_q, heads_k;
  float scale, scale_log2;
  int causal;
  int32_t* status;
};

struct Smem {
  uint8_t q[2][kQHalfBytes];          // [d half]
  uint8_t k[2][2][kKVHalfBytes];      // [stage][d half]
  uint8_t v[2][2][kKVHalfBytes];      // [stage][d half]
  unsigned long long umask[kMaxMaskWords];
  // One tcgen05.commit costs the issuing warp about as much as two MMAs, so every product
  // signals exactly one barrier and everybody interested waits on that one:
  //   qk_done[s]: S of ring slot s is complete -> the softmax warps read it, the producer may
  //               refill the K tile;  pv_done[s]: O holds the block of slot s -> the producer may
  //               refill the V tile, a rescale or the epilogue may touch O.
  uint64_t q_full, k_full[2], v_full[2], qk_done[2], pv_done[2], p_ready[2];
  uint32_t tmem_base;
  int n_blocks;
  int abort_flag;
};

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

// Highest-to-lowest walk over the set bits of the tile's union mask.
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

__global__ void __launch_bounds__(kThreads, 2)
sparse_attn_fwd_kernel(const __grid_constant__ CUtensorMap map_q,
                       const __grid_constant__ CUtensorMap map_k,
                       const __grid_constant__ CUtensorMap map_v, const FwdParams p) {
  extern __shared__ uint8_t smem_raw[];
  Smem& sm = *reinterpret_cast<Smem*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                      ~(uintptr_t)1023);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int b = blockIdx.y, h = blockIdx.z;
  const int q0 = p.cu_q[b], lq = p.cu_q[b + 1] - q0;
  // keys of the sequence: rows [k0, k0 + lk) of a packed tensor (optionally starting `leftpad_k`
  // rows into the sequence's extent, block_info.h:22-24, 40), or positions [0, lk) of a paged
  // cache whose pages the block table names
  const int pad = p.leftpad_k ? p.leftpad_k[b] : 0;
  const int k0 = p.block_table ? 0 : p.cu_k[b] + pad;
  const int lk = max(0, (p.seqused_k ? p.seqused_k[b] : p.cu_k[b + 1] - p.cu_k[b]) - pad);
  const int tok0 = ((int)gridDim.x - 1 - (int)blockIdx.x) * kTokPerTile;   // long tiles first
  if (tok0 >= lq) return;
  // an earlier CTA gave up on a wait: the launch is already failed, do not pile up more waits
  if (*reinterpret_cast<volatile int32_t*>(p.status) != 0) return;
  const int ntok = min(kTokPerTile, lq - tok0);
  const int shift = lk - lq;                        // bottom-right aligned causal diagonal
  const int nblk_k = (lk + kBlockN - 1) / kBlockN;
  const int words = (p.mask != nullptr) ? p.mask_words : min(kMaxMaskWords, (nblk_k + 63) / 64);

  // ---- union of the tile's mask rows, trimmed to the blocks any of its tokens can see
  {
    int last_blk = nblk_k - 1;
    if (p.causal) last_blk = min(last_blk, (tok0 + ntok - 1 + shift) >= 0
                                               ? (tok0 + ntok - 1 + shift) / kBlockN : -1);
    for (int w = threadIdx.x; w < words; w += kThreads) {
      unsigned long long u = 0ull;
      if (p.mask != nullptr) {
        const unsigned long long* row =
            p.mask + ((int64_t)h * p.total_q + q0 + tok0) * p.mask_words + w;
        for (int t = 0; t < ntok; ++t) u |= __ldg(row + (int64_t)t * p.mask_words);
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
    mbar_init(&sm.q_full, 1);
    for (int s = 0; s < 2; ++s) {
      mbar_init(&sm.k_full[s], 1);
      mbar_init(&sm.qk_done[s], 1);
      mbar_init(&sm.v_full[s], 1);
      mbar_init(&sm.pv_done[s], 1);
      mbar_init(&sm.p_ready[s], 4);          // one arrival per softmax warp
    }
    fence_barrier_init();
    prefetch_tensormap(&map_q);
    prefetch_tensormap(&map_k);
    prefetch_tensormap(&map_v);
  }
  if (warp == 1) {
    tmem_alloc(&sm.tmem_base, kTmemCols);
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
  const uint32_t tmem_o = tmem + 128;
  volatile int* abort_flag = &sm.abort_flag;

  if (warp == 0) {
    // ================================================================ TMA producer
    if (lane == 0 && n_blocks > 0) {
      mbar_expect_tx(&sm.q_full, 2 * kQHalfBytes);
      tma_load_3d(sm.q[0], &map_q, &sm.q_full, 0, h * kGroup, q0 + tok0);
      tma_load_3d(sm.q[1], &map_q, &sm.q_full, 64, h * kGroup, q0 + tok0);
      BlockWalk walk(sm.umask, words);
      int issued = 0;
      bool ok = true;
      for (int i = 0; i < n_blocks && ok; ++i) {
        const int blk = walk.next();
        const int s = i & 1;
        int key = k0 + blk * kBlockN;
        if (p.block_table != nullptr) {          // a 64-key block never straddles a page
          const int pos = blk * kBlockN;
          key = __ldg(p.block_table + (int64_t)b * p.bt_stride + pos / p.page_size) * p.page_size +
                pos % p.page_size;
        }
        const uint32_t par = (uint32_t)((i >> 1) & 1);
        if (i >= 2) ok = mbar_wait(&sm.qk_done[s], par ^ 1u, abort_flag, p.status, 11);
        if (!ok) break;
        mbar_expect_tx(&sm.k_full[s], 2 * kKVHalfBytes);
        tma_load_3d(sm.k[s][0], &map_k, &sm.k_full[s], 0, h, key);
        tma_load_3d(sm.k[s][1], &map_k, &sm.k_full[s], 64, h, key);
        if (i >= 2) ok = mbar_wait(&sm.pv_done[s], par ^ 1u, abort_flag, p.status, 12);
        if (!ok) { issued = i + 1; break; }
        mbar_expect_tx(&sm.v_full[s], 2 * kKVHalfBytes);
        tma_load_3d(sm.v[s][0], &map_v, &sm.v_full[s], 0, h, key);
        tma_load_3d(sm.v[s][1], &map_v, &sm.v_full[s], 64, h, key);
        issued = i + 1;
      }
      if (*abort_flag) {   // let the copies already in flight land before the CTA retires
        mbar_wait_drain(&sm.q_full, 0);
        for (int j = max(0, issued - 2); j < issued; ++j) {
          mbar_wait_drain(&sm.k_full[j & 1], (uint32_t)((j >> 1) & 1));
          mbar_wait_drain(&sm.v_full[j & 1], (uint32_t)((j >> 1) & 1));
        }
      }
    }
  } else if (warp == 1) {
    // ================================================================ MMA issuer
    // All 32 lanes run the same issue code (descriptors stay in uniform registers); `leader`
    // enables the MMA / commit instructions in one lane only.
    if (n_blocks > 0) {
      const uint32_t leader = (lane == 0) ? 1u : 0u;
      constexpr uint32_t idesc_qk = umma_idesc_bf16(128, 64, false);
      constexpr uint32_t idesc_pv = umma_idesc_bf16(128, 128, true);
      const uint64_t q_desc = umma_desc_sw128(smem_u32(sm.q[0]), 16, 1024);
      // ring stage s = stage 0 + s * kStage: plain arithmetic keeps the descriptors in registers
      // (a runtime-indexed array of descriptors would live in local memory)
      const uint64_t k_desc0 = umma_desc_sw128(smem_u32(sm.k[0][0]), 16, 1024);
      const uint64_t v_desc0 = umma_desc_sw128(smem_u32(sm.v[0][0]), kKVHalfBytes, 1024);
      constexpr uint32_t kStage = (2 * kKVHalfBytes) >> 4;
      bool ok = __all_sync(0xFFFFFFFFu, mbar_wait(&sm.q_full, 0, abort_flag, p.status, 21));
      auto issue_qk = [&](int j) -> bool {
        const int s = j & 1;
        if (!__all_sync(0xFFFFFFFFu, mbar_wait(&sm.k_full[s], (uint32_t)((j >> 1) & 1), abort_flag,
                                               p.status, 22)))
          return false;
        tc_fence_after();
#pragma unroll
        for (int kk = 0; kk < 8; ++kk) {
          const uint32_t qoff = (kk >> 2) * kQHalfBytes + (kk & 3) * 32;
          const uint32_t koff = (kk >> 2) * kKVHalfBytes + (kk & 3) * 32;
          umma_ss_pred(tmem + s * 64, q_desc + (qoff >> 4), k_desc0 + s * kStage + (koff >> 4), idesc_qk,
                       kk > 0, leader);
        }
        umma_commit_pred(&sm.qk_done[s], leader);
        return true;
      };
      if (ok) ok = issue_qk(0);
      for (int i = 0; i < n_blocks && ok; ++i) {
        const int s = i & 1;
        const uint32_t par = (uint32_t)((i >> 1) & 1);
        if (i + 1 < n_blocks) ok = issue_qk(i + 1);
        if (!ok) break;
        // (V landed long ago: its wait goes first so that it is not paid after P is ready)
        ok = __all_sync(0xFFFFFFFFu, mbar_wait(&sm.v_full[s], par, abort_flag, p.status, 24) &&
                                         mbar_wait(&sm.p_ready[s], par, abort_flag, p.status, 23));
        if (!ok) break;
        tc_fence_after();
#pragma unroll
        for (int kk = 0; kk < 4; ++kk)
          umma_ts_pred(tmem_o, tmem + s * 64 + kk * 8, v_desc0 + s * kStage + ((kk * 2048) >> 4), idesc_pv,
                       (i > 0) || (kk > 0), leader);
        umma_commit_pred(&sm.pv_done[s], leader);
      }
    }
  } else {
    // ================================================================ softmax + epilogue
    const int quad = warp & 3;                       // TMEM lane quadrant this warp may access
    const int r = quad * 32 + lane;                  // row of the tile = TMEM lane
    const int tl = r >> 4, g = r & 15;
    const int tok = tok0 + tl;                       // local token index
    const bool valid = tl < ntok;
    const uint32_t lane_off = (uint32_t)(quad * 32) << 16;
    const unsigned long long* mrow =
        (p.mask != nullptr && valid)
            ? p.mask + ((int64_t)h * p.total_q + q0 + tok) * p.mask_words : nullptr;
    const int row_limit = valid ? min(lk, p.causal ? tok + shift + 1 : lk) : 0;   // visible keys

    float m_ref = -INFINITY, l = 0.f;
    bool ok = true;
    BlockWalk walk(sm.umask, words);
    MaskRowReader mask_reader(mrow);
    for (int i = 0; i < n_blocks; ++i) {
      const int blk = walk.next();
      const int s = i & 1;
      const uint32_t par = (uint32_t)((i >> 1) & 1);
      const bool selected = valid && mask_reader.selected(blk);
      const int lim = selected ? min(max(row_limit - blk * kBlockN, 0), kBlockN) : 0;
      // only the diagonal / ragged block needs per-element masking; a row that did not select
      // the block is handled by the row-level terms below
      const bool partial = __any_sync(0xFFFFFFFFu, lim > 0 && lim < kBlockN);
      ok = __all_sync(0xFFFFFFFFu, mbar_wait(&sm.qk_done[s], par, abort_flag, p.status, 31));
      if (!ok) break;
      tc_fence_after();

      // keys of this block that exist: in the ragged last block of a sequence the K / V rows past
      // them hold the next sequence's keys or whatever an unused part of a cache page contains
      const int nk = lk - blk * kBlockN;
      uint32_t raw[64];
      tmem_ld64_wait(tmem + lane_off + s * 64, raw);
      if (partial || nk < kBlockN) {         // (every row of a ragged block: its scores may be NaN)
#pragma unroll
        for (int c = 0; c < 64; ++c)
          if (c >= lim) raw[c] = 0xFF800000u;                              // -inf
      }
      uint32_t packed[32];
      float sum = 0.f;
      // P = exp2(S * c + neg) for the row's 64 scores, packed to bf16, and their sum
      auto compute_p = [&](float neg) {
        const uint64_t c2 = pack_f32x2(p.scale_log2, p.scale_log2), n2 = pack_f32x2(neg, neg);
        uint64_t sum2[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) sum2[i] = pack_f32x2(0.f, 0.f);
#pragma unroll
        for (int c = 0; c < 64; c += 2) {
          float y0, y1;
          unpack_f32x2(fma_f32x2(pack_f32x2(raw[c], raw[c + 1]), c2, n2), y0, y1);
          const float p0 = exp2f(y0), p1 = exp2f(y1);
          sum2[(c >> 1) & 3] = add_f32x2(sum2[(c >> 1) & 3], pack_f32x2(p0, p1));
          packed[c >> 1] = pack_bf16(p0, p1);
        }
        float s_lo, s_hi;
        unpack_f32x2(add_f32x2(add_f32x2(sum2[0], sum2[1]), add_f32x2(sum2[2], sum2[3])), s_lo, s_hi);
        sum = s_lo + s_hi;
      };
      auto row_max = [&]() -> float {
        float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
        for (int c = 0; c < 64; c += 2)           // two scores per step: a three-input maximum each
          mx4[(c >> 1) & 3] = fmaxf(mx4[(c >> 1) & 3], fmaxf(__uint_as_float(raw[c]), __uint_as_float(raw[c + 1])));
        return (lim > 0) ? fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3])) : -INFINITY;
      };
      // The reference maximum moves only when the row maximum exceeds it by more than the
      // threshold, which after a row's first block almost never happens.  So once every row of the
      // warp that takes part has a reference, the exponentials are started against the current one
      // and the row maximum is computed beside them (it is off the chain S -> P); a block that does
      // move some row's reference is redone below, with the result the in-order form would give.
      bool done = false;
      if (!__any_sync(0xFFFFFFFFu, lim > 0 && m_ref == -INFINITY)) {
        compute_p((lim == 0) ? -INFINITY : -m_ref * p.scale_log2);
        const float mx = row_max();
        const bool moves = mx > m_ref && (mx - m_ref) * p.scale_log2 > kRescaleThreshold;
        done = !__any_sync(0xFFFFFFFFu, moves);
      }
      if (!done) {
        const float mx = row_max();
        // raise the reference max only when it moves by more than the threshold
        float f = 1.f;
        if (mx > m_ref && (m_ref == -INFINITY || (mx - m_ref) * p.scale_log2 > kRescaleThreshold)) {
          if (m_ref != -INFINITY) f = exp2f((m_ref - mx) * p.scale_log2);
          m_ref = mx;
          l *= f;
        }
        if (i > 0 && __any_sync(0xFFFFFFFFu, f != 1.f)) {
          // the previous block's product (slot (i-1)&1, its ((i-1)>>1)-th use).  S of this block is
          // complete, so every product up to block i-2 is too: the barrier is at most one phase
          // behind and the parity wait is unambiguous
          ok = __all_sync(0xFFFFFFFFu, mbar_wait(&sm.pv_done[(i - 1) & 1], (uint32_t)(((i - 1) >> 1) & 1),
                                                 abort_flag, p.status, 32));
          if (!ok) break;
          tc_fence_after();
#pragma unroll 1
          for (int c = 0; c < 128; c += 32) {
            uint32_t o[32];
            tmem_ld32(tmem_o + lane_off + c, o);
            tmem_wait_ld();
#pragma unroll
            for (int j = 0; j < 32; ++j) o[j] = __float_as_uint(__uint_as_float(o[j]) * f);
            tmem_st32(tmem_o + lane_off + c, o);
          }
          tmem_wait_st();
        }
        // rows that take nothing from this block get an exponent of -inf (P = 0) for every column
        compute_p((lim == 0) ? -INFINITY : -m_ref * p.scale_log2);
      }
      // The V rows past the last key of a ragged block have P = 0, but 0 x inf or 0 x NaN is not 0,
      // so those rows are cleared before the product reads them.
      if (nk < kBlockN) {
        ok = __all_sync(0xFFFFFFFFu, mbar_wait(&sm.v_full[s], par, abort_flag, p.status, 34));
        if (!ok) break;
        const int t128 = threadIdx.x - 64;                   // 0..127 among the softmax threads
        for (int i = t128; i < (kBlockN - nk) * 16; i += 128) {
          const int row = nk + (i >> 4), half = (i >> 3) & 1, chunk = i & 7;
          *reinterpret_cast<uint4*>(sm.v[s][half] + row * 128 + chunk * 16) = make_uint4(0u, 0u, 0u, 0u);
        }
        fence_proxy_async_smem();
      }
      l += sum;
      tmem_st32(tmem + lane_off + s * 64, packed);
      tmem_wait_st();
      tc_fence_before();
      mbar_arrive_warp(&sm.p_ready[s]);
    }

    // ---- epilogue: O / l -> bf16, lse
    if (ok && n_blocks > 0) {
      // the last product; as above, all but the last two are known to be complete
      ok = __all_sync(0xFFFFFFFFu,
                      mbar_wait(&sm.pv_done[(n_blocks - 1) & 1],
                                (uint32_t)(((n_blocks - 1) >> 1) & 1), abort_flag, p.status, 33));
      tc_fence_after();
    }
    if (ok) {
      const float inv = (l > 0.f) ? 1.f / l : 0.f;
      __nv_bfloat16* orow =
          p.out + ((int64_t)(q0 + tok) * p.heads_q + h * kGroup + g) * kHeadDim;
#pragma unroll 1
      for (int c = 0; c < 128; c += 32) {
        uint32_t o[32];
        if (n_blocks > 0) {
          tmem_ld32(tmem_o + lane_off + c, o);
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
            v4.x = pack_bf16(__uint_as_float(o[8 * j + 0]) * inv, __uint_as_float(o[8 * j + 1]) * inv);
            v4.y = pack_bf16(__uint_as_float(o[8 * j + 2]) * inv, __uint_as_float(o[8 * j + 3]) * inv);
            v4.z = pack_bf16(__uint_as_float(o[8 * j + 4]) * inv, __uint_as_float(o[8 * j + 5]) * inv);
            v4.w = pack_bf16(__uint_as_float(o[8 * j + 6]) * inv, __uint_as_float(o[8 * j + 7]) * inv);
            dst[j] = v4;
          }
        }
      }
      if (valid)
        p.lse[(int64_t)h * p.total_q * kGroup + (int64_t)(q0 + tok) * kGroup + g] =
            (l > 0.f) ? m_ref * p.scale + logf(l) : INFINITY;
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem, kTmemCols);
}

}  // namespace
}  // namespace ifv2

using namespace ifv2;

static int sparse_attn_fwd_impl(const void* q, const void* k, const void* v, void* out,
                                float* lse, const int64_t* fwd_mask, int mask_words,
                                const int32_t* cu_seqlens_q, const int32_t* cu_seqlens_k,
                                const int32_t* seqused_k, const int32_t* leftpad_k,
                                const int32_t* block_table, int block_table_stride, int page_size,
                                int batch, int64_t total_q, int64_t total_k, int heads_q,
                                int heads_k, int head_dim, int max_seqlen_q, int max_seqlen_k,
                                float softmax_scale, int causal, int32_t* status,
                                void* stream) {
  IFV2_REQUIRE(head_dim == kHeadDim, IFV2_ERR_UNSUPPORTED,
               "sparse_attn_fwd: head_dim %d not supported (only 128, as in the reference build)",
               head_dim);
  IFV2_REQUIRE(heads_k >= 1 && heads_q == heads_k * kGroup, IFV2_ERR_UNSUPPORTED,
               "sparse_attn_fwd: heads_q (%d) must be 16 x heads_k (%d)", heads_q, heads_k);
  IFV2_REQUIRE(batch >= 1 && total_q >= 0 && total_k >= 0 && max_seqlen_q >= 0 && max_seqlen_k >= 0,
               IFV2_ERR_INVALID_ARG, "sparse_attn_fwd: negative size or batch < 1");
  if (total_q == 0 || max_seqlen_q == 0) return IFV2_OK;
  IFV2_REQUIRE(q && k && v && out && lse && cu_seqlens_q && cu_seqlens_k && status,
               IFV2_ERR_INVALID_ARG, "sparse_attn_fwd: null pointer");
  IFV2_REQUIRE(total_q <= INT32_MAX && total_k <= INT32_MAX, IFV2_ERR_TOO_LARGE,
               "sparse_attn_fwd: more than 2^31-1 tokens");
  const int k_blocks = (max_seqlen_k + kBlockN - 1) / kBlockN;
  IFV2_REQUIRE((k_blocks + 63) / 64 <= kMaxMaskWords, IFV2_ERR_TOO_LARGE,
               "sparse_attn_fwd: max_seqlen_k %d exceeds %d keys", max_seqlen_k,
               kMaxMaskWords * 64 * kBlockN);
  IFV2_REQUIRE(fwd_mask == nullptr || (mask_words >= 1 && mask_words <= kMaxMaskWords),
               IFV2_ERR_INVALID_ARG, "sparse_attn_fwd: mask_words %d out of range [1, %d]",
               mask_words, kMaxMaskWords);
  IFV2_REQUIRE(batch <= 65535 && heads_k <= 65535, IFV2_ERR_TOO_LARGE,
               "sparse_attn_fwd: batch or heads_k > 65535");
  if (block_table != nullptr) {
    IFV2_REQUIRE(page_size >= kBlockN && page_size % kBlockN == 0 && block_table_stride >= 1,
                 IFV2_ERR_INVALID_ARG, "sparse_attn_fwd: page size must be a positive multiple of 64");
    IFV2_REQUIRE(leftpad_k == nullptr, IFV2_ERR_UNSUPPORTED,
                 "sparse_attn_fwd: a paged cache takes no leftpad_k (as in the reference)");
    IFV2_REQUIRE((int64_t)block_table_stride * page_size >= max_seqlen_k, IFV2_ERR_INVALID_ARG,
                 "sparse_attn_fwd: the block table covers fewer than max_seqlen_k positions");
  }

  CUtensorMap map_q, map_k, map_v;
  int rc = make_tensor_map_bf16_3d(&map_q, q, kHeadDim, heads_q, total_q, kHeadDim * 2,
                                   (uint64_t)heads_q * kHeadDim * 2, 64, kGroup, kTokPerTile);
  if (rc) return rc;
  rc = make_tensor_map_bf16_3d(&map_k, k, kHeadDim, heads_k, total_k > 0 ? total_k : 1,
                               kHeadDim * 2, (uint64_t)heads_k * kHeadDim * 2, 64, 1, kBlockN);
  if (rc) return rc;
  rc = make_tensor_map_bf16_3d(&map_v, v, kHeadDim, heads_k, total_k > 0 ? total_k : 1,
                               kHeadDim * 2, (uint64_t)heads_k * kHeadDim * 2, 64, 1, kBlockN);
  if (rc) return rc;

  FwdParams p;
  p.out = static_cast<__nv_bfloat16*>(out);
  p.lse = lse;
  p.mask = reinterpret_cast<const unsigned long long*>(fwd_mask);
  p.mask_words = mask_words;
  p.cu_q = cu_seqlens_q;
  p.cu_k = cu_seqlens_k;
  p.seqused_k = seqused_k;
  p.leftpad_k = leftpad_k;
  p.block_table = block_table;
  p.bt_stride = block_table_stride;
  p.page_size = page_size > 0 ? page_size : 1;
  p.total_q = total_q;
  p.heads_q = heads_q;
  p.heads_k = heads_k;
  p.scale = softmax_scale;
  p.scale_log2 = softmax_scale * 1.4426950408889634f;
  p.causal = causal ? 1 : 0;
  p.status = status;

  const size_t smem = sizeof(Smem) + 1024;
  cudaError_t e = cudaFuncSetAttribute(sparse_attn_fwd_kernel,
                                       cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return set_error((int)e, "sparse_attn_fwd: %s", cudaGetErrorString(e));
  dim3 grid((max_seqlen_q + kTokPerTile - 1) / kTokPerTile, batch, heads_k);
  rc = clear_launch_status(status, stream, "sparse_attn_fwd");
  if (rc) return rc;
  sparse_attn_fwd_kernel<<<grid, kThreads, smem, (cudaStream_t)stream>>>(map_q, map_k, map_v, p);
  return check_launch("sparse_attn_fwd");
}

extern "C" int ifv2_sparse_attn_fwd(const void* q, const void* k, const void* v, void* out,
                                    float* lse, const int64_t* fwd_mask, int mask_words,
                                    const int32_t* cu_seqlens_q, const int32_t* cu_seqlens_k,
                                    int batch, int64_t total_q, int64_t total_k, int heads_q,
                                    int heads_k, int head_dim, int max_seqlen_q, int max_seqlen_k,
                                    float softmax_scale, int causal, int32_t* status,
                                    void* stream) {
  return sparse_attn_fwd_impl(q, k, v, out, lse, fwd_mask, mask_words, cu_seqlens_q, cu_seqlens_k,
                              nullptr, nullptr, nullptr, 0, 0, batch, total_q, total_k, heads_q, heads_k,
                              head_dim, max_seqlen_q, max_seqlen_k, softmax_scale, causal, status, stream);
}

extern "C" int ifv2_sparse_attn_fwd_paged(const void* q, const void* k, const void* v, void* out,
                                          float* lse, const int64_t* fwd_mask, int mask_words,
                                          const int32_t* cu_seqlens_q, const int32_t* cu_seqlens_k,
                                          const int32_t* seqused_k, const int32_t* leftpad_k,
                                          const int32_t* block_table, int block_table_stride,
                                          int page_size, int batch, int64_t total_q, int64_t total_k,
                                          int heads_q, int heads_k, int head_dim, int max_seqlen_q,
                                          int max_seqlen_k, float softmax_scale, int causal,
                                          int32_t* status, void* stream) {
  return sparse_attn_fwd_impl(q, k, v, out, lse, fwd_mask, mask_words, cu_seqlens_q, cu_seqlens_k,
                              seqused_k, leftpad_k, block_table, block_table_stride, page_size, batch,
                              total_q, total_k, heads_q, heads_k, head_dim, max_seqlen_q, max_seqlen_k,
                              softmax_scale, causal, status, stream);
}
