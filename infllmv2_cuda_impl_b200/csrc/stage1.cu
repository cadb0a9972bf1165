// Stage-1 scorer: group-summed softmax probabilities of the queries against the compressed keys.
//
// One CTA owns 8 consecutive tokens x the 16 query heads of one KV head (128 rows, fetched by one
// 3-D TMA box from the caller's (token, head, d) layout) and streams 128-key tiles of the
// compressed keys twice:
//   pass 1:  S   = Q . Kc^T   (rows = query rows in TMEM lanes)   -> running max m and sum l per row
//   pass 2:  S^T = Kc . Q^T   (rows = keys in TMEM lanes)         -> p = exp2(s*c - m*c) / l,
//            and because the 16 heads of a token are now 16 adjacent COLUMNS of one thread's
//            row, the GQA group sum is an in-register sum: no shuffles, no shared memory.
// Both products use the same two swizzled shared-memory tiles with the operand roles swapped.
// The bf16 result row (Hk, token, key) is written straight from registers; columns past the
// last visible key are zero-filled, so the output needs no pre-zeroing, no slice and no NaN
// scrub.  Warp roles: warp 0 = TMA producer, warp 1 = MMA issuer, warps 2-5 = softmax.
#include "tc05.cuh"

namespace ifv2 {
namespace {

using namespace tc;

constexpr int kTokPerTile = 8;
constexpr int kThreads = 192;
constexpr int kKeysPerTile = 128;
constexpr uint32_t kHalfBytes = 128 * 128;    // 128 rows x 64 bf16
constexpr uint32_t kTmemCols = 256;

struct Stage1Params {
  __nv_bfloat16* out;
  const int32_t* cu_q;
  const int32_t* cu_k;
  int64_t total_q;
  int heads_q, heads_k;
  int max_seqlen_k;
  int64_t out_row_stride;
  float scale_log2;
  int causal;
  int32_t* status;
};

struct Smem {
  uint8_t q[2][kHalfBytes];          // [d half]
  uint8_t kc[2][2][kHalfBytes];      // [stage][d half]
  float2 stat[128];                  // per query row: {-m * scale_log2, 1 / l}
  uint64_t q_full, kc_full[2], kc_empty[2], acc_full[2], acc_empty[2];
  uint32_t tmem_base;
  int abort_flag;
};

// Number of leading compressed keys visible to local token i (C integer division, as the
// reference's device code): key j covers tokens [16j, 16j+32) and the pattern is aligned to the
// END of the keys when the query segment is shorter than the keys cover.
__device__ __forceinline__ int visible_limit(int i, int lq, int lc, int causal) {
  if (!causal) return lc;
  const int off = lc - (lq - 15) / 16;
  return min(lc, max(0, (i + 1) / 16 - 1 + off));
}

__global__ void __launch_bounds__(kThreads, 2)
stage1_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_kc,
              const Stage1Params p) {
  extern __shared__ uint8_t smem_raw[];
  Smem& sm = *reinterpret_cast<Smem*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                      ~(uintptr_t)1023);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int b = blockIdx.y, h = blockIdx.z;
  const int q0 = p.cu_q[b], lq = p.cu_q[b + 1] - q0;
  const int k0 = p.cu_k[b], lc = p.cu_k[b + 1] - k0;
  const int tok0 = ((int)gridDim.x - 1 - (int)blockIdx.x) * kTokPerTile;   // long tiles first
  if (tok0 >= lq) return;
  // an earlier CTA gave up on a wait: the launch is already failed, do not pile up more waits
  if (*reinterpret_cast<volatile int32_t*>(p.status) != 0) return;
  const int ntok = min(kTokPerTile, lq - tok0);
  const int lim_max = visible_limit(tok0 + ntok - 1, lq, lc, p.causal);    // limits grow with i
  const int n_tiles = (lim_max + kKeysPerTile - 1) / kKeysPerTile;
  const int n_steps = 2 * n_tiles;

  if (threadIdx.x == 0) {
    sm.abort_flag = 0;
    mbar_init(&sm.q_full, 1);
    for (int s = 0; s < 2; ++s) {
      mbar_init(&sm.kc_full[s], 1);
      mbar_init(&sm.kc_empty[s], 1);
      mbar_init(&sm.acc_full[s], 1);
      mbar_init(&sm.acc_empty[s], 128);
    }
    fence_barrier_init();
    prefetch_tensormap(&map_q);
    prefetch_tensormap(&map_kc);
  }
  if (warp == 1) {
    tmem_alloc(&sm.tmem_base, kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = sm.tmem_base;
  volatile int* abort_flag = &sm.abort_flag;

  if (warp == 0) {
    // ================================================================ TMA producer
    if (lane == 0 && n_steps > 0) {
      mbar_expect_tx(&sm.q_full, 2 * kHalfBytes);
      tma_load_3d(sm.q[0], &map_q, &sm.q_full, 0, h * kGroup, q0 + tok0);
      tma_load_3d(sm.q[1], &map_q, &sm.q_full, 64, h * kGroup, q0 + tok0);
      int issued = 0;
      for (int t = 0; t < n_steps; ++t) {
        const int s = t & 1, tile = (t < n_tiles) ? t : t - n_tiles;
        if (t >= 2 && !mbar_wait(&sm.kc_empty[s], (uint32_t)(((t >> 1) & 1) ^ 1), abort_flag,
                                 p.status, 41))
          break;
        mbar_expect_tx(&sm.kc_full[s], 2 * kHalfBytes);
        tma_load_3d(sm.kc[s][0], &map_kc, &sm.kc_full[s], 0, h, k0 + tile * kKeysPerTile);
        tma_load_3d(sm.kc[s][1], &map_kc, &sm.kc_full[s], 64, h, k0 + tile * kKeysPerTile);
        issued = t + 1;
      }
      if (*abort_flag) {
        mbar_wait_drain(&sm.q_full, 0);
        for (int j = max(0, issued - 2); j < issued; ++j)
          mbar_wait_drain(&sm.kc_full[j & 1], (uint32_t)((j >> 1) & 1));
      }
    }
  } else if (warp == 1) {
    // ================================================================ MMA issuer
    if (lane == 0 && n_steps > 0) {
      constexpr uint32_t idesc = umma_idesc_bf16(128, 128, false);
      const uint32_t q_addr = smem_u32(sm.q[0]);
      bool ok = mbar_wait(&sm.q_full, 0, abort_flag, p.status, 51);
      for (int t = 0; t < n_steps && ok; ++t) {
        const int s = t & 1;
        const uint32_t par = (uint32_t)((t >> 1) & 1);
        ok = mbar_wait(&sm.kc_full[s], par, abort_flag, p.status, 52);
        if (ok && t >= 2) ok = mbar_wait(&sm.acc_empty[s], par ^ 1u, abort_flag, p.status, 53);
        if (!ok) break;
        tc_fence_after();
        const uint32_t kc_addr = smem_u32(sm.kc[s][0]);
        const bool pass2 = t >= n_tiles;
#pragma unroll
        for (int kk = 0; kk < 8; ++kk) {
          const uint32_t off = (kk >> 2) * kHalfBytes + (kk & 3) * 32;
          const uint64_t dq = umma_desc_sw128(q_addr + off, 16, 1024);
          const uint64_t dk = umma_desc_sw128(kc_addr + off, 16, 1024);
          umma_ss(tmem + s * 128, pass2 ? dk : dq, pass2 ? dq : dk, idesc, kk > 0);
        }
        umma_commit(&sm.kc_empty[s]);
        umma_commit(&sm.acc_full[s]);
      }
    }
  } else {
    // ================================================================ softmax warps
    const int quad = warp & 3;
    const int r = quad * 32 + lane;                  // TMEM lane: pass 1 = query row, pass 2 = key
    const uint32_t lane_off = (uint32_t)(quad * 32) << 16;
    const int st = threadIdx.x - 64;                 // 0..127 among the softmax threads
    bool ok = true;

    // ---------------- pass 1: running max / sum of this thread's query row
    {
      const int tl = r >> 4;
      const int lim_row = (tl < ntok) ? visible_limit(tok0 + tl, lq, lc, p.causal) : 0;
      float m = -INFINITY, l = 0.f;
      for (int t = 0; t < n_tiles; ++t) {
        const int s = t & 1;
        ok = __all_sync(0xFFFFFFFFu, mbar_wait(&sm.acc_full[s], (uint32_t)((t >> 1) & 1),
                                               abort_flag, p.status, 61));
        if (!ok) break;
        tc_fence_after();
        const int lim = min(max(lim_row - t * kKeysPerTile, 0), kKeysPerTile);
#pragma unroll 1
        for (int c0 = 0; c0 < 128; c0 += 64) {
          uint32_t raw[2][32];
          tmem_ld32(tmem + lane_off + s * 128 + c0, raw[0]);
          tmem_ld32(tmem + lane_off + s * 128 + c0 + 32, raw[1]);
          tmem_wait_ld();
          float mx = -INFINITY;
#pragma unroll
          for (int c = 0; c < 64; ++c) {
            float x = __uint_as_float(raw[c >> 5][c & 31]);
            x = (c0 + c < lim) ? x : -INFINITY;
            raw[c >> 5][c & 31] = __float_as_uint(x);
            mx = fmaxf(mx, x);
          }
          if (mx > -INFINITY) {
            const float m_new = fmaxf(m, mx);
            const float neg = -m_new * p.scale_log2;
            float sum = 0.f;
#pragma unroll
            for (int c = 0; c < 64; ++c)
              sum += exp2f(fmaf(__uint_as_float(raw[c >> 5][c & 31]), p.scale_log2, neg));
            l = l * exp2f((m - m_new) * p.scale_log2) + sum;     // m = -inf -> factor 0, l was 0
            m = m_new;
          }
        }
        tc_fence_before();
        mbar_arrive(&sm.acc_empty[s]);
      }
      sm.stat[r] = (l > 0.f) ? make_float2(-m * p.scale_log2, 1.f / l) : make_float2(0.f, 0.f);
    }
    asm volatile("bar.sync 1, 128;" ::: "memory");    // the four softmax warps only

    // ---------------- pass 2: this thread's key against all 128 query rows
    if (ok) {
      int lim_tok[kTokPerTile];
#pragma unroll
      for (int t8 = 0; t8 < kTokPerTile; ++t8)
        lim_tok[t8] = (t8 < ntok) ? visible_limit(tok0 + t8, lq, lc, p.causal) : 0;
      __nv_bfloat16* out_base =
          p.out + ((int64_t)h * p.total_q + q0 + tok0) * p.out_row_stride;
      for (int t = n_tiles; t < n_steps; ++t) {
        const int s = t & 1;
        ok = __all_sync(0xFFFFFFFFu, mbar_wait(&sm.acc_full[s], (uint32_t)((t >> 1) & 1),
                                               abort_flag, p.status, 62));
        if (!ok) break;
        tc_fence_after();
        const int key = (t - n_tiles) * kKeysPerTile + r;
#pragma unroll
        for (int c0 = 0; c0 < 128; c0 += 32) {          // 32 columns = 2 tokens x 16 heads
          uint32_t raw[32];
          tmem_ld32(tmem + lane_off + s * 128 + c0, raw);
          tmem_wait_ld();
#pragma unroll
          for (int half = 0; half < 2; ++half) {
            const int t8 = (c0 >> 4) + half;
            float acc = 0.f;
#pragma unroll
            for (int g = 0; g < 16; ++g) {
              const float2 st2 = sm.stat[c0 + half * 16 + g];
              acc += exp2f(fmaf(__uint_as_float(raw[half * 16 + g]), p.scale_log2, st2.x)) * st2.y;
            }
            if (t8 < ntok && key < p.max_seqlen_k)
              out_base[(int64_t)t8 * p.out_row_stride + key] =
                  __float2bfloat16_rn(key < lim_tok[t8] ? acc : 0.f);
          }
        }
        tc_fence_before();
        mbar_arrive(&sm.acc_empty[s]);
      }
      // columns past the last tile are zero (rows are 16-byte aligned: stride % 8 == 0)
      const int first = n_tiles * kKeysPerTile;
      if (ok && first < p.max_seqlen_k) {
        const int vec_per_row = (p.max_seqlen_k - first + 7) / 8;   // may spill into row padding
        const uint4 z = make_uint4(0u, 0u, 0u, 0u);
        for (int t8 = 0; t8 < ntok; ++t8) {
          uint4* dst = reinterpret_cast<uint4*>(out_base + (int64_t)t8 * p.out_row_stride + first);
          for (int i = st; i < vec_per_row; i += 128) dst[i] = z;
        }
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem, kTmemCols);
}

}  // namespace
}  // namespace ifv2

using namespace ifv2;

extern "C" int ifv2_stage1_scores(const void* q, const void* kc, void* out,
                                  const int32_t* cu_seqlens_q, const int32_t* cu_seqlens_k,
                                  int batch, int64_t total_q, int64_t total_c, int heads_q,
                                  int heads_k, int head_dim, int max_seqlen_q, int max_seqlen_k,
                                  int64_t out_row_stride, float softmax_scale, int causal,
                                  int32_t* status, void* stream) {
  IFV2_REQUIRE(head_dim == kHeadDim, IFV2_ERR_UNSUPPORTED,
               "stage1_scores: head_dim %d not supported (only 128, as in the reference build)",
               head_dim);
  IFV2_REQUIRE(heads_k >= 1 && heads_q == heads_k * kGroup, IFV2_ERR_UNSUPPORTED,
               "stage1_scores: heads_q (%d) must be 16 x heads_k (%d)", heads_q, heads_k);
  IFV2_REQUIRE(batch >= 1 && total_q >= 0 && total_c >= 0 && max_seqlen_q >= 0 && max_seqlen_k >= 0,
               IFV2_ERR_INVALID_ARG, "stage1_scores: negative size or batch < 1");
  if (total_q == 0 || max_seqlen_q == 0 || max_seqlen_k == 0) return IFV2_OK;
  IFV2_REQUIRE(q && out && cu_seqlens_q && cu_seqlens_k && status && (kc || total_c == 0),
               IFV2_ERR_INVALID_ARG, "stage1_scores: null pointer");
  IFV2_REQUIRE(out_row_stride >= ((max_seqlen_k + 7) / 8) * 8 && out_row_stride % 8 == 0,
               IFV2_ERR_INVALID_ARG,
               "stage1_scores: out_row_stride (%lld) must be a multiple of 8 and >= max_seqlen_k "
               "rounded up to 8", (long long)out_row_stride);
  IFV2_REQUIRE(reinterpret_cast<uintptr_t>(out) % 16 == 0, IFV2_ERR_INVALID_ARG,
               "stage1_scores: out must be 16-byte aligned");
  IFV2_REQUIRE(total_q <= INT32_MAX && total_c <= INT32_MAX, IFV2_ERR_TOO_LARGE,
               "stage1_scores: more than 2^31-1 rows");
  IFV2_REQUIRE(batch <= 65535 && heads_k <= 65535, IFV2_ERR_TOO_LARGE,
               "stage1_scores: batch or heads_k > 65535");

  CUtensorMap map_q, map_kc;
  int rc = make_tensor_map_bf16_3d(&map_q, q, kHeadDim, heads_q, total_q, kHeadDim * 2,
                                   (uint64_t)heads_q * kHeadDim * 2, 64, kGroup, kTokPerTile);
  if (rc) return rc;
  // an empty key tensor still needs a valid map: point it at q, no tile is ever fetched
  rc = make_tensor_map_bf16_3d(&map_kc, total_c > 0 ? kc : q, kHeadDim, heads_k,
                               total_c > 0 ? total_c : 1, kHeadDim * 2,
                               (uint64_t)heads_k * kHeadDim * 2, 64, 1, kKeysPerTile);
  if (rc) return rc;

  Stage1Params p;
  p.out = static_cast<__nv_bfloat16*>(out);
  p.cu_q = cu_seqlens_q;
  p.cu_k = cu_seqlens_k;
  p.total_q = total_q;
  p.heads_q = heads_q;
  p.heads_k = heads_k;
  p.max_seqlen_k = max_seqlen_k;
  p.out_row_stride = out_row_stride;
  p.scale_log2 = softmax_scale * 1.4426950408889634f;
  p.causal = causal ? 1 : 0;
  p.status = status;

  const size_t smem = sizeof(Smem) + 1024;
  cudaError_t e =
      cudaFuncSetAttribute(stage1_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return set_error((int)e, "stage1_scores: %s", cudaGetErrorString(e));
  dim3 grid((max_seqlen_q + kTokPerTile - 1) / kTokPerTile, batch, heads_k);
  stage1_kernel<<<grid, kThreads, smem, (cudaStream_t)stream>>>(map_q, map_kc, p);
  return check_launch("stage1_scores");
}
