// Stage-1 scorer for decode: ONE query token per sequence against all of its compressed keys.
//
// The 16 query heads of a KV head are one mma.sync M tile and the work is HBM-bound (every
// compressed key is read and used by 16 rows), so the general 128-row tcgen05 kernel, which gives
// a (sequence, KV head) pair to a single CTA, is the wrong tool: here the keys of a pair are cut
// into chunks of 512 and every chunk gets a CTA (4 warps, 32-key units through a cp.async double
// buffer, ldmatrix + mma.sync m16n8k16).  A softmax over all keys needs the maximum and sum of
// the whole row before any score can be normalised; instead of reading the keys twice,
//   kernel 1 writes e = exp2(c*s - chunk max) per head as bf16 (32 bytes per key, an eighth of
//            the key row) plus the per-head (max, sum) of the chunk, and
//   kernel 2 merges the chunk statistics of the pair and forms the head-summed scores from e
//            (0 where invisible, 0 up to max_seqlen_k past the last key).
// Output layout and values are those of the general kernel (ifv2_stage1_scores); e carries 8
// mantissa bits, like the bf16 result it ends up in.
#include "mma_sync.cuh"
#include "decode_select.cuh"

namespace ifv2 {
namespace {

using namespace mmasync;

constexpr int kWarps = 4;
constexpr int kThreads = kWarps * 32;
constexpr int kChunk = 512;                       // keys per CTA
constexpr int kUnitsPerWarp = kChunk / kUnit / kWarps;
constexpr int kWarpSmem = 2 * kUnit * 256;        // two K tiles per warp (double buffer)
constexpr float kLog2e = 1.4426950408889634f;
constexpr int kMaxChunksShared = 64;              // chunk statistics staged in shared memory up to here

struct DecodeS1Params {
  const __nv_bfloat16* q;        // (batch, heads_q, 128): one token per sequence
  const __nv_bfloat16* kc;       // (total_c, heads_k, 128)
  __nv_bfloat16* out;            // (heads_k, batch, row_stride)
  const int32_t* cu_k;           // (batch + 1)
  const int32_t* seqused_k;      // (batch) keys in use per sequence, or null = all of cu_k's extent
  float2* stats;                 // (batch, heads_k, chunks, 16): (max in log2 units, sum of e)
  __nv_bfloat16* e;              // (batch, heads_k, 16, e_stride): exp2(score - chunk max)
  int64_t e_stride;              // chunks * 512
  int batch, heads_q, heads_k, chunks, max_seqlen_k, causal;
  int64_t row_stride;
  float scale_log2;
};

__device__ __forceinline__ int used_keys(const DecodeS1Params& p, int b) {
  const int extent = p.cu_k[b + 1] - p.cu_k[b];
  return p.seqused_k ? max(0, min(p.seqused_k[b], extent)) : extent;
}

// keys visible to the single query token (same rule as the general kernel with Lq = 1)
__device__ __forceinline__ int decode_limit(int lc, int causal) {
  if (!causal) return lc;
  return min(lc, max(0, (0 + 1) / 16 - 1 + lc - (1 - 15) / 16));
}

// S (16 heads x 32 keys, log2 units, -inf where invisible) of one unit from its K tile
__device__ __forceinline__ void unit_scores(float (&s)[kUnit / 8][4], uint8_t* k_tile,
                                            const uint32_t (&qf)[8][4], int key0, int lim,
                                            float scale_log2, int lane) {
  const int t = lane & 3;
#pragma unroll
  for (int nt = 0; nt < kUnit / 8; ++nt) s[nt][0] = s[nt][1] = s[nt][2] = s[nt][3] = 0.f;
#pragma unroll
  for (int nt = 0; nt < kUnit / 8; ++nt) {
#pragma unroll
    for (int kp = 0; kp < 4; ++kp) {        // two k-steps (32 d) per ldmatrix.x4
      uint32_t bf[4];
      ldmatrix_x4(bf, tile_addr(k_tile, nt * 8 + (lane & 7), kp * 4 + (lane >> 3)));
      mma_bf16(s[nt], qf[2 * kp], bf[0], bf[1]);
      mma_bf16(s[nt], qf[2 * kp + 1], bf[2], bf[3]);
    }
  }
#pragma unroll
  for (int nt = 0; nt < kUnit / 8; ++nt) {
#pragma unroll
    for (int e = 0; e < 2; ++e) {
      const bool vis = key0 + nt * 8 + 2 * t + e < lim;      // rows past `lim` were never fetched
      s[nt][e] = vis ? s[nt][e] * scale_log2 : -INFINITY;
      s[nt][2 + e] = vis ? s[nt][2 + e] * scale_log2 : -INFINITY;
    }
  }
}

__device__ __forceinline__ void load_q_fragments(uint32_t (&qf)[8][4], const __nv_bfloat16* q_row0,
                                                 int lane) {
  const int g = lane >> 2, t = lane & 3;
  const __nv_bfloat16* q0 = q_row0 + g * kHeadDim;
  const __nv_bfloat16* q1 = q0 + 8 * kHeadDim;
#pragma unroll
  for (int ks = 0; ks < 8; ++ks) {
    qf[ks][0] = *reinterpret_cast<const uint32_t*>(q0 + ks * 16 + 2 * t);
    qf[ks][1] = *reinterpret_cast<const uint32_t*>(q1 + ks * 16 + 2 * t);
    qf[ks][2] = *reinterpret_cast<const uint32_t*>(q0 + ks * 16 + 8 + 2 * t);
    qf[ks][3] = *reinterpret_cast<const uint32_t*>(q1 + ks * 16 + 8 + 2 * t);
  }
}

// Kernel 1: one CTA per 512-key chunk of a (sequence, KV head) pair.  Every warp keeps the scores
// of its four 32-key units in registers, the CTA agrees on the per-head maximum of the chunk, and
// e = exp2(c*s - max) goes to the workspace as bf16 (head-major rows, so that lanes write
// contiguous keys) together with the per-head (max, sum e) of the chunk.
__global__ void __launch_bounds__(kThreads) stage1_decode_scores_kernel(const DecodeS1Params p) {
  extern __shared__ __align__(128) uint8_t smem[];
  __shared__ float warp_max[kWarps][16];
  __shared__ float warp_sum[kWarps][16];
  const int chunk = blockIdx.x, h = blockIdx.y, b = blockIdx.z;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t = lane & 3;
  const int k0 = p.cu_k[b], lc = used_keys(p, b);
  const int lim = decode_limit(lc, p.causal);
  const int c0 = chunk * kChunk;                   // first key of this CTA
  const int64_t pair = (int64_t)b * p.heads_k + h;
  float2* my_stats = p.stats + (pair * p.chunks + chunk) * 16;
  if (c0 >= lim) {                                 // nothing visible in this chunk (uniform)
    if (threadIdx.x < 16) my_stats[threadIdx.x] = make_float2(-INFINITY, 0.f);
    return;
  }
  uint32_t qf[8][4];
  load_q_fragments(qf, p.q + ((int64_t)b * p.heads_q + h * kGroup) * kHeadDim, lane);

  uint8_t* tiles = smem + warp * kWarpSmem;
  const int64_t row_stride = (int64_t)p.heads_k * kHeadDim;
  const __nv_bfloat16* kbase = p.kc + (int64_t)k0 * row_stride + (int64_t)h * kHeadDim;
  const int w0 = c0 + warp * kUnitsPerWarp * kUnit;     // this warp's keys: w0 .. w0 + 127
  float s[kUnitsPerWarp][kUnit / 8][4];
  float mx0 = -INFINITY, mx1 = -INFINITY;               // heads g and g + 8

  if (w0 < lim) load_tile(tiles, kbase + (int64_t)w0 * row_stride, row_stride, lim - w0, lane);
  cp_async_commit();
#pragma unroll
  for (int u = 0; u < kUnitsPerWarp; ++u) {
    const int key0 = w0 + u * kUnit;
    const int key_next = key0 + kUnit;
    if (u + 1 < kUnitsPerWarp && key_next < lim)
      load_tile(tiles + ((u + 1) & 1) * kUnit * 256, kbase + (int64_t)key_next * row_stride, row_stride,
                lim - key_next, lane);
    cp_async_commit();
    cp_async_wait<1>();
    __syncwarp();
    if (key0 < lim) {
      unit_scores(s[u], tiles + (u & 1) * kUnit * 256, qf, key0, lim, p.scale_log2, lane);
    } else {
#pragma unroll
      for (int nt = 0; nt < kUnit / 8; ++nt) s[u][nt][0] = s[u][nt][1] = s[u][nt][2] = s[u][nt][3] = -INFINITY;
    }
    __syncwarp();
#pragma unroll
    for (int nt = 0; nt < kUnit / 8; ++nt) {
      mx0 = fmaxf(mx0, fmaxf(s[u][nt][0], s[u][nt][1]));
      mx1 = fmaxf(mx1, fmaxf(s[u][nt][2], s[u][nt][3]));
    }
  }
  cp_async_wait<0>();
  mx0 = fmaxf(mx0, __shfl_xor_sync(0xFFFFFFFFu, mx0, 1));
  mx0 = fmaxf(mx0, __shfl_xor_sync(0xFFFFFFFFu, mx0, 2));
  mx1 = fmaxf(mx1, __shfl_xor_sync(0xFFFFFFFFu, mx1, 1));
  mx1 = fmaxf(mx1, __shfl_xor_sync(0xFFFFFFFFu, mx1, 2));
  if (t == 0) {
    warp_max[warp][g] = mx0;
    warp_max[warp][g + 8] = mx1;
  }
  __syncthreads();
  float m0 = -INFINITY, m1 = -INFINITY;                 // chunk maxima (finite: key c0 is visible)
#pragma unroll
  for (int w = 0; w < kWarps; ++w) {
    m0 = fmaxf(m0, warp_max[w][g]);
    m1 = fmaxf(m1, warp_max[w][g + 8]);
  }
  // e rows of this pair: (16 heads, e_stride keys), head-major
  __nv_bfloat16* e0 = p.e + (pair * 16 + g) * p.e_stride;
  __nv_bfloat16* e1 = e0 + 8 * p.e_stride;
  float l0 = 0.f, l1 = 0.f;
#pragma unroll
  for (int u = 0; u < kUnitsPerWarp; ++u) {
#pragma unroll
    for (int nt = 0; nt < kUnit / 8; ++nt) {
      const int key = w0 + u * kUnit + nt * 8 + 2 * t;   // even; the e rows are padded to the chunk
      const float a0 = exp2f(s[u][nt][0] - m0), a1 = exp2f(s[u][nt][1] - m0);
      const float b0 = exp2f(s[u][nt][2] - m1), b1 = exp2f(s[u][nt][3] - m1);
      l0 += a0 + a1;
      l1 += b0 + b1;
      *reinterpret_cast<__nv_bfloat162*>(e0 + key) = __floats2bfloat162_rn(a0, a1);
      *reinterpret_cast<__nv_bfloat162*>(e1 + key) = __floats2bfloat162_rn(b0, b1);
    }
  }
  l0 += __shfl_xor_sync(0xFFFFFFFFu, l0, 1);
  l0 += __shfl_xor_sync(0xFFFFFFFFu, l0, 2);
  l1 += __shfl_xor_sync(0xFFFFFFFFu, l1, 1);
  l1 += __shfl_xor_sync(0xFFFFFFFFu, l1, 2);
  if (t == 0) {
    warp_sum[warp][g] = l0;
    warp_sum[warp][g + 8] = l1;
  }
  __syncthreads();
  if (threadIdx.x < 16) {
    float m = -INFINITY, l = 0.f;
    for (int w = 0; w < kWarps; ++w) {
      m = fmaxf(m, warp_max[w][threadIdx.x]);
      l += warp_sum[w][threadIdx.x];
    }
    my_stats[threadIdx.x] = make_float2(m, l);
  }
}

// Kernel 2: merge the chunk statistics of the pair, then out[key] = sum over the 16 heads of
// e[head][key] * 2^(chunk max - max) / sum: 32 bytes read per key instead of the 256 of a key row.
__global__ void __launch_bounds__(kThreads) stage1_decode_normalise_kernel(const DecodeS1Params p) {
  __shared__ float weight[16];
  const int chunk = blockIdx.x, h = blockIdx.y, b = blockIdx.z;
  const int lc = used_keys(p, b);
  const int lim = decode_limit(lc, p.causal);
  const int c0 = chunk * kChunk;
  const int64_t pair = (int64_t)b * p.heads_k + h;
  __nv_bfloat16* out_row = p.out + ((int64_t)h * p.batch + b) * p.row_stride;
  const int end = min(c0 + kChunk, p.max_seqlen_k);
  if (c0 >= lim) {
    for (int i = c0 + threadIdx.x; i < end; i += kThreads) out_row[i] = __float2bfloat16_rn(0.f);
    return;
  }
  // all chunk statistics of the pair come in side by side, then 16 threads merge them
  __shared__ float2 stats_s[kMaxChunksShared][16];
  const float2* st_g = p.stats + pair * p.chunks * 16;
  const bool staged = p.chunks <= kMaxChunksShared;
  if (staged) {
    for (int i = threadIdx.x; i < p.chunks * 16; i += kThreads) stats_s[i >> 4][i & 15] = __ldg(st_g + i);
    __syncthreads();
  }
  if (threadIdx.x < 16) {
    const int hh = threadIdx.x;
    auto stat = [&](int c) -> float2 { return staged ? stats_s[c][hh] : st_g[c * 16 + hh]; };
    float m = -INFINITY;
    for (int c = 0; c < p.chunks; ++c) m = fmaxf(m, stat(c).x);
    float l = 0.f;
    for (int c = 0; c < p.chunks; ++c) {
      const float2 v = stat(c);
      if (v.x > -INFINITY) l += v.y * exp2f(v.x - m);
    }
    const float mine = stat(chunk).x;
    weight[hh] = (l > 0.f) ? exp2f(mine - m) / l : 0.f;
  }
  __syncthreads();
  const __nv_bfloat16* e = p.e + pair * 16 * p.e_stride;
  for (int i = c0 + 2 * threadIdx.x; i < end; i += 2 * kThreads) {
    float a0 = 0.f, a1 = 0.f;
    if (i < lim) {
#pragma unroll
      for (int r = 0; r < 16; ++r) {
        const float2 v = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(e + r * p.e_stride + i));
        a0 = fmaf(v.x, weight[r], a0);
        a1 = fmaf(v.y, weight[r], a1);
      }
      if (i + 1 >= lim) a1 = 0.f;
    }
    if (i + 1 < p.max_seqlen_k) {
      *reinterpret_cast<__nv_bfloat162*>(out_row + i) = __floats2bfloat162_rn(a0, a1);
    } else {
      out_row[i] = __float2bfloat16_rn(a0);
    }
  }
}

// Kernel 2, fused with the block selection: one CTA per (sequence, KV head) merges the chunk
// statistics, forms the pair's whole score row in shared memory (the values kernel 2 would write,
// bf16-rounded the same way) and goes straight on to max-pool, top-k and the packed block mask
// (dsel::select_row).  The score row never reaches HBM.
constexpr int kMaxChunks = 64;                    // 32768 compressed keys

struct DecodeSelectParams {
  DecodeS1Params s1;
  const int32_t* positions;     // (batch) position of the query token in its sequence
  unsigned long long* mask;     // (batch, heads_k, words)
  int32_t* topk_idx;            // (batch, heads_k, k) or null
  int block_size;
  int row_bytes;                // bytes of the score row in shared memory (a multiple of 16)
  dsel::Args a;
};

__global__ void __launch_bounds__(dsel::kThreads)
stage1_decode_select_kernel(const DecodeSelectParams q) {
  extern __shared__ __align__(16) uint8_t row_smem[];            // the score row, bf16
  __shared__ dsel::Smem sm;
  __shared__ float weight[kMaxChunks][16];
  __shared__ float2 stats_s[kMaxChunks][16];
  const DecodeS1Params& p = q.s1;
  const int h = blockIdx.x, b = blockIdx.y, tid = threadIdx.x;
  const int lc = used_keys(p, b);
  const int lim = decode_limit(lc, p.causal);
  const int64_t pair = (int64_t)b * p.heads_k + h;
  const int chunks_used = (lim + kChunk - 1) / kChunk;
  // the chunk statistics come in side by side (one trip to memory), then 16 threads merge them
  {
    const float2* st = p.stats + pair * p.chunks * 16;
    for (int i = tid; i < chunks_used * 16; i += dsel::kThreads) stats_s[i >> 4][i & 15] = __ldg(st + i);
  }
  __syncthreads();
  if (tid < 16) {
    float m = -INFINITY;
    for (int c = 0; c < chunks_used; ++c) m = fmaxf(m, stats_s[c][tid].x);
    float l = 0.f;
    for (int c = 0; c < chunks_used; ++c) {
      const float2 v = stats_s[c][tid];
      if (v.x > -INFINITY) l += v.y * exp2f(v.x - m);
    }
    for (int c = 0; c < chunks_used; ++c)
      weight[c][tid] = (l > 0.f) ? exp2f(stats_s[c][tid].x - m) / l : 0.f;
  }
  __syncthreads();
  __nv_bfloat16* row = reinterpret_cast<__nv_bfloat16*>(row_smem);
  // staging tile behind the row: 16 head rows x 256 vectors of 8 keys.  A thread copies the 16
  // vectors of its 8 keys with cp.async (all in flight at once, whatever the register budget) and
  // is the only reader of what it copied, so a wait on its own copies is all the ordering needed.
  uint4* tile = reinterpret_cast<uint4*>(row_smem + q.row_bytes);
  const __nv_bfloat16* e = p.e + pair * 16 * p.e_stride;
  const int n_vec = (lc + 7) / 8, n_vec_vis = (lim + 7) / 8;      // 8 keys per thread and trip
  for (int v0 = 0; v0 < n_vec; v0 += dsel::kThreads) {
    const int v = v0 + tid, i = v * 8;
    if (v < n_vec_vis) {
#pragma unroll
      for (int r = 0; r < 16; ++r) cp_async16(tile + r * dsel::kThreads + tid, e + r * p.e_stride + i);
    }
    cp_async_commit();
    cp_async_wait<0>();
    if (v >= n_vec) continue;
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    if (v < n_vec_vis) {
      const float* w = weight[i / kChunk];
#pragma unroll
      for (int r = 0; r < 16; ++r) {
        const uint4 raw = tile[r * dsel::kThreads + tid];
        const __nv_bfloat162* h2 = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float2 f = __bfloat1622float2(h2[j]);
          acc[2 * j] = fmaf(f.x, w[r], acc[2 * j]);
          acc[2 * j + 1] = fmaf(f.y, w[r], acc[2 * j + 1]);
        }
      }
    }
    uint4 out;
    __nv_bfloat162* o2 = reinterpret_cast<__nv_bfloat162*>(&out);
#pragma unroll
    for (int j = 0; j < 4; ++j)
      o2[j] = __floats2bfloat162_rn(i + 2 * j < lim ? acc[2 * j] : 0.f, i + 2 * j + 1 < lim ? acc[2 * j + 1] : 0.f);
    reinterpret_cast<uint4*>(row)[v] = out;
  }
  __syncthreads();
  dsel::select_row<__nv_bfloat16>(row, true, lc, q.positions[b] / q.block_size, q.a, sm,
                                  q.mask + pair * q.a.words,
                                  q.topk_idx ? q.topk_idx + pair * q.a.k : nullptr,
                                  q.positions[b] < q.a.dense_len);
}

}  // namespace
}  // namespace ifv2

using namespace ifv2;

extern "C" int64_t ifv2_stage1_decode_workspace_bytes(int batch, int heads_k, int max_seqlen_k) {
  if (batch < 0 || heads_k < 0 || max_seqlen_k < 0) return 0;
  const int64_t chunks = (max_seqlen_k + kChunk - 1) / kChunk > 0 ? (max_seqlen_k + kChunk - 1) / kChunk : 1;
  const int64_t stats = (int64_t)batch * heads_k * chunks * 16 * (int64_t)sizeof(float2);
  const int64_t e = (int64_t)batch * heads_k * 16 * chunks * kChunk * 2;
  return ((stats + 255) / 256) * 256 + e + 256;
}

static int fill_decode_params(DecodeS1Params& p, const char* what, const void* q, const void* kc,
                              const int32_t* cu_seqlens_k, const int32_t* seqused_k, int batch,
                              int64_t total_c, int heads_q, int heads_k, int head_dim,
                              int max_seqlen_k, float softmax_scale, int causal, void* workspace,
                              int64_t workspace_bytes) {
  IFV2_REQUIRE(head_dim == kHeadDim, IFV2_ERR_UNSUPPORTED, "%s: head_dim %d not supported (only 128)", what,
               head_dim);
  IFV2_REQUIRE(heads_k >= 1 && heads_q == heads_k * kGroup, IFV2_ERR_UNSUPPORTED,
               "%s: heads_q (%d) must be 16 x heads_k (%d)", what, heads_q, heads_k);
  IFV2_REQUIRE(batch >= 1 && total_c >= 0 && max_seqlen_k >= 1, IFV2_ERR_INVALID_ARG, "%s: bad size", what);
  IFV2_REQUIRE(softmax_scale > 0.f, IFV2_ERR_INVALID_ARG, "%s: softmax_scale must be > 0", what);
  IFV2_REQUIRE(q && cu_seqlens_k && workspace && (kc || total_c == 0), IFV2_ERR_INVALID_ARG,
               "%s: null pointer", what);
  IFV2_REQUIRE(workspace_bytes >= ifv2_stage1_decode_workspace_bytes(batch, heads_k, max_seqlen_k) &&
                   reinterpret_cast<uintptr_t>(workspace) % 16 == 0,
               IFV2_ERR_INVALID_ARG, "%s: workspace too small or misaligned", what);
  IFV2_REQUIRE(batch <= 65535 && heads_k <= 65535 && total_c <= INT32_MAX, IFV2_ERR_TOO_LARGE,
               "%s: batch, heads_k or key count too large", what);
  p.q = static_cast<const __nv_bfloat16*>(q);
  p.kc = static_cast<const __nv_bfloat16*>(kc);
  p.out = nullptr;
  p.cu_k = cu_seqlens_k;
  p.seqused_k = seqused_k;
  p.stats = static_cast<float2*>(workspace);
  const int64_t n_chunks = (max_seqlen_k + kChunk - 1) / kChunk;
  const int64_t stats_bytes = (((int64_t)batch * heads_k * n_chunks * 16 * (int64_t)sizeof(float2)) + 255) / 256 * 256;
  p.e = reinterpret_cast<__nv_bfloat16*>(static_cast<uint8_t*>(workspace) + stats_bytes);
  p.e_stride = n_chunks * kChunk;
  p.batch = batch;
  p.heads_q = heads_q;
  p.heads_k = heads_k;
  p.chunks = (int)n_chunks;
  p.max_seqlen_k = max_seqlen_k;
  p.causal = causal ? 1 : 0;
  p.row_stride = 0;
  p.scale_log2 = softmax_scale * kLog2e;
  return IFV2_OK;
}

static int launch_decode_scores(const DecodeS1Params& p, cudaStream_t st) {
  const size_t smem = (size_t)kWarps * kWarpSmem;
  cudaError_t e = cudaFuncSetAttribute(stage1_decode_scores_kernel,
                                       cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return set_error((int)e, "stage1_decode_scores: %s", cudaGetErrorString(e));
  stage1_decode_scores_kernel<<<dim3(p.chunks, p.heads_k, p.batch), kThreads, smem, st>>>(p);
  return check_launch("stage1_decode_scores");
}

extern "C" int ifv2_stage1_decode_scores(const void* q, const void* kc, void* out,
                                         const int32_t* cu_seqlens_k, const int32_t* seqused_k,
                                         int batch, int64_t total_c,
                                         int heads_q, int heads_k, int head_dim, int max_seqlen_k,
                                         int64_t out_row_stride, float softmax_scale, int causal,
                                         void* workspace, int64_t workspace_bytes, void* stream) {
  IFV2_REQUIRE(batch >= 0 && max_seqlen_k >= 0, IFV2_ERR_INVALID_ARG, "stage1_decode_scores: negative size");
  if (batch == 0 || max_seqlen_k == 0) return IFV2_OK;
  DecodeS1Params p;
  int rc = fill_decode_params(p, "stage1_decode_scores", q, kc, cu_seqlens_k, seqused_k, batch, total_c,
                              heads_q, heads_k, head_dim, max_seqlen_k, softmax_scale, causal, workspace,
                              workspace_bytes);
  if (rc) return rc;
  IFV2_REQUIRE(out != nullptr && out_row_stride >= max_seqlen_k && out_row_stride % 2 == 0 &&
                   reinterpret_cast<uintptr_t>(out) % 4 == 0,
               IFV2_ERR_INVALID_ARG, "stage1_decode_scores: out_row_stride must be even and >= max_seqlen_k");
  p.out = static_cast<__nv_bfloat16*>(out);
  p.row_stride = out_row_stride;
  cudaStream_t st = (cudaStream_t)stream;
  rc = launch_decode_scores(p, st);
  if (rc) return rc;
  stage1_decode_normalise_kernel<<<dim3(p.chunks, heads_k, batch), kThreads, 0, st>>>(p);
  return check_launch("stage1_decode_normalise");
}

extern "C" int ifv2_stage1_decode_select(const void* q, const void* kc, const int32_t* cu_seqlens_k,
                                         const int32_t* seqused_k, const int32_t* positions,
                                         int64_t* mask, int32_t* topk_idx, int batch, int64_t total_c,
                                         int heads_q, int heads_k, int head_dim, int max_seqlen_k,
                                         int n_blocks, int mask_words, int k, int local_blocks,
                                         int init_blocks, int block_size, int stride, int dense_len,
                                         float softmax_scale, int causal, void* workspace,
                                         int64_t workspace_bytes, void* stream) {
  IFV2_REQUIRE(batch >= 0 && max_seqlen_k >= 0 && n_blocks >= 0 && mask_words >= 0 && k >= 0 &&
                   local_blocks >= 0 && init_blocks >= 0,
               IFV2_ERR_INVALID_ARG, "stage1_decode_select: negative size");
  IFV2_REQUIRE(block_size >= 1 && stride >= 1 && block_size % stride == 0, IFV2_ERR_INVALID_ARG,
               "stage1_decode_select: block_size must be a multiple of the compression stride");
  IFV2_REQUIRE(n_blocks <= dsel::kMaxBlocks && mask_words <= dsel::kMaxBlocks / 64, IFV2_ERR_TOO_LARGE,
               "stage1_decode_select: more than %d blocks", dsel::kMaxBlocks);
  IFV2_REQUIRE(max_seqlen_k <= kMaxChunks * kChunk, IFV2_ERR_TOO_LARGE,
               "stage1_decode_select: more than %d compressed keys per sequence", kMaxChunks * kChunk);
  if (batch == 0 || mask_words == 0) return IFV2_OK;
  IFV2_REQUIRE(positions && mask, IFV2_ERR_INVALID_ARG, "stage1_decode_select: null pointer");
  IFV2_REQUIRE(max_seqlen_k >= 1, IFV2_ERR_INVALID_ARG,
               "stage1_decode_select: needs at least one compressed key (use ifv2_decode_select on an "
               "empty score row otherwise)");
  DecodeSelectParams sp;
  int rc = fill_decode_params(sp.s1, "stage1_decode_select", q, kc, cu_seqlens_k, seqused_k, batch, total_c,
                              heads_q, heads_k, head_dim, max_seqlen_k, softmax_scale, causal, workspace,
                              workspace_bytes);
  if (rc) return rc;
  sp.positions = positions;
  sp.mask = reinterpret_cast<unsigned long long*>(mask);
  sp.topk_idx = topk_idx;
  sp.block_size = block_size;
  sp.a = dsel::Args{n_blocks, mask_words, k, local_blocks, init_blocks, block_size / stride,
                    dense_len > 0 ? dense_len : 0};
  cudaStream_t st = (cudaStream_t)stream;
  rc = launch_decode_scores(sp.s1, st);
  if (rc) return rc;
  sp.row_bytes = ((max_seqlen_k + 7) / 8) * 16;
  const size_t smem = (size_t)sp.row_bytes + 16 * dsel::kThreads * sizeof(uint4);     // row + staging tile
  cudaError_t e = cudaFuncSetAttribute(stage1_decode_select_kernel,
                                       cudaFuncAttributeMaxDynamicSharedMemorySize, 128 * 1024);
  if (e != cudaSuccess) return set_error((int)e, "stage1_decode_select: %s", cudaGetErrorString(e));
  stage1_decode_select_kernel<<<dim3(heads_k, batch), dsel::kThreads, smem, st>>>(sp);
  return check_launch("stage1_decode_select");
}
