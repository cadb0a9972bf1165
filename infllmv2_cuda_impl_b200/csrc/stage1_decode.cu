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

namespace ifv2 {
namespace {

using namespace mmasync;

constexpr int kWarps = 4;
constexpr int kThreads = kWarps * 32;
constexpr int kChunk = 512;                       // keys per CTA
constexpr int kUnitsPerWarp = kChunk / kUnit / kWarps;
constexpr int kWarpSmem = 2 * kUnit * 256;        // two K tiles per warp (double buffer)
constexpr float kLog2e = 1.4426950408889634f;

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
  if (threadIdx.x < 16) {
    const float2* st = p.stats + pair * p.chunks * 16 + threadIdx.x;
    float m = -INFINITY;
    for (int c = 0; c < p.chunks; ++c) m = fmaxf(m, st[c * 16].x);
    float l = 0.f;
    for (int c = 0; c < p.chunks; ++c) {
      const float2 v = st[c * 16];
      if (v.x > -INFINITY) l += v.y * exp2f(v.x - m);
    }
    const float mine = st[chunk * 16].x;
    weight[threadIdx.x] = (l > 0.f) ? exp2f(mine - m) / l : 0.f;
  }
  __syncthreads();
  const __nv_bfloat16* e = p.e + pair * 16 * p.e_stride;
  for (int i = c0 + 2 * threadIdx.x; i < end; i += 2 * kThreads) {
    float a0 = 0.f, a1 = 0.f;
    if (i < lim) {
#pragma unroll
      for (int r = 0; r < 16; ++r) {
        const float2 v = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(e + r * p.e_stride + i));
        a0 += v.x * weight[r];
        a1 += v.y * weight[r];
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

extern "C" int ifv2_stage1_decode_scores(const void* q, const void* kc, void* out,
                                         const int32_t* cu_seqlens_k, const int32_t* seqused_k,
                                         int batch, int64_t total_c,
                                         int heads_q, int heads_k, int head_dim, int max_seqlen_k,
                                         int64_t out_row_stride, float softmax_scale, int causal,
                                         void* workspace, int64_t workspace_bytes, void* stream) {
  IFV2_REQUIRE(head_dim == kHeadDim, IFV2_ERR_UNSUPPORTED,
               "stage1_decode_scores: head_dim %d not supported (only 128)", head_dim);
  IFV2_REQUIRE(heads_k >= 1 && heads_q == heads_k * kGroup, IFV2_ERR_UNSUPPORTED,
               "stage1_decode_scores: heads_q (%d) must be 16 x heads_k (%d)", heads_q, heads_k);
  IFV2_REQUIRE(batch >= 0 && total_c >= 0 && max_seqlen_k >= 0, IFV2_ERR_INVALID_ARG,
               "stage1_decode_scores: negative size");
  if (batch == 0 || max_seqlen_k == 0) return IFV2_OK;
  IFV2_REQUIRE(softmax_scale > 0.f, IFV2_ERR_INVALID_ARG, "stage1_decode_scores: softmax_scale must be > 0");
  IFV2_REQUIRE(q && out && cu_seqlens_k && workspace && (kc || total_c == 0), IFV2_ERR_INVALID_ARG,
               "stage1_decode_scores: null pointer");
  IFV2_REQUIRE(out_row_stride >= max_seqlen_k && out_row_stride % 2 == 0 &&
                   reinterpret_cast<uintptr_t>(out) % 4 == 0,
               IFV2_ERR_INVALID_ARG, "stage1_decode_scores: out_row_stride must be even and >= max_seqlen_k");
  IFV2_REQUIRE(workspace_bytes >= ifv2_stage1_decode_workspace_bytes(batch, heads_k, max_seqlen_k) &&
                   reinterpret_cast<uintptr_t>(workspace) % 16 == 0,
               IFV2_ERR_INVALID_ARG, "stage1_decode_scores: workspace too small or misaligned");
  IFV2_REQUIRE(batch <= 65535 && heads_k <= 65535 && total_c <= INT32_MAX, IFV2_ERR_TOO_LARGE,
               "stage1_decode_scores: batch, heads_k or key count too large");
  DecodeS1Params p;
  p.q = static_cast<const __nv_bfloat16*>(q);
  p.kc = static_cast<const __nv_bfloat16*>(kc);
  p.out = static_cast<__nv_bfloat16*>(out);
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
  p.chunks = (max_seqlen_k + kChunk - 1) / kChunk;
  p.max_seqlen_k = max_seqlen_k;
  p.causal = causal ? 1 : 0;
  p.row_stride = out_row_stride;
  p.scale_log2 = softmax_scale * kLog2e;
  const size_t smem = (size_t)kWarps * kWarpSmem;
  cudaStream_t st = (cudaStream_t)stream;
  cudaError_t e = cudaFuncSetAttribute(stage1_decode_scores_kernel,
                                       cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return set_error((int)e, "stage1_decode_scores: %s", cudaGetErrorString(e));
  const dim3 grid(p.chunks, heads_k, batch);
  stage1_decode_scores_kernel<<<grid, kThreads, smem, st>>>(p);
  int rc = check_launch("stage1_decode_scores");
  if (rc) return rc;
  stage1_decode_normalise_kernel<<<grid, kThreads, 0, st>>>(p);
  return check_launch("stage1_decode_normalise");
}
