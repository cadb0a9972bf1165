// Stage-1 scorer for decode: ONE query token per sequence against all of its compressed keys.
//
// The 16 query heads of a KV head are one mma.sync M tile and the work is HBM-bound (every
// compressed key is read and used by 16 rows), so the general 128-row tcgen05 kernel, which gives
// a (sequence, KV head) pair to a single CTA, is the wrong tool: here the keys of a pair are cut
// into chunks of 512 and every chunk gets a CTA (4 warps, 32-key units through a cp.async double
// buffer, ldmatrix + mma.sync m16n8k16).  A softmax over all keys needs two sweeps:
//   kernel 1: per chunk and head the running (max, sum) of exp2(c*s)      -> stats workspace
//   kernel 2: merge the chunk stats of the pair, recompute the products, p = exp2(c*s - c*m)/l,
//             sum the 16 heads with warp shuffles, write the bf16 score row (0 where invisible,
//             0 up to max_seqlen_k past the last key)
// The keys are read twice; kernel 2 runs over the grid in reverse so that its first reads hit
// what kernel 1 left in L2.  Output layout and values are those of the general kernel (ifv2_stage1_scores).
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
  float2* stats;                 // (batch, heads_k, chunks, 16): (max in log2 units, sum)
  int batch, heads_q, heads_k, chunks, max_seqlen_k, causal;
  int64_t row_stride;
  float scale_log2;
};

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

// kPass 1: chunk statistics.  kPass 2: normalised, head-summed scores.
template <int kPass>
__global__ void __launch_bounds__(kThreads) stage1_decode_kernel(const DecodeS1Params p) {
  extern __shared__ __align__(128) uint8_t smem[];
  __shared__ float2 warp_stat[kWarps][16];
  __shared__ float row_const[16];                  // pass 2: -(m + log2 l) per head, log2 units
  // Kernel 2 walks the grid backwards: what kernel 1 read last is still in L2 when kernel 2 starts
  // there, so only the part of the key set that does not fit L2 is fetched from DRAM twice.
  const int chunk = (kPass == 2) ? (int)(gridDim.x - 1 - blockIdx.x) : (int)blockIdx.x;
  const int h = (kPass == 2) ? (int)(gridDim.y - 1 - blockIdx.y) : (int)blockIdx.y;
  const int b = (kPass == 2) ? (int)(gridDim.z - 1 - blockIdx.z) : (int)blockIdx.z;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t = lane & 3;
  const int k0 = p.cu_k[b], lc = p.cu_k[b + 1] - k0;
  const int lim = decode_limit(lc, p.causal);
  const int c0 = chunk * kChunk;                   // first key of this CTA
  float2* my_stats = p.stats + (((int64_t)b * p.heads_k + h) * p.chunks + chunk) * 16;
  __nv_bfloat16* out_row = p.out + ((int64_t)h * p.batch + b) * p.row_stride;

  if (c0 >= lim) {                                 // nothing visible in this chunk
    if (kPass == 1) {
      if (threadIdx.x < 16) my_stats[threadIdx.x] = make_float2(-INFINITY, 0.f);
    } else {
      for (int i = c0 + threadIdx.x; i < min(c0 + kChunk, p.max_seqlen_k); i += kThreads)
        out_row[i] = __float2bfloat16_rn(0.f);
    }
    return;
  }

  if (kPass == 2) {                                // merge the statistics of every chunk of the pair
    if (threadIdx.x < 16) {
      const float2* st = p.stats + ((int64_t)b * p.heads_k + h) * p.chunks * 16 + threadIdx.x;
      float m = -INFINITY;
      for (int c = 0; c < p.chunks; ++c) m = fmaxf(m, st[c * 16].x);
      float l = 0.f;
      for (int c = 0; c < p.chunks; ++c) {
        const float2 v = st[c * 16];
        if (v.x > -INFINITY) l += v.y * exp2f(v.x - m);
      }
      row_const[threadIdx.x] = (l > 0.f) ? -(m + log2f(l)) : -INFINITY;
    }
    __syncthreads();
  }

  uint32_t qf[8][4];
  load_q_fragments(qf, p.q + ((int64_t)b * p.heads_q + h * kGroup) * kHeadDim, lane);
  const float rc0 = (kPass == 2) ? row_const[g] : 0.f, rc1 = (kPass == 2) ? row_const[g + 8] : 0.f;

  uint8_t* tiles = smem + warp * kWarpSmem;
  const int64_t row_stride = (int64_t)p.heads_k * kHeadDim;
  const __nv_bfloat16* kbase = p.kc + (int64_t)k0 * row_stride + (int64_t)h * kHeadDim;
  // this warp's units: keys c0 + (warp * kUnitsPerWarp + u) * 32
  const int w0 = c0 + warp * kUnitsPerWarp * kUnit;
  float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;

  if (w0 < lim) load_tile(tiles, kbase + (int64_t)w0 * row_stride, row_stride, lim - w0, lane);
  cp_async_commit();
#pragma unroll 1
  for (int u = 0; u < kUnitsPerWarp; ++u) {
    const int key0 = w0 + u * kUnit;
    uint8_t* k_tile = tiles + (u & 1) * kUnit * 256;
    const int key_next = key0 + kUnit;
    if (u + 1 < kUnitsPerWarp && key_next < lim)
      load_tile(tiles + ((u + 1) & 1) * kUnit * 256, kbase + (int64_t)key_next * row_stride, row_stride,
                lim - key_next, lane);
    cp_async_commit();
    if (key0 >= lim) {                             // nothing visible in this unit
      if (kPass == 2) {
        for (int i = key0 + lane; i < min(key0 + kUnit, p.max_seqlen_k); i += 32)
          out_row[i] = __float2bfloat16_rn(0.f);
      }
      cp_async_wait<0>();
      continue;
    }
    cp_async_wait<1>();
    __syncwarp();
    float s[kUnit / 8][4];
    unit_scores(s, k_tile, qf, key0, lim, p.scale_log2, lane);
    __syncwarp();
    if (kPass == 1) {
      float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
      for (int nt = 0; nt < kUnit / 8; ++nt) {
        mx0 = fmaxf(mx0, fmaxf(s[nt][0], s[nt][1]));
        mx1 = fmaxf(mx1, fmaxf(s[nt][2], s[nt][3]));
      }
      mx0 = fmaxf(mx0, __shfl_xor_sync(0xFFFFFFFFu, mx0, 1));
      mx0 = fmaxf(mx0, __shfl_xor_sync(0xFFFFFFFFu, mx0, 2));
      mx1 = fmaxf(mx1, __shfl_xor_sync(0xFFFFFFFFu, mx1, 1));
      mx1 = fmaxf(mx1, __shfl_xor_sync(0xFFFFFFFFu, mx1, 2));
      const float mn0 = fmaxf(m0, mx0), mn1 = fmaxf(m1, mx1);       // finite: the unit has a visible key
      float sum0 = 0.f, sum1 = 0.f;
#pragma unroll
      for (int nt = 0; nt < kUnit / 8; ++nt) {
        sum0 += exp2f(s[nt][0] - mn0) + exp2f(s[nt][1] - mn0);
        sum1 += exp2f(s[nt][2] - mn1) + exp2f(s[nt][3] - mn1);
      }
      l0 = l0 * ((m0 == -INFINITY) ? 0.f : exp2f(m0 - mn0)) + sum0;
      l1 = l1 * ((m1 == -INFINITY) ? 0.f : exp2f(m1 - mn1)) + sum1;
      m0 = mn0;
      m1 = mn1;
    } else {
      // p summed over this lane's two heads, then over the 8 lane groups (heads g and g + 8)
      float v[kUnit / 8][2];
#pragma unroll
      for (int nt = 0; nt < kUnit / 8; ++nt) {
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          float x = exp2f(s[nt][e] + rc0) + exp2f(s[nt][2 + e] + rc1);   // exp2(-inf) = 0 when invisible
          x += __shfl_xor_sync(0xFFFFFFFFu, x, 4);
          x += __shfl_xor_sync(0xFFFFFFFFu, x, 8);
          x += __shfl_xor_sync(0xFFFFFFFFu, x, 16);
          v[nt][e] = x;
        }
      }
      if (g == 0) {
#pragma unroll
        for (int nt = 0; nt < kUnit / 8; ++nt) {
          const int key = key0 + nt * 8 + 2 * t;
          if (key + 1 < p.max_seqlen_k) {
            *reinterpret_cast<__nv_bfloat162*>(out_row + key) = __floats2bfloat162_rn(v[nt][0], v[nt][1]);
          } else if (key < p.max_seqlen_k) {
            out_row[key] = __float2bfloat16_rn(v[nt][0]);
          }
        }
      }
    }
  }
  cp_async_wait<0>();

  if (kPass == 1) {
    l0 += __shfl_xor_sync(0xFFFFFFFFu, l0, 1);
    l0 += __shfl_xor_sync(0xFFFFFFFFu, l0, 2);
    l1 += __shfl_xor_sync(0xFFFFFFFFu, l1, 1);
    l1 += __shfl_xor_sync(0xFFFFFFFFu, l1, 2);
    if (t == 0) {
      warp_stat[warp][g] = make_float2(m0, l0);
      warp_stat[warp][g + 8] = make_float2(m1, l1);
    }
    __syncthreads();
    if (threadIdx.x < 16) {
      float m = -INFINITY;
      for (int w = 0; w < kWarps; ++w) m = fmaxf(m, warp_stat[w][threadIdx.x].x);
      float l = 0.f;
      for (int w = 0; w < kWarps; ++w) {
        const float2 v = warp_stat[w][threadIdx.x];
        if (v.x > -INFINITY) l += v.y * exp2f(v.x - m);
      }
      my_stats[threadIdx.x] = make_float2(m, l);
    }
  }
}

}  // namespace
}  // namespace ifv2

using namespace ifv2;

extern "C" int64_t ifv2_stage1_decode_workspace_bytes(int batch, int heads_k, int max_seqlen_k) {
  if (batch < 0 || heads_k < 0 || max_seqlen_k < 0) return 0;
  const int64_t chunks = (max_seqlen_k + kChunk - 1) / kChunk;
  return (int64_t)batch * heads_k * (chunks > 0 ? chunks : 1) * 16 * (int64_t)sizeof(float2) + 256;
}

extern "C" int ifv2_stage1_decode_scores(const void* q, const void* kc, void* out,
                                         const int32_t* cu_seqlens_k, int batch, int64_t total_c,
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
                   reinterpret_cast<uintptr_t>(workspace) % 8 == 0,
               IFV2_ERR_INVALID_ARG, "stage1_decode_scores: workspace too small or misaligned");
  IFV2_REQUIRE(batch <= 65535 && heads_k <= 65535 && total_c <= INT32_MAX, IFV2_ERR_TOO_LARGE,
               "stage1_decode_scores: batch, heads_k or key count too large");
  DecodeS1Params p;
  p.q = static_cast<const __nv_bfloat16*>(q);
  p.kc = static_cast<const __nv_bfloat16*>(kc);
  p.out = static_cast<__nv_bfloat16*>(out);
  p.cu_k = cu_seqlens_k;
  p.stats = static_cast<float2*>(workspace);
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
  cudaError_t e = cudaFuncSetAttribute(stage1_decode_kernel<1>,
                                       cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e == cudaSuccess)
    e = cudaFuncSetAttribute(stage1_decode_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             (int)smem);
  if (e != cudaSuccess) return set_error((int)e, "stage1_decode_scores: %s", cudaGetErrorString(e));
  const dim3 grid(p.chunks, heads_k, batch);
  stage1_decode_kernel<1><<<grid, kThreads, smem, st>>>(p);
  int rc = check_launch("stage1_decode_stats");
  if (rc) return rc;
  stage1_decode_kernel<2><<<grid, kThreads, smem, st>>>(p);
  return check_launch("stage1_decode_scores");
}
