// Single-tile checks of the tcgen05 building blocks the attention kernels rely on: TMA tiles
// with 128-byte swizzle feeding K-major and MN-major shared-memory operands, an A operand held
// in TMEM, and TMEM load/store.  Each mode computes one small product that the test-suite
// compares with a plain matmul, so a wrong descriptor shows up here and not inside a pipeline.
#include "tc05.cuh"

namespace ifv2 {
namespace {

using namespace tc;

struct SelfTestParams {
  const __nv_bfloat16* a;   // modes 2, 4: A read with plain loads
  const __nv_bfloat16* b;   // mode 4: B read with plain loads
  float* d;                 // (128, n) fp32
  int mode;
  int32_t* status;
};

// mode 0: D(128x64)  = A(128x128, K-major) * B(64x128, K-major)^T      [the Q.K^T shape]
// mode 1: D(128x128) = A(128x64,  K-major) * Bt(64x128, MN-major)      [the P.V shape, P in smem]
// mode 2: D(128x128) = A(128x64 in TMEM)   * Bt(64x128, MN-major)      [the P.V shape, P in TMEM]
// mode 3: D(128x64)  = At(128x128, MN-major)^T * Bt(128x64, MN-major)  [the dO^T.P shape of the backward]
// mode 5: as mode 4 with the 32-byte swizzle
// mode 4: D(128x64)  = A(128x16) * B(64x16)^T, both K-major WITHOUT swizzle, written by threads
//                                                                        [the row-constant K step of stage 1]
__global__ void __launch_bounds__(128)
umma_selftest_kernel(const __grid_constant__ CUtensorMap map_a,
                     const __grid_constant__ CUtensorMap map_b, const SelfTestParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~(uintptr_t)1023);
  uint8_t* sA = smem;              // up to 32 KB
  uint8_t* sB = smem + 32768;      // up to 16 KB
  __shared__ uint64_t bar_load, bar_mma;
  __shared__ uint32_t tmem_base_slot;
  __shared__ int abort_flag;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    abort_flag = 0;
    mbar_init(&bar_load, 1);
    mbar_init(&bar_mma, 1);
    fence_barrier_init();
  }
  if (warp == 0) {
    tmem_alloc(&tmem_base_slot, 256);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = tmem_base_slot;
  const uint32_t tmem_d = tmem, tmem_a = tmem + 128;
  const int mode = p.mode;
  const bool sw32 = p.mode == 5;               // mode 5 = mode 4 with the 32-byte swizzle
  const int n = (mode == 0 || mode == 3 || mode == 4 || mode == 5) ? 64 : 128;
  if (sw32) {
    for (int i = threadIdx.x; i < 128 * 16; i += 128)
      *reinterpret_cast<__nv_bfloat16*>(sA + umma_sw32_off(i >> 4, i & 15)) = p.a[i];
    for (int i = threadIdx.x; i < 64 * 16; i += 128)
      *reinterpret_cast<__nv_bfloat16*>(sB + umma_sw32_off(i >> 4, i & 15)) = p.b[i];
    fence_proxy_async_smem();
  }
  if (mode == 4) {
    for (int i = threadIdx.x; i < 128 * 16; i += 128)
      *reinterpret_cast<__nv_bfloat16*>(sA + umma_noswz16_off(i >> 4, i & 15)) = p.a[i];
    for (int i = threadIdx.x; i < 64 * 16; i += 128)
      *reinterpret_cast<__nv_bfloat16*>(sB + umma_noswz16_off(i >> 4, i & 15)) = p.b[i];
    fence_proxy_async_smem();
  }

  if (mode == 2) {   // every thread stores its A row into TMEM as packed bf16 pairs
    uint32_t regs[32];
    const uint32_t* row = reinterpret_cast<const uint32_t*>(p.a + (size_t)threadIdx.x * 64);
#pragma unroll
    for (int j = 0; j < 32; ++j) regs[j] = row[j];
    tmem_st32(tmem_a + ((uint32_t)(warp * 32) << 16), regs);
    tmem_wait_st();
    tc_fence_before();
  }
  __syncthreads();

  if (warp == 0 && lane == 0) {
    tc_fence_after();
    if (mode == 4 || mode == 5) {
      mbar_arrive(&bar_load);                                 // nothing to fetch
    } else if (mode == 0) {
      mbar_expect_tx(&bar_load, 2 * 16384 + 2 * 8192);
      tma_load_3d(sA, &map_a, &bar_load, 0, 0, 0);
      tma_load_3d(sA + 16384, &map_a, &bar_load, 64, 0, 0);
      tma_load_3d(sB, &map_b, &bar_load, 0, 0, 0);
      tma_load_3d(sB + 8192, &map_b, &bar_load, 64, 0, 0);
    } else if (mode == 3) {
      mbar_expect_tx(&bar_load, 2 * 16384 + 16384);
      tma_load_3d(sA, &map_a, &bar_load, 0, 0, 0);            // At rows 0..127, M columns 0..63
      tma_load_3d(sA + 16384, &map_a, &bar_load, 64, 0, 0);   //                  M columns 64..127
      tma_load_3d(sB, &map_b, &bar_load, 0, 0, 0);            // Bt rows 0..127, N columns 0..63
    } else if (mode == 1) {
      mbar_expect_tx(&bar_load, 16384 + 2 * 8192);
      tma_load_3d(sA, &map_a, &bar_load, 0, 0, 0);
      tma_load_3d(sB, &map_b, &bar_load, 0, 0, 0);
      tma_load_3d(sB + 8192, &map_b, &bar_load, 64, 0, 0);
    } else {
      mbar_expect_tx(&bar_load, 2 * 8192);
      tma_load_3d(sB, &map_b, &bar_load, 0, 0, 0);
      tma_load_3d(sB + 8192, &map_b, &bar_load, 64, 0, 0);
    }
    if (mbar_wait(&bar_load, 0, &abort_flag, p.status, 1)) {
      tc_fence_after();
      if (mode == 5) {
        umma_ss(tmem_d, umma_desc_sw32(smem_u32(sA)), umma_desc_sw32(smem_u32(sB)),
                umma_idesc_bf16(128, 64, false), false);
      } else if (mode == 4) {
        umma_ss(tmem_d, umma_desc_noswz16(smem_u32(sA)), umma_desc_noswz16(smem_u32(sB)),
                umma_idesc_bf16(128, 64, false), false);
      } else if (mode == 0) {
        const uint32_t idesc = umma_idesc_bf16(128, 64, false);
#pragma unroll
        for (int kk = 0; kk < 8; ++kk) {
          const uint32_t off = (kk >> 2) * 16384 + (kk & 3) * 32;
          const uint32_t offb = (kk >> 2) * 8192 + (kk & 3) * 32;
          umma_ss(tmem_d, umma_desc_sw128(smem_u32(sA) + off, 16, 1024),
                  umma_desc_sw128(smem_u32(sB) + offb, 16, 1024), idesc, kk > 0);
        }
      } else if (mode == 3) {
        const uint32_t idesc = umma_idesc_bf16(128, 64, true, true);
#pragma unroll
        for (int kk = 0; kk < 8; ++kk)
          umma_ss(tmem_d, umma_desc_sw128(smem_u32(sA) + kk * 2048, 16384, 1024),
                  umma_desc_sw128(smem_u32(sB) + kk * 2048, 16, 1024), idesc, kk > 0);
      } else {
        const uint32_t idesc = umma_idesc_bf16(128, 128, true);
#pragma unroll
        for (int kk = 0; kk < 4; ++kk) {
          const uint64_t bdesc = umma_desc_sw128(smem_u32(sB) + kk * 2048, 8192, 1024);
          if (mode == 1)
            umma_ss(tmem_d, umma_desc_sw128(smem_u32(sA) + kk * 32, 16, 1024),
                    bdesc, idesc, kk > 0);
          else
            umma_ts(tmem_d, tmem_a + kk * 8, bdesc, idesc, kk > 0);
        }
      }
      umma_commit(&bar_mma);
    }
  }
  __syncwarp();
  const bool ok = mbar_wait(&bar_mma, 0, &abort_flag, p.status, 2);
  tc_fence_after();
  if (ok) {
    for (int c = 0; c < n; c += 32) {
      uint32_t regs[32];
      tmem_ld32(tmem_d + ((uint32_t)(warp * 32) << 16) + c, regs);
      tmem_wait_ld();
      float* out = p.d + (size_t)threadIdx.x * n + c;
#pragma unroll
      for (int j = 0; j < 32; ++j) out[j] = __uint_as_float(regs[j]);
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tmem, 256);
}

// A bounded wait that is meant to run out: one CTA allocates TMEM, waits with a short cycle limit
// on an mbarrier that nothing ever arms, records the site in the status block, frees its TMEM and
// returns normally -- the teardown every pipeline kernel shares, exercised without any fault.
__global__ void __launch_bounds__(64)
wait_timeout_selftest_kernel(int32_t* status, long long limit_cycles, int site, int32_t* result) {
  __shared__ uint64_t never_armed;
  __shared__ uint32_t tmem_base_slot;
  __shared__ int abort_flag;
  const int warp = threadIdx.x >> 5;
  if (threadIdx.x == 0) {
    abort_flag = 0;
    mbar_init(&never_armed, 1);
    fence_barrier_init();
  }
  if (warp == 0) {
    tmem_alloc(&tmem_base_slot, 32);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = tmem_base_slot;
  // warp 1 waits; warp 0 then sees the CTA-wide abort flag exactly as the other roles of a
  // pipeline kernel do
  bool ok = true;
  if (warp == 1) ok = mbar_wait(&never_armed, 0, &abort_flag, status, site, limit_cycles);
  __syncthreads();
  if (threadIdx.x == 0) {
    result[0] = abort_flag;                 // 1: the wait gave up and told the CTA
    result[1] = 1;                          // the kernel reached its normal end
  }
  if (threadIdx.x == 32) result[2] = ok ? 0 : 1;
  tc_fence_before();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tmem, 32);
}

}  // namespace
}  // namespace ifv2

using namespace ifv2;

extern "C" int ifv2_selftest_wait_timeout(int32_t* status, int64_t limit_cycles, int site,
                                          int32_t* result, void* stream) {
  IFV2_REQUIRE(status && result, IFV2_ERR_INVALID_ARG, "selftest_wait_timeout: null pointer");
  IFV2_REQUIRE(limit_cycles >= 1 && limit_cycles <= (1ll << 24), IFV2_ERR_INVALID_ARG,
               "selftest_wait_timeout: limit_cycles must be in [1, 2^24] (a few milliseconds at most)");
  IFV2_REQUIRE(site > 0, IFV2_ERR_INVALID_ARG, "selftest_wait_timeout: site must be > 0");
  wait_timeout_selftest_kernel<<<1, 64, 0, (cudaStream_t)stream>>>(status, (long long)limit_cycles,
                                                                  site, result);
  return check_launch("selftest_wait_timeout");
}

// Runs one tile product.
//   mode 0: a (128,128), b (64,128)  -> d (128,64);  modes 1, 2: a (128,64), b (64,128) -> d (128,128)
//   mode 3: a (128,128) = At, b (128,64) = Bt -> d = At^T . Bt (128,64)
//   mode 4: a (128,16), b (64,16) -> d = a . b^T (128,64)
extern "C" int ifv2_selftest_umma(int mode, const void* a, const void* b, float* d, int32_t* status,
                                  void* stream) {
  IFV2_REQUIRE(mode >= 0 && mode <= 5, IFV2_ERR_INVALID_ARG, "selftest: mode must be 0..5");
  IFV2_REQUIRE(a && b && d && status, IFV2_ERR_INVALID_ARG, "selftest: null pointer");
  CUtensorMap map_a, map_b;
  int rc;
  if (mode == 0) {
    rc = make_tensor_map_bf16_3d(&map_a, a, 128, 128, 1, 256, 256 * 128, 64, 128, 1);
    if (rc) return rc;
    rc = make_tensor_map_bf16_3d(&map_b, b, 128, 64, 1, 256, 256 * 64, 64, 64, 1);
  } else if (mode == 4 || mode == 5) {       // operands are written by threads; the maps are not used
    rc = make_tensor_map_bf16_3d(&map_a, d, 64, 128, 1, 128, 128 * 128, 64, 128, 1);
    if (rc) return rc;
    rc = make_tensor_map_bf16_3d(&map_b, d, 64, 128, 1, 128, 128 * 128, 64, 128, 1);
  } else if (mode == 3) {
    rc = make_tensor_map_bf16_3d(&map_a, a, 128, 128, 1, 256, 256 * 128, 64, 128, 1);
    if (rc) return rc;
    rc = make_tensor_map_bf16_3d(&map_b, b, 64, 128, 1, 128, 128 * 128, 64, 128, 1);
  } else {
    rc = make_tensor_map_bf16_3d(&map_a, a, 64, 128, 1, 128, 128 * 128, 64, 128, 1);
    if (rc) return rc;
    rc = make_tensor_map_bf16_3d(&map_b, b, 128, 64, 1, 256, 256 * 64, 64, 64, 1);
  }
  if (rc) return rc;
  cudaError_t attr = cudaFuncSetAttribute(umma_selftest_kernel,
                                          cudaFuncAttributeMaxDynamicSharedMemorySize, 50 * 1024);
  if (attr != cudaSuccess) return set_error((int)attr, "selftest: %s", cudaGetErrorString(attr));
  SelfTestParams p{static_cast<const __nv_bfloat16*>(a), static_cast<const __nv_bfloat16*>(b), d, mode,
                   status};
  umma_selftest_kernel<<<1, 128, 50 * 1024, (cudaStream_t)stream>>>(map_a, map_b, p);
  return check_launch("umma_selftest");
}
