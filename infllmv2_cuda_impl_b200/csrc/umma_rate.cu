// Sustained issue rate of one tcgen05.mma shape / operand arrangement on a single SM.  One CTA,
// warp 0 issues `iters` groups of four K=16 steps back to back into the same accumulator (operand
// contents are irrelevant and left as zeros), one commit at the end; the cycle count between the
// first issue and the completion gives clocks per MMA.  Everything that selects the variant is a
// template parameter so the issue loop is straight-line code.  Test / tuning hook only.
#include "tc05.cuh"

namespace ifv2 {
namespace {

using namespace tc;

enum : int { kSmemK = 0, kSmemMN = 1, kTmem = 2 };

template <int kA, int kB, int kN, int kAccs, int kSteps, bool kRandom>
__global__ void __launch_bounds__(128)
umma_rate_kernel(int iters, long long* cycles, int32_t* status, int dyn, int commits) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~(uintptr_t)1023);
  uint8_t* sA = smem;              // 32 KB
  uint8_t* sB = smem + 32768;      // 64 KB
  __shared__ uint64_t bar_mma, bar_group[2];
  __shared__ uint32_t tmem_base_slot;
  __shared__ int abort_flag;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  for (int i = threadIdx.x; i < (32768 + 65536) / 16; i += 128) {
    // zeros, or bf16 values of magnitude ~1 with varying mantissas (operand contents may matter)
    const uint32_t w = kRandom ? (0x3F803F80u ^ ((uint32_t)i * 2654435761u & 0x807F807Fu)) : 0u;
    reinterpret_cast<uint4*>(smem)[i] = make_uint4(w, w ^ 0x00110022u * kRandom, w, w ^ 0x00330044u * kRandom);
  }
  fence_proxy_async_smem();
  if (threadIdx.x == 0) {
    abort_flag = 0;
    mbar_init(&bar_mma, 1);
    mbar_init(&bar_group[0], 1);
    mbar_init(&bar_group[1], 1);
    fence_barrier_init();
  }
  if (warp == 0) {
    tmem_alloc(&tmem_base_slot, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = tmem_base_slot;
  const uint32_t tmem_a = tmem + 448;          // up to 8 K steps x 8 columns
  long long t_start = 0;
  if (warp == 0) {
    const uint32_t leader = (lane == 0) ? 1u : 0u;
    constexpr uint32_t idesc = umma_idesc_bf16(128, kN, kB == kSmemMN, kA == kSmemMN);
    // K-major: K step = 32 bytes inside the 128-byte row.  MN-major: K step = 16 rows = 2 KB,
    // 64-element M/N groups 16 KB apart (64-row tiles stacked group after group).
    const uint64_t da = (kA == kSmemMN) ? umma_desc_sw128(smem_u32(sA), 16384, 1024)
                                        : umma_desc_sw128(smem_u32(sA), 16, 1024);
    const uint64_t db = (kB == kSmemMN) ? umma_desc_sw128(smem_u32(sB), 16384, 1024)
                                        : umma_desc_sw128(smem_u32(sB), 16, 1024);
    constexpr uint32_t a_step = (kA == kSmemMN) ? 128 : 2, b_step = (kB == kSmemMN) ? 128 : 2;
    t_start = clock64();
    for (int it = 0; it < iters; ++it) {
      // dyn != 0: the operand tiles alternate between two ring stages chosen at run time, as in
      // the attention kernels (the descriptors can then not be hoisted out of the loop)
      const uint32_t stage = (uint32_t)(it & 1) * (uint32_t)dyn;
#pragma unroll
      for (int kk = 0; kk < kSteps; ++kk) {
        const uint32_t d = tmem + ((kAccs > 1) ? (uint32_t)((kk % kAccs) * kN) : 0u);
        // K-major: steps 4..7 continue in the second 64-element K slab (16 KB / 32 KB further)
        const uint32_t ao = (kA == kSmemMN) ? a_step * kk : ((kk >> 2) * 1024 + (kk & 3) * 2);
        const uint32_t bo = (kB == kSmemMN) ? b_step * kk : ((kk >> 2) * 2048 + (kk & 3) * 2);
        if (kA == kTmem)
          umma_ts_pred(d, tmem_a + kk * 8, db + stage + bo, idesc, kk >= kAccs, leader);
        else
          umma_ss_pred(d, da + stage + ao, db + stage + bo, idesc, kk >= kAccs, leader);
      }
      // commits per group of K steps, as a pipelined kernel issues them (nobody waits on these)
      for (int c = 0; c < commits; ++c) umma_commit_pred(&bar_group[c & 1], leader);
    }
    umma_commit_pred(&bar_mma, leader);
  }
  __syncwarp();
  mbar_wait(&bar_mma, 0, &abort_flag, status, 2);
  tc_fence_after();
  if (threadIdx.x == 0) *cycles = clock64() - t_start;
  tc_fence_before();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tmem, 512);
}

template <int kA, int kB, int kN, int kAccs, int kSteps, bool kRandom>
int launch_rate(int iters, long long* cycles, int32_t* status, cudaStream_t stream, int dyn,
                int commits) {
  auto kern = umma_rate_kernel<kA, kB, kN, kAccs, kSteps, kRandom>;
  const int smem = 32768 + 65536 + 1024;
  cudaError_t attr = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
  if (attr != cudaSuccess) return set_error((int)attr, "umma_rate: %s", cudaGetErrorString(attr));
  kern<<<1, 128, smem, stream>>>(iters, cycles, status, dyn, commits);
  return check_launch("umma_rate");
}

}  // namespace
}  // namespace ifv2

using namespace ifv2;

// a in {0: smem K-major, 1: smem MN-major, 2: TMEM}, b in {0: K-major, 1: MN-major}; n = MMA N;
// accs = accumulators used in turn; steps = K steps per group (4 or 8); random: bit 0 = non-zero
// operand contents, bits 1..12 = run-time ring-stage stride in descriptor units (0 = fixed tiles),
// bits 16.. = tcgen05.commit instructions issued after every group of K steps.
extern "C" int ifv2_umma_rate(int a, int b, int n, int accs, int steps, int random, int iters,
                              long long* cycles, int32_t* status, void* stream) {
  IFV2_REQUIRE(cycles && status && iters > 0, IFV2_ERR_INVALID_ARG, "umma_rate: bad argument");
  cudaStream_t s = (cudaStream_t)stream;
#define IFV2_RATE_CASE(A, B, N, ACCS)                                                        \
  if (a == A && b == B && n == N && accs == ACCS) {                                          \
    if (steps == 4 && !(random & 1)) return launch_rate<A, B, N, ACCS, 4, false>(iters, cycles, status, s, (random >> 1) & 0xFFF, random >> 16); \
    if (steps == 8 && !(random & 1)) return launch_rate<A, B, N, ACCS, 8, false>(iters, cycles, status, s, (random >> 1) & 0xFFF, random >> 16); \
    if (steps == 8 && (random & 1)) return launch_rate<A, B, N, ACCS, 8, true>(iters, cycles, status, s, (random >> 1) & 0xFFF, random >> 16);   \
    if (steps == 4 && (random & 1)) return launch_rate<A, B, N, ACCS, 4, true>(iters, cycles, status, s, (random >> 1) & 0xFFF, random >> 16);   \
  }
  IFV2_RATE_CASE(0, 0, 64, 1)
  IFV2_RATE_CASE(0, 0, 128, 1)
  IFV2_RATE_CASE(0, 0, 256, 1)
  IFV2_RATE_CASE(0, 1, 64, 1)
  IFV2_RATE_CASE(0, 1, 128, 1)
  IFV2_RATE_CASE(0, 1, 256, 1)
  IFV2_RATE_CASE(0, 1, 128, 2)
  IFV2_RATE_CASE(1, 0, 64, 1)
  IFV2_RATE_CASE(1, 0, 128, 1)
  IFV2_RATE_CASE(1, 1, 64, 1)
  IFV2_RATE_CASE(1, 1, 128, 1)
  IFV2_RATE_CASE(2, 0, 64, 1)
  IFV2_RATE_CASE(2, 0, 128, 1)
  IFV2_RATE_CASE(2, 0, 256, 1)
  IFV2_RATE_CASE(2, 1, 64, 1)
  IFV2_RATE_CASE(2, 1, 128, 1)
  IFV2_RATE_CASE(2, 1, 256, 1)
  IFV2_RATE_CASE(2, 1, 128, 2)
#undef IFV2_RATE_CASE
  return set_error(IFV2_ERR_INVALID_ARG, "umma_rate: variant not instantiated");
}

// ---------------------------------------------------------------------------------------------
// Throughput of the exponential forms a softmax loop can use, on one SM: 1024 threads each run
// `iters` rounds of eight independent exponentials and keep a running sum; the clock count of the
// slowest warp over the number of values gives values per clock per SM.  mode 0: ex2.approx.ftz.f32
// (one value per instruction), 1: ex2.approx.ftz.bf16x2 (two), 2: ex2.approx.f16x2 (two),
// 3: the degree-3 polynomial on the FMA pipe (exp2_fma).  Tuning aid only.
namespace ifv2 {
namespace {

template <int kMode>
__global__ void __launch_bounds__(1024) ex2_rate_kernel(int iters, long long* cycles, float* sink) {
  float x[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) x[j] = -0.01f * (float)(threadIdx.x % 61) - 0.125f * (float)j;
  float acc = 0.f;
  uint32_t pacc = 0;
  __syncthreads();
  const long long t0 = clock64();
  for (int it = 0; it < iters; ++it) {
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      if (kMode == 0) {
        acc += exp2f(x[j]);
      } else if (kMode == 3) {
        acc += tc::exp2_fma(x[j]);
      } else {
        // two values per instruction; the packed results are folded with an xor so that the
        // measured loop holds the exponential and one cheap integer op per pair
        uint32_t in, out;
        if (kMode == 1) {
          asm volatile("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(in) : "f"(x[j]), "f"(x[j] - 0.5f));
          asm volatile("ex2.approx.ftz.bf16x2 %0, %1;" : "=r"(out) : "r"(in));
        } else {
          asm volatile("cvt.rn.f16x2.f32 %0, %1, %2;" : "=r"(in) : "f"(x[j]), "f"(x[j] - 0.5f));
          asm volatile("ex2.approx.f16x2 %0, %1;" : "=r"(out) : "r"(in));
        }
        pacc ^= out;
      }
      x[j] -= 1e-6f;
    }
  }
  const long long t1 = clock64();
  __shared__ long long worst;
  if (threadIdx.x == 0) worst = 0;
  __syncthreads();
  atomicMax(reinterpret_cast<unsigned long long*>(&worst), (unsigned long long)(t1 - t0));
  __syncthreads();
  if (threadIdx.x == 0) *cycles = worst;
  if (acc == 123.456f || pacc == 0x12345678u) *sink = acc;      // keep the results alive
}

}  // namespace
}  // namespace ifv2

// Values per instruction: 1 for modes 0 and 3, 2 for modes 1 and 2.  cycles: SM clocks of the slowest
// warp for 1024 threads x iters x 8 instructions.
extern "C" int ifv2_ex2_rate(int mode, int iters, long long* cycles, float* sink, void* stream) {
  IFV2_REQUIRE(cycles && sink && iters > 0 && mode >= 0 && mode <= 3, IFV2_ERR_INVALID_ARG,
               "ex2_rate: bad argument");
  cudaStream_t s = (cudaStream_t)stream;
  switch (mode) {
    case 0: ex2_rate_kernel<0><<<1, 1024, 0, s>>>(iters, cycles, sink); break;
    case 1: ex2_rate_kernel<1><<<1, 1024, 0, s>>>(iters, cycles, sink); break;
    case 2: ex2_rate_kernel<2><<<1, 1024, 0, s>>>(iters, cycles, sink); break;
    default: ex2_rate_kernel<3><<<1, 1024, 0, s>>>(iters, cycles, sink); break;
  }
  return check_launch("ex2_rate");
}
