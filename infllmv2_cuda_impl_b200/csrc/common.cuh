// Shared host/device helpers for the infllmv2_b200 kernels.
#pragma once
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <stdint.h>
#include <stdio.h>
#include <stdarg.h>

#include "../../include/infllmv2_b200.h"

namespace ifv2 {

constexpr int kNumSMs = 148;          // B200
constexpr int kBlockN = 64;           // tokens per KV block (the reference's n_block_dim)
constexpr int kGroup = 16;            // query heads per KV head (the reference's m_block_dim)
constexpr int kHeadDim = 128;

// Thread-local error text behind ifv2_last_error().
char* error_buffer();
int set_error(int code, const char* fmt, ...);
// Checks the launch of the kernel just enqueued; returns 0 or the positive cudaError_t.
int check_launch(const char* what);
// Clears word 0 of a kernel status block (the flag of the launch about to be enqueued) on the
// stream; word 1 keeps the first failure until ifv2_check_status.  Returns 0 or a cudaError_t.
int clear_launch_status(int32_t* status, void* stream, const char* what);

#define IFV2_REQUIRE(cond, code, ...)                          \
  do {                                                         \
    if (!(cond)) return ::ifv2::set_error((code), __VA_ARGS__); \
  } while (0)

__host__ __device__ inline int64_t ceil_div64(int64_t a, int64_t b) { return (a + b - 1) / b; }
__host__ __device__ inline int ceil_div(int a, int b) { return (a + b - 1) / b; }

// Sequence that owns global row `t` in a cumulative-length table cu[0..batch] (cu[0] == 0):
// largest b with cu[b] <= t.  Empty sequences are skipped by construction.
__device__ inline int find_sequence(const int32_t* __restrict__ cu, int batch, int t) {
  int lo = 0, hi = batch;              // invariant: cu[lo] <= t < cu[hi]
  while (hi - lo > 1) {
    int mid = (lo + hi) >> 1;
    if (cu[mid] <= t) lo = mid; else hi = mid;
  }
  return lo;
}

// Read-only 16-bit loads.  The toolkit's __ldg overloads for __half / __nv_bfloat16 are inline
// asm without `volatile`, which the compiler treats as a pure computation and may hoist above the
// bounds check guarding it: the speculated load of a lane that owns no element then reads past
// the end of the tensor and faults when the tensor ends at a mapping boundary.  The built-in
// overload for unsigned short is an ordinary load and stays behind its guard.
__device__ __forceinline__ __nv_bfloat16 ldg16(const __nv_bfloat16* p) {
  return __ushort_as_bfloat16(__ldg(reinterpret_cast<const unsigned short*>(p)));
}
__device__ __forceinline__ __half ldg16(const __half* p) {
  return __ushort_as_half(__ldg(reinterpret_cast<const unsigned short*>(p)));
}

}  // namespace ifv2
