"""Issue-rate probe for tcgen05.mma on one SM (a tuning aid, not part of the operator API).

    python -m infllmv2_cuda_impl_b200.mma_probe

One CTA issues a long run of M=128, K=16 bf16 MMAs of one shape / operand arrangement and reports
SM clocks per MMA (`ifv2_umma_rate` in csrc/umma_rate.cu).  The table answers the questions the
attention kernels' tile shapes depend on: what an N=64 step costs against N=128 or N=256, whether
an operand in TMEM or an MN-major operand changes the rate, and what a tcgen05.commit after every
group of MMAs costs the issuing warp.
"""
import ctypes
import sys

import torch

from . import _lib

_A = {0: "A smem K-major ", 1: "A smem MN-major", 2: "A in TMEM      "}
_B = {0: "B K-major ", 1: "B MN-major"}


def clocks_per_mma(a, b, n, accs=1, steps=8, nonzero=0, stage_stride=0, commits=0):
    """SM clocks per MMA for one variant (two run lengths, so launch and drain cancel out)."""
    lib = _lib.load()
    fn = lib.ifv2_umma_rate
    fn.argtypes = [ctypes.c_int] * 7 + [ctypes.c_void_p] * 3
    fn.restype = ctypes.c_int
    status = torch.zeros(4, dtype=torch.int32, device="cuda")
    cyc = torch.zeros(1, dtype=torch.int64, device="cuda")
    flags = (nonzero & 1) | ((stage_stride & 0xFFF) << 1) | (commits << 16)
    res = []
    for iters in (200, 400):
        rc = fn(a, b, n, accs, steps, flags, iters, cyc.data_ptr(), status.data_ptr(), None)
        torch.cuda.synchronize()
        if rc != 0:
            raise RuntimeError(lib.ifv2_last_error().decode(errors="replace"))
        if int(status[0]) != 0:
            raise RuntimeError(f"a device wait ran out (code {int(status[0])})")
        res.append(int(cyc[0]))
    return (res[1] - res[0]) / 200.0 / steps


def exp_values_per_clock(mode):
    """Exponentials per SM clock of one form (`ifv2_ex2_rate`: 0 ex2.f32, 1 ex2.bf16x2, 2 ex2.f16x2,
    3 degree-3 polynomial on the FMA pipe), 1024 threads on one SM, two run lengths."""
    lib = _lib.load()
    fn = lib.ifv2_ex2_rate
    fn.argtypes = [ctypes.c_int, ctypes.c_int, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p]
    fn.restype = ctypes.c_int
    cyc = torch.zeros(1, dtype=torch.int64, device="cuda")
    sink = torch.zeros(1, dtype=torch.float32, device="cuda")
    res = []
    for iters in (2000, 4000):
        if fn(mode, iters, cyc.data_ptr(), sink.data_ptr(), None) != 0:
            raise RuntimeError(lib.ifv2_last_error().decode(errors="replace"))
        torch.cuda.synchronize()
        res.append(int(cyc[0]))
    per_instr = 2 if mode in (1, 2) else 1
    return 1024 * 2000 * 8 * per_instr / (res[1] - res[0])


def main():
    if not torch.cuda.is_available():
        sys.exit("mma_probe needs a GPU")
    rows = []
    for a, b, n in [(0, 0, 64), (0, 0, 128), (0, 0, 256), (0, 1, 128), (1, 1, 64), (2, 0, 64),
                    (2, 1, 128)]:
        rows.append((a, b, n, 8, 0, clocks_per_mma(a, b, n)))
    for a, b, n in [(0, 0, 64), (0, 0, 128), (2, 1, 128)]:
        for commits in (1, 2):
            rows.append((a, b, n, 8, commits, clocks_per_mma(a, b, n, commits=commits)))
        rows.append((a, b, n, 4, 2, clocks_per_mma(a, b, n, steps=4, commits=2)))
    print("operands                         N   MMAs/group commits/group  clk/MMA  flop/clk/SM")
    for a, b, n, steps, commits, clk in rows:
        print(f"{_A[a]} {_B[b]}  {n:4d}  {steps:6d}     {commits:6d}      {clk:7.1f}  "
              f"{128 * n * 32 / clk:9.0f}")
    print("exponentials per clock per SM:")
    for mode, name in ((0, "ex2.approx.ftz.f32"), (1, "ex2.approx.ftz.bf16x2 (+ cvt)"), (2, "ex2.approx.f16x2 (+ cvt)"),
                       (3, "degree-3 polynomial, FMA pipe")):
        print(f"  {name:32s} {exp_values_per_clock(mode):6.1f}")


if __name__ == "__main__":
    main()
