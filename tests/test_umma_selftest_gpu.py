"""GPU: single-tile products through TMA + tcgen05 in each operand arrangement the attention
kernels use (both operands in swizzled smem, MN-major B, A from TMEM)."""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("mode", [0, 1, 2, 3, 4, 5])
def test_umma_tile(lib, mode):
    g = torch.Generator().manual_seed(mode)
    if mode == 0:
        a = torch.randn(128, 128, generator=g).to(torch.bfloat16)
        b = torch.randn(64, 128, generator=g).to(torch.bfloat16)
        ref = a.float() @ b.float().t()
    elif mode in (4, 5):
        a = torch.randn(128, 16, generator=g).to(torch.bfloat16)
        b = torch.randn(64, 16, generator=g).to(torch.bfloat16)
        ref = a.float() @ b.float().t()
    elif mode == 3:
        a = torch.randn(128, 128, generator=g).to(torch.bfloat16)      # At: (K rows, M)
        b = torch.randn(128, 64, generator=g).to(torch.bfloat16)       # Bt: (K rows, N)
        ref = a.float().t() @ b.float()
    else:
        a = torch.randn(128, 64, generator=g).to(torch.bfloat16)
        b = torch.randn(64, 128, generator=g).to(torch.bfloat16)
        ref = a.float() @ b.float()
    d = torch.full(ref.shape, float("nan"), device="cuda")
    status = torch.zeros(4, dtype=torch.int32, device="cuda")
    a_d, b_d = a.cuda(), b.cuda()
    fn = lib.ifv2_selftest_umma
    fn.argtypes = [ctypes.c_int] + [ctypes.c_void_p] * 5
    fn.restype = ctypes.c_int
    rc = fn(mode, a_d.data_ptr(), b_d.data_ptr(), d.data_ptr(), status.data_ptr(),
            torch.cuda.current_stream().cuda_stream)
    assert rc == 0, lib.ifv2_last_error()
    torch.cuda.synchronize()
    assert int(status[0]) == 0, f"bounded wait ran out at site {int(status[0])}"
    err = (d.cpu() - ref).abs().max().item()
    assert err < 1e-2 * max(1.0, ref.abs().max().item()), f"mode {mode}: max err {err}"
