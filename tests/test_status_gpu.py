"""GPU: the status block of the tensor-core kernels.  A bounded wait is made to run out safely (a
barrier that nothing arms, a limit of 2^16 clocks), and the documented behaviour of the two status
words is checked: word 0 belongs to the running launch and is cleared by every entry point, word 1
keeps the first failure until ifv2_check_status.  Nothing here faults, traps or hangs."""
import pytest
import torch

import infllm_v2
import oracle
from infllmv2_cuda_impl_b200 import _lib, attention
from helpers import det_tensor, cu, local_topk

pytestmark = pytest.mark.gpu
DEV = "cuda"


def test_a_wait_that_runs_out_reports_and_returns(lib):
    status = torch.zeros(4, dtype=torch.int32, device=DEV)
    result = torch.zeros(3, dtype=torch.int32, device=DEV)
    stream = torch.cuda.current_stream().cuda_stream
    _lib.call("ifv2_selftest_wait_timeout", status.data_ptr(), 1 << 16, 97, result.data_ptr(), stream)
    torch.cuda.synchronize()
    assert result.tolist() == [1, 1, 1]            # flag raised, kernel ended normally, wait gave up
    assert status.tolist()[:2] == [97, 97]
    # the context is intact and the tensor memory was returned: a tile product runs right after
    a = torch.randn(128, 128).to(torch.bfloat16).to(DEV)
    b = torch.randn(64, 128).to(torch.bfloat16).to(DEV)
    d = torch.empty(128, 64, device=DEV)
    st2 = torch.zeros(4, dtype=torch.int32, device=DEV)
    _lib.call("ifv2_selftest_umma", 0, a.data_ptr(), b.data_ptr(), d.data_ptr(), st2.data_ptr(), stream)
    torch.cuda.synchronize()
    assert int(st2[0]) == 0
    assert (d - a.float() @ b.float().t()).abs().max().item() < 1e-2 * 128
    # the check reports the site once and clears the block
    rc = lib.ifv2_check_status(status.data_ptr(), stream)
    assert rc == -5 and b"site 97" in lib.ifv2_last_error()
    assert status.tolist() == [0, 0, 0, 0]
    assert lib.ifv2_check_status(status.data_ptr(), stream) == 0
    with pytest.raises(ValueError):
        _lib.call("ifv2_selftest_wait_timeout", status.data_ptr(), 1 << 30, 1, result.data_ptr(), stream)


def test_a_stale_launch_flag_does_not_disable_later_launches():
    """Word 0 left over from a failed launch (preset here) is cleared by the next entry point: the
    forward computes its result; word 1 (preset as if an earlier launch had failed) stays until
    check_device_status raises for it, once."""
    hq, hk, d, lens = 32, 2, 128, [200, 136]
    q = det_tensor((sum(lens), hq, d), 1, 0.25)
    k = det_tensor((sum(lens), hk, d), 2, 0.25)
    v = det_tensor((sum(lens), hk, d), 3)
    idx = local_topk(hk, lens, lens, 3, 7)
    cu_q = cu(lens)
    attention.check_device_status()
    words = attention._status_words(torch.device(DEV))
    words[0] = 1
    words[1] = 33
    out = infllm_v2.infllmv2_attn_varlen_func(q.to(DEV), k.to(DEV), v.to(DEV), cu_q.to(DEV), cu_q.to(DEV),
                                              max(lens), max(lens), causal=True, topk_idx=idx.to(DEV))
    torch.cuda.synchronize()
    assert words.tolist()[:2] == [0, 33]
    ref, _ = oracle.sparse_attention_fwd(q, k, v, cu_q, cu_q, idx, causal=True)
    assert (out.float().cpu() - ref).abs().max().item() <= 2e-2
    with pytest.raises(_lib.Ifv2Error, match="site 33"):
        attention.check_device_status()
    attention.check_device_status()                # cleared by the failed check
