"""CPU: the plain-PyTorch fp32 restatements used for the large-size GPU parity checks
(tests/gpu_oracle.py, gathered keys) agree with the pinned CPU oracle (dense under the mask) on
small shapes, forward and backward."""
import numpy as np
import torch

import oracle
import gpu_oracle
from helpers import det_tensor, cu, local_topk


def test_stage1_rows_equal_oracle():
    lq, hq, hk, d = 300, 32, 2, 128
    q = det_tensor((lq, hq, d), 1, 0.5)
    k = det_tensor((lq, hk, d), 2, 0.5)
    kc, cu_c = oracle.compress_keys(k, [0, lq])
    ref = oracle.stage1_scores(q, kc, [0, lq], cu_c, cu_c[-1], True)
    toks = torch.tensor([0, 30, 31, 47, 48, 200, 299])
    got = gpu_oracle.stage1_rows(q[toks], kc, toks, lq)
    assert (got - ref[:, toks]).abs().max().item() < 1e-5


def test_attend_rows_and_decode_equal_oracle():
    lq, lk, hq, hk, d = 150, 400, 32, 2, 128
    q = det_tensor((lq, hq, d), 3, 0.25)
    k = det_tensor((lk, hk, d), 4, 0.25)
    v = det_tensor((lk, hk, d), 5)
    idx = local_topk(hk, [lq], [lk], 3, 6)
    ref, ref_lse = oracle.sparse_attention_fwd(q, k, v, [0, lq], [0, lk], idx, causal=True)
    toks = torch.tensor([0, 1, 63, 64, 149])
    got, lse = gpu_oracle.attend_rows(q[toks], toks, k, v, idx[:, toks], lq)
    assert (got - ref[toks]).abs().max().item() < 1e-5
    ref_lse = ref_lse.view(hk, lq, 16)[:, toks]
    assert torch.equal(torch.isinf(lse), torch.isinf(ref_lse))
    fin = ~torch.isinf(lse)
    assert (lse[fin] - ref_lse[fin]).abs().max().item() < 1e-4

    b, cap = 3, 300
    qd = det_tensor((b, 1, hq, d), 7, 0.25)
    kcache, vcache = det_tensor((b, cap, hk, d), 8, 0.25), det_tensor((b, cap, hk, d), 9)
    lens = torch.tensor([300, 65, 1], dtype=torch.int32)
    di = torch.tensor(np.array([[[[0, 2, 4]], [[1, 3, -1]]], [[[0, 1, -1]], [[1, -1, -1]]],
                                [[[0, -1, -1]], [[0, -1, -1]]]], dtype=np.int32))
    ref, _ = oracle.kvcache_decode(qd, kcache.clone(), vcache.clone(), lens, di)
    assert (gpu_oracle.decode_rows(qd, kcache, vcache, lens, di) - ref).abs().max().item() < 1e-5


def test_blockshared_fwd_bwd_equals_oracle():
    lens, hq, hk, d = [130, 64, 200], 32, 2, 128
    t = sum(lens)
    q = det_tensor((t, hq, d), 11, 0.25)
    k = det_tensor((t, hk, d), 12, 0.25)
    v = det_tensor((t, hk, d), 13)
    do = det_tensor((t, hq, d), 14, 0.5)
    idx = local_topk(hk, lens, lens, 2, 15, shared_per_block=True)
    out, lse, dq, dk, dv = oracle.sparse_attention_fwd_bwd(q, k, v, do, cu(lens), cu(lens), idx, causal=True)
    g_out, g_dq, g_dk, g_dv = gpu_oracle.blockshared_fwd_bwd(q, k, v, do, lens, idx)
    for a, b in ((g_out, out), (g_dq, dq), (g_dk, dk), (g_dv, dv)):
        assert (a - b).abs().max().item() < 2e-5 * max(1.0, b.abs().max().item())
