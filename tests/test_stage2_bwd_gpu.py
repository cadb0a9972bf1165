"""GPU: stage-2 backward (dQ, dK, dV) against autograd of the fp32 dense-with-mask oracle.
Tolerance (bf16 gradients): max-abs <= 2e-2 and mean-rel <= 1e-2, the tolerance the forward
uses; dK/dV sums over hundreds of rows get the same bound relative to their own scale."""
import numpy as np
import pytest
import torch

import oracle
import infllm_v2
from helpers import det_tensor, cu, local_topk, err_stats

pytestmark = pytest.mark.gpu
DEV = "cuda"
MAX_ABS, MEAN_REL = 2e-2, 1e-2


def _grads(q, k, v, do, cu_q, cu_k, idx, causal):
    qd, kd, vd = (t.to(DEV).requires_grad_(True) for t in (q, k, v))
    out = infllm_v2.infllmv2_attn_varlen_func(
        qd, kd, vd, cu_q.to(DEV), cu_k.to(DEV), int((cu_q[1:] - cu_q[:-1]).max()),
        int((cu_k[1:] - cu_k[:-1]).max()), causal=causal, topk_idx=None if idx is None else idx.to(DEV))
    out.backward(do.to(DEV))
    infllm_v2.check_device_status()
    return out.detach().cpu(), qd.grad.cpu(), kd.grad.cpu(), vd.grad.cpu()


def _check(lens_q, lens_k, k_sel, causal, dense=False, shared=False, hk=2, seed=0):
    hq, d = hk * 16, 128
    q = det_tensor((sum(lens_q), hq, d), seed + 1, 0.25)
    k = det_tensor((sum(lens_k), hk, d), seed + 2, 0.25)
    v = det_tensor((sum(lens_k), hk, d), seed + 3)
    do = det_tensor((sum(lens_q), hq, d), seed + 4, 0.5)
    idx = None if dense else local_topk(hk, lens_q, lens_k, k_sel, seed, shared_per_block=shared)
    out, dq, dk, dv = _grads(q, k, v, do, cu(lens_q), cu(lens_k), idx, causal)
    _, _, rdq, rdk, rdv = oracle.sparse_attention_fwd_bwd(q, k, v, do, cu(lens_q), cu(lens_k), idx,
                                                          causal=causal)
    for name, got, ref in (("dq", dq, rdq), ("dk", dk, rdk), ("dv", dv, rdv)):
        assert not torch.isnan(got.float()).any(), name
        mx, mr = err_stats(got, ref)
        scale = max(1.0, ref.abs().max().item())
        assert mx <= MAX_ABS * scale and mr <= MEAN_REL, (name, mx, mr, scale)
    return dq, dk, dv


@pytest.mark.parametrize("lens_q,lens_k,k_sel,causal", [
    ([128], [128], 2, True), ([200, 136], [200, 136], 3, True), ([64, 192], [160, 300], 3, True),
    ([1000], [1000], 8, True), ([77, 5, 130], [77, 5, 130], 2, True), ([256], [256], 4, False),
    ([8], [8], 1, True), ([3], [700], 4, True),
])
def test_bwd_sparse(lens_q, lens_k, k_sel, causal):
    _check(lens_q, lens_k, k_sel, causal, seed=sum(lens_q) + k_sel)


def test_bwd_dense():
    _check([300], [300], 0, True, dense=True, seed=5)


def test_bwd_shared_masks_two_words():
    _check([4500], [4500], 6, True, shared=True, seed=9)


def test_bwd_unselected_blocks_get_zero_grad_and_rerun_is_deterministic():
    hq, hk, d = 32, 2, 128
    q = det_tensor((256, hq, d), 1, 0.25)
    k = det_tensor((256, hk, d), 2, 0.25)
    v = det_tensor((256, hk, d), 3)
    do = det_tensor((256, hq, d), 4, 0.5)
    idx = torch.full((hk, 256, 2), -1, dtype=torch.int32)
    idx[:, :, 0] = 0                          # everybody attends block 0 only
    a = _grads(q, k, v, do, cu([256]), cu([256]), idx, True)
    b = _grads(q, k, v, do, cu([256]), cu([256]), idx, True)
    assert all(torch.equal(x, y) for x, y in zip(a, b))      # no atomics anywhere
    assert a[2][64:].abs().max() == 0 and a[3][64:].abs().max() == 0


def test_bwd_column_masks_with_long_empty_stretches():
    """Key blocks whose selecting tokens lie thousands of tokens apart: the dK / dV kernel's walk
    over the column-mask row has to skip runs of more than 32 empty 64-bit words and refill its
    cached words, with the second sequence starting in the middle of a word (q0 = 4200)."""
    hk, d = 1, 128
    hq = hk * 16
    lens = [4200, 600]
    rows = []
    for lq in lens:
        for t in range(lq):
            blocks = {0, t // 64}
            if lq == 4200 and (t == 200 or 4100 <= t < 4104):
                blocks.add(1)                  # block 1: its own tokens, token 200, tokens 4100-4103
            if lq == 4200 and t == 4199:
                blocks.add(30)                 # block 30: its own tokens and the very last one
            if lq == 600 and t in (70, 599):
                blocks.add(1)
            row = sorted(blocks) + [-1] * (4 - len(blocks))
            rows.append(row)
    idx = torch.tensor(rows, dtype=torch.int32).view(1, sum(lens), 4).repeat(hk, 1, 1)
    q = det_tensor((sum(lens), hq, d), 21, 0.25)
    k = det_tensor((sum(lens), hk, d), 22, 0.25)
    v = det_tensor((sum(lens), hk, d), 23)
    do = det_tensor((sum(lens), hq, d), 24, 0.5)
    out, dq, dk, dv = _grads(q, k, v, do, cu(lens), cu(lens), idx, True)
    _, _, rdq, rdk, rdv = oracle.sparse_attention_fwd_bwd(q, k, v, do, cu(lens), cu(lens), idx, causal=True)
    for name, got, ref in (("dq", dq, rdq), ("dk", dk, rdk), ("dv", dv, rdv)):
        assert not torch.isnan(got.float()).any(), name
        mx, mr = err_stats(got, ref)
        scale = max(1.0, ref.abs().max().item())
        assert mx <= MAX_ABS * scale and mr <= MEAN_REL, (name, mx, mr, scale)
    # the rows of block 1 of the first sequence get exactly the contributions of those 73 tokens
    assert dk[64:128].abs().max() > 0 and dv[64:128].abs().max() > 0
