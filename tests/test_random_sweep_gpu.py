"""GPU: seeded random sweep of the whole path against the oracle -- ragged batches of short
sequences (including ones too short for any compressed key), 1/2/4 KV heads, causal or not,
plain or compressed-LSE stage 1; then compression, fused block scores == pool(scores), top-k,
stage-2 forward and backward.  Small shapes, many combinations: the cases the fixed-shape tests
do not enumerate."""
import random

import numpy as np
import pytest
import torch

import oracle
import infllm_v2
from helpers import cu, err_stats

pytestmark = pytest.mark.gpu
DEV = "cuda"
LENGTHS = [1, 7, 31, 32, 33, 64, 100, 129, 300, 511, 600]


def _within(got, ref):
    d = (got - ref).abs()
    return bool(((d <= 2e-2) | (d <= ref.abs() * 2.0 ** -7)).all()), d.max().item()


@pytest.mark.parametrize("seed", [2, 11])
def test_random_sweep(seed):
    rnd = random.Random(seed)
    gen = torch.Generator().manual_seed(seed)
    ran = 0
    for case in range(24):
        nseq, hk = rnd.randint(1, 4), rnd.choice([1, 2, 4])
        lens = [rnd.choice(LENGTHS) for _ in range(nseq)]
        causal, coarse = rnd.random() < 0.8, rnd.random() < 0.4
        total = sum(lens)
        q = (torch.randn(total, hk * 16, 128, generator=gen) * 0.4).to(torch.bfloat16)
        k = (torch.randn(total, hk, 128, generator=gen) * 0.4).to(torch.bfloat16)
        v = torch.randn(total, hk, 128, generator=gen).to(torch.bfloat16)
        kc, cu_c = oracle.compress_keys(k, cu(lens))
        max_k = int(np.diff(cu_c).max())
        if max_k == 0:
            continue
        ran += 1
        tag = (seed, case, lens, hk, causal, coarse)
        kw = {}
        if coarse:
            kv, cu_v = oracle.compress_keys(k, cu(lens), 128, 64)
            kw = dict(lse_keys=kv, cu_seqlens_v=cu_v)
        exp = oracle.stage1_scores(q, kc, cu(lens).tolist(), cu_c, max_k, causal, **kw)
        cq, ck = cu(lens, DEV), torch.tensor(cu_c, dtype=torch.int32, device=DEV)
        qd, kcd = q.to(DEV), kc.to(DEV)
        if coarse:
            vv, cv = kv.to(DEV), torch.tensor(cu_v, dtype=torch.int32, device=DEV)
        else:
            vv, cv = kcd, ck
        got = infllm_v2.infllmv2_attn_stage1(qd, kcd, vv, cq, ck, cv, max(lens), max_k, causal=causal)
        ok, err = _within(got.float().cpu(), exp)
        assert ok, ("stage1", tag, err)

        kcg, _ = infllm_v2.compress_keys(k.to(DEV), cq)
        assert (kcg.cpu().float() - kc.float()).abs().max().item() <= 2.0 ** -7, ("compress", tag)
        if not causal:
            continue

        extra = dict(lse_keys=vv, cu_seqlens_v=cv) if coarse else {}
        pooled = infllm_v2.infllmv2_stage1_block_scores(qd, kcd, cq, ck, max(lens), max_k, 2, 1, **extra)
        ref = infllm_v2.max_pooling_1d_varlen(got, cq, ck, torch.zeros(nseq, dtype=torch.int32, device=DEV),
                                              max(lens), max_k, 2, 1)
        assert torch.equal(pooled, ref), ("fused block scores", tag)

        kk = rnd.choice([1, 3, 8])
        idx = infllm_v2.infllmv2_topk(pooled, kk, cu_seqlens_q=cq)
        qb = torch.cat([torch.arange(l) // 64 for l in lens])
        exp_idx = oracle.topk_select(pooled.float().cpu(), kk, qb)
        assert torch.equal(idx.cpu(), exp_idx), ("topk", tag, kk)

        do = torch.randn(total, hk * 16, 128, generator=gen).to(torch.bfloat16)
        qg, kg, vg = (t.to(DEV).requires_grad_(True) for t in (q, k, v))
        out = infllm_v2.infllmv2_attn_varlen_func(qg, kg, vg, cq, cq, max(lens), max(lens), causal=True,
                                                  topk_idx=idx)
        out.backward(do.to(DEV))
        ro, _, rdq, rdk, rdv = oracle.sparse_attention_fwd_bwd(q, k, v, do, cu(lens).tolist(),
                                                                cu(lens).tolist(), exp_idx)
        for name, a, b in (("out", out, ro), ("dq", qg.grad, rdq), ("dk", kg.grad, rdk), ("dv", vg.grad, rdv)):
            mx, mr = err_stats(a.detach().float().cpu(), b)
            assert mx <= 2e-2 * max(1.0, b.abs().max().item()) and mr <= 1e-2, (name, tag, kk, mx, mr)
        infllm_v2.check_device_status()
    assert ran >= 10
