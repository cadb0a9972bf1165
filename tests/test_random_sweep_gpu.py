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


def _block_lists(rnd, rng, bsz, hk, n_keys, k_sel):
    rows = np.full((bsz, hk, 1, k_sel), -1, np.int32)
    for b in range(bsz):
        nblk = (n_keys[b] + 63) // 64
        for h in range(hk):
            take = min(k_sel, nblk, rnd.randint(1, k_sel))
            if nblk:
                rows[b, h, 0, :take] = np.sort(rng.choice(nblk, size=take, replace=False))
    return torch.from_numpy(rows)


@pytest.mark.parametrize("seed", [1, 5])
def test_random_sweep_kvcache(seed):
    """infllmv2_attn_with_kvcache over random batch / heads / capacity / lengths (empty caches
    with an append included), with and without an append, a block list, cache_batch_idx +
    cache_leftpad or a paged cache, against the oracle on the equivalent dense cache."""
    rnd, rng = random.Random(seed), np.random.default_rng(seed)
    gen = torch.Generator().manual_seed(seed)
    d = 128
    for case in range(20):
        bsz, hk = rnd.randint(1, 6), rnd.choice([1, 2, 4])
        mode = rnd.choice(["plain", "plain", "slots", "paged"])
        append, use_topk, k_sel = rnd.random() < 0.5, rnd.random() < 0.7, rnd.choice([1, 3, 8, 16])
        page = rnd.choice([64, 128, 256])
        cap = page * rnd.randint(1, 8) if mode == "paged" else rnd.randint(2, 1500)
        lens = [rnd.randint(0 if append else 1, cap - (1 if append else 0)) for _ in range(bsz)]
        tag = (seed, case, bsz, hk, mode, append, use_topk, k_sel, cap, lens)
        q = (torch.randn(bsz, 1, hk * 16, d, generator=gen) * 0.3).to(torch.bfloat16)
        kn = (torch.randn(bsz, 1, hk, d, generator=gen) * 0.3).to(torch.bfloat16) if append else None
        vn = torch.randn(bsz, 1, hk, d, generator=gen).to(torch.bfloat16) if append else None
        kw, n = {}, list(lens)
        if mode == "slots":
            rows = bsz + rnd.randint(0, 3)
            slot = torch.tensor(rng.permutation(rows)[:bsz].astype(np.int32))
            pad = torch.tensor([rnd.randint(0, l if append else max(l - 1, 0)) for l in lens], dtype=torch.int32)
            kc = (torch.randn(rows, cap, hk, d, generator=gen) * 0.3).to(torch.bfloat16)
            vc = torch.randn(rows, cap, hk, d, generator=gen).to(torch.bfloat16)
            n = [l - int(p) for l, p in zip(lens, pad)]
            kd = torch.zeros(bsz, cap + 1, hk, d, dtype=kc.dtype)
            vd = torch.zeros_like(kd)
            for b in range(bsz):
                kd[b, :n[b]] = kc[slot[b], int(pad[b]):lens[b]]
                vd[b, :n[b]] = vc[slot[b], int(pad[b]):lens[b]]
            kw = dict(cache_batch_idx=slot.to(DEV), cache_leftpad=pad.to(DEV))
        elif mode == "paged":
            per = cap // page
            table = torch.tensor(rng.permutation(bsz * per + 2)[:bsz * per].reshape(bsz, per).astype(np.int32))
            kc = (torch.randn(bsz * per + 2, page, hk, d, generator=gen) * 0.3).to(torch.bfloat16)
            vc = torch.randn(bsz * per + 2, page, hk, d, generator=gen).to(torch.bfloat16)
            tail = torch.zeros(bsz, 1, hk, d, dtype=kc.dtype)
            kd = torch.cat([torch.stack([kc[table[b].long()].reshape(cap, hk, d) for b in range(bsz)]), tail], 1)
            vd = torch.cat([torch.stack([vc[table[b].long()].reshape(cap, hk, d) for b in range(bsz)]), tail], 1)
            kw = dict(block_table=table.to(DEV))
        else:
            kc = (torch.randn(bsz, cap, hk, d, generator=gen) * 0.3).to(torch.bfloat16)
            vc = torch.randn(bsz, cap, hk, d, generator=gen).to(torch.bfloat16)
            kd = torch.cat([kc, torch.zeros(bsz, 1, hk, d, dtype=kc.dtype)], 1)
            vd = torch.cat([vc, torch.zeros(bsz, 1, hk, d, dtype=vc.dtype)], 1)
        idx = _block_lists(rnd, rng, bsz, hk, [x + int(append) for x in n], k_sel) if use_topk else None
        ref, _ = oracle.kvcache_decode(q, kd, vd, torch.tensor(n, dtype=torch.int32), idx, kn, vn)
        out = infllm_v2.infllmv2_attn_with_kvcache(
            q.to(DEV), kc.to(DEV), vc.to(DEV), kn.to(DEV) if append else None, vn.to(DEV) if append else None,
            cache_seqlens=torch.tensor(lens, dtype=torch.int32, device=DEV),
            topk_idx=idx.to(DEV) if idx is not None else None, **kw)
        assert (out.float().cpu() - ref).abs().max().item() <= 2e-2, tag
        infllm_v2.check_device_status()
