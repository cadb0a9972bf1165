"""GPU: the key addressing options of the varlen forward and of the stage-1 scorer -- a paged cache
(block_table), left-padded sequences (leftpad_k) and seqused_k -- against the same call on packed
keys (same kernels, so bit for bit) and against the fp32 oracle."""
import numpy as np
import pytest
import torch

import oracle
import infllm_v2
from helpers import det_tensor, cu, local_topk, err_stats

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _paginate(x, lens, page, seed):
    """Packed rows (sum(lens), H, d) -> (pages (n_pages, page, H, d) with NaN in unused rows and a
    shuffled page order, block_table (batch, max_pages) int32)."""
    rng = np.random.default_rng(seed)
    per_seq = [(l + page - 1) // page for l in lens]
    n_pages = sum(per_seq) + 3                                 # a few pages nobody uses
    order = rng.permutation(n_pages)
    pages = torch.full((n_pages, page) + tuple(x.shape[1:]), float("nan"), dtype=x.dtype)
    table = np.zeros((len(lens), max(per_seq)), np.int32)
    start, nxt = 0, 0
    for b, l in enumerate(lens):
        for j in range(per_seq[b]):
            pg = int(order[nxt]); nxt += 1
            table[b, j] = pg
            rows = x[start + j * page:start + min(l, (j + 1) * page)]
            pages[pg, :rows.shape[0]] = rows
        start += l
    return pages, torch.from_numpy(table)


@pytest.mark.parametrize("page", [64, 256])
def test_varlen_forward_over_a_paged_cache(page):
    hq, hk, d = 32, 2, 128
    lens_q, lens_k = [200, 64, 300], [500, 129, 300]
    q = det_tensor((sum(lens_q), hq, d), 1, 0.25)
    k = det_tensor((sum(lens_k), hk, d), 2, 0.25)
    v = det_tensor((sum(lens_k), hk, d), 3)
    idx = local_topk(hk, lens_q, lens_k, 3, 4)
    cu_q, cu_k = cu(lens_q), cu(lens_k)
    ref = infllm_v2.infllmv2_attn_varlen_func(q.to(DEV), k.to(DEV), v.to(DEV), cu_q.to(DEV), cu_k.to(DEV),
                                              max(lens_q), max(lens_k), causal=True, topk_idx=idx.to(DEV))
    kp, table = _paginate(k, lens_k, page, 5)
    vp, _ = _paginate(v, lens_k, page, 5)
    out, lse, _ = infllm_v2.infllmv2_attn_varlen_func(
        q.to(DEV), kp.to(DEV), vp.to(DEV), cu_q.to(DEV), cu_k.to(DEV), max(lens_q), max(lens_k), causal=True,
        topk_idx=idx.to(DEV), block_table=table.to(DEV), return_attn_probs=True)
    infllm_v2.check_device_status()
    assert not torch.isnan(out.float()).any()
    assert torch.equal(out, ref)
    o_ref, _ = oracle.sparse_attention_fwd(q, k, v, cu_q, cu_k, idx, causal=True)
    mx, mr = err_stats(out.cpu(), o_ref)
    assert mx <= 2e-2 and mr <= 1e-2, (mx, mr)


def test_varlen_forward_leftpad_and_seqused():
    hq, hk, d = 32, 2, 128
    lens_q = [100, 70]
    extents = [300, 200]                      # rows each sequence owns in the packed key tensor
    pad = [37, 0]
    used = [300, 150]                         # seqused_k counts from the start of the extent
    k = det_tensor((sum(extents), hk, d), 2, 0.25)
    v = det_tensor((sum(extents), hk, d), 3)
    q = det_tensor((sum(lens_q), hq, d), 1, 0.25)
    lens_k = [u - p for u, p in zip(used, pad)]
    idx = local_topk(hk, lens_q, lens_k, 2, 4)
    cu_q, cu_e = cu(lens_q), cu(extents)
    out = infllm_v2.infllmv2_attn_varlen_func(
        q.to(DEV), k.to(DEV), v.to(DEV), cu_q.to(DEV), cu_e.to(DEV), max(lens_q), max(lens_k), causal=True,
        topk_idx=idx.to(DEV), leftpad_k=torch.tensor(pad, dtype=torch.int32, device=DEV),
        seqused_k=torch.tensor(used, dtype=torch.int32, device=DEV))
    # the same keys packed tightly
    rows = torch.cat([torch.arange(cu_e[b] + pad[b], cu_e[b] + used[b]) for b in range(2)])
    ref = infllm_v2.infllmv2_attn_varlen_func(q.to(DEV), k[rows].to(DEV), v[rows].to(DEV), cu_q.to(DEV),
                                              cu(lens_k).to(DEV), max(lens_q), max(lens_k), causal=True,
                                              topk_idx=idx.to(DEV))
    infllm_v2.check_device_status()
    assert torch.equal(out, ref)
    with pytest.raises(NotImplementedError):
        infllm_v2.infllmv2_attn_varlen_func(
            q.to(DEV).requires_grad_(True), k.to(DEV), v.to(DEV), cu_q.to(DEV), cu_e.to(DEV), max(lens_q),
            max(lens_k), causal=True, leftpad_k=torch.tensor(pad, dtype=torch.int32, device=DEV))


@pytest.mark.parametrize("page", [128, 256])
def test_stage1_over_a_paged_compressed_key_cache(page):
    hq, hk, d = 32, 2, 128
    lens_q = [700, 260]
    q = det_tensor((sum(lens_q), hq, d), 1, 0.5)
    k = det_tensor((sum(lens_q), hk, d), 2, 0.5)
    kc, cu_c = oracle.compress_keys(k, cu(lens_q).tolist())
    lens_c = [cu_c[i + 1] - cu_c[i] for i in range(2)]
    cu_q, cu_cd = cu(lens_q).to(DEV), torch.tensor(cu_c, dtype=torch.int32, device=DEV)
    ref = infllm_v2.infllmv2_attn_stage1(q.to(DEV), kc.to(DEV), kc.to(DEV), cu_q, cu_cd, cu_cd, max(lens_q),
                                         max(lens_c), causal=True)
    pages, table = _paginate(kc, lens_c, page, 9)
    pages = torch.nan_to_num(pages, nan=1e4)            # rows past a sequence's keys: large, never visible
    pages_d = pages.to(DEV)
    got = infllm_v2.infllmv2_attn_stage1(q.to(DEV), pages_d, pages_d, cu_q, cu_cd, cu_cd, max(lens_q),
                                         max(lens_c), causal=True, block_table=table.to(DEV))
    infllm_v2.check_device_status()
    assert torch.equal(got, ref)
    want = oracle.stage1_scores(q, kc, cu(lens_q), cu_c, max(lens_c), True)
    diff = (got.float().cpu() - want).abs()
    assert bool(((diff <= 2e-2) | (diff <= 2.0 ** -7 * want.abs())).all())
    # fused block scores over the same paged cache
    pooled_ref = infllm_v2.infllmv2_stage1_block_scores(q.to(DEV), kc.to(DEV), cu_q, cu_cd, max(lens_q), max(lens_c),
                                                        2, 1, causal=True)
    pooled = infllm_v2.infllmv2_stage1_block_scores(q.to(DEV), pages_d, cu_q, cu_cd, max(lens_q), max(lens_c),
                                                    2, 1, causal=True, block_table=table.to(DEV))
    assert torch.equal(pooled, pooled_ref)


def test_stage1_leftpad():
    hq, hk, d = 32, 2, 128
    lq = 400
    q = det_tensor((lq, hq, d), 1, 0.5)
    k = det_tensor((lq, hk, d), 2, 0.5)
    kc, cu_c = oracle.compress_keys(k, [0, lq])
    n = cu_c[-1]
    junk = det_tensor((5, hk, d), 7, 3.0)
    padded = torch.cat([junk, kc])                       # five rows in front that must be skipped
    cu_q = torch.tensor([0, lq], dtype=torch.int32, device=DEV)
    ref = infllm_v2.infllmv2_attn_stage1(q.to(DEV), kc.to(DEV), kc.to(DEV), cu_q,
                                         torch.tensor([0, n], dtype=torch.int32, device=DEV),
                                         torch.tensor([0, n], dtype=torch.int32, device=DEV), lq, n, causal=True)
    cu_p = torch.tensor([0, n + 5], dtype=torch.int32, device=DEV)
    padded_d = padded.to(DEV)
    got = infllm_v2.infllmv2_attn_stage1(q.to(DEV), padded_d, padded_d, cu_q, cu_p, cu_p, lq, n,
                                         causal=True, leftpad_k=torch.tensor([5], dtype=torch.int32, device=DEV))
    infllm_v2.check_device_status()
    assert torch.equal(got, ref)
