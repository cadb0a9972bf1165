"""GPU: sparse KV-cache decode against the fp32 oracle (max-abs <= 2e-2, mean-rel <= 1e-2)."""
import os

import numpy as np
import pytest
import torch

import oracle
import infllm_v2
from helpers import det_tensor, err_stats
from inputs import det_array, det_perm_rows

pytestmark = pytest.mark.gpu
DEV = "cuda"
MAX_ABS, MEAN_REL = 2e-2, 1e-2


def _case(bsz, hk, lens, cap, k_sel, append, seed):
    hq, d = hk * 16, 128
    q = det_tensor((bsz, 1, hq, d), seed, 0.25)
    kc = det_tensor((bsz, cap, hk, d), seed + 1, 0.25)
    vc = det_tensor((bsz, cap, hk, d), seed + 2)
    kn = det_tensor((bsz, 1, hk, d), seed + 3, 0.25) if append else None
    vn = det_tensor((bsz, 1, hk, d), seed + 4) if append else None
    lens_t = torch.tensor(lens, dtype=torch.int32)
    idx = None
    if k_sel:
        rng = np.random.default_rng(seed)
        rows = []
        for b in range(bsz):
            nblk = (lens[b] + (1 if append else 0) + 63) // 64
            per = []
            for h in range(hk):
                pick = np.sort(rng.permutation(nblk)[:k_sel])
                row = np.full(k_sel, -1, np.int32)
                row[:len(pick)] = pick
                per.append(row)
            rows.append(np.stack(per))
        idx = torch.from_numpy(np.stack(rows)).view(bsz, hk, 1, k_sel)
    kc_ref, vc_ref = kc.clone(), vc.clone()
    ref, ref_lse = oracle.kvcache_decode(q, kc_ref, vc_ref, lens_t, idx, kn, vn)
    kc_d, vc_d = kc.to(DEV), vc.to(DEV)
    out, lse = infllm_v2.infllmv2_attn_with_kvcache(
        q.to(DEV), kc_d, vc_d, k=None if kn is None else kn.to(DEV), v=None if vn is None else vn.to(DEV),
        cache_seqlens=lens_t.to(DEV), topk_idx=None if idx is None else idx.to(DEV),
        return_softmax_lse=True)
    torch.cuda.synchronize()
    assert out.shape == (bsz, 1, hq, d) and lse.shape == (bsz, hq, 1)
    mx, mr = err_stats(out.cpu(), ref)
    assert mx <= MAX_ABS and mr <= MEAN_REL, (mx, mr)
    assert (lse.cpu() - ref_lse).abs().max() < 2e-2
    if append:       # the caches were updated in place, exactly like the oracle's copies
        assert torch.equal(kc_d.cpu(), kc_ref) and torch.equal(vc_d.cpu(), vc_ref)


@pytest.mark.parametrize("bsz,hk,lens,cap,k_sel,append", [
    (1, 2, [10000], 10001, 78, True),            # the reference's own decode test shape, 50 % blocks
    (3, 2, [300, 64, 1], 400, 3, True),
    (2, 2, [500, 129], 512, 0, False),           # dense over the cache
    (4, 8, [4096, 1000, 4095, 77], 4160, 16, True),
    (2, 2, [63, 64], 128, 1, False),
])
def test_decode(bsz, hk, lens, cap, k_sel, append):
    _case(bsz, hk, lens, cap, k_sel, append, seed=bsz * 100 + hk)


def test_decode_golden(golden_dir):
    g = np.load(os.path.join(golden_dir, "stage2.npz"))
    bsz, hq, hk, d, cache = (int(x) for x in g["dec_shape"])
    q = torch.from_numpy(det_array((bsz, hq, 1, d), 301, 0.25)).to(torch.bfloat16)
    kc = torch.from_numpy(det_array((bsz, hk, cache + 1, d), 302, 0.25)).to(torch.bfloat16)
    vc = torch.from_numpy(det_array((bsz, hk, cache + 1, d), 303)).to(torch.bfloat16)
    idx = torch.from_numpy(det_perm_rows(bsz * hk, (cache + 1 + 63) // 64, 3, 304)).view(bsz, hk, 1, 3)
    out = infllm_v2.infllmv2_attn_with_kvcache(
        q.transpose(1, 2).contiguous().to(DEV), kc.transpose(1, 2).contiguous().to(DEV),
        vc.transpose(1, 2).contiguous().to(DEV),
        cache_seqlens=torch.full((bsz,), cache + 1, dtype=torch.int32, device=DEV), topk_idx=idx.to(DEV))
    mx, mr = err_stats(out.cpu(), torch.from_numpy(g["dec_out"]))
    assert mx <= MAX_ABS and mr <= MEAN_REL, (mx, mr)


def _topk(bsz, hk, lens, k_sel, seed):
    rng = np.random.default_rng(seed)
    rows = np.full((bsz, hk, 1, k_sel), -1, np.int32)
    for b in range(bsz):
        nblk = (lens[b] + 63) // 64
        for h in range(hk):
            pick = np.sort(rng.permutation(nblk)[:k_sel])
            rows[b, h, 0, :len(pick)] = pick
    return torch.from_numpy(rows)


@pytest.mark.parametrize("page,append", [(64, True), (256, False), (128, True)])
def test_decode_paged_cache(page, append):
    """A cache scattered over pages through a block table gives the results (and, with an append,
    the in-place update) of the same cache laid out contiguously."""
    bsz, hk, d, cap = 3, 2, 128, 1024
    lens = [700, 64, 1023 - (1 if append else 0)]
    q = det_tensor((bsz, 1, hk * 16, d), 41, 0.25)
    kc, vc = det_tensor((bsz, cap, hk, d), 42, 0.25), det_tensor((bsz, cap, hk, d), 43)
    kn = det_tensor((bsz, 1, hk, d), 44, 0.25) if append else None
    vn = det_tensor((bsz, 1, hk, d), 45) if append else None
    lens_t = torch.tensor(lens, dtype=torch.int32)
    idx = _topk(bsz, hk, [l + (1 if append else 0) for l in lens], 5, 46)
    ref, ref_lse = oracle.kvcache_decode(q, kc.clone(), vc.clone(), lens_t, idx, kn, vn)
    # scatter the pages
    per_seq = cap // page
    perm = torch.randperm(bsz * per_seq, generator=torch.Generator().manual_seed(3))
    table = perm.view(bsz, per_seq).to(torch.int32)
    kp = torch.zeros(bsz * per_seq, page, hk, d, dtype=kc.dtype)
    vp = torch.zeros_like(kp)
    for b in range(bsz):
        for j in range(per_seq):
            kp[table[b, j]] = kc[b, j * page:(j + 1) * page]
            vp[table[b, j]] = vc[b, j * page:(j + 1) * page]
    kp_d, vp_d = kp.to(DEV), vp.to(DEV)
    out, lse = infllm_v2.infllmv2_attn_with_kvcache(
        q.to(DEV), kp_d, vp_d, k=None if kn is None else kn.to(DEV), v=None if vn is None else vn.to(DEV),
        cache_seqlens=lens_t.to(DEV), block_table=table.to(DEV), topk_idx=idx.to(DEV),
        return_softmax_lse=True)
    mx, mr = err_stats(out.cpu(), ref)
    assert mx <= MAX_ABS and mr <= MEAN_REL, (mx, mr)
    assert (lse.cpu() - ref_lse).abs().max() < 2e-2
    if append:
        for b in range(bsz):
            pg, off = int(table[b, lens[b] // page]), lens[b] % page
            assert torch.equal(kp_d[pg, off].cpu(), kn[b, 0]) and torch.equal(vp_d[pg, off].cpu(), vn[b, 0])
    with pytest.raises(NotImplementedError):
        infllm_v2.infllmv2_attn_with_kvcache(q.to(DEV), kp_d, vp_d, cache_seqlens=lens_t.to(DEV),
                                             block_table=table.to(DEV),
                                             cache_leftpad=torch.zeros(bsz, dtype=torch.int32, device=DEV))


def test_decode_batch_idx_and_leftpad():
    """cache_batch_idx picks the cache row of each sequence; cache_leftpad shifts where its keys
    start (block indices then count from the first key)."""
    bsz, rows, hk, d, cap = 3, 5, 2, 128, 600
    q = det_tensor((bsz, 1, hk * 16, d), 51, 0.25)
    kc, vc = det_tensor((rows, cap, hk, d), 52, 0.25), det_tensor((rows, cap, hk, d), 53)
    slot = torch.tensor([4, 0, 2], dtype=torch.int32)
    pad = torch.tensor([0, 37, 130], dtype=torch.int32)
    end = torch.tensor([500, 300, 599], dtype=torch.int32)          # cache_seqlens: absolute ends
    n = [int(e - p) for e, p in zip(end, pad)]
    idx = _topk(bsz, hk, n, 4, 54)
    # dense equivalent: every sequence's keys moved to the front of its own row
    kd = torch.zeros(bsz, cap, hk, d, dtype=kc.dtype)
    vd = torch.zeros_like(kd)
    for b in range(bsz):
        kd[b, :n[b]] = kc[slot[b], pad[b]:end[b]]
        vd[b, :n[b]] = vc[slot[b], pad[b]:end[b]]
    ref, ref_lse = oracle.kvcache_decode(q, kd, vd, torch.tensor(n, dtype=torch.int32), idx)
    out, lse = infllm_v2.infllmv2_attn_with_kvcache(
        q.to(DEV), kc.to(DEV), vc.to(DEV), cache_seqlens=end.to(DEV), cache_batch_idx=slot.to(DEV),
        cache_leftpad=pad.to(DEV), topk_idx=idx.to(DEV), return_softmax_lse=True)
    mx, mr = err_stats(out.cpu(), ref)
    assert mx <= MAX_ABS and mr <= MEAN_REL, (mx, mr)
    assert (lse.cpu() - ref_lse).abs().max() < 2e-2


@pytest.mark.parametrize("rotary_dim,interleaved", [(128, True), (64, False), (32, True), (128, False)])
def test_decode_rotary_on_append(rotary_dim, interleaved):
    """rotary_cos / rotary_sin rotate the appended key and the query at the append position; the
    result equals the plain call on inputs rotated by the oracle, and the cache receives the
    rotated key."""
    bsz, hk, d, cap = 3, 2, 128, 700
    lens = [5, 300, 640]
    q = det_tensor((bsz, 1, hk * 16, d), 61, 0.25)
    kc, vc = det_tensor((bsz, cap, hk, d), 62, 0.25), det_tensor((bsz, cap, hk, d), 63)
    kn, vn = det_tensor((bsz, 1, hk, d), 64, 0.25), det_tensor((bsz, 1, hk, d), 65)
    ang = torch.arange(cap)[:, None] * (1.0 / 10000 ** (torch.arange(rotary_dim // 2) / (rotary_dim // 2)))[None, :]
    cos, sin = torch.cos(ang).to(torch.bfloat16), torch.sin(ang).to(torch.bfloat16)
    lens_t = torch.tensor(lens, dtype=torch.int32)
    idx = _topk(bsz, hk, [l + 1 for l in lens], 4, 66)
    pos = lens_t.long()
    q_rot = oracle.apply_rotary(q[:, 0], cos[pos][:, None], sin[pos][:, None], interleaved)[:, None]
    k_rot = oracle.apply_rotary(kn[:, 0], cos[pos][:, None], sin[pos][:, None], interleaved)[:, None]
    kc_ref, vc_ref = kc.clone(), vc.clone()
    ref, ref_lse = oracle.kvcache_decode(q_rot, kc_ref, vc_ref, lens_t, idx, k_rot, vn)
    kc_d, vc_d = kc.to(DEV), vc.to(DEV)
    out, lse = infllm_v2.infllmv2_attn_with_kvcache(
        q.to(DEV), kc_d, vc_d, k=kn.to(DEV), v=vn.to(DEV), rotary_cos=cos.to(DEV), rotary_sin=sin.to(DEV),
        cache_seqlens=lens_t.to(DEV), rotary_interleaved=interleaved, topk_idx=idx.to(DEV),
        return_softmax_lse=True)
    mx, mr = err_stats(out.cpu(), ref)
    assert mx <= MAX_ABS and mr <= MEAN_REL, (mx, mr)
    assert (lse.cpu() - ref_lse).abs().max() < 2e-2
    assert torch.equal(kc_d.cpu(), kc_ref) and torch.equal(vc_d.cpu(), vc_ref)     # rotated key in the cache


def test_decode_full_cache_and_lengths_beyond_the_capacity():
    """A sequence whose cache is full cannot take the new token: it is neither appended nor
    attended, so the result equals the call without k / v; a length beyond the capacity attends the
    positions that exist.  The caches sit between NaN guards, so a read past a sequence's rows
    would poison the output."""
    bsz, hk, cap, d = 3, 2, 256, 128
    hq = hk * 16
    q = det_tensor((bsz, 1, hq, d), 1, 0.25).to(DEV)
    guard = torch.full((bsz + 2, cap, hk, d), float("nan"), dtype=torch.bfloat16, device=DEV)
    kc_all, vc_all = guard.clone(), guard.clone()
    kc, vc = kc_all[1:-1], vc_all[1:-1]
    kc.copy_(det_tensor((bsz, cap, hk, d), 2, 0.25))
    vc.copy_(det_tensor((bsz, cap, hk, d), 3))
    kn = det_tensor((bsz, 1, hk, d), 4, 0.25).to(DEV)
    vn = det_tensor((bsz, 1, hk, d), 5).to(DEV)
    full = torch.tensor([cap, cap, 100], dtype=torch.int32, device=DEV)
    k_before, v_before = kc.clone(), vc.clone()
    with_new = infllm_v2.infllmv2_attn_with_kvcache(q, kc, vc, k=kn, v=vn, cache_seqlens=full)
    # sequences 0 and 1 are full: their rows are untouched; sequence 2 took the token
    assert torch.equal(kc[:2], k_before[:2]) and torch.equal(vc[:2], v_before[:2])
    assert torch.equal(kc[2, 100], kn[2, 0]) and torch.equal(vc[2, 100], vn[2, 0])
    without = infllm_v2.infllmv2_attn_with_kvcache(q, kc, vc, cache_seqlens=torch.tensor(
        [cap, cap, 101], dtype=torch.int32, device=DEV))
    assert not torch.isnan(with_new.float()).any()
    assert torch.equal(with_new, without)
    beyond = infllm_v2.infllmv2_attn_with_kvcache(q, kc, vc, cache_seqlens=torch.tensor(
        [cap + 1000, cap + 1, 101], dtype=torch.int32, device=DEV))
    assert torch.equal(beyond, without)
