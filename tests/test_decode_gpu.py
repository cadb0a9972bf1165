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
