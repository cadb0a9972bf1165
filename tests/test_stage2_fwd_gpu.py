"""GPU: stage-2 block-sparse attention forward against the fp32 dense-with-mask oracle.
Tolerance (bf16 outputs): max-abs <= 2e-2 and mean-rel <= 1e-2."""
import os

import numpy as np
import pytest
import torch

import oracle
import infllm_v2
from helpers import det_tensor, cu, local_topk, err_stats
from inputs import det_array, det_perm_rows

pytestmark = pytest.mark.gpu
DEV = "cuda"
MAX_ABS, MEAN_REL = 2e-2, 1e-2


def _run(q, k, v, cu_q, cu_k, idx, causal):
    out, lse, _ = infllm_v2.infllmv2_attn_varlen_func(
        q.to(DEV), k.to(DEV), v.to(DEV), cu_q.to(DEV), cu_k.to(DEV),
        int((cu_q[1:] - cu_q[:-1]).max()), int((cu_k[1:] - cu_k[:-1]).max()),
        causal=causal, topk_idx=None if idx is None else idx.to(DEV), return_attn_probs=True)
    infllm_v2.check_device_status()
    return out.cpu(), lse.cpu()


def _check(q, k, v, cu_q, cu_k, idx, causal):
    out, lse = _run(q, k, v, cu_q, cu_k, idx, causal)
    ref, ref_lse = oracle.sparse_attention_fwd(q, k, v, cu_q, cu_k, idx, causal=causal)
    assert not torch.isnan(out.float()).any()
    mx, mr = err_stats(out, ref)
    assert mx <= MAX_ABS and mr <= MEAN_REL, (mx, mr)
    empty = torch.isinf(ref_lse)
    assert torch.equal(torch.isinf(lse) & (lse > 0), empty)
    assert (lse[~empty] - ref_lse[~empty]).abs().max() < 2e-2
    return out


@pytest.mark.parametrize("lens_q,lens_k,k_sel,causal", [
    ([128], [128], 2, True), ([200, 136], [200, 136], 3, True), ([64, 192], [160, 300], 3, True),
    ([1000], [1000], 8, True), ([77, 5, 130], [77, 5, 130], 2, True), ([256], [256], 4, False),
    ([8], [8], 1, True), ([3], [700], 4, True),
])
def test_fwd_sparse(lens_q, lens_k, k_sel, causal):
    hq, hk, d = 32, 2, 128
    seed = sum(lens_q) + k_sel
    q = det_tensor((sum(lens_q), hq, d), seed, 0.25)
    k = det_tensor((sum(lens_k), hk, d), seed + 1, 0.25)
    v = det_tensor((sum(lens_k), hk, d), seed + 2)
    idx = local_topk(hk, lens_q, lens_k, k_sel, seed)
    _check(q, k, v, cu(lens_q), cu(lens_k), idx, causal)


def test_fwd_dense_and_large_scores():
    # dense (topk_idx=None) with scores large enough to force accumulator rescales
    hq, hk, d = 32, 2, 128
    q = det_tensor((300, hq, d), 1, 1.0)
    k = det_tensor((300, hk, d), 2, 1.0)
    v = det_tensor((300, hk, d), 3)
    _check(q, k, v, cu([300]), cu([300]), None, True)


def test_fwd_rows_without_keys_and_unselected_blocks():
    hq, hk, d = 32, 2, 128
    q = det_tensor((130, hq, d), 4, 0.25)
    k = det_tensor((130, hk, d), 5, 0.25)
    v = det_tensor((130, hk, d), 6)
    idx = torch.full((hk, 130, 2), -1, dtype=torch.int32)
    idx[:, 70:, 0] = 0                      # tokens < 70 select nothing at all
    idx[0, 100:, 1] = 1
    out = _check(q, k, v, cu([130]), cu([130]), idx, True)
    assert out[:70].abs().max() == 0


def test_fwd_golden_inputs(golden_dir):
    g = np.load(os.path.join(golden_dir, "stage2.npz"))
    step = int(g["out_row_step"])
    hq, hk, d = 32, 2, 128
    for name in ("a", "b", "c"):
        seed, k_sel = (int(x) for x in g[f"s2_{name}_seed"])
        cu_q, cu_k = torch.from_numpy(g[f"s2_{name}_cuq"]), torch.from_numpy(g[f"s2_{name}_cuk"])
        sk = int((cu_k[1:] - cu_k[:-1]).max())
        q = torch.from_numpy(det_array((int(cu_q[-1]), hq, d), seed, 0.25)).to(torch.bfloat16)
        k = torch.from_numpy(det_array((int(cu_k[-1]), hk, d), seed + 1000, 0.25)).to(torch.bfloat16)
        v = torch.from_numpy(det_array((int(cu_k[-1]), hk, d), seed + 2000)).to(torch.bfloat16)
        idx = torch.from_numpy(det_perm_rows(hk * int(cu_q[-1]), (sk + 63) // 64, k_sel, seed + 3000)
                               ).view(hk, -1, k_sel)
        for causal in (0, 1):
            key = f"s2_{name}_{causal}_out"
            if key not in g.files:
                continue
            out, _ = _run(q, k, v, cu_q, cu_k, idx, bool(causal))
            mx, mr = err_stats(out[::step], torch.from_numpy(g[key]))
            assert mx <= MAX_ABS and mr <= MEAN_REL, (key, mx, mr)


def test_fwd_multiword_mask_eight_kv_heads():
    # 8 KV heads, > 64 key blocks (two mask words), block lists shared per 64-token query block
    hq, hk, d = 128, 8, 128
    lens = [4500]
    q = det_tensor((lens[0], hq, d), 21, 0.25)
    k = det_tensor((lens[0], hk, d), 22, 0.25)
    v = det_tensor((lens[0], hk, d), 23)
    idx = local_topk(hk, lens, lens, 6, 24, shared_per_block=True)
    out, _ = _run(q, k, v, cu(lens), cu(lens), idx, True)
    sl = slice(4300, 4500)                     # check the tail rows (most blocks) on the CPU oracle
    ref, _ = oracle.sparse_attention_fwd(q, k, v, cu(lens), cu(lens), idx, causal=True)
    mx, mr = err_stats(out[sl], ref[sl])
    assert mx <= MAX_ABS and mr <= MEAN_REL, (mx, mr)
