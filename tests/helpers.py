"""Shared helpers for the parity tests."""
import numpy as np
import torch

from inputs import det_array, det_perm_rows  # tests/golden/inputs.py


def det_tensor(shape, seed, scale=1.0, dtype=torch.bfloat16, device="cpu"):
    return torch.from_numpy(det_array(shape, seed, scale)).to(dtype).to(device)


def cu(lens, device="cpu"):
    return torch.tensor(np.concatenate([[0], np.cumsum(lens)]), dtype=torch.int32, device=device)


def local_topk(hk, lens_q, lens_k, k_sel, seed, shared_per_block=False):
    """Random sorted block lists per (head, token) with indices valid for the token's own
    sequence (and not in the causal future), -1 padded: (hk, sum(lens_q), k_sel) int32."""
    rng = np.random.default_rng(seed)
    rows = []
    for h in range(hk):
        per_head = []
        for lq, lk in zip(lens_q, lens_k):
            nblk = (lk + 63) // 64
            for i in range(lq):
                if shared_per_block and i % 64 != 0:
                    per_head.append(per_head[-1])
                    continue
                lim = min(nblk, max((i + lk - lq) // 64 + 1, 0))
                pick = np.sort(rng.permutation(lim)[:k_sel]) if lim > 0 else np.zeros(0, np.int64)
                row = np.full(k_sel, -1, np.int32)
                row[:len(pick)] = pick
                per_head.append(row)
        rows.append(np.stack(per_head))
    return torch.from_numpy(np.stack(rows))


def err_stats(got, ref):
    got, ref = got.float(), ref.float()
    diff = (got - ref).abs()
    return diff.max().item(), (diff.mean() / ref.abs().mean().clamp_min(1e-12)).item()
