"""Stage-1 scorer oracle (fp32, CPU).  Test infrastructure only.

Follows tests/stage1/naive_softmax.py:4-41 and the varlen wrapper tests/test_stage1.py:11-84;
the visibility limit is the device form of csrc/flash_attn/src/mask.h:270-281 with
flash_fwd_kernel.h:1247-1265 (C integer division), which equals the Python form of the test
oracle whenever q_len >= 15.
"""
import math
import torch


def _cdiv_trunc(a: int, b: int) -> int:
    """C integer division (truncation toward zero)."""
    q = abs(a) // b
    return q if a >= 0 else -q


def stage1_visible_limit(i: torch.Tensor, q_len: int, k_len: int, causal: bool,
                         stride: int = 16) -> torch.Tensor:
    """Number of leading compressed keys visible to local query token i (mask.h:270-281):
    key j is visible iff j < limit.  Compressed key j covers tokens [stride*j, stride*j + 2*stride);
    stride 16 for the scored keys, 64 for the coarse keys of the "compressed LSE" mode."""
    if not causal:
        return torch.full_like(i, k_len)
    off = k_len - _cdiv_trunc(q_len - stride + 1, stride)
    lim = (i + 1) // stride - 1 + off
    return lim.clamp(0, k_len)


def compress_keys(k: torch.Tensor, cu_seqlens, kernel: int = 32, stride: int = 16):
    """Mean-pool keys (total_k, Hk, d) per sequence with the given window
    (tests/test_stage1_compressed_lse.py:56-99).  Returns (kc, cu_seqlens_c list)."""
    cu = [int(v) for v in cu_seqlens]
    parts, cu_c = [], [0]
    for b in range(len(cu) - 1):
        seg = k[cu[b]:cu[b + 1]].float()
        n = (seg.shape[0] - kernel) // stride + 1 if seg.shape[0] >= kernel else 0
        if n > 0:
            win = seg.unfold(0, kernel, stride)[:n]          # (n, Hk, d, kernel)
            parts.append(win.mean(dim=-1))
        cu_c.append(cu_c[-1] + max(n, 0))
    kc = torch.cat(parts, 0) if parts else k.new_zeros((0,) + k.shape[1:]).float()
    return kc.to(k.dtype), cu_c


def stage1_scores(q: torch.Tensor, kc: torch.Tensor, cu_seqlens_q, cu_seqlens_k,
                  max_seqlen_k: int, causal: bool, softmax_scale=None,
                  group: int = 16, chunk: int = 512, lse_keys=None, cu_seqlens_v=None) -> torch.Tensor:
    """q: (T, Hq, d), kc: (sum Lc, Hk, d).  Returns fp32 (Hk, T, max_seqlen_k): for every KV
    head the softmax probabilities over the visible compressed keys, summed over the `group`
    query heads that share it; invisible / padded columns and rows with no visible key are 0.

    lse_keys / cu_seqlens_v ("compressed LSE" mode, tests/stage1/complse_online_softmax.py:21-108
    and flash_fwd_kernel.h:1236-1240): the log-sum-exp of a row is taken over these keys instead
    -- with the stride-64 visibility rule when a sequence has a different number of them than of
    scored keys -- and the result is exp(q.k - lse) summed over the heads.  A row that sees no such
    key scores 0 everywhere (the reference oracle's running sum turns NaN there and NaNs are
    scrubbed to 0, complse_online_softmax.py:84-85, 104)."""
    t, hq, d = q.shape
    hk = kc.shape[1]
    assert hq == hk * group
    scale = softmax_scale if softmax_scale is not None else 1.0 / math.sqrt(d)
    cu_q = [int(v) for v in cu_seqlens_q]
    cu_k = [int(v) for v in cu_seqlens_k]
    cu_v = [int(v) for v in cu_seqlens_v] if lse_keys is not None else cu_k
    kv_all = lse_keys if lse_keys is not None else kc
    out = torch.zeros(hk, t, max_seqlen_k, dtype=torch.float32)
    for b in range(len(cu_q) - 1):
        q0, q1, k0, k1 = cu_q[b], cu_q[b + 1], cu_k[b], cu_k[b + 1]
        v0, v1 = cu_v[b], cu_v[b + 1]
        lq, lc, lcv = q1 - q0, k1 - k0, v1 - v0
        if lq <= 0 or lc <= 0:
            continue
        st1 = 16 if lcv == lc else 64
        kb = kc[k0:k1].float().permute(1, 2, 0)                       # (Hk, d, Lc)
        vb = kv_all[v0:v1].float().permute(1, 2, 0)                   # (Hk, d, Lcv)
        for s in range(0, lq, chunk):
            e = min(lq, s + chunk)
            qb = q[q0 + s:q0 + e].float().view(e - s, hk, group, d).permute(1, 2, 0, 3)
            rows = torch.arange(s, e)
            # log-sum-exp over the pass-1 keys
            s1 = torch.matmul(qb, vb[:, None]) * scale                # (Hk, g, n, Lcv)
            lim1 = stage1_visible_limit(rows, lq, lcv, causal, st1)
            s1 = s1.masked_fill((torch.arange(lcv)[None, :] >= lim1[:, None])[None, None], float("-inf"))
            lse = torch.logsumexp(s1, dim=-1, keepdim=True)           # -inf for a row that sees nothing
            # scores of the pass-2 keys against that normaliser
            sc = torch.matmul(qb, kb[:, None]) * scale                # (Hk, g, n, Lc)
            lim = stage1_visible_limit(rows, lq, lc, causal)
            hidden = (torch.arange(lc)[None, :] >= lim[:, None])[None, None]
            p = torch.exp(sc - lse)
            dead = hidden | torch.isinf(lse) | torch.isnan(p)         # no pass-1 key: 0, not +inf
            p = torch.where(dead, torch.zeros((), dtype=p.dtype), p).sum(dim=1)
            out[:, q0 + s:q0 + e, :lc] = p
    return out
