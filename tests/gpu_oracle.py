"""Plain fp32 PyTorch restatements of stage 1 and stage 2 that run ON THE GPU, for parity checks
at sizes the CPU oracle cannot finish (the BASELINE configurations).  Test infrastructure only:
nothing in the package imports this file, and it calls none of the library's kernels -- only
torch matmul / softmax in fp32 (TF32 off).

The mathematics is that of oracle/stage1.py and oracle/attention.py (dense attention under the
block mask); the only difference is that a row's keys are GATHERED (the selected blocks, cut at the
causal limit) instead of being masked inside a dense score matrix, which is the same sum.
"""
import math

import torch

import oracle


def _fp32():
    torch.backends.cuda.matmul.allow_tf32 = False
    torch.backends.cudnn.allow_tf32 = False


def stage1_rows(q_rows, kc, tok_local, lq, causal=True, softmax_scale=None, group=16):
    """Stage-1 scores of sampled tokens of ONE sequence.  q_rows: (n, Hq, d) bf16 on the GPU, the
    rows of local tokens `tok_local` (n,) of a query segment of length lq; kc: (Lc, Hk, d).
    Returns fp32 (Hk, n, Lc): softmax over the visible compressed keys, summed over the group."""
    _fp32()
    n, hq, d = q_rows.shape
    lc, hk, _ = kc.shape
    scale = softmax_scale if softmax_scale is not None else 1.0 / math.sqrt(d)
    lim = oracle.stage1_visible_limit(tok_local.cpu().long(), lq, lc, causal).to(q_rows.device)
    qf = q_rows.float().view(n, hk, group, d)
    s = torch.einsum("nhgd,chd->hngc", qf, kc.float()) * scale
    vis = torch.arange(lc, device=q_rows.device)[None, :] < lim[:, None]          # (n, Lc)
    s = s.masked_fill(~vis[None, :, None, :], float("-inf"))
    lse = torch.logsumexp(s, dim=-1, keepdim=True)
    p = torch.exp(s - lse)
    p = torch.where(vis[None, :, None, :] & ~torch.isinf(lse), p, torch.zeros((), device=p.device))
    return p.sum(dim=2)


def _gather_keys(blocks, limit, device):
    """Key positions of the selected 64-key blocks below `limit` (exclusive)."""
    blocks = blocks[blocks >= 0].long()
    keys = (blocks[:, None] * 64 + torch.arange(64, device=device)[None, :]).reshape(-1)
    return keys[keys < limit]


def attend_rows(q_rows, tok_local, k_seq, v_seq, idx_rows, lq, causal=True, softmax_scale=None, group=16):
    """Stage-2 forward of sampled tokens of one sequence.  q_rows (n, Hq, d); tok_local (n,)
    local token indices in a query segment of length lq; k_seq, v_seq (Lk, Hk, d); idx_rows
    (Hk, n, topk) int32 block lists (-1 = unused) or None for dense.  Returns fp32 out (n, Hq, d)
    and lse (Hk, n, group) (+inf for a row that sees no key)."""
    _fp32()
    n, hq, d = q_rows.shape
    lk, hk, _ = k_seq.shape
    dev = q_rows.device
    scale = softmax_scale if softmax_scale is not None else 1.0 / math.sqrt(d)
    out = torch.zeros(n, hq, d, device=dev)
    lse = torch.full((hk, n, group), float("inf"), device=dev)
    toks = tok_local.tolist()
    for i, t in enumerate(toks):
        limit = min(lk, t + lk - lq + 1) if causal else lk
        for h in range(hk):
            if idx_rows is None:
                keys = torch.arange(max(limit, 0), device=dev)
            else:
                keys = _gather_keys(idx_rows[h, i], limit, dev)
            if keys.numel() == 0:
                continue
            kg, vg = k_seq[keys, h].float(), v_seq[keys, h].float()
            s = q_rows[i, h * group:(h + 1) * group].float() @ kg.t() * scale
            l = torch.logsumexp(s, dim=-1)
            out[i, h * group:(h + 1) * group] = torch.exp(s - l[:, None]) @ vg
            lse[h, i] = l
    return out, lse


def blockshared_fwd_bwd(q, k, v, dout, lens, idx, softmax_scale=None, group=16):
    """Forward and backward of causal varlen block-sparse self-attention (Lq = Lk per sequence)
    when the 64 tokens of a query block share one block list (the layout of the varlen training
    configuration).  q, dout: (T, Hq, d); k, v: (T, Hk, d); idx: (Hk, T, topk) int32.  One fp32
    dense-under-mask problem per (sequence, KV head, query block).  Returns fp32 out, dq, dk, dv."""
    _fp32()
    t_all, hq, d = q.shape
    hk = k.shape[1]
    dev = q.device
    scale = softmax_scale if softmax_scale is not None else 1.0 / math.sqrt(d)
    out = torch.zeros(t_all, hq, d, device=dev)
    dq = torch.zeros(t_all, hq, d, device=dev)
    dk = torch.zeros(t_all, hk, d, device=dev)
    dv = torch.zeros(t_all, hk, d, device=dev)
    start = 0
    ar64 = torch.arange(64, device=dev)
    for length in lens:
        for qb in range((length + 63) // 64):
            t0 = qb * 64
            nt = min(64, length - t0)
            rows = slice(start + t0, start + t0 + nt)
            tok = (t0 + ar64[:nt])                                       # local token per row
            for h in range(hk):
                blocks = idx[h, start + t0]
                keys = _gather_keys(blocks, length, dev)
                kg, vg = k[start + keys, h].float(), v[start + keys, h].float()
                qh = q[rows, h * group:(h + 1) * group].float().reshape(nt * group, d)
                doh = dout[rows, h * group:(h + 1) * group].float().reshape(nt * group, d)
                s = qh @ kg.t() * scale
                vis = keys[None, :] <= tok.repeat_interleave(group)[:, None]
                s = s.masked_fill(~vis, float("-inf"))
                p = torch.softmax(s, dim=-1)
                o = p @ vg
                dp = doh @ vg.t()
                dsum = (doh * o).sum(dim=-1, keepdim=True)
                ds = p * (dp - dsum)
                out[rows, h * group:(h + 1) * group] = o.view(nt, group, d)
                dq[rows, h * group:(h + 1) * group] = (ds @ kg * scale).view(nt, group, d)
                dk[:, h].index_add_(0, start + keys, ds.t() @ qh * scale)
                dv[:, h].index_add_(0, start + keys, p.t() @ doh)
        start += length
    return out, dq, dk, dv


def decode_rows(q, k_cache, v_cache, lens, idx, softmax_scale=None, group=16):
    """Sparse decode: q (B, 1, Hq, d), caches (B, cap, Hk, d), lens (B,) keys per sequence, idx
    (B, Hk, 1, topk) int32 or None.  Returns fp32 out (B, 1, Hq, d)."""
    _fp32()
    b, _, hq, d = q.shape
    hk = k_cache.shape[2]
    dev = q.device
    scale = softmax_scale if softmax_scale is not None else 1.0 / math.sqrt(d)
    out = torch.zeros(b, 1, hq, d, device=dev)
    for i, n in enumerate(lens.tolist()):
        for h in range(hk):
            keys = (torch.arange(n, device=dev) if idx is None else _gather_keys(idx[i, h, 0], n, dev))
            if keys.numel() == 0:
                continue
            s = q[i, 0, h * group:(h + 1) * group].float() @ k_cache[i, keys, h].float().t() * scale
            out[i, 0, h * group:(h + 1) * group] = torch.softmax(s, dim=-1) @ v_cache[i, keys, h].float()
    return out
