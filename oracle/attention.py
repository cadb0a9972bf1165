"""Stage-2 block-sparse attention oracle (fp32 dense-with-mask, CPU).  Test infrastructure only.

Follows tests/utils.py:224-260 (convert_topk_to_base_blockmask), :1027-1085
(prepare_mixed_mask), :1133-1195 (attention_blocksparse_ref, upcast=True) for the forward and
uses autograd of the same expression for dQ/dK/dV; the visibility rule is the device rule of
csrc/flash_attn/src/mask.h:181-203 (bottom-right aligned causal mask) combined with the
per-token block mask of flash_blockmask.h:26-31.  Decode follows tests/test_kvcache_simple.py:5-15
and csrc/flash_attn/flash_api.cpp:1628 (a single query token is never causally masked).
"""
import math
import torch


def expand_topk_mask(topk_idx: torch.Tensor, k_blocks: int) -> torch.Tensor:
    """int32 (Hk, T, k) block lists (-1 = unused) -> bool (Hk, T, k_blocks)."""
    hk, t, k = topk_idx.shape
    m = torch.zeros(hk, t, k_blocks + 1, dtype=torch.bool)
    idx = topk_idx.long()
    idx = torch.where((idx < 0) | (idx >= k_blocks), torch.tensor(k_blocks), idx)
    m.scatter_(2, idx, True)
    return m[..., :k_blocks]


def _seq_attention(q, k, v, blk_mask, causal, scale, block_size):
    """q: (Lq, Hq, d) fp32, k/v: (Lk, Hk, d) fp32, blk_mask: bool (Hk, Lq, nblk) or None.
    Returns out (Lq, Hq, d) fp32 and lse (Hq, Lq) fp32 (+inf for rows that see no key)."""
    lq, hq, d = q.shape
    lk, hk, _ = k.shape
    g = hq // hk
    s = torch.einsum("thd,shd->hts", q, k.repeat_interleave(g, dim=1)) * scale   # (Hq, Lq, Lk)
    vis = torch.ones(hk, lq, lk, dtype=torch.bool)
    if blk_mask is not None:
        vis = blk_mask.repeat_interleave(block_size, dim=2)[..., :lk]
        if vis.shape[-1] < lk:                       # mask narrower than the keys: rest unselected
            vis = torch.nn.functional.pad(vis, (0, lk - vis.shape[-1]))
    if causal:
        i = torch.arange(lq)[:, None]
        j = torch.arange(lk)[None, :]
        vis = vis & (j <= i + lk - lq)[None]
    vis = vis.repeat_interleave(g, dim=0)
    s = s.masked_fill(~vis, float("-inf"))
    lse = torch.logsumexp(s, dim=-1)
    p = torch.exp(s - lse.masked_fill(lse == float("-inf"), 0.0)[..., None])
    p = torch.where(vis, p, torch.zeros((), dtype=p.dtype))
    out = torch.einsum("hts,shd->thd", p, v.repeat_interleave(g, dim=1))
    lse = torch.where(lse == float("-inf"), torch.tensor(float("inf")), lse)
    return out, lse


def sparse_attention_fwd(q, k, v, cu_seqlens_q, cu_seqlens_k, topk_idx, causal=True,
                         softmax_scale=None, block_size: int = 64):
    """Varlen block-sparse attention.  q: (T, Hq, d); k, v: (Tk, Hk, d); topk_idx: int32
    (Hk, T, k) with block indices local to each sequence's keys (rows indexed by the global
    token), or None for dense attention.  Returns fp32 out (T, Hq, d) and lse (Hk, T*g) whose
    row index is token*g + head-in-group (csrc/flash_attn/flash_api.cpp:665)."""
    t, hq, d = q.shape
    hk = k.shape[1]
    g = hq // hk
    scale = softmax_scale if softmax_scale is not None else 1.0 / math.sqrt(d)
    cu_q = [int(x) for x in cu_seqlens_q]
    cu_k = [int(x) for x in cu_seqlens_k]
    outs, lses = [], []
    for b in range(len(cu_q) - 1):
        q0, q1, k0, k1 = cu_q[b], cu_q[b + 1], cu_k[b], cu_k[b + 1]
        lk = k1 - k0
        bm = None
        if topk_idx is not None:
            bm = expand_topk_mask(topk_idx[:, q0:q1], (lk + block_size - 1) // block_size)
        o, l = _seq_attention(q[q0:q1].float(), k[k0:k1].float(), v[k0:k1].float(),
                              bm, causal, scale, block_size)
        outs.append(o)
        lses.append(l)
    out = torch.cat(outs, 0)
    lse = torch.cat(lses, 1)                                     # (Hq, T)
    lse = lse.view(hk, g, t).permute(0, 2, 1).reshape(hk, t * g)
    return out, lse


def sparse_attention_fwd_bwd(q, k, v, dout, cu_seqlens_q, cu_seqlens_k, topk_idx, causal=True,
                             softmax_scale=None, block_size: int = 64):
    """Forward plus dQ, dK, dV by autograd on the fp32 expression."""
    qf = q.detach().float().requires_grad_(True)
    kf = k.detach().float().requires_grad_(True)
    vf = v.detach().float().requires_grad_(True)
    out, lse = sparse_attention_fwd(qf, kf, vf, cu_seqlens_q, cu_seqlens_k, topk_idx, causal,
                                    softmax_scale, block_size)
    dq, dk, dv = torch.autograd.grad(out, (qf, kf, vf), dout.float())
    return out.detach(), lse.detach(), dq, dk, dv


def kvcache_decode(q, k_cache, v_cache, cache_seqlens, topk_idx=None, k_new=None, v_new=None,
                   softmax_scale=None, block_size: int = 64):
    """q: (B, 1, Hq, d); caches (B, S, Hk, d) updated in place at cache_seqlens[b] when k_new /
    v_new (B, 1, Hk, d) are given; topk_idx (B, Hk, 1, k) or None.  Returns fp32 out
    (B, 1, Hq, d) and lse (B, Hq, 1)."""
    b, sq, hq, d = q.shape
    assert sq == 1
    hk = k_cache.shape[2]
    scale = softmax_scale if softmax_scale is not None else 1.0 / math.sqrt(d)
    outs, lses = [], []
    for i in range(b):
        n = int(cache_seqlens[i])
        if k_new is not None:
            k_cache[i, n:n + 1] = k_new[i]
            v_cache[i, n:n + 1] = v_new[i]
            n += 1
        bm = None
        if topk_idx is not None:
            bm = expand_topk_mask(topk_idx[i], (n + block_size - 1) // block_size)
        o, l = _seq_attention(q[i].float(), k_cache[i, :n].float(), v_cache[i, :n].float(),
                              bm, False, scale, block_size)
        outs.append(o)
        lses.append(l)
    return torch.stack(outs, 0), torch.stack(lses, 0)


def apply_rotary(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, interleaved: bool) -> torch.Tensor:
    """Rotary embedding of rows x (..., d) with per-row cos / sin (..., rotary_dim / 2), the way the
    reference rotates q and the appended key of a decode step (csrc/flash_attn/src/rotary.h:20-79
    interleaved, :83-150 contiguous halves): fp32 arithmetic, features past rotary_dim unchanged,
    result in x's dtype.  Pinned by `apply_rotary_literal`, an element-by-element restatement of the
    two device loops (tests/golden/make_golden.py asserts equality, fixtures rotary_* in stage2.npz)."""
    half = cos.shape[-1]
    xf, c, s_ = x.float(), cos.float(), sin.float()
    out = xf.clone()
    if interleaved:
        x0, x1 = xf[..., 0:2 * half:2], xf[..., 1:2 * half:2]
        out[..., 0:2 * half:2] = x0 * c - x1 * s_
        out[..., 1:2 * half:2] = x0 * s_ + x1 * c
    else:
        x0, x1 = xf[..., :half], xf[..., half:2 * half]
        out[..., :half] = x0 * c - x1 * s_
        out[..., half:2 * half] = x0 * s_ + x1 * c
    return out.to(x.dtype)


def apply_rotary_literal(x, cos, sin, interleaved: bool):
    """Element-by-element restatement of the reference's two rotary copy loops, the pin of
    `apply_rotary`: copy_rotary_interleaved (csrc/flash_attn/src/rotary.h:20-79: pairs (2i, 2i+1),
    real = x0*cos - x1*sin, imag = x0*sin + x1*cos) and copy_rotary_contiguous (:83-150: feature j
    pairs with j +- rotary_dim/2, out = x[j]*cos + other*(-sin for the left half, +sin for the
    right)), both in fp32 with one rounding to the storage type; features at or past rotary_dim are
    copied.  x: (rows, d) array of values exactly representable in the storage type, cos / sin:
    (rows, rotary_dim / 2).  Returns float32 (rows, d) BEFORE the final rounding."""
    import numpy as np
    x = np.asarray(x, dtype=np.float32)
    cos = np.asarray(cos, dtype=np.float32)
    sin = np.asarray(sin, dtype=np.float32)
    rows, d = x.shape
    half = cos.shape[1]
    rotary_dim = 2 * half
    out = x.copy()
    for r in range(rows):
        if interleaved:
            for i in range(half):
                x0, x1 = x[r, 2 * i], x[r, 2 * i + 1]
                out[r, 2 * i] = np.float32(x0 * cos[r, i]) - np.float32(x1 * sin[r, i])
                out[r, 2 * i + 1] = np.float32(x0 * sin[r, i]) + np.float32(x1 * cos[r, i])
        else:
            for j in range(rotary_dim):
                is_left = j < half
                other = x[r, j + half] if is_left else x[r, j - half]
                i = j if is_left else j - half
                out[r, j] = np.float32(x[r, j] * cos[r, i]) + np.float32(other * (-sin[r, i] if is_left else sin[r, i]))
    return out
