"""Max-pool oracle: compressed-key scores -> 64-token block scores.  Test infrastructure only.

Follows csrc/max_pooling_1d.cuh:106-160 (fixed length) and :11-103 (varlen), with the
wrapper arithmetic of infllm_v2/max_pooling_1d.py:14-21, 93-110.  Pure comparisons, so the
result is bit-exact for bf16/fp16 inputs (computed here on the fp32 image of the values).
"""
import numpy as np
import torch


def _pool_rows(x: torch.Tensor, k_len: int, out_len: int, bq: torch.Tensor,
               local_blocks: int, init_blocks: int, stride: int) -> torch.Tensor:
    """x: (..., R, >=k_len) fp32 rows; bq: (R,) query block index per row."""
    kernel, pad = stride + 1, 1
    xs = x[..., :k_len]
    width = stride * out_len + kernel
    buf = torch.full(x.shape[:-1] + (width,), float("-inf"), dtype=torch.float32)
    n = min(k_len, width - pad)
    buf[..., pad:pad + n] = xs[..., :n]
    win = buf.unfold(-1, kernel, stride)[..., :out_len, :]       # window b = x[stride*b-1 .. stride*b+stride]
    y = win.max(dim=-1).values
    b = torch.arange(out_len)
    forced = (b[None, :] < init_blocks) | ((bq[:, None] >= b[None, :]) &
                                           (bq[:, None] <= b[None, :] + local_blocks))
    return torch.where(forced, torch.tensor(float("inf")), y)


def max_pooling_1d(x: torch.Tensor, cache_len: int, local_blocks: int, init_blocks: int,
                   block_size: int = 64, stride: int = 16) -> torch.Tensor:
    """x: (Hk, q_len, k_len) -> (Hk, q_len, ceil((q_len+cache_len)/block_size)), dtype of x."""
    hk, q_len, k_len = x.shape
    s = block_size // stride
    out_len = (q_len + cache_len + block_size - 1) // block_size
    bq = (torch.arange(q_len) + cache_len) // block_size
    y = _pool_rows(x.float(), k_len, out_len, bq, local_blocks, init_blocks, s)
    return y.to(x.dtype)


def max_pooling_1d_varlen(x: torch.Tensor, cu_seqlens_q, cu_seqlens_k, cache_lens,
                          max_seqlen_q: int, max_seqlen_k: int, local_blocks: int,
                          init_blocks: int, block_size: int = 64, stride: int = 16) -> torch.Tensor:
    """x: (Hk, total_q, max_k) packed rows; per sequence the key length and cache length differ."""
    hk, total_q, max_k = x.shape
    cu_q = [int(v) for v in cu_seqlens_q]
    cu_k = [int(v) for v in cu_seqlens_k]
    cl = [int(v) for v in cache_lens]
    s = block_size // stride
    out_len = (max_seqlen_q + max(cl) + block_size - 1) // block_size
    out = torch.zeros(hk, total_q, out_len, dtype=x.dtype)
    for b in range(len(cl)):
        q0, q1 = cu_q[b], cu_q[b + 1]
        if q1 <= q0:
            continue
        k_len = cu_k[b + 1] - cu_k[b]
        bq = (torch.arange(q1 - q0) + cl[b]) // block_size
        y = _pool_rows(x[:, q0:q1].float(), k_len, out_len, bq, local_blocks, init_blocks, s)
        out[:, q0:q1] = y.to(x.dtype)
    return out


def max_pooling_1d_literal(x: np.ndarray, cache_len: int, local_blocks: int, init_blocks: int,
                           block_size: int = 64, stride: int = 16) -> np.ndarray:
    """Loop-for-loop transliteration of the kernel body; small cases only (pins the fast form)."""
    hk, q_len, k_len = x.shape
    s, kernel, pad = block_size // stride, block_size // stride + 1, 1
    out_len = (q_len + cache_len + block_size - 1) // block_size
    y = np.zeros((hk, q_len, out_len), dtype=np.float32)
    for h in range(hk):
        for q in range(q_len):
            bq = (q + cache_len) // block_size
            for b in range(out_len):
                if b < init_blocks or (bq >= b and bq <= b + local_blocks):
                    y[h, q, b] = np.inf
                    continue
                st, en = max(b * s - pad, 0), min(b * s - pad + kernel, k_len)
                y[h, q, b] = x[h, q, st:en].max() if en > st else -np.inf
    return y
