"""Per-query top-k block selection oracle.  Test infrastructure only.

The reference leaves selection to its caller (README.md:40-42); the ordering rule restated
here is the one its own bitonic top-k uses (csrc/topk.cuh:17, 26, 37): larger value first,
equal values -> smaller index first.  That equals a stable descending sort.  No reference
test pins this function ("parity unpinned" for top-k); the rule itself is pinned by
tests/golden KATs derived from the comparison in csrc/topk.cuh.
"""
import torch


def topk_select(block_score: torch.Tensor, k: int, q_block: torch.Tensor) -> torch.Tensor:
    """block_score: (Hk, T, n_blocks) (any float dtype); q_block: (T,) block index of each
    query token (indices strictly greater than it are dropped).  Returns int32 (Hk, T, k):
    the chosen block indices ascending, -1 in the unused tail."""
    hk, t, n = block_score.shape
    kk = min(k, n)
    order = torch.sort(block_score.float(), dim=-1, descending=True, stable=True).indices[..., :kk]
    order = order.sort(dim=-1).values
    future = order > q_block.view(1, t, 1).to(order.dtype)
    big = torch.iinfo(torch.int64).max
    order = torch.where(future, torch.tensor(big), order).sort(dim=-1).values
    order = torch.where(order == big, torch.tensor(-1), order)
    out = torch.full((hk, t, k), -1, dtype=torch.int32)
    out[..., :kk] = order.to(torch.int32)
    return out
