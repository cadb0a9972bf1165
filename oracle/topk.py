"""Per-query top-k block selection oracle.  Test infrastructure only.

The reference leaves selection to its caller (README.md:40-42); the ordering rule restated
here is the one its own bitonic top-k uses (csrc/topk.cuh:17, 26, 37): larger value first,
equal values -> smaller index first.  That equals a stable descending sort.  Pinned:
`bitonic_topk_literal` below simulates the reference's kernel thread for thread, and
tests/golden/make_golden.py asserts that `topk_select` picks the same blocks in the same order
on tie-heavy rows with +-inf (fixtures bitonic_* in tests/golden/pool_topk.npz).
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


def bitonic_topk_literal(x, top: int):
    """Thread-for-thread simulation of the reference's own top-k kernel, used to pin
    `topk_select`: kernel_bitonic_topk_multiblock<T, N, false> launched by bitonic_topk with one
    block of n threads per row (csrc/topk.cuh:98-117, 141-161), i.e. warpBitonicSort (:6-23) on
    groups of N lanes, blockBitonicReduce (:43-69) with warpBitonicMerge (:24-42) over shared
    memory, and the final 32-lane sort.  Every `__shfl_xor_sync(…, j)` becomes a gather from
    thread `tid ^ j`; the predicate of each compare-exchange is restated term by term.

    x: float array (rows, n), n a multiple of 32 and <= 1024; N = `top` rounded up to a power of
    two (TOPK_SIZE_DISPATCH, :119-139; at most 32).  Returns (values, positions), each
    (rows, N), in the kernel's output order (threads 0..N-1)."""
    import numpy as np
    x = np.asarray(x, dtype=np.float32)
    rows, n = x.shape
    assert n % 32 == 0 and 32 <= n <= 1024 and 1 <= top <= 32
    N = 1
    while N < top:
        N *= 2
    tid = np.arange(n)
    v, pos = x.copy(), np.broadcast_to(tid, (rows, n)).copy()

    def first_wins(v1, p1, v2, p2):              # v1 > v2 || (v1 == v2 && pos < pos2)
        return (v1 > v2) | ((v1 == v2) & (p1 < p2))

    def second_wins(v1, p1, v2, p2):             # v1 < v2 || (v1 == v2 && pos1 > pos2)
        return (v1 < v2) | ((v1 == v2) & (p1 > p2))

    def warp_sort(v, pos, width, asc, threads):  # warpBitonicSort<T, width> run by `threads`
        lane = threads & (width - 1)
        k = 2
        while k <= width:
            desc = ((lane & k) == 0) ^ asc
            j = k // 2
            while j > 0:
                v2, p2 = v[:, threads ^ j], pos[:, threads ^ j]
                v1, p1 = v[:, threads], pos[:, threads]
                upper = (lane & j) != 0
                take = desc[None, :] ^ first_wins(v1, p1, v2, p2) ^ upper[None, :]
                v[:, threads] = np.where(take, v2, v1)
                pos[:, threads] = np.where(take, p2, p1)
                j //= 2
            k *= 2

    def warp_merge(v, pos, nv, npos, threads):   # warpBitonicMerge<T, N> run by `threads`
        lane = threads & (N - 1)
        v1, p1 = v[:, threads], pos[:, threads]
        take = second_wins(v1, p1, nv, npos)
        v[:, threads] = np.where(take, nv, v1)
        pos[:, threads] = np.where(take, npos, p1)
        j = N // 2
        while j > 0:
            v2, p2 = v[:, threads ^ j], pos[:, threads ^ j]
            v1, p1 = v[:, threads], pos[:, threads]
            upper = (lane & j) != 0
            take = second_wins(v1, p1, v2, p2) ^ upper[None, :]
            v[:, threads] = np.where(take, v2, v1)
            pos[:, threads] = np.where(take, p2, p1)
            j //= 2

    warp_sort(v, pos, N, False, tid)             # `ordered` = false: local sort, descending
    # blockBitonicReduce: shared copies, halve the number of live threads down to one warp
    sh_v, sh_p = v.copy(), pos.copy()
    i = 512
    while i >= 32:
        if n > i:
            threads = np.arange(i)
            nxt = 2 * i - threads - 1
            inside = nxt < n
            nv = np.where(inside[None, :], sh_v[:, np.minimum(nxt, n - 1)], -np.inf).astype(np.float32)
            npos = np.where(inside[None, :], sh_p[:, np.minimum(nxt, n - 1)], -1)
            warp_merge(v, pos, nv, npos, threads)
            sh_v[:, threads], sh_p[:, threads] = v[:, threads], pos[:, threads]
        i //= 2
    warp_sort(v, pos, 32, False, np.arange(32))
    return v[:, :N].copy(), pos[:, :N].copy()
