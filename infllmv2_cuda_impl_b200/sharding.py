"""Partitioning of the sparse-attention path over the GPUs of one box (one process per GPU).

The path shards along three independent axes, none of which needs cross-shard arithmetic:

* KV-head groups (tensor parallel): every kernel's grid has an independent KV-head axis and the
  masks / top-k lists are per KV head -> `head_shard`; no collective at all.
* sequences of a batch (decode, packed training batches) -> `batch_shard`; no collective.
* query-sequence chunks for long prefill when there are fewer KV heads than GPUs: rank r owns
  the zig-zag chunks {r, 2R-1-r} of the sequence (balanced causal work) and needs the keys
  BEFORE each chunk's end -> one exchange step, an all-gather of the compressed keys and of K/V
  into local HBM (NCCL over NVLink; payloads are MBs).  Each chunk is then an ordinary call with
  seqlen_q < seqlen_k: the stage-1 and stage-2 kernels align the causal diagonal bottom-right
  and the pool / top-k kernels take the chunk start as `cache_len`.

The reference has no distributed code; the chunk layout follows the contract visible in its
tests (tests/test_stage1_cp_load.py:43-47: head, tail = cp_rank + 1, 2*cp - cp_rank).
Kernels only ever read local memory; nothing here uses peer pointers or multicast.
"""
from dataclasses import dataclass
from typing import Callable, List, Optional, Sequence, Tuple

import torch
import torch.distributed as dist


_cu_cache = {}


def _cu_pair(n: int, device) -> torch.Tensor:
    """int32 [0, n] on `device`, built once per (device, n): creating it per call would be a
    blocking pageable host->device copy in the middle of a pipelined step."""
    key = (str(device), int(n))
    t = _cu_cache.get(key)
    if t is None:
        if len(_cu_cache) > 4096:
            _cu_cache.clear()
        t = torch.tensor([0, int(n)], dtype=torch.int32, device=device)
        _cu_cache[key] = t
    return t


_side_streams = {}


def _side_stream(device) -> "torch.cuda.Stream":
    """One persistent side stream per device: the caching allocator keeps a pool per stream, so a
    new stream per call would turn every gather buffer into a fresh cudaMalloc."""
    key = str(torch.device(device))
    if key not in _side_streams:
        _side_streams[key] = torch.cuda.Stream(device=device)
    return _side_streams[key]


def head_shard(num_kv_heads: int, world: int, rank: int) -> slice:
    """KV heads owned by `rank` (query heads are 16x that slice)."""
    if num_kv_heads % world != 0:
        raise ValueError(f"{num_kv_heads} KV heads do not divide over {world} ranks")
    per = num_kv_heads // world
    return slice(rank * per, (rank + 1) * per)


def batch_shard(batch: int, world: int, rank: int) -> range:
    """Sequences owned by `rank` (contiguous, sizes differ by at most one)."""
    base, rem = divmod(batch, world)
    start = rank * base + min(rank, rem)
    return range(start, start + base + (1 if rank < rem else 0))


@dataclass(frozen=True)
class Chunk:
    index: int      # position of the chunk in the sequence, 0 .. 2*world-1
    start: int      # first token
    end: int        # one past the last token


def zigzag_chunks(seqlen: int, world: int, rank: int, align: int = 64) -> List[Chunk]:
    """The two chunks of a `seqlen`-token sequence owned by `rank`: chunk r and chunk 2R-1-r of
    2R equal chunks (chunk length a multiple of `align`, so chunks start on KV-block borders)."""
    n = 2 * world
    if seqlen % (n * align) != 0:
        raise ValueError(f"seqlen {seqlen} must be a multiple of {n * align} for {world} ranks")
    clen = seqlen // n
    return [Chunk(i, i * clen, (i + 1) * clen) for i in (rank, n - 1 - rank)]


def gather_sequence(local: torch.Tensor, world: int, group=None) -> torch.Tensor:
    """All-gather per-rank zig-zag shards (2 chunks concatenated along dim 0, equal sizes on all
    ranks) and put the chunks back in sequence order."""
    if world == 1:
        return local
    parts = [torch.empty_like(local) for _ in range(world)]
    dist.all_gather(parts, local.contiguous(), group=group)
    half = local.shape[0] // 2
    chunks: List[Optional[torch.Tensor]] = [None] * (2 * world)
    for r, p in enumerate(parts):
        chunks[r] = p[:half]
        chunks[2 * world - 1 - r] = p[half:]
    return torch.cat(chunks, dim=0)


def scatter_sequence_grad(full: torch.Tensor, world: int, rank: int, group=None) -> torch.Tensor:
    """The reverse of `gather_sequence` for gradients: every rank holds a partial gradient of a
    whole-sequence tensor (rows in sequence order); the partials are summed and each rank gets the
    rows of its own two zig-zag chunks, in the order `gather_sequence` takes them.  A
    reduce-scatter over NCCL; backends without one (gloo) all-reduce and slice."""
    if world == 1:
        return full
    n = 2 * world
    clen = full.shape[0] // n
    chunks = full.reshape(n, clen, *full.shape[1:])
    order = [i for r in range(world) for i in (r, n - 1 - r)]       # rank-major zig-zag order
    send = chunks[order].contiguous()                                # (2*world, clen, ...)
    mine = torch.empty((2 * clen,) + tuple(full.shape[1:]), dtype=full.dtype, device=full.device)
    if dist.get_backend(group) == "nccl":
        dist.reduce_scatter_tensor(mine, send.view(-1, *full.shape[1:]), group=group)
    else:
        dist.all_reduce(send, group=group)
        mine.copy_(send[2 * rank:2 * rank + 2].reshape(mine.shape))
    return mine


def sharded_attention_fwd_bwd(q_local: torch.Tensor, k_local: torch.Tensor, v_local: torch.Tensor,
                              dout_local: torch.Tensor, topk_idx_local: torch.Tensor, seqlen: int,
                              world: int, rank: int, attn: Optional[Callable] = None, group=None):
    """Training step of the block-sparse attention of ONE sequence under query-chunk sharding
    (the selection that produced `topk_idx_local` carries no gradient, as in the reference's
    autograd function, infllm_v2/infllmv2_sparse_attention.py:266-385).

    Every rank passes the rows of its two zig-zag chunks: q_local / dout_local (2*clen, Hq, d),
    k_local / v_local (2*clen, Hk, d), topk_idx_local (Hk, 2*clen, k).  K and V are all-gathered,
    each chunk runs forward and backward as an ordinary seqlen_q < seqlen_k call (its dK / dV
    cover the keys before its end), and the partial dK / dV of all ranks are summed and handed
    back by rows (`scatter_sequence_grad`).  Returns (out_local, dq_local, dk_local, dv_local).
    `attn`: a differentiable stand-in for infllmv2_attn_varlen_func (tests)."""
    if attn is None:
        from . import attention
        attn = attention.infllmv2_attn_varlen_func
    chunks = zigzag_chunks(seqlen, world, rank)
    clen = chunks[0].end - chunks[0].start
    dev = q_local.device
    q = q_local.detach().requires_grad_(True)
    k = gather_sequence(k_local, world, group).detach().requires_grad_(True)
    v = gather_sequence(v_local, world, group).detach().requires_grad_(True)
    outs = []
    for i, ch in enumerate(chunks):
        cu_q, cu_k = _cu_pair(clen, dev), _cu_pair(ch.end, dev)
        idx = topk_idx_local[:, i * clen:(i + 1) * clen].contiguous()
        outs.append(attn(q[i * clen:(i + 1) * clen], k[:ch.end], v[:ch.end], cu_q, cu_k, clen, ch.end,
                         causal=True, topk_idx=idx))
    out = torch.cat(outs, dim=0)
    out.backward(dout_local.to(out.dtype))
    dk = scatter_sequence_grad(k.grad, world, rank, group)
    dv = scatter_sequence_grad(v.grad, world, rank, group)
    return out.detach(), q.grad, dk, dv


def compressed_range(chunk: Chunk, stride: int = 16) -> Tuple[int, int]:
    """Compressed-key slots [lo, hi) that a rank contributes for a chunk: key j (tokens
    [16j, 16j+32)) belongs to the chunk that holds its first token."""
    return chunk.start // stride, chunk.end // stride


@dataclass
class PrefillOps:
    """The operators of the prefill path; defaults are the CUDA ones.  `block_scores`, when set,
    replaces stage1 + max_pool by the fused kernel (same block scores, bit for bit)."""
    stage1: Callable
    max_pool: Callable
    topk: Callable
    attn: Callable
    block_scores: Optional[Callable] = None

    @staticmethod
    def cuda() -> "PrefillOps":
        from . import attention, ops
        return PrefillOps(attention.infllmv2_attn_stage1, ops.max_pooling_1d, ops.infllmv2_topk,
                          attention.infllmv2_attn_varlen_func,
                          attention.infllmv2_stage1_block_scores)


def chunk_selection(q_chunk: torch.Tensor, kc: torch.Tensor, chunk: Chunk, topk: int, init_blocks: int,
                    local_blocks: int, ops: Optional[PrefillOps] = None, block_size: int = 64,
                    kernel: int = 32, stride: int = 16) -> torch.Tensor:
    """Stage 1 + pool + top-k for the query tokens [chunk.start, chunk.end) of one sequence: needs
    the compressed keys of the prefix up to chunk.end only.  Returns topk_idx (Hk, lq, topk)."""
    ops = ops or PrefillOps.cuda()
    dev = q_chunk.device
    lq, lk = chunk.end - chunk.start, chunk.end
    n_comp = (lk - kernel) // stride + 1 if lk >= kernel else 0
    cu_q, cu_c = _cu_pair(lq, dev), _cu_pair(n_comp, dev)
    kc_p = kc[:n_comp]
    if ops.block_scores is not None and block_size == 64 and stride == 16:
        pooled = ops.block_scores(q_chunk, kc_p, cu_q, cu_c, lq, n_comp, local_blocks, init_blocks,
                                  cache_len=chunk.start, causal=True)
    else:
        score = ops.stage1(q_chunk, kc_p, kc_p, cu_q, cu_c, cu_c, lq, n_comp, causal=True)
        pooled = ops.max_pool(score, chunk.start, local_blocks, init_blocks, block_size, stride)
    return ops.topk(pooled, topk, chunk.start)


def chunk_attention(q_chunk: torch.Tensor, k: torch.Tensor, v: torch.Tensor, chunk: Chunk,
                    idx: torch.Tensor, ops: Optional[PrefillOps] = None) -> torch.Tensor:
    """Stage 2 for the same chunk against the keys / values of the prefix up to chunk.end."""
    ops = ops or PrefillOps.cuda()
    dev = q_chunk.device
    lq, lk = chunk.end - chunk.start, chunk.end
    cu_q, cu_k = _cu_pair(lq, dev), _cu_pair(lk, dev)
    return ops.attn(q_chunk, k[:lk], v[:lk], cu_q, cu_k, lq, lk, causal=True, topk_idx=idx)


def prefill_chunk(q_chunk: torch.Tensor, kc: torch.Tensor, k: torch.Tensor, v: torch.Tensor,
                  chunk: Chunk, topk: int, init_blocks: int, local_blocks: int,
                  ops: Optional[PrefillOps] = None, block_size: int = 64, kernel: int = 32,
                  stride: int = 16) -> Tuple[torch.Tensor, torch.Tensor]:
    """Full two-stage pipeline for the query tokens [chunk.start, chunk.end) of one sequence
    against the keys before chunk.end.  kc, k, v hold (at least) the sequence prefix up to
    chunk.end.  Returns (out_chunk, topk_idx_chunk)."""
    idx = chunk_selection(q_chunk, kc, chunk, topk, init_blocks, local_blocks, ops, block_size, kernel, stride)
    return chunk_attention(q_chunk, k, v, chunk, idx, ops), idx


def sharded_prefill(q_local: torch.Tensor, k_local: torch.Tensor, v_local: torch.Tensor,
                    kc_local: torch.Tensor, seqlen: int, world: int, rank: int, topk: int,
                    init_blocks: int, local_blocks: int, ops: Optional[PrefillOps] = None,
                    group=None, stride: int = 16, overlap: bool = True) -> torch.Tensor:
    """Query-chunk-parallel prefill of ONE sequence.  Every rank passes the rows of its two
    zig-zag chunks (concatenated): q_local (2*clen, Hq, d), k_local / v_local (2*clen, Hk, d) and
    kc_local (2*clen/stride, Hk, d) -- the compressed keys whose first token lies in the chunk;
    the slot of the sequence's last, incomplete window is padding.  Returns the attention output
    for the local rows, in the same order.

    The small compressed keys are gathered first and the selection of both chunks starts on them;
    on CUDA the all-gather of K and V runs on a side stream meanwhile and stage 2 waits for it."""
    chunks = zigzag_chunks(seqlen, world, rank)
    clen = chunks[0].end - chunks[0].start
    kc = gather_sequence(kc_local, world, group)
    side = ready = None
    if overlap and q_local.is_cuda and world > 1:
        cur = torch.cuda.current_stream(q_local.device)
        side = _side_stream(q_local.device)
        side.wait_stream(cur)
        with torch.cuda.stream(side):
            k = gather_sequence(k_local, world, group)
            v = gather_sequence(v_local, world, group)
            ready = torch.cuda.Event()
            ready.record(side)
    else:
        k = gather_sequence(k_local, world, group)
        v = gather_sequence(v_local, world, group)
    idxs = [chunk_selection(q_local[i * clen:(i + 1) * clen], kc, ch, topk, init_blocks, local_blocks, ops,
                            stride=stride) for i, ch in enumerate(chunks)]
    if ready is not None:
        cur.wait_event(ready)
        k.record_stream(cur)                      # allocated on the side stream, consumed on this one
        v.record_stream(cur)
    outs = [chunk_attention(q_local[i * clen:(i + 1) * clen], k, v, ch, idxs[i], ops)
            for i, ch in enumerate(chunks)]
    return torch.cat(outs, dim=0)


class StreamedPrefill:
    """Prefill of one sequence whose q / k / v / compressed k live in pinned HOST memory, result to
    pinned host memory: the query is processed in chunks (each an ordinary seqlen_q < seqlen_k call,
    as in `prefill_chunk`), and the host->device copy of chunk i+1, the kernels of chunk i and the
    device->host copy of chunk i-1 run on three streams, so a step costs about
    max(copy in, compute, copy out) instead of their sum.  Device buffers are allocated once."""

    def __init__(self, seqlen: int, heads_q: int, heads_k: int, head_dim: int, n_comp: int,
                 device, chunk_tokens: int = 16384, dtype=torch.bfloat16):
        if seqlen % chunk_tokens != 0 or chunk_tokens % 64 != 0:
            raise ValueError("seqlen must be a multiple of chunk_tokens, itself a multiple of 64")
        self.seqlen, self.chunk = seqlen, chunk_tokens
        self.device = torch.device(device)
        self.q = torch.empty(seqlen, heads_q, head_dim, dtype=dtype, device=device)
        self.k = torch.empty(seqlen, heads_k, head_dim, dtype=dtype, device=device)
        self.v = torch.empty_like(self.k)
        self.kc = torch.empty(n_comp, heads_k, head_dim, dtype=dtype, device=device)
        self.s_in, self.s_out = torch.cuda.Stream(device), torch.cuda.Stream(device)
        # the per-chunk cu_seqlens tables, created up front (see _cu_pair)
        for c in range(seqlen // chunk_tokens):
            lk = (c + 1) * chunk_tokens
            _cu_pair(chunk_tokens, self.device)
            _cu_pair(lk, self.device)
            _cu_pair((lk - 32) // 16 + 1 if lk >= 32 else 0, self.device)

    @staticmethod
    def middle_out(n: int) -> List[int]:
        """Chunk order n/2, n/2-1, n/2+1, ...: the cost of a chunk grows with its index (causal) while
        its copy does not, so starting with cheap chunks leaves the GPU waiting for copies and
        starting with the last one pays for the whole K/V up front; alternating around the middle
        keeps both the copy stream and the kernels busy."""
        order, lo, hi = [], n // 2 - 1, n // 2
        while lo >= 0 or hi < n:
            if hi < n:
                order.append(hi)
                hi += 1
            if lo >= 0:
                order.append(lo)
                lo -= 1
        return order

    def pieces(self, order: Sequence[int], split_ends: int) -> List[Tuple[int, int]]:
        """Token ranges in processing order.  The first and the last chunk of `order` are cut into
        `split_ends` equal pieces: the kernels can start after a quarter of a chunk has been copied
        in, and only a quarter of a chunk is left to copy out when the last kernel has finished."""
        out = []
        for pos, c in enumerate(order):
            start = c * self.chunk
            parts = split_ends if pos in (0, len(order) - 1) else 1
            if parts < 1 or self.chunk % (parts * 64) != 0:
                parts = 1
            step = self.chunk // parts
            out += [(start + j * step, start + (j + 1) * step) for j in range(parts)]
        return out

    def __call__(self, q_host, k_host, v_host, kc_host, out_host, topk: int, init_blocks: int,
                 local_blocks: int, ops: Optional[PrefillOps] = None, kernel: int = 32,
                 stride: int = 16, order: Optional[Sequence[int]] = None, split_ends: int = 4):
        """Enqueue one full prefill; returns when everything is ENQUEUED (synchronise the device, or
        the returned event, before reading out_host).  `order`: the sequence in which the query
        chunks are processed (default `middle_out`); chunks are independent given the keys before
        their end, which are copied on demand.  `split_ends`: see `pieces`."""
        main = torch.cuda.current_stream(self.device)
        n = self.seqlen // self.chunk
        order = list(order) if order is not None else self.middle_out(n)
        if sorted(order) != list(range(n)):
            raise ValueError("order must be a permutation of the chunk indices")
        pieces = self.pieces(order, split_ends)
        self.s_in.wait_stream(main)
        self.s_out.wait_stream(main)
        ev_in = {}
        with torch.cuda.stream(self.s_in):
            kv_done, kc_done = 0, 0                 # tokens / compressed keys already on the device
            for start, lk in pieces:
                # a piece needs the keys before its own end: K / V / compressed K travel piecewise
                # too, so the first kernels start after a fraction of the input has landed
                if lk > kv_done:
                    self.k[kv_done:lk].copy_(k_host[kv_done:lk], non_blocking=True)
                    self.v[kv_done:lk].copy_(v_host[kv_done:lk], non_blocking=True)
                    kv_done = lk
                n_c = min(self.kc.shape[0], (lk - kernel) // stride + 1 if lk >= kernel else 0)
                if n_c > kc_done:
                    self.kc[kc_done:n_c].copy_(kc_host[kc_done:n_c], non_blocking=True)
                    kc_done = n_c
                sl = slice(start, lk)
                self.q[sl].copy_(q_host[sl], non_blocking=True)
                ev = torch.cuda.Event()
                ev.record(self.s_in)
                ev_in[start] = ev
        keep = []
        for start, end in pieces:
            ch = Chunk(start // self.chunk, start, end)
            main.wait_event(ev_in[start])
            out, _ = prefill_chunk(self.q[ch.start:ch.end], self.kc, self.k, self.v, ch, topk,
                                   init_blocks, local_blocks, ops)
            ev = torch.cuda.Event()
            ev.record(main)
            self.s_out.wait_event(ev)
            with torch.cuda.stream(self.s_out):
                out_host[ch.start:ch.end].copy_(out, non_blocking=True)
            out.record_stream(self.s_out)
            keep.append(out)
        done = torch.cuda.Event()
        done.record(self.s_out)
        main.wait_event(done)
        return done
