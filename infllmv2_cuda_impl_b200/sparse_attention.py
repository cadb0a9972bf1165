"""Caller-side glue for the hot path: what a model's attention layer does around the operators.

The reference ships operators only; the layer that strings them together lives in the model code
that imports `infllm_v2` (the calls it makes are the ones the reference's tests replay:
tests/test_stage1_compressed_lse.py:57-99 for the compression, tests/test_infllmv2.py for stage 2,
tests/test_kvcache_simple.py for decode).  This module is that layer, for callers that do not
bring their own:

    prefill / training   compress keys -> stage-1 block scores -> top-k -> block-sparse attention
                         (selection runs without gradients; attention is differentiable), and
                         optionally fills a DecodeCache
    decode               one launch appends the new key / value and updates the compressed keys,
                         then stage-1 scores over the cache in place (`seqused_k`), max-pool,
                         top-k and sparse attention over the selected blocks

Short sequences (<= dense_len tokens) attend densely, as the selection cannot drop anything
useful there.  Everything stays on the caller's stream; the only host <-> device traffic is the
optional read of the total number of compressed keys when the caller does not pass the lengths.
"""
from dataclasses import dataclass
from typing import Optional, Sequence

import torch

from . import ops
from .attention import (infllmv2_attn_stage1, infllmv2_stage1_decode_select, infllmv2_attn_varlen_func, infllmv2_attn_with_kvcache,
                        infllmv2_stage1_block_scores, GROUP, HEAD_DIM)

__all__ = ["SparseConfig", "DecodeCache", "SparseAttention"]


@dataclass
class SparseConfig:
    topk: int = 64                 # blocks kept per (token, KV head), forced ones included
    init_blocks: int = 1           # leading blocks always kept
    local_blocks: int = 32         # blocks bq-local_blocks .. bq always kept (a 2048-token window)
    block_size: int = 64
    kernel_size: int = 32          # key compression of the scorer
    kernel_stride: int = 16
    coarse_lse: bool = False       # row sums over a second compression (the "compressed LSE" mode)
    coarse_kernel_size: int = 128
    coarse_kernel_stride: int = 64
    dense_len: int = 8192          # at most this many tokens -> dense attention

    def windows(self, length: int, coarse: bool = False) -> int:
        k, s = ((self.coarse_kernel_size, self.coarse_kernel_stride) if coarse
                else (self.kernel_size, self.kernel_stride))
        return (length - k) // s + 1 if length >= k else 0


class DecodeCache:
    """Per-sequence caches of keys, values and compressed keys at a fixed capacity, plus the
    small integer tensors a decode step needs (all device-resident; `max_len` is the only host
    copy of the lengths and is an upper bound)."""

    def __init__(self, batch: int, capacity: int, heads_k: int, config: SparseConfig, device="cuda"):
        dev = torch.device(device)
        self.config, self.batch, self.capacity, self.heads_k = config, batch, capacity, heads_k
        shape = (batch, capacity, heads_k, HEAD_DIM)
        self.k = torch.zeros(shape, dtype=torch.bfloat16, device=dev)
        self.v = torch.zeros(shape, dtype=torch.bfloat16, device=dev)
        self.c_capacity = max(config.windows(capacity), 1)
        self.kc = torch.zeros(batch, self.c_capacity, heads_k, HEAD_DIM, dtype=torch.bfloat16, device=dev)
        self.kc2 = self.n_comp2 = self.cu_c2 = None
        self.c2_capacity = 0
        if config.coarse_lse:
            self.c2_capacity = max(config.windows(capacity, coarse=True), 1)
            self.kc2 = torch.zeros(batch, self.c2_capacity, heads_k, HEAD_DIM, dtype=torch.bfloat16, device=dev)
            self.n_comp2 = torch.zeros(batch, dtype=torch.int32, device=dev)
            self.cu_c2 = torch.arange(batch + 1, dtype=torch.int32, device=dev) * self.c2_capacity
        self.seqlens = torch.zeros(batch, dtype=torch.int32, device=dev)
        self.positions = torch.zeros(batch, dtype=torch.int32, device=dev)   # lengths before the last append
        self.n_comp = torch.zeros(batch, dtype=torch.int32, device=dev)
        self.cu_q = torch.arange(batch + 1, dtype=torch.int32, device=dev)
        self.cu_c = self.cu_q * self.c_capacity
        self.max_len = 0

    def fill(self, k, v, kc, cu_seqlens, cu_seqlens_c, max_seqlen, kc2=None, cu_seqlens_c2=None):
        """Load the caches from packed prefill tensors (rows past the capacity are dropped)."""
        ops.cache_fill(k, self.k, cu_seqlens, self.seqlens)
        ops.cache_fill(v, self.v, cu_seqlens)
        ops.cache_fill(kc, self.kc, cu_seqlens_c, self.n_comp)
        if self.kc2 is not None:
            ops.cache_fill(kc2, self.kc2, cu_seqlens_c2, self.n_comp2)
        self.max_len = min(int(max_seqlen), self.capacity)


class SparseAttention:
    """Prefill / training and decode on top of the operators, for 16 query heads per KV head
    and head dimension 128 (the reference build's only configuration)."""

    def __init__(self, config: Optional[SparseConfig] = None):
        self.config = config or SparseConfig()
        if self.config.block_size != 64 or self.config.kernel_stride != 16:
            raise NotImplementedError("block_size 64 over compression stride 16 only, as in the reference")

    # ------------------------------------------------------------------ selection (no gradients)
    @torch.no_grad()
    def compress(self, k, cu_seqlens, seqlens: Optional[Sequence[int]] = None, coarse: bool = False):
        """Compressed keys of packed sequences; `seqlens` (host ints) avoids a device read."""
        c = self.config
        ks, st = ((c.coarse_kernel_size, c.coarse_kernel_stride) if coarse else (c.kernel_size, c.kernel_stride))
        total_c = sum(c.windows(int(l), coarse) for l in seqlens) if seqlens is not None else None
        return ops.compress_keys(k, cu_seqlens, ks, st, total_c=total_c)

    @torch.no_grad()
    def select(self, q, kc, cu_seqlens_q, cu_seqlens_c, max_seqlen_q, max_c, kc2=None,
               cu_seqlens_c2=None, cache_len: int = 0):
        """Block selection of packed sequences: int32 (Hk, total_q, topk), ascending, -1 padded."""
        c = self.config
        pooled = infllmv2_stage1_block_scores(q, kc, cu_seqlens_q, cu_seqlens_c, max_seqlen_q, max_c,
                                              c.local_blocks, c.init_blocks, cache_len=cache_len,
                                              lse_keys=kc2, cu_seqlens_v=cu_seqlens_c2)
        return ops.infllmv2_topk(pooled, c.topk, cache_len=cache_len, cu_seqlens_q=cu_seqlens_q)

    # ------------------------------------------------------------------ prefill / training
    def prefill(self, q, k, v, cu_seqlens, max_seqlen: int, seqlens: Optional[Sequence[int]] = None,
                cache: Optional[DecodeCache] = None, softmax_scale: Optional[float] = None):
        """Causal self-attention over packed sequences: q (total, Hq, 128), k / v (total, Hk, 128)
        bf16, cu_seqlens (B+1) int32.  Differentiable in q, k, v through the attention itself; the
        selection sees detached tensors.  With `cache`, the keys, values and compressed keys are
        also stored for decoding."""
        c = self.config
        max_c = c.windows(max_seqlen)
        need_comp = cache is not None or (max_seqlen > c.dense_len and max_c > 0)
        kc = cu_c = kc2 = cu_c2 = None
        if need_comp:
            kc, cu_c = self.compress(k.detach(), cu_seqlens, seqlens)
            if c.coarse_lse:
                kc2, cu_c2 = self.compress(k.detach(), cu_seqlens, seqlens, coarse=True)
        idx = None
        if max_seqlen > c.dense_len and max_c > 0:
            idx = self.select(q.detach(), kc, cu_seqlens, cu_c, max_seqlen, max_c, kc2, cu_c2)
        out = infllmv2_attn_varlen_func(q, k, v, cu_seqlens, cu_seqlens, max_seqlen, max_seqlen,
                                        softmax_scale=softmax_scale, causal=True, topk_idx=idx)
        if cache is not None:
            cache.fill(k.detach(), v.detach(), kc, cu_seqlens, cu_c, max_seqlen, kc2, cu_c2)
        return out

    # ------------------------------------------------------------------ decode
    @torch.no_grad()
    def decode(self, q, k_new, v_new, cache: DecodeCache, softmax_scale: Optional[float] = None,
               static_shapes: bool = False):
        """One token per sequence: q (B, Hq, 128) or (B, 1, Hq, 128); k_new / v_new (B, Hk, 128)
        or (B, 1, Hk, 128).  Appends to the cache, then attends over it (the new token included).
        Returns (B, 1, Hq, 128).  static_shapes: size every intermediate for the cache capacity
        instead of the current maximum length, so that the step launches the same kernels with the
        same arguments every time (what a CUDA graph needs; see `capture_decode`)."""
        c = self.config
        b, hk = cache.batch, cache.heads_k
        if cache.max_len >= cache.capacity:
            raise RuntimeError("DecodeCache is full")
        q3 = q.reshape(b, hk * GROUP, HEAD_DIM)
        ops.decode_append(k_new.reshape(b, hk, HEAD_DIM), v_new.reshape(b, hk, HEAD_DIM), cache.k, cache.v,
                          cache.seqlens, cache.positions, cache.kc, cache.n_comp, c.kernel_size,
                          c.kernel_stride, cache.kc2, cache.n_comp2, c.coarse_kernel_size,
                          c.coarse_kernel_stride)
        cache.max_len += 1
        bound = cache.capacity if static_shapes else cache.max_len       # >= every sequence length
        max_c = c.windows(bound)
        mask = None
        # Dense or sparse is decided per sequence on the device (a sequence of at most dense_len
        # tokens gets every block), so a captured step, which is sized for the capacity, and an
        # eager one agree; the eager step merely skips the selection when no sequence can need it.
        if bound > c.dense_len and max_c > 0:
            kc_flat = cache.kc.view(-1, hk, HEAD_DIM)
            if cache.kc2 is not None:
                score = infllmv2_attn_stage1(q3, kc_flat, cache.kc2.view(-1, hk, HEAD_DIM), cache.cu_q, cache.cu_c,
                                             cache.cu_c2, 1, max_c, causal=False, seqused_k=cache.n_comp,
                                             seqused_v=cache.n_comp2)
                # pool + top-k + packed mask of the few decode rows in one launch
                mask = ops.decode_select(score, cache.positions, c.topk, cache.capacity, c.local_blocks,
                                         c.init_blocks, seqused_c=cache.n_comp, dense_len=c.dense_len)
            else:
                # scores, pool, top-k and mask in two launches; the score rows stay on chip
                mask = infllmv2_stage1_decode_select(q3, kc_flat, cache.cu_c, cache.positions, max_c,
                                                     cache.capacity, c.topk, c.local_blocks, c.init_blocks,
                                                     seqused_k=cache.n_comp, dense_len=c.dense_len)
        return infllmv2_attn_with_kvcache(q3.view(b, 1, hk * GROUP, HEAD_DIM), cache.k, cache.v,
                                          cache_seqlens=cache.seqlens, softmax_scale=softmax_scale,
                                          block_mask=mask)

    def capture_decode(self, cache: DecodeCache, softmax_scale: Optional[float] = None):
        """Capture one decode step for `cache` in a CUDA graph.  Returns `step(q, k_new, v_new)`,
        which copies its arguments into the graph's input buffers, replays it and returns the
        graph's output tensor (B, 1, Hq, 128), valid until the next call.  The step is sized for
        the cache capacity (`static_shapes`); the lengths live on the device and advance with
        every replay."""
        b, hk = cache.batch, cache.heads_k
        dev = cache.k.device
        q_in = torch.zeros(b, hk * GROUP, HEAD_DIM, dtype=torch.bfloat16, device=dev)
        k_in = torch.zeros(b, hk, HEAD_DIM, dtype=torch.bfloat16, device=dev)
        v_in = torch.zeros(b, hk, HEAD_DIM, dtype=torch.bfloat16, device=dev)
        # one eager step on a side stream (first-use initialisation must not happen under capture),
        # then the lengths are put back: what the step wrote lies past them
        saved = (cache.seqlens.clone(), cache.n_comp.clone(),
                 cache.n_comp2.clone() if cache.n_comp2 is not None else None, cache.max_len)
        side = torch.cuda.Stream(device=dev)
        side.wait_stream(torch.cuda.current_stream(dev))
        with torch.cuda.stream(side):
            self.decode(q_in, k_in, v_in, cache, softmax_scale, static_shapes=True)
        torch.cuda.current_stream(dev).wait_stream(side)

        def restore():
            cache.seqlens.copy_(saved[0])
            cache.n_comp.copy_(saved[1])
            if saved[2] is not None:
                cache.n_comp2.copy_(saved[2])
            cache.max_len = saved[3]

        restore()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            out = self.decode(q_in, k_in, v_in, cache, softmax_scale, static_shapes=True)
        cache.max_len = saved[3]                   # capturing does not run the step

        def step(q, k_new, v_new):
            if cache.max_len >= cache.capacity:
                raise RuntimeError("DecodeCache is full")
            q_in.copy_(q.reshape(q_in.shape))
            k_in.copy_(k_new.reshape(k_in.shape))
            v_in.copy_(v_new.reshape(v_in.shape))
            graph.replay()
            cache.max_len += 1
            return out

        step.graph, step.inputs = graph, (q_in, k_in, v_in)
        return step
