"""Stage-1 scorer, stage-2 block-sparse attention (forward + backward) and KV-cache decode with the
reference's Python signatures (infllm_v2/infllmv2_sparse_attention.py:388-406, 483-501, 609-630).

The bodies differ from the reference on purpose: the kernels read q / write out in the caller's
(token, head, d) layout, so none of the GQA reshape-transpose-contiguous copies remain, the
backward mask comes from one bit-transpose kernel, and nothing synchronises the device.
Features the reference's build compiles out (dropout, softcap, ALiBi, sliding window, fp16,
head_dim != 128, GQA group != 16) raise on the host, as its TORCH_CHECKs do.
"""
import math
import os
from typing import Optional, Tuple, Union

import torch

from . import _lib
from .ops import topk_to_uint64, transpose_blockmask

BLOCK_N = 64      # tokens per KV block (the reference's N_BLOCK_DIM)
GROUP = 16        # query heads per KV head (the reference's m_block_dim)
HEAD_DIM = 128

_status = {}
_CHECK_STATUS = os.environ.get("IFV2_CHECK_STATUS", "0") == "1"


def _status_words(device) -> torch.Tensor:
    """Per-device int32[4] that kernels write when one of their bounded waits runs out."""
    dev = torch.device(device)
    idx = dev.index if dev.index is not None else torch.cuda.current_device()
    if idx not in _status:
        _status[idx] = torch.zeros(4, dtype=torch.int32, device=torch.device("cuda", idx))
    return _status[idx]


def check_device_status(device=None) -> None:
    """Wait for the current stream and raise if any kernel launched through this module since the
    last check gave up on one of its bounded waits (the outputs of that launch are undefined; later
    launches ran normally).  Not called on the hot path because it synchronises: tests, the smoke
    entry and the benchmark call it, and so does the backward of infllmv2_attn_varlen_func when the
    environment variable IFV2_CHECK_STATUS=1 is set."""
    devices = list(_status) if device is None else [torch.device(device).index or 0]
    for idx in devices:
        if idx in _status:
            with torch.cuda.device(idx):
                torch.cuda.synchronize(idx)
                _lib.call("ifv2_check_status", _status[idx].data_ptr(),
                          torch.cuda.current_stream(idx).cuda_stream)


def _stream(device) -> int:
    return torch.cuda.current_stream(device).cuda_stream


def maybe_contiguous(x):
    return x.contiguous() if x is not None and x.stride(-1) != 1 else x


def round_multiple(x, m):
    return (x + m - 1) // m * m


def _check_common(q, k, dropout_p, window_size, softcap, alibi_slopes, block_table, what):
    if not q.is_cuda:
        raise RuntimeError(f"{what}: tensors must be on a CUDA device; this library has no CPU path")
    if q.dtype != torch.bfloat16 or k.dtype != torch.bfloat16:
        raise RuntimeError(f"{what}: only bf16 is supported (as in the reference build)")
    if dropout_p != 0.0:
        raise RuntimeError(f"{what}: dropout is not supported (compiled out in the reference)")
    if softcap != 0.0:
        raise RuntimeError(f"{what}: softcap is not supported (compiled out in the reference)")
    if alibi_slopes is not None:
        raise RuntimeError(f"{what}: ALiBi is not supported (compiled out in the reference)")
    if tuple(window_size) != (-1, -1):
        raise RuntimeError(f"{what}: sliding-window attention is not supported (compiled out in the reference)")
    if block_table is not None:
        if block_table.dtype != torch.int32 or block_table.dim() != 2 or k.dim() != 4:
            raise ValueError(f"{what}: with block_table (batch, max_pages) int32 the keys are "
                             "(num_pages, page_size, nheads_k, 128)")
    if q.shape[-1] != HEAD_DIM or k.shape[-1] != HEAD_DIM:
        raise RuntimeError(f"{what}: head_dim must be {HEAD_DIM}")
    if q.shape[-2] != GROUP * k.shape[-2]:
        raise RuntimeError(f"{what}: the number of query heads must be {GROUP} x the number of KV heads")


def _dense(x):
    """(T, H, d) with unit stride in d and H, i.e. rows of H*d contiguous elements."""
    return x if x.is_contiguous() else x.contiguous()


# ------------------------------------------------------------------------------------ stage 1 --

def infllmv2_attn_stage1(
    q, k, v, cu_seqlens_q, cu_seqlens_k, cu_seqlens_v, max_seqlen_q, max_seqlen_k,
    dropout_p=0.0, softmax_scale=None, causal=False, window_size=(-1, -1), softcap=0.0,
    alibi_slopes=None, deterministic=False, return_attn_probs=True, block_table=None,
    seqused_k=None, seqused_v=None, leftpad_k=None,
):
    """Stage-1 scores: for every KV head, softmax(q . k_compressed) summed over its 16 query heads.

    q: (total_q, nheads, 128) bf16; k: (total_c, nheads_k, 128) bf16 compressed keys;
    v / cu_seqlens_v: the keys the log-sum-exp is taken over.  Normally the same tensor as k.
    A differently compressed v (kernel 128 / stride 64, the reference's "compressed LSE" mode,
    flash_fwd_kernel.h:1236-1240, oracle tests/stage1/complse_online_softmax.py) makes the row
    maxima and sums come from v and the returned scores exp(q.k - lse_v), summed over the heads.
    Returns (nheads_k, total_q, max_seqlen_k) bf16; entries a token cannot see are 0.
    The returned tensor is a column slice of a buffer whose rows are padded to a multiple of
    128 elements, like the reference's (infllm_v2/infllmv2_sparse_attention.py:587).
    seqused_k: optional (batch,) int32 -- only that many keys of each sequence are used
    (flash_api.cpp:792, 906-911); cu_seqlens_k then only says where a sequence's keys start, so a
    per-sequence cache (batch, capacity, nheads_k, 128) can be scored in place as
    k = cache.view(-1, nheads_k, 128), cu_seqlens_k = arange(batch + 1) * capacity.
    seqused_v: the same for v / cu_seqlens_v.
    block_table: (batch, max_pages) int32 -- k is then a paged cache of compressed keys
    (num_pages, page_size, nheads_k, 128), page_size a multiple of 128 (the reference wants 256,
    flash_api.cpp:906-911), and cu_seqlens_k / seqused_k give each sequence's key count; v must be
    k.  leftpad_k: (batch,) int32 -- the keys of a sequence start that many rows into its
    cu_seqlens_k extent (flash_api.cpp:1001-1008).
    """
    _check_common(q, k, dropout_p, window_size, softcap, alibi_slopes, block_table,
                  "infllmv2_attn_stage1")
    if block_table is not None or leftpad_k is not None:
        return _stage1_paged(q, k, v, cu_seqlens_q, cu_seqlens_k, max_seqlen_q, max_seqlen_k, softmax_scale,
                             causal, block_table, seqused_k, leftpad_k)
    lse_keys = None
    if v is not None and v is not k and (v.shape != k.shape or v.data_ptr() != k.data_ptr()):
        if v.dtype != k.dtype or v.dim() != 3 or v.shape[1:] != k.shape[1:]:
            raise ValueError("infllmv2_attn_stage1: v must be (total_v, nheads_k, 128) in k's dtype")
        assert cu_seqlens_v is not None and cu_seqlens_v.dtype == torch.int32
        lse_keys = _dense(maybe_contiguous(v))
    if softmax_scale is None:
        softmax_scale = q.shape[-1] ** (-0.5)
    q, k = _dense(maybe_contiguous(q)), _dense(maybe_contiguous(k))
    total_q, nheads, _ = q.shape
    nheads_k = k.shape[1]
    batch = cu_seqlens_q.numel() - 1
    assert cu_seqlens_q.dtype == torch.int32 and cu_seqlens_k.dtype == torch.int32
    used_ptr = None
    if seqused_k is not None:
        assert seqused_k.dtype == torch.int32 and seqused_k.numel() == batch
        seqused_k = seqused_k.contiguous()
        used_ptr = seqused_k.data_ptr()
    used_v_ptr = None
    if seqused_v is not None and lse_keys is not None:
        assert seqused_v.dtype == torch.int32 and seqused_v.numel() == batch
        seqused_v = seqused_v.contiguous()
        used_v_ptr = seqused_v.data_ptr()
    row_stride = max(round_multiple(max_seqlen_k, 128), 128)
    buf = torch.empty(nheads_k, total_q, row_stride, dtype=torch.bfloat16, device=q.device)
    if max_seqlen_q == 1 and total_q == batch and lse_keys is None and max_seqlen_k > 0:
        # decode: one token per sequence -> the bandwidth-oriented kernel pair (same values)
        lib = _lib.load()
        ws_bytes = int(lib.ifv2_stage1_decode_workspace_bytes(batch, nheads_k, max_seqlen_k))
        ws = torch.empty(ws_bytes, dtype=torch.uint8, device=q.device)
        with torch.cuda.device(q.device):
            _lib.call("ifv2_stage1_decode_scores", q.data_ptr(), k.data_ptr(), buf.data_ptr(),
                      cu_seqlens_k.contiguous().data_ptr(), used_ptr, batch, k.shape[0], nheads,
                      nheads_k, q.shape[-1], max_seqlen_k, row_stride, float(softmax_scale), int(bool(causal)),
                      ws.data_ptr(), ws_bytes, _stream(q.device))
        return buf[:, :, :max_seqlen_k]
    with torch.cuda.device(q.device):
        _lib.call("ifv2_stage1_scores", q.data_ptr(), k.data_ptr(),
                  lse_keys.data_ptr() if lse_keys is not None else None, buf.data_ptr(),
                  cu_seqlens_q.contiguous().data_ptr(), cu_seqlens_k.contiguous().data_ptr(),
                  cu_seqlens_v.contiguous().data_ptr() if lse_keys is not None else None,
                  lse_keys.shape[0] if lse_keys is not None else 0, used_ptr, used_v_ptr, batch,
                  total_q, k.shape[0], nheads, nheads_k, q.shape[-1], max_seqlen_q, max_seqlen_k,
                  row_stride, float(softmax_scale), int(bool(causal)),
                  _status_words(q.device).data_ptr(), _stream(q.device))
    return buf[:, :, :max_seqlen_k]


def _stage1_paged(q, k, v, cu_seqlens_q, cu_seqlens_k, max_seqlen_q, max_seqlen_k, softmax_scale, causal,
                  block_table, seqused_k, leftpad_k, pool_args=None):
    """Stage 1 over a paged or left-padded compressed-key cache (ifv2_stage1_paged).  pool_args:
    (n_blocks, cache_len, cache_lens, local_blocks, init_blocks) for fused block scores."""
    if v is not None and v is not k and v.data_ptr() != k.data_ptr():
        raise NotImplementedError("infllmv2_attn_stage1: separate row-sum keys are not supported with "
                                  "block_table / leftpad_k")
    if softmax_scale is None:
        softmax_scale = q.shape[-1] ** (-0.5)
    q = _dense(maybe_contiguous(q))
    total_q, nheads, d = q.shape
    batch = cu_seqlens_q.numel() - 1
    bt_ptr, bt_stride, page = None, 0, 0
    if block_table is not None:
        if leftpad_k is not None:
            raise NotImplementedError("infllmv2_attn_stage1: a paged cache takes no leftpad_k")
        page = k.shape[1]
        if page % 128 != 0:
            raise NotImplementedError("infllmv2_attn_stage1: page size must be a multiple of 128 compressed keys")
        assert block_table.shape[0] == batch
        block_table = block_table.contiguous()
        bt_ptr, bt_stride = block_table.data_ptr(), block_table.shape[1]
        k = k.contiguous().view(-1, k.shape[2], k.shape[3])
    else:
        k = _dense(maybe_contiguous(k))
    nheads_k = k.shape[1]
    for name, t in (("seqused_k", seqused_k), ("leftpad_k", leftpad_k)):
        if t is not None:
            assert t.dtype == torch.int32 and t.numel() == batch, f"{name} must be (batch,) int32"
    row_stride = max(round_multiple(max_seqlen_k, 128), 128)
    buf = pooled = None
    n_blocks = cache_len = local_blocks = init_blocks = 0
    cache_lens = None
    if pool_args is None:
        buf = torch.empty(nheads_k, total_q, row_stride, dtype=torch.bfloat16, device=q.device)
    else:
        n_blocks, cache_len, cache_lens, local_blocks, init_blocks = pool_args
        pooled = torch.empty(nheads_k, total_q, n_blocks, dtype=torch.bfloat16, device=q.device)
    with torch.cuda.device(q.device):
        _lib.call("ifv2_stage1_paged", q.data_ptr(), k.data_ptr(), buf.data_ptr() if buf is not None else None,
                  pooled.data_ptr() if pooled is not None else None, cu_seqlens_q.contiguous().data_ptr(),
                  cu_seqlens_k.contiguous().data_ptr(),
                  seqused_k.contiguous().data_ptr() if seqused_k is not None else None,
                  leftpad_k.contiguous().data_ptr() if leftpad_k is not None else None, bt_ptr, bt_stride, page,
                  cache_lens.data_ptr() if cache_lens is not None else None, batch, total_q, k.shape[0],
                  nheads, nheads_k, d, max_seqlen_q, max_seqlen_k, row_stride if buf is not None else 0,
                  n_blocks, int(cache_len), int(local_blocks), int(init_blocks), float(softmax_scale),
                  int(bool(causal)), _status_words(q.device).data_ptr(), _stream(q.device))
    return buf[:, :, :max_seqlen_k] if buf is not None else pooled


def infllmv2_stage1_decode_select(q, k, cu_seqlens_k, positions, max_seqlen_k, cache_capacity, topk,
                                  local_blocks, init_blocks, seqused_k=None, softmax_scale=None,
                                  causal=False, block_size=64, stride=16, return_topk=False, dense_len=0):
    """Block selection of a decode step straight from the compressed keys (an addition to the
    reference API): stage-1 scores of ONE query token per sequence (q: (B, Hq, 128)), 64-token
    max-pool, top-k and the packed block mask, in two launches and without the score rows ever
    reaching HBM.  k / cu_seqlens_k / seqused_k / max_seqlen_k: the compressed keys as in
    infllmv2_attn_stage1; positions (B,) int32: position of each query token in its sequence;
    cache_capacity: key capacity of the KV cache the mask is for.  Returns the int64 mask
    (B, Hk, 1, words) that infllmv2_attn_with_kvcache takes as `block_mask` [, topk_idx
    (B, Hk, 1, topk) int32]; both equal infllmv2_attn_stage1 -> ops.decode_select.  dense_len: as in
    ops.decode_select."""
    _check_common(q, k, 0.0, (-1, -1), 0.0, None, None, "infllmv2_stage1_decode_select")
    q, k = _dense(maybe_contiguous(q)), _dense(maybe_contiguous(k))
    if q.dim() != 3:
        raise ValueError("infllmv2_stage1_decode_select: q must be (batch, nheads, 128), one token per sequence")
    batch, nheads, d = q.shape
    nheads_k = k.shape[1]
    assert cu_seqlens_k.dtype == torch.int32 and cu_seqlens_k.numel() == batch + 1
    assert positions.dtype == torch.int32 and positions.numel() == batch
    if seqused_k is not None:
        assert seqused_k.dtype == torch.int32 and seqused_k.numel() == batch
        seqused_k = seqused_k.contiguous()
    if softmax_scale is None:
        softmax_scale = d ** (-0.5)
    n_blocks = (cache_capacity + block_size - 1) // block_size
    words = (n_blocks + 63) // 64
    mask = torch.empty(batch, nheads_k, 1, words, dtype=torch.int64, device=q.device)
    idx = torch.empty(batch, nheads_k, 1, topk, dtype=torch.int32, device=q.device) if return_topk else None
    lib = _lib.load()
    ws_bytes = int(lib.ifv2_stage1_decode_workspace_bytes(batch, nheads_k, max_seqlen_k))
    ws = torch.empty(max(ws_bytes, 16), dtype=torch.uint8, device=q.device)
    with torch.cuda.device(q.device):
        _lib.call("ifv2_stage1_decode_select", q.data_ptr(), k.data_ptr(), cu_seqlens_k.contiguous().data_ptr(),
                  seqused_k.data_ptr() if seqused_k is not None else None, positions.contiguous().data_ptr(),
                  mask.data_ptr(), idx.data_ptr() if idx is not None else None, batch, k.shape[0], nheads,
                  nheads_k, d, max_seqlen_k, n_blocks, words, topk, local_blocks, init_blocks, block_size,
                  stride, int(dense_len), float(softmax_scale), int(bool(causal)), ws.data_ptr(), ws_bytes,
                  _stream(q.device))
    return (mask, idx) if return_topk else mask


def infllmv2_stage1_block_scores(q, k, cu_seqlens_q, cu_seqlens_k, max_seqlen_q, max_seqlen_k,
                                 local_blocks, init_blocks, cache_len=0, cache_lens=None,
                                 max_cache_len=None, softmax_scale=None, causal=True,
                                 block_size=64, stride=16, return_scores=False,
                                 lse_keys=None, cu_seqlens_v=None, seqused_k=None, seqused_v=None,
                                 block_table=None, leftpad_k=None):
    """Stage 1 and the 64-token max-pool in one kernel (an addition to the reference API).

    Returns block scores (nheads_k, total_q, ceil((max_seqlen_q + cache) / 64)) bf16 equal, bit
    for bit, to `max_pooling_1d[_varlen](infllmv2_attn_stage1(...), ...)`; the
    (nheads_k, total_q, max_seqlen_k) score tensor is only materialised with return_scores=True
    (then the result is (block_scores, scores)).  cache_lens: optional per-sequence int32 tensor
    (pass max_cache_len to avoid a device->host read); otherwise the scalar cache_len applies.
    lse_keys / cu_seqlens_v: optional coarser compressed keys for the log-sum-exp (the `v` of
    infllmv2_attn_stage1).  seqused_k / seqused_v / block_table / leftpad_k: as in
    infllmv2_attn_stage1 (a paged or left-padded cache returns the block scores only).
    """
    _check_common(q, k, 0.0, (-1, -1), 0.0, None, block_table, "infllmv2_stage1_block_scores")
    if block_table is not None or leftpad_k is not None:
        if lse_keys is not None or return_scores:
            raise NotImplementedError("infllmv2_stage1_block_scores: a paged / left-padded cache takes neither "
                                      "lse_keys nor return_scores")
        if block_size != BLOCK_N or stride != 16:
            raise NotImplementedError("infllmv2_stage1_block_scores: only block_size 64 / stride 16")
        batch = cu_seqlens_q.numel() - 1
        if cache_lens is not None:
            assert cache_lens.dtype == torch.int32 and cache_lens.numel() == batch
            if max_cache_len is None:
                max_cache_len = int(cache_lens.max().item())
            cache_lens = cache_lens.contiguous()
        else:
            max_cache_len = cache_len
        n_blocks = (max_seqlen_q + max_cache_len + BLOCK_N - 1) // BLOCK_N
        return _stage1_paged(q, k, None, cu_seqlens_q, cu_seqlens_k, max_seqlen_q, max_seqlen_k, softmax_scale,
                             causal, block_table, seqused_k, leftpad_k,
                             pool_args=(n_blocks, cache_len, cache_lens, local_blocks, init_blocks))
    if lse_keys is not None:
        assert cu_seqlens_v is not None and cu_seqlens_v.dtype == torch.int32
        lse_keys = _dense(maybe_contiguous(lse_keys))
    if block_size != BLOCK_N or stride != 16:
        raise NotImplementedError("infllmv2_stage1_block_scores: only block_size 64 / stride 16")
    if softmax_scale is None:
        softmax_scale = q.shape[-1] ** (-0.5)
    q, k = _dense(maybe_contiguous(q)), _dense(maybe_contiguous(k))
    total_q, nheads, _ = q.shape
    nheads_k = k.shape[1]
    batch = cu_seqlens_q.numel() - 1
    if cache_lens is not None:
        assert cache_lens.dtype == torch.int32 and cache_lens.numel() == batch
        if max_cache_len is None:
            max_cache_len = int(cache_lens.max().item())
        cache_lens = cache_lens.contiguous()
    else:
        max_cache_len = cache_len
    n_blocks = (max_seqlen_q + max_cache_len + BLOCK_N - 1) // BLOCK_N
    pooled = torch.empty(nheads_k, total_q, n_blocks, dtype=torch.bfloat16, device=q.device)
    buf, row_stride = None, 0
    if return_scores:
        row_stride = max(round_multiple(max_seqlen_k, 128), 128)
        buf = torch.empty(nheads_k, total_q, row_stride, dtype=torch.bfloat16, device=q.device)
    with torch.cuda.device(q.device):
        _lib.call("ifv2_stage1_block_scores", q.data_ptr(), k.data_ptr(),
                  lse_keys.data_ptr() if lse_keys is not None else None,
                  buf.data_ptr() if buf is not None else None, pooled.data_ptr(),
                  cu_seqlens_q.contiguous().data_ptr(), cu_seqlens_k.contiguous().data_ptr(),
                  cu_seqlens_v.contiguous().data_ptr() if lse_keys is not None else None,
                  lse_keys.shape[0] if lse_keys is not None else 0,
                  seqused_k.contiguous().data_ptr() if seqused_k is not None else None,
                  seqused_v.contiguous().data_ptr() if (seqused_v is not None and lse_keys is not None) else None,
                  cache_lens.data_ptr() if cache_lens is not None else None, batch, total_q,
                  k.shape[0], nheads, nheads_k, q.shape[-1], max_seqlen_q, max_seqlen_k, row_stride,
                  n_blocks, int(cache_len), int(local_blocks), int(init_blocks), float(softmax_scale),
                  int(bool(causal)), _status_words(q.device).data_ptr(), _stream(q.device))
    return (pooled, buf[:, :, :max_seqlen_k]) if return_scores else pooled


# ------------------------------------------------------------------------------------ stage 2 --

def _fwd(q, k, v, cu_seqlens_q, cu_seqlens_k, max_seqlen_q, max_seqlen_k, softmax_scale, causal,
         fwd_mask, block_table=None, leftpad_k=None, seqused_k=None):
    total_q, nheads, d = q.shape
    batch = cu_seqlens_q.numel() - 1
    out = torch.empty_like(q)
    if block_table is not None or leftpad_k is not None or seqused_k is not None:
        bt_ptr, bt_stride, page = None, 0, 0
        if block_table is not None:
            if leftpad_k is not None:
                raise NotImplementedError("infllmv2_attn_varlen_func: a paged cache takes no leftpad_k")
            page = k.shape[1]
            if page % BLOCK_N != 0:
                raise NotImplementedError("infllmv2_attn_varlen_func: page size must be a multiple of 64")
            assert block_table.shape[0] == batch
            block_table = block_table.contiguous()
            bt_ptr, bt_stride = block_table.data_ptr(), block_table.shape[1]
            k = k.contiguous().view(-1, k.shape[2], k.shape[3])
            v = v.contiguous().view(-1, v.shape[2], v.shape[3])
        for name, t in (("seqused_k", seqused_k), ("leftpad_k", leftpad_k)):
            if t is not None:
                assert t.dtype == torch.int32 and t.numel() == batch, f"{name} must be (batch,) int32"
        nheads_k = k.shape[1]
        lse = torch.empty(nheads_k, total_q * GROUP, dtype=torch.float32, device=q.device)
        with torch.cuda.device(q.device):
            _lib.call("ifv2_sparse_attn_fwd_paged", q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(),
                      lse.data_ptr(), fwd_mask.data_ptr() if fwd_mask is not None else None,
                      fwd_mask.shape[-1] if fwd_mask is not None else 0,
                      cu_seqlens_q.data_ptr(), cu_seqlens_k.data_ptr(),
                      seqused_k.contiguous().data_ptr() if seqused_k is not None else None,
                      leftpad_k.contiguous().data_ptr() if leftpad_k is not None else None,
                      bt_ptr, bt_stride, page, batch, total_q, k.shape[0], nheads, nheads_k, d,
                      max_seqlen_q, max_seqlen_k, float(softmax_scale), int(bool(causal)),
                      _status_words(q.device).data_ptr(), _stream(q.device))
        return out, lse
    nheads_k = k.shape[1]
    lse = torch.empty(nheads_k, total_q * GROUP, dtype=torch.float32, device=q.device)
    with torch.cuda.device(q.device):
        _lib.call("ifv2_sparse_attn_fwd", q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(),
                  lse.data_ptr(), fwd_mask.data_ptr() if fwd_mask is not None else None,
                  fwd_mask.shape[-1] if fwd_mask is not None else 0,
                  cu_seqlens_q.data_ptr(), cu_seqlens_k.data_ptr(), batch, total_q, k.shape[0],
                  nheads, nheads_k, d, max_seqlen_q, max_seqlen_k, float(softmax_scale),
                  int(bool(causal)), _status_words(q.device).data_ptr(), _stream(q.device))
    return out, lse


def _bwd(dout, q, k, v, out, lse, cu_seqlens_q, cu_seqlens_k, max_seqlen_q, max_seqlen_k,
         softmax_scale, causal, fwd_mask, bwd_mask):
    total_q, nheads, d = q.shape
    nheads_k = k.shape[1]
    batch = cu_seqlens_q.numel() - 1
    dq, dk, dv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
    lib = _lib.load()
    ws_bytes = int(lib.ifv2_sparse_attn_bwd_workspace_bytes(total_q, nheads, d))
    ws = torch.empty(ws_bytes, dtype=torch.uint8, device=q.device)
    with torch.cuda.device(q.device):
        _lib.call("ifv2_sparse_attn_bwd", dout.data_ptr(), q.data_ptr(), k.data_ptr(), v.data_ptr(),
                  out.data_ptr(), lse.data_ptr(), dq.data_ptr(), dk.data_ptr(), dv.data_ptr(),
                  fwd_mask.data_ptr() if fwd_mask is not None else None,
                  fwd_mask.shape[-1] if fwd_mask is not None else 0,
                  bwd_mask.data_ptr() if bwd_mask is not None else None,
                  bwd_mask.shape[-1] if bwd_mask is not None else 0,
                  cu_seqlens_q.data_ptr(), cu_seqlens_k.data_ptr(), batch, total_q, k.shape[0],
                  nheads, nheads_k, d, max_seqlen_q, max_seqlen_k, float(softmax_scale),
                  int(bool(causal)), ws.data_ptr(), ws_bytes, _status_words(q.device).data_ptr(),
                  _stream(q.device))
    return dq, dk, dv


@torch.library.custom_op("infllmv2_attn::_infllmv2_attn_varlen_forward", mutates_args=(),
                         device_types="cuda")
def _infllmv2_attn_varlen_forward(
    q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, cu_seqlens_q: torch.Tensor,
    cu_seqlens_k: torch.Tensor, max_seqlen_q: int, max_seqlen_k: int, softmax_scale: float,
    causal: bool, topk_idx: Optional[torch.Tensor] = None, block_mask: Optional[torch.Tensor] = None,
) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """Returns (out, softmax_lse (nheads_k, total_q*16), fwd_blockmask int64 or an empty tensor)."""
    q, k, v = [_dense(maybe_contiguous(x)) for x in (q, k, v)]
    if block_mask is not None:
        words = ((max_seqlen_k + BLOCK_N - 1) // BLOCK_N + 63) // 64
        if topk_idx is not None or block_mask.dtype != torch.int64 or \
                tuple(block_mask.shape) != (k.shape[1], q.shape[0], words):
            raise ValueError(f"block_mask must be int64 (nheads_k, total_q, {words}) and excludes topk_idx")
        fwd_mask = block_mask.contiguous()
    elif topk_idx is not None:
        assert topk_idx.dtype == torch.int32
        fwd_mask, _ = topk_to_uint64(topk_idx, max_seqlen_k, BLOCK_N)
    else:
        fwd_mask = None
    out, lse = _fwd(q, k, v, cu_seqlens_q.contiguous(), cu_seqlens_k.contiguous(), max_seqlen_q,
                    max_seqlen_k, softmax_scale, causal, fwd_mask)
    if fwd_mask is None or block_mask is not None:
        # (an operator output may not alias an input: the caller keeps its own block_mask)
        fwd_mask = torch.empty(0, dtype=torch.int64, device=q.device)
    return out, lse, fwd_mask


@_infllmv2_attn_varlen_forward.register_fake
def _(q, k, v, cu_seqlens_q, cu_seqlens_k, max_seqlen_q, max_seqlen_k, softmax_scale, causal,
      topk_idx=None, block_mask=None):
    words = ((max_seqlen_k + BLOCK_N - 1) // BLOCK_N + 63) // 64
    mask = (q.new_empty((k.shape[1], q.shape[0], words), dtype=torch.int64)
            if (topk_idx is not None and block_mask is None) else q.new_empty((0,), dtype=torch.int64))
    return (torch.empty_like(q),
            q.new_empty((k.shape[1], q.shape[0] * GROUP), dtype=torch.float32), mask)


@torch.library.custom_op("infllmv2_attn::_infllmv2_attn_varlen_backward", mutates_args=(),
                         device_types="cuda")
def _infllmv2_attn_varlen_backward(
    dout: torch.Tensor, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, out: torch.Tensor,
    softmax_lse: torch.Tensor, cu_seqlens_q: torch.Tensor, cu_seqlens_k: torch.Tensor,
    max_seqlen_q: int, max_seqlen_k: int, softmax_scale: float, causal: bool,
    fwd_blockmask: torch.Tensor,
) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    dout = _dense(maybe_contiguous(dout))
    fwd_mask = bwd_mask = None
    if fwd_blockmask.numel() > 0:
        k_blocks = (max_seqlen_k + BLOCK_N - 1) // BLOCK_N
        fwd_mask = fwd_blockmask
        bwd_mask = transpose_blockmask(fwd_blockmask, k_blocks)
    return _bwd(dout, q, k, v, out, softmax_lse, cu_seqlens_q.contiguous(),
                cu_seqlens_k.contiguous(), max_seqlen_q, max_seqlen_k, softmax_scale, causal,
                fwd_mask, bwd_mask)


@_infllmv2_attn_varlen_backward.register_fake
def _(dout, q, k, v, out, softmax_lse, cu_seqlens_q, cu_seqlens_k, max_seqlen_q, max_seqlen_k,
      softmax_scale, causal, fwd_blockmask):
    return torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)


class Infllmv2AttnVarlenFunc(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, cu_seqlens_q, cu_seqlens_k, max_seqlen_q, max_seqlen_k, dropout_p,
                softmax_scale, causal, window_size, softcap, alibi_slopes, deterministic,
                return_softmax, block_table, topk_idx, block_mask=None):
        _check_common(q, k, dropout_p, window_size, softcap, alibi_slopes, block_table,
                      "infllmv2_attn_varlen_func")
        if softmax_scale is None:
            softmax_scale = q.shape[-1] ** (-0.5)
        out, lse, fwd_mask = _infllmv2_attn_varlen_forward(
            q, k, v, cu_seqlens_q, cu_seqlens_k, max_seqlen_q, max_seqlen_k, softmax_scale, causal,
            topk_idx, block_mask)
        if block_mask is not None:
            fwd_mask = block_mask.contiguous()
        ctx.save_for_backward(q, k, v, out, lse, cu_seqlens_q, cu_seqlens_k, fwd_mask)
        ctx.max_seqlen_q, ctx.max_seqlen_k = max_seqlen_q, max_seqlen_k
        ctx.softmax_scale, ctx.causal = softmax_scale, causal
        return out if not return_softmax else (out, lse, None)

    @staticmethod
    def backward(ctx, dout, *args):
        q, k, v, out, lse, cu_seqlens_q, cu_seqlens_k, fwd_mask = ctx.saved_tensors
        dq, dk, dv = _infllmv2_attn_varlen_backward(
            dout, q, k, v, out, lse, cu_seqlens_q, cu_seqlens_k, ctx.max_seqlen_q,
            ctx.max_seqlen_k, ctx.softmax_scale, ctx.causal, fwd_mask)
        if _CHECK_STATUS:
            check_device_status(q.device)
        return (dq, dk, dv) + (None,) * 15


def infllmv2_attn_varlen_func(
    q, k, v, cu_seqlens_q, cu_seqlens_k, max_seqlen_q, max_seqlen_k, dropout_p=0.0,
    softmax_scale=None, causal=False, window_size=(-1, -1), softcap=0.0, alibi_slopes=None,
    deterministic=False, return_attn_probs=False, block_table=None, topk_idx=None, block_mask=None,
    leftpad_k=None, seqused_k=None,
):
    """Block-sparse varlen attention (stage 2), differentiable.

    q: (total_q, nheads, 128); k, v: (total_k, nheads_k, 128), bf16, nheads = 16 * nheads_k.
    cu_seqlens_q / cu_seqlens_k: (batch + 1,) int32.  topk_idx: int32 (nheads_k, total_q, topk)
    block indices local to each sequence's keys (64-token blocks, -1 = unused); None = dense
    attention.  block_mask (an addition): the same selection already packed, int64 (nheads_k,
    total_q, ceil(ceil(max_seqlen_k / 64) / 64)) as topk_to_uint64 / infllmv2_topk_mask return it.  causal=True aligns the diagonal to the bottom right when seqlen_q != seqlen_k.
    Rows that see no key return 0.  Returns out (total_q, nheads, 128), or
    (out, softmax_lse (nheads_k, total_q * 16), None) with return_attn_probs=True.
    block_table (batch, max_pages) int32: k and v are a paged cache (num_pages, page_size, nheads_k,
    128), page_size a multiple of 64 (the reference wants 256, flash_api.cpp:592-596), and
    cu_seqlens_k / seqused_k give each sequence's key count.  leftpad_k (batch,) int32: the keys of a
    sequence start that many rows into its cu_seqlens_k extent; seqused_k (batch,) int32: keys in
    use per sequence (flash_api.cpp:717-742, block_info.h:22-24).  These three are forward-only, as
    in the reference, whose backward takes none of them.
    """
    if block_table is not None or leftpad_k is not None or seqused_k is not None:
        _check_common(q, k, dropout_p, window_size, softcap, alibi_slopes, block_table,
                      "infllmv2_attn_varlen_func")
        if any(t.requires_grad for t in (q, k, v)) and torch.is_grad_enabled():
            raise NotImplementedError("infllmv2_attn_varlen_func: block_table / leftpad_k / seqused_k are "
                                      "forward-only (the reference's backward takes none of them)")
        if softmax_scale is None:
            softmax_scale = q.shape[-1] ** (-0.5)
        q = _dense(maybe_contiguous(q))
        if block_table is None:
            k, v = _dense(maybe_contiguous(k)), _dense(maybe_contiguous(v))
        nheads_k = k.shape[-2]
        words = ((max_seqlen_k + BLOCK_N - 1) // BLOCK_N + 63) // 64
        if block_mask is not None:
            if topk_idx is not None or block_mask.dtype != torch.int64 or \
                    tuple(block_mask.shape) != (nheads_k, q.shape[0], words):
                raise ValueError(f"block_mask must be int64 (nheads_k, total_q, {words}) and excludes topk_idx")
            fwd_mask = block_mask.contiguous()
        elif topk_idx is not None:
            assert topk_idx.dtype == torch.int32
            fwd_mask, _ = topk_to_uint64(topk_idx, max_seqlen_k, BLOCK_N)
        else:
            fwd_mask = None
        out, lse = _fwd(q, k, v, cu_seqlens_q.contiguous(), cu_seqlens_k.contiguous(), max_seqlen_q,
                        max_seqlen_k, softmax_scale, causal, fwd_mask, block_table, leftpad_k, seqused_k)
        return (out, lse, None) if return_attn_probs else out
    return Infllmv2AttnVarlenFunc.apply(
        q, k, v, cu_seqlens_q, cu_seqlens_k, max_seqlen_q, max_seqlen_k, dropout_p, softmax_scale,
        causal, window_size, softcap, alibi_slopes, deterministic, return_attn_probs, block_table,
        topk_idx, block_mask)


# ------------------------------------------------------------------------------------ decode --

def infllmv2_attn_with_kvcache(
    q, k_cache, v_cache, k=None, v=None, rotary_cos=None, rotary_sin=None,
    cache_seqlens: Optional[Union[int, torch.Tensor]] = None,
    cache_batch_idx: Optional[torch.Tensor] = None, cache_leftpad: Optional[torch.Tensor] = None,
    block_table: Optional[torch.Tensor] = None, softmax_scale=None, causal=False,
    window_size=(-1, -1), softcap=0.0, rotary_interleaved=True, alibi_slopes=None, num_splits=0,
    return_softmax_lse=False, topk_idx=None, block_mask=None,
):
    """Sparse decode step over a KV cache (one new query token per sequence).

    q: (batch, 1, nheads, 128); k_cache, v_cache: (batch_cache, seqlen_cache, nheads_k, 128), or
    (num_pages, page_size, nheads_k, 128) with block_table (batch, max_pages) int32;
    k, v: optional (batch, 1, nheads_k, 128), written in place at cache_seqlens first;
    cache_seqlens: int or (batch,) int32; cache_batch_idx (batch,) int32: the cache row each
    sequence uses; cache_leftpad (batch,) int32: position of each sequence's first key;
    topk_idx: int32 (batch, nheads_k, 1, topk) blocks of the sequence to attend (None = all of
    it), counted from its first key.  block_mask (an addition): the same selection already packed
    into 64-bit words, (batch, nheads_k, 1, words) int64 as ops.decode_select returns it.
    A single query token is never causally masked
    (csrc/flash_attn/flash_api.cpp:1628).  Returns out (batch, 1, nheads, 128)
    [, softmax_lse (batch, nheads, 1)].
    """
    assert k_cache.stride(-1) == 1, "k_cache must have contiguous last dimension"
    assert v_cache.stride(-1) == 1, "v_cache must have contiguous last dimension"
    _check_common(q, k_cache, 0.0, window_size, softcap, alibi_slopes, None,
                  "infllmv2_attn_with_kvcache")
    if (rotary_cos is None) != (rotary_sin is None):
        raise ValueError("infllmv2_attn_with_kvcache: pass both rotary_cos and rotary_sin, or neither")
    if q.shape[1] != 1:
        raise NotImplementedError("infllmv2_attn_with_kvcache: only one query token per sequence is supported")
    q, k, v = [maybe_contiguous(x) for x in (q, k, v)]
    if softmax_scale is None:
        softmax_scale = q.shape[-1] ** (-0.5)
    batch, _, nheads, d = q.shape
    nheads_k = k_cache.shape[2]
    bt_ptr, bt_stride, page_size = None, 0, 0
    if block_table is not None:
        if cache_batch_idx is not None or cache_leftpad is not None:
            raise NotImplementedError(
                "infllmv2_attn_with_kvcache: a paged cache takes neither cache_batch_idx nor cache_leftpad")
        assert block_table.dtype == torch.int32 and block_table.shape[0] == batch
        block_table = block_table.contiguous()
        page_size = k_cache.shape[1]
        if page_size % BLOCK_N != 0:
            raise NotImplementedError("infllmv2_attn_with_kvcache: page size must be a multiple of 64")
        bt_ptr, bt_stride = block_table.data_ptr(), block_table.shape[1]
        cap = bt_stride * page_size
    else:
        cap = k_cache.shape[1]
    if cache_seqlens is None:
        cache_seqlens = cap
    if isinstance(cache_seqlens, int):
        cache_seqlens = torch.full((batch,), cache_seqlens, dtype=torch.int32, device=q.device)
    cache_seqlens = cache_seqlens.contiguous()
    assert cache_seqlens.dtype == torch.int32
    for name, t in (("cache_batch_idx", cache_batch_idx), ("cache_leftpad", cache_leftpad)):
        if t is not None:
            assert t.dtype == torch.int32 and t.numel() == batch, f"{name} must be (batch,) int32"
    for c in (k_cache, v_cache):
        if c.stride(2) != d or c.stride(1) != nheads_k * d:
            raise RuntimeError("infllmv2_attn_with_kvcache: caches must be dense in (seqlen, heads, d)")
    mask = None
    if block_mask is not None:
        # an already packed selection (ops.decode_select): (batch, nheads_k, [1,] words) int64
        words = ((cap + BLOCK_N - 1) // BLOCK_N + 63) // 64
        if topk_idx is not None or block_mask.dtype != torch.int64 or block_mask.numel() != batch * nheads_k * words:
            raise ValueError("infllmv2_attn_with_kvcache: block_mask must be (batch, nheads_k, 1, "
                             f"{words}) int64 and excludes topk_idx")
        mask = block_mask.contiguous().view(batch, nheads_k, 1, words)
    elif topk_idx is not None:
        assert topk_idx.dtype == torch.int32
        mask, _ = topk_to_uint64(topk_idx, cap, BLOCK_N)
    q2 = q.reshape(batch, nheads, d).contiguous()
    if rotary_cos is not None and k is not None:
        # as in the reference, the rotation applies to the appended key and to the query, both at
        # the position of the append; without an append nothing is rotated
        if rotary_cos.dtype != q.dtype or rotary_cos.shape != rotary_sin.shape or rotary_cos.dim() != 2:
            raise ValueError("infllmv2_attn_with_kvcache: rotary_cos / rotary_sin must be "
                             "(seqlen_ro, rotary_dim / 2) in the dtype of q")
        k2 = k.reshape(batch, nheads_k, d).contiguous()
        q_rot, k_rot = torch.empty_like(q2), torch.empty_like(k2)
        with torch.cuda.device(q.device):
            _lib.call("ifv2_decode_rotary", q2.data_ptr(), k2.data_ptr(), q_rot.data_ptr(), k_rot.data_ptr(),
                      rotary_cos.contiguous().data_ptr(), rotary_sin.contiguous().data_ptr(),
                      cache_seqlens.data_ptr(), batch, nheads, nheads_k, d, 2 * rotary_cos.shape[1],
                      rotary_cos.shape[0], int(bool(rotary_interleaved)), _stream(q.device))
        q2, k = q_rot, k_rot
    out = torch.empty_like(q2)
    lse = torch.empty(batch, nheads, dtype=torch.float32, device=q.device)
    lib = _lib.load()
    max_blocks = (cap + BLOCK_N - 1) // BLOCK_N
    ws_bytes = int(lib.ifv2_decode_workspace_bytes(batch, nheads, d, max_blocks))
    ws = torch.empty(max(ws_bytes, 16), dtype=torch.uint8, device=q.device)
    with torch.cuda.device(q.device):
        _lib.call("ifv2_decode_paged", q2.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(),
                  k.contiguous().data_ptr() if k is not None else None,
                  v.contiguous().data_ptr() if v is not None else None, out.data_ptr(),
                  lse.data_ptr(), mask.data_ptr() if mask is not None else None,
                  mask.shape[-1] if mask is not None else 0, cache_seqlens.data_ptr(), batch,
                  nheads, nheads_k, d, cap, k_cache.stride(0), bt_ptr, bt_stride, page_size,
                  cache_batch_idx.contiguous().data_ptr() if cache_batch_idx is not None else None,
                  cache_leftpad.contiguous().data_ptr() if cache_leftpad is not None else None,
                  float(softmax_scale), ws.data_ptr(), ws_bytes, _stream(q.device))
    out = out.view(batch, 1, nheads, d)
    return (out, lse.view(batch, nheads, 1)) if return_softmax_lse else out
