"""Selection and bitmask operators with the reference's Python signatures.

Same names, argument order, defaults and return values as infllm_v2/{topk_to_uint64,
blockmask_to_uint64, uint64_to_bool, max_pooling_1d}.py of the reference; every call goes to
the CUDA library through the C ABI on the current stream.  `infllmv2_topk` and
`transpose_blockmask` are additions (the reference leaves top-k to its caller and builds the
backward mask through a bool round trip).
"""
from typing import Optional, Tuple

import torch

from . import _lib


def _stream(device) -> int:
    return torch.cuda.current_stream(device).cuda_stream


def _require_cuda(t: torch.Tensor, name: str):
    if not t.is_cuda:
        raise RuntimeError(f"{name} must be a CUDA tensor (got {t.device}); this library has no CPU path")


def topk_to_uint64(topk_idx: torch.Tensor, max_seqlen_k: int, block_size: int,
                   memory_buffer: Optional[torch.Tensor] = None) -> Tuple[torch.Tensor, int]:
    """Top-k block indices -> packed int64 bitmask rows.

    topk_idx: int32 [num_heads, total_seqlen, k] or [batch, num_heads, seqlen, k]; -1 = unused.
    Returns (int64 tensor with the last dim replaced by ceil(k_blocks/64), k_blocks).
    Mirrors infllm_v2/topk_to_uint64.py:5-72.
    """
    assert topk_idx.dtype == torch.int32
    _require_cuda(topk_idx, "topk_idx")
    if topk_idx.dim() not in (3, 4):
        raise ValueError("topk_idx must be 3-D or 4-D")
    k_blocks = (max_seqlen_k + block_size - 1) // block_size
    words = (k_blocks + 63) // 64
    topk_idx = topk_idx.contiguous()
    out_shape = tuple(topk_idx.shape[:-1]) + (words,)
    rows = topk_idx.numel() // max(topk_idx.shape[-1], 1) if topk_idx.shape[-1] else \
        int(torch.Size(topk_idx.shape[:-1]).numel())
    if (memory_buffer is not None and memory_buffer.dtype == torch.int64
            and tuple(memory_buffer.shape) == out_shape and memory_buffer.is_contiguous()
            and memory_buffer.device == topk_idx.device):
        result = memory_buffer
    else:
        result = torch.empty(out_shape, dtype=torch.int64, device=topk_idx.device)
    with torch.cuda.device(topk_idx.device):
        _lib.call("ifv2_topk_to_uint64", topk_idx.data_ptr(), result.data_ptr(), rows,
                  topk_idx.shape[-1], k_blocks, words, _stream(topk_idx.device))
    return result, k_blocks


def blockmask_to_uint64(blockmask: torch.Tensor) -> Tuple[torch.Tensor, int]:
    """Bool mask [..., n] -> (int64 [..., ceil(n/64)], n).  Mirrors infllm_v2/blockmask_to_uint64.py:5-42."""
    _require_cuda(blockmask, "blockmask")
    if blockmask.dtype != torch.bool:
        raise TypeError("blockmask must be a bool tensor")
    blockmask = blockmask.contiguous()
    last = blockmask.shape[-1]
    words = (last + 63) // 64
    rows = int(torch.Size(blockmask.shape[:-1]).numel())
    result = torch.empty(tuple(blockmask.shape[:-1]) + (words,), dtype=torch.int64,
                         device=blockmask.device)
    with torch.cuda.device(blockmask.device):
        _lib.call("ifv2_blockmask_to_uint64", blockmask.data_ptr(), result.data_ptr(), rows, last,
                  words, _stream(blockmask.device))
    return result, last


def uint64_to_bool(uint64_array: torch.Tensor, last_dim_size: int) -> torch.Tensor:
    """Packed int64 rows -> bool [..., last_dim_size].  Mirrors infllm_v2/uint64_to_bool.py:5-38."""
    _require_cuda(uint64_array, "uint64_array")
    if uint64_array.dtype != torch.int64:
        raise TypeError("uint64_array must be an int64 tensor")
    uint64_array = uint64_array.contiguous()
    words = uint64_array.shape[-1]
    rows = int(torch.Size(uint64_array.shape[:-1]).numel())
    result = torch.empty(tuple(uint64_array.shape[:-1]) + (last_dim_size,), dtype=torch.bool,
                         device=uint64_array.device)
    with torch.cuda.device(uint64_array.device):
        _lib.call("ifv2_uint64_to_bool", uint64_array.data_ptr(), result.data_ptr(), rows,
                  last_dim_size, words, _stream(uint64_array.device))
    return result


def transpose_blockmask(fwd_mask: torch.Tensor, k_blocks: int) -> torch.Tensor:
    """Row mask (Hk, T, ceil(k_blocks/64)) -> column mask (Hk, k_blocks, ceil(T/64)) in one kernel:
    out[h, blk, t//64] bit t%64 = in[h, t, blk//64] bit blk%64.  Equals the reference's
    uint64_to_bool -> transpose(1, 2) -> blockmask_to_uint64 sequence
    (infllm_v2/infllmv2_sparse_attention.py:343-350) without the bool tensors or the sync."""
    _require_cuda(fwd_mask, "fwd_mask")
    if fwd_mask.dtype != torch.int64 or fwd_mask.dim() != 3:
        raise TypeError("fwd_mask must be a 3-D int64 tensor")
    fwd_mask = fwd_mask.contiguous()
    hk, t, words = fwd_mask.shape
    if words != (k_blocks + 63) // 64:
        raise ValueError(f"fwd_mask has {words} words per row, k_blocks={k_blocks} needs {(k_blocks + 63) // 64}")
    out = torch.empty(hk, k_blocks, (t + 63) // 64, dtype=torch.int64, device=fwd_mask.device)
    with torch.cuda.device(fwd_mask.device):
        _lib.call("ifv2_transpose_blockmask", fwd_mask.data_ptr(), out.data_ptr(), hk, t, k_blocks,
                  _stream(fwd_mask.device))
    return out


def _row_view(x: torch.Tensor):
    """Accept (H, R, C) tensors whose rows are contiguous and evenly strided (e.g. a column
    slice of a padded buffer) without copying; anything else is made contiguous.
    Returns (tensor, elements between consecutive rows)."""
    h, r, c = x.shape
    if x.numel() and x.stride(2) == 1 and x.stride(1) >= c and x.stride(0) == x.stride(1) * r:
        return x, x.stride(1)
    return x.contiguous(), c


def max_pooling_1d(input: torch.Tensor, cache_len: int, local_blocks: int, init_blocks: int,
                   block_size: int = 64, stride: int = 16) -> torch.Tensor:
    """input: (num_heads, q_len, k_len) bf16/fp16 stage-1 scores -> (num_heads, q_len,
    ceil((q_len + cache_len) / block_size)).  Mirrors infllm_v2/max_pooling_1d.py:4-46."""
    assert input.dtype == torch.float16 or input.dtype == torch.bfloat16
    _require_cuda(input, "input")
    if input.dim() != 3:
        raise ValueError(f"Expected 3D input, got {input.dim()}D")
    input, row_stride = _row_view(input)
    pool_stride = block_size // stride
    kernel_size, padding = pool_stride + 1, 1
    num_heads, q_len, k_len = input.shape
    out_len = (q_len + cache_len + block_size - 1) // block_size
    output = torch.empty(num_heads, q_len, out_len, device=input.device, dtype=input.dtype)
    with torch.cuda.device(input.device):
        _lib.call("ifv2_max_pooling_1d", input.data_ptr(), output.data_ptr(),
                  int(input.dtype == torch.bfloat16), num_heads, q_len, k_len, row_stride, out_len,
                  cache_len, kernel_size, pool_stride, padding, block_size, local_blocks,
                  init_blocks, _stream(input.device))
    return output


def max_pooling_1d_varlen(input: torch.Tensor, cu_seqlens_q: torch.Tensor,
                          cu_seqlens_k: torch.Tensor, cache_lens: torch.Tensor,
                          max_seqlen_q: int, max_seqlen_k: int, local_blocks: int,
                          init_blocks: int, block_size: int = 64, stride: int = 16,
                          max_cache_len: Optional[int] = None) -> torch.Tensor:
    """Packed-sequence max-pool.  input: (num_heads, total_q, max_k).  Mirrors
    infllm_v2/max_pooling_1d.py:49-138.  `max_cache_len` (an addition) lets the caller pass
    max(cache_lens) and so avoid the device->host read the output shape otherwise needs."""
    assert input.dtype == torch.float16 or input.dtype == torch.bfloat16
    assert cu_seqlens_q.dtype == torch.int32
    assert cu_seqlens_k.dtype == torch.int32
    assert cache_lens.dtype == torch.int32
    assert input.dim() == 3, f"Expected 3D input, got {input.dim()}D"
    _require_cuda(input, "input")
    input, row_stride = _row_view(input)
    cu_seqlens_q, cu_seqlens_k = cu_seqlens_q.contiguous(), cu_seqlens_k.contiguous()
    cache_lens = cache_lens.contiguous()
    pool_stride = block_size // stride
    kernel_size, padding = pool_stride + 1, 1
    batch_size = cu_seqlens_q.shape[0] - 1
    num_heads, total_q, max_k = input.shape
    assert max_k == max_seqlen_k, f"max_k mismatch: {max_k} vs {max_seqlen_k}"
    assert cache_lens.shape[0] == batch_size, \
        f"cache_lens batch size mismatch: {cache_lens.shape[0]} vs {batch_size}"
    if max_cache_len is None:
        max_cache_len = int(cache_lens.max().item())
    out_len = (max_seqlen_q + max_cache_len + block_size - 1) // block_size
    output = torch.empty(num_heads, total_q, out_len, device=input.device, dtype=input.dtype)
    with torch.cuda.device(input.device):
        _lib.call("ifv2_max_pooling_1d_varlen", input.data_ptr(), output.data_ptr(),
                  cu_seqlens_q.data_ptr(), cu_seqlens_k.data_ptr(), cache_lens.data_ptr(),
                  int(input.dtype == torch.bfloat16), batch_size, num_heads, total_q, max_seqlen_k,
                  row_stride, out_len, kernel_size, pool_stride, padding, block_size, local_blocks,
                  init_blocks, _stream(input.device))
    return output


def infllmv2_topk(block_score: torch.Tensor, k: int, cache_len: int = 0,
                  cu_seqlens_q: Optional[torch.Tensor] = None,
                  cache_lens: Optional[torch.Tensor] = None, block_size: int = 64) -> torch.Tensor:
    """Per-query top-k of block scores (Hk, T, n_blocks) -> int32 (Hk, T, k).

    Picks the k entries first in (value descending, index ascending) order -- the ordering of
    the reference's bitonic top-k, csrc/topk.cuh:17 -- and returns their indices ascending, -1
    in the unused tail.  Indices greater than the query's own block
    ((local token + cache_len) // block_size) are replaced by -1.  With cu_seqlens_q the token
    index is local to its sequence and cache_lens (optional) gives a per-sequence cache length.
    """
    assert block_score.dtype == torch.float16 or block_score.dtype == torch.bfloat16
    _require_cuda(block_score, "block_score")
    if block_score.dim() != 3:
        raise ValueError("block_score must be (num_heads, total_q, n_blocks)")
    block_score, row_stride = _row_view(block_score)
    hk, t, n = block_score.shape
    out = torch.empty(hk, t, k, dtype=torch.int32, device=block_score.device)
    batch = 1
    cu_ptr = cl_ptr = None
    if cu_seqlens_q is not None:
        assert cu_seqlens_q.dtype == torch.int32
        cu_seqlens_q = cu_seqlens_q.contiguous()
        batch = cu_seqlens_q.shape[0] - 1
        cu_ptr = cu_seqlens_q.data_ptr()
        if cache_lens is not None:
            assert cache_lens.dtype == torch.int32 and cache_lens.shape[0] == batch
            cache_lens = cache_lens.contiguous()
            cl_ptr = cache_lens.data_ptr()
    elif cache_lens is not None:
        raise ValueError("cache_lens needs cu_seqlens_q")
    with torch.cuda.device(block_score.device):
        _lib.call("ifv2_topk_select", block_score.data_ptr(), out.data_ptr(),
                  int(block_score.dtype == torch.bfloat16), hk, t, n, row_stride, k, cu_ptr, cl_ptr,
                  batch, cache_len, block_size, _stream(block_score.device))
    return out


def infllmv2_topk_mask(block_score: torch.Tensor, k: int, max_seqlen_k: int, cache_len: int = 0,
                       cu_seqlens_q: Optional[torch.Tensor] = None,
                       cache_lens: Optional[torch.Tensor] = None, block_size: int = 64,
                       return_idx: bool = False, return_col_mask: bool = False):
    """Top-k of block scores straight to the packed block mask (an addition to the reference API):
    the selection of `infllmv2_topk` and the words of `topk_to_uint64(idx, max_seqlen_k, block_size)`
    from one kernel, without the int32 list in between.  Returns (row_mask int64 (Hk, T,
    ceil(k_blocks / 64)), k_blocks) followed, when asked for, by topk_idx (Hk, T, k) int32 and by
    the column mask (Hk, k_blocks, ceil(T / 64)) that the backward reads (`transpose_blockmask`
    of the row mask, run inside the same call).  Pass the row mask to infllmv2_attn_varlen_func
    as `block_mask`."""
    assert block_score.dtype == torch.float16 or block_score.dtype == torch.bfloat16
    _require_cuda(block_score, "block_score")
    if block_score.dim() != 3:
        raise ValueError("block_score must be (num_heads, total_q, n_blocks)")
    block_score, row_stride = _row_view(block_score)
    hk, t, n = block_score.shape
    dev = block_score.device
    k_blocks = (max_seqlen_k + block_size - 1) // block_size
    words = (k_blocks + 63) // 64
    mask = torch.empty(hk, t, words, dtype=torch.int64, device=dev)
    idx = torch.empty(hk, t, k, dtype=torch.int32, device=dev) if return_idx else None
    col = torch.empty(hk, k_blocks, (t + 63) // 64, dtype=torch.int64, device=dev) if return_col_mask else None
    batch = 1
    cu_ptr = cl_ptr = None
    if cu_seqlens_q is not None:
        assert cu_seqlens_q.dtype == torch.int32
        cu_seqlens_q = cu_seqlens_q.contiguous()
        batch = cu_seqlens_q.shape[0] - 1
        cu_ptr = cu_seqlens_q.data_ptr()
        if cache_lens is not None:
            assert cache_lens.dtype == torch.int32 and cache_lens.shape[0] == batch
            cache_lens = cache_lens.contiguous()
            cl_ptr = cache_lens.data_ptr()
    elif cache_lens is not None:
        raise ValueError("cache_lens needs cu_seqlens_q")
    with torch.cuda.device(dev):
        _lib.call("ifv2_topk_select_mask", block_score.data_ptr(), idx.data_ptr() if idx is not None else None,
                  mask.data_ptr(), col.data_ptr() if col is not None else None,
                  int(block_score.dtype == torch.bfloat16), hk, t, n, row_stride, k, k_blocks, cu_ptr, cl_ptr,
                  batch, cache_len, block_size, _stream(dev))
    out = (mask, k_blocks)
    if return_idx:
        out += (idx,)
    if return_col_mask:
        out += (col,)
    return out


def compressed_lengths(cu_seqlens_k: torch.Tensor, kernel_size: int = 32,
                       kernel_stride: int = 16) -> torch.Tensor:
    """Cumulative number of compressed keys per sequence (int32, same device, no host sync):
    a sequence of length L has (L - kernel_size) // kernel_stride + 1 full windows, none when
    L < kernel_size (tests/test_stage1_compressed_lse.py:11-55, calc_chunks_with_stride)."""
    lens = (cu_seqlens_k[1:] - cu_seqlens_k[:-1]).to(torch.int64)
    n = torch.where(lens >= kernel_size, (lens - kernel_size) // kernel_stride + 1,
                    torch.zeros_like(lens))
    cu_c = torch.zeros_like(cu_seqlens_k, dtype=torch.int32)
    cu_c[1:] = n.cumsum(0).to(torch.int32)
    return cu_c


def compress_keys(k: torch.Tensor, cu_seqlens_k: Optional[torch.Tensor] = None, kernel_size: int = 32,
                  kernel_stride: int = 16, cu_seqlens_c: Optional[torch.Tensor] = None,
                  total_c: Optional[int] = None) -> Tuple[torch.Tensor, Optional[torch.Tensor]]:
    """Mean-pool keys (total_k, Hk, 128) bf16 into compressed keys (total_c, Hk, 128): window j of
    a sequence covers its tokens [stride*j, stride*j + kernel), full windows only -- what the
    reference's tests build with `compress_tensor` (tests/test_stage1_compressed_lse.py:57-99)
    before calling infllmv2_attn_stage1 (there in (heads, tokens, d) layout).

    Returns (kc, cu_seqlens_c).  Without cu_seqlens_k the input is one sequence and cu_seqlens_c is
    None.  With it, pass cu_seqlens_c / total_c when known; otherwise they are computed here and
    total_c costs one device->host read.
    """
    _require_cuda(k, "k")
    if k.dtype != torch.bfloat16 or k.dim() != 3:
        raise ValueError("k must be (total_k, heads_k, head_dim) bf16")
    k = k.contiguous()
    total_k, hk, d = k.shape
    if cu_seqlens_k is None:
        total_c = (total_k - kernel_size) // kernel_stride + 1 if total_k >= kernel_size else 0
        batch, cu_k_ptr, cu_c_ptr = 1, None, None
    else:
        assert cu_seqlens_k.dtype == torch.int32
        cu_seqlens_k = cu_seqlens_k.contiguous()
        batch = cu_seqlens_k.shape[0] - 1
        if cu_seqlens_c is None:
            cu_seqlens_c = compressed_lengths(cu_seqlens_k, kernel_size, kernel_stride)
        cu_seqlens_c = cu_seqlens_c.contiguous()
        if total_c is None:
            total_c = int(cu_seqlens_c[-1].item())
        cu_k_ptr, cu_c_ptr = cu_seqlens_k.data_ptr(), cu_seqlens_c.data_ptr()
    kc = torch.empty(total_c, hk, d, dtype=k.dtype, device=k.device)
    with torch.cuda.device(k.device):
        _lib.call("ifv2_compress_keys", k.data_ptr(), kc.data_ptr(), cu_k_ptr, cu_c_ptr, batch,
                  total_k, total_c, hk, d, kernel_size, kernel_stride, _stream(k.device))
    return kc, cu_seqlens_c


def compress_keys_append(k_cache: torch.Tensor, cache_seqlens: torch.Tensor, kc_cache: torch.Tensor,
                         kernel_size: int = 32, kernel_stride: int = 16) -> None:
    """Decode-time update, in place: for every sequence whose length (AFTER the append of the new
    token, `cache_seqlens`) completes a window -- L >= kernel and (L - kernel) % stride == 0 --
    write that window's mean into kc_cache[b, (L - kernel) // stride].
    k_cache (B, cap, Hk, 128), kc_cache (B, c_cap, Hk, 128), both bf16 and contiguous."""
    _require_cuda(k_cache, "k_cache")
    _require_cuda(kc_cache, "kc_cache")
    if (k_cache.dtype != torch.bfloat16 or kc_cache.dtype != torch.bfloat16 or k_cache.dim() != 4
            or kc_cache.dim() != 4 or not k_cache.is_contiguous() or not kc_cache.is_contiguous()):
        raise ValueError("k_cache / kc_cache must be contiguous (batch, capacity, heads_k, 128) bf16")
    assert cache_seqlens.dtype == torch.int32 and cache_seqlens.shape[0] == k_cache.shape[0]
    b, cap, hk, d = k_cache.shape
    if kc_cache.shape[0] != b or kc_cache.shape[2] != hk or kc_cache.shape[3] != d:
        raise ValueError("kc_cache does not match k_cache")
    with torch.cuda.device(k_cache.device):
        _lib.call("ifv2_compress_keys_append", k_cache.data_ptr(), kc_cache.data_ptr(),
                  cache_seqlens.contiguous().data_ptr(), b, cap, kc_cache.shape[1], hk, d,
                  kernel_size, kernel_stride, _stream(k_cache.device))


def cache_fill(src: torch.Tensor, cache: torch.Tensor, cu_seqlens: torch.Tensor,
               seqlens_out: Optional[torch.Tensor] = None) -> None:
    """Copy the packed rows of every sequence (src: (total, Hk, 128) bf16, cu_seqlens (B+1) int32)
    to rows [0, len_b) of its slot of cache (B, capacity, Hk, 128), in place; rows past the
    capacity are dropped.  seqlens_out (B,) int32, optional: min(len_b, capacity)."""
    _require_cuda(src, "src")
    _require_cuda(cache, "cache")
    if (src.dtype != torch.bfloat16 or cache.dtype != torch.bfloat16 or src.dim() != 3 or cache.dim() != 4
            or not cache.is_contiguous() or cache.shape[2:] != src.shape[1:]):
        raise ValueError("cache_fill: src (total, heads_k, 128) and contiguous cache (batch, capacity, heads_k, 128), bf16")
    assert cu_seqlens.dtype == torch.int32 and cu_seqlens.numel() == cache.shape[0] + 1
    if seqlens_out is not None:
        assert seqlens_out.dtype == torch.int32 and seqlens_out.is_contiguous() and seqlens_out.numel() == cache.shape[0]
    src = src.contiguous()
    with torch.cuda.device(src.device):
        _lib.call("ifv2_cache_fill", src.data_ptr(), cache.data_ptr(), cu_seqlens.contiguous().data_ptr(),
                  seqlens_out.data_ptr() if seqlens_out is not None else None, cache.shape[0],
                  src.shape[0], cache.shape[1], cache.shape[2], cache.shape[3], _stream(src.device))


def decode_append(k_new: torch.Tensor, v_new: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor,
                  cache_seqlens: torch.Tensor, positions: Optional[torch.Tensor] = None,
                  kc_cache: Optional[torch.Tensor] = None, n_comp: Optional[torch.Tensor] = None,
                  kernel_size: int = 32, kernel_stride: int = 16,
                  kc2_cache: Optional[torch.Tensor] = None, n_comp2: Optional[torch.Tensor] = None,
                  kernel2_size: int = 128, kernel2_stride: int = 64) -> None:
    """One decode step of cache bookkeeping, one launch, all in place: k_new / v_new (B, Hk, 128)
    are written at position cache_seqlens[b] of k_cache / v_cache (B, capacity, Hk, 128); a
    sequence whose new length completes a compression window gets that window's mean in kc_cache
    (B, c_capacity, Hk, 128) (and kc2_cache for the second compression); cache_seqlens (B,) int32
    is advanced in place, positions (B,) int32 receives the old lengths (the `cache_lens` of the
    pool and top-k), n_comp / n_comp2 the number of valid compressed keys (the `seqused_k` of the
    stage-1 scorer).  No pointer changes from step to step.  A sequence whose cache is full is
    left as it is."""
    for name, t in (("k_new", k_new), ("v_new", v_new), ("k_cache", k_cache), ("v_cache", v_cache)):
        _require_cuda(t, name)
        if t.dtype != torch.bfloat16 or not t.is_contiguous():
            raise ValueError(f"decode_append: {name} must be contiguous bf16")
    b, cap, hk, d = k_cache.shape
    if v_cache.shape != k_cache.shape or k_new.numel() != b * hk * d or v_new.numel() != b * hk * d:
        raise ValueError("decode_append: shapes of the new rows and the caches do not match")
    for t in (cache_seqlens, positions, n_comp, n_comp2):
        assert t is None or (t.dtype == torch.int32 and t.is_contiguous() and t.numel() == b)
    for c in (kc_cache, kc2_cache):
        if c is not None and (c.dtype != torch.bfloat16 or not c.is_contiguous() or c.dim() != 4
                              or c.shape[0] != b or c.shape[2:] != k_cache.shape[2:]):
            raise ValueError("decode_append: a compressed cache must be contiguous (batch, c_capacity, heads_k, 128) bf16")
    ptr = lambda t: t.data_ptr() if t is not None else None
    with torch.cuda.device(k_cache.device):
        _lib.call("ifv2_decode_append", k_new.data_ptr(), v_new.data_ptr(), k_cache.data_ptr(),
                  v_cache.data_ptr(), ptr(kc_cache), ptr(kc2_cache), cache_seqlens.data_ptr(),
                  ptr(positions), ptr(n_comp), ptr(n_comp2), b, cap,
                  kc_cache.shape[1] if kc_cache is not None else 0,
                  kc2_cache.shape[1] if kc2_cache is not None else 0, hk, d, kernel_size, kernel_stride,
                  kernel2_size, kernel2_stride, _stream(k_cache.device))


def decode_select(score: torch.Tensor, positions: torch.Tensor, k: int, max_seqlen_k: int,
                  local_blocks: int, init_blocks: int, seqused_c: Optional[torch.Tensor] = None,
                  block_size: int = 64, stride: int = 16, return_topk: bool = False, dense_len: int = 0):
    """Block selection of a decode step in one launch: max-pool of the stage-1 scores of ONE query
    token per sequence (score: (Hk, B, n_comp) bf16/fp16, e.g. from infllmv2_attn_stage1), top-k
    and the uint64 block mask (B, Hk, 1, ceil(ceil(max_seqlen_k / block_size) / 64)) int64 that
    infllmv2_attn_with_kvcache takes as `block_mask`.  positions (B,) int32: position of the query
    token in its sequence; seqused_c (B,) int32: compressed keys per sequence (default: all
    columns).  Equal to max_pooling_1d_varlen -> infllmv2_topk -> topk_to_uint64.  With
    return_topk also returns topk_idx (B, Hk, 1, k) int32.  dense_len: sequences whose query position
    is below it get every block up to their own (dense attention for short sequences)."""
    assert score.dtype == torch.float16 or score.dtype == torch.bfloat16
    _require_cuda(score, "score")
    if score.dim() != 3:
        raise ValueError("score must be (num_heads_k, batch, n_comp)")
    score, row_stride = _row_view(score)
    hk, b, n_c = score.shape
    assert positions.dtype == torch.int32 and positions.numel() == b
    if seqused_c is not None:
        assert seqused_c.dtype == torch.int32 and seqused_c.numel() == b
        seqused_c = seqused_c.contiguous()
    n_blocks = (max_seqlen_k + block_size - 1) // block_size
    words = (n_blocks + 63) // 64
    mask = torch.empty(b, hk, 1, words, dtype=torch.int64, device=score.device)
    idx = torch.empty(b, hk, 1, k, dtype=torch.int32, device=score.device) if return_topk else None
    with torch.cuda.device(score.device):
        _lib.call("ifv2_decode_select", score.data_ptr(), int(score.dtype == torch.bfloat16), row_stride,
                  seqused_c.data_ptr() if seqused_c is not None else None, positions.contiguous().data_ptr(),
                  mask.data_ptr(), idx.data_ptr() if idx is not None else None, b, hk, n_c, n_blocks, words,
                  k, local_blocks, init_blocks, block_size, stride, int(dense_len), _stream(score.device))
    return (mask, idx) if return_topk else mask
