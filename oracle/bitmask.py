"""Bitmask pack / unpack / transpose oracles (NumPy, bit-exact).  Test infrastructure only.

Follows:
  * topk_to_uint64      csrc/topk_to_uint64.cuh:19-51   (NumPy twin: tests/test_topk_to_uint64.py:42-99)
  * blockmask_to_uint64 csrc/blockmask_to_uint64.cuh:28-50 (tests/test_blockmask.py:6-57)
  * uint64_to_bool      csrc/uint64_to_bool.cuh:24-42   (tests/test_uint64_to_bool.py:6-49)
  * transpose_blockmask infllm_v2/infllmv2_sparse_attention.py:343-350 (unpack -> transpose(1,2) -> pack)
"""
import numpy as np


def topk_to_uint64(topk_idx: np.ndarray, max_seqlen_k: int, block_size: int):
    """Rows of block indices (-1 = empty slot) -> rows of 64-bit words, bit (idx % 64) of word
    (idx // 64) set.  Returns (int64 array [..., words], k_blocks)."""
    topk_idx = np.asarray(topk_idx)
    assert topk_idx.dtype == np.int32
    k_blocks = (max_seqlen_k + block_size - 1) // block_size
    words = (k_blocks + 63) // 64
    lead = topk_idx.shape[:-1]
    flat = topk_idx.reshape(-1, topk_idx.shape[-1]).astype(np.int64)
    out = np.zeros((flat.shape[0], words), dtype=np.uint64)
    rows = np.repeat(np.arange(flat.shape[0]), flat.shape[1])
    idx = flat.reshape(-1)
    # the kernel tests each index against the word's range, so anything outside
    # [0, 64*words) is dropped, not only -1
    ok = (idx >= 0) & (idx < 64 * words)
    np.bitwise_or.at(out, (rows[ok], idx[ok] // 64),
                     np.uint64(1) << (idx[ok] % 64).astype(np.uint64))
    return out.view(np.int64).reshape(lead + (words,)), k_blocks


def blockmask_to_uint64(mask: np.ndarray):
    """Bool array [..., n] -> (int64 array [..., ceil(n/64)], n); element 64w+b is bit b of word w."""
    mask = np.asarray(mask).astype(bool)
    n = mask.shape[-1]
    words = (n + 63) // 64
    flat = mask.reshape(-1, n)
    padded = np.zeros((flat.shape[0], words * 64), dtype=bool)
    padded[:, :n] = flat
    bits = np.packbits(padded.reshape(-1, words, 8, 8), axis=-1, bitorder="little")
    out = np.ascontiguousarray(bits.reshape(-1, words, 8)).view("<u8").reshape(-1, words)
    return out.view(np.int64).reshape(mask.shape[:-1] + (words,)), n


def uint64_to_bool(words: np.ndarray, last_dim: int) -> np.ndarray:
    """Inverse of blockmask_to_uint64 restricted to the first `last_dim` bits of each row."""
    words = np.ascontiguousarray(np.asarray(words)).view(np.uint64)
    nw = words.shape[-1]
    by = words.reshape(-1, nw).astype("<u8").view(np.uint8).reshape(-1, nw * 8)
    bits = np.unpackbits(by, axis=-1, bitorder="little").astype(bool)
    if bits.shape[1] < last_dim:
        bits = np.pad(bits, ((0, 0), (0, last_dim - bits.shape[1])))
    return bits[:, :last_dim].reshape(words.shape[:-1] + (last_dim,))


def transpose_blockmask(fwd_words: np.ndarray, k_blocks: int) -> np.ndarray:
    """Row mask (Hk, T, ceil(k_blocks/64)) -> column mask (Hk, k_blocks, ceil(T/64)):
    out[h, blk, t // 64] bit (t % 64) = in[h, t, blk // 64] bit (blk % 64)."""
    b = uint64_to_bool(fwd_words, k_blocks)            # (Hk, T, k_blocks)
    bt = np.ascontiguousarray(np.swapaxes(b, 1, 2))    # (Hk, k_blocks, T)
    return blockmask_to_uint64(bt)[0]
