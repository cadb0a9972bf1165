"""Deterministic, platform-independent test inputs shared by the fixture generator and the tests.

Values are small multiples of 1/64 in [-2, 2), so they are exact in bf16, fp16 and fp32 and a
fixture only has to store the expected OUTPUT: the input is recomputed from (shape, seed).
"""
import numpy as np


def det_array(shape, seed: int, scale: float = 1.0) -> np.ndarray:
    """float32 array of the given shape from an integer hash of (flat index, seed)."""
    n = int(np.prod(shape))
    i = np.arange(n, dtype=np.uint64) + np.uint64(seed) * np.uint64(0x9E3779B97F4A7C15 & 0xFFFFFFFF)
    x = (i ^ (i >> np.uint64(15))) * np.uint64(0x2C1B3C6D) & np.uint64(0xFFFFFFFF)
    x = (x ^ (x >> np.uint64(12))) * np.uint64(0x297A2D39) & np.uint64(0xFFFFFFFF)
    x = x ^ (x >> np.uint64(15))
    k = (x & np.uint64(0xFF)).astype(np.int64) - 128
    return (k.astype(np.float32) / 64.0 * scale).reshape(shape)


def det_perm_rows(rows: int, n: int, k: int, seed: int) -> np.ndarray:
    """`rows` sorted k-subsets of range(n) as int32 (rows, k), from the same hash."""
    keys = det_array((rows, n), seed) + np.arange(n, dtype=np.float32)[None, :] * 1e-4
    idx = np.argsort(keys, axis=1, kind="stable")[:, :k]
    return np.sort(idx, axis=1).astype(np.int32)
