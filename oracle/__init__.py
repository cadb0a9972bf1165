"""CPU oracle for the InfLLM-V2 sparse-attention path.  TEST INFRASTRUCTURE ONLY.

This package restates, in plain NumPy / fp32 PyTorch on the CPU, the algorithm of the
reference's hot path (stage-1 scorer -> 64-token max-pool -> top-k -> uint64 bitmask ->
stage-2 block-sparse attention forward/backward -> KV-cache decode).  Each function cites
the reference file:line it follows.

It is the checker, never the product: only the test-suite, the smoke entry and the
benchmark's CPU-baseline leg may import it.  The library proper fails loudly when its CUDA
extension is missing and never routes through this package.

Parity pin: the restatements are checked against the reference's own pure-Python oracle
functions (imported from the reference's tests/ directory when it is present) by
tests/golden/make_golden.py, which also writes the committed fixtures under tests/golden/.
The reference has no Python twin of its top-k; that function is pinned by a thread-for-thread
simulation of the reference's bitonic top-k kernel (csrc/topk.cuh:6-117, oracle/topk.py).
"""
from .bitmask import (topk_to_uint64, blockmask_to_uint64, uint64_to_bool,
                      transpose_blockmask)
from .pooling import max_pooling_1d, max_pooling_1d_varlen
from .topk import topk_select
from .stage1 import stage1_scores, stage1_visible_limit, compress_keys
from .attention import (expand_topk_mask, sparse_attention_fwd, sparse_attention_fwd_bwd,
                        kvcache_decode, apply_rotary, apply_rotary_literal)

__all__ = [
    "topk_to_uint64", "blockmask_to_uint64", "uint64_to_bool", "transpose_blockmask",
    "max_pooling_1d", "max_pooling_1d_varlen", "topk_select",
    "stage1_scores", "stage1_visible_limit", "compress_keys",
    "expand_topk_mask", "sparse_attention_fwd", "sparse_attention_fwd_bwd", "kvcache_decode", "apply_rotary", "apply_rotary_literal",
]
