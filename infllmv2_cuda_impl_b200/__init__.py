"""B200-native (sm_100a) InfLLM-V2 two-stage sparse attention behind the reference's `infllm_v2`
Python API.  Every operator runs hand-written CUDA through the C ABI of
include/infllmv2_b200.h; there is no CPU or library fallback."""
__version__ = "0.1.0"

from .ops import (blockmask_to_uint64, topk_to_uint64, uint64_to_bool, max_pooling_1d,
                  max_pooling_1d_varlen, infllmv2_topk, infllmv2_topk_mask, transpose_blockmask, compress_keys,
                  compress_keys_append, compressed_lengths, cache_fill, decode_append, decode_select)
from .attention import (infllmv2_attn_varlen_func, infllmv2_attn_stage1,
                        infllmv2_attn_with_kvcache, infllmv2_stage1_block_scores,
                        infllmv2_stage1_decode_select,
                        check_device_status)
from .sparse_attention import SparseConfig, DecodeCache, SparseAttention

__all__ = [
    "blockmask_to_uint64", "topk_to_uint64", "uint64_to_bool", "max_pooling_1d",
    "max_pooling_1d_varlen", "infllmv2_attn_varlen_func", "infllmv2_attn_stage1",
    "infllmv2_attn_with_kvcache", "infllmv2_topk", "infllmv2_topk_mask", "infllmv2_stage1_block_scores", "infllmv2_stage1_decode_select", "transpose_blockmask", "check_device_status",
    "compress_keys", "compress_keys_append", "compressed_lengths", "cache_fill", "decode_append", "decode_select",
    "SparseConfig", "DecodeCache", "SparseAttention",
]
