"""CPU: the C-ABI library loads without a GPU, exports every symbol the header declares, and
rejects bad arguments before touching the device."""
import ctypes

import pytest

from infllmv2_cuda_impl_b200 import _lib


def test_exports_every_declared_symbol(lib):
    names = _lib.declared_symbols()
    assert len(names) >= 15
    for name in names:
        assert hasattr(lib, name), f"{name} is declared in include/infllmv2_b200.h but not exported"
    assert set(_lib.SIGNATURES) | set(_lib._INT64_RETURNS) | {"ifv2_last_error", "ifv2_version"} == set(names)


def test_version_and_error_text(lib):
    assert lib.ifv2_version() >= 100
    rc = lib.ifv2_topk_to_uint64(None, None, -1, 4, 64, 1, None)
    assert rc == -1
    assert b"negative" in lib.ifv2_last_error()


@pytest.mark.parametrize("name,args,code", [
    ("ifv2_topk_to_uint64", (None, None, 4, 4, 64, 3, None), -1),            # words != ceil(k_blocks/64)
    ("ifv2_blockmask_to_uint64", (None, None, 4, 65, 1, None), -1),          # null pointers
    ("ifv2_uint64_to_bool", (8, 8, 4, 200, 2, None), -1),                    # last_dim > 64*words
    ("ifv2_max_pooling_1d", (8, 8, 1, 2, 4, 16, 8, 1, 0, 5, 4, 1, 64, 1, 1, None), -1),  # stride < k_len
    ("ifv2_topk_select", (8, 8, 1, 2, 4, 9000, 9000, 64, None, None, 1, 0, 64, None), -3),  # too many blocks
    ("ifv2_stage1_scores", (8, 8, None, 8, 8, 8, None, 0, None, None, 1, 4, 4, 32, 2, 64, 4, 4, 8, 0.1, 1, 8, None), -2),  # d != 128
    ("ifv2_stage1_scores", (8, 8, None, 8, 8, 8, None, 0, None, None, 1, 4, 4, 24, 2, 128, 4, 4, 8, 0.1, 1, 8, None), -2),  # group != 16
    ("ifv2_sparse_attn_fwd", (8, 8, 8, 8, 8, None, 0, 8, 8, 1, 4, 4, 32, 2, 96, 4, 4, 0.1, 1, 8, None), -2),
    ("ifv2_sparse_attn_fwd", (8, 8, 8, 8, 8, 8, 999, 8, 8, 1, 4, 4, 32, 2, 128, 4, 4, 0.1, 1, 8, None), -1),
])
def test_argument_errors(lib, name, args, code):
    assert getattr(lib, name)(*args) == code
    assert len(lib.ifv2_last_error()) > 0


def test_empty_inputs_are_noops(lib):
    assert lib.ifv2_topk_to_uint64(None, None, 0, 4, 64, 1, None) == 0
    assert lib.ifv2_uint64_to_bool(None, None, 0, 64, 1, None) == 0
    assert lib.ifv2_transpose_blockmask(None, None, 2, 0, 5, None) == 0


def test_python_wrappers_refuse_cpu_tensors():
    import torch
    import infllm_v2
    with pytest.raises(RuntimeError):
        infllm_v2.blockmask_to_uint64(torch.zeros(2, 64, dtype=torch.bool))
    q = torch.zeros(4, 32, 128, dtype=torch.bfloat16)
    k = torch.zeros(4, 2, 128, dtype=torch.bfloat16)
    c = torch.tensor([0, 4], dtype=torch.int32)
    with pytest.raises(RuntimeError):
        infllm_v2.infllmv2_attn_varlen_func(q, k, k, c, c, 4, 4, causal=True)
    with pytest.raises(RuntimeError):
        infllm_v2.infllmv2_attn_stage1(q, k, k, c, c, c, 4, 4, causal=True)
