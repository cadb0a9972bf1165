"""GPU: bitmask kernels, bit-exact against the NumPy oracle and the golden vectors."""
import os

import numpy as np
import pytest
import torch

import oracle
import infllm_v2

pytestmark = pytest.mark.gpu
DEV = "cuda"


def test_topk_to_uint64_golden(golden_dir):
    g = np.load(os.path.join(golden_dir, "bitmask.npz"))
    for key in [k for k in g.files if k.endswith("_idx")]:
        base = key[:-4]
        got, kb = infllm_v2.topk_to_uint64(torch.from_numpy(g[key]).to(DEV), int(g[base + "_maxk"]), 64)
        assert got.dtype == torch.int64
        assert np.array_equal(got.cpu().numpy(), g[base + "_out"]), key


@pytest.mark.parametrize("shape,max_k", [((2, 300, 64), 32768), ((8, 257, 64), 131072),
                                         ((2, 3, 5, 7), 64 * 130), ((1, 1, 1), 64), ((2, 33, 16), 4096)])
def test_topk_to_uint64_random(shape, max_k):
    rng = np.random.default_rng(hash(shape) % 2**32)
    kb = (max_k + 63) // 64
    idx = rng.integers(-1, kb, size=shape).astype(np.int32)
    exp, _ = oracle.topk_to_uint64(idx, max_k, 64)
    got, k_blocks = infllm_v2.topk_to_uint64(torch.from_numpy(idx).to(DEV), max_k, 64)
    assert k_blocks == kb and np.array_equal(got.cpu().numpy(), exp)


@pytest.mark.parametrize("shape", [(3, 63), (2, 2, 64), (4, 65), (2, 3, 200), (5, 1), (1, 1024),
                                   (7, 128), (3, 4, 4096), (2, 1000), (16, 16), (9, 20)])
def test_blockmask_roundtrip(shape):
    rng = np.random.default_rng(sum(shape))
    m = rng.random(shape) < 0.4
    exp, n = oracle.blockmask_to_uint64(m)
    got, last = infllm_v2.blockmask_to_uint64(torch.from_numpy(m).to(DEV))
    assert last == shape[-1] and np.array_equal(got.cpu().numpy(), exp)
    back = infllm_v2.uint64_to_bool(got, last)
    assert back.dtype == torch.bool and np.array_equal(back.cpu().numpy(), m)


def test_blockmask_golden(golden_dir):
    g = np.load(os.path.join(golden_dir, "bitmask.npz"))
    for key in [k for k in g.files if k.endswith("_mask")]:
        got, _ = infllm_v2.blockmask_to_uint64(torch.from_numpy(g[key]).to(DEV))
        assert np.array_equal(got.cpu().numpy(), g[key[:-5] + "_out"]), key


def test_blockmask_large_idempotent():
    # size-independent property at a large size: pack(unpack(pack(x))) == pack(x)
    g = torch.Generator(device=DEV).manual_seed(0)
    m = torch.rand(64, 1 << 20, device=DEV, generator=g) < 0.5
    w, n = infllm_v2.blockmask_to_uint64(m)
    b = infllm_v2.uint64_to_bool(w, n)
    assert torch.equal(b, m)
    assert int(sum(bin(int(x) & (2**64 - 1)).count("1") for x in w[0, :8].cpu())) == int(m[0, :512].sum())


@pytest.mark.parametrize("hk,t,kb", [(2, 130, 70), (1, 64, 64), (3, 1, 129), (2, 1000, 384), (2, 513, 65)])
def test_transpose_blockmask(hk, t, kb):
    rng = np.random.default_rng(t + kb)
    m = rng.random((hk, t, kb)) < 0.3
    fwd, _ = oracle.blockmask_to_uint64(m)
    exp = oracle.transpose_blockmask(fwd, kb)
    got = infllm_v2.transpose_blockmask(torch.from_numpy(fwd).to(DEV), kb)
    assert np.array_equal(got.cpu().numpy(), exp)
    # and it equals the reference's unpack -> transpose -> pack sequence done with our kernels
    b = infllm_v2.uint64_to_bool(torch.from_numpy(fwd).to(DEV), kb).transpose(1, 2).contiguous()
    ref_path, _ = infllm_v2.blockmask_to_uint64(b)
    assert torch.equal(ref_path, got)
