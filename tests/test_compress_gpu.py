"""GPU parity of the key-compression kernels (through the C ABI) with the oracle and with the
fixtures made from the reference's compress_tensor test helper."""
import os

import numpy as np
import pytest
import torch

import infllm_v2
import oracle
from helpers import cu, det_tensor

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def test_compress_golden(golden_dir):
    g = np.load(os.path.join(golden_dir, "compress.npz"))
    for key in [k for k in g.files if k.endswith("_lens")]:
        base = key[:-5]
        lens = [int(x) for x in g[key]]
        kernel, stride, seed, hk = (int(x) for x in g[base + "_cfg"])
        k = det_tensor((sum(lens), hk, 128), seed, device=DEV)
        kc, cu_c = infllm_v2.compress_keys(k, cu(lens, DEV), kernel, stride)
        assert cu_c.cpu().tolist() == [int(x) for x in g[base + "_cu_c"]], key
        assert kc.dtype == torch.bfloat16
        # inputs are multiples of 1/64: every partial sum is exact, so the result is bit-exact
        assert np.array_equal(kc.float().cpu().numpy(), g[base + "_out"]), key


@pytest.mark.parametrize("lens,hk,kernel,stride", [
    ([4096], 2, 32, 16), ([1000, 33, 31, 2048], 8, 32, 16), ([700, 128, 127], 2, 128, 64),
    ([50], 1, 24, 8),
])
def test_compress_random(lens, hk, kernel, stride):
    g = torch.Generator().manual_seed(sum(lens) + kernel)
    k = torch.randn(sum(lens), hk, 128, generator=g).to(torch.bfloat16)
    exp, cu_c = oracle.compress_keys(k, cu(lens).tolist(), kernel, stride)
    got, cu_got = infllm_v2.compress_keys(k.to(DEV), cu(lens, DEV), kernel, stride)
    assert cu_got.cpu().tolist() == cu_c and got.shape == exp.shape
    # fp32 sums in a different order than the oracle's: equal up to one bf16 step
    diff = (got.float().cpu() - exp.float()).abs()
    assert (diff <= exp.float().abs() * 2.0 ** -7 + 1e-6).all()
    assert (diff == 0).float().mean() > 0.98


def test_compress_single_sequence_and_empty():
    k = det_tensor((200, 2, 128), 5, device=DEV)
    kc, cu_c = infllm_v2.compress_keys(k)
    assert cu_c is None and kc.shape == (11, 2, 128)
    exp, _ = oracle.compress_keys(k.cpu(), [0, 200])
    assert torch.equal(kc.cpu(), exp)
    short = det_tensor((20, 2, 128), 6, device=DEV)
    kc, _ = infllm_v2.compress_keys(short)
    assert kc.shape == (0, 2, 128)
    kc, cu_c = infllm_v2.compress_keys(short, cu([5, 15], DEV))
    assert kc.shape == (0, 2, 128) and cu_c.cpu().tolist() == [0, 0, 0]
    with pytest.raises(ValueError):
        infllm_v2.compress_keys(short.float())


def test_compress_feeds_stage1():
    """compress_keys -> infllmv2_attn_stage1 equals the oracle fed with the oracle's compression."""
    lens = [300, 129]
    q = det_tensor((sum(lens), 32, 128), 11, 0.25, device=DEV)
    k = det_tensor((sum(lens), 2, 128), 12, device=DEV)
    kc, cu_c = infllm_v2.compress_keys(k, cu(lens, DEV))
    n_c = [int(x) for x in (cu_c[1:] - cu_c[:-1]).cpu()]
    score = infllm_v2.infllmv2_attn_stage1(q, kc, kc, cu(lens, DEV), cu_c, cu_c, max(lens), max(n_c),
                                           causal=True)
    kc_o, cu_o = oracle.compress_keys(k.cpu(), cu(lens).tolist())
    exp = oracle.stage1_scores(q.cpu(), kc_o, cu(lens).tolist(), cu_o, max(n_c), True)
    err = (score.float().cpu() - exp).abs()
    assert (err <= torch.maximum(torch.tensor(2e-2), exp.abs() * 2.0 ** -7)).all()


def test_compress_append_equals_recompute():
    """Appending tokens one at a time and updating the compressed cache in place gives the same
    compressed keys as compressing the final cache in one go."""
    b, cap, hk, steps = 3, 160, 2, 40
    kcache = det_tensor((b, cap, hk, 128), 21, device=DEV)
    start = torch.tensor([31, 40, 95], dtype=torch.int32, device=DEV)
    c_cap = (cap - 32) // 16 + 1
    kc_cache = torch.zeros(b, c_cap, hk, 128, dtype=torch.bfloat16, device=DEV)
    for i in range(b):                                   # the prefix present before decoding starts
        n0 = (int(start[i]) - 32) // 16 + 1 if int(start[i]) >= 32 else 0
        if n0:
            kc_cache[i, :n0] = infllm_v2.compress_keys(kcache[i, :int(start[i])].contiguous())[0]
    lens = start.clone()
    for _ in range(steps):
        lens += 1                                        # the new token is already in the cache
        infllm_v2.compress_keys_append(kcache, lens, kc_cache)
    for i in range(b):
        full, _ = oracle.compress_keys(kcache[i, :int(lens[i])].cpu(), [0, int(lens[i])])
        assert torch.equal(kc_cache[i, :full.shape[0]].cpu(), full)
        assert (kc_cache[i, full.shape[0]:] == 0).all()
