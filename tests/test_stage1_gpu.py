"""GPU: stage-1 scorer against the fp32 oracle and the golden vectors.
Tolerance: |got - ref| <= 2e-2, or within 2^-7 relative where a score is large (the output is
bf16 and a row's 16 units of probability can sit on a handful of keys: one bf16 step at 8..16
is 2^-4, already above 2e-2)."""
import os

import numpy as np
import pytest
import torch

import oracle
import infllm_v2
from helpers import det_tensor, cu
from inputs import det_array

pytestmark = pytest.mark.gpu
DEV = "cuda"
MAX_ABS, REL = 2e-2, 2.0 ** -7


def _within(got, ref):
    got, ref = torch.as_tensor(got).float(), torch.as_tensor(ref).float()
    diff = (got - ref).abs()
    ok = (diff <= MAX_ABS) | (diff <= REL * ref.abs())
    return bool(ok.all()), diff.max().item()


def _run(q, kc, cu_q, cu_k, max_q, max_k, causal):
    s = infllm_v2.infllmv2_attn_stage1(q.to(DEV), kc.to(DEV), kc.to(DEV), cu_q.to(DEV), cu_k.to(DEV),
                                       cu_k.to(DEV), max_q, max_k, causal=causal)
    infllm_v2.check_device_status()
    assert s.dtype == torch.bfloat16 and s.shape == (kc.shape[1], q.shape[0], max_k)
    return s.float().cpu()


def test_stage1_golden(golden_dir):
    g = np.load(os.path.join(golden_dir, "stage1.npz"))
    for key in [k for k in g.files if k.endswith("_shape")]:
        base = key[:-6]
        lq, lc, seed = (int(x) for x in g[key][:3])
        if len(g[key]) == 4:                 # "compressed LSE" case: row sums over coarser keys
            lcv = int(g[key][3])
            q = torch.from_numpy(det_array((lq, 32, 128), seed, 0.5)).to(torch.bfloat16)
            k = torch.from_numpy(det_array((lc, 2, 128), seed + 1000)).to(torch.bfloat16)
            kv = torch.from_numpy(det_array((lcv, 2, 128), seed + 2000)).to(torch.bfloat16)
            got = infllm_v2.infllmv2_attn_stage1(q.to(DEV), k.to(DEV), kv.to(DEV), cu([lq], DEV),
                                                 cu([lc], DEV), cu([lcv], DEV), lq, lc,
                                                 causal=bool(g[base + "_causal"])).float().cpu()
            infllm_v2.check_device_status()
            ok, err = _within(got, g[base + "_out"])
            assert ok, (base, err)
            continue
        q = torch.from_numpy(det_array((lq, 32, 128), seed)).to(torch.bfloat16)
        k = torch.from_numpy(det_array((lc, 2, 128), seed + 1000)).to(torch.bfloat16)
        got = _run(q, k, cu([lq]), cu([lc]), lq, lc, bool(g[base + "_causal"]))
        ok, err = _within(got, g[base + "_out"])
        assert ok, (base, err)
        assert not np.isnan(got.numpy()).any()


@pytest.mark.parametrize("lens_q,causal", [([4096], True), ([700, 33, 1500], True), ([513], False),
                                           ([40], True), ([4096 + 64], True)])
def test_stage1_vs_oracle(lens_q, causal):
    hq, hk, d = 32, 2, 128
    seed = sum(lens_q)
    q = det_tensor((sum(lens_q), hq, d), seed, 0.5)
    k = det_tensor((sum(lens_q), hk, d), seed + 1, 0.5)
    kc, cu_c = oracle.compress_keys(k, cu(lens_q))
    max_k = int(np.diff(cu_c).max())
    if max_k == 0:
        pytest.skip("no compressed key")
    cu_c_t = torch.tensor(cu_c, dtype=torch.int32)
    got = _run(q, kc, cu(lens_q), cu_c_t, max(lens_q), max_k, causal)
    ref = oracle.stage1_scores(q, kc, cu(lens_q), cu_c_t, max_k, causal)
    ok, err = _within(got, ref)
    assert ok, err
    rows = ref.sum(-1)
    assert ((got.sum(-1) - rows).abs() < 0.25).all()          # visible rows sum to 16, others to 0


def test_stage1_query_chunk_bottom_right_alignment():
    # a query chunk shorter than the span of the keys (context-parallel prefix scoring)
    hq, hk, d = 32, 2, 128
    full = 1024
    q = det_tensor((full, hq, d), 31, 0.5)
    k = det_tensor((full, hk, d), 32, 0.5)
    kc, cu_c = oracle.compress_keys(k, cu([full]))
    whole = _run(q, kc, cu([full]), torch.tensor(cu_c, dtype=torch.int32), full, cu_c[-1], True)
    tail = _run(q[512:], kc, cu([512]), torch.tensor(cu_c, dtype=torch.int32), 512, cu_c[-1], True)
    assert (whole[:, 512:] - tail).abs().max() <= 1e-2


@pytest.mark.parametrize("lens_q,cache,local,init", [([4096], 0, 2, 1), ([700, 33, 1500], 0, 32, 1),
                                                     ([513], 0, 1, 0), ([40], 0, 2, 1),
                                                     ([2048 + 64], 0, 32, 1)])
def test_fused_block_scores_equal_pool_of_scores(lens_q, cache, local, init):
    """The fused stage-1 + max-pool kernel against the two separate kernels: bit-exact."""
    hq, hk, d = 32, 2, 128
    seed = sum(lens_q) + 5
    q = det_tensor((sum(lens_q), hq, d), seed, 0.5).to(DEV)
    k = det_tensor((sum(lens_q), hk, d), seed + 1, 0.5)
    kc, cu_c = oracle.compress_keys(k, cu(lens_q))
    max_k = int(np.diff(cu_c).max())
    cu_q, cu_ct = cu(lens_q).to(DEV), torch.tensor(cu_c, dtype=torch.int32, device=DEV)
    kc = kc.to(DEV)
    pooled, scores = infllm_v2.infllmv2_stage1_block_scores(
        q, kc, cu_q, cu_ct, max(lens_q), max_k, local, init, cache_len=cache, return_scores=True)
    infllm_v2.check_device_status()
    plain = infllm_v2.infllmv2_attn_stage1(q, kc, kc, cu_q, cu_ct, cu_ct, max(lens_q), max_k, causal=True)
    assert torch.equal(scores, plain)
    if len(lens_q) == 1:
        ref = infllm_v2.max_pooling_1d(plain, cache, local, init)
    else:
        ref = infllm_v2.max_pooling_1d_varlen(plain, cu_q, cu_ct, torch.zeros(len(lens_q), dtype=torch.int32, device=DEV),
                                              max(lens_q), max_k, local, init)
    assert pooled.shape == ref.shape
    assert torch.equal(pooled, ref)
    only = infllm_v2.infllmv2_stage1_block_scores(q, kc, cu_q, cu_ct, max(lens_q), max_k, local, init,
                                                  cache_len=cache)
    assert torch.equal(only, ref)


def test_fused_block_scores_query_chunk_with_cache_len():
    hq, hk, d, full = 32, 2, 128, 2048
    q = det_tensor((full, hq, d), 41, 0.5).to(DEV)
    k = det_tensor((full, hk, d), 42, 0.5)
    kc, cu_c = oracle.compress_keys(k, cu([full]))
    kc = kc.to(DEV)
    cu_ct = torch.tensor(cu_c, dtype=torch.int32, device=DEV)
    start = 1024
    got = infllm_v2.infllmv2_stage1_block_scores(q[start:], kc, cu([full - start]).to(DEV), cu_ct, full - start,
                                                 cu_c[-1], 2, 1, cache_len=start)
    plain = infllm_v2.infllmv2_attn_stage1(q[start:], kc, kc, cu([full - start]).to(DEV), cu_ct, cu_ct,
                                           full - start, cu_c[-1], causal=True)
    assert torch.equal(got, infllm_v2.max_pooling_1d(plain, start, 2, 1))


@pytest.mark.parametrize("lens,causal", [([1000, 130, 64, 700], True), ([2048], True), ([300, 500], False)])
def test_stage1_compressed_lse_vs_oracle(lens, causal):
    """Row sums over a coarser compression of the same keys (kernel 128 / stride 64), packed
    ragged sequences including ones with no coarse key at all; scores and fused block scores."""
    hq, hk = 32, 2
    seed = sum(lens) + 5
    q = det_tensor((sum(lens), hq, 128), seed, 0.5)
    k = det_tensor((sum(lens), hk, 128), seed + 1, 0.5)
    kc, cu_c = oracle.compress_keys(k, cu(lens), 32, 16)
    kv, cu_v = oracle.compress_keys(k, cu(lens), 128, 64)
    max_k = int(np.diff(cu_c).max())
    exp = oracle.stage1_scores(q, kc, cu(lens).tolist(), cu_c, max_k, causal, lse_keys=kv, cu_seqlens_v=cu_v)
    cq = cu(lens, DEV)
    ck = torch.tensor(cu_c, dtype=torch.int32, device=DEV)
    cv = torch.tensor(cu_v, dtype=torch.int32, device=DEV)
    got = infllm_v2.infllmv2_attn_stage1(q.to(DEV), kc.to(DEV), kv.to(DEV), cq, ck, cv, max(lens), max_k,
                                         causal=causal)
    infllm_v2.check_device_status()
    ok, err = _within(got.float().cpu(), exp)
    assert ok, err
    if causal:
        pooled = infllm_v2.infllmv2_stage1_block_scores(q.to(DEV), kc.to(DEV), cq, ck, max(lens), max_k, 2, 1,
                                                        lse_keys=kv.to(DEV), cu_seqlens_v=cv)
        ref = infllm_v2.max_pooling_1d_varlen(got, cq, ck, torch.zeros(len(lens), dtype=torch.int32, device=DEV),
                                              max(lens), max_k, 2, 1)
        assert torch.equal(pooled, ref)


def test_stage1_compressed_lse_without_any_coarse_key():
    """Sequences all shorter than the coarse window: the row-sum tensor is empty (its pointer is
    null), cu_seqlens_v is all zeros and every score is 0, as in the oracle."""
    lens, hq, hk = [100, 40, 127], 32, 2
    q = det_tensor((sum(lens), hq, 128), 3, 0.5)
    k = det_tensor((sum(lens), hk, 128), 4, 0.5)
    kc, cu_c = oracle.compress_keys(k, cu(lens), 32, 16)
    kv, cu_v = oracle.compress_keys(k, cu(lens), 128, 64)
    assert kv.shape[0] == 0 and not any(cu_v)
    max_k = int(np.diff(cu_c).max())
    exp = oracle.stage1_scores(q, kc, cu(lens).tolist(), cu_c, max_k, True, lse_keys=kv, cu_seqlens_v=cu_v)
    assert not exp.any()
    got = infllm_v2.infllmv2_attn_stage1(q.to(DEV), kc.to(DEV), kv.to(DEV), cu(lens, DEV),
                                         torch.tensor(cu_c, dtype=torch.int32, device=DEV),
                                         torch.tensor(cu_v, dtype=torch.int32, device=DEV), max(lens), max_k,
                                         causal=True)
    infllm_v2.check_device_status()
    assert got.shape == exp.shape and not got.float().cpu().any()


@pytest.mark.parametrize("lens_c,hk,causal", [([700, 1, 512, 513, 33], 2, False), ([2047, 16], 8, False),
                                              ([40, 0, 1025], 2, False),
                                              ([300, 64, 5], 2, True)])
def test_stage1_decode_path(lens_c, hk, causal):
    """One query token per sequence takes the chunk-parallel kernel pair: same scores as the
    oracle, zeros past every sequence's keys, and as the general kernel (forced by giving one
    sequence two tokens, which leaves the rows of the single-token sequences unchanged)."""
    bsz = len(lens_c)
    seed = sum(lens_c) + hk
    q = det_tensor((bsz, hk * 16, 128), seed, 0.5)
    kc = det_tensor((sum(lens_c), hk, 128), seed + 1, 0.5)
    cu_q, cu_c = cu([1] * bsz), cu(lens_c)
    max_c = max(lens_c)
    exp = oracle.stage1_scores(q, kc, cu_q.tolist(), cu_c.tolist(), max_c, causal)
    got = infllm_v2.infllmv2_attn_stage1(q.to(DEV), kc.to(DEV), kc.to(DEV), cu_q.to(DEV), cu_c.to(DEV),
                                         cu_c.to(DEV), 1, max_c, causal=causal)
    infllm_v2.check_device_status()
    assert got.shape == (hk, bsz, max_c)
    ok, err = _within(got.float().cpu(), exp)
    assert ok, err
    for b, n in enumerate(lens_c):                       # nothing but zeros past a sequence's keys
        assert (got[:, b, n:] == 0).all()
    if not causal:
        # the general kernel on the same rows: append a second token to the last sequence
        q2 = torch.cat([q, q[-1:]], 0)
        cu_q2 = cu([1] * (bsz - 1) + [2])
        ref = infllm_v2.infllmv2_attn_stage1(q2.to(DEV), kc.to(DEV), kc.to(DEV), cu_q2.to(DEV), cu_c.to(DEV),
                                             cu_c.to(DEV), 2, max_c, causal=False)
        diff = (got.float() - ref[:, :bsz].float()).abs()
        assert (diff <= torch.maximum(torch.tensor(2e-2, device=DEV), ref[:, :bsz].float().abs() * 2.0 ** -7)).all()
