"""GPU: parity at the sizes the benchmark is quoted on (selection micro-benchmark at 32768 tokens,
varlen training forward + backward at 65536 tokens in four packed sequences, the 131072-token
prefill with 128 query / 8 KV heads, and decode at batch 64 with 32k-128k caches), inputs built
as the benchmark builds them.

Integer results (block scores, top-k lists, masks) are compared bit for bit with the CPU oracle on
the GPU's own scores -- all rows where the CPU finishes in seconds, else row chunks spread over
the sequence.  Floating-point results are compared with plain fp32 PyTorch restatements running on
the GPU (tests/gpu_oracle.py): every row for the training configuration, sampled tokens (sequence
ends, block borders, the last octet) elsewhere.  Tolerances: stage-1 scores |d| <= 2e-2 or
<= 2^-7 relative; stage-2 outputs and gradients max-abs <= 2e-2 (x the gradient's own scale) and
mean-rel <= 1e-2.
"""
import math

import numpy as np
import pytest
import torch

import oracle
import gpu_oracle
import infllm_v2
from infllmv2_cuda_impl_b200 import attention
from helpers import err_stats

pytestmark = pytest.mark.gpu
DEV = "cuda"
D, BLOCK, TOPK, INIT, LOCAL = 128, 64, 64, 1, 32
MAX_ABS, MEAN_REL = 2e-2, 1e-2


def _randn(shape, gen, scale):
    return (torch.randn(*shape, device=DEV, generator=gen) * scale).to(torch.bfloat16)


def _stage1_close(got, ref):
    diff = (got.float() - ref).abs()
    return bool(((diff <= 2e-2) | (diff <= 2.0 ** -7 * ref.abs())).all()), diff.max().item()


def _check_selection_chunk(q, kc, seqlen, rows, block_scores, topk_idx, mask):
    """Rows [rows.start, rows.stop) of one sequence: scores of that query chunk from the unfused
    scorer (bottom-right aligned), then pool / top-k / pack on the CPU oracle, bit for bit against
    what the fused pipeline produced for the whole sequence."""
    n_comp = kc.shape[0]
    lq = rows.stop - rows.start
    cu_q = torch.tensor([0, lq], dtype=torch.int32, device=DEV)
    cu_c = torch.tensor([0, n_comp], dtype=torch.int32, device=DEV)
    # the chunk is scored against the compressed keys of its prefix, as a sharded prefill does
    n_pre = (rows.stop - 32) // 16 + 1
    cu_p = torch.tensor([0, n_pre], dtype=torch.int32, device=DEV)
    score = infllm_v2.infllmv2_attn_stage1(q[rows], kc[:n_pre], kc[:n_pre], cu_q, cu_p, cu_p, lq, n_pre,
                                           causal=True)
    pooled_ref = oracle.max_pooling_1d(score.cpu(), rows.start, LOCAL, INIT)
    n_blk = block_scores.shape[-1]
    got = block_scores[:, rows].cpu()
    # blocks past the chunk's own (future blocks) exist in the full-sequence output only
    assert torch.equal(got[..., :pooled_ref.shape[-1]], pooled_ref)
    qb = (torch.arange(lq) + rows.start) // BLOCK
    idx_ref = oracle.topk_select(got, TOPK, qb)
    assert torch.equal(topk_idx[:, rows].cpu(), idx_ref)
    words_ref, _ = oracle.topk_to_uint64(idx_ref.numpy(), seqlen, BLOCK)
    assert np.array_equal(mask[:, rows].cpu().numpy(), words_ref)
    return n_blk


def test_selection_at_32768_tokens():
    """Scores of sampled tokens against fp32; pool, top-64 (1 init + 32 local forced) and the
    packed mask bit for bit on ALL rows; the fused stage-1 + pool kernel equals the two-kernel path."""
    L, hk = 32768, 2
    g = torch.Generator(device=DEV).manual_seed(0)
    s = 1.0 / math.sqrt(D)
    q = _randn((L, hk * 16, D), g, s)
    k = _randn((L, hk, D), g, s)
    kc = infllm_v2.compress_keys(k)[0]
    n_comp = kc.shape[0]
    assert n_comp == 2047
    cu_q = torch.tensor([0, L], dtype=torch.int32, device=DEV)
    cu_c = torch.tensor([0, n_comp], dtype=torch.int32, device=DEV)
    score = infllm_v2.infllmv2_attn_stage1(q, kc, kc, cu_q, cu_c, cu_c, L, n_comp, causal=True)
    toks = torch.tensor(sorted(set([0, 1, 30, 31, 32, 47, 48, 63, 64, 65, 4095, 4096, 16383, 16384, 20000,
                                    32704, 32760, 32766, 32767] + list(range(1000, 32768, 1500)))), device=DEV)
    ref = gpu_oracle.stage1_rows(q[toks], kc, toks, L)
    ok, worst = _stage1_close(score[:, toks], ref)
    assert ok, worst
    pooled = infllm_v2.max_pooling_1d(score, 0, LOCAL, INIT, BLOCK, 16)
    assert torch.equal(pooled.cpu(), oracle.max_pooling_1d(score.cpu(), 0, LOCAL, INIT))
    fused = infllm_v2.infllmv2_stage1_block_scores(q, kc, cu_q, cu_c, L, n_comp, LOCAL, INIT, causal=True)
    assert torch.equal(fused, pooled)
    idx = infllm_v2.infllmv2_topk(pooled, TOPK)
    idx_ref = oracle.topk_select(pooled.cpu(), TOPK, torch.arange(L) // BLOCK)
    assert torch.equal(idx.cpu(), idx_ref)
    words, kb = infllm_v2.topk_to_uint64(idx, L, BLOCK)
    words_ref, kb_ref = oracle.topk_to_uint64(idx_ref.numpy(), L, BLOCK)
    assert kb == kb_ref and np.array_equal(words.cpu().numpy(), words_ref)
    fused_mask, _, col = infllm_v2.infllmv2_topk_mask(pooled, TOPK, L, return_col_mask=True)
    assert torch.equal(fused_mask, words)
    assert np.array_equal(col.cpu().numpy(), oracle.transpose_blockmask(words_ref, kb_ref))
    infllm_v2.check_device_status()


def test_varlen_training_at_65536_tokens():
    """Forward and backward of the four packed sequences {8192, 16384, 24576, 16384}, 6-word masks:
    out, dQ, dK and dV of EVERY row against fp32."""
    from bench import config3_topk
    lens, hk = [8192, 16384, 24576, 16384], 2
    T = sum(lens)
    g = torch.Generator(device=DEV).manual_seed(0)
    s = 1.0 / math.sqrt(D)
    q, k, v = _randn((T, hk * 16, D), g, s), _randn((T, hk, D), g, s), _randn((T, hk, D), g, s)
    do = _randn((T, hk * 16, D), g, 1.0)
    cu = torch.tensor([0] + list(np.cumsum(lens)), dtype=torch.int32, device=DEV)
    idx = config3_topk(lens, hk, TOPK, seed=1).to(DEV)
    max_l = max(lens)
    o, lse, mask = attention._infllmv2_attn_varlen_forward(q, k, v, cu, cu, max_l, max_l, D ** -0.5, True, idx)
    assert mask.shape[-1] == 6
    dq, dk, dv = attention._infllmv2_attn_varlen_backward(do, q, k, v, o, lse, cu, cu, max_l, max_l,
                                                          D ** -0.5, True, mask)
    infllm_v2.check_device_status()
    # no atomics and a fixed order of accumulation: a second run gives the same bits
    again = attention._infllmv2_attn_varlen_backward(do, q, k, v, o, lse, cu, cu, max_l, max_l,
                                                     D ** -0.5, True, mask)
    assert all(torch.equal(a, b) for a, b in zip((dq, dk, dv), again[:3]))
    r_o, r_dq, r_dk, r_dv = gpu_oracle.blockshared_fwd_bwd(q, k, v, do, lens, idx)
    for name, got, ref in (("out", o, r_o), ("dq", dq, r_dq), ("dk", dk, r_dk), ("dv", dv, r_dv)):
        assert not torch.isnan(got.float()).any(), name
        mx, mr = err_stats(got, ref)
        assert mx <= MAX_ABS * max(1.0, ref.abs().max().item()) and mr <= MEAN_REL, (name, mx, mr)
    # rows at the borders of the packed sequences, checked on their own
    borders = torch.tensor([0, 8191, 8192, 24575, 24576, 49151, 49152, 65535], device=DEV)
    mx, mr = err_stats(o[borders], r_o[borders])
    assert mx <= MAX_ABS and mr <= MEAN_REL, (mx, mr)
    # key blocks: first, diagonal-heavy and last of every sequence
    start = 0
    for length in lens:
        for blk in (0, length // 128, length // 64 - 1):
            rows = slice(start + blk * 64, start + blk * 64 + 64)
            for name, got, ref in (("dk", dk, r_dk), ("dv", dv, r_dv)):
                mx, mr = err_stats(got[rows], ref[rows])
                assert mx <= MAX_ABS * max(1.0, ref[rows].abs().max().item()) and mr <= 2 * MEAN_REL, (name, blk, mx, mr)
        start += length


def test_prefill_at_131072_tokens_128q_8kv():
    """The benchmark's own step (fused stage 1 + pool, top-64, 32-word mask, stage-2 forward) on
    all 8 KV heads: stage-1 scores and attention outputs of sampled tokens (incl. the last octet)
    against fp32, selection bit for bit on row chunks at the start, middle and end."""
    L, hk = 131072, 8
    g = torch.Generator(device=DEV).manual_seed(0)
    s = 1.0 / math.sqrt(D)
    q, k, v = _randn((L, hk * 16, D), g, s), _randn((L, hk, D), g, s), _randn((L, hk, D), g, s)
    kc = infllm_v2.compress_keys(k)[0]
    n_comp = kc.shape[0]
    assert n_comp == 8191
    cu_q = torch.tensor([0, L], dtype=torch.int32, device=DEV)
    cu_c = torch.tensor([0, n_comp], dtype=torch.int32, device=DEV)
    pooled = infllm_v2.infllmv2_stage1_block_scores(q, kc, cu_q, cu_c, L, n_comp, LOCAL, INIT, causal=True)
    idx = infllm_v2.infllmv2_topk(pooled, TOPK)
    mask, _ = infllm_v2.topk_to_uint64(idx, L, BLOCK)
    assert mask.shape == (hk, L, 32)
    fused_mask, _ = infllm_v2.infllmv2_topk_mask(pooled, TOPK, L)      # top-k and pack in one kernel
    assert torch.equal(fused_mask, mask)
    del fused_mask
    out, lse, _ = infllm_v2.infllmv2_attn_varlen_func(q, k, v, cu_q, cu_q, L, L, causal=True, topk_idx=idx,
                                                      return_attn_probs=True)
    infllm_v2.check_device_status()
    for rows in (slice(0, 256), slice(65408, 65664), slice(130816, 131072)):
        _check_selection_chunk(q, kc, L, rows, pooled, idx, mask)
    del pooled
    toks = torch.tensor([0, 31, 63, 64, 2111, 40000, 65535, 65536, 99999] + list(range(131064, 131072)),
                        device=DEV)
    # stage-1 scores of sampled 16-token chunks (the unfused scorer, bottom-right aligned on the
    # compressed keys of the chunk's prefix) against fp32 of the full sequence
    for t in (48, 40000, 99984, 131056):
        rows = slice(t, t + 16)
        n_pre = (rows.stop - 32) // 16 + 1
        cu16 = torch.tensor([0, 16], dtype=torch.int32, device=DEV)
        cu_p = torch.tensor([0, n_pre], dtype=torch.int32, device=DEV)
        sc = infllm_v2.infllmv2_attn_stage1(q[rows], kc[:n_pre], kc[:n_pre], cu16, cu_p, cu_p, 16, n_pre, causal=True)
        local = torch.arange(t, t + 16, device=DEV)
        ref = gpu_oracle.stage1_rows(q[rows], kc, local, L)[:, :, :n_pre]
        ok, worst = _stage1_close(sc, ref)
        assert ok, (t, worst)
    ref_out, ref_lse = gpu_oracle.attend_rows(q[toks], toks, k, v, idx[:, toks], L)
    mx, mr = err_stats(out[toks], ref_out)
    assert mx <= MAX_ABS and mr <= MEAN_REL, (mx, mr)
    got_lse = lse.view(hk, L, 16)[:, toks]
    assert (got_lse - ref_lse).abs().max().item() < 2e-2


def test_decode_at_batch_64_long_caches():
    """All 64 sequences (cache lengths uniform in [32768, 131072]): the sparse decode step with a
    given top-64 list, and the whole step with the selection from the compressed keys (scores
    against fp32, then pool / top-k / mask bit for bit on the GPU's scores)."""
    B, hk, lo, hi = 64, 2, 32768, 131072
    cap = hi + 64
    g = torch.Generator(device=DEV).manual_seed(0)
    s = 1.0 / math.sqrt(D)
    lens = torch.randint(lo, hi + 1, (B,), generator=torch.Generator().manual_seed(0)).to(torch.int32)
    kcache, vcache = _randn((B, cap, hk, D), g, s), _randn((B, cap, hk, D), g, s)
    q = _randn((B, 1, hk * 16, D), g, s)
    rng = np.random.default_rng(0)
    rows = np.full((B, hk, 1, TOPK), -1, np.int32)
    for b in range(B):
        nblk = (int(lens[b]) + BLOCK - 1) // BLOCK
        for h in range(hk):
            forced = [0] + list(range(nblk - 33, nblk))
            rest = rng.choice(np.arange(1, nblk - 33), size=TOPK - len(forced), replace=False)
            rows[b, h, 0] = np.sort(np.array(forced + list(rest), dtype=np.int32))
    idx = torch.from_numpy(rows).to(DEV)
    lens_d = lens.to(DEV)
    out = infllm_v2.infllmv2_attn_with_kvcache(q, kcache, vcache, cache_seqlens=lens_d, topk_idx=idx)
    ref = gpu_oracle.decode_rows(q, kcache, vcache, lens, idx)
    mx, mr = err_stats(out, ref)
    assert mx <= MAX_ABS and mr <= MEAN_REL, (mx, mr)

    # the whole step: compressed keys of every sequence, one query token each (the last token)
    n_c = [(int(l) - 32) // 16 + 1 for l in lens]
    cu_k = torch.tensor([0] + list(np.cumsum([int(l) for l in lens])), dtype=torch.int32, device=DEV)
    kc_parts = [infllm_v2.compress_keys(kcache[b, :int(lens[b])].contiguous())[0] for b in range(B)]
    kc = torch.cat(kc_parts, 0)
    cu_c = torch.tensor([0] + list(np.cumsum(n_c)), dtype=torch.int32, device=DEV)
    cu_q = torch.arange(B + 1, dtype=torch.int32, device=DEV)
    max_c, q2 = max(n_c), q.view(B, hk * 16, D)
    score = infllm_v2.infllmv2_attn_stage1(q2, kc, kc, cu_q, cu_c, cu_c, 1, max_c, causal=False)
    for b in (0, 17, 63):
        ref_s = gpu_oracle.stage1_rows(q2[b:b + 1], kc_parts[b], torch.zeros(1, dtype=torch.long), 1, causal=False)
        ok, worst = _stage1_close(score[:, b:b + 1, :n_c[b]], ref_s)
        assert ok, (b, worst)
        assert float(score[:, b, n_c[b]:].abs().max()) == 0.0 if n_c[b] < max_c else True
    positions = (lens_d - 1).contiguous()
    n_c_dev = torch.tensor(n_c, dtype=torch.int32, device=DEV)
    mask, sel = infllm_v2.decode_select(score, positions, TOPK, cap, LOCAL, INIT, seqused_c=n_c_dev,
                                        return_topk=True)
    sc = score.cpu()
    for b in range(B):
        pooled = oracle.max_pooling_1d(sc[:, b:b + 1, :n_c[b]], int(lens[b]) - 1, LOCAL, INIT)
        idx_ref = oracle.topk_select(pooled, TOPK, torch.tensor([(int(lens[b]) - 1) // BLOCK]))
        assert torch.equal(sel[b, :, 0].cpu(), idx_ref[:, 0]), b
        words_ref, _ = oracle.topk_to_uint64(idx_ref.numpy(), cap, BLOCK)
        assert np.array_equal(mask[b, :, 0].cpu().numpy(), words_ref[:, 0]), b
    out2 = infllm_v2.infllmv2_attn_with_kvcache(q, kcache, vcache, cache_seqlens=lens_d, block_mask=mask)
    ref2 = gpu_oracle.decode_rows(q, kcache, vcache, lens, sel)
    mx, mr = err_stats(out2, ref2)
    assert mx <= MAX_ABS and mr <= MEAN_REL, (mx, mr)
    # two-launch selection straight from the compressed keys gives the same mask
    mask2 = infllm_v2.infllmv2_stage1_decode_select(q2, kc, cu_c, positions, max_c, cap, TOPK, LOCAL, INIT)
    assert torch.equal(mask2, mask)
