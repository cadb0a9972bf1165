"""GPU: the caller-side layer (compress -> stage 1 -> pool -> top-k -> attention, cache fill,
decode step) against the oracle composed the same way, and decode against prefill."""
import numpy as np
import pytest
import torch

import oracle
import infllm_v2
from helpers import det_tensor, cu, err_stats

pytestmark = pytest.mark.gpu
DEV = "cuda"
HQ, HK, D = 32, 2, 128


def _config(**kw):
    base = dict(topk=4, init_blocks=1, local_blocks=1, dense_len=0)
    base.update(kw)
    return infllm_v2.SparseConfig(**base)


def _oracle_selection(q, k, lens, cfg, last_only=False):
    """Selection by the oracle, stage by stage.  Returns (idx, pooled)."""
    kc, cu_c = oracle.compress_keys(k, cu(lens), cfg.kernel_size, cfg.kernel_stride)
    kw = {}
    if cfg.coarse_lse:
        kv, cu_v = oracle.compress_keys(k, cu(lens), cfg.coarse_kernel_size, cfg.coarse_kernel_stride)
        kw = dict(lse_keys=kv, cu_seqlens_v=cu_v)
    max_k = int(np.diff(cu_c).max())
    s = oracle.stage1_scores(q, kc, cu(lens).tolist(), cu_c, max_k, True, **kw).to(torch.bfloat16)
    pooled = oracle.max_pooling_1d_varlen(s, cu(lens).tolist(), cu_c, [0] * len(lens), max(lens), max_k,
                                          cfg.local_blocks, cfg.init_blocks)
    qb = torch.cat([torch.arange(l) // 64 for l in lens])
    return oracle.topk_select(pooled.float(), cfg.topk, qb), pooled


def test_cache_fill_and_append_match_recompression():
    """cache_fill places packed rows; 70 decode_append steps keep keys, values and both compressed
    caches equal to compressing the grown sequences from scratch."""
    lens, cap = [100, 31, 257], 400
    cfg = _config(coarse_lse=True)
    g = torch.Generator().manual_seed(5)
    steps = 70
    k_all = [(torch.randn(l + steps, HK, D, generator=g) * 0.5).to(torch.bfloat16) for l in lens]
    v_all = [torch.randn(l + steps, HK, D, generator=g).to(torch.bfloat16) for l in lens]
    cache = infllm_v2.DecodeCache(len(lens), cap, HK, cfg, DEV)
    k0 = torch.cat([k[:l] for k, l in zip(k_all, lens)])
    v0 = torch.cat([v[:l] for v, l in zip(v_all, lens)])
    kc0, cu_c = oracle.compress_keys(k0, cu(lens), 32, 16)
    kv0, cu_v = oracle.compress_keys(k0, cu(lens), 128, 64)
    cache.fill(k0.to(DEV), v0.to(DEV), kc0.to(DEV), cu(lens, DEV), torch.tensor(cu_c, dtype=torch.int32, device=DEV),
               max(lens), kv0.to(DEV), torch.tensor(cu_v, dtype=torch.int32, device=DEV))
    assert cache.seqlens.tolist() == lens
    assert cache.n_comp.tolist() == list(np.diff(cu_c)) and cache.n_comp2.tolist() == list(np.diff(cu_v))
    for b, l in enumerate(lens):
        assert torch.equal(cache.k[b, :l].cpu(), k_all[b][:l]) and torch.equal(cache.v[b, :l].cpu(), v_all[b][:l])
    for s in range(steps):
        kn = torch.stack([k[l + s] for k, l in zip(k_all, lens)]).to(DEV)
        vn = torch.stack([v[l + s] for v, l in zip(v_all, lens)]).to(DEV)
        infllm_v2.decode_append(kn, vn, cache.k, cache.v, cache.seqlens, cache.positions, cache.kc, cache.n_comp,
                                32, 16, cache.kc2, cache.n_comp2, 128, 64)
    torch.cuda.synchronize()
    assert cache.seqlens.tolist() == [l + steps for l in lens]
    assert cache.positions.tolist() == [l + steps - 1 for l in lens]
    for b, l in enumerate(lens):
        n = l + steps
        assert torch.equal(cache.k[b, :n].cpu(), k_all[b]) and torch.equal(cache.v[b, :n].cpu(), v_all[b])
        for kc_cache, count, (ks, st) in ((cache.kc, cache.n_comp, (32, 16)), (cache.kc2, cache.n_comp2, (128, 64))):
            ref, _ = oracle.compress_keys(k_all[b], [0, n], ks, st)
            assert int(count[b]) == ref.shape[0]
            if ref.shape[0] == 0:
                continue
            got = kc_cache[b, :ref.shape[0]].cpu().float()
            assert (got - ref.float()).abs().max().item() <= 2.0 ** -7      # one bf16 step: summation order


@pytest.mark.parametrize("coarse", [False, True])
def test_prefill_matches_composed_oracle(coarse):
    lens = [700, 130, 1000]
    cfg = _config(coarse_lse=coarse)
    q = det_tensor((sum(lens), HQ, D), 11, 0.5)
    k = det_tensor((sum(lens), HK, D), 12, 0.5)
    v = det_tensor((sum(lens), HK, D), 13, 1.0)
    layer = infllm_v2.SparseAttention(cfg)
    cq = cu(lens, DEV)
    qd, kd, vd = (t.to(DEV).requires_grad_(True) for t in (q, k, v))
    out = layer.prefill(qd, kd, vd, cq, max(lens), seqlens=lens)
    do = det_tensor((sum(lens), HQ, D), 14, 1.0)
    out.backward(do.to(DEV))
    infllm_v2.check_device_status()
    # the layer's own selection, recomputed through its public pieces
    kc, cu_c = layer.compress(kd.detach(), cq, lens)
    kc2 = cu_c2 = None
    if coarse:
        kc2, cu_c2 = layer.compress(kd.detach(), cq, lens, coarse=True)
    idx = layer.select(qd.detach(), kc, cq, cu_c, max(lens), cfg.windows(max(lens)), kc2, cu_c2).cpu()
    exp_idx, _ = _oracle_selection(q, k, lens, cfg)
    same = (idx == exp_idx).all(-1).float().mean().item()
    assert same > 0.97, same                   # bf16 block scores that tie differently pick another block
    ro, _, rdq, rdk, rdv = oracle.sparse_attention_fwd_bwd(q, k, v, do, cu(lens).tolist(), cu(lens).tolist(), idx)
    for name, a, b in (("out", out, ro), ("dq", qd.grad, rdq), ("dk", kd.grad, rdk), ("dv", vd.grad, rdv)):
        mx, mr = err_stats(a.detach().float().cpu(), b)
        assert mx <= 2e-2 * max(1.0, b.abs().max().item()) and mr <= 1e-2, (name, mx, mr)


def test_short_sequences_attend_densely():
    lens = [300, 64]
    layer = infllm_v2.SparseAttention(_config(dense_len=512))
    q = det_tensor((sum(lens), HQ, D), 21, 0.5)
    k = det_tensor((sum(lens), HK, D), 22, 0.5)
    v = det_tensor((sum(lens), HK, D), 23, 1.0)
    out = layer.prefill(q.to(DEV), k.to(DEV), v.to(DEV), cu(lens, DEV), max(lens), seqlens=lens)
    ref, _ = oracle.sparse_attention_fwd(q, k, v, cu(lens).tolist(), cu(lens).tolist(), None)
    mx, mr = err_stats(out.float().cpu(), ref)
    assert mx <= 2e-2 and mr <= 1e-2


@pytest.mark.parametrize("hk,lens,topk,local,init", [(1, [65, 257, 31], 4, 0, 2), (4, [130], 6, 2, 1),
                                                     (2, [16, 40], 3, 1, 1)])
def test_decode_other_shapes(hk, lens, topk, local, init):
    """Other head counts, forced-block settings and sequences that start below one compression
    window: 24 decoded tokens each against the oracle's dense-with-mask attention under the
    oracle's own selection for that token (rows whose bf16 block scores tie differently excepted)."""
    cfg = _config(topk=topk, local_blocks=local, init_blocks=init)
    layer = infllm_v2.SparseAttention(cfg)
    steps, cap = 24, 320
    g = torch.Generator().manual_seed(sum(lens) + hk)
    qs = [(torch.randn(l + steps, hk * 16, D, generator=g) * 0.5).to(torch.bfloat16) for l in lens]
    ks = [(torch.randn(l + steps, hk, D, generator=g) * 0.5).to(torch.bfloat16) for l in lens]
    vs = [torch.randn(l + steps, hk, D, generator=g).to(torch.bfloat16) for l in lens]
    pack = lambda ts, n: torch.cat([t[:l + n] for t, l in zip(ts, lens)])
    cache = infllm_v2.DecodeCache(len(lens), cap, hk, cfg, DEV)
    layer.prefill(pack(qs, 0).to(DEV), pack(ks, 0).to(DEV), pack(vs, 0).to(DEV), cu(lens, DEV), max(lens),
                  seqlens=lens, cache=cache)
    agree = []
    for s in range(steps):
        stack = lambda ts: torch.stack([t[l + s] for t, l in zip(ts, lens)])
        out = layer.decode(stack(qs).to(DEV), stack(ks).to(DEV), stack(vs).to(DEV), cache)
        if s % 5:
            continue
        grown = [l + s + 1 for l in lens]
        exp_idx, _ = _oracle_selection(pack(qs, s + 1), pack(ks, s + 1), grown, cfg)
        ref, _ = oracle.sparse_attention_fwd(pack(qs, s + 1), pack(ks, s + 1), pack(vs, s + 1), cu(grown).tolist(),
                                             cu(grown).tolist(), exp_idx)
        last = torch.tensor(np.cumsum(grown) - 1)
        err = (out[:, 0].float().cpu() - ref[last]).abs().amax(-1)
        agree.append((err <= 2e-2).float().mean().item())
    infllm_v2.check_device_status()
    assert cache.seqlens.tolist() == [l + steps for l in lens]
    assert np.mean(agree) > 0.9, agree


@pytest.mark.parametrize("coarse", [False, True])
def test_decode_continues_prefill(coarse):
    """Prefill L tokens into a cache, decode 40 more one at a time: every decoded token equals the
    last row of a prefill over the sequence grown by that token (same selection rule, same
    attention), and the decode selection equals the oracle's for that row."""
    lens, cap, steps = [200, 460, 150], 512, 40
    cfg = _config(coarse_lse=coarse, topk=5)
    layer = infllm_v2.SparseAttention(cfg)
    g = torch.Generator().manual_seed(9)
    qs = [(torch.randn(l + steps, HQ, D, generator=g) * 0.5).to(torch.bfloat16) for l in lens]
    ks = [(torch.randn(l + steps, HK, D, generator=g) * 0.5).to(torch.bfloat16) for l in lens]
    vs = [torch.randn(l + steps, HK, D, generator=g).to(torch.bfloat16) for l in lens]
    pack = lambda ts, n: torch.cat([t[:l + n] for t, l in zip(ts, lens)])
    cache = infllm_v2.DecodeCache(len(lens), cap, HK, cfg, DEV)
    layer.prefill(pack(qs, 0).to(DEV), pack(ks, 0).to(DEV), pack(vs, 0).to(DEV), cu(lens, DEV), max(lens),
                  seqlens=lens, cache=cache)
    agree = []
    for s in range(steps):
        qn = torch.stack([q[l + s] for q, l in zip(qs, lens)]).to(DEV)
        kn = torch.stack([k[l + s] for k, l in zip(ks, lens)]).to(DEV)
        vn = torch.stack([v[l + s] for v, l in zip(vs, lens)]).to(DEV)
        out = layer.decode(qn, kn, vn, cache)
        if s % 13 and s != steps - 1:
            continue
        grown = [l + s + 1 for l in lens]
        full = layer.prefill(pack(qs, s + 1).to(DEV), pack(ks, s + 1).to(DEV), pack(vs, s + 1).to(DEV),
                             cu(grown, DEV), max(grown), seqlens=grown)
        last = torch.tensor(np.cumsum(grown) - 1)
        err = (out[:, 0].float().cpu() - full[last.to(DEV)].float().cpu()).abs().amax(-1)    # (B, Hq)
        agree.append((err <= 2e-2).float().mean().item())
    infllm_v2.check_device_status()
    assert cache.seqlens.tolist() == [l + steps for l in lens]
    assert np.mean(agree) > 0.9, agree          # a tie that flips selects another block for 16 heads


def test_decode_graph_replay_equals_eager_steps():
    """The captured decode step (sized for the capacity) against eager steps on a twin cache."""
    lens, cap, steps = [300, 90, 411], 448, 20
    cfg = _config(topk=5)
    layer = infllm_v2.SparseAttention(cfg)
    g = torch.Generator().manual_seed(3)
    qs = [(torch.randn(l + steps, HQ, D, generator=g) * 0.5).to(torch.bfloat16) for l in lens]
    ks = [(torch.randn(l + steps, HK, D, generator=g) * 0.5).to(torch.bfloat16) for l in lens]
    vs = [torch.randn(l + steps, HK, D, generator=g).to(torch.bfloat16) for l in lens]
    pack = lambda ts: torch.cat([t[:l] for t, l in zip(ts, lens)]).to(DEV)
    caches = [infllm_v2.DecodeCache(len(lens), cap, HK, cfg, DEV) for _ in range(2)]
    for c in caches:
        layer.prefill(pack(qs), pack(ks), pack(vs), cu(lens, DEV), max(lens), seqlens=lens, cache=c)
    step = layer.capture_decode(caches[1])
    assert caches[1].seqlens.tolist() == lens and caches[1].max_len == max(lens)
    for s in range(steps):
        qn = torch.stack([q[l + s] for q, l in zip(qs, lens)]).to(DEV)
        kn = torch.stack([k[l + s] for k, l in zip(ks, lens)]).to(DEV)
        vn = torch.stack([v[l + s] for v, l in zip(vs, lens)]).to(DEV)
        eager = layer.decode(qn, kn, vn, caches[0])
        replayed = step(qn, kn, vn)
        assert torch.equal(eager, replayed), s
    infllm_v2.check_device_status()
    assert caches[1].seqlens.tolist() == [l + steps for l in lens]
    assert torch.equal(caches[0].kc, caches[1].kc) and torch.equal(caches[0].k, caches[1].k)


@pytest.mark.parametrize("coarse", [False, True])
def test_decode_graph_equals_eager_with_a_dense_length(coarse):
    """dense_len > 0 with sequences on both sides of it: the captured step (sized for the capacity)
    and eager steps give the same outputs, and a sequence of at most dense_len tokens attends every
    block (its output equals dense attention over its cache)."""
    lens, cap, steps = [700, 90, 300], 768, 6
    cfg = _config(topk=3, dense_len=384, coarse_lse=coarse)
    layer = infllm_v2.SparseAttention(cfg)
    g = torch.Generator().manual_seed(5)
    qs = [(torch.randn(l + steps, HQ, D, generator=g) * 0.5).to(torch.bfloat16) for l in lens]
    ks = [(torch.randn(l + steps, HK, D, generator=g) * 0.5).to(torch.bfloat16) for l in lens]
    vs = [torch.randn(l + steps, HK, D, generator=g).to(torch.bfloat16) for l in lens]
    pack = lambda ts: torch.cat([t[:l] for t, l in zip(ts, lens)]).to(DEV)
    caches = [infllm_v2.DecodeCache(len(lens), cap, HK, cfg, DEV) for _ in range(2)]
    for c in caches:
        layer.prefill(pack(qs), pack(ks), pack(vs), cu(lens, DEV), max(lens), seqlens=lens, cache=c)
    step = layer.capture_decode(caches[1])
    for s in range(steps):
        qn = torch.stack([q[l + s] for q, l in zip(qs, lens)]).to(DEV)
        kn = torch.stack([k[l + s] for k, l in zip(ks, lens)]).to(DEV)
        vn = torch.stack([v[l + s] for v, l in zip(vs, lens)]).to(DEV)
        eager = layer.decode(qn, kn, vn, caches[0])
        replayed = step(qn, kn, vn)
        assert torch.equal(eager, replayed), s
        # sequences 1 and 2 (91.. and 301.. tokens) are below dense_len: dense attention
        dense = infllm_v2.infllmv2_attn_with_kvcache(qn.view(len(lens), 1, HQ, D), caches[0].k, caches[0].v,
                                                     cache_seqlens=caches[0].seqlens)
        assert torch.equal(eager[1:], dense[1:]), s
        assert not torch.equal(eager[0], dense[0]), s       # 700+ tokens, 3 of 11+ blocks: sparse
    infllm_v2.check_device_status()


@pytest.mark.parametrize("cap,topk", [(2048, 8), (40000, 64)])
def test_stage1_decode_select_equals_scores_then_select(cap, topk):
    """The two-launch decode selection (scores stay on chip) against scorer -> decode_select, bit
    for bit, on a per-sequence cache of compressed keys scored in place (seqused_k)."""
    b, hk = 5, 2
    rng = np.random.default_rng(cap)
    lens = rng.integers(40, cap + 1, size=b)
    lens[0], lens[-1] = 33, cap
    n_c = np.where(lens >= 32, (lens - 32) // 16 + 1, 0).astype(np.int32)
    c_cap = (cap - 32) // 16 + 1
    max_c = int(n_c.max())
    g = torch.Generator().manual_seed(cap)
    kc = (torch.randn(b, c_cap, hk, D, generator=g) * 0.6).to(torch.bfloat16).to(DEV)
    q = (torch.randn(b, hk * 16, D, generator=g) * 0.6).to(torch.bfloat16).to(DEV)
    used = torch.tensor(n_c, device=DEV)
    positions = torch.tensor(lens - 1, dtype=torch.int32, device=DEV)
    cu_q = torch.arange(b + 1, dtype=torch.int32, device=DEV)
    cu_c = cu_q * c_cap
    flat = kc.view(-1, hk, D)
    mask, idx = infllm_v2.infllmv2_stage1_decode_select(q, flat, cu_c, positions, max_c, cap, topk, 2, 1,
                                                        seqused_k=used, return_topk=True)
    score = infllm_v2.infllmv2_attn_stage1(q, flat, flat, cu_q, cu_c, cu_c, 1, max_c, causal=False, seqused_k=used)
    ref_mask, ref_idx = infllm_v2.decode_select(score, positions, topk, cap, 2, 1, seqused_c=used, return_topk=True)
    infllm_v2.check_device_status()
    assert torch.equal(idx, ref_idx)
    assert torch.equal(mask, ref_mask)
    # the scores themselves against the oracle on the packed keys (seqused_k semantics)
    packed = torch.cat([kc[i, :n_c[i]] for i in range(b)]).cpu()
    cu_p = np.concatenate([[0], np.cumsum(n_c)])
    exp = oracle.stage1_scores(q.cpu(), packed, list(range(b + 1)), cu_p.tolist(), max_c, False)
    assert (score.float().cpu() - exp).abs().max().item() <= 2e-2


def test_cache_capacity_limits():
    """Rows past the capacity are dropped by cache_fill; a full cache is left untouched by
    decode_append and refused by the layer before anything is launched."""
    cfg = _config()
    lens, cap = [100, 40], 64
    k = det_tensor((sum(lens), HK, D), 71, 0.5)
    v = det_tensor((sum(lens), HK, D), 72, 1.0)
    kc, cu_c = oracle.compress_keys(k, cu(lens), 32, 16)
    cache = infllm_v2.DecodeCache(len(lens), cap, HK, cfg, DEV)
    cache.fill(k.to(DEV), v.to(DEV), kc.to(DEV), cu(lens, DEV), torch.tensor(cu_c, dtype=torch.int32, device=DEV),
               max(lens))
    assert cache.seqlens.tolist() == [64, 40] and cache.max_len == 64
    assert cache.n_comp.tolist() == [min(5, cache.c_capacity), 1]
    assert torch.equal(cache.k[0].cpu(), k[:64]) and torch.equal(cache.k[1, :40].cpu(), k[100:])
    before = cache.k.clone()
    kn = det_tensor((2, HK, D), 73, 0.5).to(DEV)
    infllm_v2.decode_append(kn, kn, cache.k, cache.v, cache.seqlens, cache.positions, cache.kc, cache.n_comp)
    torch.cuda.synchronize()
    assert cache.seqlens.tolist() == [64, 41] and cache.positions.tolist() == [64, 40]
    assert torch.equal(cache.k[0], before[0]) and torch.equal(cache.k[1, 40].cpu(), kn[1].cpu())
    with pytest.raises(RuntimeError):
        infllm_v2.SparseAttention(cfg).decode(det_tensor((2, HQ, D), 74, 0.5).to(DEV), kn, kn, cache)
