"""CPU: the oracle restatements against the committed golden vectors (made by running the
reference's own Python oracles, tests/golden/make_golden.py)."""
import os

import numpy as np
import torch

import oracle
from oracle.pooling import max_pooling_1d_literal
from inputs import det_array, det_perm_rows


def _load(golden_dir, name):
    return np.load(os.path.join(golden_dir, name))


def test_bitmask_golden(golden_dir):
    g = _load(golden_dir, "bitmask.npz")
    for key in [k for k in g.files if k.endswith("_idx")]:
        base = key[:-4]
        got, kb = oracle.topk_to_uint64(g[key], int(g[base + "_maxk"]), 64)
        assert np.array_equal(got, g[base + "_out"]), key
    for key in [k for k in g.files if k.endswith("_mask")]:
        base = key[:-5]
        got, n = oracle.blockmask_to_uint64(g[key])
        assert np.array_equal(got, g[base + "_out"]), key
        assert np.array_equal(oracle.uint64_to_bool(got, n), g[key]), key


def test_transpose_matches_roundtrip():
    rng = np.random.default_rng(3)
    for hk, t, kb in ((2, 130, 70), (1, 64, 64), (3, 1, 129)):
        m = rng.random((hk, t, kb)) < 0.3
        fwd, _ = oracle.blockmask_to_uint64(m)
        bwd = oracle.transpose_blockmask(fwd, kb)
        assert bwd.shape == (hk, kb, (t + 63) // 64)
        assert np.array_equal(oracle.uint64_to_bool(bwd, t), np.swapaxes(m, 1, 2))


def test_stage1_golden(golden_dir):
    g = _load(golden_dir, "stage1.npz")
    for key in [k for k in g.files if k.endswith("_shape")]:
        base = key[:-6]
        lq, lc, seed = (int(x) for x in g[key][:3])
        if len(g[key]) == 4:                 # "compressed LSE" case: row sums over coarser keys
            lcv = int(g[key][3])
            q = torch.from_numpy(det_array((lq, 32, 128), seed, 0.5))
            k = torch.from_numpy(det_array((lc, 2, 128), seed + 1000))
            kv = torch.from_numpy(det_array((lcv, 2, 128), seed + 2000))
            got = oracle.stage1_scores(q, k, [0, lq], [0, lc], lc, bool(g[base + "_causal"]),
                                       lse_keys=kv, cu_seqlens_v=[0, lcv])
            ref = g[base + "_out"]
            assert np.abs(got.numpy() - ref).max() <= 1e-5 * max(1.0, np.abs(ref).max()), base
            continue
        q = torch.from_numpy(det_array((lq, 32, 128), seed))
        k = torch.from_numpy(det_array((lc, 2, 128), seed + 1000))
        got = oracle.stage1_scores(q, k, [0, lq], [0, lc], lc, bool(g[base + "_causal"]))
        assert np.abs(got.numpy() - g[base + "_out"]).max() < 2e-6, base


def test_stage1_varlen_equals_per_sequence():
    q = torch.from_numpy(det_array((96 + 40, 32, 128), 7))
    k = torch.from_numpy(det_array((5 + 1, 2, 128), 8))
    both = oracle.stage1_scores(q, k, [0, 96, 136], [0, 5, 6], 5, True)
    a = oracle.stage1_scores(q[:96], k[:5], [0, 96], [0, 5], 5, True)
    b = oracle.stage1_scores(q[96:], k[5:], [0, 40], [0, 1], 5, True)
    assert torch.equal(both[:, :96], a) and torch.equal(both[:, 96:], b)


def test_stage2_and_decode_golden(golden_dir):
    g = _load(golden_dir, "stage2.npz")
    step = int(g["out_row_step"])
    hq, hk, d = 32, 2, 128
    for name in ("a", "b", "c"):
        seed, k_sel = (int(x) for x in g[f"s2_{name}_seed"])
        cu_q, cu_k = g[f"s2_{name}_cuq"], g[f"s2_{name}_cuk"]
        sk = int(np.diff(cu_k).max())
        q = torch.from_numpy(det_array((int(cu_q[-1]), hq, d), seed, 0.25))
        k = torch.from_numpy(det_array((int(cu_k[-1]), hk, d), seed + 1000, 0.25))
        v = torch.from_numpy(det_array((int(cu_k[-1]), hk, d), seed + 2000))
        idx = torch.from_numpy(det_perm_rows(hk * int(cu_q[-1]), (sk + 63) // 64, k_sel, seed + 3000)
                               ).view(hk, -1, k_sel)
        for causal in (0, 1):
            key = f"s2_{name}_{causal}_out"
            if key not in g.files:
                continue
            got, _ = oracle.sparse_attention_fwd(q, k, v, cu_q, cu_k, idx, causal=bool(causal))
            # the reference turns rows without a visible key into NaN -> 0 as well
            lens = np.diff(cu_q)
            per_seq = torch.cat([got[cu_q[b]:cu_q[b + 1]][:] for b in range(len(lens))], 0)
            # golden rows were subsampled per sequence-concatenated tensor
            assert np.abs(per_seq[::step].numpy() - g[key]).max() < 5e-6, key
    bsz, hq, hk, d, cache = (int(x) for x in g["dec_shape"])
    q = torch.from_numpy(det_array((bsz, hq, 1, d), 301, 0.25))
    kc = torch.from_numpy(det_array((bsz, hk, cache + 1, d), 302, 0.25))
    vc = torch.from_numpy(det_array((bsz, hk, cache + 1, d), 303))
    idx = torch.from_numpy(det_perm_rows(bsz * hk, (cache + 1 + 63) // 64, 3, 304)).view(bsz, hk, 1, 3)
    got, _ = oracle.kvcache_decode(q.transpose(1, 2), kc.transpose(1, 2).contiguous(),
                                   vc.transpose(1, 2).contiguous(),
                                   torch.full((bsz,), cache + 1, dtype=torch.int32), idx)
    assert np.abs(got.numpy() - g["dec_out"]).max() < 5e-6


def test_pool_topk_golden(golden_dir):
    g = _load(golden_dir, "pool_topk.npz")
    for name in ("a", "b", "c", "d"):
        x = torch.from_numpy(g[f"pool_{name}_x"]).to(torch.bfloat16)
        cache, local, init = (int(v) for v in g[f"pool_{name}_args"])
        y = oracle.max_pooling_1d(x, cache, local, init).float().numpy()
        assert np.array_equal(y, g[f"pool_{name}_y"]), name
    y = torch.from_numpy(g["topk_y"])
    assert np.array_equal(oracle.topk_select(y, 5, torch.tensor([7, 7, 7])).numpy(), g["topk_exp_all"])
    assert np.array_equal(oracle.topk_select(y, 5, torch.from_numpy(g["topk_bq_cut"])).numpy(),
                          g["topk_exp_cut"])


def test_topk_oracle_equals_reference_bitonic_kernel(golden_dir):
    """The pin of the top-k oracle: on tie-heavy rows with +-inf it selects the blocks that the
    reference's bitonic kernel (csrc/topk.cuh:6-117, simulated thread for thread when the fixture
    was made) selects, in the same order; the simulation itself is re-run here on two of the cases."""
    from oracle.topk import bitonic_topk_literal
    g = _load(golden_dir, "pool_topk.npz")
    names = sorted(k[len("bitonic_"):-2] for k in g.files if k.startswith("bitonic_") and k.endswith("_x"))
    assert len(names) >= 6
    for name in names:
        x = torch.from_numpy(g[f"bitonic_{name}_x"].astype(np.float32))
        pos = g[f"bitonic_{name}_pos"]
        n, k = x.shape[1], pos.shape[1]
        order = torch.sort(x, dim=-1, descending=True, stable=True).indices[:, :k].numpy()
        assert np.array_equal(order, pos), name
        sel = oracle.topk_select(x[None], k, torch.full((x.shape[0],), n))[0].numpy()
        assert np.array_equal(sel, np.sort(pos, axis=1)), name
        if name in ("b", "c"):
            _, again = bitonic_topk_literal(x.numpy(), k)
            assert np.array_equal(again, pos), name


def test_pool_varlen_equals_fixed():
    rng = np.random.default_rng(5)
    x = torch.from_numpy(rng.random((2, 150, 9)).astype(np.float32)).to(torch.bfloat16)
    cu_q, cu_k, cl = [0, 100, 150], [0, 9, 15], [0, 64]
    y = oracle.max_pooling_1d_varlen(x, cu_q, cu_k, cl, 100, 9, 2, 1)
    a = oracle.max_pooling_1d(x[:, :100], 0, 2, 1)
    b = oracle.max_pooling_1d(x[:, 100:, :6], 64, 2, 1)
    assert torch.equal(y[:, :100, :a.shape[2]], a)
    assert torch.equal(y[:, 100:, :b.shape[2]], b)


def test_backward_oracle_matches_finite_difference():
    torch.manual_seed(0)
    q = torch.randn(20, 16, 8, dtype=torch.float64) * 0.5
    k = torch.randn(70, 1, 8, dtype=torch.float64) * 0.5
    v = torch.randn(70, 1, 8, dtype=torch.float64)
    idx = torch.tensor([[[0, 1]] * 20], dtype=torch.int32)
    do = torch.randn(20, 16, 8, dtype=torch.float64)

    def f(q_, k_, v_):
        from oracle.attention import _seq_attention
        bm = oracle.expand_topk_mask(idx, 2)
        return _seq_attention(q_, k_, v_, bm, True, 0.3, 64)[0]

    assert torch.autograd.gradcheck(f, (q.requires_grad_(), k.requires_grad_(), v.requires_grad_()),
                                    eps=1e-6, atol=1e-5)


def test_compress_golden(golden_dir):
    """Key compression against the outputs of the reference's compress_tensor test helper."""
    g = _load(golden_dir, "compress.npz")
    for key in [k for k in g.files if k.endswith("_lens")]:
        base = key[:-5]
        lens = [int(x) for x in g[key]]
        kernel, stride, seed, hk = (int(x) for x in g[base + "_cfg"])
        k = torch.from_numpy(det_array((sum(lens), hk, 128), seed)).to(torch.bfloat16)
        cu = [0] + list(np.cumsum(lens))
        got, cu_c = oracle.compress_keys(k, cu, kernel, stride)
        assert cu_c == [int(x) for x in g[base + "_cu_c"]], key
        assert np.array_equal(got.float().numpy(), g[base + "_out"]), key


def test_rotary_golden(golden_dir):
    """The rotary helper against fixtures made from the element-by-element restatement of the
    reference's device loops (csrc/flash_attn/src/rotary.h:20-150); the restatement is re-run."""
    from inputs import det_array
    g = _load(golden_dir, "stage2.npz")
    names = sorted(k[len("rotary_"):-4] for k in g.files if k.startswith("rotary_") and k.endswith("_cfg"))
    assert len(names) == 4
    for name in names:
        rows, rd, inter, sx, sa = (int(v) for v in g[f"rotary_{name}_cfg"])
        x = torch.from_numpy(det_array((rows, 128), sx)).to(torch.bfloat16)
        ang = torch.from_numpy(det_array((rows, rd // 2), sa, 3.0))
        c, s_ = torch.cos(ang).to(torch.bfloat16), torch.sin(ang).to(torch.bfloat16)
        got = oracle.apply_rotary(x, c, s_, bool(inter)).float().numpy()
        assert np.array_equal(got, g[f"rotary_{name}_out"]), name
        lit = oracle.apply_rotary_literal(x.float().numpy(), c.float().numpy(), s_.float().numpy(), bool(inter))
        assert np.array_equal(torch.from_numpy(lit).to(torch.bfloat16).float().numpy(), g[f"rotary_{name}_out"]), name
