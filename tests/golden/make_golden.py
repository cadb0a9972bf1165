#!/usr/bin/env python
"""Generate the committed golden fixtures by RUNNING THE REFERENCE'S OWN PYTHON ORACLES.

Run where the reference checkout is available:

    python tests/golden/make_golden.py --reference /path/to/infllmv2_cuda_impl

It imports, unmodified, from the reference's tests/ directory:
  tests/stage1/naive_softmax.py::torch_naive_softmax
  tests/stage1/complse_online_softmax.py::compresssed_lse_online_softmax
  tests/test_topk_to_uint64.py::topk_to_uint64_numpy
  tests/test_blockmask.py::py_blockmask_to_uint64
  tests/test_uint64_to_bool.py::py_uint64_to_bool
  tests/utils.py::convert_topk_to_base_blockmask, prepare_mixed_mask, attention_blocksparse_ref
  tests/test_kvcache_simple.py::naive_attention
  tests/test_stage1_compressed_lse.py::compress_tensor (+ calc_chunks_with_stride)
(the `infllm_v2` CUDA module and matplotlib those files import at the top are replaced by
empty stand-ins; none of the functions above touches them), feeds them seeded inputs and
stores the expected outputs as small .npz files next to this script (the inputs are recomputed
from tests/golden/inputs.py, a platform-independent integer hash, so they need not be stored).  The max-pool and top-k
fixtures come from a loop-for-loop transliteration of csrc/max_pooling_1d.cuh:122-159 and from
a thread-for-thread simulation of the reference's bitonic top-k kernel, csrc/topk.cuh:6-117
(the reference has no Python twin of either).
The fixtures then travel with the repository; nothing at test time reads the reference.
"""
import argparse
import importlib
import os
import sys
import tempfile
import types

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))
sys.path.insert(0, HERE)
from inputs import det_array, det_perm_rows  # noqa: E402


def _import_reference(ref_root):
    for name in ("matplotlib", "matplotlib.pyplot", "matplotlib.colors", "seaborn"):
        sys.modules.setdefault(name, types.ModuleType(name))
    stub = types.ModuleType("infllm_v2")
    for fn in ("infllmv2_attn_stage1", "infllmv2_attn_varlen_func", "infllmv2_attn_with_kvcache",
               "topk_to_uint64", "blockmask_to_uint64", "uint64_to_bool", "max_pooling_1d",
               "max_pooling_1d_varlen"):
        setattr(stub, fn, None)
    sys.modules["infllm_v2"] = stub
    sys.path.insert(0, os.path.join(ref_root, "tests"))
    os.chdir(tempfile.mkdtemp())          # tests/utils.py creates a directory in the cwd on import
    mods = {}
    for m in ("stage1.naive_softmax", "stage1.complse_online_softmax", "test_topk_to_uint64",
              "test_blockmask", "test_uint64_to_bool", "utils", "test_kvcache_simple",
              "test_stage1_compressed_lse"):
        mods[m] = importlib.import_module(m)
    return mods


OUT_ROW_STEP = 16     # stage-2 outputs are stored for every 16th token only (keeps the files small)


def gen_bitmask(mods, out):
    rng = np.random.default_rng(0)
    cases = {}
    # topk_to_uint64: 3-D, 4-D, multi-word, with -1 padding
    for name, shape, max_k in (("a", (2, 5, 4), 64 * 6), ("b", (2, 3, 8), 64 * 200),
                               ("c", (2, 2, 3, 8), 64 * 70), ("d", (1, 7, 16), 64 * 64)):
        kb = (max_k + 63) // 64
        idx = np.stack([rng.permutation(kb)[: shape[-1]] for _ in range(int(np.prod(shape[:-1])))])
        idx = np.sort(idx, -1).astype(np.int32).reshape(shape)
        idx[..., -1] = np.where(rng.random(shape[:-1]) < 0.5, -1, idx[..., -1])
        ref, _ = mods["test_topk_to_uint64"].topk_to_uint64_numpy(idx, max_k, 64)
        cases[f"t2u_{name}_idx"] = idx
        cases[f"t2u_{name}_maxk"] = np.int64(max_k)
        cases[f"t2u_{name}_out"] = ref.view(np.int64)
    for name, shape in (("a", (3, 63)), ("b", (2, 2, 64)), ("c", (4, 65)), ("d", (2, 3, 200)),
                        ("e", (5, 1)), ("f", (1, 1024))):
        m = rng.random(shape) < 0.5
        ref, _ = mods["test_blockmask"].py_blockmask_to_uint64(torch.from_numpy(m))
        back = mods["test_uint64_to_bool"].py_uint64_to_bool(ref, shape[-1])
        assert (back.numpy() == m).all()
        cases[f"b2u_{name}_mask"] = m
        cases[f"b2u_{name}_out"] = ref.numpy()
    np.savez_compressed(os.path.join(out, "bitmask.npz"), **cases)

    import oracle
    for key in [k for k in cases if k.endswith("_idx")]:
        base = key[:-4]
        got, _ = oracle.topk_to_uint64(cases[key], int(cases[base + "_maxk"]), 64)
        assert (got == cases[base + "_out"]).all(), key
    for key in [k for k in cases if k.endswith("_mask")]:
        base = key[:-5]
        got, n = oracle.blockmask_to_uint64(cases[key])
        assert (got == cases[base + "_out"]).all(), key
        assert (oracle.uint64_to_bool(got, n) == cases[key]).all(), key
    print("bitmask: oracle == reference python twins")


def gen_stage1(mods, out):
    import oracle
    naive = mods["stage1.naive_softmax"].torch_naive_softmax
    cases = {}
    worst = 0.0
    for name, lq, lc, causal in (("a", 64, 15, True), ("b", 64, 16, True), ("c", 256, 17, True),
                                 ("d", 256, 15, False), ("e", 100, 5, True), ("f", 272, 16, True),
                                 ("g", 33, 1, True), ("h", 48, 40, True), ("i", 1000, 61, True)):
        seed = 100 + ord(name)
        q = torch.from_numpy(det_array((lq, 32, 128), seed))
        k = torch.from_numpy(det_array((lc, 2, 128), seed + 1000))
        ref = naive(q, k, causal=causal)                              # (2, lq, lc) fp32
        got = oracle.stage1_scores(q, k, [0, lq], [0, lc], lc, causal)
        worst = max(worst, (got - ref).abs().max().item())
        cases[f"s1_{name}_shape"] = np.array([lq, lc, seed], dtype=np.int64)
        cases[f"s1_{name}_causal"] = np.bool_(causal)
        cases[f"s1_{name}_out"] = ref.numpy()
    assert worst < 2e-6, worst
    print(f"stage1: oracle vs torch_naive_softmax max|diff| = {worst:.2e}")
    # "compressed LSE" mode: row sums over coarser keys (kernel 128 / stride 64 of the same tokens)
    complse = mods["stage1.complse_online_softmax"].compresssed_lse_online_softmax
    worst = 0.0
    for name, lq, causal in (("ca", 256, True), ("cb", 512, True), ("cc", 256, False), ("cd", 1024, True)):
        seed = 300 + ord(name[1])
        lc, lcv = (lq - 32) // 16 + 1, (lq - 128) // 64 + 1
        q = torch.from_numpy(det_array((lq, 32, 128), seed, 0.5))
        k = torch.from_numpy(det_array((lc, 2, 128), seed + 1000))
        kv = torch.from_numpy(det_array((lcv, 2, 128), seed + 2000))
        ref = complse(q, k, kv, 16, 16, causal=causal)                # (2, lq, lc) fp32
        got = oracle.stage1_scores(q, k, [0, lq], [0, lc], lc, causal, lse_keys=kv, cu_seqlens_v=[0, lcv])
        worst = max(worst, (got - ref).abs().max().item() / max(1.0, ref.abs().max().item()))
        cases[f"s1_{name}_shape"] = np.array([lq, lc, seed, lcv], dtype=np.int64)
        cases[f"s1_{name}_causal"] = np.bool_(causal)
        cases[f"s1_{name}_out"] = ref.numpy()
    assert worst < 1e-5, worst
    print(f"stage1 compressed-LSE: oracle vs compresssed_lse_online_softmax max rel diff = {worst:.2e}")
    np.savez_compressed(os.path.join(out, "stage1.npz"), **cases)


def gen_stage2(mods, out):
    import oracle
    u = mods["utils"]
    cases = {}
    worst = 0.0
    for name, lens_q, lens_k, k_sel in (("a", [128], [128], 2), ("b", [200, 136], [200, 136], 2),
                                        ("c", [64, 192], [160, 300], 3)):
        hq, hk, d, bs = 32, 2, 128, 64
        seed = 200 + ord(name)
        bsz = len(lens_q)
        cu_q = np.concatenate([[0], np.cumsum(lens_q)]).astype(np.int32)
        cu_k = np.concatenate([[0], np.cumsum(lens_k)]).astype(np.int32)
        sq, sk = max(lens_q), max(lens_k)
        q = torch.from_numpy(det_array((int(cu_q[-1]), hq, d), seed, 0.25))
        k = torch.from_numpy(det_array((int(cu_k[-1]), hk, d), seed + 1000, 0.25))
        v = torch.from_numpy(det_array((int(cu_k[-1]), hk, d), seed + 2000))
        kb = (sk + bs - 1) // bs
        idx = torch.from_numpy(det_perm_rows(hk * int(cu_q[-1]), kb, k_sel, seed + 3000)).view(hk, -1, k_sel)
        # reference path: padded tensors + expanded token-level mask (True = masked out)
        base = u.convert_topk_to_base_blockmask(idx, sk, bs, device="cpu")
        mixed = u.prepare_mixed_mask(base, torch.from_numpy(cu_q), torch.from_numpy(cu_k), sq, sk, bsz,
                                     nheads=hq, nheads_k=hk, m_block_dim=1, n_block_dim=bs)
        qp = torch.zeros(bsz, sq, hq, d); kp = torch.zeros(bsz, sk, hk, d); vp = torch.zeros(bsz, sk, hk, d)
        qmask = torch.zeros(bsz, sq, dtype=torch.bool); kmask = torch.zeros(bsz, sk, dtype=torch.bool)
        for b in range(bsz):
            qp[b, :lens_q[b]] = q[cu_q[b]:cu_q[b + 1]]; qmask[b, :lens_q[b]] = True
            kp[b, :lens_k[b]] = k[cu_k[b]:cu_k[b + 1]]; kmask[b, :lens_k[b]] = True
            vp[b, :lens_k[b]] = v[cu_k[b]:cu_k[b + 1]]
        # the reference's mask has no causal term of its own when Lq != Lk; its attention_blocksparse_ref
        # applies a top-left window via construct_local_mask, so compare the non-causal form here and
        # the causal form only on Lq == Lk cases (where top-left == bottom-right).
        for causal in (False, True):
            if causal and any(a != b_ for a, b_ in zip(lens_q, lens_k)):
                continue
            ref, _ = u.attention_blocksparse_ref(qp, kp, vp, mixed, qmask, kmask, 0.0, None, causal=causal)
            ref = torch.where(torch.isnan(ref), torch.zeros(()), ref)
            ref_un = torch.cat([ref[b, :lens_q[b]] for b in range(bsz)], 0)
            got, _ = oracle.sparse_attention_fwd(q, k, v, cu_q, cu_k, idx, causal=causal)
            worst = max(worst, (got - ref_un).abs().max().item())
            cases[f"s2_{name}_{int(causal)}_out"] = ref_un[::OUT_ROW_STEP].numpy()
        cases[f"s2_{name}_seed"] = np.array([seed, k_sel], dtype=np.int64)
        cases[f"s2_{name}_cuq"] = cu_q; cases[f"s2_{name}_cuk"] = cu_k
    assert worst < 5e-6, worst
    print(f"stage2: oracle vs attention_blocksparse_ref max|diff| = {worst:.2e}")

    # decode (tests/test_kvcache_simple.py::naive_attention)
    naive = mods["test_kvcache_simple"].naive_attention
    bsz, hq, hk, d, cache = 2, 32, 2, 128, 300
    q = torch.from_numpy(det_array((bsz, hq, 1, d), 301, 0.25))
    kc = torch.from_numpy(det_array((bsz, hk, cache + 1, d), 302, 0.25))
    vc = torch.from_numpy(det_array((bsz, hk, cache + 1, d), 303))
    nb = (cache + 1 + 63) // 64
    idx = torch.from_numpy(det_perm_rows(bsz * hk, nb, 3, 304)).view(bsz, hk, 1, 3)
    bm = torch.zeros(bsz, hk, 1, cache + 1, dtype=torch.bool)
    for b in range(bsz):
        for h in range(hk):
            for i in idx[b, h, 0]:
                bm[b, h, 0, int(i) * 64:(int(i) + 1) * 64] = True
    bm = bm.repeat_interleave(hq // hk, dim=1)
    ref = naive(q, kc, vc, bm).transpose(1, 2)                       # (B, 1, Hq, d)
    got, _ = oracle.kvcache_decode(q.transpose(1, 2), kc.transpose(1, 2).contiguous(),
                                   vc.transpose(1, 2).contiguous(),
                                   torch.full((bsz,), cache + 1, dtype=torch.int32), idx)
    err = (got - ref).abs().max().item()
    assert err < 5e-6, err
    print(f"decode: oracle vs naive_attention max|diff| = {err:.2e}")
    cases.update(dec_shape=np.array([bsz, hq, hk, d, cache], dtype=np.int64),
                 dec_out=ref.numpy(), out_row_step=np.int64(OUT_ROW_STEP))
    # rotary helper: the vectorised oracle against the element-by-element restatement of the
    # reference's device loops (csrc/flash_attn/src/rotary.h:20-150), both layouts, rotary_dim < d
    for name, rows_, rd, inter in (("a", 6, 128, True), ("b", 5, 64, True), ("c", 6, 128, False), ("d", 5, 32, False)):
        x = torch.from_numpy(det_array((rows_, 128), 900 + ord(name))).to(torch.bfloat16)
        ang = torch.from_numpy(det_array((rows_, rd // 2), 950 + ord(name), 3.0))
        c, s_ = torch.cos(ang).to(torch.bfloat16), torch.sin(ang).to(torch.bfloat16)
        lit = oracle.apply_rotary_literal(x.float().numpy(), c.float().numpy(), s_.float().numpy(), inter)
        got = oracle.apply_rotary(x, c, s_, inter)
        want = torch.from_numpy(lit).to(torch.bfloat16)
        assert torch.equal(got.view(torch.int16), want.view(torch.int16)), f"rotary {name}"
        cases[f"rotary_{name}_cfg"] = np.array([rows_, rd, int(inter), 900 + ord(name), 950 + ord(name)], dtype=np.int64)
        cases[f"rotary_{name}_out"] = want.float().numpy()
    np.savez_compressed(os.path.join(out, "stage2.npz"), **cases)


def gen_pool_topk(out):
    import oracle
    from oracle.pooling import max_pooling_1d_literal
    rng = np.random.default_rng(1)
    cases = {}
    for name, hk, ql, kl, cache, local, init in (("a", 2, 70, 3, 0, 1, 1), ("b", 1, 130, 7, 64, 2, 1),
                                                 ("c", 2, 200, 11, 0, 0, 0), ("d", 1, 65, 2, 190, 3, 2)):
        x = torch.from_numpy(rng.random((hk, ql, kl)).astype(np.float32)).to(torch.bfloat16)
        lit = max_pooling_1d_literal(x.float().numpy(), cache, local, init)
        fast = oracle.max_pooling_1d(x, cache, local, init).float().numpy()
        assert np.array_equal(lit, fast), name
        cases[f"pool_{name}_x"] = x.float().numpy()
        cases[f"pool_{name}_args"] = np.array([cache, local, init], dtype=np.int64)
        cases[f"pool_{name}_y"] = lit
    # top-k KATs: ordering rule of csrc/topk.cuh:17 -> (value desc, index asc)
    y = torch.tensor([[[0, 1, 1, float("inf"), .5, 1, float("inf"), 0],
                       [3, 3, 3, 3, 3, 3, 3, 3],
                       [float("inf"), 0, 0, 0, 0, 0, float("inf"), float("inf")]]])
    exp5 = np.array([[[1, 2, 3, 5, 6], [0, 1, 2, 3, 4], [0, 1, 2, 6, 7]]], dtype=np.int32)
    got = oracle.topk_select(y, 5, torch.tensor([7, 7, 7])).numpy()
    assert np.array_equal(got, exp5), got
    got2 = oracle.topk_select(y, 5, torch.tensor([7, 2, 6])).numpy()
    exp2 = np.array([[[1, 2, 3, 5, 6], [0, 1, 2, -1, -1], [0, 1, 2, 6, -1]]], dtype=np.int32)
    assert np.array_equal(got2, exp2), got2
    cases.update(topk_y=y.numpy(), topk_exp_all=exp5, topk_exp_cut=exp2,
                 topk_bq_cut=np.array([7, 2, 6]))
    # top-k pin: the reference's own bitonic kernel (csrc/topk.cuh), simulated thread for thread,
    # on tie-heavy rows with +-inf; the oracle must pick the same blocks in the same order
    from oracle.topk import bitonic_topk_literal
    for name, n, top in (("a", 1024, 32), ("b", 256, 16), ("c", 96, 8), ("d", 160, 5), ("e", 64, 1),
                         ("f", 512, 17), ("g", 32, 32)):
        x = rng.integers(0, 4, size=(12, n)).astype(np.float32)
        x[rng.random((12, n)) < 0.04] = np.inf
        # -inf only where it cannot reach the top (a padded thread of the kernel holds
        # (-inf, position -1), which would win a tie against a real -inf)
        low = rng.random((12, n)) < 0.04
        low[:, :40 if n >= 64 else 0] = False
        x[low & (np.arange(n)[None, :] >= 32)] = -np.inf
        x[0] = 1.0                                                  # a row of all-equal scores
        x[1, : n // 2] = np.inf                                     # more +inf than selected
        val, pos = bitonic_topk_literal(x, top)
        n_sel = pos.shape[1]
        assert np.isfinite(val).any() and (val > -np.inf).all(), name
        xt = torch.from_numpy(x)
        order = torch.sort(xt, dim=-1, descending=True, stable=True).indices[:, :n_sel].numpy()
        assert np.array_equal(pos, order), f"top-k order differs from the reference kernel ({name})"
        sel = oracle.topk_select(xt[None].to(torch.bfloat16), n_sel, torch.full((12,), n))[0].numpy()
        assert np.array_equal(np.sort(pos, axis=1), sel), f"top-k set differs from the reference kernel ({name})"
        cases[f"bitonic_{name}_x"] = x.astype(np.float16)            # values 0..3 and +-inf: exact
        cases[f"bitonic_{name}_pos"] = pos.astype(np.int32)
    np.savez_compressed(os.path.join(out, "pool_topk.npz"), **cases)
    print("pool/topk: fast forms == literal transliterations / hand KATs; top-k == the reference's "
          "bitonic kernel simulated thread for thread")


def gen_compress(mods, out):
    """Key compression (mean over token windows): the reference's test helper on bf16 inputs,
    packed sequences of ragged lengths, both window shapes."""
    import oracle
    ref_fn = mods["test_stage1_compressed_lse"].compress_tensor
    cases = {}
    for name, lens, kernel, stride in (("a", [64], 32, 16), ("b", [31, 32, 33, 100], 32, 16),
                                       ("c", [300, 5, 257], 128, 64), ("d", [47, 48, 49], 32, 16),
                                       ("e", [10, 20], 32, 16)):
        seed = 700 + ord(name)
        total, hk = sum(lens), 2
        k = torch.from_numpy(det_array((total, hk, 128), seed)).to(torch.bfloat16)
        cu = torch.tensor(np.concatenate([[0], np.cumsum(lens)]), dtype=torch.int32)
        ref, cu_ref = ref_fn(k.transpose(0, 1).contiguous(), cu, kernel, stride, hk, 128)
        ref = ref.transpose(0, 1).contiguous()                     # (total_c, hk, 128)
        got, cu_c = oracle.compress_keys(k, cu.tolist(), kernel, stride)
        assert list(cu_ref.tolist()) == cu_c, (cu_ref, cu_c)
        assert ref.shape == got.shape and torch.equal(ref.view(torch.int16), got.view(torch.int16)), name
        cases[f"ck_{name}_lens"] = np.array(lens, dtype=np.int64)
        cases[f"ck_{name}_cfg"] = np.array([kernel, stride, seed, hk], dtype=np.int64)
        cases[f"ck_{name}_cu_c"] = np.array(cu_c, dtype=np.int64)
        cases[f"ck_{name}_out"] = ref.float().numpy()
    print("compress: oracle == reference compress_tensor bit for bit")
    np.savez_compressed(os.path.join(out, "compress.npz"), **cases)


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", default=os.environ.get("INFLLMV2_REFERENCE"), required="INFLLMV2_REFERENCE" not in os.environ,
                    help="checkout of OpenBMB/infllmv2_cuda_impl (or set INFLLMV2_REFERENCE)")
    args = ap.parse_args()
    torch.set_num_threads(8)
    mods = _import_reference(args.reference)
    gen_bitmask(mods, HERE)
    gen_stage1(mods, HERE)
    gen_stage2(mods, HERE)
    gen_pool_topk(HERE)
    gen_compress(mods, HERE)
    print("golden fixtures written to", HERE)
