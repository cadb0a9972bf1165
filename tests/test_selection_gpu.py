"""GPU: max-pool and top-k kernels, bit-exact against the oracle."""
import os

import numpy as np
import pytest
import torch

import oracle
import infllm_v2

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _scores(shape, seed, dtype=torch.bfloat16):
    g = torch.Generator().manual_seed(seed)
    return torch.rand(shape, generator=g).to(dtype)


def test_pool_golden(golden_dir):
    g = np.load(os.path.join(golden_dir, "pool_topk.npz"))
    for name in ("a", "b", "c", "d"):
        x = torch.from_numpy(g[f"pool_{name}_x"]).to(torch.bfloat16)
        cache, local, init = (int(v) for v in g[f"pool_{name}_args"])
        y = infllm_v2.max_pooling_1d(x.to(DEV), cache, local, init)
        assert np.array_equal(y.float().cpu().numpy(), g[f"pool_{name}_y"]), name


@pytest.mark.parametrize("hk,ql,kl,cache,local,init,dtype", [
    (2, 256, 15, 0, 2, 1, torch.bfloat16), (2, 1000, 61, 0, 32, 1, torch.bfloat16),
    (1, 333, 255, 4096, 2, 1, torch.float16), (2, 64, 2047, 32704, 32, 1, torch.bfloat16),
    (1, 70, 3, 0, 0, 0, torch.bfloat16), (3, 129, 8, 1, 1, 2, torch.bfloat16),
])
def test_pool_random(hk, ql, kl, cache, local, init, dtype):
    x = _scores((hk, ql, kl), ql + kl, dtype)
    exp = oracle.max_pooling_1d(x, cache, local, init)
    got = infllm_v2.max_pooling_1d(x.to(DEV), cache, local, init)
    assert got.dtype == dtype and torch.equal(got.cpu(), exp)


def test_pool_strided_view_fast_path():
    # a column slice of a padded buffer (what stage 1 returns) takes the vector path, no copy
    buf = _scores((2, 300, 128), 11)
    x = buf[:, :, :61]
    exp = oracle.max_pooling_1d(x.contiguous(), 0, 2, 1)
    got = infllm_v2.max_pooling_1d(buf.to(DEV)[:, :, :61], 0, 2, 1)
    assert torch.equal(got.cpu(), exp)


def test_pool_varlen():
    lens_q, lens_c, cl = [100, 37, 200], [5, 1, 11], [0, 64, 130]
    x = _scores((2, sum(lens_q), 11), 3)
    cu_q = torch.tensor(np.concatenate([[0], np.cumsum(lens_q)]), dtype=torch.int32)
    cu_k = torch.tensor(np.concatenate([[0], np.cumsum(lens_c)]), dtype=torch.int32)
    cache = torch.tensor(cl, dtype=torch.int32)
    exp = oracle.max_pooling_1d_varlen(x, cu_q, cu_k, cache, 200, 11, 2, 1)
    got = infllm_v2.max_pooling_1d_varlen(x.to(DEV), cu_q.to(DEV), cu_k.to(DEV), cache.to(DEV),
                                          200, 11, 2, 1)
    assert torch.equal(got.cpu(), exp)


def test_topk_equals_reference_bitonic_kernel(golden_dir):
    """Tie-heavy rows with +-inf whose expected selection was produced by a thread-for-thread
    simulation of the reference's bitonic top-k kernel (csrc/topk.cuh), see make_golden.py."""
    g = np.load(os.path.join(golden_dir, "pool_topk.npz"))
    names = sorted(k[len("bitonic_"):-2] for k in g.files if k.startswith("bitonic_") and k.endswith("_x"))
    assert len(names) >= 6
    for name in names:
        x = torch.from_numpy(g[f"bitonic_{name}_x"].astype(np.float32))
        pos = g[f"bitonic_{name}_pos"]
        n, k = x.shape[1], pos.shape[1]
        got = infllm_v2.infllmv2_topk(x[None].to(torch.bfloat16).to(DEV), k, cache_len=64 * n)
        assert np.array_equal(got[0].cpu().numpy(), np.sort(pos, axis=1)), name


def test_topk_kats(golden_dir):
    g = np.load(os.path.join(golden_dir, "pool_topk.npz"))
    y = torch.from_numpy(g["topk_y"]).to(torch.bfloat16).to(DEV)          # (1, 3, 8)
    # rows are tokens 0..2; pick cache_len so that every index stays visible
    got = infllm_v2.infllmv2_topk(y, 5, cache_len=7 * 64)
    assert np.array_equal(got.cpu().numpy(), g["topk_exp_all"])


@pytest.mark.parametrize("hk,t,n,k,dtype", [
    (2, 300, 512, 64, torch.bfloat16), (2, 130, 2048, 64, torch.bfloat16), (1, 70, 40, 64, torch.bfloat16),
    (2, 100, 384, 16, torch.float16), (1, 64, 2049, 64, torch.bfloat16), (1, 33, 4100, 64, torch.bfloat16),
    (2, 200, 100, 1, torch.bfloat16), (1, 50, 257, 64, torch.bfloat16),
])
def test_topk_random_with_ties(hk, t, n, k, dtype):
    g = torch.Generator().manual_seed(n + k)
    # few distinct values -> many ties, plus forced +inf entries and -inf tails
    y = (torch.randint(0, 12, (hk, t, n), generator=g).float() / 8).to(dtype)
    y[:, :, 0] = float("inf")
    y[:, : t // 2, n // 2:] = float("-inf")
    y[:, 1::3, 3:9] = float("inf")
    q_block = (torch.arange(t) + 64 * (n - 1)) // 64          # nothing is in the future
    exp = oracle.topk_select(y, k, q_block)
    got = infllm_v2.infllmv2_topk(y.to(DEV), k, cache_len=64 * (n - 1))
    assert got.dtype == torch.int32 and torch.equal(got.cpu(), exp)


def test_topk_future_blocks_and_varlen():
    lens = [130, 64, 200]
    t = sum(lens)
    y = _scores((2, t, 8), 9)
    cu = torch.tensor(np.concatenate([[0], np.cumsum(lens)]), dtype=torch.int32)
    cl = torch.tensor([0, 128, 64], dtype=torch.int32)
    qb = torch.cat([(torch.arange(l) + int(c)) // 64 for l, c in zip(lens, cl)])
    exp = oracle.topk_select(y, 4, qb)
    got = infllm_v2.infllmv2_topk(y.to(DEV), 4, cu_seqlens_q=cu.to(DEV), cache_lens=cl.to(DEV))
    assert torch.equal(got.cpu(), exp)
    # pool -> topk composition on the forced-block pattern: block 0 and the local blocks always win
    x = _scores((2, 640, 39), 10)
    pooled = infllm_v2.max_pooling_1d(x.to(DEV), 0, 2, 1)
    sel = infllm_v2.infllmv2_topk(pooled, 6).cpu()
    for tok in (0, 63, 64, 300, 639):
        bq = tok // 64
        forced = {0} | {b for b in range(max(bq - 2, 0), bq + 1)}
        assert forced <= set(sel[0, tok].tolist()) and sel[0, tok].max() <= bq


@pytest.mark.parametrize("tail", ["random", "zero", "neg_inf"])
@pytest.mark.parametrize("t,n,k", [(700, 600, 64), (520, 2048, 64), (300, 40, 16)])
def test_topk_causal_restriction(t, n, k, tail):
    """Entries past the query's own block: arbitrary values there must displace earlier entries
    exactly as a full-width selection would (and come out as -1); the stage-1 pattern (0 / -inf
    there) must give the same lists as selecting among the visible blocks only."""
    g = torch.Generator().manual_seed(t + n + k)
    y = (torch.randint(0, 40, (2, t, n), generator=g).float() / 16).to(torch.bfloat16)
    y[:, :, 0] = float("inf")
    q_block = torch.arange(t) // 64
    if tail != "random":
        future = torch.arange(n)[None, :] > q_block[:, None]                 # (t, n)
        y[:, future] = 0.0 if tail == "zero" else float("-inf")
    exp = oracle.topk_select(y, k, q_block)
    got = infllm_v2.infllmv2_topk(y.to(DEV), k)
    assert torch.equal(got.cpu(), exp)


def _guarded(x, guard_value, guard_elems=4096):
    """x copied into the middle of a larger device buffer whose elements before and after it hold
    `guard_value`: a kernel that reads outside its input then computes a wrong result instead of
    faulting.  Returns the view of x inside the buffer."""
    buf = torch.full((x.numel() + 2 * guard_elems,), guard_value, dtype=x.dtype, device=DEV)
    view = buf[guard_elems:guard_elems + x.numel()].view(x.shape)
    view.copy_(x)
    return view


@pytest.mark.parametrize("guard", [float("inf"), float("nan")])
def test_neither_kernel_reads_outside_its_input(guard):
    """Block scores of unaligned width (5 columns: rows start at odd 2-byte offsets, and the lanes
    of a warp that own no element of such a row must not load anything) and scores whose first
    row has no element in front of it (max-pool: the halo of block 0).  The input sits between
    guard regions of +inf / NaN, so a read outside it changes the selected blocks or the pooled
    maxima and the comparison with the oracle fails."""
    hk, t, n, k = 4, 307, 5, 1
    x = _scores((hk, t, n), 77)
    x[:, :, 0] = float("inf")
    cu_q = torch.tensor([0, 7, t], dtype=torch.int32, device=DEV)
    got = infllm_v2.infllmv2_topk(_guarded(x, guard), k, cu_seqlens_q=cu_q)
    qb = torch.cat([torch.arange(7) // 64, torch.arange(t - 7) // 64])
    assert torch.equal(got.cpu(), oracle.topk_select(x.float(), k, qb))
    # three selected of five columns: a stray +inf / NaN read past a row's end would displace one
    got3 = infllm_v2.infllmv2_topk(_guarded(x[-1:, -3:].contiguous(), guard), 3, cache_len=64 * n)
    assert torch.equal(got3.cpu(), oracle.topk_select(x[-1:, -3:].float(), 3, torch.full((3,), n)))

    s = _scores((2, 200, 24), 78)
    view = _guarded(s, guard)
    pooled = infllm_v2.max_pooling_1d(view[:, :, :21], 0, 2, 0)          # no forced first block
    assert torch.equal(pooled.cpu(), oracle.max_pooling_1d(s[:, :, :21], 0, 2, 0))
    pooled = infllm_v2.max_pooling_1d(view, 0, 0, 0)
    assert torch.equal(pooled.cpu(), oracle.max_pooling_1d(s, 0, 0, 0))


@pytest.mark.parametrize("hk,b,cap,k,local,init,dtype", [
    (2, 5, 4096, 8, 2, 1, torch.bfloat16), (1, 3, 131072, 64, 32, 1, torch.bfloat16),
    (4, 6, 1000, 16, 0, 0, torch.float16), (2, 4, 64 * 70, 96, 1, 2, torch.bfloat16),
])
def test_decode_select_equals_pool_topk_pack(hk, b, cap, k, local, init, dtype):
    """One launch against the three kernels it replaces, bit for bit: ragged lengths (one
    sequence shorter than a compression window, one at the capacity), heavy ties."""
    rng = np.random.default_rng(cap + k)
    lens = rng.integers(40, cap + 1, size=b)
    lens[0], lens[-1] = 20, cap
    n_c = np.where(lens >= 32, (lens - 32) // 16 + 1, 0).astype(np.int32)
    max_c = int(n_c.max())
    g = torch.Generator().manual_seed(int(cap))
    score = (torch.randint(0, 12, (hk, b, max_c), generator=g).float() / 8).to(dtype)     # many equal values
    for i in range(b):
        score[:, i, n_c[i]:] = 0
    score = score.to(DEV)
    if k % 16 == 0:        # rows padded to 128 scores, as the scorer writes them (staged in shared memory)
        buf = torch.full((hk, b, (max_c + 127) // 128 * 128), float("nan"), dtype=dtype, device=DEV)
        buf[:, :, :max_c] = score
        score = buf[:, :, :max_c]
    positions = torch.tensor(lens - 1, dtype=torch.int32, device=DEV)
    used = torch.tensor(n_c, device=DEV)
    mask, idx = infllm_v2.decode_select(score, positions, k, cap, local, init, seqused_c=used, return_topk=True)
    cu_q = torch.arange(b + 1, dtype=torch.int32, device=DEV)
    cu_c = torch.tensor(np.concatenate([[0], np.cumsum(n_c)]), dtype=torch.int32, device=DEV)
    pooled = infllm_v2.max_pooling_1d_varlen(score, cu_q, cu_c, positions, 1, max_c, local, init,
                                             max_cache_len=cap - 1)
    assert pooled.shape[-1] == (cap + 63) // 64
    ref_idx = infllm_v2.infllmv2_topk(pooled, k, cu_seqlens_q=cu_q, cache_lens=positions)
    ref_idx = ref_idx.permute(1, 0, 2).unsqueeze(2).contiguous()
    ref_mask, _ = infllm_v2.topk_to_uint64(ref_idx, cap, 64)
    assert torch.equal(idx, ref_idx)
    assert torch.equal(mask, ref_mask)
    # and against the oracle for one row
    exp = oracle.topk_select(oracle.max_pooling_1d_varlen(score.cpu(), cu_q.tolist(), cu_c.tolist(), (lens - 1).tolist(),
                                                          1, max_c, local, init).float(), k,
                             torch.tensor((lens - 1) // 64))
    assert torch.equal(idx[:, :, 0].cpu().permute(1, 0, 2), exp)


@pytest.mark.parametrize("hk,t,n,k,max_k,dtype", [
    (2, 300, 512, 64, 512 * 64, torch.bfloat16), (2, 130, 2048, 64, 2048 * 64, torch.bfloat16),
    (1, 70, 40, 64, 40 * 64, torch.bfloat16), (2, 100, 384, 16, 384 * 64 - 5, torch.float16),
    (1, 64, 2049, 64, 2049 * 64, torch.bfloat16), (1, 33, 4100, 64, 4100 * 64, torch.bfloat16),
    (2, 200, 100, 1, 100 * 64, torch.bfloat16), (1, 50, 257, 64, 300 * 64, torch.bfloat16),
    (1, 40, 200, 8, 130 * 64, torch.bfloat16),
])
def test_topk_mask_equals_topk_then_pack_then_transpose(hk, t, n, k, max_k, dtype):
    """The fused entry (top-k straight to the packed row mask, column mask in the same call) against
    the three separate operators, on tie-heavy scores, with the mask narrower / wider than the
    score rows and queries whose later blocks are cut off."""
    g = torch.Generator().manual_seed(n + k)
    y = (torch.randint(0, 12, (hk, t, n), generator=g).float() / 8).to(dtype)
    y[:, :, 0] = float("inf")
    y[:, : t // 2, n // 2:] = float("-inf")
    y[:, 1::3, 3:9] = float("inf")
    yd = y.to(DEV)
    for cache_len in (64 * (n - 1), 64 * (n // 3)):            # nothing cut off / most blocks cut off
        idx = infllm_v2.infllmv2_topk(yd, k, cache_len=cache_len)
        words, kb = infllm_v2.topk_to_uint64(idx, max_k, 64)
        col = infllm_v2.transpose_blockmask(words, kb)
        mask, kb2, idx2, col2 = infllm_v2.infllmv2_topk_mask(yd, k, max_k, cache_len=cache_len, return_idx=True,
                                                            return_col_mask=True)
        assert kb2 == kb and torch.equal(idx2, idx)
        assert torch.equal(mask, words)
        assert torch.equal(col2, col)
        only_mask, _ = infllm_v2.infllmv2_topk_mask(yd, k, max_k, cache_len=cache_len)
        assert torch.equal(only_mask, words)


def test_topk_mask_varlen_and_attention_takes_the_mask():
    lens = [130, 64, 200]
    t = sum(lens)
    y = _scores((2, t, 8), 9).to(DEV)
    cu = torch.tensor(np.concatenate([[0], np.cumsum(lens)]), dtype=torch.int32, device=DEV)
    cl = torch.tensor([0, 128, 64], dtype=torch.int32, device=DEV)
    idx = infllm_v2.infllmv2_topk(y, 4, cu_seqlens_q=cu, cache_lens=cl)
    words, kb = infllm_v2.topk_to_uint64(idx, 8 * 64, 64)
    mask, kb2 = infllm_v2.infllmv2_topk_mask(y, 4, 8 * 64, cu_seqlens_q=cu, cache_lens=cl)
    assert kb == kb2 and torch.equal(mask, words)
    # the attention accepts the packed mask in place of the list, same result bit for bit
    from helpers import det_tensor
    L = 512
    q = det_tensor((L, 32, 128), 1, 0.25).to(DEV)
    k = det_tensor((L, 2, 128), 2, 0.25).to(DEV)
    v = det_tensor((L, 2, 128), 3).to(DEV)
    sc = _scores((2, L, 8), 11).to(DEV)
    cu1 = torch.tensor([0, L], dtype=torch.int32, device=DEV)
    idx = infllm_v2.infllmv2_topk(sc, 3)
    m, _ = infllm_v2.infllmv2_topk_mask(sc, 3, L)
    a = infllm_v2.infllmv2_attn_varlen_func(q, k, v, cu1, cu1, L, L, causal=True, topk_idx=idx)
    b = infllm_v2.infllmv2_attn_varlen_func(q, k, v, cu1, cu1, L, L, causal=True, block_mask=m)
    assert torch.equal(a, b)
