"""CPU: the multi-GPU host logic (KV-head / batch partition, zig-zag query chunks, all-gather and
re-ordering, per-chunk call geometry) with world_size-2 gloo ranks.  The chunk pipeline runs on the
CPU oracle here, and the sharded result must equal the unsharded oracle on the whole sequence."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

import oracle
from infllmv2_cuda_impl_b200 import sharding

L, HQ, HK, D, TOPK, INIT, LOCAL = 512, 16, 1, 32, 4, 1, 1


def _oracle_ops():
    def stage1(q, kc, _v, cu_q, cu_c, _cu_v, lq, n_comp, causal=True):
        return oracle.stage1_scores(q, kc, cu_q, cu_c, n_comp, causal).to(torch.bfloat16)

    def max_pool(score, cache_len, local_blocks, init_blocks, block_size, stride):
        return oracle.max_pooling_1d(score, cache_len, local_blocks, init_blocks, block_size, stride)

    def topk(pooled, k, cache_len):
        t = pooled.shape[1]
        return oracle.topk_select(pooled, k, (torch.arange(t) + cache_len) // 64)

    def attn(q, k, v, cu_q, cu_k, lq, lk, causal=True, topk_idx=None):
        return oracle.sparse_attention_fwd(q, k, v, cu_q, cu_k, topk_idx, causal=causal)[0]

    return sharding.PrefillOps(stage1, max_pool, topk, attn)


def _inputs():
    g = torch.Generator().manual_seed(0)
    q = (torch.randn(L, HQ, D, generator=g) * 0.5).to(torch.bfloat16)
    k = (torch.randn(L, HK, D, generator=g) * 0.5).to(torch.bfloat16)
    v = torch.randn(L, HK, D, generator=g).to(torch.bfloat16)
    kc, cu_c = oracle.compress_keys(k, [0, L])
    return q, k, v, kc


def _worker(rank, world, port, result_dir):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        q, k, v, kc = _inputs()
        chunks = sharding.zigzag_chunks(L, world, rank)
        rows = torch.cat([torch.arange(c.start, c.end) for c in chunks])
        kc_pad = torch.cat([kc, kc.new_zeros((L // 16 - kc.shape[0],) + kc.shape[1:])])   # slot L/16-1 is padding
        kc_rows = torch.cat([torch.arange(*sharding.compressed_range(c)) for c in chunks])
        out = sharding.sharded_prefill(q[rows], k[rows], v[rows], kc_pad[kc_rows], L, world, rank, TOPK,
                                       INIT, LOCAL, ops=_oracle_ops())
        torch.save({"rows": rows, "out": out}, os.path.join(result_dir, f"r{rank}.pt"))
    finally:
        dist.destroy_process_group()


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def test_partitions():
    assert sharding.head_shard(8, 4, 3) == slice(6, 8)
    with pytest.raises(ValueError):
        sharding.head_shard(8, 3, 0)
    got = [list(sharding.batch_shard(10, 4, r)) for r in range(4)]
    assert sum(got, []) == list(range(10)) and max(map(len, got)) - min(map(len, got)) <= 1
    ch = [sharding.zigzag_chunks(1024, 4, r) for r in range(4)]
    idx = sorted(c.index for pair in ch for c in pair)
    assert idx == list(range(8)) and all(c.end - c.start == 128 for pair in ch for c in pair)
    assert [c.index for c in ch[1]] == [1, 6]
    with pytest.raises(ValueError):
        sharding.zigzag_chunks(1000, 4, 0)


def test_query_chunk_prefill_world2_matches_unsharded(tmp_path):
    world = 2
    mp.spawn(_worker, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    q, k, v, kc = _inputs()
    ops = _oracle_ops()
    full_out, full_idx = sharding.prefill_chunk(q, kc, k, v, sharding.Chunk(0, 0, L), TOPK, INIT, LOCAL, ops)
    seen = torch.zeros(L, dtype=torch.bool)
    for r in range(world):
        res = torch.load(os.path.join(str(tmp_path), f"r{r}.pt"))
        assert (res["out"] - full_out[res["rows"]]).abs().max() < 1e-5
        seen[res["rows"]] = True
    assert bool(seen.all())


def _bwd_worker(rank, world, port, result_dir):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        q, k, v, kc = _inputs()
        dout = torch.randn(L, HQ, D, generator=torch.Generator().manual_seed(1))
        idx = _full_topk(q, k, v, kc)
        rows = torch.cat([torch.arange(c.start, c.end) for c in sharding.zigzag_chunks(L, world, rank)])

        def attn(qc, kk, vv, cu_q, cu_k, lq, lk, causal=True, topk_idx=None):
            return oracle.sparse_attention_fwd(qc, kk, vv, cu_q, cu_k, topk_idx, causal=causal)[0]

        out, dq, dk, dv = sharding.sharded_attention_fwd_bwd(
            q[rows].float(), k[rows].float(), v[rows].float(), dout[rows], idx[:, rows], L, world, rank,
            attn=attn)
        torch.save({"rows": rows, "out": out, "dq": dq, "dk": dk, "dv": dv},
                   os.path.join(result_dir, f"b{rank}.pt"))
    finally:
        dist.destroy_process_group()


def _full_topk(q, k, v, kc):
    return sharding.prefill_chunk(q, kc, k, v, sharding.Chunk(0, 0, L), TOPK, INIT, LOCAL, _oracle_ops())[1]


def test_query_chunk_backward_world2_matches_unsharded(tmp_path):
    """Forward + backward under query-chunk sharding (all-gather of K/V, per-chunk backward,
    summed and re-scattered dK/dV) against the unsharded oracle gradients."""
    world = 2
    mp.spawn(_bwd_worker, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    q, k, v, kc = _inputs()
    dout = torch.randn(L, HQ, D, generator=torch.Generator().manual_seed(1))
    idx = _full_topk(q, k, v, kc)
    out, _, dq, dk, dv = oracle.sparse_attention_fwd_bwd(q, k, v, dout, [0, L], [0, L], idx)
    for r in range(world):
        res = torch.load(os.path.join(str(tmp_path), f"b{r}.pt"))
        rows = res["rows"]
        for name, ref in (("out", out), ("dq", dq), ("dk", dk), ("dv", dv)):
            assert (res[name] - ref[rows]).abs().max() < 1e-4, (name, r)
