"""GPU: the operators chained as a caller chains them (stage 1 -> pool -> top-k -> stage 2), each
stage checked against the oracle on the previous stage's ACTUAL output, and a query chunk of a
longer sequence against the same tokens of the full run."""
import numpy as np
import pytest
import torch

import oracle
import infllm_v2
from infllmv2_cuda_impl_b200 import sharding
from helpers import det_tensor, cu, err_stats

pytestmark = pytest.mark.gpu
DEV = "cuda"


def test_pipeline_config1_shape():
    # BASELINE config 1 shapes (4096 tokens, 32q/2kv, top-16, 1 init + 2 local), bf16 on the GPU
    L, hq, hk, d, topk = 4096, 32, 2, 128, 16
    g = torch.Generator().manual_seed(0)
    q = (torch.randn(L, hq, d, generator=g) / d ** 0.5 * 4).to(torch.bfloat16)
    k = (torch.randn(L, hk, d, generator=g) / d ** 0.5 * 4).to(torch.bfloat16)
    v = torch.randn(L, hk, d, generator=g).to(torch.bfloat16)
    kc, cu_c = oracle.compress_keys(k, [0, L])
    cu_q, cu_ct = cu([L]), torch.tensor(cu_c, dtype=torch.int32)
    score = infllm_v2.infllmv2_attn_stage1(q.to(DEV), kc.to(DEV), kc.to(DEV), cu_q.to(DEV), cu_ct.to(DEV),
                                           cu_ct.to(DEV), L, cu_c[-1], causal=True)
    ref = oracle.stage1_scores(q, kc, cu_q, cu_ct, cu_c[-1], True)
    diff = (score.float().cpu() - ref).abs()
    assert bool(((diff <= 2e-2) | (diff <= 2.0 ** -7 * ref.abs())).all())
    pooled = infllm_v2.max_pooling_1d(score, 0, 2, 1)
    assert torch.equal(pooled.cpu(), oracle.max_pooling_1d(score.cpu(), 0, 2, 1))
    idx = infllm_v2.infllmv2_topk(pooled, topk)
    assert torch.equal(idx.cpu(), oracle.topk_select(pooled.cpu(), topk, torch.arange(L) // 64))
    out = infllm_v2.infllmv2_attn_varlen_func(q.to(DEV), k.to(DEV), v.to(DEV), cu_q.to(DEV), cu_q.to(DEV),
                                              L, L, causal=True, topk_idx=idx)
    infllm_v2.check_device_status()
    sl = slice(L - 256, L)
    ref_out, _ = oracle.sparse_attention_fwd(q, k, v, cu_q, cu_q, idx.cpu(), causal=True)
    mx, mr = err_stats(out.cpu()[sl], ref_out[sl])
    assert mx <= 2e-2 and mr <= 1e-2, (mx, mr)


def test_query_chunk_equals_full_run():
    L, hq, hk, d, topk = 2048, 32, 2, 128, 8
    q = det_tensor((L, hq, d), 1, 0.5).to(DEV)
    k = det_tensor((L, hk, d), 2, 0.5).to(DEV)
    v = det_tensor((L, hk, d), 3).to(DEV)
    kc, _ = oracle.compress_keys(k.cpu(), [0, L])
    kc = kc.to(DEV)
    full_out, full_idx = sharding.prefill_chunk(q, kc, k, v, sharding.Chunk(0, 0, L), topk, 1, 2)
    for ch in sharding.zigzag_chunks(L, 2, 1):                    # chunks 1 and 2 of 4
        out, idx = sharding.prefill_chunk(q[ch.start:ch.end], kc, k, v, ch, topk, 1, 2)
        infllm_v2.check_device_status()
        same = (idx == full_idx[:, ch.start:ch.end]).all(dim=-1).float().mean().item()
        assert same > 0.98, same            # bf16 scores differ only through accumulation order
        rows = (idx == full_idx[:, ch.start:ch.end]).all(dim=-1).all(dim=0)
        err = (out.float() - full_out[ch.start:ch.end].float()).abs()[rows].max().item()
        assert err <= 2e-2, err


def test_streamed_prefill_from_host_equals_resident_run():
    L, hq, hk, d, topk = 2048, 32, 2, 128, 8
    q = det_tensor((L, hq, d), 11, 0.5).pin_memory()
    k = det_tensor((L, hk, d), 12, 0.5).pin_memory()
    v = det_tensor((L, hk, d), 13).pin_memory()
    kc = oracle.compress_keys(k, [0, L])[0].pin_memory()
    out_host = torch.empty_like(q).pin_memory()
    runner = sharding.StreamedPrefill(L, hq, hk, d, kc.shape[0], DEV, chunk_tokens=512)
    for _ in range(2):                                   # second call reuses the device buffers
        runner(q, k, v, kc, out_host, topk, 1, 2)
        torch.cuda.synchronize()
    infllm_v2.check_device_status()
    outs = [sharding.prefill_chunk(q.to(DEV)[s:s + 512], kc.to(DEV), k.to(DEV), v.to(DEV),
                                   sharding.Chunk(i, s, s + 512), topk, 1, 2)[0]
            for i, s in enumerate(range(0, L, 512))]
    assert torch.equal(out_host, torch.cat(outs).cpu())
