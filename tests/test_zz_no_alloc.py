"""GPU: the allocation-free backward entry point against the regular one.

Some hosts of this library cannot allocate device memory when they call it: an inference or
training engine that handed all of HBM to its own pools at start-up has nothing left for
cudaMalloc, and cudaMalloc/cudaFree stall every stream of the device.  For them
`ifv2_sparse_attn_bwd_noalloc` keeps its scratch in an array inside the library.  This test
drives both entry points through the C ABI on the same inputs, twice in a row (the second call
reuses whatever the first left in the shared scratch; a second, different problem runs in
between so that stale scratch rows would show), and expects the same gradients bit for bit:
both entry points run the same deterministic kernels, only the scratch address differs.  With
more than one GPU the same is repeated on the second device, whose scratch address is looked up
separately.  It lives in a file pytest collects last so that a run that stops at the first
failure has already been through every other test.
"""
import pytest
import torch

import infllm_v2
from infllmv2_cuda_impl_b200 import _lib, attention
from helpers import det_tensor, cu, local_topk

pytestmark = pytest.mark.gpu


def _bwd_call(name, extra, t, masks, cu_q, cu_k, sizes, status):
    dq, dk, dv = torch.empty_like(t["q"]), torch.empty_like(t["k"]), torch.empty_like(t["v"])
    fwd_mask, bwd_mask = masks
    batch, total_q, total_k, hq, hk, d, max_q, max_k = sizes
    args = [t["do"].data_ptr(), t["q"].data_ptr(), t["k"].data_ptr(), t["v"].data_ptr(),
            t["out"].data_ptr(), t["lse"].data_ptr(), dq.data_ptr(), dk.data_ptr(), dv.data_ptr(),
            fwd_mask.data_ptr(), fwd_mask.shape[-1], bwd_mask.data_ptr(), bwd_mask.shape[-1],
            cu_q.data_ptr(), cu_k.data_ptr(), batch, total_q, total_k, hq, hk, d, max_q, max_k,
            float(d ** -0.5), 1] + extra + [status.data_ptr(), torch.cuda.current_stream().cuda_stream]
    _lib.call(name, *args)
    return dq, dk, dv


def _problem(dev, lens_q, lens_k, seed):
    hk, d = 2, 128
    hq = hk * 16
    t = {"q": det_tensor((sum(lens_q), hq, d), seed, 0.25).to(dev),
         "k": det_tensor((sum(lens_k), hk, d), seed + 1, 0.25).to(dev),
         "v": det_tensor((sum(lens_k), hk, d), seed + 2).to(dev),
         "do": det_tensor((sum(lens_q), hq, d), seed + 3, 0.5).to(dev)}
    cu_q, cu_k = cu(lens_q, dev), cu(lens_k, dev)
    idx = local_topk(hk, lens_q, lens_k, 3, seed + 6).to(dev)
    max_q, max_k = max(lens_q), max(lens_k)
    t["out"], t["lse"], _ = infllm_v2.infllmv2_attn_varlen_func(
        t["q"], t["k"], t["v"], cu_q, cu_k, max_q, max_k, causal=True, topk_idx=idx,
        return_attn_probs=True)
    fwd_mask, k_blocks = infllm_v2.topk_to_uint64(idx, max_k, 64)
    bwd_mask = infllm_v2.transpose_blockmask(fwd_mask, k_blocks)
    sizes = (len(lens_q), sum(lens_q), sum(lens_k), hq, hk, d, max_q, max_k)
    return t, (fwd_mask, bwd_mask), cu_q, cu_k, sizes


def _check_device(dev):
    with torch.cuda.device(dev):
        first = _problem(dev, [200, 136], [200, 136], 1)
        other = _problem(dev, [90, 300], [90, 300], 11)
        status = torch.zeros(4, dtype=torch.int32, device=dev)
        lib = _lib.load()
        refs = []
        for prob in (first, other):
            ws_bytes = int(lib.ifv2_sparse_attn_bwd_workspace_bytes(prob[4][1], prob[4][3], 128))
            ws = torch.empty(ws_bytes, dtype=torch.uint8, device=dev)
            refs.append(_bwd_call("ifv2_sparse_attn_bwd", [ws.data_ptr(), ws_bytes], *prob, status))
        # first problem, the other one (it overwrites the shared scratch), the first again
        for attempt, (prob, ref) in enumerate(((first, refs[0]), (other, refs[1]), (first, refs[0]))):
            got = _bwd_call("ifv2_sparse_attn_bwd_noalloc", [], *prob, status)
            torch.cuda.synchronize(dev)
            assert int(status[0]) == 0 and int(status[1]) == 0
            for name, a, b in zip(("dq", "dk", "dv"), got, ref):
                assert not torch.isnan(a.float()).any(), (dev, attempt, name)
                assert torch.equal(a, b), (dev, attempt, name, (a.float() - b.float()).abs().max().item())


def test_noalloc_backward_matches_workspace_backward_twice():
    _check_device(torch.device("cuda", 0))


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs a second GPU")
def test_noalloc_backward_on_a_second_device():
    """The scratch address is per device: the table entry of device 1 is filled by the first call
    made with device 1 current, and device 0 keeps working afterwards."""
    _check_device(torch.device("cuda", 1))
    _check_device(torch.device("cuda", 0))


def test_noalloc_rejects_oversized_calls():
    lib = _lib.load()
    fn = lib.ifv2_sparse_attn_bwd_noalloc
    # 8 Mi query rows > the 4 Mi-row built-in scratch: refused before anything is touched
    rc = fn(8, 8, 8, 8, 8, 8, 8, 8, 8, None, 0, None, 0, 8, 8, 1, 1 << 18, 1 << 18, 32, 2, 128,
            1 << 18, 1 << 18, 0.1, 1, 8, None)
    assert rc == -3 and b"exceed" in lib.ifv2_last_error()
