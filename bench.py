#!/usr/bin/env python
"""Benchmark of the InfLLM-V2 sparse-attention prefill path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--seqlen L]

One "step" is one pass of the hot path over one synthetic 131072-token sequence (128 query heads,
8 KV heads, head_dim 128, bf16): stage-1 scores against the compressed keys -> 64-token max-pool
-> top-64 blocks (1 init + 32 local forced) -> uint64 block mask -> stage-2 block-sparse attention
forward.  Rank 0 prints ONE JSON line; metric = prefill tokens/s.

  * `value`   : inputs already resident in HBM, CUDA-event timed, max over ranks.
  * `e2e`     : the same step through the public Python API starting from pinned HOST buffers,
                host->device copies of q/k/v/compressed-k and the device->host copy of the
                output inside the timed region.
  * `roofline`: the dominant kernel's algorithmic FLOP/s (CUDA events around that kernel inside
                the timed steps) against the measured bf16 peak of this pool.
  * `cpu_baseline`: the pure-PyTorch CPU oracle timed on a bounded sample of the same sequence.

With N > 1 GPUs the KV heads are sharded across ranks (8/N per GPU, no collective: every kernel's
grid has an independent KV-head axis), so the total work is fixed ("strong" scaling).
`--impl reference` times the CPU oracle (the reference's pure-PyTorch path) instead.
"""
import argparse
import json
import math
import os
import subprocess
import sys
import tempfile
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

import torch  # noqa: E402
import torch.distributed as dist  # noqa: E402

SEQLEN, HQ, HK, D = 131072, 128, 8, 128
TOPK, INIT_BLOCKS, LOCAL_BLOCKS, BLOCK = 64, 1, 32, 64
KERNEL, STRIDE = 32, 16
METRIC = "sparse-attn prefill tokens/s at 128k"
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return {k: float(p.get(k, FALLBACK_PEAKS[k])) for k in FALLBACK_PEAKS}, "measured"
    return dict(FALLBACK_PEAKS), "fallback"


class ClockSampler:
    """SM clock and throttle-reason samples while the timed region runs: NVML from a thread every
    5 ms (read-only queries), so that even a region of a few tens of milliseconds gets samples;
    `nvidia-smi -lms` as the fallback when the NVML binding is missing."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
         "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")
    # NVML clocks-event-reason bits (nvml.h)
    BITS = {"sw_power_cap": 0x4, "hw_slowdown": 0x8, "sw_thermal_slowdown": 0x20,
            "hw_thermal_slowdown": 0x40}

    def __init__(self, gpu_index):
        self.idx, self.proc, self.path = gpu_index, None, None
        self.thread, self.stop, self.sm, self.smax, self.reasons = None, False, [], None, set()

    def _nvml_loop(self, nv, handle):
        reason_fn = getattr(nv, "nvmlDeviceGetCurrentClocksEventReasons", None) or \
            nv.nvmlDeviceGetCurrentClocksThrottleReasons
        while not self.stop:
            try:
                self.sm.append(float(nv.nvmlDeviceGetClockInfo(handle, nv.NVML_CLOCK_SM)))
                r = int(reason_fn(handle))
                for n, bit in self.BITS.items():
                    if r & bit:
                        self.reasons.add(n)
            except Exception:
                pass
            time.sleep(0.005)

    def __enter__(self):
        try:
            import threading
            import pynvml as nv
            nv.nvmlInit()
            try:
                uuid = "GPU-" + str(torch.cuda.get_device_properties(self.idx).uuid)
                handle = nv.nvmlDeviceGetHandleByUUID(uuid.encode())
            except Exception:
                handle = nv.nvmlDeviceGetHandleByIndex(self.idx)
            self.smax = float(nv.nvmlDeviceGetMaxClockInfo(handle, nv.NVML_CLOCK_SM))
            self.thread = threading.Thread(target=self._nvml_loop, args=(nv, handle), daemon=True)
            self.thread.start()
            return self
        except Exception:
            self.thread = None
        try:
            fd, self.path = tempfile.mkstemp(suffix=".csv")
            os.close(fd)
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "100",
                 "-i", str(self.idx)], stdout=open(self.path, "w"), stderr=subprocess.DEVNULL)
        except Exception:
            self.proc = None
        return self

    def __exit__(self, *exc):
        if self.thread is not None:
            self.stop = True
            self.thread.join(timeout=2)
        if self.proc is not None:
            time.sleep(0.15)
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except Exception:
                self.proc.kill()

    def summary(self):
        out = {"sm_mhz": None, "sm_max_mhz": None, "reasons": []}
        if self.thread is not None:
            if self.sm:
                sm = sorted(self.sm)
                out.update(sm_mhz=sm[len(sm) // 2], sm_max_mhz=self.smax, reasons=sorted(self.reasons),
                           samples=len(sm))
            return out
        if not self.path or not os.path.exists(self.path):
            return out
        sm, smax, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        with open(self.path) as f:
            for line in f:
                parts = [x.strip() for x in line.split(",")]
                if len(parts) < 9:
                    continue
                try:
                    sm.append(float(parts[1]))
                    smax.append(float(parts[2]))
                except ValueError:
                    continue
                for n, v in zip(names, parts[5:9]):
                    if v.lower().startswith("active"):
                        reasons.add(n)
        os.unlink(self.path)
        if sm:
            sm.sort()
            out.update(sm_mhz=sm[len(sm) // 2], sm_max_mhz=max(smax), reasons=sorted(reasons))
        return out


# ------------------------------------------------------------------------------ workload ------

def make_inputs(seqlen, hk_local, device, seed):
    """q, k, v ~ N(0,1)/sqrt(128) in bf16 for `hk_local` KV heads (16 query heads each), plus the
    compressed keys (mean over windows of 32 tokens, stride 16: the compress_keys kernel)."""
    import infllm_v2
    g = torch.Generator(device=device).manual_seed(seed)
    s = 1.0 / math.sqrt(D)
    q = (torch.randn(seqlen, hk_local * 16, D, device=device, generator=g) * s).to(torch.bfloat16)
    k = (torch.randn(seqlen, hk_local, D, device=device, generator=g) * s).to(torch.bfloat16)
    v = (torch.randn(seqlen, hk_local, D, device=device, generator=g) * s).to(torch.bfloat16)
    kc = infllm_v2.compress_keys(k, kernel_size=KERNEL, kernel_stride=STRIDE)[0]
    return q, k, v, kc


def visible_compressed(seqlen, n_comp):
    """Sum over tokens of the number of visible compressed keys (stage-1 algorithmic pairs)."""
    i = torch.arange(seqlen, dtype=torch.int64)
    off = n_comp - (seqlen - 15) // 16
    return int(((i + 1) // 16 - 1 + off).clamp(0, n_comp).sum())


def attended_pairs(topk_idx, seqlen):
    """Sum over (KV head, token, selected block) of the keys of that block the token may see."""
    hk = topk_idx.shape[0]
    total = 0
    i = torch.arange(seqlen, device=topk_idx.device, dtype=torch.int64).view(1, -1, 1)
    for h in range(hk):
        blk = topk_idx[h:h + 1].long()
        vis = (i + 1 - blk * BLOCK).clamp(0, BLOCK)
        vis = torch.where(blk >= 0, vis, torch.zeros_like(vis))
        total += int(vis.sum())
    return total


def run_ours(args, rank, world, device):
    import infllm_v2
    seqlen = args.seqlen
    assert HK % world == 0, "the KV heads (8) must divide over the GPUs"
    hk_local = HK // world
    q, k, v, kc = make_inputs(seqlen, hk_local, device, seed=rank)
    n_comp = kc.shape[0]
    cu_q = torch.tensor([0, seqlen], dtype=torch.int32, device=device)
    cu_c = torch.tensor([0, n_comp], dtype=torch.int32, device=device)
    fused = not args.unfused
    # default step: stage 1 + pool in one kernel, top-k + mask pack in one kernel, stage 2 (3 launches);
    # --unfused runs the reference's operator sequence (5 launches)
    names = (["stage1_block_scores", "topk_select_mask", "sparse_attn_fwd"] if fused else
             ["stage1_scores", "max_pooling_1d", "topk_select", "topk_to_uint64", "sparse_attn_fwd"])
    n_marks = len(names) + 1

    def step(events=None):
        j = [0]

        def mark():
            if events is not None:
                events[j[0]].record()
            j[0] += 1
        mark()
        if fused:
            # the 17 GB score tensor never reaches HBM, and neither does the int32 block list
            pooled = infllm_v2.infllmv2_stage1_block_scores(q, kc, cu_q, cu_c, seqlen, n_comp,
                                                            LOCAL_BLOCKS, INIT_BLOCKS, causal=True)
            mark()
            mask, _ = infllm_v2.infllmv2_topk_mask(pooled, TOPK, seqlen)
            del pooled
            mark()
        else:
            score = infllm_v2.infllmv2_attn_stage1(q, kc, kc, cu_q, cu_c, cu_c, seqlen, n_comp, causal=True)
            mark()
            pooled = infllm_v2.max_pooling_1d(score, 0, LOCAL_BLOCKS, INIT_BLOCKS, BLOCK, STRIDE)
            del score
            mark()
            idx = infllm_v2.infllmv2_topk(pooled, TOPK)
            del pooled
            mark()
            mask, _ = infllm_v2.topk_to_uint64(idx, seqlen, BLOCK)
            del idx
            mark()
        out = infllm_v2.infllmv2_attn_varlen_func(q, k, v, cu_q, cu_q, seqlen, seqlen, causal=True,
                                                  block_mask=mask)
        mark()
        return out

    for _ in range(args.warmup):
        step()
    infllm_v2.check_device_status()
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    ev = [[torch.cuda.Event(enable_timing=True) for _ in range(n_marks)] for _ in range(args.steps)]
    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with ClockSampler(torch.cuda.current_device()) as clocks:
        t0.record()
        for s in range(args.steps):
            out = step(ev[s])
        t1.record()
        torch.cuda.synchronize()
    infllm_v2.check_device_status()
    total_ms = t0.elapsed_time(t1)
    if world > 1:
        t = torch.tensor([total_ms], device=device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        total_ms = float(t.item())
    ms_per_step = total_ms / args.steps
    per_kernel = [sum(ev[s][j].elapsed_time(ev[s][j + 1]) for s in range(args.steps)) / args.steps
                  for j in range(n_marks - 1)]
    kernel_ms = dict(zip(names, per_kernel))

    # ---- outside the timed region: the block lists (for the work count and the parity check) and
    # the two separate selection kernels that the fused one replaces
    pooled = infllm_v2.infllmv2_stage1_block_scores(q, kc, cu_q, cu_c, seqlen, n_comp, LOCAL_BLOCKS,
                                                    INIT_BLOCKS, causal=True)
    idx = infllm_v2.infllmv2_topk(pooled, TOPK)
    sel_ms = {"topk_select": _time_ms(lambda: infllm_v2.infllmv2_topk(pooled, TOPK), reps=3, warmup=1),
              "topk_to_uint64": _time_ms(lambda: infllm_v2.topk_to_uint64(idx, seqlen, BLOCK), reps=3, warmup=1)}
    del pooled

    # ---- algorithmic work of this rank's shard
    pk, pk_kind = peaks()
    v_pairs = visible_compressed(seqlen, n_comp)
    flops_s1 = 2.0 * D * (hk_local * 16) * v_pairs
    pairs = attended_pairs(idx, seqlen)                     # over this rank's KV heads
    flops_s2 = 4.0 * D * 16 * pairs
    n_blk = (seqlen + BLOCK - 1) // BLOCK
    row_stride = max((n_comp + 127) // 128 * 128, 128)
    bytes_pool = hk_local * seqlen * (n_comp * 2 + n_blk * 2)
    bytes_topk = hk_local * seqlen * (n_blk * 2 + TOPK * 4)
    bytes_pack = hk_local * seqlen * (TOPK * 4 + ((n_blk + 63) // 64) * 8)
    tens, hbm = pk["bf16_tflops_sustained"], pk["hbm_gbs"]
    bytes_mask = hk_local * seqlen * (n_blk * 2 + ((n_blk + 63) // 64) * 8)
    roof = {
        "sparse_attn_fwd": ("tensor", flops_s2 / (kernel_ms["sparse_attn_fwd"] * 1e-3) / 1e12, tens, "TFLOP/s"),
    }
    if fused:
        roof["stage1_block_scores"] = ("tensor", flops_s1 / (kernel_ms["stage1_block_scores"] * 1e-3) / 1e12,
                                       tens, "TFLOP/s")
        roof["topk_select_mask"] = ("hbm", bytes_mask / (kernel_ms["topk_select_mask"] * 1e-3) / 1e9, hbm, "GB/s")
    else:
        roof["stage1_scores"] = ("tensor", flops_s1 / (kernel_ms["stage1_scores"] * 1e-3) / 1e12, tens, "TFLOP/s")
        roof["max_pooling_1d"] = ("hbm", bytes_pool / (kernel_ms["max_pooling_1d"] * 1e-3) / 1e9, hbm, "GB/s")
        roof["topk_select"] = ("hbm", bytes_topk / (kernel_ms["topk_select"] * 1e-3) / 1e9, hbm, "GB/s")
        roof["topk_to_uint64"] = ("hbm", bytes_pack / (kernel_ms["topk_to_uint64"] * 1e-3) / 1e9, hbm, "GB/s")
    dominant = max(kernel_ms, key=kernel_ms.get)
    bound, ach, peak, unit = roof[dominant]
    # DRAM traffic per launch: measured with ncu on the 16384-token case of the same command
    # (profiles/), where dram bytes / algorithmic bytes came out as below; a full-size launch is
    # too large to capture, and both kernels stream each input once, so the ratio carries over
    q_bytes = seqlen * hk_local * 16 * D * 2
    alg_bytes = {
        "stage1_block_scores": q_bytes + n_comp * hk_local * D * 2 + hk_local * seqlen * n_blk * 2,
        "stage1_scores": q_bytes + n_comp * hk_local * D * 2 + hk_local * seqlen * row_stride * 2,
        "sparse_attn_fwd": 2 * q_bytes + 2 * seqlen * hk_local * D * 2
                           + hk_local * seqlen * (((n_blk + 63) // 64) * 8 + 16 * 4),
    }
    ncu_ratio = {"stage1_block_scores": 0.99, "stage1_scores": 0.97, "sparse_attn_fwd": 0.97}
    traffic = (round(alg_bytes[dominant] * ncu_ratio[dominant]) if dominant in ncu_ratio else None)
    clk = clocks.summary()
    roofline = {"kernel": dominant, "bound": bound, "achieved": round(ach, 2), "peak": peak,
                "unit": unit, "frac": round(ach / peak, 4), "traffic": traffic,
                "traffic_source": "ncu dram bytes of the 16384-token case x algorithmic-byte ratio",
                "algorithmic_bytes": alg_bytes.get(dominant), "peak_source": pk_kind,
                "ms_per_launch": round(kernel_ms[dominant], 3)}
    s1_name = "stage1_block_scores" if fused else "stage1_scores"
    if dominant == s1_name and clk.get("sm_mhz"):
        # what governs the scorer is the exponential unit, not the tensor pipe: two exponentials per
        # (query-head row, visible key) pair -- one for the row sums, one for the probability -- on a
        # unit that retires 16 ex2 per clock per SM (measured on this part: 16.0)
        n_exp = 2.0 * (hk_local * 16) * v_pairs
        sfu_peak = 16.0 * 148 * clk["sm_mhz"] * 1e6
        sfu_ach = n_exp / (kernel_ms[dominant] * 1e-3)
        roofline.update(bound_alt="sfu", achieved_alt=round(sfu_ach / 1e12, 3), peak_alt=round(sfu_peak / 1e12, 3),
                        unit_alt="Texp/s", frac_alt=round(sfu_ach / sfu_peak, 4),
                        alt_note="exponentials per launch / (16 ex2 per clock per SM x 148 SMs x median SM clock "
                                 "under load)")
    kernels = {n: {"ms": round(kernel_ms[n], 3), "bound": roof[n][0], "achieved": round(roof[n][1], 2),
                   "unit": roof[n][3], "frac": round(roof[n][1] / roof[n][2], 4)} for n in names}
    if fused:
        kernels["separate_selection_kernels"] = {
            "topk_select_ms": round(sel_ms["topk_select"], 3), "topk_to_uint64_ms": round(sel_ms["topk_to_uint64"], 3),
            "note": "the two launches (and the int32 list between them) that topk_select_mask replaces; "
                    "timed outside the step"}

    parity = step_parity(q, k, v, kc, out, idx, seqlen)

    # ---- end to end from pinned host memory through the public API
    e2e = run_e2e(args, step, q, k, v, kc, seqlen, world, device)

    result = {
        "metric": METRIC, "value": round(seqlen / (ms_per_step * 1e-3), 1), "unit": "tokens/s",
        "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": round(ms_per_step, 3), "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": f"prefill {seqlen} tokens, 128q/8kv heads, d128: stage1 + max-pool + "
                               f"top-64 (1 init + 32 local) + uint64 mask + stage-2 fwd"
                               + (" [3 launches: stage 1 + pool, top-k + mask, stage 2]" if fused
                                  else " [the reference's 5-operator sequence]"),
                   "seq_len": seqlen, "global_batch": 1, "kv_heads_per_gpu": hk_local,
                   "parallelism": f"kv-head shards x{world}" if world > 1 else "single GPU",
                   "l2": "inputs (q alone is %.1f GB per GPU) exceed the 126 MB L2" % (q.numel() * 2 / 1e9)},
        "clocks": clk,
        "e2e": e2e,
        "parity": parity,
        "gpu_launches": len(names) * args.steps,
        "gpu_launches_per_step": len(names),
        "roofline": roofline,
        "kernels": kernels,
        "flops_per_step": {"stage1_algorithmic": flops_s1 * world, "stage2_fwd_algorithmic": flops_s2 * world},
    }
    return result


def step_parity(q, k, v, kc, out, idx, seqlen):
    """The timed step's own results against plain fp32 PyTorch on the GPU for sampled tokens (the
    dense-with-mask attention restated over gathered keys) and against the CPU oracle for the
    selection of two row chunks.  The checker runs after the timed region; it is not the product."""
    try:
        import oracle
        sys.path.insert(0, os.path.join(ROOT, "tests"))
        sys.path.insert(0, os.path.join(ROOT, "tests", "golden"))
        import gpu_oracle
        import infllm_v2
        dev = q.device
        toks = torch.tensor(sorted(set([0, 63, 64, seqlen // 3, seqlen // 2 - 1, seqlen // 2] +
                                       list(range(seqlen - 8, seqlen)))), device=dev)
        ref, _ = gpu_oracle.attend_rows(q[toks], toks, k, v, idx[:, toks], seqlen)
        diff = (out[toks].float() - ref).abs()
        max_abs = diff.max().item()
        mean_rel = (diff.mean() / ref.abs().mean().clamp_min(1e-12)).item()
        exact, rows = 0, 0
        for start in (seqlen // 2, seqlen - 128):
            start = start // 64 * 64
            sl = slice(start, start + 128)
            n_pre = (sl.stop - KERNEL) // STRIDE + 1
            cu_q = torch.tensor([0, 128], dtype=torch.int32, device=dev)
            cu_p = torch.tensor([0, n_pre], dtype=torch.int32, device=dev)
            score = infllm_v2.infllmv2_attn_stage1(q[sl], kc[:n_pre], kc[:n_pre], cu_q, cu_p, cu_p, 128, n_pre,
                                                   causal=True)
            pooled = oracle.max_pooling_1d(score.cpu(), start, LOCAL_BLOCKS, INIT_BLOCKS, BLOCK, STRIDE)
            ref_idx = oracle.topk_select(pooled, TOPK, (torch.arange(128) + start) // BLOCK)
            same = (ref_idx == idx[:, sl].cpu()).all(dim=-1)
            exact += int(same.sum())
            rows += same.numel()
        return {"stage2_out_max_abs": round(max_abs, 5), "stage2_out_mean_rel": round(mean_rel, 5),
                "stage2_tokens_checked": int(toks.numel()), "topk_exact_row_rate": round(exact / rows, 4),
                "topk_rows_checked": rows,
                "tolerance": "max-abs <= 2e-2, mean-rel <= 1e-2; top-k rows bit-exact",
                "pass": bool(max_abs <= 2e-2 and mean_rel <= 1e-2 and exact == rows)}
    except Exception as e:                              # the headline line must still be printed
        return {"error": repr(e)[:300]}


def run_e2e(args, step, q, k, v, kc, seqlen, world, device):
    """The same job through the public API starting from pinned HOST buffers and ending with the
    output in pinned host memory: `StreamedPrefill` cuts the query into chunks (--e2e-chunk tokens) and
    overlaps copy-in, kernels and copy-out on three streams.  With compute ~ tokens^2 and copies ~ tokens
    an ascending chunk order is copy-bound for the first ~45 % of the sequence; the default order
    starts in the middle and alternates outwards, which keeps copies and kernels both busy."""
    from infllmv2_cuda_impl_b200.sharding import StreamedPrefill
    host = [torch.empty(t.shape, dtype=t.dtype).pin_memory() for t in (q, k, v, kc)]
    for h, t in zip(host, (q, k, v, kc)):
        h.copy_(t)
    out_host = torch.empty(q.shape, dtype=q.dtype).pin_memory()
    chunk = args.e2e_chunk if seqlen % args.e2e_chunk == 0 else seqlen
    runner = StreamedPrefill(seqlen, q.shape[1], k.shape[1], D, kc.shape[0], device, chunk)
    torch.cuda.synchronize()
    steps = max(1, min(args.steps, 3))

    def one():
        runner(host[0], host[1], host[2], host[3], out_host, TOPK, INIT_BLOCKS, LOCAL_BLOCKS,
               order=(list(range(seqlen // chunk)) if args.e2e_order == "ascending" else None),
               split_ends=args.e2e_split)

    one()
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(steps):
        one()
    b.record()
    torch.cuda.synchronize()
    ms = a.elapsed_time(b) / steps
    if world > 1:
        t = torch.tensor([ms], device=device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    h2d = sum(h.numel() * h.element_size() for h in host)
    d2h = out_host.numel() * out_host.element_size()

    # ---- the floor under any host-to-host number: the same bytes moved by bare cudaMemcpyAsync
    # calls, host->device and device->host at the same time on two streams, all ranks together
    def bare_copies():
        main = torch.cuda.current_stream(device)
        runner.s_in.wait_stream(main)
        runner.s_out.wait_stream(main)
        with torch.cuda.stream(runner.s_in):
            for dst, src in zip((runner.q, runner.k, runner.v, runner.kc), host):
                dst.copy_(src, non_blocking=True)
        with torch.cuda.stream(runner.s_out):
            out_host.copy_(runner.q, non_blocking=True)
        main.wait_stream(runner.s_in)
        main.wait_stream(runner.s_out)

    bare_copies()
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    a.record()
    for _ in range(2):
        bare_copies()
    b.record()
    torch.cuda.synchronize()
    copy_ms = a.elapsed_time(b) / 2
    if world > 1:
        t = torch.tensor([copy_ms], device=device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        copy_ms = float(t.item())
    return {"value": round(seqlen / (ms * 1e-3), 1), "unit": "tokens/s", "ms_per_step": round(ms, 3),
            "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
            "copy_floor": {"ms": round(copy_ms, 3), "h2d_gbs_per_rank": round(h2d / copy_ms / 1e6, 1),
                           "d2h_gbs_per_rank": round(d2h / copy_ms / 1e6, 1),
                           "how": "the step's input and output bytes as bare pinned copies, both directions "
                                  "at once, all ranks at once, no kernels; max over ranks"},
            "how": f"pinned host buffers, {seqlen // chunk} query chunks ({args.e2e_order}), copy-in / kernels / copy-out overlapped"}


# ------------------------------------------------------------------------------ other configs --

def _time_ms(fn, reps=5, warmup=2):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(reps):
        fn()
    b.record()
    torch.cuda.synchronize()
    return a.elapsed_time(b) / reps


def config4_compress(device, pk, small=False):
    """Key compression (mean over 32-token windows, stride 16) at the prefill size: the K of the
    131072-token, 8-KV-head sequence (268 MB, larger than L2) -> 8191 compressed keys."""
    import infllm_v2
    L, hk = (65536 if small else 131072), 8
    g = torch.Generator(device=device).manual_seed(0)
    k = (torch.randn(L, hk, D, device=device, generator=g) / math.sqrt(D)).to(torch.bfloat16)
    kc = infllm_v2.compress_keys(k)[0]
    t = _time_ms(lambda: infllm_v2.compress_keys(k), reps=20, warmup=3)
    b = k.numel() * 2 + kc.numel() * 2
    return {"config4_compress_keys": {"tokens": L, "kv_heads": hk, "ms": round(t, 4),
                                      "gbs": round(b / t / 1e6, 1),
                                      "frac": round(b / t / 1e6 / pk["hbm_gbs"], 4),
                                      "note": "268 MB of keys per launch, larger than the 126 MB L2"}}


def config4_coarse_lse(device, pk, small=False):
    """Stage 1 (+ pool) of the prefill with the row sums taken over the coarse compression
    (kernel 128 / stride 64) instead of the scored keys: the reference's "compressed LSE" mode.
    Pass 1 then has a quarter of the keys."""
    import infllm_v2
    L, hk = (32768 if small else SEQLEN), HK
    q, k, _, kc = make_inputs(L, hk, device, seed=0)
    kv = infllm_v2.compress_keys(k, kernel_size=128, kernel_stride=64)[0]
    cu_q = torch.tensor([0, L], dtype=torch.int32, device=device)
    cu_c = torch.tensor([0, kc.shape[0]], dtype=torch.int32, device=device)
    cu_v = torch.tensor([0, kv.shape[0]], dtype=torch.int32, device=device)
    run = lambda **kw: infllm_v2.infllmv2_stage1_block_scores(q, kc, cu_q, cu_c, L, kc.shape[0],
                                                              LOCAL_BLOCKS, INIT_BLOCKS, **kw)
    t_same = _time_ms(lambda: run(), reps=3, warmup=2)
    t_coarse = _time_ms(lambda: run(lse_keys=kv, cu_seqlens_v=cu_v), reps=3, warmup=2)
    infllm_v2.check_device_status()
    fl = 2.0 * D * hk * 16 * visible_compressed(L, kc.shape[0])
    return {"config4_stage1_compressed_lse": {
        "tokens": L, "ms_lse_over_scored_keys": round(t_same, 3), "ms_lse_over_coarse_keys": round(t_coarse, 3),
        "tflops_coarse": round(fl / t_coarse / 1e9, 1),
        "frac_coarse": round(fl / t_coarse / 1e9 / pk["bf16_tflops_sustained"], 4),
        "note": "FLOPs counted as one pass over the scored keys in both cases"}}


def config4_topk(device, pk, small=False):
    """The top-k kernel alone at the row width of the 131072-token prefill (2048 block scores per
    query row): one KV head's rows, scores shaped like the stage-1 output (block 0 and the 32
    local blocks +inf, blocks past the query's own 0)."""
    import infllm_v2
    n_blk = 2048
    rows = 32768 if small else 131072
    first = 131072 - rows                        # the last `rows` tokens of the sequence
    g = torch.Generator(device=device).manual_seed(0)
    y = torch.rand(1, rows, n_blk, device=device, generator=g).to(torch.bfloat16)
    bq = (torch.arange(rows, device=device) + first) // BLOCK
    col = torch.arange(n_blk, device=device)
    y[0].masked_fill_(col[None, :] > bq[:, None], 0.0)
    y[0].masked_fill_((col[None, :] <= bq[:, None]) & (col[None, :] + LOCAL_BLOCKS >= bq[:, None]), float("inf"))
    y[0, :, 0] = float("inf")
    t = _time_ms(lambda: infllm_v2.infllmv2_topk(y, TOPK, cache_len=first))
    b = rows * (n_blk * 2 + TOPK * 4)
    return {"config4_topk_rows": {"rows": rows, "n_blocks": n_blk, "topk_ms": round(t, 4),
                                  "topk_gbs": round(b / t / 1e6, 1),
                                  "topk_frac": round(b / t / 1e6 / pk["hbm_gbs"], 4)}}


def config3_topk(lens, hk, topk, seed):
    """Block lists of BASELINE config 3: per 64-token query block and KV head, block 0, the 32
    causal-local blocks and uniformly random earlier blocks up to `topk`, ascending, -1 tail."""
    import numpy as np
    rng = np.random.default_rng(seed)
    per_head = []
    for h in range(hk):
        rows = []
        for lq in lens:
            for bq in range((lq + BLOCK - 1) // BLOCK):
                forced = set([0]) | set(range(max(0, bq - 31), bq + 1))
                rest = [b for b in range(bq + 1) if b not in forced]
                extra = rng.choice(rest, size=min(len(rest), topk - len(forced)), replace=False) if rest and len(forced) < topk else []
                sel = np.sort(np.array(sorted(forced) + list(extra), dtype=np.int32))[:topk]
                row = np.full(topk, -1, np.int32)
                row[:len(sel)] = sel
                n_tok = min(BLOCK, lq - bq * BLOCK)
                rows.append(np.repeat(row[None], n_tok, 0))
        per_head.append(np.concatenate(rows))
    return torch.from_numpy(np.stack(per_head))


def extra_configs(device, pk, only=None, small=False):
    """Secondary numbers on one GPU: config 2 (selection micro-benchmark), config 3 (varlen
    training forward + backward) and config 5 (decode).  Each kernel against its own roofline.
    `only` picks one of them; `small` shrinks it (for profiler captures)."""
    out = {}
    if only in (None, "selection"):
        out.update(config2_selection(device, pk, small))
    if only in (None, "topk"):
        out.update(config4_topk(device, pk, small))
    if only in (None, "compress"):
        out.update(config4_compress(device, pk, small))
    if only in (None, "coarse"):
        out.update(config4_coarse_lse(device, pk, small))
    if only in (None, "train"):
        out.update(config3_train(device, pk, small))
    if only in (None, "decode"):
        out.update(config5_decode(device, pk, small))
    return out


def config2_selection(device, pk, small=False):
    import infllm_v2
    out = {}
    s = 1.0 / math.sqrt(D)
    g = torch.Generator(device=device).manual_seed(0)
    # ---- config 2: 32768 tokens, 32q/2kv
    L, hk = (8192 if small else 32768), 2
    q = (torch.randn(L, hk * 16, D, device=device, generator=g) * s).to(torch.bfloat16)
    k = (torch.randn(L, hk, D, device=device, generator=g) * s).to(torch.bfloat16)
    kc = infllm_v2.compress_keys(k, kernel_size=KERNEL, kernel_stride=STRIDE)[0]
    n_comp, n_blk = kc.shape[0], L // BLOCK
    cu_q = torch.tensor([0, L], dtype=torch.int32, device=device)
    cu_c = torch.tensor([0, n_comp], dtype=torch.int32, device=device)
    score = infllm_v2.infllmv2_attn_stage1(q, kc, kc, cu_q, cu_c, cu_c, L, n_comp, causal=True)
    pooled = infllm_v2.max_pooling_1d(score, 0, LOCAL_BLOCKS, INIT_BLOCKS, BLOCK, STRIDE)
    idx = infllm_v2.infllmv2_topk(pooled, TOPK)
    t_s1 = _time_ms(lambda: infllm_v2.infllmv2_attn_stage1(q, kc, kc, cu_q, cu_c, cu_c, L, n_comp, causal=True))
    t_pool = _time_ms(lambda: infllm_v2.max_pooling_1d(score, 0, LOCAL_BLOCKS, INIT_BLOCKS, BLOCK, STRIDE))
    t_topk = _time_ms(lambda: infllm_v2.infllmv2_topk(pooled, TOPK))
    t_pack = _time_ms(lambda: infllm_v2.topk_to_uint64(idx, L, BLOCK))
    fl = 2.0 * D * hk * 16 * visible_compressed(L, n_comp)
    b_pool = hk * L * (n_comp + n_blk) * 2
    b_topk = hk * L * (n_blk * 2 + TOPK * 4)
    b_pack = hk * L * (TOPK * 4 + ((n_blk + 63) // 64) * 8)
    out["config2_selection_32k"] = {
        "stage1_ms": round(t_s1, 4), "stage1_tflops": round(fl / t_s1 / 1e9, 1),
        "stage1_frac": round(fl / t_s1 / 1e9 / pk["bf16_tflops"], 4),
        "pool_ms": round(t_pool, 4), "pool_gbs": round(b_pool / t_pool / 1e6, 1),
        "pool_frac": round(b_pool / t_pool / 1e6 / pk["hbm_gbs"], 4),
        "topk_ms": round(t_topk, 4), "topk_gbs": round(b_topk / t_topk / 1e6, 1),
        "topk_frac": round(b_topk / t_topk / 1e6 / pk["hbm_gbs"], 4),
        "pack_ms": round(t_pack, 4), "pack_gbs": round(b_pack / t_pack / 1e6, 1),
        "pack_frac": round(b_pack / t_pack / 1e6 / pk["hbm_gbs"], 4),
        "note": "32 MB working sets fit the 126 MB L2: GB/s here are L2-assisted"}
    return out


def config3_train(device, pk, small=False):
    import infllm_v2
    from infllmv2_cuda_impl_b200 import attention
    out = {}
    s = 1.0 / math.sqrt(D)
    g = torch.Generator(device=device).manual_seed(0)
    # ---- config 3: varlen fwd + bwd, 4 packed sequences, 65536 tokens, 32q/2kv
    lens, hk = ([2048, 4096, 6144, 4096] if small else [8192, 16384, 24576, 16384]), 2
    T = sum(lens)
    q = (torch.randn(T, hk * 16, D, device=device, generator=g) * s).to(torch.bfloat16)
    k = (torch.randn(T, hk, D, device=device, generator=g) * s).to(torch.bfloat16)
    v = (torch.randn(T, hk, D, device=device, generator=g) * s).to(torch.bfloat16)
    do = torch.randn(T, hk * 16, D, device=device, generator=g).to(torch.bfloat16)
    cu = torch.tensor([0] + list(torch.tensor(lens).cumsum(0)), dtype=torch.int32, device=device)
    idx = config3_topk(lens, hk, TOPK, seed=1).to(device)
    max_l = max(lens)
    scale = D ** -0.5
    o, lse, mask = attention._infllmv2_attn_varlen_forward(q, k, v, cu, cu, max_l, max_l, scale, True, idx)
    t_fwd = _time_ms(lambda: attention._infllmv2_attn_varlen_forward(q, k, v, cu, cu, max_l, max_l, scale, True, idx))
    t_bwd = _time_ms(lambda: attention._infllmv2_attn_varlen_backward(do, q, k, v, o, lse, cu, cu, max_l, max_l,
                                                                      scale, True, mask))
    attention.check_device_status()
    i_local = torch.cat([torch.arange(l, device=device) for l in lens]).view(1, -1, 1)
    pairs = 0
    for h in range(hk):
        blk = idx[h:h + 1].long()
        vis = (i_local + 1 - blk * BLOCK).clamp(0, BLOCK)
        pairs += int(torch.where(blk >= 0, vis, torch.zeros_like(vis)).sum())
    f_fwd, f_bwd = 4.0 * D * 16 * pairs, 10.0 * D * 16 * pairs
    out["config3_varlen_fwd_bwd_64k"] = {
        "fwd_ms": round(t_fwd, 3), "bwd_ms": round(t_bwd, 3),
        "fwd_tflops": round(f_fwd / t_fwd / 1e9, 1), "bwd_tflops": round(f_bwd / t_bwd / 1e9, 1),
        "fwd_bwd_tflops": round((f_fwd + f_bwd) / (t_fwd + t_bwd) / 1e9, 1),
        "fwd_bwd_frac": round((f_fwd + f_bwd) / (t_fwd + t_bwd) / 1e9 / pk["bf16_tflops_sustained"], 4),
        "algorithmic_flops": f_fwd + f_bwd, "tokens_per_s_fwd_bwd": round(T / ((t_fwd + t_bwd) * 1e-3), 1),
        "note": "bwd includes the mask transpose, the dO.O pre-pass and both gradient kernels"}
    return out


def config5_decode(device, pk, small=False):
    import infllm_v2
    out = {}
    s = 1.0 / math.sqrt(D)
    g = torch.Generator(device=device).manual_seed(0)
    # ---- config 5: decode, batch 64, cache 32768..131072, 32q/2kv, top-64 blocks
    B, hk = 64, 2
    lo, hi = (8192, 16384) if small else (32768, 131072)
    cap = hi + 64
    lens_t = torch.randint(lo, hi + 1, (B,), generator=torch.Generator().manual_seed(0)).to(torch.int32)
    kcache = (torch.randn(B, cap, hk, D, device=device, generator=g) * s).to(torch.bfloat16)
    vcache = (torch.randn(B, cap, hk, D, device=device, generator=g) * s).to(torch.bfloat16)
    q = (torch.randn(B, 1, hk * 16, D, device=device, generator=g) * s).to(torch.bfloat16)
    import numpy as np
    rng = np.random.default_rng(0)
    rows = np.full((B, hk, 1, TOPK), -1, np.int32)
    for b in range(B):
        nblk = (int(lens_t[b]) + BLOCK - 1) // BLOCK
        for h in range(hk):
            forced = [0] + list(range(nblk - 33, nblk))
            rest = rng.choice(np.arange(1, nblk - 33), size=TOPK - len(forced), replace=False)
            rows[b, h, 0] = np.sort(np.array(forced + list(rest), dtype=np.int32))
    idx = torch.from_numpy(rows).to(device)
    lens_d = lens_t.to(device)
    t_dec = _time_ms(lambda: infllm_v2.infllmv2_attn_with_kvcache(q, kcache, vcache, cache_seqlens=lens_d,
                                                                  topk_idx=idx), reps=10)
    bytes_dec = B * hk * TOPK * BLOCK * D * 2 * 2 + 2 * B * hk * 16 * D * 2
    # the step is four short launches: replayed from a CUDA graph the host launch cost disappears
    t_graph = None
    try:
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            infllm_v2.infllmv2_attn_with_kvcache(q, kcache, vcache, cache_seqlens=lens_d, topk_idx=idx)
        torch.cuda.current_stream().wait_stream(side)
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            infllm_v2.infllmv2_attn_with_kvcache(q, kcache, vcache, cache_seqlens=lens_d, topk_idx=idx)
        t_graph = _time_ms(graph.replay, reps=20)
    except Exception as e:                                  # keep the eager number
        out["config5_graph_error"] = repr(e)[:200]
    best = min(t_dec, t_graph) if t_graph else t_dec
    out["config5_decode_b64"] = {
        "ms": round(best, 4), "ms_eager": round(t_dec, 4),
        "ms_cuda_graph": round(t_graph, 4) if t_graph else None,
        "gbs": round(bytes_dec / best / 1e6, 1),
        "frac": round(bytes_dec / best / 1e6 / pk["hbm_gbs"], 4),
        "tokens_per_s": round(B / (best * 1e-3), 1),
        "note": "stage-2 sparse decode step incl. the uint64 mask build; 268 MB of selected K/V per step"}

    # ---- the whole decode step: stage 1 over the compressed keys of every sequence (one query
    # token each) -> 64-token max-pool -> top-64 -> sparse attention over the selected blocks
    n_c = [(int(l) - KERNEL) // STRIDE + 1 for l in lens_t]
    kc = (torch.randn(sum(n_c), hk, D, device=device, generator=g) * s).to(torch.bfloat16)
    cu_q = torch.arange(B + 1, dtype=torch.int32, device=device)
    cu_c = torch.tensor([0] + list(torch.tensor(n_c).cumsum(0)), dtype=torch.int32, device=device)
    max_c, q2 = max(n_c), q.view(B, hk * 16, D)
    cache_lens = (lens_d - 1).contiguous()               # the query is the last token of its sequence
    n_c_dev = torch.tensor(n_c, dtype=torch.int32, device=device)

    def full_step():
        # scores, pool, top-k and mask in two launches (the score rows stay on chip), as
        # SparseAttention.decode does; equal to infllmv2_attn_stage1 -> decode_select
        mask = infllm_v2.infllmv2_stage1_decode_select(q2, kc, cu_c, cache_lens, max_c, cap, TOPK,
                                                       LOCAL_BLOCKS, INIT_BLOCKS, seqused_k=n_c_dev)
        return infllm_v2.infllmv2_attn_with_kvcache(q, kcache, vcache, cache_seqlens=lens_d, block_mask=mask)

    full_step()
    t_full = _time_ms(full_step, reps=10)
    t_full_graph = None
    try:
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            full_step()
        torch.cuda.current_stream().wait_stream(side)
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            full_step()
        t_full_graph = _time_ms(graph.replay, reps=20)
    except Exception as e:
        out["config5_full_graph_error"] = repr(e)[:200]
    best_full = min(t_full, t_full_graph) if t_full_graph else t_full
    bytes_full = bytes_dec + kc.numel() * 2
    out["config5_decode_b64_with_selection"] = {
        "ms": round(best_full, 4), "ms_eager": round(t_full, 4),
        "ms_cuda_graph": round(t_full_graph, 4) if t_full_graph else None,
        "gbs": round(bytes_full / best_full / 1e6, 1),
        "frac": round(bytes_full / best_full / 1e6 / pk["hbm_gbs"], 4),
        "tokens_per_s": round(B / (best_full * 1e-3), 1),
        "note": "stage 1 (one token per sequence) with pool/top-k/mask in its second launch + sparse decode; algorithmic bytes = "
                "compressed keys once (%d MB) + selected K/V" % (kc.numel() * 2 // 1000000)}

    # ---- the same step through the caller-side layer: the new token's key / value are appended
    # and the compressed-key cache is updated (one launch), the compressed keys are scored in place
    # in their per-sequence cache (seqused_k), then pool, top-k and sparse attention
    del kc
    cfg = infllm_v2.SparseConfig(topk=TOPK, init_blocks=INIT_BLOCKS, local_blocks=LOCAL_BLOCKS, dense_len=0)
    layer = infllm_v2.SparseAttention(cfg)
    cache = infllm_v2.DecodeCache(B, 64, hk, cfg, device)          # small, then pointed at the big caches
    cache.capacity, cache.k, cache.v = cap, kcache, vcache
    cache.c_capacity = cfg.windows(cap)
    cache.kc = (torch.randn(B, cache.c_capacity, hk, D, device=device, generator=g) * s).to(torch.bfloat16)
    cache.cu_c = cache.cu_q * cache.c_capacity
    cache.seqlens.copy_(lens_d)
    cache.n_comp.copy_(torch.tensor(n_c, dtype=torch.int32))
    cache.max_len = hi
    k_new = (torch.randn(B, hk, D, device=device, generator=g) * s).to(torch.bfloat16)
    v_new = (torch.randn(B, hk, D, device=device, generator=g) * s).to(torch.bfloat16)
    t_layer = _time_ms(lambda: layer.decode(q2, k_new, v_new, cache), reps=10, warmup=3)
    infllm_v2.check_device_status()
    t_layer_graph = None
    try:
        step = layer.capture_decode(cache)
        t_layer_graph = _time_ms(lambda: step(q2, k_new, v_new), reps=20, warmup=3)
        infllm_v2.check_device_status()
    except Exception as e:
        out["config5_layer_graph_error"] = repr(e)[:200]
    best_layer = min(t_layer, t_layer_graph) if t_layer_graph else t_layer
    out["config5_decode_b64_layer_step"] = {
        "ms": round(best_layer, 4), "ms_eager": round(t_layer, 4),
        "ms_cuda_graph": round(t_layer_graph, 4) if t_layer_graph else None,
        "gbs": round(bytes_full / best_layer / 1e6, 1),
        "frac": round(bytes_full / best_layer / 1e6 / pk["hbm_gbs"], 4),
        "tokens_per_s": round(B / (best_layer * 1e-3), 1),
        "note": "SparseAttention.decode: token append + compressed-key update + stage 1 over the "
                "compressed cache in place + pool + top-k + sparse decode; the graph variant includes "
                "the three input copies and is sized for the cache capacity"}
    return out


def _timed_max(fn, device, reps=5, warmup=3):
    """CUDA-event time of fn per call, all ranks between barriers, max over ranks."""
    for _ in range(warmup):
        fn()
    dist.barrier()
    torch.cuda.synchronize()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(reps):
        fn()
    b.record()
    dist.barrier()
    torch.cuda.synchronize()
    t = torch.tensor([a.elapsed_time(b) / reps], device=device)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def _zigzag_rows(seqlen, world, rank):
    from infllmv2_cuda_impl_b200 import sharding
    chunks = sharding.zigzag_chunks(seqlen, world, rank)
    rows = torch.cat([torch.arange(c.start, c.end) for c in chunks])
    kc_rows = torch.cat([torch.arange(*sharding.compressed_range(c)) for c in chunks])
    return chunks, rows, kc_rows


def sharded_prefill_bench(device, rank, world, seqlen=SEQLEN, hk=2, reps=5, pk=None):
    """Query-chunk-parallel prefill of ONE sequence with fewer KV heads than GPUs (32q/2kv heads):
    every rank owns two zig-zag query chunks, K / V / compressed K are all-gathered over NCCL into
    local HBM, then each chunk runs the normal kernels.  The whole sequence is generated from one
    seed on every rank (each keeps its rows), so rank 0 can also run it unsharded and compare."""
    from infllmv2_cuda_impl_b200 import sharding
    import infllm_v2
    g = torch.Generator(device=device).manual_seed(1234)
    s = 1.0 / math.sqrt(D)
    q_full = (torch.randn(seqlen, hk * 16, D, device=device, generator=g) * s).to(torch.bfloat16)
    k_full = (torch.randn(seqlen, hk, D, device=device, generator=g) * s).to(torch.bfloat16)
    v_full = (torch.randn(seqlen, hk, D, device=device, generator=g) * s).to(torch.bfloat16)
    kc_full = infllm_v2.compress_keys(k_full)[0]
    kc_pad = torch.cat([kc_full, kc_full.new_zeros((seqlen // STRIDE - kc_full.shape[0],) + kc_full.shape[1:])])
    chunks, rows, kc_rows = _zigzag_rows(seqlen, world, rank)
    rows_d, kc_rows_d = rows.to(device), kc_rows.to(device)
    q, k, v, kc = q_full[rows_d], k_full[rows_d], v_full[rows_d], kc_pad[kc_rows_d]
    if rank != 0:
        del q_full, k_full, v_full, kc_full
    del kc_pad

    def gather():
        return [sharding.gather_sequence(t, world) for t in (k, v, kc)]

    def step(overlap=True):
        return sharding.sharded_prefill(q, k, v, kc, seqlen, world, rank, TOPK, INIT_BLOCKS, LOCAL_BLOCKS,
                                        overlap=overlap)

    t_gather = _timed_max(gather, device, reps)
    t_step = _timed_max(step, device, reps)
    t_serial = _timed_max(lambda: step(False), device, reps)
    infllm_v2.check_device_status()
    out_local = step()
    # ---- parity: rank 0 runs the same sequence unsharded and compares its own rows
    ok = torch.ones(1, device=device)
    parity = None
    if rank == 0:
        full, _ = sharding.prefill_chunk(q_full, kc_full, k_full, v_full, sharding.Chunk(0, 0, seqlen), TOPK,
                                         INIT_BLOCKS, LOCAL_BLOCKS)
        diff = (out_local.float() - full[rows_d].float()).abs().amax(dim=(1, 2))
        parity = {"rows": int(rows.numel()), "rows_bit_identical": round(float((diff == 0).float().mean()), 4),
                  "rows_within_2e-2": round(float((diff <= 2e-2).float().mean()), 4),
                  "max_abs": round(float(diff.max()), 5)}
        parity["pass"] = bool(parity["rows_within_2e-2"] >= 0.999)
        ok[0] = 1.0 if parity["pass"] else 0.0
        del full
    infllm_v2.check_device_status()
    gathered = (2 * seqlen * hk * D + (seqlen // STRIDE) * hk * D) * 2
    recv = gathered * (world - 1) // world                     # bytes that cross NVLink into one rank
    # algorithmic work of the whole sequence: stage 1 over the visible compressed keys, stage 2 over
    # min(64, bq + 1) selected blocks per token, the diagonal one partly visible
    n_comp = (seqlen - KERNEL) // STRIDE + 1
    t_idx = torch.arange(seqlen, dtype=torch.int64)
    nsel = ((t_idx // BLOCK) + 1).clamp(max=TOPK)
    pairs = int(((nsel - 1) * BLOCK + t_idx % BLOCK + 1).sum())
    flops = 2.0 * D * hk * 16 * visible_compressed(seqlen, n_comp) + 4.0 * D * hk * 16 * pairs
    res = {
        "n_gpus": world, "ms_step": round(t_step, 3), "ms_step_gather_first": round(t_serial, 3),
        "ms_allgather": round(t_gather, 3),
        "tokens_per_s": round(seqlen / (t_step * 1e-3), 1),
        "tflops": round(flops / t_step / 1e9, 1),
        "allgather_bytes_per_rank": gathered, "allgather_received_bytes_per_rank": recv,
        "allgather_gbs": round(gathered / t_gather / 1e6, 1),
        "allgather_received_gbs_per_rank": round(recv / t_gather / 1e6, 1),
        "parity_vs_unsharded_rank0": parity,
        "note": "one sequence, query chunks in zig-zag order over the ranks; step = all-gather of K, V and "
                "compressed K into local HBM (compressed K first, K / V on a side stream under the selection) "
                "+ fused stage 1 / top-k / mask / stage-2 forward per chunk; gather_first = everything "
                "gathered before any kernel; max over ranks"}
    if pk is not None:
        res["frac_of_n_gpu_tensor_roofline"] = round(flops / t_step / 1e9 / (world * pk["bf16_tflops_sustained"]), 4)
    return {f"sharded_prefill_{seqlen}_32q2kv": res}


def sharded_training_parity(device, rank, world, seqlen=16384, hk=2):
    """Forward + backward of one sequence under query-chunk sharding (all-gather of K / V, per-chunk
    backward, reduce-scatter of dK / dV over NCCL) against the same step on rank 0 alone."""
    from infllmv2_cuda_impl_b200 import sharding
    import infllm_v2
    g = torch.Generator(device=device).manual_seed(4321)
    s = 1.0 / math.sqrt(D)
    q = (torch.randn(seqlen, hk * 16, D, device=device, generator=g) * s).to(torch.bfloat16)
    k = (torch.randn(seqlen, hk, D, device=device, generator=g) * s).to(torch.bfloat16)
    v = (torch.randn(seqlen, hk, D, device=device, generator=g) * s).to(torch.bfloat16)
    do = torch.randn(seqlen, hk * 16, D, device=device, generator=g).to(torch.bfloat16)
    kc = infllm_v2.compress_keys(k)[0]
    # the selection is input to the training step (it carries no gradient): every rank computes the
    # same lists from the same tensors
    _, idx = sharding.prefill_chunk(q, kc, k, v, sharding.Chunk(0, 0, seqlen), TOPK, INIT_BLOCKS, LOCAL_BLOCKS)
    _, rows, _ = _zigzag_rows(seqlen, world, rank)
    rows_d = rows.to(device)
    fn = lambda: sharding.sharded_attention_fwd_bwd(q[rows_d], k[rows_d], v[rows_d], do[rows_d],
                                                    idx[:, rows_d].contiguous(), seqlen, world, rank)
    out, dq, dk, dv = fn()
    t = _timed_max(fn, device, reps=3, warmup=1)
    infllm_v2.check_device_status()
    res = {"n_gpus": world, "tokens": seqlen, "ms_fwd_bwd_step": round(t, 3)}
    if rank == 0:
        qd, kd, vd = (x.detach().clone().requires_grad_(True) for x in (q, k, v))
        cu = torch.tensor([0, seqlen], dtype=torch.int32, device=device)
        ref_out = infllm_v2.infllmv2_attn_varlen_func(qd, kd, vd, cu, cu, seqlen, seqlen, causal=True, topk_idx=idx)
        ref_out.backward(do)
        worst = {}
        good = True
        for name, a, b in (("out", out, ref_out.detach()), ("dq", dq, qd.grad), ("dk", dk, kd.grad), ("dv", dv, vd.grad)):
            b = b[rows_d].float()
            err = float((a.float() - b).abs().max())
            tol = 2e-2 * max(1.0, float(b.abs().max()))
            worst[name] = round(err, 5)
            good = good and err <= tol
        res.update(max_abs_vs_single_gpu=worst, tolerance="2e-2 x max(1, |ref|max)", **{"pass": bool(good)})
    return {"sharded_training_step_parity": res}


def sharded_decode_bench(device, rank, world, pk):
    """Decode at batch 64 with the sequences sharded over the ranks (64 / N per GPU, cache lengths
    uniform in [32768, 131072], 32q/2kv heads): stage 1 over the compressed keys, one-launch pool /
    top-64 / mask, sparse decode; replayed from a CUDA graph.  No collective: sequences are
    independent.  Throughput = 64 sequences / the slowest rank's step."""
    from infllmv2_cuda_impl_b200 import sharding
    import infllm_v2
    B, hk, lo, hi = 64, 2, 32768, 131072
    mine = list(sharding.batch_shard(B, world, rank))
    lens_all = torch.randint(lo, hi + 1, (B,), generator=torch.Generator().manual_seed(0)).to(torch.int32)
    lens = lens_all[mine]
    nb = len(mine)
    cap = hi + 64
    g = torch.Generator(device=device).manual_seed(100 + rank)
    s = 1.0 / math.sqrt(D)
    kcache = (torch.randn(nb, cap, hk, D, device=device, generator=g) * s).to(torch.bfloat16)
    vcache = (torch.randn(nb, cap, hk, D, device=device, generator=g) * s).to(torch.bfloat16)
    q = (torch.randn(nb, 1, hk * 16, D, device=device, generator=g) * s).to(torch.bfloat16)
    n_c = [(int(l) - KERNEL) // STRIDE + 1 for l in lens]
    kc = (torch.randn(sum(n_c), hk, D, device=device, generator=g) * s).to(torch.bfloat16)
    cu_q = torch.arange(nb + 1, dtype=torch.int32, device=device)
    cu_c = torch.tensor([0] + list(torch.tensor(n_c).cumsum(0)), dtype=torch.int32, device=device)
    lens_d = lens.to(device)
    positions = (lens_d - 1).contiguous()
    n_c_dev = torch.tensor(n_c, dtype=torch.int32, device=device)
    max_c, q2 = max(n_c), q.view(nb, hk * 16, D)

    def full_step():
        mask = infllm_v2.infllmv2_stage1_decode_select(q2, kc, cu_c, positions, max_c, cap, TOPK,
                                                       LOCAL_BLOCKS, INIT_BLOCKS, seqused_k=n_c_dev)
        return infllm_v2.infllmv2_attn_with_kvcache(q, kcache, vcache, cache_seqlens=lens_d, block_mask=mask)

    full_step()
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        full_step()
    torch.cuda.current_stream().wait_stream(side)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        full_step()
    t = _timed_max(graph.replay, device, reps=20, warmup=3)
    nbytes = torch.tensor([float(nb * hk * TOPK * BLOCK * D * 2 * 2 + kc.numel() * 2)], device=device)
    dist.all_reduce(nbytes)
    total = float(nbytes.item())
    return {"sharded_decode_b64_with_selection": {
        "n_gpus": world, "sequences_per_gpu": nb, "ms": round(t, 4), "tokens_per_s": round(B / (t * 1e-3), 1),
        "gbs_all_gpus": round(total / t / 1e6, 1),
        "frac_of_n_gpu_hbm": round(total / t / 1e6 / (world * pk["hbm_gbs"]), 4),
        "note": "batch sharded, no collective; CUDA-graph replay; max over ranks"}}


def multi_gpu_configs(device, rank, world, pk):
    """What the path does across GPUs besides the KV-head sharding of the headline step."""
    out = {}
    for name, fn in (("sharded_prefill", lambda: sharded_prefill_bench(device, rank, world, SEQLEN, pk=pk)),
                     ("sharded_training", lambda: sharded_training_parity(device, rank, world)),
                     ("sharded_decode", lambda: sharded_decode_bench(device, rank, world, pk))):
        try:
            out.update(fn())
        except Exception as e:                               # every rank takes the same branch or none
            out[name + "_error"] = repr(e)[:300]
        torch.cuda.empty_cache()
    return out


# ------------------------------------------------------------------------------ CPU baseline --

def _reference_functions():
    """The reference's own pure-PyTorch functions (its test oracles), when a checkout is reachable
    through INFLLMV2_REFERENCE (or at the default location below): torch_naive_softmax (stage 1) and
    convert_topk_to_base_blockmask / prepare_mixed_mask / attention_blocksparse_ref (stage 2).
    Returns None where there is no checkout (the GPU box): the CPU port in oracle/ is timed then."""
    import importlib
    import types
    root = os.environ.get("INFLLMV2_REFERENCE") or "/root/reference"
    tests_dir = os.path.join(root, "tests")
    if not os.path.isdir(tests_dir):
        return None
    try:
        for name in ("matplotlib", "matplotlib.pyplot", "matplotlib.colors", "seaborn"):
            sys.modules.setdefault(name, types.ModuleType(name))
        if "infllm_v2" not in sys.modules:            # the reference's tests import its CUDA module
            stub = types.ModuleType("infllm_v2")
            for fn in ("infllmv2_attn_stage1", "infllmv2_attn_varlen_func", "infllmv2_attn_with_kvcache",
                       "topk_to_uint64", "blockmask_to_uint64", "uint64_to_bool", "max_pooling_1d",
                       "max_pooling_1d_varlen"):
                setattr(stub, fn, None)
            sys.modules["infllm_v2"] = stub
        sys.path.insert(0, tests_dir)
        cwd = os.getcwd()
        os.chdir(tempfile.mkdtemp())                  # tests/utils.py creates a directory on import
        try:
            ns = importlib.import_module("stage1.naive_softmax")
            ut = importlib.import_module("utils")
        finally:
            os.chdir(cwd)
        return {"stage1": ns.torch_naive_softmax, "to_blockmask": ut.convert_topk_to_base_blockmask,
                "mixed_mask": ut.prepare_mixed_mask, "attention": ut.attention_blocksparse_ref}
    except Exception:
        return None


def cpu_chunk_starts(seqlen, n_chunks, chunk=16):
    """Starts of `n_chunks` chunks of `chunk` query tokens spread evenly over the sequence (the
    cost of a token grows with its position, so the sample must not sit at one end)."""
    return [min(seqlen - chunk, int((i + 0.5) * seqlen / n_chunks) // 64 * 64) for i in range(n_chunks)]


def cpu_sample(seqlen, sample_tokens, threads, ref=None):
    """The reference's pure-PyTorch CPU path (fp32, dense attention under the block mask) for
    `sample_tokens` query tokens of one `seqlen`-token sequence, all 128 query heads, taken as
    16-token chunks spread evenly over the sequence; each chunk is scored against the keys before
    its end (bottom-right alignment), exactly the work those tokens cost inside the full job.
    `ref`: the reference's own functions (stage 1 and stage 2; pool, top-k and the mask pack have
    no CPU form in the reference and come from oracle/ either way).  Returns seconds."""
    import oracle
    torch.set_num_threads(threads)
    g = torch.Generator().manual_seed(0)
    s = 1.0 / math.sqrt(D)
    k = (torch.randn(seqlen, HK, D, generator=g) * s).to(torch.bfloat16)
    v = (torch.randn(seqlen, HK, D, generator=g) * s).to(torch.bfloat16)
    chunk = 16
    starts = cpu_chunk_starts(seqlen, max(1, sample_tokens // chunk), chunk)
    qs = [(torch.randn(chunk, HQ, D, generator=g) * s).to(torch.bfloat16) for _ in starts]
    kc, _ = oracle.compress_keys(k, [0, seqlen], KERNEL, STRIDE)       # input preparation, not timed
    t0 = time.perf_counter()
    for st, q in zip(starts, qs):
        end = st + chunk
        n_pre = (end - KERNEL) // STRIDE + 1
        if ref is not None:
            score = ref["stage1"](q.float(), kc[:n_pre].float(), causal=True).to(torch.bfloat16)
        else:
            score = oracle.stage1_scores(q, kc[:n_pre], [0, chunk], [0, n_pre], n_pre, True).to(torch.bfloat16)
        pooled = oracle.max_pooling_1d(score, st, LOCAL_BLOCKS, INIT_BLOCKS, BLOCK, STRIDE)
        idx = oracle.topk_select(pooled, TOPK, (torch.arange(chunk) + st) // BLOCK)
        _mask = oracle.topk_to_uint64(idx.numpy(), end, BLOCK)
        if ref is not None:
            base = ref["to_blockmask"](idx, end, BLOCK, device="cpu")
            cu_q, cu_k = torch.tensor([0, chunk]), torch.tensor([0, end])
            mixed = ref["mixed_mask"](base, cu_q, cu_k, chunk, end, 1, nheads=HQ, nheads_k=HK,
                                      m_block_dim=16, n_block_dim=BLOCK)
            ref["attention"](q[None], k[None, :end], v[None, :end], mixed, causal=True)
        else:
            oracle.sparse_attention_fwd(q, k[:end], v[:end], [0, chunk], [0, end], idx, causal=True)
    return time.perf_counter() - t0


def cpu_baseline_object(seqlen, sample_tokens, threads, sec, kind):
    n = max(1, sample_tokens // 16) * 16
    how = ("the reference's own torch_naive_softmax + attention_blocksparse_ref" if kind == "reference"
           else "the CPU port of the reference's PyTorch path (oracle/)")
    return {"value": round(n / sec, 2), "unit": "tokens/s", "cores": threads, "kind": kind,
            "sample": f"{n} query tokens in 16-token chunks spread evenly over the {seqlen}-token sequence, "
                      f"all 128 query heads, fp32, {how}; stage1 + pool + top-64 + mask + dense-with-mask "
                      f"attention, {sec:.1f} s"}


def run_reference(args, rank, world):
    if rank != 0:
        return None
    threads = os.cpu_count() or 1
    sample = args.cpu_tokens
    ref = _reference_functions()
    kind = "reference" if ref is not None else "port"
    for _ in range(min(args.warmup, 1)):
        cpu_sample(args.seqlen, sample, threads, ref)
    times = [cpu_sample(args.seqlen, sample, threads, ref) for _ in range(args.steps)]
    sec = sum(times) / len(times)
    n = max(1, sample // 16) * 16
    val = n / sec
    return {
        "impl": "reference", "metric": METRIC, "value": round(val, 2), "unit": "tokens/s",
        "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": round(sec * 1e3, 2), "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": f"prefill {args.seqlen} tokens, 128q/8kv heads, d128 (CPU sample)",
                   "seq_len": args.seqlen, "global_batch": 1},
        "cpu_baseline": cpu_baseline_object(args.seqlen, sample, threads, sec, kind),
        "e2e": {"value": round(val, 2), "unit": "tokens/s", "h2d_bytes_per_step": 0,
                "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--seqlen", type=int, default=SEQLEN)
    ap.add_argument("--cpu-tokens", type=int, default=128,
                    help="query tokens in the CPU sample (cpu_baseline / --impl reference), in 16-token chunks")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--unfused", action="store_true",
                    help="run the reference's operator sequence: stage 1, max-pool, top-k, mask pack, stage 2")
    ap.add_argument("--only", default=None, choices=["selection", "topk", "compress", "coarse", "train", "decode", "sharded"],
                    help="run just one secondary config and print its numbers (profiling aid)")
    ap.add_argument("--small", action="store_true", help="with --only: a reduced size")
    ap.add_argument("--e2e-order", default="middle-out", choices=["middle-out", "ascending"],
                    help="order in which the host-to-host pipeline processes the query chunks")
    ap.add_argument("--e2e-chunk", type=int, default=4096,
                    help="query tokens per chunk of the host-to-host (e2e) pipeline")
    ap.add_argument("--e2e-split", type=int, default=4,
                    help="pieces into which the first and the last chunk of the e2e pipeline are cut")
    ap.add_argument("--no-extras", action="store_true",
                    help="skip the secondary configs (selection micro-benchmark, varlen fwd+bwd, decode)")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup
    # stdout carries the JSON line and nothing else: libraries that print to file descriptor 1
    # (NCCL's version banner) go to stderr for the length of the run
    sys.stdout.flush()
    json_fd = os.dup(1)
    os.dup2(2, 1)
    sys.stdout = os.fdopen(json_fd, "w")

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))

    if args.impl == "reference":
        res = run_reference(args, rank, world)
        if res is not None:
            print(json.dumps(res), flush=True)
        return

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the library has no CPU path "
                         "(use --impl reference for the CPU oracle)")
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=device)
    if args.only == "sharded":
        if world < 2:
            raise SystemExit("--only sharded needs at least two ranks (torchrun)")
        res = multi_gpu_configs(device, rank, world, peaks()[0])
        if rank == 0:
            print(json.dumps(res), flush=True)
        dist.barrier()
        dist.destroy_process_group()
        return
    if args.only is not None:
        print(json.dumps(extra_configs(device, peaks()[0], args.only, args.small)), flush=True)
        return
    res = run_ours(args, rank, world, device)
    multi = None
    if world > 1 and not args.no_extras and args.seqlen == SEQLEN:
        torch.cuda.empty_cache()
        multi = multi_gpu_configs(device, rank, world, peaks()[0])
    if rank == 0:
        if multi is not None:
            res["other_configs"] = multi
        if world == 1 and not args.no_extras and args.seqlen == SEQLEN:
            torch.cuda.empty_cache()
            try:
                res["other_configs"] = extra_configs(device, peaks()[0])
            except Exception as e:                         # the headline line must still be printed
                res["other_configs"] = {"error": repr(e)[:300]}
        if not args.no_cpu_baseline:
            threads = os.cpu_count() or 1
            ref = _reference_functions()
            sec = cpu_sample(args.seqlen, args.cpu_tokens, threads, ref)
            res["cpu_baseline"] = cpu_baseline_object(args.seqlen, args.cpu_tokens, threads, sec,
                                                      "reference" if ref is not None else "port")
        print(json.dumps(res), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
