#!/usr/bin/env python3
"""Benchmark of the fused Matmul -> row-Softmax chain.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload cfg2] [--impl reference]

One step = one call of the chain on one batch of synthetic input.  The headline
workload is the f16-native chain A[4096,1024] . B[1024,1024], scale 1/32, f16
probabilities; with N GPUs every rank runs its own 4096 rows against a replicated B
(rows are independent: no data-path collective, weak scaling).  The same JSON line
carries, under `scaling_cfg3` and `scaling_cfg4`, the two splits of a FIXED problem
over the N GPUs: the 64 batches of the attention-score chain (no collective) and the
columns of the vocab-wide chain (one all-gather of per-row (max, sum) pairs).
Prints ONE JSON line (rank 0).  `--impl reference` times the CPU restatement of the
chain (scalar loop nest, all host threads) on the same workload.
"""
from __future__ import annotations

import argparse
import json
import math
import os
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

# name -> batch, M, N, K, scale, sigma of B, B batched?, how N GPUs share it
WORKLOADS = {
    "cfg1": dict(batch=1, M=128, N=128, K=128, scale=1.0, sigma_b=1.0, b_batched=False, dtype="f32", shard="replica",
                 desc="decomposed f32 chain 128x128x128"),
    "cfg2": dict(batch=1, M=4096, N=1024, K=1024, scale=1.0 / 32, sigma_b=1.0, b_batched=False, dtype="f16", shard="rows",
                 desc="f16 native chain 4096x1024x1024, f32 accumulate, scale 1/32"),
    "cfg3": dict(batch=64, M=2048, N=2048, K=128, scale=128 ** -0.5, sigma_b=1.0, b_batched=True, dtype="f16", shard="batch",
                 desc="batched attention scores 64 x (2048x128 . 128x2048), scale 1/sqrt(128)"),
    "cfg4": dict(batch=1, M=8192, N=32000, K=4096, scale=1.0, sigma_b=0.02, b_batched=False, dtype="f16", shard="cols",
                 desc="vocab-wide logits 8192x4096 . 4096x32000, online two-pass"),
    "cfg5": dict(batch=1, M=16, N=32000, K=4096, scale=1.0, sigma_b=0.02, b_batched=False, dtype="f16", shard="replica",
                 desc="skinny decode 16x4096 . 4096x32000"),
    "cfg4s": dict(batch=1, M=1024, N=32000, K=4096, scale=1.0, sigma_b=0.02, b_batched=False, dtype="f16", shard="cols",
                  desc="vocab-wide logits at an eighth of the rows (1024x4096 . 4096x32000): the size profiler captures of the two-pass kernels use"),
    "ref": dict(batch=1, M=8192, N=128, K=64, scale=1.0, sigma_b=1.0, b_batched=False, dtype="f16", shard="rows",
                desc="the reference's own shape 8192x64 . 64x128"),
}
SHARDING_TEXT = {"rows": "each GPU its own M rows, B replicated, no collective",
                 "batch": "batches split over the GPUs, no collective",
                 "cols": "N split on 256-column tile boundaries, one all-gather of per-row (max,sum)",
                 "replica": "independent replicas"}
L2_BYTES = 126 * 1024 * 1024
HBM_BOUND = ("cfg3", "cfg5")

# DRAM traffic of the dominant kernel, bytes per launch, from the ncu captures summarised under
# profiles/ (dram__bytes_read.sum + dram__bytes_write.sum of ONE captured launch; output lines that
# are still in L2 when the launch ends are not in the write figure).
NCU_TRAFFIC = {
    "cfg2": dict(bytes=10550016, capture="profiles/fused_tc_kernel_cfg2_4096x1024x1024.md",
                 note="single cold launch, write-back not counted: the 8.39 MB of output was still in L2 when it ended"),
    "cfg3": dict(bytes=546158336, capture="profiles/fused_tc_kernel_cfg3_batched_64x2048x2048x128.md",
                 note="single launch; 58 MB of the output was still in L2 when it ended"),
    "cfg4": dict(bytes=2172000000, capture="profiles/fused_tc_kernel_cfg4_tiled_pair_1024x32000x4096.md",
                 note="both kernels, scaled from a capture at M = 1024 by the rows processed (B streamed once per 4096 rows)"),
    "cfg4s": dict(bytes=407866368, capture="profiles/fused_tc_kernel_cfg4_tiled_pair_1024x32000x4096.md",
                  note="both kernels, single launches"),
    "cfg5": dict(bytes=266929664, capture="profiles/fused_tc_kernel_cfg5_skinny_16x32000x4096.md",
                 note="both kernels, single launches"),
}


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        p = json.load(open(path))
        return dict(hbm_gbs=float(p["hbm_gbs"]), tflops=float(p["bf16_tflops"]), source="measured")
    return dict(hbm_gbs=6650.0, tflops=1590.0, source="fallback")


def algorithmic(wl, batch=None, M=None, N=None):
    b = wl["batch"] if batch is None else batch
    M = wl["M"] if M is None else M
    N = wl["N"] if N is None else N
    K = wl["K"]
    es = 2 if wl["dtype"] == "f16" else 4
    flops = 2.0 * b * M * N * K
    bytes_ = es * (b * M * K + (b if wl["b_batched"] else 1) * K * N + b * M * N)
    return flops, bytes_


def config_for(name, wl, world):
    """The `config` object: the same in both arms (ours and --impl reference)."""
    return dict(workload=f"{name}: {wl['desc']}",
                problem=dict(batch=wl["batch"], M=wl["M"], N=wl["N"], K=wl["K"], scale=wl["scale"], in_dtype=wl["dtype"],
                             accumulate="f32", out_dtype=wl["dtype"]),
                sharding=SHARDING_TEXT[wl["shard"]], n_gpus=world,
                timing="mean over the timed steps, back to back; the GPU arm rotates buffer sets larger than L2 between steps")


def host_threads():
    """Threads this process may run on (the affinity mask, not OMP_NUM_THREADS: launchers such as
    torchrun set that variable to 1 for every rank)."""
    try:
        return max(1, len(os.sched_getaffinity(0)))
    except AttributeError:
        return max(1, os.cpu_count() or 1)


class ClockSampler(threading.Thread):
    """Samples SM clock and throttle reasons of one GPU through NVML while the timed region runs."""

    def __init__(self, index):
        super().__init__(daemon=True)
        self.index = index
        self.samples, self.reasons, self.max_mhz = [], set(), None
        self._stop_evt = threading.Event()
        self.ok = False
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            self.h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM)
            self.ok = True
        except Exception:
            self.ok = False

    def run(self):
        if not self.ok:
            return
        nv = self.nv
        names = {
            getattr(nv, "nvmlClocksThrottleReasonHwSlowdown", 0x8): "hw_slowdown",
            getattr(nv, "nvmlClocksThrottleReasonHwThermalSlowdown", 0x40): "hw_thermal_slowdown",
            getattr(nv, "nvmlClocksThrottleReasonSwThermalSlowdown", 0x20): "sw_thermal_slowdown",
            getattr(nv, "nvmlClocksThrottleReasonSwPowerCap", 0x4): "sw_power_cap",
        }
        self._names = names
        while not self._stop_evt.is_set():
            self._sample()
            time.sleep(0.02)

    def _sample(self):
        try:
            nv = self.nv
            self.samples.append(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM))
            r = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h)
            for bit, name in self._names.items():
                if r & bit:
                    self.reasons.add(name)
        except Exception:
            pass

    def mark(self):
        """Start of a timed region: forget what was sampled before it."""
        self.samples, self.reasons = [], set()

    def snapshot(self):
        """Call with the timed work still in flight: takes one more sample (short regions fall
        between two polls of the thread) and reports the region's clocks."""
        if self.ok and hasattr(self, "_names"):
            self._sample()
        if not self.samples:
            return dict(sm_mhz=None, sm_max_mhz=self.max_mhz, reasons=sorted(self.reasons))
        s = sorted(self.samples)
        return dict(sm_mhz=s[len(s) // 2], sm_max_mhz=self.max_mhz, reasons=sorted(self.reasons))

    def stop(self):
        self._stop_evt.set()
        if self.is_alive():
            self.join(timeout=1)


def run_reference(args, wl):
    """CPU arm: the loop-nest restatement of the chain on all host threads.  A step is the whole
    workload when that takes about a second or less on this host, else a row sample of it (rows
    are independent, so a row sample scales)."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    import numpy as np
    from oracle import oracle
    threads = host_threads()
    dt = np.float16 if wl["dtype"] == "f16" else np.float32
    total_rows = wl["batch"] * wl["M"]
    B = oracle.normal((wl["K"], wl["N"]), 2, wl["sigma_b"], dt)
    # calibrate on a small slice, then size a step to about one second at most
    probe = max(1, min(total_rows, int(2.0e8 / (2.0 * wl["N"] * wl["K"])) or 1))
    Ap = oracle.normal((probe, wl["K"]), 1, 1.0, dt)
    oracle.chain_loops_f32(Ap, B, wl["scale"], threads)
    t0 = time.perf_counter()
    oracle.chain_loops_f32(Ap, B, wl["scale"], threads)
    per_row = max(1e-9, (time.perf_counter() - t0) / probe)
    rows = max(1, min(total_rows, int(1.0 / per_row)))
    A = oracle.normal((rows, wl["K"]), 1, 1.0, dt)
    for _ in range(max(1, min(args.warmup, 2))):
        oracle.chain_loops_f32(A, B, wl["scale"], threads)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        oracle.chain_loops_f32(A, B, wl["scale"], threads)
    dt_s = (time.perf_counter() - t0) / args.steps
    flops = 2.0 * rows * wl["N"] * wl["K"]
    value = flops / dt_s / 1e12
    sample = (f"{rows} of {total_rows} rows per step" + (" (the whole workload)" if rows == total_rows else
              " (rows are independent; throughput is per-row work / time)") +
              f"; scalar loop nest, f32 accumulate, separate max/exp/sum/div passes, {threads} threads")
    line = dict(impl="reference", metric="fused_matmul_softmax_tflops", value=value, unit="TFLOP/s",
                n_gpus=args.gpus, steps=args.steps, warmup=args.warmup, ms_per_step=dt_s * 1e3,
                higher_is_better=True, scaling="weak", vs_baseline=None, dtype=wl["dtype"], data="synthetic",
                config=config_for(args.workload, wl, args.gpus),
                cpu_baseline=dict(value=value, unit="TFLOP/s", cores=threads, kind="port", sample=sample),
                e2e=dict(value=value, unit="TFLOP/s", h2d_bytes_per_step=0, d2h_bytes_per_step=0),
                gpu_launches=0)
    print(json.dumps(line), flush=True)


class Ctx:
    """What every measurement needs: the process group (if any), this rank's device, the library."""

    def __init__(self):
        import torch
        import torch.distributed as dist
        import welder_typical_chain_b200 as wtc
        self.torch, self.dist, self.wtc = torch, dist, wtc
        self.world = int(os.environ.get("WORLD_SIZE", "1"))
        self.rank = int(os.environ.get("RANK", "0"))
        self.local = int(os.environ.get("LOCAL_RANK", "0"))
        if not torch.cuda.is_available():
            raise SystemExit("bench.py needs a CUDA device: the chain has no CPU path (use --impl reference for the CPU baseline)")
        torch.cuda.set_device(self.local)
        self.dev = torch.device("cuda", self.local)
        if self.world > 1:
            dist.init_process_group("nccl", device_id=self.dev)
        self.sampler = ClockSampler(self.local)
        self.sampler.start()

    def barrier(self):
        if self.world > 1:
            self.dist.barrier()
        self.torch.cuda.synchronize()

    def max_over_ranks(self, x):
        t = self.torch.tensor([x], device=self.dev, dtype=self.torch.float64)
        if self.world > 1:
            self.dist.all_reduce(t, op=self.dist.ReduceOp.MAX)
        return float(t.item())

    def sum_over_ranks(self, x):
        t = self.torch.tensor([x], device=self.dev, dtype=self.torch.float64)
        if self.world > 1:
            self.dist.all_reduce(t, op=self.dist.ReduceOp.SUM)
        return float(t.item())

    def close(self):
        self.sampler.stop()
        if self.world > 1:
            self.dist.destroy_process_group()


def measure(ctx, name, steps, warmup, parity=True, e2e=False, isolated=False):
    """Times `steps` back-to-back calls of workload `name` on this job's GPUs (device events, max
    over ranks) after a parity check against the CPU checker.  Returns a dict (the same on every
    rank for the reduced figures)."""
    import numpy as np
    torch, dist, wtc = ctx.torch, ctx.dist, ctx.wtc
    from welder_typical_chain_b200 import sharding
    wl = WORKLOADS[name]
    world, rank, dev = ctx.world, ctx.rank, ctx.dev
    tdt = torch.float16 if wl["dtype"] == "f16" else torch.float32
    out_code = wtc.F16 if wl["dtype"] == "f16" else wtc.F32
    batch, M, N, K, scale = wl["batch"], wl["M"], wl["N"], wl["K"], wl["scale"]
    shard = wl["shard"]
    scaling = "weak"
    n_local, c0 = N, 0
    if shard == "batch" and world > 1:           # fixed 64 batches split over the ranks
        b0, b1 = sharding.split_batches(batch, world)[rank]
        batch = b1 - b0
        scaling = "strong"
    elif shard == "cols" and world > 1:          # N split on 256-column tile boundaries
        c0, c1 = sharding.split_columns(N, world)[rank]
        n_local = c1 - c0
        scaling = "strong"
    elif shard in ("batch", "cols"):
        scaling = "strong"                       # one GPU runs the whole fixed problem
    col_sharded = shard == "cols" and world > 1

    flops_step, bytes_step = algorithmic(wl, batch=batch, N=n_local)
    # rotating buffer sets so that consecutive steps never find their operands in L2
    set_bytes = bytes_step
    nsets = max(2, min(64, math.ceil(2.4 * L2_BYTES / max(set_bytes, 1))))
    if set_bytes > 2 * L2_BYTES:
        nsets = 1 if set_bytes > 8e9 else 2
    g = torch.Generator(device=dev)
    # a column shard must see the SAME A and B as its peers (it owns a slice of B's columns): one seed
    g.manual_seed(1234 + (0 if col_sharded else rank))
    a_shape = (batch, M, K) if batch > 1 else (M, K)
    b_full_shape = (batch, K, N) if (wl["b_batched"] and batch > 1) else (K, N)
    o_shape = (batch, M, n_local) if batch > 1 else (M, n_local)
    sets, full_b0 = [], None
    for i in range(nsets):
        A = torch.randn(a_shape, device=dev, dtype=torch.float32, generator=g).to(tdt)
        B = (torch.randn(b_full_shape, device=dev, dtype=torch.float32, generator=g) * wl["sigma_b"]).to(tdt)
        if col_sharded:
            if i == 0 and rank == 0 and parity:
                full_b0 = B.cpu().numpy()
            B = B[:, c0:c0 + n_local].contiguous()
        O = torch.empty(o_shape, device=dev, dtype=tdt)
        sets.append((A, B, O))
    desc = wtc.launch._desc_for(sets[0][0], sets[0][1], out_code, scale, wtc.F32, wtc.VARIANT_FUSED, 0, None)
    plan = wtc.plan_query(desc)
    ws_bytes = wtc.workspace_bytes(desc)
    ws = torch.empty(max(ws_bytes, 16), device=dev, dtype=torch.uint8)
    rows_total = batch * M
    sptr = wtc.current_stream_ptr()
    if col_sharded:
        row_stats = torch.empty((rows_total, 2), device=dev, dtype=torch.float32)
        all_stats = torch.empty((world * rows_total, 2), device=dev, dtype=torch.float32)   # rank-major [world][rows][2]
        shard_calls = [wtc.PreparedShardCall(A, B, O, scale, ws, row_stats, all_stats, world) for (A, B, O) in sets]

        def step(i):
            c = shard_calls[i % nsets]
            c.partial(sptr)
            dist.all_gather_into_tensor(all_stats, row_stats)      # [M,2] f32 per rank over NVLink
            c.finish(sptr)
    else:
        prepared = [wtc.PreparedCall(A, B, O, scale, workspace=ws) for (A, B, O) in sets]

        def step(i):
            prepared[i % nsets].launch(sptr)

    # ---- parity on this job's first buffer set (sampled rows, CPU checker) ----
    par = None
    if parity:
        from oracle import oracle
        step(0)
        torch.cuda.synchronize()
        A, B, O = sets[0]
        if col_sharded:
            # the sampled rows' columns of every rank are put side by side on rank 0 and checked
            # as whole rows against the checker run on the whole B
            idx = sorted(set(int(x) for x in np.linspace(0, M - 1, 8)))
            mine = O[idx].cpu().numpy()
            parts = [None] * world
            dist.all_gather_object(parts, mine)
            if rank == 0:
                got = np.concatenate(parts, axis=1)
                par = oracle.compare(got, oracle.chain(A[idx].cpu().numpy(), full_b0, scale))
                par["rows_checked"] = len(idx)
                par["note"] = "whole rows assembled from every rank's columns"
            flag = [par["ok"] if rank == 0 else None]
            dist.broadcast_object_list(flag, src=0)
            if not flag[0]:
                raise SystemExit(f"{name}: column-sharded parity check failed: {par}")
        else:
            A2 = A.reshape(-1, M, K)[0]
            B2 = B.reshape(-1, K, n_local)[0]
            O2 = O.reshape(-1, M, n_local)[0]
            rows_n = 24 if N * K <= (1 << 22) else 8
            idx = sorted(set(int(x) for x in np.linspace(0, M - 1, rows_n)))
            par = oracle.compare(O2[idx].cpu().numpy(), oracle.chain(A2[idx].cpu().numpy(), B2.cpu().numpy(), scale))
            par["rows_checked"] = len(idx)
            if not par["ok"]:
                raise SystemExit(f"{name}: parity check failed before timing: {par}")

    for i in range(warmup):
        step(i)
    wtc.check_device_status()
    ctx.barrier()
    ctx.sampler.mark()
    stream = torch.cuda.current_stream()
    e0 = torch.cuda.Event(enable_timing=True)
    e1 = torch.cuda.Event(enable_timing=True)
    e0.record(stream)
    for i in range(steps):
        step(i)
    e1.record(stream)
    clocks = ctx.sampler.snapshot()    # the queue is still draining: this sample is under load
    ctx.barrier()
    ms = e0.elapsed_time(e1)
    wtc.check_device_status()
    ms_max = ctx.max_over_ranks(ms)
    total_flops_step = ctx.sum_over_ranks(flops_step)
    total_bytes_step = ctx.sum_over_ranks(bytes_step)
    ms_per_step = ms_max / steps
    value = total_flops_step / (ms_per_step * 1e-3) / 1e12

    res = dict(name=name, wl=wl, plan=plan, scaling=scaling, batch=batch, M=M, n_local=n_local, K=K, nsets=nsets, set_bytes=set_bytes,
               ms_per_step=ms_per_step, value=value, parity=par, clocks=clocks, flops_step=flops_step, bytes_step=bytes_step,
               total_flops_step=total_flops_step, total_bytes_step=total_bytes_step, rank_ms_per_step=ms / steps,
               launches_per_step=plan.launches + (1 if col_sharded else 0), steps=steps)

    # ---- column-sharded: where a step's time goes on this rank's device (a few steps with events between the phases)
    if col_sharded:
        ph = []
        for i in range(5):
            ev = [torch.cuda.Event(enable_timing=True) for _ in range(4)]
            c = shard_calls[i % nsets]
            ev[0].record(stream); c.partial(sptr); ev[1].record(stream)
            dist.all_gather_into_tensor(all_stats, row_stats); ev[2].record(stream)
            c.finish(sptr); ev[3].record(stream)
            torch.cuda.synchronize()
            ph.append([ev[k].elapsed_time(ev[k + 1]) * 1e3 for k in range(3)])
        ph = np.median(np.array(ph), axis=0)
        res["phases_us"] = dict(partial=ctx.max_over_ranks(float(ph[0])), gather=ctx.max_over_ranks(float(ph[1])),
                                finish=ctx.max_over_ranks(float(ph[2])),
                                note="median of 5 steps with events between the phases, max over ranks; "
                                     "the gather is one NCCL all-gather of [rows,2] f32 per rank")

    # ---- HBM-bound workloads: what a plain fill of this rank's output buffer takes.  The copy figure
    #      that `roofline.peak` holds counts reads and writes together; a stream of writes alone is
    #      slower on this part, and a kernel whose traffic is nearly all output cannot beat it.
    if name in HBM_BOUND and 2 * sets[0][2].numel() * sets[0][2].element_size() >= res["bytes_step"]:
        O = sets[0][2]
        fills = []
        for i in range(8):
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record(stream)
            sets[i % len(sets)][2].fill_(0.5)
            b.record(stream)
            b.synchronize()
            fills.append(a.elapsed_time(b) * 1e3)
        fill_us = ctx.max_over_ranks(float(min(fills[2:])))
        res["fill_us"] = fill_us
        res["fill_bytes"] = int(O.numel() * O.element_size())

    # ---- isolated calls (the stream is idle before each), each between its own pair of events, this rank
    if isolated:
        single = []
        for i in range(min(steps, 30)):
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record(stream)
            step(i)
            b.record(stream)
            b.synchronize()
            single.append(a.elapsed_time(b) * 1e3)
        single.sort()
        res["isolated_us"] = (single[0], single[len(single) // 2])
        # the same loop with the opt-in promise that the operands do not depend on earlier work on the
        # stream (true here: they are resident before the loop): loads then run under the previous call's
        # tail.  Reported beside the headline, which does not use the flag.
        if not col_sharded and wl["dtype"] == "f16":
            ready = [wtc.PreparedCall(A, B, O, scale, workspace=ws, flags=wtc.FLAG_OPERANDS_READY) for (A, B, O) in sets]
            for i in range(max(3, warmup)):
                ready[i % nsets].launch(sptr)
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            ctx.barrier()
            torch.cuda.synchronize()
            a.record(stream)
            for i in range(steps):
                ready[i % nsets].launch(sptr)
            b.record(stream)
            torch.cuda.synchronize()
            res["operands_ready_us"] = ctx.max_over_ranks(a.elapsed_time(b) * 1e3 / steps)

    # ---- end to end: host buffers in, host buffer out, through the C-ABI host entry point ----
    if e2e and not col_sharded:
        A, B, O = sets[0]
        hA = torch.empty(A.shape, dtype=tdt, pin_memory=True).copy_(A)
        hB = torch.empty(B.shape, dtype=tdt, pin_memory=True).copy_(B)
        hO = torch.empty(O.shape, dtype=tdt, pin_memory=True)
        hO2 = torch.empty(O.shape, dtype=tdt, pin_memory=True)
        nA, nB, nO = hA.numpy(), hB.numpy(), (hO.numpy(), hO2.numpy())
        e2e_steps = max(3, min(steps, int(2.0 / max(1e-4, (hA.nbytes + hB.nbytes + hO.nbytes) / 20e9))))
        # (a) one call at a time: copy in, kernels, copy back, wait -- the latency of a lone call
        for _ in range(3):
            wtc.matmul_softmax_host(nA, nB, scale, out=nO[0], out_dtype=out_code)
        ctx.barrier()
        t0 = time.perf_counter()
        for _ in range(e2e_steps):
            wtc.matmul_softmax_host(nA, nB, scale, out=nO[0], out_dtype=out_code)
        dt_sync = ctx.max_over_ranks((time.perf_counter() - t0) / e2e_steps)
        # (b) a stream of calls through the same entry point's two halves, two in flight: while the
        #     rows of step i travel back, the operands of step i+1 travel in.  Every step still moves
        #     its own operands host -> device and its own result device -> host inside the timed region.
        hc = wtc.HostChain(A.shape[0] if A.dim() == 3 else 1, A.shape[-2], B.shape[-1], A.shape[-1], scale,
                           in_dtype=out_code, out_dtype=out_code, shared_b=(A.dim() == 3 and B.dim() == 2))
        for i in range(4):
            hc.wait(hc.submit(nA, nB, nO[i & 1]))
        ctx.barrier()
        t0 = time.perf_counter()
        prev = -1
        for i in range(e2e_steps):
            t = hc.submit(nA, nB, nO[i & 1])
            hc.wait(prev)
            prev = t
        hc.wait(prev)
        dt_s = ctx.max_over_ranks((time.perf_counter() - t0) / e2e_steps)
        ok_e2e = bool(torch.equal(hO, hO2))          # both slots' results, same inputs
        moved = hA.nbytes + hB.nbytes + hO.nbytes
        res["e2e"] = dict(value=total_flops_step / dt_s / 1e12, unit="TFLOP/s",
                          h2d_bytes_per_step=int(hA.nbytes + hB.nbytes), d2h_bytes_per_step=int(hO.nbytes),
                          ms_per_step=dt_s * 1e3, steps=e2e_steps,
                          pcie_gbs_per_rank=moved / dt_s / 1e9,
                          one_call_at_a_time=dict(ms_per_step=dt_sync * 1e3, value=total_flops_step / dt_sync / 1e12),
                          results_identical_across_slots=ok_e2e,
                          api="wtc_matmul_softmax_host_submit / _wait, two calls in flight (pinned host buffers; every step's "
                              "copies inside the timed region); one_call_at_a_time = wtc_matmul_softmax_host",
                          note="every rank moves its own operands and result over its own PCIe link; the ranks of one "
                               "host share the host's memory and root ports, which is what limits this figure at N > 1")
    del sets
    torch.cuda.empty_cache()
    return res


def measure_row_chains(ctx, pk, steps):
    """The two row-only chains of the reference's backend inputs (row softmax of a given matrix; row
    variance broadcast along the row) on this rank's GPU: microseconds per call over rotating buffers
    larger than L2, bytes read + written per second against the measured copy rate, and a check of a
    few rows against the CPU checker.  Rank 0 only (the chains shard by rows without any exchange)."""
    import numpy as np
    from oracle import oracle
    torch, wtc = ctx.torch, ctx.wtc
    out = {}
    cases = [("row_softmax", "f16", 65536, 2048), ("row_softmax", "f32", 65536, 2048), ("row_softmax", "f16", 8192, 32000),
             ("row_variance", "f32", 16384, 8192), ("row_variance", "f16", 8192, 32000)]
    for kind, dt, rows, n in cases:
        tdt = torch.float16 if dt == "f16" else torch.float32
        xs = [torch.randn((rows, n), device=ctx.dev, dtype=torch.float32).mul_(2.0).to(tdt) for _ in range(3)]
        outs = [torch.empty_like(x) for x in xs]
        fn = wtc.row_softmax if kind == "row_softmax" else wtc.row_variance
        for i in range(3):
            fn(xs[i], out=outs[i])
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        k = max(6, min(steps, 30))
        a.record()
        for i in range(k):
            fn(xs[i % 3], out=outs[i % 3])
        b.record()
        torch.cuda.synchronize()
        us = a.elapsed_time(b) * 1e3 / k
        nbytes = 2 * rows * n * xs[0].element_size()
        sample = [0, 1, rows // 2, rows - 1]
        x = xs[(k - 1) % 3][sample].cpu().numpy()
        got = outs[(k - 1) % 3][sample].cpu().numpy().astype(np.float64)
        if kind == "row_softmax":
            ok = bool(oracle.compare(got, oracle.row_softmax(x))["ok"])
        else:
            ref = oracle.row_variance(x)
            ok = bool(np.abs(got - ref).max() <= (2e-3 if dt == "f16" else 1e-4) * np.abs(ref).max())
        out[f"{kind}_{dt}_{rows}x{n}"] = dict(us_per_call=us, gbs=nbytes / us / 1e3, frac_of_copy_rate=nbytes / us / 1e3 / pk["hbm_gbs"],
                                              bytes=nbytes, parity_ok=ok)
        del xs, outs
        torch.cuda.empty_cache()
    return out


def roofline_of(res, pk):
    name = res["name"]
    launch_s = res["ms_per_step"] * 1e-3
    if name in HBM_BOUND:
        achieved = res["total_bytes_step"] / launch_s / 1e9 / max(1, res.get("world", 1))
        roof = dict(bound="hbm", achieved=achieved, peak=pk["hbm_gbs"], unit="GB/s", frac=achieved / pk["hbm_gbs"])
    else:
        achieved = res["total_flops_step"] / launch_s / 1e12 / max(1, res.get("world", 1))
        roof = dict(bound="tensor", achieved=achieved, peak=pk["tflops"], unit="TFLOP/s", frac=achieved / pk["tflops"])
    roof["peak_source"] = pk["source"]
    roof["per"] = "GPU (whole-job figure / n_gpus); step time = max over ranks"
    t = NCU_TRAFFIC.get(name)
    world = max(1, res.get("world", 1))
    strong = WORKLOADS[name]["shard"] in ("batch", "cols")      # the whole workload is cut over the GPUs
    roof["traffic"] = (t["bytes"] // world if strong else t["bytes"]) if t else None
    if t:
        roof["traffic_source"] = f"{t['capture']}: {t['note']}" + (f"; divided by the {world} GPUs that share the workload" if strong and world > 1 else "")
    roof["algorithmic_per_launch"] = dict(flops=res["flops_step"], bytes=res["bytes_step"])
    if res.get("fill_us"):
        roof["write_stream"] = dict(fill_us=res["fill_us"], fill_gbs=res["fill_bytes"] / res["fill_us"] / 1e3,
                                    output_bytes_per_gpu=res["fill_bytes"], call_us=res["ms_per_step"] * 1e3,
                                    fill_over_call=res["fill_us"] / (res["ms_per_step"] * 1e3),
                                    note="a torch fill_ of this GPU's output buffer, timed here with CUDA events: the time "
                                         "the output alone needs as a plain stream of writes")
    return roof


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=400)
    ap.add_argument("--warmup", type=int, default=20)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="cfg2", choices=sorted(WORKLOADS))
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-parity", action="store_true")
    ap.add_argument("--no-splits", action="store_true", help="skip the scaling_cfg3 / scaling_cfg4 measurements")
    ap.add_argument("--no-siblings", action="store_true", help="skip the row-only chains (row softmax, row variance)")
    args = ap.parse_args()
    wl = WORKLOADS[args.workload]
    if args.warmup < 3:
        args.warmup = 3

    if args.impl == "reference":
        run_reference(args, wl)
        return

    import numpy as np
    ctx = Ctx()
    wtc = ctx.wtc
    world, rank = ctx.world, ctx.rank
    pk = peaks()

    head = measure(ctx, args.workload, args.steps, args.warmup, parity=not args.no_parity, e2e=not args.no_e2e, isolated=True)
    head["world"] = world

    # the two splits of a fixed problem over the N GPUs, in the same record
    splits = {}
    if args.workload == "cfg2" and not args.no_splits:
        for nm, st in (("cfg3", min(args.steps, 50)), ("cfg4", min(args.steps, 20))):
            r = measure(ctx, nm, st, max(3, min(args.warmup, 5)), parity=not args.no_parity)
            r["world"] = world
            splits[nm] = r

    if rank != 0:
        ctx.close()
        return

    plan = head["plan"]
    roof = roofline_of(head, pk)
    roof["kernel"] = wtc.launch.KERNEL_NAMES[plan.kernel]
    # (rank 0 alone from here on: the other ranks have left; nothing below is a collective)
    siblings = None
    if args.workload == "cfg2" and not args.no_siblings and world == 1:
        siblings = measure_row_chains(ctx, pk, args.steps)

    cpu = None
    if not args.no_cpu_baseline and world == 1:
        from oracle import oracle
        M, N, K, scale = wl["M"], wl["N"], wl["K"], wl["scale"]
        threads = host_threads()
        rows = max(1, min(M, int(6.0e9 / (2.0 * N * K))))
        dtn = np.float16 if wl["dtype"] == "f16" else np.float32
        A = oracle.normal((rows, K), 1, 1.0, dtn)
        B = oracle.normal((K, N), 2, wl["sigma_b"], dtn)
        oracle.chain_loops_f32(A, B, scale, threads)
        reps, t0 = 0, time.perf_counter()
        while reps < 3 or time.perf_counter() - t0 < 8.0:
            oracle.chain_loops_f32(A, B, scale, threads)
            reps += 1
            if time.perf_counter() - t0 > 25.0:
                break
        dt_s = (time.perf_counter() - t0) / reps
        cpu = dict(value=2.0 * rows * N * K / dt_s / 1e12, unit="TFLOP/s", cores=threads, kind="port",
                   sample=f"{rows} of {wl['batch'] * M} rows, {reps} repetitions of the scalar loop-nest restatement "
                          f"(f32 accumulate, separate max/exp/sum/div passes), rows spread over {threads} threads")
        # the same loop nest on ONE thread (what a plain linalg-to-loops lowering runs as), on a smaller slice
        rows1 = max(1, min(rows, int(2.0e9 / (2.0 * N * K))))
        t1 = time.perf_counter()
        oracle.chain_loops_f32(A[:rows1], B, scale, 1)
        dt1 = time.perf_counter() - t1
        cpu["single_thread"] = dict(value=2.0 * rows1 * N * K / dt1 / 1e12, unit="TFLOP/s", cores=1,
                                    sample=f"{rows1} rows, one pass")

    def plan_dict(r):
        p = r["plan"]
        return dict(kernel=wtc.launch.KERNEL_NAMES[p.kernel], cluster_n=p.cluster_n, tile=[p.tile_m, p.tile_n, p.tile_k],
                    stages=p.stages, threads=p.threads, launches_per_step=r["launches_per_step"],
                    per_gpu=dict(batch=r["batch"], M=r["M"], N=r["n_local"], K=r["K"]),
                    l2=f"{r['nsets']} rotating buffer sets of {r['set_bytes'] / 1e6:.1f} MB per GPU "
                       f"({r['nsets'] * r['set_bytes'] / 1e6:.0f} MB vs 126 MB L2); timed region = {r['steps']} back-to-back calls")

    iso = head.get("isolated_us")
    line = dict(metric="fused_matmul_softmax_tflops", value=head["value"], unit="TFLOP/s", n_gpus=world, steps=args.steps,
                warmup=args.warmup, ms_per_step=head["ms_per_step"], us_per_call=head["ms_per_step"] * 1e3,
                us_isolated_call_min=iso[0] if iso else None, us_isolated_call_median=iso[1] if iso else None,
                us_per_call_operands_ready=head.get("operands_ready_us"),
                higher_is_better=True, scaling=head["scaling"], vs_baseline=None, dtype=wl["dtype"], data="synthetic",
                config=config_for(args.workload, wl, world), plan=plan_dict(head),
                roofline=roof, cpu_baseline=cpu, e2e=head.get("e2e"), clocks=head["clocks"],
                gpu_launches=args.steps * head["launches_per_step"], parity=head["parity"])
    for nm, r in splits.items():
        rf = roofline_of(r, pk)
        obj = dict(workload=f"{nm}: {WORKLOADS[nm]['desc']}", scaling="strong", n_gpus=world, steps=r["steps"],
                   ms_per_step=r["ms_per_step"], us_per_call=r["ms_per_step"] * 1e3, value=r["value"], unit="TFLOP/s",
                   sharding=SHARDING_TEXT[WORKLOADS[nm]["shard"]], plan=plan_dict(r), roofline=rf, parity=r["parity"],
                   clocks=r["clocks"])
        if "phases_us" in r:
            obj["phases_us"] = r["phases_us"]
        line[f"scaling_{nm}"] = obj
    if siblings:
        line["row_chains"] = siblings
    print(json.dumps(line), flush=True)
    ctx.close()


if __name__ == "__main__":
    main()
