#!/usr/bin/env python3
"""Benchmark of the fused Matmul -> row-Softmax chain.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload cfg2] [--impl reference]

One step = one call of the chain on one batch of synthetic input.  The default
workload is the f16-native chain A[4096,1024] . B[1024,1024], scale 1/32, f16
probabilities, on one GPU; with N GPUs every rank runs its own 4096 rows against
a replicated B (rows are independent: no data-path collective).  Prints ONE JSON
line (rank 0).  `--impl reference` times the CPU restatement of the chain (scalar
loop nest, all host threads) on a bounded sample of the same workload.
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
    "ref": dict(batch=1, M=8192, N=128, K=64, scale=1.0, sigma_b=1.0, b_batched=False, dtype="f16", shard="rows",
                desc="the reference's own shape 8192x64 . 64x128"),
}
L2_BYTES = 126 * 1024 * 1024

# DRAM traffic of the dominant kernel, bytes per launch, from the ncu captures
# summarised under profiles/ (dram__bytes_read.sum + dram__bytes_write.sum).
NCU_TRAFFIC = {"cfg2": 10555648, "cfg3": 545029632, "cfg5": 267214336}


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
        """Start of the timed region: forget what was sampled during warm-up."""
        self.samples, self.reasons = [], set()

    def finish(self):
        """Call with the timed work still in flight: takes one more sample (short regions fall
        between two polls of the thread), then stops the thread."""
        if self.ok and hasattr(self, "_names"):
            self._sample()
        self._stop_evt.set()
        if self.is_alive():
            self.join(timeout=1)
        if not self.samples:
            return dict(sm_mhz=None, sm_max_mhz=self.max_mhz, reasons=sorted(self.reasons))
        s = sorted(self.samples)
        return dict(sm_mhz=s[len(s) // 2], sm_max_mhz=self.max_mhz, reasons=sorted(self.reasons))


def run_reference(args, wl):
    """CPU arm: the loop-nest restatement of the chain on all host threads, a bounded
    sample of the workload per step (rows are independent, so a row sample scales)."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    import numpy as np
    from oracle import oracle
    threads = oracle.max_threads()
    dt = np.float16 if wl["dtype"] == "f16" else np.float32
    # about 2 GFLOP of scalar work per step
    rows = max(1, min(wl["M"], int(2.0e9 / (2.0 * wl["N"] * wl["K"]))))
    A = oracle.normal((rows, wl["K"]), 1, 1.0, dt)
    B = oracle.normal((wl["K"], wl["N"]), 2, wl["sigma_b"], dt)
    for _ in range(max(1, min(args.warmup, 2))):
        oracle.chain_loops_f32(A, B, wl["scale"], threads)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        oracle.chain_loops_f32(A, B, wl["scale"], threads)
    dt_s = (time.perf_counter() - t0) / args.steps
    flops = 2.0 * rows * wl["N"] * wl["K"]
    value = flops / dt_s / 1e12
    sample = f"{rows} of {wl['batch'] * wl['M']} rows per step (rows are independent; throughput is per-row work / time)"
    line = dict(impl="reference", metric="fused_matmul_softmax_tflops", value=value, unit="TFLOP/s",
                n_gpus=args.gpus, steps=args.steps, warmup=args.warmup, ms_per_step=dt_s * 1e3,
                higher_is_better=True, scaling="weak", vs_baseline=None, dtype="f32", data="synthetic",
                config=dict(workload=f"{args.workload}: {wl['desc']}", sample=sample),
                cpu_baseline=dict(value=value, unit="TFLOP/s", cores=threads, kind="port", sample=sample),
                e2e=dict(value=value, unit="TFLOP/s", h2d_bytes_per_step=0, d2h_bytes_per_step=0),
                gpu_launches=0)
    print(json.dumps(line), flush=True)


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
    args = ap.parse_args()
    wl = WORKLOADS[args.workload]
    if args.warmup < 3:
        args.warmup = 3

    if args.impl == "reference":
        run_reference(args, wl)
        return

    import numpy as np
    import torch
    import torch.distributed as dist
    import welder_typical_chain_b200 as wtc

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the chain has no CPU path (use --impl reference for the CPU baseline)")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)

    tdt = torch.float16 if wl["dtype"] == "f16" else torch.float32
    out_code = wtc.F16 if wl["dtype"] == "f16" else wtc.F32
    batch, M, N, K, scale = wl["batch"], wl["M"], wl["N"], wl["K"], wl["scale"]
    shard = wl["shard"]
    scaling = "weak"
    n_local = N
    from welder_typical_chain_b200 import sharding
    if shard == "batch" and world > 1:           # fixed 64 batches split over the ranks
        b0, b1 = sharding.split_batches(batch, world)[rank]
        batch = b1 - b0
        scaling = "strong"
    elif shard == "cols" and world > 1:          # N split on 256-column tile boundaries
        c0, c1 = sharding.split_columns(N, world)[rank]
        n_local = c1 - c0
        scaling = "strong"
    # rows / replica: every rank runs the whole per-GPU workload (weak scaling)

    flops_step, bytes_step = algorithmic(wl, batch=batch, N=n_local)
    # rotating buffer sets so that consecutive steps never find their operands in L2
    set_bytes = bytes_step
    nsets = max(2, min(64, math.ceil(2.4 * L2_BYTES / max(set_bytes, 1))))
    if set_bytes > 2 * L2_BYTES:
        nsets = 1 if set_bytes > 8e9 else 2
    g = torch.Generator(device=dev)
    g.manual_seed(1234 + rank)
    a_shape = (batch, M, K) if batch > 1 else (M, K)
    b_shape = (batch, K, n_local) if (wl["b_batched"] and batch > 1) else (K, n_local)
    o_shape = (batch, M, n_local) if batch > 1 else (M, n_local)
    sets = []
    for _ in range(nsets):
        A = torch.randn(a_shape, device=dev, dtype=torch.float32, generator=g).to(tdt)
        B = (torch.randn(b_shape, device=dev, dtype=torch.float32, generator=g) * wl["sigma_b"]).to(tdt)
        O = torch.empty(o_shape, device=dev, dtype=tdt)
        sets.append((A, B, O))
    desc = wtc.launch._desc_for(sets[0][0], sets[0][1], out_code, scale, wtc.F32, wtc.VARIANT_FUSED, 0, None)
    plan = wtc.plan_query(desc)
    ws_bytes = wtc.workspace_bytes(desc)
    ws = torch.empty(max(ws_bytes, 16), device=dev, dtype=torch.uint8)
    col_sharded = shard == "cols" and world > 1
    rows_total = batch * M
    if col_sharded:
        row_stats = torch.empty((rows_total, 2), device=dev, dtype=torch.float32)
        all_stats = torch.empty((world * rows_total, 2), device=dev, dtype=torch.float32)   # rank-major [world][rows][2]

    sptr = wtc.current_stream_ptr()
    if col_sharded:
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

    # ---- parity spot check on this rank's first buffer set (sampled rows, CPU checker) ----
    parity = None
    if not args.no_parity and not col_sharded:
        from oracle import oracle
        step(0)
        torch.cuda.synchronize()
        A, B, O = sets[0]
        A2 = A.reshape(-1, M, K)[0]
        B2 = B.reshape(-1, K, n_local)[0]
        O2 = O.reshape(-1, M, n_local)[0]
        idx = sorted(set(int(x) for x in np.linspace(0, M - 1, 24)))
        ref = oracle.chain(A2[idx].cpu().numpy(), B2.cpu().numpy(), scale)
        parity = oracle.compare(O2[idx].cpu().numpy(), ref)
        parity["rows_checked"] = len(idx)
        if not parity["ok"]:
            raise SystemExit(f"parity check failed before timing: {parity}")

    if not args.no_parity and col_sharded:
        # every rank checks its own columns of a few rows: the whole-row (max, sum) comes from
        # float64 partials of all ranks, exchanged as Python objects
        step(0)
        torch.cuda.synchronize()
        A, B, O = sets[0]
        idx = sorted(set(int(x) for x in np.linspace(0, M - 1, 8)))
        v = scale * 1.4426950408889634 * (A[idx].double().cpu().numpy() @ B.double().cpu().numpy())
        m_loc = v.max(1) if n_local else np.full(len(idx), -np.inf)
        l_loc = np.exp2(v - m_loc[:, None]).sum(1) if n_local else np.zeros(len(idx))
        parts = [None] * world
        dist.all_gather_object(parts, (m_loc, l_loc))
        gm = np.max([q[0] for q in parts], axis=0)
        gl = np.sum([q[1] * np.exp2(q[0] - gm) for q in parts], axis=0)
        ref = np.exp2(v - gm[:, None]) / gl[:, None]
        got = O[idx].float().cpu().numpy().astype(np.float64)
        err = float(np.abs(got - ref).max()) if n_local else 0.0
        parity = dict(ok=bool(err <= 2e-3), max_abs=err, rows_checked=len(idx), note="this rank's columns against the whole-row statistics")
        if not parity["ok"]:
            raise SystemExit(f"rank {rank}: column-sharded parity check failed: {parity}")

    # the sampler thread starts before the warm-up so that its start-up (NVML first calls) is
    # not inside the timed region; its samples are cleared when the timed region begins
    sampler = ClockSampler(local)
    sampler.start()
    for i in range(args.warmup):
        step(i)
    wtc.check_device_status()
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    sampler.mark()
    stream = torch.cuda.current_stream()
    e0 = torch.cuda.Event(enable_timing=True)
    e1 = torch.cuda.Event(enable_timing=True)
    e0.record(stream)
    for i in range(args.steps):
        step(i)
    e1.record(stream)
    clocks = sampler.finish()          # the queue is still draining: this sample is under load
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1)
    wtc.check_device_status()
    t = torch.tensor([ms], device=dev, dtype=torch.float64)
    fl = torch.tensor([flops_step], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        dist.all_reduce(fl, op=dist.ReduceOp.SUM)
    ms_max = float(t.item())
    total_flops_step = float(fl.item())
    ms_per_step = ms_max / args.steps
    value = total_flops_step / (ms_per_step * 1e-3) / 1e12

    # ---- isolated calls (the stream is idle before each), each between its own pair of events, this rank:
    #      minimum and median; these include the launch latency the back-to-back loop hides
    #      beside the mean of the back-to-back loop above (the reference harness reports a mean only)
    single = []
    for i in range(min(args.steps, 30)):
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record(stream)
        step(i)
        b.record(stream)
        b.synchronize()
        single.append(a.elapsed_time(b) * 1e3)
    single.sort()

    # ---- end to end: host buffers in, host buffer out, through the C-ABI host entry point ----
    e2e = None
    if not args.no_e2e and not col_sharded:
        A, B, O = sets[0]
        hA = torch.empty(A.shape, dtype=tdt, pin_memory=True).copy_(A)
        hB = torch.empty(B.shape, dtype=tdt, pin_memory=True).copy_(B)
        hO = torch.empty(O.shape, dtype=tdt, pin_memory=True)
        nA, nB, nO = hA.numpy(), hB.numpy(), hO.numpy()
        e2e_steps = max(3, min(args.steps, int(2.0 / max(1e-4, (hA.nbytes + hB.nbytes + hO.nbytes) / 20e9))))
        for _ in range(3):
            wtc.matmul_softmax_host(nA, nB, scale, out=nO, out_dtype=out_code)
        if world > 1:
            dist.barrier()
        t0 = time.perf_counter()
        for _ in range(e2e_steps):
            wtc.matmul_softmax_host(nA, nB, scale, out=nO, out_dtype=out_code)
        dt_s = time.perf_counter() - t0
        te = torch.tensor([dt_s / e2e_steps], device=dev, dtype=torch.float64)
        if world > 1:
            dist.all_reduce(te, op=dist.ReduceOp.MAX)
        e2e = dict(value=total_flops_step / float(te.item()) / 1e12, unit="TFLOP/s",
                   h2d_bytes_per_step=int(hA.nbytes + hB.nbytes), d2h_bytes_per_step=int(hO.nbytes),
                   ms_per_step=float(te.item()) * 1e3, steps=e2e_steps,
                   api="wtc_matmul_softmax_host (pinned host buffers; copies inside the timed region)")

    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return

    pk = peaks()
    hbm_bound = args.workload in ("cfg3", "cfg5")
    launch_s = ms / args.steps * 1e-3          # this rank's average call duration on its stream
    if hbm_bound:
        achieved = bytes_step / launch_s / 1e9
        roof = dict(bound="hbm", achieved=achieved, peak=pk["hbm_gbs"], unit="GB/s", frac=achieved / pk["hbm_gbs"])
    else:
        achieved = flops_step / launch_s / 1e12
        roof = dict(bound="tensor", achieved=achieved, peak=pk["tflops"], unit="TFLOP/s", frac=achieved / pk["tflops"])
    roof["peak_source"] = pk["source"]
    roof["traffic"] = NCU_TRAFFIC.get(args.workload)
    roof["kernel"] = wtc.launch.KERNEL_NAMES[plan.kernel]
    roof["algorithmic_per_launch"] = dict(flops=flops_step, bytes=bytes_step)

    cpu = None
    if not args.no_cpu_baseline and world == 1:
        from oracle import oracle
        threads = oracle.max_threads()
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

    line = dict(metric="fused_matmul_softmax_tflops", value=value, unit="TFLOP/s", n_gpus=world, steps=args.steps,
                warmup=args.warmup, ms_per_step=ms_per_step, us_per_call=ms_per_step * 1e3,
                us_isolated_call_min=single[0] if single else None, us_isolated_call_median=single[len(single) // 2] if single else None,
                higher_is_better=True, scaling=scaling, vs_baseline=None, dtype=wl["dtype"], data="synthetic",
                config=dict(workload=f"{args.workload}: {wl['desc']}",
                            per_gpu=dict(batch=batch, M=M, N=n_local, K=K),
                            sharding={"rows": "each GPU its own M rows, B replicated, no collective",
                                      "batch": "batches split over the GPUs, no collective",
                                      "cols": "N split on 256-column tile boundaries, one all-gather of per-row (max,sum)",
                                      "replica": "independent replicas"}[shard],
                            l2=f"{nsets} rotating buffer sets of {set_bytes / 1e6:.1f} MB "
                               f"({nsets * set_bytes / 1e6:.0f} MB vs 126 MB L2); timed region = {args.steps} back-to-back calls",
                            kernel=wtc.launch.KERNEL_NAMES[plan.kernel], cluster_n=plan.cluster_n,
                            tile=[plan.tile_m, plan.tile_n, plan.tile_k], stages=plan.stages),
                roofline=roof, cpu_baseline=cpu, e2e=e2e, clocks=clocks,
                gpu_launches=args.steps * plan.launches, parity=parity)
    print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
