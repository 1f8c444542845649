"""Where one call of the tensor-core kernel spends its time, from the bring-up build's stamps.

    make -C welder_typical_chain_b200/csrc bringup
    python -m welder_typical_chain_b200.stamps [--batch B --M M --N N --K K --flags F --sets S]

The bring-up library (csrc/build/bringup/libwtc_bringup.so, compiled with -DWTC_BRINGUP) makes
every CTA write globaltimer and clock64 at the phases of its first tile: entry, set-up done,
dependency wait returned, first loads issued, first stage landed, accumulator complete,
exponentials done, cluster statistics in, tile staged, stores read, exit.  This tool runs the
chain back to back over rotating buffer sets larger than L2 (as bench.py does), prints the time
per call, then captures a few stamped launches and prints the median / min / max length of each
phase over the CTAs in clocks and microseconds, and the first / median / last absolute time of
each stamp for consecutive launches (to see how launches overlap).  The stamps cost about
0.3 us per call; the default library has none.
"""
import argparse
import ctypes as C
import os

import numpy as np

SLOTS = ["entry", "setup", "deps", "tma0", "full0", "mma_done", "accum", "exp", "stats", "staged", "stored", "exit",
         "loaded", "max", "teardown", "clsync", "mma_ready", "packed", "producer_end"]
PHASES = [("entry -> set-up done", "setup", "entry"), ("entry -> dependency wait returns", "deps", "entry"),
          ("wait returns -> first loads issued", "tma0", "deps"), ("first loads issued -> first stage landed", "full0", "tma0"),
          ("first stage landed -> accumulator complete", "accum", "full0"), ("accumulator -> exponentials done", "exp", "accum"),
          ("exponentials -> cluster statistics in", "stats", "exp"), ("statistics -> tile staged, store issued", "staged", "stats"),
          ("store issued -> staging read", "stored", "staged"),
          ("staging read -> exit (other warps' stores, barriers, TMEM freed)", "exit", "stored"),
          ("entry -> exit", "exit", "entry"), ("wait returns -> exit", "exit", "deps")]


def main():
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--batch", type=int, default=1)
    ap.add_argument("--M", type=int, default=4096)
    ap.add_argument("--N", type=int, default=1024)
    ap.add_argument("--K", type=int, default=1024)
    ap.add_argument("--flags", type=int, default=0)
    ap.add_argument("--sets", type=int, default=16, help="rotating operand/output sets (their total should exceed L2)")
    ap.add_argument("--calls", type=int, default=200)
    ap.add_argument("--lib", default=os.path.join(os.path.dirname(os.path.abspath(__file__)), "csrc", "build", "bringup", "libwtc_bringup.so"))
    a = ap.parse_args()
    if not os.path.exists(a.lib):
        raise SystemExit(f"{a.lib} not found: run `make -C welder_typical_chain_b200/csrc bringup` first")
    import torch
    from . import launch
    launch.lib_path = lambda: a.lib
    L = launch.lib()
    L.wtc_bringup_set_timeline.argtypes = [C.c_void_p]
    dev = torch.device("cuda:0")
    scale = 1.0 / 32

    def mk():
        lead = (a.batch,) if a.batch > 1 else ()
        return (torch.randn(lead + (a.M, a.K), device=dev, dtype=torch.float16), torch.randn(lead + (a.K, a.N), device=dev, dtype=torch.float16),
                torch.empty(lead + (a.M, a.N), device=dev, dtype=torch.float16))
    sets = [mk() for _ in range(a.sets)]
    calls = [launch.PreparedCall(A, B, O, scale, flags=a.flags) for (A, B, O) in sets]
    sp = launch.current_stream_ptr()
    for i in range(20):
        calls[i % a.sets].launch(sp)
    launch.check_device_status()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(a.calls):
        calls[i % a.sets].launch(sp)
    e1.record()
    torch.cuda.synchronize()
    print(f"batch={a.batch} M={a.M} N={a.N} K={a.K} flags={a.flags}: {e0.elapsed_time(e1) / a.calls * 1e3:.2f} us per call, back to back over {a.sets} buffer sets (stamps compiled in)")
    A, B, O = sets[(a.calls - 1) % a.sets]
    ref = torch.softmax((A.float() @ B.float()) * scale, dim=-1)
    print(f"max abs error against torch fp32: {float((O.float() - ref).abs().max()):.3g}")

    # four consecutive stamped launches (the library keeps four regions of 148 CTAs x 48 slots)
    tl = torch.zeros(4 * 148 * 48, dtype=torch.int64, device=dev)
    L.wtc_bringup_set_timeline(C.c_void_p(tl.data_ptr()))
    for i in range(4):
        calls[i % a.sets].launch(sp)
    torch.cuda.synchronize()
    L.wtc_bringup_set_timeline(None)
    t = tl.cpu().numpy().reshape(4, 148, 48).astype(np.float64)
    idx = {n: i for i, n in enumerate(SLOTS)}
    last = t[3]
    last = last[last[:, 0] > 0]
    g, c = last[:, :24], last[:, 24:]
    print(f"\nphases of the fourth launch, over its {len(last)} CTAs:")
    for label, hi, lo in PHASES:
        m = (g[:, idx[hi]] > 0) & (g[:, idx[lo]] > 0)
        if not m.any():
            continue
        dc = c[m, idx[hi]] - c[m, idx[lo]]
        dg = (g[m, idx[hi]] - g[m, idx[lo]]) / 1e3
        print(f"  {label:66s} clocks median {np.median(dc):7.0f}  min {dc.min():7.0f}  max {dc.max():7.0f}   us median {np.median(dg):6.2f}")
    m = (g[:, idx["accum"]] > 0) & (g[:, idx["full0"]] > 0)
    if m.any():
        mhz = np.median((c[m, idx["exit"]] - c[m, idx["entry"]]) / (g[m, idx["exit"]] - g[m, idx["entry"]])) * 1e3
        print(f"  main loop: {np.median(c[m, idx['accum']] - c[m, idx['full0']]) / max(1, (a.K + 63) // 64):.0f} clocks per 64-deep K block; SM clock {mhz:.0f} MHz")
    print("\nabsolute times (us after the first stamp; first / median / last CTA) of launches 2-4:")
    t0 = min(x[x[:, 0] > 0][:, 0].min() for x in t if (x[:, 0] > 0).any())
    for k in (1, 2, 3):
        x = t[k]
        x = x[x[:, 0] > 0]
        cols = []
        for n in ("entry", "deps", "full0", "accum", "stats", "stored", "exit"):
            v = x[:, idx[n]]
            v = (v[v > 0] - t0) / 1e3
            if len(v):
                cols.append(f"{n}[{v.min():6.2f} {np.median(v):6.2f} {v.max():6.2f}]")
        print("  " + " ".join(cols))


if __name__ == "__main__":
    main()
