"""Benchmark of the verify-step hot path on B200.

Default workload ("c2-moe"): BASELINE config 2, the verify-step MoE microbench: hidden 2048, 512 experts top-10,
expert FFN 512 + a shared expert of FFN 512, K+1 = 4 rows of N(0,1) activations rounded to bf16, expert weights EXL3 at
3 bits a weight (--format exl3, the default) or IQ3_S / Q8_0.  One "step" is one MoE sublayer pass over the 4 rows.
`--layers` distinct layers (default 8, ~5 GB) are cycled so each step streams expert weights that are not in the 126 MB L2.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--format exl3|iq3_s|q8_0] [--impl reference]

Prints one JSON line (rank 0).  `--impl reference` times the CPU restatement of the reference's scalar path (the oracle)
on the host cores for the same workload.
"""
import argparse
import ctypes as C
import json
import os
import subprocess
import sys
import tempfile
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

C2 = dict(hidden=2048, n_expert=512, top_k=10, expert_ff=512, shared_ff=512, rows=4)
METRIC = "verify-step us (MoE sublayer, K+1=4 rows, spec K=3)"


def peaks():
    try:
        p = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))
        return float(p["hbm_gbs"]), "measured"
    except Exception:
        return 6650.0, "fallback"


def type_of(fmt, szlib):
    return {"exl3": szlib.TYPE_EXL3(3), "iq3_s": szlib.TYPE_IQ3_S, "q8_0": szlib.TYPE_Q8_0}[fmt]


def expert_bytes(fmt, H, FF):
    """Bytes of one expert (gate + up + down) in the format's own layout: the algorithmic bytes per distinct expert."""
    if fmt == "exl3":
        return 3 * (2 * H + 2 * FF + 4 + H * FF * 3 // 8)
    if fmt == "iq3_s":
        return 3 * (H * FF // 256 * 110)
    return 3 * (H * FF // 32 * 34)


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index = index
        self.f = tempfile.NamedTemporaryFile("w+", suffix=".csv", delete=False)
        self.p = None

    def start(self):
        try:
            self.p = subprocess.Popen(["nvidia-smi", "-i", str(self.index), "--query-gpu=" + self.Q, "--format=csv,noheader,nounits",
                                       "-lms", "100"], stdout=self.f, stderr=subprocess.DEVNULL)
        except Exception:
            self.p = None

    def stop(self):
        if self.p is not None:
            self.p.terminate()
            try:
                self.p.wait(timeout=5)
            except Exception:
                self.p.kill()
        self.f.flush()
        rows = [l.strip().split(", ") for l in open(self.f.name).read().splitlines() if l.strip()]
        os.unlink(self.f.name)
        sm, mx, reasons = [], [], set()
        for r in rows:
            try:
                sm.append(float(r[1])); mx.append(float(r[2]))
                for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), r[5:9]):
                    if v.strip().lower() == "active":
                        reasons.add(name)
            except Exception:
                pass
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        sm.sort()
        return {"sm_mhz": sm[len(sm) // 2], "sm_max_mhz": max(mx), "reasons": sorted(reasons), "samples": len(sm)}


def build_layers(fmt, n_layers, device, seed=1):
    import __graft_entry__ as graft
    pkg = graft.load_package()
    ty = type_of(fmt, pkg.lib)
    layers, host0 = [], None
    for l in range(n_layers):
        L = pkg.synth.make_moe_layer(C2["hidden"], C2["n_expert"], C2["top_k"], C2["expert_ff"], C2["shared_ff"], ty, ty,
                                     seed=seed + l, device=device, name="blk.%d" % l)
        layers.append(pkg.moe.MoeLayer(L, device, max_rows=C2["rows"]))
        if l == 0:
            host0 = pkg.synth.to_numpy_layer(L)
        del L
    return pkg, layers, host0


def make_x(seed=11):
    import torch
    g = torch.Generator().manual_seed(seed)
    return torch.randn(C2["rows"], C2["hidden"], generator=g).to(torch.bfloat16).to(torch.float32)


def cpu_step_seconds(host_layer, x, threads, budget_s):
    """Times the oracle's MoE (Session::moe per row, rows split over `threads` threads as the reference's matvec does)."""
    from oracle import binding as ob
    xs = x.numpy()
    reps, t0 = 0, time.perf_counter()
    while True:
        for j in range(xs.shape[0]):
            ob.moe(host_layer, xs[j], threads=threads)
        reps += 1
        el = time.perf_counter() - t0
        if el >= budget_s or reps >= 50:
            return el / reps, reps


def run_reference(args):
    """The reference arm: the reference's own CPU implementation of the path, i.e. its scalar f64-accumulating Session::moe
    restated in C (the reference itself is Rust and cannot be built here), on all host cores."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    import torch  # noqa: F401
    import __graft_entry__ as graft
    from oracle import binding as ob
    ob.lib()
    pkg = graft.load_package()
    ty = type_of(args.format, pkg.lib)
    L = pkg.synth.make_moe_layer(C2["hidden"], C2["n_expert"], C2["top_k"], C2["expert_ff"], C2["shared_ff"], ty, ty, seed=1,
                                 device="cpu", name="blk.0")
    host = pkg.synth.to_numpy_layer(L)
    x = make_x()
    threads = os.cpu_count() or 1
    for _ in range(max(args.warmup, 1)):
        for j in range(C2["rows"]):
            ob.moe(host, x[j].numpy(), threads=threads)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        for j in range(C2["rows"]):
            ob.moe(host, x[j].numpy(), threads=threads)
    sec = (time.perf_counter() - t0) / args.steps
    us = sec * 1e6
    sample = "%d steps of the full 4-row MoE pass on one layer (weights in the CPU caches/DRAM)" % args.steps
    print(json.dumps({
        "impl": "reference", "metric": METRIC, "value": us, "unit": "us", "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": us / 1e3, "higher_is_better": False, "scaling": "weak", "vs_baseline": None, "dtype": "f32 (f64 accumulate)",
        "data": "synthetic", "config": {"workload": "c2-moe", "format": args.format, **C2},
        "cpu_baseline": {"value": us, "unit": "us", "cores": threads, "kind": "port", "sample": sample},
        "e2e": {"value": us, "unit": "us", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}))


def time_format(fmt, args, device, rank, world):
    import torch
    pkg, layers, host0 = build_layers(fmt, args.layers, device)
    szlib = pkg.lib
    x = make_x()
    xd = x.to(device)
    yd = torch.empty_like(xd)
    nl = len(layers)
    stream = torch.cuda.Stream(device)
    H, FF, k, m = C2["hidden"], C2["expert_ff"], C2["top_k"], C2["rows"]

    # routing is a function of (layer, x): count the distinct experts each layer's step touches
    distinct = []
    for layer in layers:
        _, ridx, _ = layer.moe_batch(xd, want_routing=True)
        torch.cuda.synchronize()
        distinct.append(int(torch.unique(ridx).numel()))
    be = expert_bytes(fmt, H, FF)

    def step(i, st):
        layers[i % nl].moe_batch(xd, yd, stream=st)

    with torch.cuda.stream(stream):
        for i in range(max(args.warmup, 3)):
            step(i, stream)
        stream.synchronize()
        graph = None
        if not args.no_graph:
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=stream):
                for i in range(args.steps):
                    step(i, stream)
            graph.replay()  # untimed warm replay
            stream.synchronize()
        if world > 1:
            import torch.distributed as dist
            dist.barrier()
        torch.cuda.synchronize()
        sampler = ClockSampler(torch.cuda.current_device())
        sampler.start()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        reps = max(1, args.reps)
        best = None
        for _ in range(reps):
            e0.record(stream)
            if graph is not None:
                graph.replay()
            else:
                for i in range(args.steps):
                    step(i, stream)
            e1.record(stream)
            stream.synchronize()
            ms = e0.elapsed_time(e1)
            best = ms if best is None else min(best, ms)
        torch.cuda.synchronize()
        clocks = sampler.stop()
        ms_per_step = best / args.steps

        # per-kernel attribution: a traced (serialised) pass
        nev = args.steps * layers[0].launches() + 2
        evs = [torch.cuda.Event(enable_timing=True) for _ in range(nev)]
        for e in evs:
            e.record(stream)  # creates the handles
        stream.synchronize()
        arr = (C.c_uint64 * nev)(*[e.cuda_event for e in evs])
        L = szlib.load()
        szlib.check(L.sz_trace_begin(arr, nev, stream.cuda_stream))
        for i in range(args.steps):
            step(i, stream)
        n = L.sz_trace_end()
        stream.synchronize()
        per = {}
        for i in range(1, n):
            nm = L.sz_trace_name(i).decode()
            per.setdefault(nm, []).append(evs[i - 1].elapsed_time(evs[i]) * 1e3)
        kern = {nm: {"launches": len(v), "avg_us": sum(v) / len(v)} for nm, v in per.items()}

        # end to end: host buffers, copies inside the timed region
        xh = x.clone().pin_memory()
        yh = torch.empty_like(xh).pin_memory()
        for i in range(3):
            layers[i % nl].moe_batch_host(xh, yh, xd, yd, stream=stream)
        t0 = time.perf_counter()
        for i in range(args.steps):
            layers[i % nl].moe_batch_host(xh, yh, xd, yd, stream=stream)
        e2e_us = (time.perf_counter() - t0) / args.steps * 1e6

    davg = sum(distinct[i % nl] for i in range(args.steps)) / args.steps
    res = dict(fmt=fmt, ms_per_step=ms_per_step, e2e_us=e2e_us, distinct=davg, expert_bytes=be, kernels=kern, clocks=clocks,
               launches=args.steps * layers[0].launches(), host0=host0, x=x)
    return res


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours")
    ap.add_argument("--format", default="exl3", choices=["exl3", "iq3_s", "q8_0"])
    ap.add_argument("--also", default="iq3_s", help="comma list of further formats to time and report under 'also' ('' for none)")
    ap.add_argument("--layers", type=int, default=8)
    ap.add_argument("--reps", type=int, default=3, help="timed repetitions of the K-step region; the fastest is reported")
    ap.add_argument("--no-graph", action="store_true", help="launch eagerly instead of replaying a CUDA graph of the K steps")
    ap.add_argument("--cpu-seconds", type=float, default=12.0)
    args = ap.parse_args()
    if args.impl == "reference":
        return run_reference(args)

    import torch
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the library has no CPU path")
    torch.cuda.set_device(local)
    device = "cuda:%d" % local
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl")
    hbm, peak_kind = peaks()

    main_res = time_format(args.format, args, device, rank, world)
    also = []
    for f in [t for t in args.also.split(",") if t and t != args.format]:
        r = time_format(f, args, device, rank, world)
        also.append(r)

    def roofline(r):
        # the dominant kernel: gate+up of the routed experts (2/3 of an expert's bytes per distinct expert)
        name = "gateup_exl3" if r["fmt"] == "exl3" else "gateup_rows"
        ks = r["kernels"].get(name)
        # two launches carry that name (routed, shared): the routed one is the first of each pair; both are averaged here with
        # bytes of both, so the figure is the pair's
        bytes_pair = (r["distinct"] + 1) * r["expert_bytes"] * 2 / 3
        out = {"bound": "hbm", "peak": hbm, "unit": "GB/s", "peak_kind": peak_kind, "traffic": None, "kernel": name}
        if ks:
            dur_us = ks["avg_us"] * 2  # the pair
            out["achieved"] = bytes_pair / (dur_us * 1e-6) / 1e9
            out["frac"] = out["achieved"] / hbm
            out["kernel_us"] = dur_us
        step_bytes = r["distinct"] * r["expert_bytes"]
        out["step_bytes"] = step_bytes
        out["step_achieved"] = step_bytes / (r["ms_per_step"] * 1e-3) / 1e9
        out["step_frac"] = out["step_achieved"] / hbm
        return out

    if world > 1:
        import torch.distributed as dist
        t = torch.tensor([main_res["ms_per_step"]], device=device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        main_res["ms_per_step"] = float(t.item())
    if rank != 0:
        return
    cpu = None
    if world == 1:
        threads = os.cpu_count() or 1
        sec, reps = cpu_step_seconds(main_res["host0"], main_res["x"], threads, args.cpu_seconds)
        cpu = {"value": sec * 1e6, "unit": "us", "cores": threads, "kind": "port",
               "sample": "%d full 4-row MoE passes of layer 0 by the C restatement of Session::moe" % reps}
    us = main_res["ms_per_step"] * 1e3
    line = {
        "metric": METRIC, "value": us, "unit": "us", "n_gpus": args.gpus, "steps": args.steps, "warmup": max(args.warmup, 3),
        "ms_per_step": main_res["ms_per_step"], "higher_is_better": False, "scaling": "weak", "vs_baseline": None,
        "dtype": "f32 activations, f16 codebook weights, f32 accumulate (router and combine in f64)", "data": "synthetic",
        "config": {"workload": "c2-moe", "format": args.format, **C2, "layers_cycled": args.layers,
                   "l2": "inputs larger than L2: %d layers of expert weights cycled" % args.layers,
                   "graph": not args.no_graph, "distinct_experts_per_step": main_res["distinct"]},
        "roofline": roofline(main_res), "cpu_baseline": cpu,
        "e2e": {"value": main_res["e2e_us"], "unit": "us", "h2d_bytes_per_step": C2["rows"] * C2["hidden"] * 4,
                "d2h_bytes_per_step": C2["rows"] * C2["hidden"] * 4},
        "gpu_launches": main_res["launches"], "clocks": main_res["clocks"], "kernels": main_res["kernels"],
        "also": [{"format": r["fmt"], "value": r["ms_per_step"] * 1e3, "unit": "us", "e2e_us": r["e2e_us"],
                  "roofline": roofline(r), "kernels": r["kernels"]} for r in also],
    }
    print(json.dumps(line))


if __name__ == "__main__":
    main()
