"""Benchmark of the speculative-decoding verify path on B200.

Default workload ("c3"): benchmark config 3 - the full-size seeded hybrid MoE (48 layers 3:1 DeltaNet : gated attention, hidden
2048, 512 experts top-10 of FFN 512 + a shared expert, EXL3 3-bit experts, Q8_0 dense matrices, a 4-bit EXL3 head screened by
its 2-bit proxy (`--head q8` / `exl3`: a Q8_0 or an EXL3 head read in full), vocab 151936, Q8_KV cache) decoding greedily at spec K=3, batch 1, at context 24576.  One "step" is one draft / verify / accept round: the suffix
drafter proposes up to 3 tokens, one verify pass runs over the 1..4 rows, acceptance and rollback happen on the device.  The
metric is accepted tokens per second (every emitted token: accepted drafts and the pass's own token).  With --gpus N (under
torchrun) the experts of every layer are sharded over the N ranks (expert parallelism); one sequence, so scaling is "strong".

`--workload c2-moe`: benchmark config 2, the verify-step MoE microbench (one MoE sublayer pass over K+1 = 4 rows per step).
`--workload prefill-dense`: the batched / prompt form of a DeltaNet layer's input projection (12,288 x 2,048 Q8_0) over 256 or more token
rows on tcgen05 (`sz_mma_cols`); TFLOP/s against the measured dense bf16 rate.
`--workload c5-concurrent`: B sequences decoded at once on every GPU (config 5's batched serving, without batching the kernels): each
sequence has a verify session, stream and CUDA graphs of its own over the one resident model, and the GPU overlaps their passes.
`--workload c5-batch`: B sequences decoding in lockstep on every GPU (`sz_batch_gen_run`): sessions of their own, the reads, projections
and MoE sublayers of every layer run once over the rows of all sequences.
`--workload c5-moe`: the MoE sublayer over the verify rows of many sequences at once (64 sequences x K+1 = 4 rows = 256 rows), every
distinct expert decoded once (`sz_moe_rows`), next to the same rows as 64 passes of 4.
`--workload c4-tree`: benchmark config 4's mechanism on the config-3 model: one verify pass over a draft tree (8 rows), greedy
acceptance on the device and rejection sampling on the host; reports us per verify and the accepted length.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload c3|c2-moe] [--impl reference]

Prints one JSON line (rank 0).  `--impl reference` times the CPU restatement of the reference's scalar path (the oracle) on the
host cores for the same workload.
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

# benchmark config 3
C3 = dict(n_layer=48, hidden=2048, streams=4, hc_rank=256, vocab=151936, n_head=16, n_kv_head=2, head_dim=256, rope_dims=64,
          n_expert=512, n_expert_used=10, expert_ff=512, shared_ff=512, ssm_k_heads=16, ssm_v_heads=32, ssm_head_dim=128, conv_k=4,
          attn_interval=4, eps=1e-6, rope_theta=1e7)
C3_CTX = 24576
C3_INDEXER = dict(idx_heads=4, idx_dim=128, idx_budget=2048, idx_ratio=4)   # docs/ARCH.md:142-157 of the reference


def c3_model_cfg(args, n_layer):
    cfg = dict(C3, n_layer=n_layer)
    if getattr(args, "indexer", False):
        cfg.update(C3_INDEXER)
    return cfg
GATEUP_PROFILE = os.path.join(ROOT, "profiles", "c2_moe_gateup_exl3_full.md")


def gateup_traffic(experts_per_launch):
    """DRAM bytes (read + written) a launch of the EXL3 gate/up kernel moves, from the committed ncu capture of that kernel on
    these expert shapes: the capture's `traffic:` line gives the bytes of one launch and how many experts it covered; traffic grows
    in proportion to the experts a launch streams, so it is scaled to `experts_per_launch`.  None when the profile has no such line."""
    import re
    try:
        m = re.search(r"^traffic:\s*(\d+)\s*bytes a launch over\s*(\d+)\s*experts", open(GATEUP_PROFILE).read(), re.M)
        return int(m.group(1)) / int(m.group(2)) * experts_per_launch
    except Exception:
        return None
C3_METRIC = "accepted tok/s at spec K=3"


class QuietStdout:
    """Everything libraries write to file descriptor 1 while this is active goes to stderr (NCCL prints its version line there when
    NCCL_DEBUG is set in the environment); `emit` writes the one JSON line to the real stdout."""

    def __init__(self):
        sys.stdout.flush()
        self.real = os.dup(1)
        os.dup2(2, 1)

    def emit(self, line):
        sys.stdout.flush()
        os.write(self.real, (line + "\n").encode())


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


# ---- workload c3: accepted tok/s on the full-size model ---------------------------------------------------------------------------
# How strongly the synthetic model continues its token cycles, per kind of head (the two constructions differ: with a Q8_0 head the
# head is made from the embedding, with an EXL3 head the embedding from the decoded head).  Chosen so that a 200-round run accepts
# about as many tokens a round as the reference reports for its suffix drafter (2.8): 3.1 and 2.9.
C3_ALPHA = 0.85
C3_ALPHA_BY_HEAD = {"q8": 0.85, "exl3": 0.95, "proxy": 0.95}
# ... and how strongly it leans towards skipping a token of the cycle: what makes a draft right at a position only some of the
# time.  Measured with the screened head at 0.6 / 0.8 / 0.9: drafts right at positions 1, 2, 3 in 90 / 93 / 88 %, 65 / 69 / 79 % and
# 56 / 55 / 47 % of the tries; 0.7 sits near the reference's 75 / 75 / 83 % on real text (docs/SPECULATION.md:95-98).
C3_BETA_BY_HEAD = {"q8": 0.7, "exl3": 0.7, "proxy": 0.7}


def c3_config(args, cfg, ctx, bytes_all=None):
    """The `config` object of a c3 line: both arms (the library and the CPU reference) print the same one."""
    world = args.gpus
    return {"workload": "c3", "n_layer": cfg["n_layer"], "hidden": cfg["hidden"], "n_expert": cfg["n_expert"], "top_k": cfg["n_expert_used"],
            "expert_ff": cfg["expert_ff"], "vocab": cfg["vocab"], "experts": "exl3-3bit", "dense": "q8_0", "kv": "q8_kv",
            "head": {"q8": "q8_0, read in full", "exl3": "exl3-4bit, read in full", "proxy": "exl3-4bit screened by its 2-bit proxy (128 blocks a row)"}[args.head],
            "context": ctx, "spec_k": 3, "batch": 1, "greedy": True,
            "indexer": ({k: cfg[k] for k in C3_INDEXER} if cfg.get("idx_heads", 0) else None),
            "requests": "256-token prompts (a token cycle of the model repeated, 10%% random substitutions), %d tokens decoded each; "
                        "prompt passes and the cache fill are outside the timed region" % args.request_tokens,
            "acceptance_knobs": {"cycle_alpha": args.alpha, "cycle_beta": args.beta, "prompt_substitution": 0.1},
            "parallelism": ("replicas%d" % world if args.parallelism == "replicas" else "ep%d" % world) if world > 1 else "single",
            "exchange": args.exchange if world > 1 and args.parallelism != "replicas" else None,
            "l2": "inputs larger than L2: a pass streams about 5 GB of weights and cache"}


def c3_bytes(cfg, ctx, distinct_per_layer, dense_bytes):
    """Algorithmic bytes of one verify pass: every distinct routed expert and the shared expert once (EXL3 3-bit blobs), the
    Q8_KV cache of the attention layers once, and - counted apart - `dense_bytes`: the projections, hyper-connection weights,
    routers and the head, each read once."""
    H, FF = cfg["hidden"], cfg["expert_ff"]
    be = expert_bytes("exl3", H, FF)
    n_attn = cfg["n_layer"] // cfg["attn_interval"]
    hb = cfg["head_dim"] + ((cfg["head_dim"] // 32 * 2 + 15) & ~15)
    experts = sum(distinct_per_layer) * be + cfg["n_layer"] * expert_bytes("exl3", H, cfg["shared_ff"])
    kv = n_attn * ctx * cfg["n_kv_head"] * hb * 2
    if cfg.get("idx_heads", 0) and ctx > cfg["idx_budget"]:
        # the sparse indexer: a row attends to the budget's positions; the pooled keys (one per block of positions) are read instead
        kv = n_attn * (cfg["idx_budget"] * cfg["n_kv_head"] * hb * 2 + ctx // cfg["idx_ratio"] * cfg["idx_dim"] * 4)
    return {"experts": experts, "kv": kv, "experts_kv": experts + kv, "dense_and_head": dense_bytes, "all": experts + kv + dense_bytes}


def run_c3(args):
    out = QuietStdout()
    import torch
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the library has no CPU path")
    torch.cuda.set_device(local)
    device = "cuda:%d" % local
    import __graft_entry__ as graft
    pkg = graft.load_package()
    md, szlib, ep = pkg.model, pkg.lib, pkg.ep
    replicas = world > 1 and args.parallelism == "replicas"   # every GPU holds the whole model and decodes requests of its own: no exchange
    if world > 1:
        import torch.distributed as dist
        os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
        os.environ.setdefault("NCCL_DEBUG_FILE", "/dev/stderr")   # stdout carries the one JSON line
        dist.init_process_group("nccl")
        if replicas:
            pass
        elif args.exchange == "nccl":
            ep.init_from_process_group()
        else:
            peer = ep.PeerExchange(C3["hidden"])
    hbm, peak_kind = peaks()
    cfg = c3_model_cfg(args, args.n_layer)
    head_type = szlib.TYPE_Q8_0 if args.head == "q8" else szlib.TYPE_EXL3(4)
    M = md.make_model(cfg, dense_type=szlib.TYPE_Q8_0, expert_type=szlib.TYPE_EXL3(3), seed=1, device=device, cycle_alpha=args.alpha,
                      cycle_beta=args.beta, head_type=head_type)
    dm = md.DeviceModel(M, device, ep=(rank, world) if world > 1 and not replicas else None)
    # every tensor outside the experts is read once a pass, except the embedding table (m rows gathered)
    dense_bytes = sum(t[3].numel() * t[3].element_size() for n, t in M["tensors"].items() if n != "token_embd.weight")
    if args.head == "proxy":
        # the screened head reads its 2-bit proxy and the kept blocks, not the whole blob: at most 4 rows x 128 blocks of 128 outputs
        blob = M["tensors"]["output.weight"][3].numel()
        dense_bytes += cfg["vocab"] * cfg["hidden"] // 4 + cfg["vocab"] * (cfg["hidden"] // 128) * 2 + 512 * 128 * cfg["hidden"] // 2 - blob
    dense_bytes += sum(Ld["router"].numel() * 4 + Ld["shared_router"].numel() * 4 for Ld in M["moe"])
    del M
    torch.cuda.empty_cache()
    ctx = args.ctx
    K, W = args.steps, max(args.warmup, 3)
    n_prompt, n_new = 256, args.request_tokens
    sess = md.Session(dm, ctx + n_new + 64, kv_q8=True, head_proxy=args.head == "proxy")
    _, cyc = md.token_cycles(cfg["vocab"], 1)
    stream = sess._stream

    def request(i):
        """Request i of the workload: the cache up to ctx - 256 filled in place with seeded values of the cache's own distribution
        (the long context), then a 256-token prompt of its own - one of the model's token cycles repeated, 10% of the tokens
        substituted at random - fed through the model.  Returns the generator, positioned after the prompt."""
        sess.fill_synthetic(ctx - n_prompt, seed=3)
        # (replicas: every rank takes requests of its own; expert parallelism: every rank the same ones)
        return md.Generator(sess, md.make_prompt(n_prompt, cfg["vocab"], seed=1 + (i * world + rank if replicas else i), cycles=cyc), n_new, spec_k=3)

    if args.profile_passes > 0:
        # for a profiler: N verify passes of 4 rows and nothing else (run with SZ_SESSION_GRAPHS=0 to see every launch by name)
        sess.fill_synthetic(ctx - n_prompt, seed=3)
        prompt = md.make_prompt(n_prompt, cfg["vocab"], seed=1, cycles=cyc)
        for i in range(args.profile_passes):
            sess.verify([int(t) for t in prompt[4 * i:4 * i + 4]], accept=1)
            (keep, _), _, _ = sess.result()
            sess.commit(keep)
        torch.cuda.synchronize()
        out.emit(json.dumps({"profile_passes": args.profile_passes, "rows": 4, "context": ctx, "n_layer": cfg["n_layer"]}))
        return

    def barrier():
        if world > 1:
            import torch.distributed as dist
            dist.barrier()
        torch.cuda.synchronize()

    def agree(v, op="max"):
        if world == 1:
            return v
        import torch.distributed as dist
        t = torch.tensor([v], device=device, dtype=torch.float64)
        dist.all_reduce(t, op={"max": dist.ReduceOp.MAX, "min": dist.ReduceOp.MIN, "sum": dist.ReduceOp.SUM}[op])
        return float(t[0])

    def agree_max(v):
        return agree(v, "max")

    # --- the workload: a stream of requests.  Every request decodes n_new tokens after its prompt through the public loop (host
    # drafter, ids host -> device, result device -> host every round).  Only decode rounds are timed - the prompt passes and the
    # cache fill between requests are not - and the rounds of whole requests are added up:
    #   value = tokens / the device time of the passes (events on the session's stream around each pass: the graph of the pass
    #           with acceptance and commit; cache and weights resident);  e2e = tokens / wall clock of the loop.
    # Warm-up: whole requests, untimed, until at least W rounds ran (the first request also records the CUDA graphs).  Timed: whole
    # requests until at least K rounds and a second of device time; every rank runs the same requests (the tokens are the same
    # bits on every rank), and the decision to go on is taken on the slowest rank's clock.
    tot = dict(n=0, rounds=0, passes=0, drafted=0, accepted=0, dev_ms=0.0, wall_s=0.0, draft_ms=0.0, verify_ms=0.0, commit_ms=0.0,
               tried=[0] * 8, right=[0] * 8, requests=0)

    def run_request(i, acc):
        gen = request(i)
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        st = gen.run(0)
        stream.synchronize()
        wall = time.perf_counter() - t0
        if acc is not None:
            acc["n"] += st.n_tokens; acc["rounds"] += st.rounds; acc["passes"] += st.passes; acc["drafted"] += st.drafted
            acc["accepted"] += st.accepted; acc["dev_ms"] += st.device_ms; acc["wall_s"] += wall
            acc["draft_ms"] += st.draft_ms; acc["verify_ms"] += st.verify_ms; acc["commit_ms"] += st.commit_ms
            for j in range(8):
                acc["tried"][j] += st.pos_tried[j]; acc["right"][j] += st.pos_right[j]
            acc["requests"] += 1
        rounds = st.rounds
        del gen
        return rounds

    req, warm_rounds = 0, 0
    while warm_rounds < W or req == 0:
        warm_rounds += run_request(req, None)
        req += 1
    barrier()
    sampler = ClockSampler(torch.cuda.current_device())
    sampler.start()
    while True:
        run_request(req, tot)
        req += 1
        # every rank runs the same number of requests: the run ends when the slowest-to-fill rank has its K rounds and its second
        if agree(1.0 if tot["rounds"] >= K and tot["dev_ms"] >= 1000.0 else 0.0, "min") > 0.5 or tot["requests"] >= 400:
            break
    barrier()
    clocks = sampler.stop()
    dev_ms, wall_s = agree_max(tot["dev_ms"]), agree_max(tot["wall_s"])
    rounds, toks = tot["rounds"], tot["n"]
    if replicas:   # the job's tokens: every rank's
        toks = int(agree(toks, "sum"))
        for k_ in ("rounds", "passes", "drafted", "accepted", "requests"):
            tot[k_] = int(agree(tot[k_], "sum"))
        for j in range(8):
            tot["tried"][j] = int(agree(tot["tried"][j], "sum")); tot["right"][j] = int(agree(tot["right"][j], "sum"))
        rounds_all = tot["rounds"]
    else:
        rounds_all = rounds
    gen_stats = dict(tokens=toks, rounds=rounds_all, requests=tot["requests"], warmup_rounds=warm_rounds, drafting_rounds=tot["passes"],
                     drafted=tot["drafted"], accepted=tot["accepted"], tokens_per_round=toks / max(rounds_all, 1),
                     right_by_position=tot["right"][:3], tried_by_position=tot["tried"][:3],
                     accept_rate_by_position=[tot["right"][j] / max(tot["tried"][j], 1) for j in range(3)],
                     draft_ms=tot["draft_ms"], verify_ms=tot["verify_ms"], commit_ms=tot["commit_ms"])
    rows_avg = 1 + gen_stats["drafted"] / max(rounds_all, 1)   # rows of a pass: its own token and the drafts
    gen_stats["accept_rate"] = gen_stats["accepted"] / max(gen_stats["drafted"], 1)
    sess.fill_synthetic(ctx - n_prompt, seed=3)
    prompt = md.make_prompt(n_prompt, cfg["vocab"], seed=1, cycles=cyc)
    sess.prefill(prompt)
    sess.result()
    sess.commit((n_prompt - 1) % 8 + 1)

    # --- the verify step alone: one pass of m rows, device time, for m = 1 and m = 4 (spec K=3), median of 15
    def pass_us(m, n=15):
        # the prompt's first token and drafts from another token cycle: rejected, so the pass carries acceptance, replay and commit
        # and keeps one row, while its rows route like those of any pass (distinct tokens)
        ids = [int(prompt[0])] + [int(t) for t in other[:m - 1]]
        ts = []
        for i in range(n + 3):
            p0, p1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            p0.record(stream)
            sess.verify(ids, accept=1)
            p1.record(stream)
            (kept, _), _, _ = sess.result()
            sess.commit(kept)
            if i >= 3:
                ts.append(p0.elapsed_time(p1) * 1e3)
        ts.sort()
        return ts[len(ts) // 2]

    other = md.make_prompt(16, cfg["vocab"], seed=977, cycles=cyc, substitute=0.0)
    step_us = {m: pass_us(m) for m in (1, 4)}
    # --- routing of one 4-row pass: distinct experts per layer (the bytes the pass must read)
    sess.trace_routes(True)
    sess.verify([int(prompt[0])] + [int(t) for t in other[:3]], accept=0)
    sess.result()
    ridx, _ = sess.routes()
    sess.commit(1)
    sess.trace_routes(False)
    import numpy as np
    distinct = [int(np.unique(ridx[l]).size) for l in range(cfg["n_layer"])]
    # --- per-kernel attribution of one 4-row pass (eager, an event between launches: durations include the launch gap)
    nev = 4096
    evs = [torch.cuda.Event(enable_timing=True) for _ in range(nev)]
    for e in evs:
        e.record(stream)
    stream.synchronize()
    arr = (C.c_uint64 * nev)(*[e.cuda_event for e in evs])
    L = szlib.load()
    n_k = 0
    for rep in range(2):
        szlib.check(L.sz_trace_begin(arr, nev, sess.stream))
        sess.verify([int(prompt[0])] + [int(t) for t in other[:args.trace_rows - 1]], accept=1)
        n_k = L.sz_trace_end()
        (kept, _), _, _ = sess.result()
        sess.commit(kept)
    per = {}
    for i in range(1, n_k):
        per.setdefault(L.sz_trace_name(i).decode(), []).append(evs[i - 1].elapsed_time(evs[i]) * 1e3)
    kern = {nm: {"launches": len(v), "avg_us": sum(v) / len(v), "total_us": sum(v)} for nm, v in per.items()}
    del sess
    if world > 1:
        import torch.distributed as dist
        dist.barrier()
        if replicas:
            pass
        elif args.exchange == "nccl":
            szlib.check(L.sz_ep_destroy())
        else:
            assert peer.status() == 0, "a wait of the peer exchange ran out"
            peer.close()
    if rank != 0:
        return

    by = c3_bytes(cfg, ctx, distinct, dense_bytes)
    be = expert_bytes("exl3", cfg["hidden"], cfg["expert_ff"])
    # traffic: dram__bytes_read + write of one launch of this kernel on these shapes (39 + 1 experts), from an ncu --set full capture
    roof = {"bound": "hbm", "peak": hbm, "unit": "GB/s", "peak_kind": peak_kind,
            "traffic": gateup_traffic(sum(distinct) / len(distinct) / (1 if replicas else world) + 1),
            "traffic_source": "profiles/c2_moe_gateup_exl3_full.md: ncu capture of the same kernel and expert shapes on the c2-moe workload, "
                              "scaled by the experts a launch streams", "kernel": "gateup_exl3s"}
    ks = kern.get("gateup_exl3s")
    if ks:
        # gate + up of a layer's distinct routed experts and of the shared expert: 2/3 of their bytes, one launch a layer
        per_launch = (sum(distinct) / len(distinct) / (1 if replicas else world) + 1) * be * 2 / 3
        roof.update(achieved=per_launch / (ks["avg_us"] * 1e-6) / 1e9, kernel_us=ks["avg_us"], bytes_per_launch=per_launch)
        roof["frac"] = roof["achieved"] / hbm
    roof.update(step_bytes=by["experts_kv"], step_bytes_all=by["all"], step_us=step_us[4],
                step_achieved=by["experts_kv"] / (step_us[4] * 1e-6) / 1e9, step_achieved_all=by["all"] / (step_us[4] * 1e-6) / 1e9)
    roof["step_frac"] = roof["step_achieved"] / hbm
    roof["step_frac_all"] = roof["step_achieved_all"] / hbm
    value = toks / (dev_ms * 1e-3)
    cpu = None
    if world == 1 and args.cpu_seconds > 0:
        cpu = cpu_c3(pkg, args.cpu_seconds, os.cpu_count() or 1, args.head, ctx, C3_INDEXER if args.indexer else None)
    line = {
        "metric": C3_METRIC, "value": value, "unit": "tok/s", "n_gpus": args.gpus, "steps": K, "warmup": W, "rounds_timed": rounds,
        "ms_per_step": dev_ms / max(rounds, 1), "higher_is_better": True, "scaling": "weak" if replicas else "strong", "vs_baseline": None,
        "dtype": "f32 activations, f16 EXL3 codebook weights, int8 Q8_0 / Q8_KV, f32 accumulate (router, norms, combine in f64)",
        "data": "synthetic",
        "config": c3_config(args, cfg, ctx, by["all"]),
        "speculation": gen_stats, "verify_step_us": {"rows_1": step_us[1], "rows_4": step_us[4]},
        "roofline": roof, "cpu_baseline": cpu,
        "e2e": {"value": toks / wall_s, "unit": "tok/s", "h2d_bytes_per_step": 128, "d2h_bytes_per_step": 8 + 512 * rows_avg,
                "wall_ms_per_step": wall_s * 1e3 / max(rounds, 1)},
        "gpu_launches": (n_k - 1) * rounds, "launches_per_pass": n_k - 1, "clocks": clocks,
        "kernels": {k: v for k, v in sorted(kern.items(), key=lambda kv: -kv[1]["total_us"])},
    }
    out.emit(json.dumps(line))


# ---- workload c4-tree: one verify pass over a draft tree on the config-3 model ------------------------------------------------------
# Benchmark config 4 asks for a 16-node tree (depth 4, branching [4, 2, 1, 1]).  A pass of this library - like the reference's - has
# at most 8 rows (MAX_VERIFY), the root included, so the tree here has 7 drafted nodes: depth 4, branching [3, 2, 1, 1].
C4_PARENTS = [-1, 0, 0, 0, 1, 1, 4, 6]
C4_METRIC = "verify-step us (draft tree, 8 rows, depth 4)"


def run_c4(args):
    out = QuietStdout()
    import numpy as np
    import torch
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the library has no CPU path")
    if int(os.environ.get("WORLD_SIZE", "1")) > 1:
        raise SystemExit("the c4-tree workload runs on one GPU")
    torch.cuda.set_device(0)
    device = "cuda:0"
    import __graft_entry__ as graft
    pkg = graft.load_package()
    md, szlib = pkg.model, pkg.lib
    hbm, peak_kind = peaks()
    cfg = dict(C3, n_layer=args.n_layer)
    head_type = szlib.TYPE_Q8_0 if args.head == "q8" else szlib.TYPE_EXL3(4)
    M = md.make_model(cfg, dense_type=szlib.TYPE_Q8_0, expert_type=szlib.TYPE_EXL3(3), seed=1, device=device, cycle_alpha=args.alpha,
                      cycle_beta=args.beta, head_type=head_type)
    dm = md.DeviceModel(M, device)
    del M
    torch.cuda.empty_cache()
    ctx, n_prompt = args.ctx, 256
    K, W = args.steps, max(args.warmup, 3)
    sess = md.Session(dm, ctx + 8 * (K + W) * 3 + 64, kv_q8=True, head_proxy=args.head == "proxy")
    stream = sess._stream
    _, cyc = md.token_cycles(cfg["vocab"], 1)
    sess.fill_synthetic(ctx - n_prompt, seed=3)
    prompt = md.make_prompt(n_prompt, cfg["vocab"], seed=1, cycles=cyc)
    sess.prefill(prompt)
    _, top, _ = sess.result()
    sess.commit((n_prompt - 1) % 8 + 1)
    nxt = int(top[(n_prompt - 1) % 8][64])
    rng = np.random.default_rng(4)
    parents = C4_PARENTS
    m = len(parents)
    L = szlib.load()
    sampler = md.Sampler(0.7, 64, 0.9, 0.0, 17)

    def tree_ids(root):
        return [int(root)] + [int(t) for t in rng.integers(0, cfg["vocab"], m - 1)]   # draft tokens uniform over the vocabulary

    def greedy_pass(root):
        """device acceptance: ids host -> device, {kept, next} and the path device -> host"""
        ids = tree_ids(root)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0 = time.perf_counter()
        e0.record(stream)
        sess.verify_tree(ids, parents, accept=1)
        e1.record(stream)
        (keep, nx), _, _ = sess.result()
        sess.commit(keep)
        stream.synchronize()
        return e0.elapsed_time(e1) * 1e3, (time.perf_counter() - t0) * 1e6, keep, nx

    def sampled_pass(root, pos):
        """host acceptance by rejection sampling against uniform-random draft probabilities, then the path commit"""
        ids = tree_ids(root)
        q = rng.random(m).astype(np.float32)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0 = time.perf_counter()
        e0.record(stream)
        sess.verify_tree(ids, parents, accept=0)
        _, top, _ = sess.result()
        a, p = np.array(ids, dtype=np.uint32), np.array(parents, dtype=np.int32)
        path = np.zeros(m, dtype=np.int32)
        nx = C.c_uint32()
        n = L.sz_tree_accept_sampled(C.byref(sampler), top.ctypes.data, a.ctypes.data, p.ctypes.data, m, q.ctypes.data, pos, -1, path.ctypes.data, C.byref(nx))
        sess.commit_path([int(t) for t in path[:n]])
        e1.record(stream)
        stream.synchronize()
        return e0.elapsed_time(e1) * 1e3, (time.perf_counter() - t0) * 1e6, n, int(nx.value)

    for _ in range(W):
        _, _, _, nxt = greedy_pass(nxt)
    clock = ClockSampler(torch.cuda.current_device())
    clock.start()
    dev, wall, kept = [], [], []
    for _ in range(K):
        d, w_, k_, nxt = greedy_pass(nxt)
        dev.append(d); wall.append(w_); kept.append(k_)
    sdev, swall, skept = [], [], []
    for i in range(K):
        d, w_, k_, nxt = sampled_pass(nxt, 1000 + 8 * i)
        sdev.append(d); swall.append(w_); skept.append(k_)
    clocks = clock.stop()
    # routing of one tree pass: distinct experts per layer (the bytes the pass must read)
    sess.trace_routes(True)
    sess.verify_tree(tree_ids(nxt), parents)
    sess.result()
    ridx, _ = sess.routes()
    sess.commit_path([0])
    sess.trace_routes(False)
    distinct = [int(np.unique(ridx[l]).size) for l in range(cfg["n_layer"])]
    # launches of one tree pass (eager, counted by the library's trace)
    nev = 4096
    evs = [torch.cuda.Event(enable_timing=True) for _ in range(nev)]
    for e in evs:
        e.record(stream)
    stream.synchronize()
    arr = (C.c_uint64 * nev)(*[e.cuda_event for e in evs])
    szlib.check(L.sz_trace_begin(arr, nev, sess.stream))
    sess.verify_tree(tree_ids(nxt), parents, accept=1)
    n_k = L.sz_trace_end()
    (kept1, _), _, _ = sess.result()
    sess.commit(kept1)
    by = c3_bytes(cfg, ctx, distinct, 0)
    med = sorted(dev)[len(dev) // 2]
    line = {
        "metric": C4_METRIC, "value": med, "unit": "us", "n_gpus": 1, "steps": K, "warmup": W, "ms_per_step": med / 1e3, "higher_is_better": False,
        "scaling": "weak", "vs_baseline": None, "dtype": "f32 activations, f16 EXL3 codebook weights, int8 Q8_0 / Q8_KV, f32 accumulate", "data": "synthetic",
        "config": {"workload": "c4-tree", "n_layer": cfg["n_layer"], "context": ctx, "tree_rows": m, "parents": parents, "depth": 4, "branching": [3, 2, 1, 1],
                   "note": "benchmark config 4 names 16 nodes with branching [4, 2, 1, 1]; a pass holds at most 8 rows (the root included), so the tree has 7 "
                           "drafted nodes; draft tokens uniform over the vocabulary, draft probabilities uniform random; parity of tree passes is against "
                           "this repository's own CPU restatement (the reference has no tree verification)",
                   "l2": "inputs larger than L2: a pass streams several GB of weights and cache"},
        "tree": {"greedy": {"us_per_verify": med, "accepted_len_mean": sum(kept) / len(kept)},
                 "sampled_T0.7_top_p0.9": {"us_per_verify": sorted(sdev)[len(sdev) // 2], "accepted_len_mean": sum(skept) / len(skept),
                                            "note": "pass without device acceptance, top-64 rows to the host, rejection sampling there, commit of the kept path"}},
        "roofline": {"bound": "hbm", "peak": hbm, "unit": "GB/s", "peak_kind": peak_kind, "step_bytes": by["experts_kv"], "achieved": by["experts_kv"] / (med * 1e-6) / 1e9,
                     "frac": by["experts_kv"] / (med * 1e-6) / 1e9 / hbm, "traffic": None, "distinct_experts_per_layer": sum(distinct) / len(distinct)},
        "cpu_baseline": None,
        "e2e": {"value": sorted(wall)[len(wall) // 2], "unit": "us", "h2d_bytes_per_step": 4 * m + 128, "d2h_bytes_per_step": 8 + 64 + 512 * m},
        "gpu_launches": (n_k - 1) * 2 * K, "launches_per_pass": n_k - 1, "clocks": clocks,
    }
    out.emit(json.dumps(line))


def cpu_c3(pkg, budget_s, threads, head="q8", ctx=C3_CTX, extra=None):
    """Accepted tok/s of the CPU restatement of the reference's scalar path on the config-3 shapes, at the benchmark's context.
    The CPU path verifies one token at a time (a batched pass is bitwise the one-at-a-time pass there), so its accepted tok/s is
    1 / (seconds a token).  Sample: models of 4 and of 8 layers (one and two periods of the 3:1 pattern) with the full-size layers,
    vocabulary and head; the attention layers' caches are filled to the benchmark's context with the same seeded history the GPU
    arm uses, then a few tokens are stepped; a token of the 48-layer model costs t4 + 11 * (t8 - t4)."""
    import torch  # noqa: F401
    from oracle import binding as ob
    md, szlib = pkg.model, pkg.lib
    per = {}
    ntok = 0
    for nl in (4, 8):
        cfg = dict(C3, n_layer=nl, **(extra or {}))
        # (the time of a token does not depend on which tokens come out: with an EXL3 head, whose token cycles need a GPU to build,
        # the sample's model has none; the CPU path always evaluates the head in full, as the reference's --exact does)
        M = md.make_model(cfg, dense_type=szlib.TYPE_Q8_0, expert_type=szlib.TYPE_EXL3(3), seed=1, device="cpu",
                          cycle_alpha=C3_ALPHA if head == "q8" else 0.0, head_type=szlib.TYPE_Q8_0 if head == "q8" else szlib.TYPE_EXL3(4))
        hm = md.HostModel(M)
        s = ob.Session(hm, kv_q8=True, threads=threads)
        s.fill_synthetic(max(ctx - 32, 0), seed=3)
        s.step(1, want_logits=True)  # warm: page the weights in
        t0, n = time.perf_counter(), 0
        while True:
            s.step(2 + n, want_logits=True)
            n += 1
            if time.perf_counter() - t0 > budget_s / 3 or n >= 16:
                break
        per[nl] = (time.perf_counter() - t0) / n
        ntok += n
        del s, hm, M
    t_tok = per[4] + 11 * max(per[8] - per[4], 0.0)
    return {"value": 1.0 / t_tok, "unit": "tok/s", "cores": threads, "kind": "port",
            "sample": "%d tokens through 4- and 8-layer slices of the model (full-size layers, vocabulary, head) at context %d; "
                      "seconds a token extrapolated to 48 layers: %.3f" % (ntok, ctx, t_tok),
            "seconds_per_token": t_tok, "t4": per[4], "t8": per[8]}


def run_reference_c3(args):
    """The reference arm: the reference's own CPU implementation of the path - its scalar Session restated in C (the reference is
    Rust and cannot be built here) - on all host cores, on a bounded sample of the config-3 workload at the same context."""
    if int(os.environ.get("RANK", "0")) != 0:
        return
    import __graft_entry__ as graft
    pkg = graft.load_package()
    threads = os.cpu_count() or 1
    cpu = cpu_c3(pkg, max(10.0, min(60.0, 2.0 * args.steps)), threads, args.head, args.ctx, C3_INDEXER if args.indexer else None)
    v = cpu["value"]
    cpu_line = {k: cpu[k] for k in ("value", "unit", "cores", "kind", "sample")}
    print(json.dumps({
        "impl": "reference", "metric": C3_METRIC, "value": v, "unit": "tok/s", "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": 1e3 / v, "higher_is_better": True, "scaling": "weak" if args.gpus > 1 and args.parallelism == "replicas" else "strong",
        "vs_baseline": None, "dtype": "f32 (f64 accumulate)",
        "data": "synthetic", "config": c3_config(args, c3_model_cfg(args, args.n_layer), args.ctx),
        "cpu_baseline": cpu_line, "e2e": {"value": v, "unit": "tok/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}))


# ---- workload c5-concurrent: B sequences at once on every GPU ----------------------------------------------------------------------
def run_c5(args):
    """Config 5's shape of load - many sequences decoding at once, spec K=3 each - served by B independent verify sessions a GPU over
    one resident model: a session, a stream, CUDA graphs and a host thread (drafter + loop) per sequence.  A single pass leaves most
    of the GPU idle (it is a chain of short dependent kernels), so the passes of different sequences overlap.  Kernels are NOT
    batched across sequences: every sequence streams its own experts.  N > 1: every GPU holds the whole model and B sequences of its
    own (no exchange on the data path).  Waves: every sequence takes a request (cache filled to the context, 256-token prompt fed:
    untimed), then all decode their tokens at once (timed, device time between events around the wave)."""
    import threading
    out = QuietStdout()
    import torch
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        raise SystemExit("--gpus %d but WORLD_SIZE=%d (launch with torch.distributed.run for N > 1)" % (args.gpus, world))
    torch.cuda.set_device(local)
    device = "cuda:%d" % local
    import __graft_entry__ as graft
    pkg = graft.load_package()
    md, szlib = pkg.model, pkg.lib
    if world > 1:
        import torch.distributed as dist
        os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
        os.environ.setdefault("NCCL_DEBUG_FILE", "/dev/stderr")
        dist.init_process_group("nccl")
    cfg = c3_model_cfg(args, args.n_layer)
    head_type = szlib.TYPE_Q8_0 if args.head == "q8" else szlib.TYPE_EXL3(4)
    M = md.make_model(cfg, dense_type=szlib.TYPE_Q8_0, expert_type=szlib.TYPE_EXL3(3), seed=1, device=device, cycle_alpha=args.alpha,
                      cycle_beta=args.beta, head_type=head_type)
    dm = md.DeviceModel(M, device)
    del M
    torch.cuda.empty_cache()
    B, ctx, n_prompt, n_new = args.sequences, args.ctx, 256, args.request_tokens
    _, cyc = md.token_cycles(cfg["vocab"], 1)
    sessions = [md.Session(dm, ctx + n_new + 64, kv_q8=True, head_proxy=args.head == "proxy") for _ in range(B)]
    gens = [None] * B
    stats = [None] * B
    errors = []

    def prepare(b, wave):
        try:
            sessions[b].fill_synthetic(ctx - n_prompt, seed=3)
            gens[b] = md.Generator(sessions[b], md.make_prompt(n_prompt, cfg["vocab"], seed=1 + (wave * B + b) * world + rank, cycles=cyc), n_new, spec_k=3)
        except Exception as e:   # noqa: BLE001
            errors.append(repr(e))

    def decode(b):
        try:
            stats[b] = gens[b].run(0)
            sessions[b]._stream.synchronize()
        except Exception as e:   # noqa: BLE001
            errors.append(repr(e))

    def in_threads(fn, *a):
        ts = [threading.Thread(target=fn, args=(b,) + a) for b in range(B)]
        for t in ts:
            t.start()
        for t in ts:
            t.join()
        if errors:
            raise SystemExit("c5-concurrent: " + errors[0])

    def barrier():
        if world > 1:
            import torch.distributed as dist
            dist.barrier()
        torch.cuda.synchronize()

    tot = dict(n=0, rounds=0, drafted=0, accepted=0, dev_ms=0.0, wall_s=0.0, pass_ms=0.0)
    clocks = None
    for wave in range(-1, args.waves):     # wave -1: warm-up (records every session's graphs)
        in_threads(prepare, wave + 1)
        barrier()
        if wave == 0:
            sampler = ClockSampler(torch.cuda.current_device())
            sampler.start()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        t0 = time.perf_counter()
        in_threads(decode)
        torch.cuda.synchronize()
        wall = time.perf_counter() - t0
        e1.record()
        torch.cuda.synchronize()
        if wave >= 0:
            tot["dev_ms"] += e0.elapsed_time(e1); tot["wall_s"] += wall
            for st in stats:
                tot["n"] += st.n_tokens; tot["rounds"] += st.rounds; tot["drafted"] += st.drafted; tot["accepted"] += st.accepted
                tot["pass_ms"] += st.device_ms
        for b in range(B):
            gens[b] = None
    barrier()
    clocks = sampler.stop()

    def agree(v, op):
        if world == 1:
            return v
        import torch.distributed as dist
        t = torch.tensor([v], device=device, dtype=torch.float64)
        dist.all_reduce(t, op={"max": dist.ReduceOp.MAX, "sum": dist.ReduceOp.SUM}[op])
        return float(t[0])

    dev_ms, wall_s = agree(tot["dev_ms"], "max"), agree(tot["wall_s"], "max")
    toks, rounds = int(agree(tot["n"], "sum")), int(agree(tot["rounds"], "sum"))
    drafted, accepted = int(agree(tot["drafted"], "sum")), int(agree(tot["accepted"], "sum"))
    if rank != 0:
        return
    hbm, peak_kind = peaks()
    line = {
        "metric": "accepted tok/s at spec K=3, %d sequences at once a GPU" % B, "value": toks / (dev_ms * 1e-3), "unit": "tok/s", "n_gpus": args.gpus,
        "steps": rounds, "warmup": B, "ms_per_step": dev_ms / max(rounds, 1), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "f32 activations, f16 EXL3 codebook weights, int8 Q8_0 / Q8_KV, f32 accumulate (router, norms, combine in f64)", "data": "synthetic",
        "config": dict(c3_config(args, cfg, ctx), workload="c5-concurrent", sequences_per_gpu=B, batch=B * world, waves=args.waves,
                       parallelism="replicas%d x %d sequences" % (world, B) if world > 1 else "%d sequences, one GPU" % B,
                       batching="none across sequences: a session, stream and CUDA graphs per sequence; passes of different sequences overlap on the GPU"),
        "speculation": {"tokens": toks, "rounds": rounds, "drafted": drafted, "accepted": accepted, "tokens_per_round": toks / max(rounds, 1)},
        "sequence_pass_ms": tot["pass_ms"] / max(tot["rounds"], 1),
        "roofline": {"bound": "hbm", "achieved": None, "peak": hbm, "unit": "GB/s", "frac": None, "traffic": None, "peak_kind": peak_kind,
                     "note": "the kernels are those of the c3 workload (see its line for the per-kernel roofline); this line measures how many of their chains one GPU overlaps"},
        "cpu_baseline": None,
        "e2e": {"value": toks / wall_s, "unit": "tok/s", "h2d_bytes_per_step": 128, "d2h_bytes_per_step": 8 + 512 * (1 + drafted / max(rounds, 1))},
        "gpu_launches": None, "clocks": clocks,
    }
    out.emit(json.dumps(line))


# ---- workload c5-moe: the MoE sublayer over the rows of many sequences -----------------------------------------------------------------
def run_c5_moe(args):
    """Config 2's layer shape (hidden 2048, 512 experts top-10 of FFN 512 + a shared expert, EXL3 3-bit) with config 5's batch:
    `rows` = 256 rows a step.  Timed: sz_moe_rows, a graph of K steps over `layers` distinct layers (weights larger than L2), and
    for comparison the same rows as rows / 4 verify-pass calls of 4 rows."""
    if args.gpus != 1:
        raise SystemExit("the c5-moe workload runs on one GPU")
    out = QuietStdout()
    import torch
    import __graft_entry__ as graft
    pkg = graft.load_package()
    szlib = pkg.lib
    torch.cuda.set_device(0)
    R, nl, K, W = args.rows, max(2, min(args.layers, 4)), max(4, min(args.steps, 32)), max(args.warmup, 3)
    ty = szlib.TYPE_EXL3(3)
    layers = [pkg.moe.MoeLayer(pkg.synth.make_moe_layer(C2["hidden"], C2["n_expert"], C2["top_k"], C2["expert_ff"], C2["shared_ff"], ty, ty, seed=1 + i,
                                                        device="cuda"), "cuda:0") for i in range(nl)]
    x = pkg.synth.normal((R, C2["hidden"]), 1.0, 5, "c5moe.x", device="cuda").to(torch.bfloat16).to(torch.float32).contiguous()
    y = torch.empty_like(x)
    stream = torch.cuda.Stream()
    with torch.cuda.stream(stream):
        for i in range(W):
            _, ridx, _ = layers[i % nl].moe_rows(x, y, want_routing=True, stream=stream)
        stream.synchronize()
        distinct = int(torch.unique(ridx).numel())
        ev = [torch.cuda.Event(enable_timing=True) for _ in range(4)]
        ev[0].record(stream)
        for i in range(K):
            layers[i % nl].moe_rows(x, y, stream=stream)
        ev[1].record(stream)
        stream.synchronize()
        rows_ms = ev[0].elapsed_time(ev[1]) / K
        # the same rows as verify passes of 4 rows (what a server without the batched form would run)
        for i in range(2):
            layers[i % nl].moe_batch(x[:4].contiguous(), stream=stream)
        xs = [x[c:c + 4].contiguous() for c in range(0, R, 4)]
        ys = torch.empty((4, C2["hidden"]), device="cuda")
        ev[2].record(stream)
        for i in range(2):
            for xc in xs:
                layers[i % nl].moe_batch(xc, ys, stream=stream)
        ev[3].record(stream)
        stream.synchronize()
        pass_ms = ev[2].elapsed_time(ev[3]) / 2
        # end to end: host rows up, result back, every step
        xh, yh = x.cpu().pin_memory(), torch.empty(x.shape, dtype=torch.float32).pin_memory()
        t0 = time.perf_counter()
        for i in range(K):
            x.copy_(xh, non_blocking=True)
            layers[i % nl].moe_rows(x, y, stream=stream)
            yh.copy_(y, non_blocking=True)
            stream.synchronize()
        e2e_us = (time.perf_counter() - t0) / K * 1e6
        # per-kernel attribution of one step (eager, an event between launches: durations include the launch gap)
        nev = 256
        evs = [torch.cuda.Event(enable_timing=True) for _ in range(nev)]
        for e in evs:
            e.record(stream)
        stream.synchronize()
        arr = (C.c_uint64 * nev)(*[e.cuda_event for e in evs])
        Lb = szlib.load()
        szlib.check(Lb.sz_trace_begin(arr, nev, stream.cuda_stream))
        layers[0].moe_rows(x, y, stream=stream)
        n_k = Lb.sz_trace_end()
        stream.synchronize()
        per = {}
        for i in range(1, n_k):
            per.setdefault(Lb.sz_trace_name(i).decode(), []).append(evs[i - 1].elapsed_time(evs[i]) * 1e3)
        kern = {nm: {"launches": len(v), "total_us": sum(v), "max_us": max(v)} for nm, v in per.items()}
    for l in layers:
        assert l.moe_rows_status(R) == 0
    hbm, peak_kind = peaks()
    be = expert_bytes("exl3", C2["hidden"], C2["expert_ff"])
    step_bytes = (distinct + 1) * be + C2["n_expert"] * C2["hidden"] * 4
    us = rows_ms * 1e3
    line = {"metric": "verify-step us (MoE sublayer, %d rows = %d sequences x K+1 = 4)" % (R, R // 4), "value": us, "unit": "us", "n_gpus": 1, "steps": K, "warmup": W,
            "ms_per_step": rows_ms, "higher_is_better": False, "scaling": "weak", "vs_baseline": None,
            "dtype": "f32 activations, f16 codebook weights, f32 accumulate (router and combine in f64)", "data": "synthetic",
            "config": {"workload": "c5-moe", "format": "exl3", **{k: v for k, v in C2.items() if k != "rows"}, "rows": R, "layers_cycled": nl,
                       "distinct_experts_per_step": distinct, "l2": "inputs larger than L2: %d layers of %d MB of expert weights cycled" % (nl, C2["n_expert"] * be >> 20)},
            "us_per_row": us / R, "as_passes_of_4_rows_us": pass_ms * 1e3, "speedup_over_passes_of_4": pass_ms / rows_ms,
            "roofline": {"bound": "hbm", "achieved": step_bytes / (us * 1e-6) / 1e9, "peak": hbm, "unit": "GB/s", "frac": step_bytes / (us * 1e-6) / 1e9 / hbm,
                         "peak_kind": peak_kind, "traffic": None, "step_bytes": step_bytes,
                         "note": "bytes = every distinct expert once + the router; the expert kernels are the verify pass's (decode-bound, see the c2-moe line)"},
            "cpu_baseline": None,
            "e2e": {"value": e2e_us, "unit": "us", "h2d_bytes_per_step": R * C2["hidden"] * 4, "d2h_bytes_per_step": R * C2["hidden"] * 4},
            "gpu_launches": K * (n_k - 1), "launches_per_step": n_k - 1, "kernels": kern,
            "clocks": {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}}
    out.emit(json.dumps(line))


# ---- workload c5-batch: B sequences in lockstep, what reads weights shared -----------------------------------------------------------
def run_c5_batch(args):
    """Config 5's batch on the config-3 model: B sequences a GPU, every one with a session of its own (cache filled to the context,
    a 256-token prompt fed through it: untimed), then all decode `request_tokens` tokens in lockstep, spec K=3 each, through
    sz_batch_gen_run: a step runs every sequence's attention and head, and the reads, projections, scans and MoE sublayer of a
    layer ONCE over the rows of all of them.
    N > 1: every GPU holds the whole model and B sequences of its own.  Timed: the steps' device time (events around each step) and
    the wall clock of the loop."""
    out = QuietStdout()
    import torch
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        raise SystemExit("--gpus %d but WORLD_SIZE=%d (launch with torch.distributed.run for N > 1)" % (args.gpus, world))
    torch.cuda.set_device(local)
    device = "cuda:%d" % local
    import __graft_entry__ as graft
    pkg = graft.load_package()
    md, szlib = pkg.model, pkg.lib
    if world > 1:
        import torch.distributed as dist
        os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
        os.environ.setdefault("NCCL_DEBUG_FILE", "/dev/stderr")
        dist.init_process_group("nccl")
    cfg = c3_model_cfg(args, args.n_layer)
    head_type = szlib.TYPE_Q8_0 if args.head == "q8" else szlib.TYPE_EXL3(4)
    M = md.make_model(cfg, dense_type=szlib.TYPE_Q8_0, expert_type=szlib.TYPE_EXL3(3), seed=1, device=device, cycle_alpha=args.alpha,
                      cycle_beta=args.beta, head_type=head_type)
    dm = md.DeviceModel(M, device)
    del M
    torch.cuda.empty_cache()
    B, ctx, n_prompt, n_new = args.sequences, args.ctx, 256, args.request_tokens
    _, cyc = md.token_cycles(cfg["vocab"], 1)
    # --contexts a,b,c: every sequence's context (history + prompt) is one of these, drawn with a fixed seed (benchmark config 5:
    # 3k, 9.6k or 15k tokens before the decode); default: every sequence at --ctx
    if args.contexts:
        choices = [int(v) for v in args.contexts.split(",")]
        rng_c = __import__("numpy").random.default_rng(5 + rank)
        ctx_of = [int(choices[int(rng_c.integers(0, len(choices)))]) for _ in range(B)]
        ctx = max(ctx_of)
    else:
        ctx_of = [ctx] * B
    batch = md.Batch(dm, B, ctx + n_new + 64, head_proxy=args.head == "proxy")

    def barrier():
        if world > 1:
            import torch.distributed as dist
            dist.barrier()
        torch.cuda.synchronize()

    if args.profile_steps > 0:
        # for a profiler: N steps of the B sequences with 1..4 rows each (no prompts, no timing); the last step sits between
        # cudaProfilerStart and cudaProfilerStop, so `ncu --profile-from-start off` lists exactly its launches
        for s in batch.sessions:
            s.fill_synthetic(ctx - n_prompt, seed=3)
        prompts = [md.make_prompt(n_prompt, cfg["vocab"], seed=1 + b, cycles=cyc) for b in range(B)]
        at = [0] * B
        rows_of = 0
        for step in range(args.profile_steps):
            ms = [1 + (b + step) % 4 for b in range(B)]
            rows = [[int(t) for t in prompts[b][at[b]:at[b] + ms[b]]] for b in range(B)]
            last = step == args.profile_steps - 1
            torch.cuda.synchronize()
            if last:
                torch.cuda.profiler.start()
            batch.verify(rows, accept=1)
            torch.cuda.synchronize()
            if last:
                torch.cuda.profiler.stop()
                rows_of = sum(ms)
            for b, sess in enumerate(batch.sessions):
                (keep, _), _, _ = sess.result()
                sess.commit(keep)
                at[b] += keep
        out.emit(json.dumps({"profile_steps": args.profile_steps, "sequences": B, "rows_of_last_step": rows_of, "context": ctx, "n_layer": cfg["n_layer"]}))
        return

    tot = dict(n=0, rounds=0, steps=0, drafted=0, accepted=0, dev_ms=0.0, wall_s=0.0, prefill_s=0.0, prefill_tokens=0)
    sampler = None
    for wave in range(-1, args.waves):     # wave -1: warm-up
        for s, cb in zip(batch.sessions, ctx_of):
            s.fill_synthetic(cb - n_prompt, seed=3)
        prompts = [md.make_prompt(n_prompt, cfg["vocab"], seed=1 + ((wave + 1) * B + b) * world + rank, cycles=cyc) for b in range(B)]
        torch.cuda.synchronize()
        tp = time.perf_counter()
        if args.feed == "alone":
            gens = [md.Generator(s, p, n_new, spec_k=3) for s, p in zip(batch.sessions, prompts)]   # the prompts, one session at a time
        else:
            gens = batch.begin(prompts, n_new, spec_k=3)                                            # ... or in lockstep (sz_batch_prefill)
        torch.cuda.synchronize()
        if wave >= 0:
            tot["prefill_s"] += time.perf_counter() - tp
            tot["prefill_tokens"] += B * n_prompt
        barrier()
        if wave == 0:
            sampler = ClockSampler(torch.cuda.current_device())
            sampler.start()
        n = len(gens)
        gh = (C.c_void_p * n)(*[g.h for g in gens])
        outs = (C.c_void_p * n)(*[C.cast(g.out, C.c_void_p) for g in gens])
        sts = (C.c_void_p * n)(*[C.cast(C.pointer(g.stats), C.c_void_p) for g in gens])
        dev = C.c_double(0.0)
        t0 = time.perf_counter()
        szlib.check(batch.lib.sz_batch_gen_run(gh, n, 0, outs, sts, batch.rows_max, batch.scratch, batch.scratch_bytes, C.byref(dev), batch.stream))
        torch.cuda.synchronize()
        wall = time.perf_counter() - t0
        if wave >= 0:
            tot["dev_ms"] += dev.value; tot["wall_s"] += wall
            tot["steps"] += max(g.stats.rounds for g in gens)
            for g in gens:
                tot["n"] += g.stats.n_tokens; tot["rounds"] += g.stats.rounds; tot["drafted"] += g.stats.drafted; tot["accepted"] += g.stats.accepted
        del gens
    barrier()
    clocks = sampler.stop()

    def agree(v, op):
        if world == 1:
            return v
        import torch.distributed as dist
        t = torch.tensor([v], device=device, dtype=torch.float64)
        dist.all_reduce(t, op={"max": dist.ReduceOp.MAX, "sum": dist.ReduceOp.SUM}[op])
        return float(t[0])

    dev_ms, wall_s = agree(tot["dev_ms"], "max"), agree(tot["wall_s"], "max")
    toks, rounds = int(agree(tot["n"], "sum")), int(agree(tot["rounds"], "sum"))
    drafted, accepted = int(agree(tot["drafted"], "sum")), int(agree(tot["accepted"], "sum"))
    if rank != 0:
        return
    hbm, peak_kind = peaks()
    steps = tot["steps"]
    line = {
        "metric": "accepted tok/s at spec K=3, %d sequences in lockstep a GPU" % B, "value": toks / (dev_ms * 1e-3), "unit": "tok/s", "n_gpus": args.gpus,
        "steps": steps, "warmup": B, "ms_per_step": dev_ms / max(steps, 1), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "f32 activations, f16 EXL3 codebook weights, int8 Q8_0 / Q8_KV, f32 accumulate (router, norms, combine in f64)", "data": "synthetic",
        "config": dict(c3_config(args, cfg, ctx), workload="c5-batch", sequences_per_gpu=B, batch=B * world, waves=args.waves,
                       contexts=sorted(set(ctx_of)), request_tokens=n_new,
                       parallelism="replicas%d x %d sequences" % (world, B) if world > 1 else "%d sequences, one GPU" % B,
                       batching="a step = every sequence's own attention and head (its session's kernels) + the reads, projections, scans and MoE "
                                "sublayer of a layer once over the rows of all sequences; launched eagerly"),
        "prefill": {"feed": args.feed, "tokens": tot["prefill_tokens"], "tok_s": tot["prefill_tokens"] / max(tot["prefill_s"], 1e-9),
                    "note": "the 256-token prompts of the sequences (untimed in `value`), wall clock on rank 0"},
        "speculation": {"tokens": toks, "rounds": rounds, "drafted": drafted, "accepted": accepted, "tokens_per_round": toks / max(rounds, 1),
                        "rows_per_step": (rounds + drafted) / max(steps, 1)},
        "roofline": {"bound": "hbm", "achieved": None, "peak": hbm, "unit": "GB/s", "frac": None, "traffic": None, "peak_kind": peak_kind,
                     "note": "see the c3 line for the per-kernel roofline of the sessions' kernels and the c5-moe line for the shared MoE sublayer"},
        "cpu_baseline": None,
        "e2e": {"value": toks / wall_s, "unit": "tok/s", "h2d_bytes_per_step": 128 * B + 1600, "d2h_bytes_per_step": B * (8 + 512 * (1 + drafted / max(rounds, 1)))},
        "gpu_launches": None, "clocks": clocks,
    }
    out.emit(json.dumps(line))


# ---- workload prefill-dense: many token rows through one dense projection on tcgen05 ------------------------------------------------
PD = dict(rows=12288, cols=2048)     # attn_qkv (8,192) + attn_gate (4,096) of a config-3 DeltaNet layer, one Q8_0 matrix
PD_METRIC = "dense projection TFLOP/s (Q8_0 weights, many token rows, tcgen05)"


def cpu_prefill_dense(tokens, seconds, wb):
    """The restated arithmetic of the reference's tensor-core projection on the host cores (numpy, f32 matmul of the f16-rounded
    operands), on a bounded sample: as many token rows as fit the time box."""
    import numpy as np
    from oracle import binding as ob
    w = ob.dequant(ob.Q8_0, wb).reshape(PD["rows"], PD["cols"]).astype(np.float16).astype(np.float32)
    n = min(tokens, 64)
    x = np.random.default_rng(1).standard_normal((n, PD["cols"])).astype(np.float16).astype(np.float32)
    x @ w.T
    t0, reps = time.perf_counter(), 0
    while time.perf_counter() - t0 < max(seconds, 0.5):
        x @ w.T
        reps += 1
    dt = (time.perf_counter() - t0) / reps
    return {"value": 2.0 * n * PD["rows"] * PD["cols"] / dt / 1e12, "unit": "TFLOP/s", "cores": os.cpu_count() or 1, "kind": "port",
            "sample": "%d token rows of the same matrix, numpy f32 matmul of the f16-rounded operands (the arithmetic of kernels/matvec.cu mma_core)" % n}


def run_prefill_dense(args):
    if args.impl == "reference":
        import numpy as np
        sys.path.insert(0, ROOT)
        import __graft_entry__ as graft
        pkg = graft.load_package()
        wb = pkg.synth.quantize_q8_0(pkg.synth.normal((PD["rows"], PD["cols"]), 0.02, 1, "pd.w0")).numpy()
        c = cpu_prefill_dense(args.tokens, 10.0, wb)
        print(json.dumps({"impl": "reference", "metric": PD_METRIC, "value": c["value"], "unit": "TFLOP/s", "n_gpus": args.gpus, "steps": args.steps,
                          "warmup": args.warmup, "higher_is_better": True, "config": {"workload": "prefill-dense", **PD, "tokens": args.tokens},
                          "cpu_baseline": c, "e2e": {"value": c["value"], "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}))
        return
    if args.gpus != 1:
        raise SystemExit("the prefill-dense workload runs on one GPU")
    out = QuietStdout()
    import torch
    import __graft_entry__ as graft
    pkg = graft.load_package()
    torch.cuda.set_device(0)
    T, K, W = args.tokens, args.steps, max(args.warmup, 3)
    n_mat = 6                                                    # 6 x 26.7 MB of weights cycled: more than the 126 MB of L2
    mats = [pkg.synth.quantize_q8_0(pkg.synth.normal((PD["rows"], PD["cols"]), 0.02, 1, "pd.w%d" % i, device="cuda")) for i in range(n_mat)]
    ops = [pkg.mma_cols.MmaCols(wb, PD["rows"], PD["cols"], T) for wb in mats]
    x = pkg.synth.normal((T, PD["cols"]), 1.0, 2, "pd.x", device="cuda")
    y = torch.empty((T, PD["rows"]), dtype=torch.float32, device="cuda")
    xh = x.cpu().pin_memory()
    yh = torch.empty((T, PD["rows"]), dtype=torch.float32).pin_memory()
    for i in range(W):
        ops[i % n_mat](x, out=y)
    torch.cuda.synchronize()
    flops = 2.0 * T * PD["rows"] * PD["cols"]
    sampler = ClockSampler(0)
    sampler.start()
    ev = [torch.cuda.Event(enable_timing=True) for _ in range(2)]
    torch.cuda.synchronize()
    ev[0].record()
    for i in range(K):
        ops[i % n_mat](x, out=y)
    ev[1].record()
    torch.cuda.synchronize()
    dev_ms = ev[0].elapsed_time(ev[1])
    # the same through host buffers: the rows go up, the result comes back, every step
    t0 = time.perf_counter()
    for i in range(K):
        x.copy_(xh, non_blocking=True)
        ops[i % n_mat](x, out=y)
        yh.copy_(y, non_blocking=True)
        torch.cuda.synchronize()
    wall_s = time.perf_counter() - t0
    clocks = sampler.stop()
    for o in ops:
        assert o.status() == 0
    tf = flops * K / (dev_ms * 1e-3) / 1e12
    try:
        pk = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))
        peak, kind = float(pk["bf16_tflops"]), "measured"
    except Exception:
        peak, kind = 1590.0, "fallback"
    cpu = cpu_prefill_dense(T, args.cpu_seconds, mats[0].cpu().numpy()) if args.cpu_seconds > 0 else None
    line = {"metric": PD_METRIC, "value": tf, "unit": "TFLOP/s", "n_gpus": 1, "steps": K, "warmup": W, "ms_per_step": dev_ms / K, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "f16 operands (Q8_0 weights decoded d * q then rounded, inputs rounded), f32 accumulate in tensor memory",
            "data": "synthetic",
            "config": {"workload": "prefill-dense", **PD, "tokens": T, "weight_bytes": PD["rows"] * PD["cols"] // 32 * 34,
                       "l2": "inputs larger than L2: %d matrices of 26.7 MB cycled" % n_mat},
            "roofline": {"bound": "tensor", "achieved": tf, "peak": peak, "unit": "TFLOP/s", "frac": tf / peak, "peak_kind": kind, "traffic": None,
                         "kernel": "sz_mma_cols_q8_kernel (+ sz_x16_pack_kernel, in the same timed step)",
                         "hbm_side": {"bytes_per_step": PD["rows"] * PD["cols"] // 32 * 34 + T * PD["cols"] * 4 + T * PD["rows"] * 4,
                                      "gbs": (PD["rows"] * PD["cols"] // 32 * 34 + T * PD["cols"] * 4 + T * PD["rows"] * 4) * K / (dev_ms * 1e-3) / 1e9}},
            "cpu_baseline": cpu,
            "e2e": {"value": flops * K / wall_s / 1e12, "unit": "TFLOP/s", "h2d_bytes_per_step": T * PD["cols"] * 4, "d2h_bytes_per_step": T * PD["rows"] * 4},
            "gpu_launches": 2 * K, "clocks": clocks}
    out.emit(json.dumps(line))


# ---- workload c2-moe: the MoE sublayer microbench ---------------------------------------------------------------------------------
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


def run_reference_c2(args):
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
    ap.add_argument("--workload", default="c3", choices=["c3", "c2-moe", "c4-tree", "prefill-dense", "c5-concurrent", "c5-moe", "c5-batch"])
    ap.add_argument("--rows", type=int, default=256, help="c5-moe: rows a step (64 sequences x 4 rows)")
    ap.add_argument("--sequences", type=int, default=8, help="c5-concurrent: sequences decoded at once on every GPU")
    ap.add_argument("--waves", type=int, default=2, help="c5-concurrent: timed waves of requests (one request a sequence a wave)")
    ap.add_argument("--tokens", type=int, default=256, help="prefill-dense: token rows a step (256 = 64 sequences x K+1 = 4 rows)")
    ap.add_argument("--alpha", type=float, default=None,
                    help="c3: how strongly the synthetic model continues its token cycles (default: by kind of head, see C3_ALPHA_BY_HEAD)")
    ap.add_argument("--exchange", default="peer", choices=["peer", "nccl"],
                    help="c3, N > 1: the expert-parallel exchange - stores into the peers' memory from the combine kernel (default) or an NCCL all-reduce")
    ap.add_argument("--parallelism", default="replicas", choices=["ep", "replicas"],
                    help="c3, N > 1: every GPU with the whole 33 GB model and requests of its own, no exchange on the data path (default: "
                         "weak scaling, the throughput form), or experts sharded over the GPUs and ONE sequence (strong scaling: batch-1 "
                         "expert parallelism, which pays an exchange a layer and cannot scale)")
    ap.add_argument("--trace-rows", type=int, default=4, help="c3: rows of the pass whose launches are timed one by one (the line's `kernels`)")
    ap.add_argument("--contexts", default="", help="c5-batch: comma list of context lengths the sequences draw theirs from (config 5: 3000,9600,15000); default: all at --ctx")
    ap.add_argument("--feed", default="batch", choices=["batch", "alone"], help="c5-batch: the prompts in lockstep (sz_batch_prefill) or one session at a time")
    ap.add_argument("--profile-steps", type=int, default=0, help="c5-batch: only run this many batched steps (the last one between cudaProfilerStart/Stop), no timing")
    ap.add_argument("--profile-passes", type=int, default=0, help="c3: only run this many 4-row verify passes (for ncu), no timing")
    ap.add_argument("--head", default="proxy", choices=["q8", "exl3", "proxy"],
                    help="c3: output.weight as Q8_0 read in full, as 4-bit EXL3 read in full, or EXL3 screened by its 2-bit proxy (Q2_P)")
    ap.add_argument("--ctx", type=int, default=C3_CTX, help="c3: context length the decode runs at")
    ap.add_argument("--request-tokens", type=int, default=96, help="c3: tokens decoded after each request's 256-token prompt")
    ap.add_argument("--beta", type=float, default=None, help="c3: how strongly the synthetic model leans towards skipping a token of its cycle")
    ap.add_argument("--indexer", action="store_true",
                    help="c3: the model has the reference's sparse indexer (4 heads of 128, blocks of 4 positions, a budget of 2,048 positions); "
                         "BASELINE's configs describe a model without one, so this is off by default")
    ap.add_argument("--n-layer", type=int, default=C3["n_layer"], help="c3: layers (a smaller model for a quick check; not the benchmark)")
    ap.add_argument("--format", default="exl3", choices=["exl3", "iq3_s", "q8_0"])
    ap.add_argument("--also", default="iq3_s", help="comma list of further formats to time and report under 'also' ('' for none)")
    ap.add_argument("--layers", type=int, default=8)
    ap.add_argument("--reps", type=int, default=3, help="timed repetitions of the K-step region; the fastest is reported")
    ap.add_argument("--no-graph", action="store_true", help="launch eagerly instead of replaying a CUDA graph of the K steps")
    ap.add_argument("--cpu-seconds", type=float, default=12.0)
    args = ap.parse_args()
    if args.alpha is None:
        args.alpha = C3_ALPHA_BY_HEAD[args.head]
    if args.beta is None:
        args.beta = C3_BETA_BY_HEAD[args.head]
    if args.workload == "c4-tree":
        if args.impl == "reference":
            print(json.dumps({"impl": "reference", "unavailable": "the reference has no tree verification (its verify pass is a chain); the CPU restatement of a tree pass is a test oracle only"}))
            return
        return run_c4(args)
    if args.workload == "c3":
        return run_reference_c3(args) if args.impl == "reference" else run_c3(args)
    if args.workload == "prefill-dense":
        return run_prefill_dense(args)
    if args.workload == "c5-moe":
        if args.impl == "reference":
            return run_reference_c2(args)
        return run_c5_moe(args)
    if args.workload == "c5-batch":
        if args.impl == "reference":
            print(json.dumps({"impl": "reference", "unavailable": "the reference's CPU path serves one sequence at a time; see the c3 workload's reference arm for its tok/s"}))
            return
        return run_c5_batch(args)
    if args.workload == "c5-concurrent":
        if args.impl == "reference":
            print(json.dumps({"impl": "reference", "unavailable": "the reference's CPU path serves one sequence at a time; see the c3 workload's reference arm for its tok/s"}))
            return
        return run_c5(args)
    if args.impl == "reference":
        return run_reference_c2(args)

    out = QuietStdout()
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
        # (the trace name of whichever gate/up kernel ran: the streaming EXL3 kernel takes routed and shared experts in one launch,
        # the block-format kernels and the generic ones in one launch each; all launches of a step are added up with the bytes of both)
        names = ["gateup_exl3s", "gateup_exl3"] if r["fmt"] == "exl3" else ["gateup_blk", "gateup_rows"]
        name = next((n for n in names if n in r["kernels"]), names[0])
        ks = r["kernels"].get(name)
        bytes_pair = (r["distinct"] + 1) * r["expert_bytes"] * 2 / 3
        out = {"bound": "hbm", "peak": hbm, "unit": "GB/s", "peak_kind": peak_kind,
               "traffic": gateup_traffic(r["distinct"] + 1) if name == "gateup_exl3s" else None, "kernel": name}
        if ks:
            per_step = max(1, round(ks["launches"] / max(args.steps, 1)))
            dur_us = ks["avg_us"] * per_step
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
    out.emit(json.dumps(line))


if __name__ == "__main__":
    main()
