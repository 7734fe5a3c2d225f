"""Benchmark of the quantized GEMV / MoE decode hot path on N B200 GPUs of one node.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference] [--workload dense|gemv|moe|mul1|gemm] ...

Default workload (the headline): the NVFP4 dense decode layer stack (27B-shaped, 64 layers, M = 1). A step is one
token through the whole stack (4 GEMV launches per layer, one CUDA-graph replay). `value` = algorithmic bytes of a
step (every weight byte once + activations) / device time of a step, inputs resident in HBM; `e2e` = the same through
the host-facing call with pinned host buffers copied in and out every step. The same JSON line carries a `moe` block:
the routed-expert decode steps of the MoE configurations measured in the same process (on N > 1 GPUs expert-parallel,
all-to-all over peer memory), with both scaling definitions. One JSON line on stdout (rank 0).

Timing: W >= 3 warm-up steps, then blocks of K steps between two CUDA events (as many blocks as half a second needs);
ms_per_step is the median block, the spread is reported. Every multi-rank figure is the max over ranks.
"""
import argparse
import json
import math
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

METRIC = "nvfp4_gemv_hbm_gbs"
UNIT = "GB/s"
# DRAM bytes moved per algorithmic byte by the M = 1 kernel: dram__bytes_read.sum + dram__bytes_write.sum of one
# captured gate/up launch (100.3 MB read + 4.6 MB written = 104.9 MB) over its algorithmic bytes (100.3 MB); the capture is
# summarised in profiles/nvfp4_gemv_m1_kernel_gateup_17408x5120.md
TRAFFIC_RATIO = 1.046
MIN_TIMED_S = 0.5


def measured_peak(key="hbm_gbs", fallback=6650.0):
    try:
        return float(json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))[key]), "measured"
    except Exception:
        return fallback, "fallback"


class ClockSampler:
    """nvidia-smi clocks and throttle reasons sampled every 100 ms while the timed region runs."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index=0):
        self.rows, self.proc, self.index = [], None, index

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "100",
                                          "-i", str(self.index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.t = threading.Thread(target=self._read, daemon=True)
            self.t.start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([f.strip() for f in line.split(",")])

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.25)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        sm = sorted(float(r[1]) for r in self.rows if len(r) >= 9 and r[1].replace(".", "").isdigit())
        reasons = set()
        for r in self.rows:
            if len(r) >= 9:
                for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), r[5:9]):
                    if v.lower().startswith("active"):
                        reasons.add(name)
        mx = [float(r[2]) for r in self.rows if len(r) >= 9 and r[2].replace(".", "").isdigit()]
        # under load: the upper half of the samples (the sampler also sees the idle gaps between the parts of the run)
        load = sm[len(sm) // 2:]
        return {"sm_mhz": load[len(load) // 2] if load else None, "sm_max_mhz": mx[0] if mx else None, "reasons": sorted(reasons),
                "samples": len(sm)}


class Timer:
    """Blocks of `steps` steps between two CUDA events on the current stream, repeated until MIN_TIMED_S is covered
    (at most 50 blocks); barrier + synchronize on both sides of the whole region; max over ranks per block."""

    def __init__(self, world):
        self.world = world

    def barrier(self):
        import torch
        torch.cuda.synchronize()
        if self.world > 1:
            import torch.distributed as dist
            dist.barrier()
            torch.cuda.synchronize()

    def run(self, step, steps, warmup):
        import torch
        self.barrier()  # the ranks start their first step together (set-up times differ, device-side waits are bounded)
        for _ in range(warmup):
            step()
        self.barrier()
        # one probe block sizes the repeat count
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            step()
        e1.record()
        self.barrier()
        probe = max(e0.elapsed_time(e1) * 1e-3, 1e-6)
        blocks = max(1, min(50, int(math.ceil(MIN_TIMED_S / probe))))
        if self.world > 1:
            import torch.distributed as dist
            t = torch.tensor([blocks], device="cuda")
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            blocks = int(t.item())
        ev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(blocks)]
        self.barrier()
        for a, b in ev:
            a.record()
            for _ in range(steps):
                step()
            b.record()
        self.barrier()
        ms = torch.tensor([a.elapsed_time(b) for a, b in ev], dtype=torch.float64, device="cuda")
        if self.world > 1:
            import torch.distributed as dist
            dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        ms = sorted(ms.tolist())
        return {"ms_per_step": ms[len(ms) // 2] / steps, "blocks": blocks, "ms_per_step_min": ms[0] / steps, "ms_per_step_max": ms[-1] / steps}

    def wall(self, step, steps):
        """End-to-end: wall clock over `steps` host-facing calls (each synchronises), max over ranks."""
        import torch
        for _ in range(2):
            step()
        self.barrier()
        t0 = time.perf_counter()
        for _ in range(steps):
            step()
        self.barrier()
        s = time.perf_counter() - t0
        if self.world > 1:
            import torch.distributed as dist
            t = torch.tensor([s], dtype=torch.float64, device="cuda")
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            s = float(t.item())
        return s / steps


# ---------------------------------------------------------------------------------------------- CPU baselines
def _median_calls(fn, budget_s, min_calls=24, max_calls=200):
    """median seconds of `fn(i)` over at least `min_calls` calls (more while the budget lasts)"""
    fn(0)  # page faults, worker start
    ts, t_all = [], 0.0
    i = 0
    while i < max_calls and (i < min_calls or t_all < budget_s):
        t0 = time.perf_counter()
        fn(i)
        dt = time.perf_counter() - t0
        ts.append(dt)
        t_all += dt
        i += 1
        if t_all > 3 * budget_s and i >= 3:
            break
    ts.sort()
    return ts[len(ts) // 2], len(ts)


def cpu_dense_baseline(host_layers, m, budget_s=10.0):
    """The CPU checker's NVFP4 GEMV (AVX2 arm of the reference's operation order, rows split over the threads, parked
    worker pool) over whole layers, rotating over distinct layers (each 186 MB, beyond any L3): thread counts 1 / 8 /
    all, median of >= 24 layer passes each where the budget allows - the reference's own method
    (engine/src/cpu_nvfp4.rs:729-777)."""
    import numpy as np
    import oracle
    rng = np.random.default_rng(0)
    xs = {}
    for mats in host_layers:
        for _, (_, _, k) in mats.items():
            xs.setdefault(k, rng.standard_normal((m, k)).astype(np.float32))
    path = 1 if oracle.lib().cn_o_have_avx2() else 0
    layer_bytes = sum(w.size for w, _, _ in host_layers[0].values())
    cores = os.cpu_count() or 1
    sweep = {}
    for threads in sorted({1, min(8, cores), cores}):
        def one(i, threads=threads):
            for _, (w, rows, k) in host_layers[i % len(host_layers)].items():
                oracle.nvfp4_gemv(w, rows, k, 1.0, xs[k], threads=threads, path=path)
        share = budget_s * (0.5 if threads == cores else 0.25)
        med, calls = _median_calls(one, share, min_calls=24 if threads > 1 else 4)
        sweep[str(threads)] = {"gbs": layer_bytes / med / 1e9, "calls": calls}
    return {"value": sweep[str(cores)]["gbs"], "unit": UNIT, "cores": cores, "kind": "port",
            "sample": f"median of {sweep[str(cores)]['calls']} passes over one whole layer ({layer_bytes} B: qkv, o, gate, up, down), "
                      f"{len(host_layers)} distinct layers rotated, AVX2 arm, parked worker pool",
            "threads_sweep": sweep}


def cpu_moe_baseline(kind, wl, budget_s=6.0):
    """The routed-expert step on the host cores: every (token, expert) combo of rank 0's batch through the CPU
    checker's expert FFN (cn_o_nvfp4_ffn / cn_o_mul1_expert_ffn), all threads inside each FFN, median of the passes."""
    import numpy as np
    import oracle
    import torch
    from crownest_b200 import moe
    cores = os.cpu_count() or 1
    ids, _ = moe.route_softmax_topk(wl.logits, wl.topk)
    ids = ids.cpu().numpy().reshape(-1)
    x = wl.x.float().cpu().numpy()
    picked = sorted(set(int(e) for e in ids))
    if kind == "moe":
        rb = wl.hidden // 64 * 36
        gu = {e: wl.w.keep[0][e].cpu().numpy() for e in picked}
        dn = {e: wl.w.keep[3][e].cpu().numpy() for e in picked}
        sh = [t.cpu().numpy() for t in wl.w.shared]

        def one(_):
            for c, e in enumerate(ids):
                oracle.nvfp4_ffn(gu[e][: wl.inter * rb], gu[e][wl.inter * rb:], dn[e], wl.hidden, wl.inter, [1.0, 1.0, 1.0],
                                 x[c // wl.topk: c // wl.topk + 1], threads=cores, path=1)
            oracle.nvfp4_ffn(sh[0], sh[1], sh[2], wl.hidden, wl.shared_inter, [1.0, 1.0, 1.0], x, threads=cores, path=1)
    else:
        recs = {e: wl.recs[e].cpu().numpy() for e in picked}

        def one(_):
            for c, e in enumerate(ids):
                oracle.mul1_expert_ffn(recs[e], wl.hidden, wl.inter, wl.K, x[c // wl.topk: c // wl.topk + 1], limit=10.0, threads=cores)
    med, calls = _median_calls(one, budget_s, min_calls=3, max_calls=24)
    return {"value": wl.tokens / med, "unit": "tok/s", "cores": cores, "kind": "port",
            "sample": f"median of {calls} passes over the step's {len(ids)} (token, expert) FFNs ({len(picked)} distinct experts), all threads per FFN"}


# ---------------------------------------------------------------------------------------------- reference arm
def reference_arm(args, rank):
    """`--impl reference`: the reference's CPU implementation of the path (its Rust source cannot be built here - no
    Rust toolchain - so the C port under oracle/ stands in, kind "port"), all host threads, each step one layer of the
    stack's shapes (186 MB of NVFP4)."""
    if rank != 0:
        return
    import numpy as np
    from crownest_b200 import synth
    threads = os.cpu_count() or 1
    rng = np.random.default_rng(0)
    layers = [{n: (synth.nvfp4_matrix(r, k, rng), r, k) for n, r, k in synth.dense_layer_shapes()} for _ in range(2)]
    import oracle
    path = 1 if oracle.lib().cn_o_have_avx2() else 0
    xs = {k: rng.standard_normal((args.m, k)).astype(np.float32) for _, _, k in synth.dense_layer_shapes()}
    for s in range(max(1, args.warmup)):
        for name, (w, rows, k) in layers[s % len(layers)].items():
            oracle.nvfp4_gemv(w, rows, k, 1.0, xs[k], threads=threads, path=path)
    t0 = time.perf_counter()
    for s in range(args.steps):
        for name, (w, rows, k) in layers[s % len(layers)].items():
            oracle.nvfp4_gemv(w, rows, k, 1.0, xs[k], threads=threads, path=path)
    dt = time.perf_counter() - t0
    gbs = synth.dense_layer_bytes() * args.steps / dt / 1e9
    sample = f"{args.steps} steps, each one layer of the stack (qkv, o, gate, up, down = {synth.dense_layer_bytes()} B), 2 distinct layers rotated"
    line = {"impl": "reference", "metric": METRIC, "value": gbs, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": dt / args.steps * 1e3, "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": "nvfp4 dense decode stack 27B-shaped, M=%d (CPU: one layer per step)" % args.m},
            "cpu_baseline": {"value": gbs, "unit": UNIT, "cores": threads, "kind": "port", "sample": sample},
            "e2e": {"value": gbs, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line), flush=True)


# ---------------------------------------------------------------------------------------------- MoE parts
MOE_SHAPES = {"moe": "hidden 2048, 512 experts, inter 512, shared expert 512, softmax top-10, NVFP4",
              "mul1": "hidden 4096, 64 experts, inter 1536, top-4, EXL3 MUL1 K=3"}


def moe_measure(kind, tokens, rank, world, local, steps, warmup, cpu=False, e2e=True):
    """One routed-expert decode configuration: `tokens` rows per rank, experts spread over the ranks (all-to-all dispatch
    and return over peer memory when world > 1). Returns the figures of one block of the JSON line (rank 0) or None."""
    import torch
    import torch.distributed as dist
    from crownest_b200 import _lib, moe, workloads
    cls = workloads.MoeDecode if kind == "moe" else workloads.Mul1MoeDecode
    wl = cls(tokens, device=f"cuda:{local}", rank=rank, world=world, group=None)
    x_host = wl.x.cpu().pin_memory()
    y_host = torch.empty_like(x_host).pin_memory()
    st = torch.cuda.Stream()
    with torch.cuda.stream(st):
        wl.step()
        st.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=st):
            wl.step()
    torch.cuda.synchronize()
    tm = Timer(world)
    t = tm.run(graph.replay, steps, warmup)

    def host_step():
        wl.x.copy_(x_host, non_blocking=True)
        graph.replay()
        y_host.copy_(wl.y, non_blocking=True)
        torch.cuda.current_stream().synchronize()

    e2e_s = tm.wall(host_step, steps) if e2e else None
    # algorithmic bytes of the whole job: every distinct routed expert once (an expert lives on one rank), the shared
    # expert once per rank, activations in and out
    ids, _ = moe.route_softmax_topk(wl.logits, wl.topk)
    distinct = torch.tensor([float(torch.unique(ids).numel())], device="cuda")
    if world > 1:
        allids = [torch.empty_like(ids) for _ in range(world)]
        dist.all_gather(allids, ids)
        distinct = torch.tensor([float(torch.unique(torch.cat(allids)).numel())], device="cuda")
    distinct = int(distinct.item())
    if kind == "moe":
        per_expert = 3 * wl.inter * wl.hidden // 64 * 36
        nbytes = distinct * per_expert + world * (3 * wl.shared_inter * wl.hidden // 64 * 36) + tokens * world * (2 * wl.hidden * 2 + wl.experts * 4)
    else:
        from crownest_b200 import mul1
        nbytes = distinct * mul1.record_bytes(wl.hidden, wl.inter, wl.K) + tokens * world * (2 * wl.hidden * 2 + wl.experts * 4)
    status = _lib.device_status()
    out = None
    if rank == 0:
        peak, peak_kind = measured_peak()
        ms = t["ms_per_step"]
        gbs = nbytes / (ms * 1e-3) / 1e9
        out = {"workload": f"routed-expert decode step ({MOE_SHAPES[kind]})", "tokens_per_rank": tokens, "global_batch": tokens * world,
               "tok_s": tokens * world / (ms * 1e-3), "ms_per_step": ms, "blocks": t["blocks"], "ms_per_step_min": t["ms_per_step_min"],
               "ms_per_step_max": t["ms_per_step_max"], "distinct_experts": distinct, "algorithmic_bytes": nbytes,
               "roofline": {"bound": "hbm", "achieved": gbs / world, "peak": peak, "unit": "GB/s", "frac": gbs / world / peak, "peak_kind": peak_kind,
                            "scope": "per GPU", "kernel": "nvfp4_gemv_m1_kernel (routed form)" if kind == "moe" else "mul1_gemv_kernel"},
               "parallelism": f"ep{world}: all-to-all dispatch / return over peer memory" if world > 1 else "none",
               "launches_per_step": wl.launches_per_step, "device_status": status}
        if e2e_s is not None:
            out["e2e_tok_s"] = tokens * world / e2e_s
            out["h2d_bytes_per_step"] = x_host.numel() * 2
            out["d2h_bytes_per_step"] = y_host.numel() * 2
        if cpu and world == 1:
            out["cpu_baseline"] = cpu_moe_baseline(kind, wl)
    del graph, wl
    torch.cuda.empty_cache()
    return out


def moe_block(rank, world, local, steps, warmup, cpu):
    """The MoE figures that ride on the default line. Weak scaling: 64 (NVFP4) / 16 (MUL1) tokens per rank, the global
    batch grows with the ranks. Strong scaling: a global batch of 64 split over the ranks."""
    block = {"scaling_definitions": {"weak": "fixed tokens per rank; tok/s over the global batch", "strong": "global batch 64 split over the ranks"}}
    block["nvfp4_weak_64_per_rank"] = moe_measure("moe", 64, rank, world, local, steps, warmup, cpu=cpu)
    if world > 1:
        block["nvfp4_strong_global_64"] = moe_measure("moe", max(1, 64 // world), rank, world, local, steps, warmup, e2e=False)
    block["mul1_weak_16_per_rank"] = moe_measure("mul1", 16, rank, world, local, steps, warmup, cpu=cpu)
    return block


def moe_arm(args, rank, world, local):
    """`--workload moe` / `mul1`: one routed-expert configuration as the line's own metric, `--tokens` rows per rank."""
    out = moe_measure(args.workload, args.tokens, rank, world, local, args.steps, args.warmup, cpu=not args.no_cpu_baseline)
    if rank == 0:
        line = {"metric": "moe_decode_tok_s", "value": out["tok_s"], "unit": "tok/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
                "ms_per_step": out["ms_per_step"], "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
                "config": {"workload": f"{out['workload']}, {args.tokens} tokens per rank", "parallelism": out["parallelism"],
                           "l2": "the expert set changes with the routing; the weights of one step (%.0f MB) are larger than L2 from 64 tokens on" % (out["algorithmic_bytes"] / 1e6),
                           "launch": "CUDA graph replay", "distinct_experts": out["distinct_experts"]},
                "roofline": dict(out["roofline"], traffic=None), "blocks": out["blocks"],
                "e2e": {"value": out.get("e2e_tok_s"), "unit": "tok/s", "h2d_bytes_per_step": out.get("h2d_bytes_per_step"), "d2h_bytes_per_step": out.get("d2h_bytes_per_step")},
                "gpu_launches": args.steps * out["blocks"] * out["launches_per_step"], "device_status": out["device_status"]}
        if "cpu_baseline" in out:
            line["cpu_baseline"] = out["cpu_baseline"]
        print(json.dumps(line), flush=True)
    leave(world)


# ---------------------------------------------------------------------------------------------- single GEMV
def gemv_arm(args, rank, world, local):
    """`--workload gemv`: one NVFP4 GEMV shape (default: the single 4096 x 4096 matrix at M = 1) the reference's way
    (engine/src/glm5_model.rs:2414-2432): distinct weight copies of at least 512 MiB in all rotated launch by launch, so
    that nothing is served from L2, and at least 64 launches per graph replay between the two events."""
    import numpy as np
    import torch
    from crownest_b200 import _lib, dense, ops, synth
    torch.cuda.set_device(local)
    dev = f"cuda:{local}"
    rows, k, m = args.rows, args.cols, args.m
    nb = rows * k // 64 * 36
    copies = max(2, int(math.ceil(512 * 2 ** 20 / nb)))
    per_graph = max(64, copies)
    gen = torch.Generator(device=dev)
    gen.manual_seed(0)
    one = torch.ones(1, device=dev)
    op = args.op
    if op == "fp8":
        nb = rows * k
        copies = max(2, int(math.ceil(512 * 2 ** 20 / nb)))
        per_graph = max(64, copies)
        ws = [torch.randint(0, 120, (rows * k,), dtype=torch.uint8, device=dev, generator=gen) for _ in range(copies)]
        sc = torch.rand(((rows + 127) // 128) * ((k + 127) // 128), device=dev, generator=gen) * 0.01 + 0.005
        launch = lambda w, xx, yy: ops.fp8_gemv(w, sc, xx, rows, k, yy)
    elif op == "gu":  # fused gate/up: `rows` outputs from two [rows][k] matrices
        nb *= 2
        copies = max(2, int(math.ceil(512 * 2 ** 20 / nb)))
        per_graph = max(64, copies)
        ws = [(ops.Fp4(dense._rand_nvfp4_device(rows, k, gen, dev), one, rows, k), ops.Fp4(dense._rand_nvfp4_device(rows, k, gen, dev), one, rows, k))
              for _ in range(copies)]
        launch = lambda w, xx, yy: ops.launch_gemv_gu(w[0], w[1], xx, yy)
    else:
        ws = [ops.Fp4(dense._rand_nvfp4_device(rows, k, gen, dev), one, rows, k) for _ in range(copies)]
        launch = lambda w, xx, yy: ops.launch_gemv(w, xx, yy)
    x_host = torch.randn((m, k), generator=torch.Generator().manual_seed(1)).to(torch.bfloat16).pin_memory()
    x = x_host.to(dev)
    y = torch.empty((m, rows), dtype=torch.bfloat16, device=dev)
    y_host = torch.empty((m, rows), dtype=torch.bfloat16).pin_memory()
    st = torch.cuda.Stream()
    with torch.cuda.stream(st):
        launch(ws[0], x, y)
        st.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=st):
            for i in range(per_graph):
                launch(ws[i % copies], x, y)
    tm = Timer(1)
    sampler = ClockSampler(local)
    sampler.start()
    t = tm.run(graph.replay, args.steps, args.warmup)
    i = [0]

    def host_step():
        x.copy_(x_host, non_blocking=True)
        launch(ws[i[0] % copies], x, y)
        i[0] += 1
        y_host.copy_(y, non_blocking=True)
        torch.cuda.current_stream().synchronize()

    e2e_s = tm.wall(host_step, max(args.steps, 50))
    clocks = sampler.stop()
    bytes_launch = nb + 4 + m * (k + rows) * 2
    us = t["ms_per_step"] * 1e3 / per_graph
    gbs = bytes_launch / us / 1e3
    peak, peak_kind = measured_peak()
    line = {"metric": METRIC, "value": gbs, "unit": UNIT, "n_gpus": 1, "steps": args.steps, "warmup": args.warmup, "ms_per_step": t["ms_per_step"],
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": f"single {'FP8' if op == 'fp8' else 'NVFP4'} {'fused gate/up ' if op == 'gu' else ''}GEMV [{rows} x {k}], M={m}; a step = {per_graph} launches",
                       "activations": "bf16 in/out, f32 accumulate",
                       "l2": f"{copies} distinct weight copies ({copies * nb / 2 ** 20:.0f} MiB) rotated launch by launch: larger than L2",
                       "launch": f"CUDA graph replay of {per_graph} launches"},
            "roofline": {"bound": "hbm", "achieved": gbs, "peak": peak, "unit": "GB/s", "frac": gbs / peak, "traffic": None, "peak_kind": peak_kind,
                         "kernel": "fp8_gemv_tc_kernel" if op == "fp8" else "nvfp4_gemv_m1_kernel", "bytes_per_launch": bytes_launch, "us_per_launch": us},
            "blocks": t["blocks"], "ms_per_step_min": t["ms_per_step_min"], "ms_per_step_max": t["ms_per_step_max"],
            "e2e": {"value": bytes_launch / e2e_s / 1e9, "unit": UNIT, "h2d_bytes_per_step": x_host.numel() * 2, "d2h_bytes_per_step": y_host.numel() * 2,
                    "note": "one launch per host call"},
            "gpu_launches": args.steps * t["blocks"] * per_graph, "clocks": clocks, "device_status": _lib.device_status()}
    if not args.no_cpu_baseline and op == "gemv":
        import oracle
        cores = os.cpu_count() or 1
        hw = [w.w.cpu().numpy() for w in ws[:min(copies, 24)]]
        xf = x_host.float().numpy()
        sweep = {}
        for threads in sorted({1, min(8, cores), cores}):
            med, calls = _median_calls(lambda j: oracle.nvfp4_gemv(hw[j % len(hw)], rows, k, 1.0, xf, threads=threads, path=1), 3.0)
            sweep[str(threads)] = {"gbs": nb / med / 1e9, "calls": calls}
        line["cpu_baseline"] = {"value": sweep[str(cores)]["gbs"], "unit": UNIT, "cores": cores, "kind": "port",
                                "sample": f"median of {sweep[str(cores)]['calls']} calls rotating over {len(hw)} weight copies ({len(hw) * nb / 2 ** 20:.0f} MiB)",
                                "threads_sweep": sweep}
    print(json.dumps(line), flush=True)


# ---------------------------------------------------------------------------------------------- interval table
def intervals_arm(args, rank=0, world=1, local=0):
    """`--workload intervals`: where the time of a projection goes inside the dense stack. Needs the diagnostic build of the
    library (`make -C crow-nest_b200/csrc trace`), whose one-row GEMV kernel stamps %globaltimer per CTA at entry, after the
    wait on the predecessor grid, after the activations are staged, when its first stage has landed, at its end, and in the
    producer warp at its first and after its last bulk copy; under torchrun the exchange kernel of the tensor-parallel stack
    stamps its own steps too. Prints markdown tables (ns after the previous launch's last CTA ended; medians over the CTAs
    of a launch, mean over the last layers) and one JSON line with the same figures."""
    import numpy as np
    import torch
    import torch.distributed as dist
    from crownest_b200 import _lib
    _lib.use_trace_library()
    from crownest_b200 import dense
    torch.cuda.set_device(local)
    group = None
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
        group = dist.group.WORLD
    layers = max(3, min(args.layers, 8))
    st = dense.DenseStack(layers=layers, seed=0, device=f"cuda:{local}", rank=rank, world=world, group=group,
                          exchange=args.exchange if args.exchange != "nccl" else "peer",
                          gather_q=True)  # all four vectors exchanged: one exchange kernel per projection in the tables
    if world > 1 and st.peer is None:
        raise SystemExit("intervals: the peer-memory exchange is not available between these GPUs")
    st.x.copy_(torch.randn((1, st.hidden), device=f"cuda:{local}").to(torch.bfloat16))
    n = 4 * layers
    tr = torch.zeros((n, 512, 8), dtype=torch.int64, device=f"cuda:{local}")
    tx = torch.zeros((n, 8), dtype=torch.int64, device=f"cuda:{local}")
    s = torch.cuda.Stream()
    with torch.cuda.stream(s):
        for _ in range(3):
            st.run_layers(1)
        s.synchronize()
        # the launches captured next keep their slot of the buffers in the graph
        _lib.lib().cn_m1_trace(tr.data_ptr(), n)
        _lib.lib().cn_tp_trace(tx.data_ptr(), n)
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=s):
            st.run_layers(1)
    for _ in range(3):
        g.replay()
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    tr.zero_()
    tx.zero_()
    g.replay()
    torch.cuda.synchronize()
    t = tr.cpu().numpy().astype(np.float64)
    x = tx.cpu().numpy().astype(np.float64)
    shapes = [("qkv", 7168, 5120), ("o", 5120, 5120), ("gate/up", 2 * 17408, 5120), ("down", 5120, 17408)]
    names = [f"{nm} {r // world}x{k}" for nm, r, k in shapes]
    cols = ["ctas", "entry", "predecessor_wait_over", "activations_staged", "first_stage_landed", "first_cta_ends", "median_cta_ends", "last_cta_ends",
            "first_bulk_copy", "last_bulk_copy_median", "last_bulk_copy_max"]
    xcols = ["entry", "predecessor_wait_over", "slice_stores_issued", "flag_stored", "peer_flag_seen", "all_flags_seen", "next_gemv_wait_over"]
    rows = {nm: [] for nm in names}
    xrows = {nm: [] for nm in names}
    prev_end = None
    for i in range(n):
        a = t[i][t[i][:, 0] > 0]
        end = a[:, 4].max()
        if prev_end is not None and i >= 8:
            pr = a[a[:, 5] > 0]
            rel = lambda c: float(np.median(a[:, c] - prev_end))
            rows[names[i % 4]].append([len(a), rel(0), rel(1), rel(2), rel(3), a[:, 4].min() - prev_end, rel(4), end - prev_end,
                                       float(np.median(pr[:, 5] - prev_end)), float(np.median(pr[:, 6] - prev_end)), float(np.max(pr[:, 6] - prev_end))])
        if world > 1 and i >= 8 and i + 1 < n:
            # the exchange that follows launch i, against the end of launch i's last CTA; then the next launch's wait
            nxt = t[i + 1][t[i + 1][:, 0] > 0]
            xrows[names[i % 4]].append([x[i][c] - end for c in range(6)] + [float(np.median(nxt[:, 1])) - end])
        prev_end = end if world == 1 else (x[i][5] if x[i][5] > 0 else end)
    out = {"gemv": {}, "exchange": {}}
    if rank == 0:
        print("| projection | " + " | ".join(cols) + " |")
        print("|---|" + "---|" * len(cols))
        for nm in names:
            v = np.mean(np.array(rows[nm]), axis=0)
            out["gemv"][nm] = {c: float(q) for c, q in zip(cols, v)}
            print(f"| {nm} | " + " | ".join(f"{q:.0f}" for q in v) + " |")
        if world > 1:
            print()
            print("| exchange after | " + " | ".join(xcols) + " |")
            print("|---|" + "---|" * len(xcols))
            for nm in names:
                v = np.mean(np.array(xrows[nm]), axis=0)
                out["exchange"][nm] = {c: float(q) for c, q in zip(xcols, v)}
                print(f"| {nm} | " + " | ".join(f"{q:.0f}" for q in v) + " |")
        print(json.dumps({"metric": "m1_gemv_intervals_ns", "n_gpus": world, "layers": layers,
                          "unit": "ns after the previous launch's last CTA ended (N > 1: after the previous exchange ended; exchange table: after the GEMV's last CTA ended)",
                          "intervals": out, "device_status": _lib.device_status()}), flush=True)
    if world > 1:
        leave(world, st)


# ---------------------------------------------------------------------------------------------- batched GEMM
def gemm_arm(args, rank, world, local):
    """`--workload gemm`: the batched NVFP4 GEMM (W [17408 x 5120] then [5120 x 17408], --m rows), output columns split over
    the ranks with an all-gather (tensor parallel). A step = both GEMMs once."""
    import torch
    import torch.distributed as dist
    from crownest_b200 import _lib, dense, ops
    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    _lib.lib()
    dev = f"cuda:{local}"
    m, hidden, inter = args.m, 5120, 17408
    gen = torch.Generator(device=dev)
    one = torch.ones(1, device=dev)
    ncopy = 3  # distinct weight copies rotated step by step: 3 x 100 MB per rank, beyond L2 together with the activations
    ups, downs = [], []
    for c in range(ncopy):
        gen.manual_seed(100 * c + rank)
        ups.append(ops.Fp4(dense._rand_nvfp4_device(inter // world, hidden, gen, dev), one, inter // world, hidden))
        downs.append(ops.Fp4(dense._rand_nvfp4_device(hidden // world, inter, gen, dev), one, hidden // world, inter))
    x_host = torch.randn((m, hidden), generator=torch.Generator().manual_seed(7)).to(torch.bfloat16).pin_memory()
    x = x_host.to(dev)
    h = torch.empty((m, inter), dtype=torch.bfloat16, device=dev)
    y = torch.empty((m, hidden), dtype=torch.bfloat16, device=dev)
    hp = torch.empty((m, inter // world), dtype=torch.bfloat16, device=dev) if world > 1 else h
    yp = torch.empty((m, hidden // world), dtype=torch.bfloat16, device=dev) if world > 1 else y
    y_host = torch.empty((m, hidden), dtype=torch.bfloat16).pin_memory()
    # engine: the block-scaled FP4 MMA (kind::mxf4nvf4 + five-level activation cascade) up to 128 rows, where one pass over
    # the weights serves every token; beyond that its operand traffic (five cascade columns per token) binds on L2 and the f16
    # MMA on losslessly widened weights is faster (both are tcgen05)
    fp4 = args.engine == "fp4" or (args.engine == "auto" and m <= 128)
    raw_rows = ups[0].w[: 1024 * (hidden // 64 * 36)].cpu().numpy() if world == 1 and not args.no_cpu_baseline else None
    if fp4:
        ups, downs = [ops.Fp4Packed(w) for w in ups], [ops.Fp4Packed(w) for w in downs]
        nws = max(int(_lib.lib().cn_nvfp4_bs_workspace_bytes(inter // world, hidden, m)), int(_lib.lib().cn_nvfp4_bs_workspace_bytes(hidden // world, inter, m)))
        ws = torch.empty(nws, dtype=torch.uint8, device=dev)
        gemm = ops.launch_gemm_fp4
    else:
        ws = torch.empty(ops.gemm_workspace_bytes(inter, m), dtype=torch.uint8, device=dev)
        gemm = ops.launch_gemm
    it = [0]

    def step():
        i = it[0]
        it[0] += 1
        gemm(ups[i % ncopy], x, hp, workspace=ws)
        if world > 1:
            dense.gather_rows(hp, h, m, world)
        gemm(downs[i % ncopy], h, yp, workspace=ws)
        if world > 1:
            dense.gather_rows(yp, y, m, world)

    def host_step():
        x.copy_(x_host, non_blocking=True)
        step()
        y_host.copy_(y, non_blocking=True)
        torch.cuda.current_stream().synchronize()

    tm = Timer(world)
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    t = tm.run(step, args.steps, args.warmup)
    e2e_s = tm.wall(host_step, args.steps)
    clocks = sampler.stop() if rank == 0 else None
    if rank == 0:
        flops = 2.0 * m * hidden * inter * 2
        ms_step = t["ms_per_step"]
        tf = flops / (ms_step * 1e-3) / 1e12
        peak, kind = measured_peak("bf16_tflops", 1590.0)
        line = {"metric": "nvfp4_gemm_tflops", "value": tf, "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
                "ms_per_step": ms_step, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
                "dtype": "e2m1 x e2m1 block-scaled -> f32" if fp4 else "f16 x f16 -> f32", "data": "synthetic",
                "config": {"workload": f"nvfp4 GEMM pair [17408 x 5120] and [5120 x 17408], M={m}", "parallelism": f"tp{world} column split + all-gather" if world > 1 else "none",
                           "l2": "three weight copies rotated (300 MB per rank) plus the activations: larger than L2", "launch": "plain launches"},
                "roofline": {"bound": "tensor", "achieved": tf / world, "peak": peak, "unit": "TFLOP/s", "frac": tf / world / peak, "traffic": None,
                             "peak_kind": kind + " (bf16 GEMM, burst)", "scope": "per GPU",
                             "kernel": "nvfp4_gemm_bs_kernel (tcgen05 kind::mxf4nvf4)" if fp4 else "nvfp4_gemm_tc5_kernel (tcgen05 kind::f16)", "flops_per_launch": flops / 2 / world, "us_per_launch": ms_step * 1e3 / 2,
                             "hbm_gbs": (2 * hidden * inter // 64 * 36 / world + 2.0 * m * (hidden + inter) * 2) / (ms_step * 1e-3) / 1e9},
                "blocks": t["blocks"], "ms_per_step_min": t["ms_per_step_min"], "ms_per_step_max": t["ms_per_step_max"],
                "e2e": {"value": flops / e2e_s / 1e12, "unit": "TFLOP/s", "h2d_bytes_per_step": x_host.numel() * 2, "d2h_bytes_per_step": y_host.numel() * 2},
                "gpu_launches": args.steps * t["blocks"] * 4, "clocks": clocks, "device_status": _lib.device_status()}
        if world == 1 and not args.no_cpu_baseline:
            import numpy as np
            import oracle
            cores = os.cpu_count() or 1
            rows_s, toks = 1024, min(m, 8)  # a bounded sample: 1024 output rows of the first matrix for 8 tokens
            wsub = raw_rows
            xf = x_host[:toks].float().numpy()
            med, calls = _median_calls(lambda j: oracle.nvfp4_gemv(wsub, rows_s, hidden, 1.0, xf, threads=cores, path=1), 3.0)
            line["cpu_baseline"] = {"value": 2.0 * toks * rows_s * hidden / med / 1e12, "unit": "TFLOP/s", "cores": cores, "kind": "port",
                                    "sample": f"median of {calls} calls of the CPU GEMV over {rows_s} rows of W [17408 x 5120] for {toks} tokens (its token tile)"}
        print(json.dumps(line), flush=True)
    leave(world)


def leave(world, *holders):
    """End of a multi-rank run. A captured graph that holds NCCL kernels keeps the communicator busy:
    destroy_process_group() then waits for ever, so the ranks meet once more and exit without tearing it down."""
    if world <= 1:
        return
    import torch
    import torch.distributed as dist
    torch.cuda.synchronize()
    dist.barrier()
    torch.cuda.synchronize()
    sys.stdout.flush()
    sys.stderr.flush()
    os._exit(0)


def exchange_check(rank, world, local):
    """N >= 2: the peer-memory exchange of the tensor-parallel stack against the NCCL all-gather path on a three-layer
    stack (same weights, same input): every replicated vector must agree bit for bit, replay after replay."""
    import torch
    import torch.distributed as dist
    from crownest_b200 import _lib, dense
    res = "ok"
    try:
        a = dense.DenseStack(layers=3, device=f"cuda:{local}", seed=5, rank=rank, world=world, exchange="nccl")
        b = dense.DenseStack(layers=3, device=f"cuda:{local}", seed=5, rank=rank, world=world, exchange="peer")
        if b.peer is None:
            res = "peer exchange unavailable: " + getattr(b, "peer_error", "?")
        else:
            x = torch.randn((1, a.hidden), generator=torch.Generator().manual_seed(1)).to(torch.bfloat16).cuda()
            a.x.copy_(x), b.x.copy_(x)
            a.run_layers(1)
            b.capture(1)
            for it in range(2):
                b.graph.replay()
                torch.cuda.synchronize()
                for name in ("q", "o", "h", "y"):
                    va, vb = getattr(a, name), getattr(b, name)
                    if name in a.local_only:  # not exchanged: every rank holds its own slice only
                        lo, hi = dense.tp_rows(va.shape[1], rank, world)
                        va, vb = va[:, lo:hi].contiguous(), vb[:, lo:hi].contiguous()
                    if not torch.equal(va.view(torch.int16), vb.view(torch.int16)):
                        res = f"replay {it}: vector {name} differs from the all-gather path"
                dist.barrier()  # nobody starts the next replay (and overwrites its slices in the peers' copies) before all have looked
            if _lib.device_status() != 0:
                res = "device status"
    except Exception as e:  # noqa: BLE001 - reported in the line
        res = f"{type(e).__name__}: {e}"
    flag = torch.tensor([0 if res == "ok" else 1], device="cuda")
    dist.all_reduce(flag)
    torch.cuda.synchronize()
    return res if int(flag.item()) == 0 or res != "ok" else "a peer rank reported a mismatch"


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=100)
    ap.add_argument("--warmup", type=int, default=5)
    # "--act-rows": the spelling to use under torch.distributed.run, whose own parser takes "--m" for an abbreviation
    ap.add_argument("--m", "--act-rows", dest="m", type=int, default=1, help="activation rows per step (1 decode, 4 = MTP verify)")
    ap.add_argument("--layers", type=int, default=64)
    ap.add_argument("--impl", default="crownest")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--min-time", type=float, default=MIN_TIMED_S,
                    help="seconds of device time the timed blocks cover (0 = one block: for a profiler capture of a few launches)")
    ap.add_argument("--no-moe", action="store_true", help="dense workload: leave the MoE block out of the line")
    ap.add_argument("--exchange", default="peer", choices=["peer", "peer-lines", "peer-flags", "nccl"],
                    help="tensor parallel: output rows stored by the GEMV itself as 16-byte lines that carry a sequence number into the peers' memory (peer), "
                         "the same lines pushed by a separate kernel (peer-lines), data followed by a flag (peer-flags), or NCCL all-gather")
    ap.add_argument("--eager", action="store_true", help="plain launches instead of a CUDA-graph replay")
    ap.add_argument("--gather-q", action="store_true",
                    help="tensor parallel: exchange the QKV output as well (by default every rank keeps its heads: attention is per head)")
    ap.add_argument("--fuse", default="none", choices=["none", "gemv", "layer", "token"],
                    help="dense, one GPU, M = 1: projections through the balanced-share kernel, one launch per projection / layer / token")
    ap.add_argument("--workload", default="dense", choices=["dense", "gemv", "moe", "mul1", "gemm", "intervals"],
                    help="dense = the headline (layer stack); gemv = one matrix (default 4096 x 4096); moe / mul1 = routed experts; gemm = batched rows")
    ap.add_argument("--tokens", type=int, default=8, help="moe / mul1: token rows per rank")
    ap.add_argument("--engine", default="auto", choices=["auto", "fp4", "f16"], help="gemm: block-scaled FP4 MMA, f16 MMA on widened weights, or by row count")
    ap.add_argument("--op", default="gemv", choices=["gemv", "gu", "fp8"], help="gemv workload: plain NVFP4 GEMV, fused gate/up, or the FP8 GEMV")
    ap.add_argument("--rows", type=int, default=4096, help="gemv: output rows")
    ap.add_argument("--cols", type=int, default=4096, help="gemv: k")
    args = ap.parse_args()
    globals()["MIN_TIMED_S"] = max(0.0, args.min_time)
    rank, world = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))
    local = int(os.environ.get("LOCAL_RANK", 0))
    if args.impl == "reference":
        return reference_arm(args, rank)
    args.warmup = max(args.warmup, 3)
    if args.workload == "intervals":
        return intervals_arm(args, rank, world, local)
    if args.workload == "gemm":
        return gemm_arm(args, rank, world, local)
    if args.workload == "gemv":
        return gemv_arm(args, rank, world, local)

    import torch
    import torch.distributed as dist
    from crownest_b200 import _lib, dense
    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    _lib.lib()  # fail loudly when the CUDA library is missing: there is no fallback
    if args.workload != "dense":
        return moe_arm(args, rank, world, local)

    stack = dense.DenseStack(layers=args.layers, device=f"cuda:{local}", seed=0, rank=rank, world=world, group=None, max_m=args.m,
                             exchange=args.exchange, gather_q=args.gather_q)
    m = args.m
    if args.fuse != "none" and world == 1 and m == 1:
        stack.fuse(args.fuse)
    gen = torch.Generator(device="cpu").manual_seed(1)
    x_host = torch.randn((m, stack.hidden), generator=gen).to(torch.bfloat16).pin_memory()
    y_host = torch.empty((m, stack.hidden), dtype=torch.bfloat16).pin_memory()
    stack.x[:m].copy_(x_host)
    # the whole step (256 launches, with their exchanges when tensor parallel) replays as one CUDA graph
    use_graph = not args.eager
    if use_graph:
        stack.capture(m)
    step = (lambda: stack.graph.replay()) if use_graph else (lambda: stack.run_layers(m))
    tm = Timer(world)
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    t = tm.run(step, args.steps, args.warmup)
    # end to end through the host-facing call: pinned host in, pinned host out, every step
    e2e_s = tm.wall(lambda: stack.decode_step(x_host, y_host), args.steps)
    clocks = sampler.stop() if rank == 0 else None
    status = _lib.device_status()
    line = None
    if rank == 0:
        bytes_step = stack.bytes_per_step(m)
        ms_step = t["ms_per_step"]
        value = bytes_step / (ms_step * 1e-3) / 1e9
        peak, peak_kind = measured_peak()
        per_gpu = value / world
        fused = stack.chains is not None
        line = {"metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
                "ms_per_step": ms_step, "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32",
                "data": "synthetic",
                "config": {"workload": f"nvfp4 dense decode stack 27B-shaped (hidden 5120, qkv 7168, inter 17408, {stack.layers} layers), M={m}",
                           "activations": "bf16 in/out, f32 accumulate", "parallelism": (f"tp{world} row split + " + ("exchange over peer memory fused into the GEMV" if stack.peer is not None and stack.peer.fused
                                                                        else "peer-memory exchange" if stack.peer is not None else "NCCL all-gather")
                                           + (" after o, gate/up and down (QKV heads stay on their rank)" if stack.local_only else " after every projection")) if world > 1 else "none",
                           "l2": "inputs larger than L2: %.2f GB of weights streamed per step" % (bytes_step / 1e9),
                           "launch": ("CUDA graph replay" if use_graph else "eager launches") + (f", projections fused per {args.fuse}" if fused else ""),
                           "tokens_per_s": m / (ms_step * 1e-3)},
                "roofline": {"bound": "hbm", "achieved": per_gpu, "peak": peak, "unit": "GB/s", "frac": per_gpu / peak, "scope": "per GPU",
                             "traffic": TRAFFIC_RATIO * bytes_step / world / (4 * stack.layers) if m == 1 else None,
                             "traffic_note": "dram read+write bytes of one ncu capture of the gate/up launch (profiles/), scaled to the average projection by bytes",
                             "peak_kind": peak_kind, "kernel": "nvfp4_gemv_seq_kernel" if fused else "nvfp4_gemv_m1_kernel", "bytes_per_launch": bytes_step / world / (4 * stack.layers),
                             "us_per_launch": ms_step * 1e3 / (4 * stack.layers)},
                "blocks": t["blocks"], "ms_per_step_min": t["ms_per_step_min"], "ms_per_step_max": t["ms_per_step_max"],
                "e2e": {"value": bytes_step / e2e_s / 1e9, "unit": UNIT, "h2d_bytes_per_step": x_host.numel() * 2,
                        "d2h_bytes_per_step": y_host.numel() * 2, "ms_per_step": e2e_s * 1e3},
                "gpu_launches": stack.launches_per_step * args.steps * t["blocks"], "clocks": clocks, "device_status": status}
        if world == 1 and not args.no_cpu_baseline:
            host_layers = [stack.host_copy(i) for i in range(min(3, stack.layers))]
            line["cpu_baseline"] = cpu_dense_baseline(host_layers, m)
    del stack
    torch.cuda.empty_cache()
    if world > 1:
        chk = exchange_check(rank, world, local)
        if rank == 0:
            line["exchange_check"] = chk
        torch.cuda.empty_cache()
    if not args.no_moe:
        block = moe_block(rank, world, local, max(10, args.steps // 2), args.warmup, cpu=not args.no_cpu_baseline)
        if rank == 0:
            line["moe"] = block
    if rank == 0:
        print(json.dumps(line), flush=True)
    leave(world)


if __name__ == "__main__":
    main()
