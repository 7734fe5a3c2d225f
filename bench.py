"""Benchmark of the quantized GEMV hot path: the NVFP4 dense decode layer stack (27B-shaped, 64
layers, M = 1) on N B200 GPUs of one node.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--m M] [--impl reference]

A step is one token through the whole stack (4 GEMV launches per layer). `value` is the algorithmic
bytes of a step (every weight byte once + activations) over the device time of a step, inputs
resident in HBM; `e2e` is the same through the host-facing call with pinned host buffers copied in
and out every step. One JSON line on stdout (rank 0).
"""
import argparse
import json
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
# captured gate/up launch (103.4 MB) over its algorithmic bytes (100.3 MB); the capture is summarised under profiles/
TRAFFIC_RATIO = 1.031


def measured_peak():
    try:
        return float(json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))["hbm_gbs"]), "measured"
    except Exception:
        return 6650.0, "fallback"


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
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": mx[0] if mx else None, "reasons": sorted(reasons),
                "samples": len(sm)}


def cpu_baseline_run(host_layers, threads, seconds_budget, m=1):
    """The CPU checker's NVFP4 GEMV (AVX2 arm of the reference's operation order, rows split over
    `threads`) over whole layers, rotating over the given distinct layers. Returns (GB/s, passes)."""
    import numpy as np
    import oracle
    rng = np.random.default_rng(0)
    xs = {}
    for mats in host_layers:
        for _, (_, _, k) in mats.items():
            xs.setdefault(k, rng.standard_normal((m, k)).astype(np.float32))
    path = 1 if oracle.lib().cn_o_have_avx2() else 0
    layer_bytes = sum(w.size for w, _, _ in host_layers[0].values())
    t_total, passes = 0.0, 0
    # one untimed pass: page faults, thread start
    for name, (w, rows, k) in host_layers[0].items():
        oracle.nvfp4_gemv(w, rows, k, 1.0, xs[k], threads=threads, path=path)
    while t_total < seconds_budget and passes < 64:
        mats = host_layers[passes % len(host_layers)]
        t0 = time.perf_counter()
        for name, (w, rows, k) in mats.items():
            oracle.nvfp4_gemv(w, rows, k, 1.0, xs[k], threads=threads, path=path)
        t_total += time.perf_counter() - t0
        passes += 1
    return (layer_bytes * passes / t_total / 1e9 if t_total > 0 else 0.0), passes


def reference_arm(args, rank):
    """`--impl reference`: the reference's CPU implementation of the path (its Rust source cannot be
    built here - no Rust toolchain - so the C port under oracle/ stands in, kind "port"), all host
    threads, each step one layer of the stack's shapes (186 MB of NVFP4)."""
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


def moe_arm(args, rank, world, local):
    """`--workload moe` / `mul1`: the routed-expert decode step (BASELINE configs 2 and 3), `--tokens` rows per rank,
    experts placed expert-parallel over the ranks (weak scaling: the global batch grows with the ranks)."""
    import torch
    import torch.distributed as dist
    from crownest_b200 import _lib, workloads
    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    _lib.lib()
    cls = workloads.MoeDecode if args.workload == "moe" else workloads.Mul1MoeDecode
    wl = cls(args.tokens, device=f"cuda:{local}", rank=rank, world=world, group=None)
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

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize()

    for _ in range(max(args.warmup, 3)):
        graph.replay()
    barrier()
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        graph.replay()
    e1.record()
    barrier()
    ms = e0.elapsed_time(e1)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        wl.x.copy_(x_host, non_blocking=True)
        graph.replay()
        y_host.copy_(wl.y, non_blocking=True)
        torch.cuda.current_stream().synchronize()
    barrier()
    e2e_s = time.perf_counter() - t0
    clocks = sampler.stop() if rank == 0 else None
    nbytes, distinct = wl.bytes_per_step()
    t = torch.tensor([ms, e2e_s, float(nbytes), float(distinct)], dtype=torch.float64, device="cuda")
    if world > 1:
        mx = t.clone()
        dist.all_reduce(mx, op=dist.ReduceOp.MAX)
        ms, e2e_s = float(mx[0]), float(mx[1])
    if rank == 0:
        ms_step = ms / args.steps
        toks = args.tokens * world
        peak, peak_kind = measured_peak()
        gbs = nbytes / (ms_step * 1e-3) / 1e9
        shape = ("hidden 2048, 512 experts, inter 512, shared expert 512, softmax top-10, NVFP4" if args.workload == "moe" else
                 "hidden 4096, 64 experts, inter 1536, top-4, EXL3 MUL1 K=3")
        line = {"metric": "moe_decode_tok_s", "value": toks / (ms_step * 1e-3), "unit": "tok/s", "n_gpus": world, "steps": args.steps,
                "warmup": max(args.warmup, 3), "ms_per_step": ms_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
                "dtype": "f32", "data": "synthetic",
                "config": {"workload": f"routed-expert decode step ({shape}), {args.tokens} tokens per rank", "parallelism": f"ep{world}" if world > 1 else "none",
                           "l2": "the expert set changes with the routing; weights of one step (%.0f MB on rank 0) fit L2, so the working set is flushed "
                                 "only by its own size at larger batches" % (nbytes / 1e6), "launch": "CUDA graph replay",
                           "distinct_experts_rank0_tokens": distinct},
                "roofline": {"bound": "hbm", "achieved": gbs, "peak": peak, "unit": "GB/s", "frac": gbs / peak, "traffic": None, "peak_kind": peak_kind,
                             "kernel": "nvfp4_gemv_m1_kernel (routed form)" if args.workload == "moe" else "mul1_gemv_kernel",
                             "note": "algorithmic bytes = distinct experts of rank 0's tokens x expert bytes + shared expert + activations"},
                "e2e": {"value": toks / (e2e_s / args.steps), "unit": "tok/s", "h2d_bytes_per_step": x_host.numel() * 2, "d2h_bytes_per_step": y_host.numel() * 2},
                "gpu_launches": args.steps * getattr(wl, "launches_per_step", 8), "clocks": clocks, "device_status": _lib.device_status()}
        print(json.dumps(line), flush=True)
    leave(world, graph)


def gemm_arm(args, rank, world, local):
    """`--workload gemm`: the batched NVFP4 GEMM (BASELINE config 4): W [17408 x 5120] then [5120 x 17408], --m rows,
    output columns split over the ranks with an all-gather (tensor parallel). A step = both GEMMs once."""
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
    gen.manual_seed(7)
    x_host = torch.randn((m, hidden), generator=torch.Generator().manual_seed(7)).to(torch.bfloat16).pin_memory()
    x = x_host.to(dev)
    h = torch.empty((m, inter), dtype=torch.bfloat16, device=dev)
    y = torch.empty((m, hidden), dtype=torch.bfloat16, device=dev)
    hp = torch.empty((m, inter // world), dtype=torch.bfloat16, device=dev) if world > 1 else h
    yp = torch.empty((m, hidden // world), dtype=torch.bfloat16, device=dev) if world > 1 else y
    y_host = torch.empty((m, hidden), dtype=torch.bfloat16).pin_memory()
    ws = torch.empty(ops.gemm_workspace_bytes(inter, m), dtype=torch.uint8, device=dev)

    def step(i):
        ops.launch_gemm(ups[i % ncopy], x, hp, workspace=ws)
        if world > 1:
            dense.gather_rows(hp, h, m, world)
        ops.launch_gemm(downs[i % ncopy], h, yp, workspace=ws)
        if world > 1:
            dense.gather_rows(yp, y, m, world)

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize()

    for i in range(max(args.warmup, 3)):
        step(i)
    barrier()
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(args.steps):
        step(i)
    e1.record()
    barrier()
    ms = e0.elapsed_time(e1)
    t0 = time.perf_counter()
    for i in range(args.steps):
        x.copy_(x_host, non_blocking=True)
        step(i)
        y_host.copy_(y, non_blocking=True)
        torch.cuda.current_stream().synchronize()
    barrier()
    e2e_s = time.perf_counter() - t0
    clocks = sampler.stop() if rank == 0 else None
    if world > 1:
        t = torch.tensor([ms, e2e_s], dtype=torch.float64, device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms, e2e_s = float(t[0]), float(t[1])
    if rank == 0:
        flops = 2.0 * m * hidden * inter * 2
        ms_step = ms / args.steps
        tf = flops / (ms_step * 1e-3) / 1e12
        try:
            peak, kind = float(json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))["bf16_tflops"]), "measured (bf16 GEMM, burst)"
        except Exception:
            peak, kind = 1590.0, "fallback"
        line = {"metric": "nvfp4_gemm_tflops", "value": tf, "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3),
                "ms_per_step": ms_step, "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f16 x f16 -> f32", "data": "synthetic",
                "config": {"workload": f"nvfp4 GEMM pair [17408 x 5120] and [5120 x 17408], M={m}", "parallelism": f"tp{world} column split + all-gather" if world > 1 else "none",
                           "l2": "three weight copies rotated (300 MB per rank) plus the activations: larger than L2", "launch": "plain launches"},
                "roofline": {"bound": "tensor", "achieved": tf / world, "peak": peak, "unit": "TFLOP/s", "frac": tf / world / peak, "traffic": None, "peak_kind": kind,
                             "kernel": "nvfp4_gemm_tc5_kernel", "flops_per_launch": flops / 2 / world, "us_per_launch": ms_step * 1e3 / 2,
                             "hbm_gbs": (2 * hidden * inter // 64 * 36 / world + 2.0 * m * (hidden + inter) * 2) / (ms_step * 1e-3) / 1e9},
                "e2e": {"value": flops / (e2e_s / args.steps) / 1e12, "unit": "TFLOP/s", "h2d_bytes_per_step": x_host.numel() * 2, "d2h_bytes_per_step": y_host.numel() * 2},
                "gpu_launches": args.steps * 4, "clocks": clocks, "device_status": _lib.device_status()}
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


def trace(msg):
    """Progress lines on stderr when CN_BENCH_TRACE is set (to see where a multi-rank run stops)."""
    if os.environ.get("CN_BENCH_TRACE"):
        print(f"[bench rank {os.environ.get('RANK', 0)} +{time.perf_counter() - T0:.1f}s] {msg}", file=sys.stderr, flush=True)


T0 = time.perf_counter()


def main():
    if os.environ.get("CN_BENCH_TRACE"):
        import faulthandler
        faulthandler.dump_traceback_later(int(os.environ["CN_BENCH_TRACE"]), exit=True)
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=5)
    # "--act-rows": the spelling to use under torch.distributed.run, whose own parser takes "--m" for an abbreviation
    ap.add_argument("--m", "--act-rows", dest="m", type=int, default=1, help="activation rows per step (1 decode, 4 = MTP verify)")
    ap.add_argument("--layers", type=int, default=64)
    ap.add_argument("--impl", default="crownest")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--exchange", default="peer", choices=["peer", "nccl"], help="tensor parallel: slices pushed over peer memory, or NCCL all-gather")
    ap.add_argument("--eager", action="store_true", help="plain launches instead of a CUDA-graph replay")
    ap.add_argument("--workload", default="dense", choices=["dense", "moe", "mul1", "gemm"], help="dense = the headline (config 1); moe / mul1 = configs 2 / 3")
    ap.add_argument("--tokens", type=int, default=8, help="moe / mul1: token rows per rank")
    args = ap.parse_args()
    rank, world = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))
    local = int(os.environ.get("LOCAL_RANK", 0))
    if args.impl == "reference":
        return reference_arm(args, rank)
    args.warmup = max(args.warmup, 3)
    if args.workload == "gemm":
        return gemm_arm(args, rank, world, local)
    if args.workload != "dense":
        return moe_arm(args, rank, world, local)

    import torch
    import torch.distributed as dist
    from crownest_b200 import _lib, dense
    torch.cuda.set_device(local)
    group = None
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    _lib.lib()  # fail loudly when the CUDA library is missing: there is no fallback
    trace("process group up")

    stack = dense.DenseStack(layers=args.layers, device=f"cuda:{local}", seed=0, rank=rank, world=world, group=group, max_m=args.m,
                             exchange=args.exchange)
    m = args.m
    gen = torch.Generator(device="cpu").manual_seed(1)
    x_host = torch.randn((m, stack.hidden), generator=gen).to(torch.bfloat16).pin_memory()
    y_host = torch.empty((m, stack.hidden), dtype=torch.bfloat16).pin_memory()
    stack.x[:m].copy_(x_host)
    # the whole step (256 launches, with their all-gathers when tensor parallel) replays as one CUDA graph
    use_graph = not args.eager
    if use_graph:
        stack.capture(m)
    step = (lambda: stack.graph.replay()) if use_graph else (lambda: stack.run_layers(m))

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize()

    trace("captured" if use_graph else "eager")
    for _ in range(args.warmup):
        step()
    barrier()
    trace("warm")
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        step()
    e1.record()
    barrier()
    ms = e0.elapsed_time(e1)
    # end to end through the host-facing call: pinned host in, pinned host out, every step
    for _ in range(2):
        stack.decode_step(x_host, y_host)
    barrier()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        stack.decode_step(x_host, y_host)
    barrier()
    e2e_s = time.perf_counter() - t0
    clocks = sampler.stop() if rank == 0 else None
    if world > 1:
        t = torch.tensor([ms, e2e_s], dtype=torch.float64, device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms, e2e_s = float(t[0]), float(t[1])
    status = _lib.device_status()

    if rank == 0:
        bytes_step = stack.bytes_per_step(m)
        ms_step = ms / args.steps
        value = bytes_step / (ms_step * 1e-3) / 1e9
        peak, peak_kind = measured_peak()
        per_gpu = value / world
        line = {"metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
                "ms_per_step": ms_step, "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32",
                "data": "synthetic",
                "config": {"workload": f"nvfp4 dense decode stack 27B-shaped (hidden 5120, qkv 7168, inter 17408, {stack.layers} layers), M={m}",
                           "activations": "bf16 in/out, f32 accumulate", "parallelism": (f"tp{world} row split + " + ("peer-memory exchange" if stack.peer is not None else "NCCL all-gather")) if world > 1 else "none",
                           "l2": "inputs larger than L2: %.2f GB of weights streamed per step" % (bytes_step / 1e9),
                           "launch": "CUDA graph replay" if use_graph else "eager launches", "tokens_per_s": m / (ms_step * 1e-3)},
                "roofline": {"bound": "hbm", "achieved": per_gpu, "peak": peak, "unit": "GB/s", "frac": per_gpu / peak, "traffic": TRAFFIC_RATIO * bytes_step / world / stack.launches_per_step if m == 1 else None,
                             "traffic_note": "dram read+write bytes of one ncu capture of the gate/up launch (profiles/), scaled to the average launch by bytes",
                             "peak_kind": peak_kind, "kernel": "nvfp4_gemv_m1_kernel" if m == 1 else "nvfp4_gemv_mma_kernel", "bytes_per_launch": bytes_step / world / stack.launches_per_step,
                             "us_per_launch": ms_step * 1e3 / stack.launches_per_step},
                "e2e": {"value": bytes_step / (e2e_s / args.steps) / 1e9, "unit": UNIT, "h2d_bytes_per_step": x_host.numel() * 2,
                        "d2h_bytes_per_step": y_host.numel() * 2, "ms_per_step": e2e_s / args.steps * 1e3},
                "gpu_launches": stack.launches_per_step * args.steps, "clocks": clocks, "device_status": status}
        if world == 1 and not args.no_cpu_baseline:
            host_layers = [stack.host_copy(i) for i in range(min(3, stack.layers))]
            threads = os.cpu_count() or 1
            gbs, passes = cpu_baseline_run(host_layers, threads, 12.0, m)
            line["cpu_baseline"] = {"value": gbs, "unit": UNIT, "cores": threads, "kind": "port",
                                    "sample": f"{passes} passes over whole layers ({host_layers and sum(w.size for w, _, _ in host_layers[0].values())} B each), "
                                              f"{len(host_layers)} distinct layers rotated, AVX2 arm"}
        print(json.dumps(line), flush=True)
    leave(world, stack)


if __name__ == "__main__":
    main()
