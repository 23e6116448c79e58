#!/usr/bin/env python
"""Benchmark of the GGUF quantized-matmul decode path on B200.

One "step" is one token's worth of quantized matmuls of a Llama-3-shaped Q4_K_M model at batch 1: per layer
attn_q/k/v, attn_output, ffn_gate/up/down, plus the output head. On one GPU that is the 8B shape (225 GEMVs over
4.88 GB of packed weights); on N > 1 GPUs the 70B shape, tensor-parallel as the reference splits it (q/k/v, gate/up and
the head by output rows; attn_output and ffn_down by input columns in whole superblocks, each followed by a sum
all-reduce of the [1, hidden] partial output). Every layer has its own weights, so each step streams far more than the
126 MB L2. Attention, norms and sampling are not part of the path and are not run. Weights are random well-formed GGUF
blocks, activations ~N(0,1) bf16.

  value        tok/s with inputs resident in HBM, timed with CUDA events over K steps (CUDA-graph replay of the step)
  e2e          the same through the host-buffer call: every step copies the token's activations from pinned host memory
               and reads the logits back
  roofline     the dominant launch (ffn_gate + ffn_up) timed alone over all layers' distinct weights
  cpu_baseline / --impl reference   the CPU oracle (a C restatement of the reference's k_quants::matmul) on the host cores
  reference_cuda   the reference's own CUDA kernels (generic dp4a / mma.sync, compiled for sm_100a from the reference
               checkout into oracle/_ref) on the same chain and shapes, when that library was built

Prints one JSON line on rank 0.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

METRIC = "q4_k_m_decode_matmul_tok_per_s"
UNIT = "tok/s"


def load_peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        with open(p) as fh:
            d = json.load(fh)
        return float(d["hbm_gbs"]), float(d["bf16_tflops"]), "measured"
    return 6650.0, 1590.0, "fallback"


def host_threads() -> int:
    """Host cores this process may use. Not OMP_NUM_THREADS: torch.distributed.run sets that to 1 for its children."""
    try:
        return max(1, len(os.sched_getaffinity(0)))
    except AttributeError:
        return max(1, os.cpu_count() or 1)


def workload_name(model, world: int) -> str:
    """The same string in both arms (ours and --impl reference) at a given N."""
    gemvs = model.layers * len(model.layer_projections()) + 1
    gb = model.weight_bytes_per_token() / 1e9
    tp = "" if world == 1 else f", tensor-parallel over {world} GPUs"
    return f"{model.name} Q4_K_M decode matmul chain, batch 1{tp} ({gemvs} GEMVs, {gb:.2f} GB of weights per token)"


class ClockSampler:
    """Samples nvidia-smi clocks and throttle reasons while the timed region runs."""

    QUERY = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index = index
        self.samples = []
        self._stop = threading.Event()
        self._thread = None

    def _run(self):
        while not self._stop.is_set():
            try:
                out = subprocess.run(["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits", "-i",
                                      str(self.index)], capture_output=True, text=True, timeout=5).stdout.strip()
                if out:
                    self.samples.append([f.strip() for f in out.split(",")])
            except Exception:
                pass
            self._stop.wait(0.1)

    def __enter__(self):
        self._thread = threading.Thread(target=self._run, daemon=True)
        self._thread.start()
        return self

    def __exit__(self, *exc):
        self._stop.set()
        self._thread.join(timeout=6)

    def summary(self):
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for s in self.samples:
            try:
                sm.append(float(s[0]))
                mx.append(float(s[1]))
            except (ValueError, IndexError):
                continue
            for name, val in zip(names, s[3:7]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def random_blocks_device(torch, dtype, n, k, gen):
    """Random well-formed packed blocks on the device, padded like the reference's device buffers."""
    nb = n * (k // dtype.block_size)
    bb = dtype.type_size
    pad = 512 * bb // dtype.block_size
    buf = torch.zeros(nb * bb + pad, dtype=torch.uint8, device="cuda")
    raw = buf[: nb * bb].view(nb, bb)
    raw.copy_(torch.randint(0, 256, (nb, bb), dtype=torch.uint8, device="cuda", generator=gen))

    def half_bytes(lo, hi):
        v = (torch.rand(nb, device="cuda", generator=gen) * (hi - lo) + lo).to(torch.float16)
        return v.view(torch.uint8).view(nb, 2)

    if dtype.name == "Q8_0":
        raw[:, 0:2] = half_bytes(2e-4, 6e-4)
    elif dtype.name == "Q4K":
        raw[:, 0:2] = half_bytes(5e-5, 2e-4)
        raw[:, 2:4] = half_bytes(5e-5, 2e-4)
    else:
        raw[:, 208:210] = half_bytes(-3e-5, 3e-5)
    return buf


def time_launch_list(torch, stream, launches, reps):
    """Captures the launches (callables on the current stream) into one CUDA graph, replays it `reps` times and
    returns the mean device time of one launch in microseconds (CUDA events on `stream`)."""
    for fn in launches:
        fn()  # eager once: first-launch attribute set-up may not run under capture
    stream.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g, stream=stream):
        for fn in launches:
            fn()
    g.replay()
    stream.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(stream)
    for _ in range(reps):
        g.replay()
    e1.record(stream)
    stream.synchronize()
    return e0.elapsed_time(e1) * 1000.0 / (reps * len(launches))


def register_launch_order(ops, seq):
    """seq: one (key weight, first weight, dtype, k, n) per launch, in stream order; the order is cyclic (the last
    launch of a token is followed by the first of the next). Tells the library which matrix follows which."""
    for i, (key, _, _, _, _) in enumerate(seq):
        _, nxt, ndt, nk, nn = seq[(i + 1) % len(seq)]
        ops.set_weight_successor(key, nxt, ndt, nk, nn)


# DRAM bytes per launch measured by ncu (dram__bytes_read.sum + dram__bytes_write.sum); the summaries are under profiles/
NCU_TRAFFIC_GEMV_Q4K_4096_14336 = 33085184
NCU_TRAFFIC_GROUP_GATE_UP = 66316288

TYPE_TAGS = {"q4_k": "Q4K", "q6_k": "Q6K", "q8_0": "Q8_0"}


def run_single(args):
    """--single TYPE K N B: one GEMV shape over rotating weight copies (> L2 in total); prints one JSON line. This is
    the small case profiler captures run on."""
    import torch

    import inference_rs_b200 as pkg
    from inference_rs_b200 import ops

    tname, k, n, b = args.single[0], int(args.single[1]), int(args.single[2]), int(args.single[3])
    dt = getattr(pkg.GgmlDType, TYPE_TAGS[tname])
    torch.cuda.set_device(0)
    gen = torch.Generator(device="cuda").manual_seed(7)
    wbytes = n * dt.row_bytes(k)
    copies = args.copies or max(2, min(64, int(400e6 // wbytes) + 1))
    ws = [random_blocks_device(torch, dt, n, k, gen) for _ in range(copies)]
    x = torch.randn(b, k, device="cuda", generator=gen).to(torch.bfloat16)
    out = torch.empty(b, n, dtype=torch.bfloat16, device="cuda")
    if not args.no_prefetch and not args.tc:
        register_launch_order(ops, [(w, w, dt, k, n) for w in ws])
    stream = torch.cuda.Stream()
    with torch.cuda.stream(stream):
        if args.two_launch:
            def mk(w):
                def fn():
                    vy = ops.quantize_q8_1(x)
                    ops.mmvq_plain(dt, w, vy, n, k, b, torch.bfloat16)
                return fn
        elif args.group2:
            outs2 = [torch.empty(b, n, dtype=torch.bfloat16, device="cuda") for _ in range(2)]

            def mk(w):
                return lambda: ops.gemv_group([dt, dt], [ws[0], w], x, [n, n], outs=outs2)
        elif args.tc:
            tc_ws = ops.gemv_tc_workspace(dt, k)

            def mk(w):
                return lambda: ops.gemv_tc(dt, w, x, n, out=out, workspace=tc_ws)
        else:
            def mk(w):
                return lambda: ops.gemv(dt, w, x, n, out=out, act_quant=args.act_quant)
        launches = [mk(w) for w in ws]
        if args.no_graph:
            for fn in launches:
                fn()
            stream.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(stream)
            for _ in range(args.steps):
                for fn in launches:
                    fn()
            e1.record(stream)
            stream.synchronize()
            us = e0.elapsed_time(e1) * 1000.0 / (args.steps * len(launches))
        else:
            us = time_launch_list(torch, stream, launches, args.steps)
    peak, _, src = load_peaks()
    alg = wbytes + b * k * 2 + b * n * 2
    if args.group2:
        alg = 2 * wbytes + b * k * 2 + 2 * b * n * 2
    print(json.dumps({"single": tname, "k": k, "n": n, "b": b, "copies": copies, "us_per_launch": us,
                      "GBps": alg / us / 1e3, "frac_of_" + src: alg / us / 1e3 / peak, "algorithmic_bytes": alg,
                      "kernel": "gemv_tc" if args.tc else ("gemv_group x2" if args.group2 else "gemv"),
                      "l2_prefetch_bytes": 0 if args.no_prefetch else ops.get_option("l2_prefetch_bytes"), "pdl": ops.get_option("pdl"),
                      "plan": None if (args.tc or b > 8) else ops.gemv_plan(dt, k, n, b),
                      "device_status": list(pkg.kernel_library.device_status())}),
          flush=True)


def run_gemm_single(args):
    """--gemm TYPE K N M: one prefill GEMM shape; prints one JSON line with TFLOP/s against the measured bf16 peak."""
    import torch

    import inference_rs_b200 as pkg
    from inference_rs_b200 import ops

    tname, k, n, m = args.gemm[0], int(args.gemm[1]), int(args.gemm[2]), int(args.gemm[3])
    dt = getattr(pkg.GgmlDType, TYPE_TAGS[tname])
    torch.cuda.set_device(0)
    gen = torch.Generator(device="cuda").manual_seed(11)
    w = random_blocks_device(torch, dt, n, k, gen)
    x = torch.randn(m, k, device="cuda", generator=gen).to(torch.bfloat16)
    y = torch.empty(m, n, dtype=torch.bfloat16, device="cuda")
    stream = torch.cuda.Stream()
    with torch.cuda.stream(stream):
        for _ in range(3):
            ops.gemm(dt, w, x, n, out=y)
        stream.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        for _ in range(args.steps):
            ops.gemm(dt, w, x, n, out=y)
        e1.record(stream)
        stream.synchronize()
    us = e0.elapsed_time(e1) * 1000.0 / args.steps
    tflops = 2.0 * m * n * k / us / 1e6
    _, peak, _ = load_peaks()
    print(json.dumps({"gemm": tname, "k": k, "n": n, "m": m, "us": us, "TFLOPs": tflops, "frac_of_measured_bf16": tflops / peak,
                      "device_status": list(pkg.kernel_library.device_status())}), flush=True)


def cpu_chain_sample(model, threads, seconds_budget=12.0):
    """Times the CPU oracle on one layer's projections plus a slice of the output head at batch 1 and scales to a
    token. Returns (tok/s, description)."""
    import numpy as np
    from oracle import kquants as kq
    type_of = {"Q8_0": kq.Q8_0, "Q4K": kq.Q4_K, "Q6K": kq.Q6_K}
    rng = np.random.default_rng(0)
    projs = model.layer_projections()
    head = model.output_projection()
    # a 1/8 slice of the head keeps the sample's memory small; its time is scaled back up
    head_rows = head.n // 8

    def blocks(p, rows):
        t = type_of[p.dtype.name]
        nb = rows * (p.k // kq.BLOCK_ELEMS[t])
        raw = rng.integers(0, 256, size=(nb, kq.BLOCK_BYTES[t]), dtype=np.uint8)
        d = rng.uniform(5e-5, 2e-4, nb).astype(np.float16).view(np.uint8).reshape(nb, 2)
        if t == kq.Q6_K:
            raw[:, 208:210] = d
        else:
            raw[:, 0:2] = d
            if t == kq.Q4_K:
                raw[:, 2:4] = d
        return t, raw.reshape(rows, -1)

    layer_w = [blocks(p, p.n) for p in projs]
    head_w = blocks(head, head_rows)
    xs = {k: rng.standard_normal((1, k)).astype(np.float32) for k in {p.k for p in projs} | {head.k}}

    def one_pass():
        t0 = time.perf_counter()
        for p, (t, w) in zip(projs, layer_w):
            kq.matmul(t, xs[p.k], w, p.n, threads)
        t_layer = time.perf_counter() - t0
        t0 = time.perf_counter()
        kq.matmul(head_w[0], xs[head.k], head_w[1], head_rows, threads)
        t_head = (time.perf_counter() - t0) * (head.n / head_rows)
        return t_layer, t_head

    one_pass()
    best_layer, best_head = float("inf"), float("inf")
    t_start = time.perf_counter()
    reps = 0
    while reps < 3 or (time.perf_counter() - t_start < seconds_budget and reps < 200):
        tl, th = one_pass()
        best_layer, best_head = min(best_layer, tl), min(best_head, th)
        reps += 1
    tok_s = 1.0 / (best_layer * model.layers + best_head)
    desc = (f"{model.name}: 1 of {model.layers} layers (7 projections, unsharded) + 1/8 of the output head at batch 1, best of {reps} "
            f"passes, scaled to a token; scalar/auto-vectorised C port of k_quants::matmul, {threads} threads")
    return tok_s, desc


def run_reference(args, rank, world):
    """--impl reference: the reference's CPU path on the host cores (the oracle port: the Rust reference cannot be built
    here), on the same model as our arm runs at this N - the whole model on one host, as the CPU path has no tensor
    parallelism."""
    if rank != 0:
        return
    from inference_rs_b200 import workloads
    threads = host_threads()
    model = workloads.LLAMA3_70B if world > 1 else workloads.LLAMA3_8B
    vals = []
    desc = ""
    t0 = time.perf_counter()
    for _ in range(args.warmup):
        cpu_chain_sample(model, threads, seconds_budget=0.0)
    for _ in range(args.steps):
        v, desc = cpu_chain_sample(model, threads, seconds_budget=max(1.0, 60.0 / max(1, args.steps)))
        vals.append(v)
    value = max(vals)
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": 1000.0 / value, "higher_is_better": True, "scaling": "strong" if world > 1 else "weak",
        "vs_baseline": None, "dtype": "int8 dot, f32 accumulate", "data": "synthetic",
        "config": {"workload": workload_name(model, world)},
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": threads, "kind": "port", "sample": desc},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "wall_s": time.perf_counter() - t0,
    }
    print(json.dumps(line), flush=True)


class Chain:
    """One rank's share of a model's decode matmul chain: weights, activations, outputs and the step that launches it."""

    def __init__(self, torch, pkg, ops, workloads, model, shards, seed, group=True, act_quant=0, weights_of=None):
        self.torch, self.ops, self.model, self.shards = torch, ops, model, shards
        self.act_quant = act_quant
        gen = torch.Generator(device="cuda").manual_seed(seed)
        self.projs = [workloads.shard(p, shards) for p in model.layer_projections()]
        self.head = workloads.shard(model.output_projection(), shards)
        if weights_of is not None:  # another chain's weights (same model and sharding)
            self.layers, self.head_w = weights_of.layers, weights_of.head_w
        else:
            self.layers = [[random_blocks_device(torch, p.dtype, p.n, p.k, gen) for p in self.projs] for _ in range(model.layers)]
            self.head_w = random_blocks_device(torch, self.head.dtype, self.head.n, self.head.k, gen)
        self.ks = sorted({p.k for p in self.projs} | {self.head.k})
        self.x_host = {k: torch.randn(1, k, generator=torch.Generator().manual_seed(k)).to(torch.bfloat16).pin_memory() for k in self.ks}
        self.x_dev = {k: v.cuda() for k, v in self.x_host.items()}
        self.outs = [[torch.empty(1, p.n, dtype=torch.bfloat16, device="cuda") for p in self.projs] for _ in range(model.layers)]
        self.logits = torch.empty(1, self.head.n, dtype=torch.bfloat16, device="cuda")
        self.bytes_per_step = model.layers * sum(p.weight_bytes for p in self.projs) + self.head.weight_bytes  # per GPU
        # projections that read the same input go out in one launch: q/k/v, gate/up (the reference's fused_qkv / fused_glu
        # matvec launches, crates/inference-quant/src/lib.rs:2441-2776)
        self.groups = []
        if group:
            names = [p.name for p in self.projs]
            for members in (("attn_q", "attn_k", "attn_v"), ("ffn_gate", "ffn_up")):
                self.groups.append([names.index(m) for m in members])
        self.grouped = {i for g in self.groups for i in g}
        self.launches_per_step = model.layers * (len(self.projs) - len(self.grouped) + len(self.groups)) + 1
        self.gemvs_per_step = model.layers * len(self.projs) + 1

    def launch_sequence(self):
        """(key weight, first weight, dtype, k, n) per launch, in the order step() issues them."""
        seq = []
        for li in range(self.model.layers):
            for g in self.groups:
                first, last = g[0], g[-1]
                seq.append((self.layers[li][last], self.layers[li][first], self.projs[first].dtype, self.projs[first].k, self.projs[first].n))
            for i, p in enumerate(self.projs):
                if i not in self.grouped:
                    seq.append((self.layers[li][i], self.layers[li][i], p.dtype, p.k, p.n))
        seq.append((self.head_w, self.head_w, self.head.dtype, self.head.k, self.head.n))
        return seq

    def step(self, row_parallel=None, after_head=None):
        """row_parallel(i, p, w, x, out): launches projection i's matmul and its exchange (tensor parallel), or None."""
        ops = self.ops
        for li in range(self.model.layers):
            for g in self.groups:
                ops.gemv_group([self.projs[i].dtype for i in g], [self.layers[li][i] for i in g], self.x_dev[self.projs[g[0]].k],
                               [self.projs[i].n for i in g], outs=[self.outs[li][i] for i in g], act_quant=self.act_quant)
            for i, (p, w, o) in enumerate(zip(self.projs, self.layers[li], self.outs[li])):
                if i in self.grouped:
                    continue
                if row_parallel is not None and p.split == "row":
                    row_parallel(i, p, w, self.x_dev[p.k], o)
                else:
                    ops.gemv(p.dtype, w, self.x_dev[p.k], p.n, out=o, act_quant=self.act_quant)
        ops.gemv(self.head.dtype, self.head_w, self.x_dev[self.head.k], self.head.n, out=self.logits, act_quant=self.act_quant)
        if after_head is not None:
            after_head()

    def free(self):
        self.ops.clear_weight_successors()
        self.layers = self.head_w = self.outs = None


def time_chain(torch, stream, step, steps, warmup, use_graph=True):
    """ms per step of `step` (CUDA events on `stream`), after one eager run, capture and `warmup` replays."""
    with torch.cuda.stream(stream):
        step()
        stream.synchronize()
        graph = None
        if use_graph:
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=stream):
                step()
        run = graph.replay if graph is not None else step
        for _ in range(warmup):
            run()
        stream.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        for _ in range(steps):
            run()
        e1.record(stream)
        stream.synchronize()
        return e0.elapsed_time(e1) / steps


def gguf_round_trip(torch, pkg, ops, chain):
    """The benched weights as FILE bytes: the first layer's seven projections are written to a llama-shaped GGUF file
    (tensor names and metadata as llama.cpp writes them), read back through the container reader and the llama name map,
    uploaded, and multiplied: the outputs must equal, bit for bit, those of the buffers the chain runs on."""
    import os
    import tempfile

    from inference_rs_b200 import llama_gguf
    from inference_rs_b200.gguf_file import Content

    model = chain.model
    projs = model.layer_projections()
    layer0 = {p.name: w for p, w in zip(chain.projs, chain.layers[0])}

    def make(name, p):
        buf = layer0[name.split(".")[2]]
        return buf[: p.n * p.dtype.row_bytes(p.k)].cpu().numpy()

    fd, path = tempfile.mkstemp(suffix=".gguf")
    try:
        with os.fdopen(fd, "wb") as f:
            llama_gguf.write_random_llama(f, model, 1, make, include_output=False)
        size = os.path.getsize(path)
        with open(path, "rb") as f:
            content = Content.read(f)
            loaded = llama_gguf.load_projections(f, content, "cuda")
    finally:
        os.unlink(path)
    identical = True
    for p in projs:
        q = loaded[llama_gguf.checkpoint_name(f"blk.0.{p.name}.weight")]
        x = chain.x_dev[p.k]
        a = ops.gemv(p.dtype, q.data, x, p.n)
        b = ops.gemv(p.dtype, layer0[p.name], x, p.n)
        identical = identical and bool(torch.equal(a, b))
    torch.cuda.synchronize()
    return {"layers": 1, "tensors": len(projs), "file_bytes": size, "outputs_identical": identical}


def reference_cuda_numbers(torch, pkg, chain, stream, peak, bf16_peak, steps):
    """The reference's own CUDA kernels on this GPU (oracle/_ref, built from the reference checkout): its decode chain
    as its host would launch it - one Q8_1 quantize per distinct input, plain matvecs for q/k/v (mixed types), the
    fused gate/up matvec, plain matvecs for attn_output, ffn_down and the head - and its prefill path (quantize + MMQ)
    on a few shapes. Returns None when the library is not there."""
    try:
        from oracle import refkernels as rk
        if not rk.available():
            return None
    except Exception as exc:  # missing file, unloadable library
        return {"unavailable": f"{type(exc).__name__}: {exc}"}
    model, projs = chain.model, chain.projs
    names = [p.name for p in projs]
    idx = {n: names.index(n) for n in names}
    x = chain.x_dev
    bf = torch.bfloat16

    def step():
        for li in range(model.layers):
            w = chain.layers[li]
            vy = rk.quantize_q8_1(x[projs[0].k])
            for nme in ("attn_q", "attn_k", "attn_v"):
                p = projs[idx[nme]]
                rk.mmvq_plain(int(p.dtype), w[idx[nme]], vy, p.n, p.k, 1, bf)
            p = projs[idx["attn_output"]]
            rk.mmvq_plain(int(p.dtype), w[idx["attn_output"]], rk.quantize_q8_1(x[p.k]), p.n, p.k, 1, bf)
            p = projs[idx["ffn_gate"]]
            rk.fused_glu(int(p.dtype), w[idx["ffn_gate"]], w[idx["ffn_up"]], x[p.k], p.n)
            p = projs[idx["ffn_down"]]
            rk.mmvq_plain(int(p.dtype), w[idx["ffn_down"]], rk.quantize_q8_1(x[p.k]), p.n, p.k, 1, bf)
        rk.mmvq_plain(int(chain.head.dtype), chain.head_w, rk.quantize_q8_1(x[chain.head.k]), chain.head.n, chain.head.k, 1, bf)

    ms = time_chain(torch, stream, step, max(3, steps // 4), 3)
    out = {"kernels": "reference mmvq_gguf dp4a matvecs + fused_glu, compiled for sm_100a with the reference's nvcc flags",
           "decode_chain_tok_per_s": 1000.0 / ms, "decode_chain_ms": ms,
           "decode_chain_hbm_frac_of_measured": chain.bytes_per_step / (ms * 1e-3) / 1e9 / peak}
    # prefill: quantize + MMQ, a few shapes
    pre = []
    gen = torch.Generator(device="cuda").manual_seed(5)
    with torch.cuda.stream(stream):
        for dt, k, n in ((pkg.GgmlDType.Q4K, 4096, 4096), (pkg.GgmlDType.Q4K, 14336, 4096), (pkg.GgmlDType.Q6K, 14336, 4096)):
            wq = random_blocks_device(torch, dt, n, k, gen)
            for m in (512, 2048, 8192):
                xm = torch.randn(m, k, device="cuda", generator=gen).to(bf)
                for _ in range(2):
                    rk.mmq_forward(int(dt), wq, xm, n)
                stream.synchronize()
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record(stream)
                for _ in range(5):
                    rk.mmq_forward(int(dt), wq, xm, n)
                e1.record(stream)
                stream.synchronize()
                us = e0.elapsed_time(e1) * 200.0
                tf = 2.0 * m * n * k / us / 1e6
                pre.append({"type": dt.name, "k": k, "n": n, "m": m, "us": round(us, 1), "TFLOPs": round(tf, 1),
                            "frac_of_measured_bf16_peak": round(tf / bf16_peak, 3)})
            del wq
    out["prefill_mmq"] = pre
    return out


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-graph", action="store_true", help="launch the step eagerly instead of replaying a CUDA graph")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-group", action="store_true", help="one launch per projection instead of grouped q/k/v and gate/up")
    ap.add_argument("--no-prefetch", action="store_true", help="do not register the launch order (no L2 prefetch of the next matrix)")
    ap.add_argument("--quick", action="store_true", help="the headline numbers only (no prefill / small-batch / reference_cuda / tp_base keys)")
    ap.add_argument("--sweep", action="store_true", help="also time every shape of the decode sweep")
    ap.add_argument("--single", nargs=4, metavar=("TYPE", "K", "N", "B"), help="time one GEMV shape only (q4_k|q6_k|q8_0)")
    ap.add_argument("--act-quant", type=int, default=0, help="--single: 0 = Q8_1 activations, 1 = the CPU path's format")
    ap.add_argument("--unfused-allreduce", action="store_true", help="N > 1: the peer-memory all-reduce as a launch of its own")
    ap.add_argument("--shard-of", type=int, default=0, help="N = 1 only: run one rank's share of the N-way 70B chain, no exchanges")
    ap.add_argument("--nccl-allreduce", action="store_true", help="N > 1: NCCL all-reduce instead of the peer-memory kernel")
    ap.add_argument("--group2", action="store_true", help="with --single: two matrices of the shape in one grouped launch (B = 1)")
    ap.add_argument("--tc", action="store_true", help="with --single: the small-batch tensor-core kernel (B up to 16)")
    ap.add_argument("--gemm", nargs=4, metavar=("TYPE", "K", "N", "M"), help="time one prefill GEMM shape only")
    ap.add_argument("--copies", type=int, default=0, help="--single: number of rotating weight copies")
    ap.add_argument("--two-launch", action="store_true", help="--single: quantize launcher + GEMV launcher instead of one launch")
    ap.add_argument("--pdl", type=int, default=1,
                    help="programmatic dependent launch for the decode chain (the library's 'pdl' option; its default is 0 because it "
                         "assumes that the weights are not written by the work just before a launch - true of a decoder's weights)")
    ap.add_argument("--stage-bytes", type=int, default=None, help="GEMV planner: target bytes per shared-memory stage")
    ap.add_argument("--prefetch-bytes", type=int, default=None, help="bytes of the next matrix each CTA asks L2 for")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup

    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))

    if args.impl == "reference":
        run_reference(args, rank, world)
        return
    from inference_rs_b200 import ops as _ops
    if args.pdl is not None:
        _ops.set_option("pdl", args.pdl)
    if args.stage_bytes is not None:
        _ops.set_option("gemv_stage_bytes", args.stage_bytes)
    if args.prefetch_bytes is not None:
        _ops.set_option("l2_prefetch_bytes", args.prefetch_bytes)
    if args.single:
        run_single(args)
        return
    if args.gemm:
        run_gemm_single(args)
        return

    import torch
    import torch.distributed as dist

    import inference_rs_b200 as pkg
    from inference_rs_b200 import ops, workloads

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: there is no CPU fallback for the product path")
    torch.cuda.set_device(local_rank)
    if world > 1:
        # NCCL only carries the logits all-gather, the checks and the timing reductions here; without in-switch (NVLS)
        # buffers no rank's memory stays bound to an NVLink multicast object when the processes leave
        os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    pkg.library()
    peak, bf16_peak, peak_src = load_peaks()

    tp = world > 1
    # --shard-of N on one GPU: one rank's share of the N-way tensor-parallel 70B chain without the exchanges (what the
    # compute alone costs at those shard shapes)
    shards = args.shard_of if (args.shard_of and not tp) else world
    model = workloads.LLAMA3_70B if (tp or shards > 1) else workloads.LLAMA3_8B
    chain = Chain(torch, pkg, ops, workloads, model, shards, 1234 + rank, group=not args.no_group)
    if not args.no_prefetch:
        register_launch_order(ops, chain.launch_sequence())
    projs, head = chain.projs, chain.head
    logits_all = torch.empty(world, head.n, dtype=torch.bfloat16, device="cuda") if tp else chain.logits
    logits_host = torch.empty(1, head.n * world, dtype=torch.bfloat16).pin_memory()
    allreduces_per_step = model.layers * sum(1 for p in projs if p.split == "row") if tp else 0

    peer_ar = None
    if tp and not args.nccl_allreduce:
        from inference_rs_b200.tensor_parallel import PeerSumAllReduce
        made = 1
        try:
            peer_ar = PeerSumAllReduce(capacity=1 << 16)
        except Exception as exc:  # no peer mappings on this machine: every rank falls back to NCCL together
            print(f"[bench] rank {rank}: peer-memory exchange unavailable ({type(exc).__name__}: {exc}); using NCCL", file=sys.stderr)
            made = 0
        agree = torch.tensor([made], device="cuda")
        dist.all_reduce(agree, op=dist.ReduceOp.MIN)
        if int(agree.item()) == 0:
            peer_ar = None
    fused_ok = {}  # projection index -> the fused matmul + exchange launch takes this shape (found out on the first, eager step)

    def row_parallel(i, p, w, x, o):
        if peer_ar is not None and not args.unfused_allreduce and fused_ok.get(i, True):
            try:
                peer_ar.gemv_sum(p.dtype, w, x, p.n, out=o)  # matmul + exchange in one launch
                return
            except pkg.KernelLibraryError:
                fused_ok[i] = False  # the same on every rank (same shapes): two launches for this projection
        ops.gemv(p.dtype, w, x, p.n, out=o)
        if peer_ar is not None:
            peer_ar.sum_all_reduce_(o)
        else:
            dist.all_reduce(o)

    def after_head():
        dist.all_gather_into_tensor(logits_all, chain.logits)

    def step():
        chain.step(row_parallel if tp else None, after_head if tp else None)

    stream = torch.cuda.Stream()
    torch.cuda.synchronize()

    # ---- tensor parallel: the exchange is checked on every rank count the bench runs at, before anything is timed: one
    # row-parallel matmul per shape through the path the step uses, against ops.gemv + an f32 NCCL all-reduce, and the
    # result must be the same bits on every rank
    tp_check = None
    if tp:
        tp_check = "ok"
        with torch.cuda.stream(stream):
            for i, p in enumerate(projs):
                if p.split != "row":
                    continue
                o = torch.empty(1, p.n, dtype=torch.bfloat16, device="cuda")
                row_parallel(i, p, chain.layers[0][i], chain.x_dev[p.k], o)
                part = ops.gemv(p.dtype, chain.layers[0][i], chain.x_dev[p.k], p.n).float()
                stream.synchronize()
                ref = part.clone()
                dist.all_reduce(ref)
                gathered = [torch.empty_like(o) for _ in range(world)]
                dist.all_gather(gathered, o)
                stream.synchronize()
                same_bits = all(torch.equal(gathered[0], t) for t in gathered)
                # partial outputs are rounded to bf16 before they are added (as the reference's all-reduce of bf16
                # tensors does), the sum once more: (world + 1) roundings of 2^-9 relative to the largest term
                tol = (world + 1) * 2.0 ** -9 * float(part.abs().max()) * world ** 0.5 + 2.0 ** -8 * float(ref.abs().max())
                err = float((o.float() - ref).abs().max())
                if not same_bits or not err <= tol:
                    tp_check = f"FAILED at {p.name}: max err {err:.4g} (tolerance {tol:.4g}), identical bits on all ranks: {same_bits}"
        flag = torch.tensor([1 if tp_check == "ok" else 0], device="cuda")
        dist.all_reduce(flag, op=dist.ReduceOp.MIN)
        if int(flag.item()) == 0 and tp_check == "ok":
            tp_check = "FAILED on another rank"

    with torch.cuda.stream(stream):
        step()  # first launch sets kernel attributes; must precede capture
        stream.synchronize()
        graph = None
        if not args.no_graph:
            try:
                graph = torch.cuda.CUDAGraph()
                with torch.cuda.graph(graph, stream=stream):
                    step()
            except Exception as exc:  # e.g. a collective that cannot be captured: run the step eagerly
                print(f"[bench] CUDA graph capture failed ({type(exc).__name__}: {exc}); running eagerly", file=sys.stderr)
                graph = None
                torch.cuda.synchronize()

        def run_step():
            if graph is not None:
                graph.replay()
            else:
                step()

        def barrier():
            torch.cuda.synchronize()
            if world > 1:
                dist.barrier()
            torch.cuda.synchronize()

        clocks = ClockSampler(local_rank)
        clocks.__enter__()
        for _ in range(args.warmup):
            run_step()
        barrier()
        ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        ev0.record(stream)
        for _ in range(args.steps):
            run_step()
        ev1.record(stream)
        barrier()
        ms = ev0.elapsed_time(ev1)
        if world > 1:
            t = torch.tensor([ms], device="cuda")
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        ms_per_step = ms / args.steps
        tok_s = 1000.0 / ms_per_step  # tensor parallel: all ranks work on the same token

        # ---- end to end: host buffers in, logits out, every step
        def e2e_step():
            for k in chain.ks:
                chain.x_dev[k].copy_(chain.x_host[k], non_blocking=True)
            run_step()
            logits_host.view(-1)[: logits_all.numel()].copy_(logits_all.view(-1), non_blocking=True)

        for _ in range(3):
            e2e_step()
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        for _ in range(args.steps):
            e2e_step()
            stream.synchronize()  # the caller reads the logits before the next token
        e1.record(stream)
        barrier()
        e2e_ms = e0.elapsed_time(e1)
        if world > 1:
            t = torch.tensor([e2e_ms], device="cuda")
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            e2e_ms = float(t.item())
        e2e_tok_s = 1000.0 * args.steps / e2e_ms
        h2d = sum(v.numel() * v.element_size() for v in chain.x_host.values())
        d2h = logits_host.numel() * logits_host.element_size()

        # ---- roofline of the dominant launch (largest share of the step's device time in the ncu launch list): the
        # ffn_gate + ffn_up GEMVs, one grouped launch per layer when grouping is on, timed alone over all layers'
        # distinct weights (2 GB, far beyond L2). The launch order is re-registered for this loop (each layer's launch is
        # followed by the next layer's) and put back afterwards.
        gate_idx = [i for i, p in enumerate(projs) if p.name in ("ffn_gate", "ffn_up")]
        gp = projs[gate_idx[0]]
        nl = min(model.layers, 32)
        if not args.no_group and len(gate_idx) == 2 and chain.groups:
            dom_kernel = "gemv_group_kernel<bf16, b=1> (ffn_gate + ffn_up, Q4_K)"
            dom_outs = [torch.empty(1, gp.n, dtype=torch.bfloat16, device="cuda") for _ in gate_idx]
            dom_list = [(lambda li=li: ops.gemv_group([gp.dtype, gp.dtype], [chain.layers[li][i] for i in gate_idx], chain.x_dev[gp.k],
                                                      [gp.n, gp.n], outs=dom_outs)) for li in range(nl)]
            dom_seq = [(chain.layers[li][gate_idx[1]], chain.layers[li][gate_idx[0]], gp.dtype, gp.k, gp.n) for li in range(nl)]
            dom_bytes = 2 * gp.weight_bytes + gp.k * 2 + 2 * gp.n * 2
            # dram__bytes_read.sum + dram__bytes_write.sum of one launch of this kernel at this shape (ncu capture
            # summarised in profiles/gemv_group_q4k_gate_up.txt)
            dom_traffic = NCU_TRAFFIC_GROUP_GATE_UP if (gp.k, gp.n) == (4096, 14336) else None
        else:
            dom_kernel = "gemv_staged_kernel<Q4_K, b=1, bf16>"
            dom_out = torch.empty(1, gp.n, dtype=torch.bfloat16, device="cuda")
            dom_w = [chain.layers[li][i] for li in range(nl) for i in gate_idx[:1 if tp else 2]]
            dom_list = [(lambda w=w: ops.gemv(gp.dtype, w, chain.x_dev[gp.k], gp.n, out=dom_out)) for w in dom_w]
            dom_seq = [(w, w, gp.dtype, gp.k, gp.n) for w in dom_w]
            dom_bytes = gp.weight_bytes + gp.k * 2 + gp.n * 2
            dom_traffic = NCU_TRAFFIC_GEMV_Q4K_4096_14336 if (gp.k, gp.n) == (4096, 14336) else None
        if not args.no_prefetch:
            register_launch_order(ops, dom_seq)
        dom_us = time_launch_list(torch, stream, dom_list, 10)
        if not args.no_prefetch:
            register_launch_order(ops, chain.launch_sequence())
        achieved = dom_bytes / (dom_us * 1e-6) / 1e9

        # ---- every other launch of a layer the same way (one GPU): each kind timed alone over the layers' distinct
        # weights, with its own algorithmic bytes. All of them are launches of the same kernel.
        by_launch = None
        if not tp and not args.shard_of:
            by_launch = []
            kinds = [[chain.projs[i] for i in g] for g in chain.groups] + [[p] for i, p in enumerate(chain.projs) if i not in chain.grouped]
            for members in kinds:
                idx = [chain.projs.index(p) for p in members]
                k0 = members[0].k
                outs_k = [torch.empty(1, p.n, dtype=torch.bfloat16, device="cuda") for p in members]
                if len(members) > 1:
                    fns = [(lambda li=li: ops.gemv_group([p.dtype for p in members], [chain.layers[li][i] for i in idx], chain.x_dev[k0],
                                                         [p.n for p in members], outs=outs_k)) for li in range(nl)]
                else:
                    fns = [(lambda li=li: ops.gemv(members[0].dtype, chain.layers[li][idx[0]], chain.x_dev[k0], members[0].n, out=outs_k[0]))
                           for li in range(nl)]
                seq_k = [(chain.layers[li][idx[-1]], chain.layers[li][idx[0]], members[0].dtype, k0, members[0].n) for li in range(nl)]
                if not args.no_prefetch:
                    register_launch_order(ops, seq_k)
                us_k = time_launch_list(torch, stream, fns, 10)
                nbytes = sum(p.weight_bytes for p in members) + k0 * 2 + sum(p.n for p in members) * 2
                by_launch.append({"launch": " + ".join(p.name for p in members), "types": "/".join(p.dtype.name for p in members),
                                  "k": k0, "n": [p.n for p in members], "us_per_launch": round(us_k, 2), "algorithmic_bytes": nbytes,
                                  "GBps": round(nbytes / us_k / 1e3, 1), "frac_of_measured_hbm": round(nbytes / us_k / 1e3 / peak, 3)})
            if not args.no_prefetch:
                register_launch_order(ops, chain.launch_sequence())
        clocks.__exit__(None, None, None)

        extras = not tp and not args.quick and not args.shard_of

        # ---- tensor parallel, the configuration's other two legs: decode at batch 32 and a 2048-token prefill through the
        # operator (QMatMul routes both to the tile GEMM), the [rows, hidden] sums of the row-parallel projections by NCCL
        # (512 KiB and 32 MiB: bandwidth-sized, beyond the peer kernel's capacity). Eager launches, CUDA events, max over ranks.
        tp_extra = None
        if tp and not args.quick:
            tp_extra = {}
            qms = [[pkg.QMatMul.from_qtensor(pkg.QTensor(w, p.dtype, (p.n, p.k))) for p, w in zip(projs, layer)] for layer in chain.layers]
            head_qm = pkg.QMatMul.from_qtensor(pkg.QTensor(chain.head_w, head.dtype, (head.n, head.k)))
            for label, rows, reps in (("decode_batch_32", 32, 5), ("prefill_2048", 2048, 2)):
                xs = {k: torch.randn(rows, k, device="cuda", generator=torch.Generator(device="cuda").manual_seed(k)).to(torch.bfloat16)
                      for k in chain.ks}

                def big_step():
                    for layer in qms:
                        for p, qm in zip(projs, layer):
                            y = qm.forward(xs[p.k])
                            if p.split == "row":
                                dist.all_reduce(y)
                    head_qm.forward(xs[head.k][-1:] if rows > 32 else xs[head.k])  # a prefill samples from its last token only

                big_step()
                barrier()
                b0, b1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                b0.record(stream)
                for _ in range(reps):
                    big_step()
                b1.record(stream)
                barrier()
                t = torch.tensor([b0.elapsed_time(b1) / reps], device="cuda")
                dist.all_reduce(t, op=dist.ReduceOp.MAX)
                ms_big = float(t.item())
                flops = 2.0 * rows * sum(p.n * p.k for p in projs) * model.layers
                tp_extra[label] = {"rows": rows, "ms_per_step": round(ms_big, 3), "tok_per_s": round(rows * 1000.0 / ms_big, 1),
                                   "TFLOPs_per_gpu": round(flops / (ms_big * 1e-3) / 1e12, 1),
                                   "allreduce": f"NCCL, {rows * model.hidden * 2 // 1024} KiB per sum"}
                del xs
            del qms, head_qm

        # ---- the element-wise-exact mode: the same chain with activations quantized to the CPU path's format (Q8_K /
        # Q8_0) in the kernel prologue, grouped and routed like the headline chain
        cpu_format = None
        if extras:
            ops.clear_weight_successors()
            exact = Chain(torch, pkg, ops, workloads, model, 1, 99, group=not args.no_group, act_quant=1, weights_of=chain)
            if not args.no_prefetch:
                register_launch_order(ops, exact.launch_sequence())
            ms_exact = time_chain(torch, stream, exact.step, max(3, args.steps // 4), 3)
            cpu_format = {"value": 1000.0 / ms_exact, "unit": UNIT, "ms_per_step": ms_exact, "launches_per_step": exact.launches_per_step,
                          "note": "act_quant=1: activations in the reference CPU path's Q8_K / Q8_0 format, element-wise within 1e-2 / 1e-3 of it; same grouping and kernel routing as the headline"}
            ops.clear_weight_successors()
            if not args.no_prefetch:
                register_launch_order(ops, chain.launch_sequence())

        prefill = None
        if extras:
            prefill = []
            gen = torch.Generator(device="cuda").manual_seed(76)
            for dt in (pkg.GgmlDType.Q4K, pkg.GgmlDType.Q6K):
                for (k, n) in workloads.SWEEP_SHAPES:
                    wq = random_blocks_device(torch, dt, n, k, gen)
                    for m in (512, 2048, 8192):
                        xm = torch.randn(m, k, device="cuda", generator=gen).to(torch.bfloat16)
                        ym = torch.empty(m, n, dtype=torch.bfloat16, device="cuda")
                        for _ in range(3):
                            ops.gemm(dt, wq, xm, n, out=ym)
                        barrier()
                        reps = 10 if m * n * k < 2e12 else 4
                        g0, g1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                        g0.record(stream)
                        for _ in range(reps):
                            ops.gemm(dt, wq, xm, n, out=ym)
                        g1.record(stream)
                        barrier()
                        us = g0.elapsed_time(g1) * 1000.0 / reps
                        tf = 2.0 * m * n * k / us / 1e6
                        prefill.append({"type": dt.name, "k": k, "n": n, "m": m, "us": round(us, 1), "TFLOPs": round(tf, 1),
                                        "frac_of_measured_bf16_peak": round(tf / bf16_peak, 3)})
                        del xm, ym
                    del wq

        small = None
        if extras:
            # the decode sweep's batch 4 and 16 through the operator (QMatMul picks the kernel): weights-only GB/s
            small = []
            gen = torch.Generator(device="cuda").manual_seed(77)
            from inference_rs_b200 import qmatmul as _qm
            for dt, k, n in ((pkg.GgmlDType.Q4K, 4096, 6144), (pkg.GgmlDType.Q4K, 4096, 28672), (pkg.GgmlDType.Q4K, 14336, 4096),
                             (pkg.GgmlDType.Q6K, 14336, 4096), (pkg.GgmlDType.Q6K, 4096, 128256)):
                wbytes = n * dt.row_bytes(k)
                copies = max(2, min(8, int(600e6 // wbytes) + 1))
                qms = [pkg.QMatMul.from_qtensor(pkg.QTensor(random_blocks_device(torch, dt, n, k, gen), dt, (n, k))) for _ in range(copies)]
                for b in (4, 16):
                    xb = torch.randn(b, k, device="cuda", generator=gen).to(torch.bfloat16)
                    qms[0].forward(xb)
                    us = time_launch_list(torch, stream, [(lambda q=q: q.forward(xb)) for q in qms], max(3, int(2e9 // (wbytes * copies))))
                    kern = ("gemv_tc" if _qm.prefers_tensor_core_rows(dt, b, n, k) else ("gemv" if b <= 8 else "gemm"))
                    small.append({"type": dt.name, "k": k, "n": n, "b": b, "kernel": kern, "us": round(us, 2),
                                  "GBps": round((wbytes + b * k * 2 + b * n * 2) / us / 1e3, 1),
                                  "frac_of_measured_hbm": round((wbytes + b * k * 2 + b * n * 2) / us / 1e3 / peak, 3)})
                del qms

        sweep = None
        if args.sweep:
            sweep = []
            gen = torch.Generator(device="cuda").manual_seed(78)
            for dt in (pkg.GgmlDType.Q4K, pkg.GgmlDType.Q6K, pkg.GgmlDType.Q8_0):
                for (k, n) in workloads.SWEEP_SHAPES:
                    wbytes = n * dt.row_bytes(k)
                    copies = max(2, min(8, int(600e6 // wbytes) + 1))
                    ws = [random_blocks_device(torch, dt, n, k, gen) for _ in range(copies)]
                    if not args.no_prefetch:
                        register_launch_order(ops, [(w, w, dt, k, n) for w in ws])
                    for b in (1, 4, 8):
                        xb = torch.randn(b, k, device="cuda", generator=gen).to(torch.bfloat16)
                        ob = torch.empty(b, n, dtype=torch.bfloat16, device="cuda")
                        iters = max(3, int(3e9 // (wbytes * copies)))
                        if not ops.gemv_plan(dt, k, n, b)["staged"]:
                            sweep.append({"type": dt.name, "k": k, "n": n, "b": b, "us": None, "GBps": None,
                                          "note": "activations do not fit beside the ring: two-launch path only"})
                            continue
                        us = time_launch_list(torch, stream, [(lambda w=w: ops.gemv(dt, w, xb, n, out=ob)) for w in ws], iters)
                        sweep.append({"type": dt.name, "k": k, "n": n, "b": b, "us": round(us, 2),
                                      "GBps": round((wbytes + b * k * 2 + b * n * 2) / us / 1e3, 1),
                                      "frac_of_measured_hbm": round((wbytes + b * k * 2 + b * n * 2) / us / 1e3 / peak, 3)})
                    for w in ws:
                        ops.set_weight_successor(w, None)
                    del ws

        gguf_trip = None
        if extras:
            try:
                gguf_trip = gguf_round_trip(torch, pkg, ops, chain)
            except Exception as exc:
                gguf_trip = {"unavailable": f"{type(exc).__name__}: {exc}"}

        ref_cuda = None
        if extras:
            try:
                ref_cuda = reference_cuda_numbers(torch, pkg, chain, stream, peak, bf16_peak, args.steps)
            except Exception as exc:
                ref_cuda = {"unavailable": f"{type(exc).__name__}: {exc}"}
        status = pkg.kernel_library.device_status()

    launches_per_step, bytes_per_step = chain.launches_per_step, chain.bytes_per_step

    # ---- strong-scaling base for the tensor-parallel curve (one GPU only): the full 70B chain on this GPU and one rank's
    # share of the 2- / 4- / 8-way split without any exchange (the compute-only floor of each N)
    tp_base = None
    if extras:
        chain.free()
        del chain
        torch.cuda.empty_cache()
        tp_base = []
        for sh in (1, 2, 4, 8):
            c70 = Chain(torch, pkg, ops, workloads, workloads.LLAMA3_70B, sh, 4321, group=True)
            if not args.no_prefetch:
                register_launch_order(ops, c70.launch_sequence())
            ms70 = time_chain(torch, stream, c70.step, 10 if sh == 1 else 20, 3)
            tp_base.append({"shard_of": sh, "ms_per_step": round(ms70, 4), "tok_per_s": round(1000.0 / ms70, 2),
                            "GB_per_step": round(c70.bytes_per_step / 1e9, 3), "launches": c70.launches_per_step,
                            "hbm_frac_of_measured": round(c70.bytes_per_step / (ms70 * 1e-3) / 1e9 / peak, 3)})
            c70.free()
            del c70
            torch.cuda.empty_cache()

    line = {
        "metric": METRIC, "value": tok_s, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "strong" if tp else "weak", "vs_baseline": None,
        "dtype": "int8 dot, f32 accumulate", "data": "synthetic",
        "config": {"workload": workload_name(model, world) if not args.shard_of else f"one rank's share of the {shards}-way split: " + workload_name(model, shards),
                   "launches_per_step": launches_per_step,
                   "weights_GB_per_token_and_gpu": round(bytes_per_step / 1e9, 3),
                   "l2": "inputs larger than L2: every step streams its GBs of distinct weights",
                   "parallelism": (f"tp{world}: column / row split, {allreduces_per_step} "
                                   f"{('peer-memory all-reduces fused into the row-parallel GEMVs (b200q_gemv_allreduce)' if not args.unfused_allreduce else 'peer-memory all-reduces (b200q_peer_allreduce)') if peer_ar is not None else 'NCCL all-reduces'} per token") if tp else "1 gpu",
                   "cuda_graph": graph is not None, "pdl": ops.get_option("pdl"),
                   "l2_prefetch_bytes": 0 if args.no_prefetch else ops.get_option("l2_prefetch_bytes"),
                   "grouped_launches": not args.no_group},
        "weights_GBps_per_gpu": bytes_per_step * tok_s / 1e9,
        "e2e": {"value": e2e_tok_s, "unit": UNIT, "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h},
        "gpu_launches": launches_per_step * args.steps,
        "roofline": {"bound": "hbm", "kernel": dom_kernel, "shape": f"K={gp.k} N={gp.n}",
                     "achieved": achieved, "peak": peak, "peak_source": peak_src, "unit": "GB/s", "frac": achieved / peak,
                     "us_per_launch": dom_us, "algorithmic_bytes": dom_bytes, "traffic": dom_traffic,
                     "traffic_note": "dram read + write of one launch under ncu with the L2 prefetch of the next matrix off; with it on, "
                                     "a launch also fetches up to 148 x l2_prefetch_bytes of the NEXT launch's rows, which that launch then "
                                     "does not read from DRAM: over a layer's four launches the DRAM traffic measured in the chain "
                                     "equals the algorithmic bytes (profiles/gemv_group_q4k_gate_up.txt)"},
        "clocks": clocks.summary(),
        "device_status": list(status),
    }
    line["hbm_frac_of_measured"] = line["weights_GBps_per_gpu"] / peak
    line["hbm_frac_of_nominal_8TBps"] = line["weights_GBps_per_gpu"] / 8000.0
    if by_launch is not None:
        line["roofline_by_launch"] = by_launch
    if tp_check is not None:
        line["tp_check"] = tp_check
    if tp_extra is not None:
        line["tp_other_legs"] = tp_extra
    if cpu_format is not None:
        line["cpu_format_activations"] = cpu_format
    if prefill is not None:
        line["prefill_gemm"] = prefill
    if small is not None:
        line["small_batch"] = small
    if sweep is not None:
        line["sweep"] = sweep
    if gguf_trip is not None:
        line["gguf_round_trip"] = gguf_trip
    if ref_cuda is not None:
        line["reference_cuda"] = ref_cuda
    if tp_base is not None:
        line["tp_base"] = tp_base
    if rank == 0 and not args.no_cpu_baseline:
        v, desc = cpu_chain_sample(model, host_threads())
        line["cpu_baseline"] = {"value": v, "unit": UNIT, "cores": host_threads(), "kind": "port", "sample": desc}
    if rank == 0:
        print(json.dumps(line), flush=True)
    failed = tp_check is not None and tp_check != "ok"
    if world > 1:
        # leave without tearing NCCL down: destroying a process group whose collectives were captured into a CUDA graph
        # can block at exit, and nothing is left to flush
        torch.cuda.synchronize()
        dist.barrier()
        sys.stdout.flush()
        sys.stderr.flush()
        os._exit(1 if failed else 0)
    if failed:
        raise SystemExit(1)


if __name__ == "__main__":
    main()
