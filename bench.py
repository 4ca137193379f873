"""Benchmark of the quantized decode path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload NAME] [--impl reference]

Prints ONE JSON line (rank 0). Workloads:

  decode_8b       (default) BASELINE config 5: random-init Llama-3-8B, attention int8, MLP int4
                  (group 128), lm_head int8, int8 KV cache, batch 1, 4096-token uniform-random
                  prompt, greedy decode. A step is one decoded token through the fused decoder
                  (one CUDA-graph replay). value = decoded tokens per second.
  decode_1b       BASELINE config 3: the same for the Llama-3.2-1B shape, 512-token prompt.

  gemv_one / attn_one / prefill_gemm
                  one GEMV shape, one attention shape, the prefill GEMM shapes (BASELINE config 4):
                  the small cases kernel profiles are taken on; each prints its own JSON line.

  gemv_sweep_1b   BASELINE config 2: the Llama-3.2-1B linear shapes at M=1 (q/o, k/v, gate/up,
                  down as int4 and int8, lm_head int8), bf16 activations, group 128. A step is
                  one pass over a pool of distinct weight copies of every shape (the pool of
                  each shape exceeds L2, so every launch streams from HBM). value = algorithmic
                  bytes moved per second over the whole pass.

`--impl reference` times the reference's own real mode on the host cores -- the staged copy of
the reference package under oracle/_ref when it is there (`python oracle/make_ref.py`), else
the oracle's restatement of it -- on a bounded sample of the same workload, on all host threads.
"""

import argparse
import ctypes
import json
import os
import subprocess
import sys
import tempfile
import threading
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

L2_BYTES = 126 * 1024 * 1024

# (name, N, K, bits) -- BASELINE config 2
SWEEP_1B = [
    ("q_o.int4", 2048, 2048, 4), ("k_v.int4", 512, 2048, 4), ("gate_up.int4", 8192, 2048, 4),
    ("down.int4", 2048, 8192, 4),
    ("q_o.int8", 2048, 2048, 8), ("k_v.int8", 512, 2048, 8), ("gate_up.int8", 8192, 2048, 8),
    ("down.int8", 2048, 8192, 8),
    ("lm_head.int8", 128256, 2048, 8),
]


# The same projections as a decode step launches them: q|k|v and gate|up as one weight each. Timed
# and reported next to the sweep (not part of its aggregate: BASELINE config 2 names the single shapes).
SWEEP_1B_FUSED = [("qkv.int8", 3072, 2048, 8), ("gate_up.int4", 16384, 2048, 4), ("gate_up.int8", 16384, 2048, 8)]


def algorithmic_bytes(n, k, bits, m=1, out_bytes=2):
    """Packed codes + one fp32 scale per (row, group of 128) + bf16 x + the output."""
    return n * k * bits // 8 + n * (-(-k // 128)) * 4 + m * k * 2 + m * n * out_bytes


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as fh:
            return json.load(fh), "measured"
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}, "fallback"


class ClockSampler:
    """nvidia-smi clocks / throttle reasons sampled every 200 ms while the timed region runs."""

    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
             "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index = index
        self.proc = None
        self.path = None

    def __enter__(self):
        try:
            fd, self.path = tempfile.mkstemp(suffix=".csv")
            os.close(fd)
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits",
                 "-lms", "200", "-i", str(self.index)],
                stdout=open(self.path, "w"), stderr=subprocess.DEVNULL)
        except OSError:
            self.proc = None
        return self

    def __exit__(self, *exc):
        if self.proc is not None:
            time.sleep(0.25)
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()

    def summary(self):
        out = {"sm_mhz": None, "sm_max_mhz": None, "reasons": []}
        if not self.path or not os.path.exists(self.path):
            return out
        sm, reasons = [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        with open(self.path) as fh:
            for line in fh:
                cols = [c.strip() for c in line.split(",")]
                if len(cols) < 9:
                    continue
                try:
                    sm.append(float(cols[1]))
                    out["sm_max_mhz"] = float(cols[2])
                except ValueError:
                    continue
                for name, col in zip(names, cols[5:9]):
                    if col.lower().startswith("active"):
                        reasons.add(name)
        os.unlink(self.path)
        if sm:
            sm.sort()
            out["sm_mhz"] = sm[len(sm) // 2]
        out["reasons"] = sorted(reasons)
        return out


# --------------------------------------------------------------------------- GPU arm
def build_pool(device, shapes=None):
    """For every shape: enough distinct quantized copies to exceed twice the L2 size."""
    from llmquant_b200.core import QuantizationArgs, QuantizationScheme
    from llmquant_b200.quantizers import KernelQuantLinear

    pool = []
    for name, n, k, bits in (shapes or SWEEP_1B):
        scheme = QuantizationScheme(
            weights=QuantizationArgs(num_bits=bits, strategy="group", group_size=128),
            input_activations=None)
        g = torch.Generator(device="cpu").manual_seed(len(pool))
        per_copy = algorithmic_bytes(n, k, bits)
        copies = max(2, -(-2 * L2_BYTES // per_copy))
        # two distinct random weights, cloned to fill the pool (values do not affect speed)
        base = []
        for _ in range(2):
            w = (torch.randn(n, k, generator=g) * 0.02).to(torch.bfloat16).to(device)
            lin = torch.nn.Linear(k, n, bias=False, device="meta")
            lin.weight = torch.nn.Parameter(w, requires_grad=False)
            base.append(KernelQuantLinear.from_linear(lin, scheme))
            del w, lin
        weights = [(m.codes, m.scale_tiles) for m in base]
        while len(weights) < copies:
            src = base[len(weights) % 2]
            weights.append((src.codes.clone(), src.scale_tiles.clone()))
        x = (torch.randn(1, k, generator=g)).to(torch.bfloat16).to(device)
        pool.append({"name": name, "n": n, "k": k, "bits": bits, "mod": base[0], "weights": weights,
                     "x": x, "bytes": per_copy})
    return pool


def capture_shape_graph(entry):
    """One CUDA graph that launches the GEMV once per weight copy of this shape."""
    x = entry["x"]
    outs = [torch.empty(1, entry["n"], dtype=torch.bfloat16, device=x.device) for _ in entry["weights"]]
    entry["outs"] = outs
    mod = entry["mod"]

    def run():
        from llmquant_b200 import native
        for (codes, scale_tiles), out in zip(entry["weights"], outs):
            # programmatic dependent launch: a launch streams its first weights while the one
            # before it drains, as consecutive linears of a decode step do
            a = native.GemvArgs(x=x.data_ptr(), ldx=x.stride(0), codes=codes.data_ptr(),
                                scale_tiles=scale_tiles.data_ptr(), out=out.data_ptr(),
                                out_dtype=native.LQ_BF16, M=1, N=mod.out_features, K=mod.in_features,
                                Kd=mod._kd, span=mod._span, bits=mod.num_bits, pdl=1)
            native.call("lq_wq_gemv_fused", ctypes.byref(a), native.stream_ptr(x.device))

    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        run()
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        run()
    entry["graph"] = graph


def run_gpu(args, rank, world, device):
    import torch.distributed as dist

    pool = build_pool(device)
    for entry in pool:
        capture_shape_graph(entry)
    launches_per_step = sum(len(e["weights"]) for e in pool)
    bytes_per_step = sum(e["bytes"] * len(e["weights"]) for e in pool)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(args.warmup):
        for entry in pool:
            entry["graph"].replay()
    barrier()

    # ---- value: inputs resident in HBM, one event pair per shape per step
    events = [[(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True))
               for _ in pool] for _ in range(args.steps)]
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with ClockSampler(torch.cuda.current_device()) as clocks:
        barrier()
        start.record()
        for s in range(args.steps):
            for entry, (e0, e1) in zip(pool, events[s]):
                e0.record()
                entry["graph"].replay()
                e1.record()
        stop.record()
        barrier()
    total_ms = start.elapsed_time(stop)
    shape_ms = [sum(events[s][i][0].elapsed_time(events[s][i][1]) for s in range(args.steps)) / args.steps
                for i in range(len(pool))]
    kernel_ms = sum(shape_ms)

    # ---- e2e: the module call a user makes, x from pinned host memory, y read back
    host_x = [e["x"].cpu().pin_memory() for e in pool]
    host_y = [torch.empty(1, e["n"], dtype=torch.bfloat16).pin_memory() for e in pool]
    h2d = sum(x.numel() * 2 for x in host_x)
    d2h = sum(y.numel() * 2 for y in host_y)

    def e2e_step(step):
        for i, entry in enumerate(pool):
            xd = host_x[i].to(device, non_blocking=True)
            host_y[i].copy_(entry["mod"](xd), non_blocking=True)
        torch.cuda.synchronize()

    for s in range(max(3, args.warmup)):
        e2e_step(s)
    barrier()
    t0 = time.perf_counter()
    for s in range(args.steps):
        e2e_step(s)
    barrier()
    e2e_s = (time.perf_counter() - t0) / args.steps
    e2e_bytes = sum(e["bytes"] for e in pool)

    times = torch.tensor([total_ms, kernel_ms, e2e_s], dtype=torch.float64, device=device)
    if world > 1:
        dist.all_reduce(times, op=dist.ReduceOp.MAX)
    total_ms, kernel_ms, e2e_s = times.tolist()
    ms_per_step = total_ms / args.steps
    peaks, peak_kind = measured_peaks()

    value = world * bytes_per_step / (ms_per_step * 1e-3) / 1e9
    achieved = bytes_per_step / (kernel_ms * 1e-3) / 1e9
    line = {
        "metric": "quant_gemv_hbm_gbs", "value": round(value, 1), "unit": "GB/s",
        "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": round(ms_per_step, 4), "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "int4/int8 codes x bf16, fp32 accumulate", "data": "synthetic",
        "config": {"workload": "gemv_sweep_1b (BASELINE config 2: Llama-3.2-1B linear shapes, M=1)",
                   "group_size": 128, "launches_per_step": launches_per_step,
                   "l2_policy": "each shape cycles a pool of distinct weight copies > 2x L2",
                   "parallelism": f"replicas x{world}" if world > 1 else "single"},
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": peaks["hbm_gbs"],
                     "unit": "GB/s", "frac": round(achieved / peaks["hbm_gbs"], 4),
                     "frac_of_nominal_8TBs": round(achieved / 8000.0, 4), "peak_kind": peak_kind,
                     "traffic": None, "kernel": "gemv_stream_kernel"},
        "shapes": {e["name"]: {"us_per_launch": round(ms * 1e3 / len(e["weights"]), 3),
                               "gbs": round(e["bytes"] * len(e["weights"]) / (ms * 1e-3) / 1e9, 1),
                               "frac": round(e["bytes"] * len(e["weights"]) / (ms * 1e-3) / 1e9 / peaks["hbm_gbs"], 4)}
                   for e, ms in zip(pool, shape_ms)},
        "e2e": {"value": round(world * e2e_bytes / e2e_s / 1e9, 2), "unit": "GB/s",
                "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h},
        "gpu_launches": launches_per_step * args.steps,
        "clocks": clocks.summary(),
    }
    # the fused projections of a decode step, the same way (after the timed region)
    del pool
    torch.cuda.empty_cache()
    fused = build_pool(device, SWEEP_1B_FUSED)
    line["fused_shapes"] = {}
    for entry in fused:
        capture_shape_graph(entry)
        for _ in range(3):
            entry["graph"].replay()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(args.steps):
            entry["graph"].replay()
        e1.record()
        torch.cuda.synchronize()
        us = e0.elapsed_time(e1) * 1e3 / (args.steps * len(entry["weights"]))
        line["fused_shapes"][entry["name"]] = {"us_per_launch": round(us, 3), "gbs": round(entry["bytes"] / us / 1e3, 1),
                                               "frac": round(entry["bytes"] / us / 1e3 / peaks["hbm_gbs"], 4)}
    if rank == 0:
        if world == 1 and not args.skip_cpu_baseline:
            line["cpu_baseline"] = cpu_baseline(sample_seconds=12.0)
        print(json.dumps(line), flush=True)


# --------------------------------------------------------------------------- one GEMV shape
def run_gemv_one(args, device):
    """One shape, a few weight copies (> L2 together), back-to-back launches: the small case
    used for kernel profiles. Prints a short JSON line of its own."""
    from llmquant_b200.core import QuantizationArgs, QuantizationScheme
    from llmquant_b200.quantizers import KernelQuantLinear

    n, k, bits = args.n, args.k, args.bits
    scheme = QuantizationScheme(
        weights=QuantizationArgs(num_bits=bits, strategy="group", group_size=128), input_activations=None)
    per_copy = algorithmic_bytes(n, k, bits)
    copies = max(2, -(-int(1.5 * L2_BYTES) // per_copy))
    g = torch.Generator(device=device).manual_seed(0)
    mods = []
    for _ in range(copies):
        w = (torch.randn(n, k, generator=g, device=device) * 0.02).to(torch.bfloat16)
        lin = torch.nn.Linear(k, n, bias=False, device="meta")
        lin.weight = torch.nn.Parameter(w, requires_grad=False)
        mods.append(KernelQuantLinear.from_linear(lin, scheme))
        del w, lin
    x = torch.randn(args.batch, k, generator=g, device=device).to(torch.bfloat16)
    gamma = torch.ones(k, dtype=torch.bfloat16, device=device) if args.norm else None
    n_out = n // 2 if args.epilogue else n
    out = torch.empty(args.batch, n_out, dtype=torch.bfloat16, device=device)

    def once():
        for m in mods:
            m.gemv(x, norm_weight=gamma, epilogue=args.epilogue, pdl=True, out=out)

    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        for _ in range(args.warmup):
            once()
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        once()
    graph.replay()
    torch.cuda.synchronize()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for _ in range(args.steps):
        graph.replay()
    stop.record()
    torch.cuda.synchronize()
    us = start.elapsed_time(stop) * 1e3 / (args.steps * copies)
    print(json.dumps({"workload": "gemv_one", "n": n, "k": k, "bits": bits, "rows": args.batch,
                      "copies": copies, "us_per_launch": round(us, 2),
                      "gbs": round(per_copy / us / 1e3, 1), "graph_replay": True}), flush=True)


# --------------------------------------------------------------------------- one attention shape
def run_attn_one(args, device):
    """The fused decode-attention block by itself at one shape and context (the small case for
    kernel profiles): `layers` caches of random codes (together larger than L2), one launch per
    cache in a CUDA graph with dependent launches. Prints a short JSON line of its own."""
    from llmquant_b200 import native

    lib = native.library()
    B, D, T = args.batch, args.head_dim, args.prompt or 4111
    Hq, Hkv = args.heads, args.kv_heads
    tmax = T + 64
    per_layer = 2 * B * Hkv * T * (D + 4)
    layers = max(2, -(-int(1.5 * L2_BYTES) // per_layer))
    g = torch.Generator(device=device).manual_seed(0)
    caches = []
    for _ in range(layers):
        kc = torch.randint(-127, 128, (B, Hkv, tmax, D), dtype=torch.int8, device=device, generator=g)
        vc = torch.randint(-127, 128, (B, Hkv, tmax, D), dtype=torch.int8, device=device, generator=g)
        ks = torch.rand(B, Hkv, tmax, 1, device=device, generator=g) * 0.02 + 0.001
        vs = torch.rand(B, Hkv, tmax, 1, device=device, generator=g) * 0.02 + 0.001
        caches.append((kc, vc, ks, vs))
    qkv = torch.randn(B, (Hq + 2 * Hkv) * D, device=device, generator=g).to(torch.bfloat16)
    cos = torch.randn(tmax, D, device=device, generator=g).to(torch.bfloat16)
    sin = torch.randn(tmax, D, device=device, generator=g).to(torch.bfloat16)
    out = torch.zeros(B, Hq, D, dtype=torch.bfloat16, device=device)
    pos = torch.tensor([T], dtype=torch.long, device=device)
    splits = args.splits or max(1, 2 * 148 // (B * Hkv))
    nbytes = lib.lq_attn_fused_scratch_bytes(B, Hq, Hkv, D, splits)
    scratch = torch.zeros(-(-nbytes // 4), dtype=torch.float32, device=device)

    def once():
        stream = native.stream_ptr(device)
        for kc, vc, ks, vs in caches:
            native.call("lq_attn_decode_fused", qkv.data_ptr(), cos.data_ptr(), sin.data_ptr(), kc.data_ptr(),
                        vc.data_ptr(), ks.data_ptr(), vs.data_ptr(), out.data_ptr(), scratch.data_ptr(), B, Hq,
                        Hkv, D, tmax, tmax, pos.data_ptr(), 0, 8, D ** -0.5, splits, args.attn_impl, 1, stream)

    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        for _ in range(args.warmup):
            once()
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        once()
    graph.replay()
    torch.cuda.synchronize()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for _ in range(args.steps):
        graph.replay()
    stop.record()
    torch.cuda.synchronize()
    us = start.elapsed_time(stop) * 1e3 / (args.steps * layers)
    peaks, _ = measured_peaks()
    print(json.dumps({"workload": "attn_one", "batch": B, "heads": Hq, "kv_heads": Hkv, "head_dim": D,
                      "context": T, "slices": splits, "impl": args.attn_impl, "caches": layers,
                      "us_per_launch": round(us, 2), "algorithmic_bytes": per_layer,
                      "gbs": round(per_layer / us / 1e3, 1),
                      "frac_of_measured_hbm_peak": round(per_layer / us / 1e3 / peaks["hbm_gbs"], 4),
                      "device_error": lib.lq_attn_device_error()}), flush=True)


# --------------------------------------------------------------------------- prefill GEMM shapes
def run_gemm_sweep(args, device):
    """BASELINE config 4: W4 group-128 weights at the Llama-3-8B shapes, M in {16, 128, 512, 2048},
    bf16 activations quantized per token per group to int8 (A8) and left in bf16 (A16); the
    tensor-core GEMM next to the reference's own choice (dequantize to bf16 + library GEMM)."""
    from llmquant_b200.core import QuantizationArgs, QuantizationScheme
    from llmquant_b200.quantizers import KernelQuantLinear

    shapes = [("q_o", 4096, 4096), ("k_v", 1024, 4096), ("gate_up", 14336, 4096), ("down", 4096, 14336)]
    scheme = QuantizationScheme(
        weights=QuantizationArgs(num_bits=args.bits, strategy="group", group_size=128), input_activations=None)
    g = torch.Generator(device=device).manual_seed(0)
    peaks, peak_kind = measured_peaks()
    rows = []

    def timed(fn):
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(args.steps):
            fn()
        b.record()
        torch.cuda.synchronize()
        return a.elapsed_time(b) / args.steps

    for name, n, k in shapes:
        w = (torch.randn(n, k, generator=g, device=device) * 0.02).to(torch.bfloat16)
        lin = torch.nn.Linear(k, n, bias=False, device="meta")
        lin.weight = torch.nn.Parameter(w, requires_grad=False)
        mod = KernelQuantLinear.from_linear(lin, scheme)
        del w, lin
        for m in ([int(v) for v in args.rows.split(',')] if args.rows else (16, 128, 512, 2048)):
            x = torch.randn(m, k, generator=g, device=device).to(torch.bfloat16)
            flops = 2.0 * m * n * k
            t8 = timed(lambda: mod.gemm(x, a8=True))
            t16 = timed(lambda: mod.gemm(x, fold_scales=True))
            t16x = timed(lambda: mod.gemm(x))
            tlib = timed(lambda: x @ mod._dequantized_weight(torch.bfloat16).T)
            tfwd = timed(lambda: mod(x))  # the module's own choice at this row count
            rows.append({"shape": name, "M": m, "N": n, "K": k, "forward_tflops": round(flops / tfwd / 1e9, 1),
                         "forward_ms": round(tfwd, 4),
                         "a8_tflops": round(flops / t8 / 1e9, 1), "a16_tflops": round(flops / t16 / 1e9, 1),
                         "a16_exact_tflops": round(flops / t16x / 1e9, 1),
                         "dequant_plus_library_tflops": round(flops / tlib / 1e9, 1),
                         "a8_ms": round(t8, 4), "a16_ms": round(t16, 4), "dequant_plus_library_ms": round(tlib, 4)})
    best = max(r["a8_tflops"] for r in rows)  # (`forward` may be the library GEMM at large row counts)
    print(json.dumps({"workload": "prefill_gemm (BASELINE config 4)", "bits": args.bits, "rows": rows,
                      "roofline": {"bound": "tensor", "achieved": best, "peak": peaks["bf16_tflops"],
                                   "unit": "TFLOP/s", "frac": round(best / peaks["bf16_tflops"], 4),
                                   "peak_kind": peak_kind + " bf16 cuBLAS burst"}}), flush=True)


# --------------------------------------------------------------------------- decode workload
DECODE = {
    "decode_8b": dict(shape="llama-3-8b", prompt=4096, label="BASELINE config 5: random-init Llama-3-8B"),
    "decode_1b": dict(shape="llama-3.2-1b", prompt=512, label="BASELINE config 3: random-init Llama-3.2-1B"),
}


def decode_step_bytes(dec, context):
    """Algorithmic HBM bytes of one decoded token: packed codes + scales of every linear, the
    int8 K and V rows and their scales read by attention, the embedding row."""
    total = 0
    for spec in dec.layers:
        for key in ("qkv", "o", "gate_up", "down"):
            total += spec[key].weight_bytes()
    if hasattr(dec.lm_head, "weight_bytes"):
        total += dec.lm_head.weight_bytes()
    else:
        total += dec.lm_head.weight.numel() * 2
    kv = 2 * dec.B * dec.Hkv * context * (dec.D + 4)
    return total + kv * len(dec.layers) + dec.B * dec.hidden * 2


def decode_margins(dec, ids, n):
    """Top-2 logit margin (bf16 logits, sequence 0) of the first `n` generated tokens, decoded
    again from the prompt with eager launches and the logits gathered on every rank."""
    dec.use_graph, dec.graph, dec.gather_logits = False, None, True
    dec.prefill(ids)
    margins = []
    for i in range(n):
        top = dec.logits[0].float().topk(2).values
        margins.append(round(float(top[0] - top[1]), 4))
        if i + 1 < n:
            dec.step()
    return margins


def decode_at_batch(model, batch, prompt, host_ids, device, steps=8, warmup=3):
    """Greedy decode of `batch` sequences (the first sequence's prompt, rotated, for each) with
    the fused decoder: prefill, graph capture, `warmup` steps, `steps` timed steps."""
    from llmquant_b200.runtime.decoder import FusedLlamaDecoder

    dec = FusedLlamaDecoder(model, batch, prompt + warmup + steps + 16, kv_bits=8)
    ids = torch.stack([torch.roll(host_ids[0], shifts=i) for i in range(batch)]).to(device)
    # the prompt goes through the transformers modules: in chunks of sequences to bound memory
    dec.prefill(ids) if batch <= 8 else prefill_in_chunks(dec, ids, 8)
    dec.capture()
    for _ in range(warmup):
        dec.step()
    torch.cuda.synchronize()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(steps):
        dec.step()
    b.record()
    torch.cuda.synchronize()
    ms = a.elapsed_time(b) / steps
    context = prompt + warmup + steps // 2
    out = {"tok_per_s": round(batch / (ms * 1e-3), 1), "ms_per_step": round(ms, 3), "steps": steps,
           "context": context, "launches_per_linear": 3 if dec.decode_gemm else 1,
           "kv_bytes_per_step": 2 * batch * dec.Hkv * context * (dec.D + 4) * len(dec.layers)}
    dec.check_device_errors()
    del dec
    torch.cuda.empty_cache()
    return out


def prefill_in_chunks(dec, ids, chunk):
    """Prefill a large batch a few sequences at a time: each chunk runs through the model with a
    cache of its own, whose integer rows are then copied into the decoder's cache."""
    from llmquant_b200.quantizers import KernelQuantCache

    batch, prompt = ids.shape
    dec._begin_sequence()
    firsts = []
    full = None
    for b0 in range(0, batch, chunk):
        part = KernelQuantCache(dec.kv_bits, max_cache_len=dec.max_len)
        with torch.no_grad():
            out = dec.model(ids[b0:b0 + chunk], past_key_values=part, use_cache=True, logits_to_keep=1)
        firsts.append(out.logits[:, -1].argmax(-1))
        if full is None:
            full = [dict(k=torch.zeros(batch, *l.k_codes.shape[1:], dtype=torch.int8, device=ids.device),
                         v=torch.zeros(batch, *l.v_codes.shape[1:], dtype=torch.int8, device=ids.device),
                         ks=torch.zeros(batch, *l.k_scales.shape[1:], device=ids.device),
                         vs=torch.zeros(batch, *l.v_scales.shape[1:], device=ids.device)) for l in part.layers]
        for dst, l in zip(full, part.layers):
            dst["k"][b0:b0 + chunk], dst["v"][b0:b0 + chunk] = l.k_codes, l.v_codes
            dst["ks"][b0:b0 + chunk], dst["vs"][b0:b0 + chunk] = l.k_scales, l.v_scales
        del part, out
    # hand the assembled rows to the decoder's cache layers
    proto = torch.zeros(batch, dec.Hkv, 1, dec.D, dtype=torch.bfloat16, device=ids.device)
    while len(dec.cache.layers) < len(dec.layers):
        dec.cache.layers.append(dec.cache.layer_class_to_replicate())
    for layer, src in zip(dec.cache.layers, full):
        if not layer.is_initialized:
            layer.lazy_initialization(proto, proto)
        layer.k_codes, layer.v_codes, layer.k_scales, layer.v_scales = src["k"], src["v"], src["ks"], src["vs"]
        layer.capacity, layer.length = src["k"].shape[2], prompt
    first = torch.cat(firsts)
    dec.tokens.copy_(first)
    dec.pos.fill_(prompt)
    dec.history.zero_()
    dec.history[:, :prompt] = ids
    dec.history[:, prompt] = first


def run_decode(args, rank, world, device):
    import torch.distributed as dist

    from llmquant_b200.core import QuantConfig
    from llmquant_b200.runtime.decoder import FusedLlamaDecoder
    from llmquant_b200.runtime.random_init import llama_config, random_quantized_llama

    from llmquant_b200.runtime import tp as tpmod

    spec = DECODE[args.workload]
    batch, prompt = args.batch, args.prompt or spec["prompt"]
    quant = QuantConfig(attn_weight="int8", mlp_weight="int4", head_weight="int8", kv_cache="int8")
    config = llama_config(spec["shape"])
    ctx = tpmod.TPContext(rank, world) if world > 1 else None
    if ctx:
        tpmod.check_divisible(config, world)
        ctx.peer_allreduce = args.allreduce == "peer"
    # every rank draws the same full weights (same seed) and keeps its slice
    model = random_quantized_llama(
        config, quant, device, seed=0,
        shard=(lambda name, w: tpmod.shard_weight(name, w, rank, world)) if ctx else None)
    if ctx:
        tpmod.wrap_for_prefill_(model, ctx)
    new = args.warmup + 2 * args.steps + 16
    dec = FusedLlamaDecoder(model, batch, prompt + new + 8, kv_bits=8, tp=ctx)
    g = torch.Generator().manual_seed(1)
    host_ids = torch.randint(0, model.config.vocab_size, (batch, prompt), generator=g).pin_memory()

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # the prompt goes through the transformers modules: a large batch in chunks of sequences
    dev_ids = host_ids.to(device, non_blocking=True)
    dec.prefill(dev_ids) if batch <= 8 else prefill_in_chunks(dec, dev_ids, 8)
    dec.capture()
    for _ in range(args.warmup):
        dec.step()
    barrier()

    # ---- value: the token loop entirely on the device
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    cursor = dec.pos.clone()
    with ClockSampler(torch.cuda.current_device()) as clocks:
        barrier()
        start.record()
        for _ in range(args.steps):
            dec.step()
        stop.record()
        barrier()
    step_ms = start.elapsed_time(stop) / args.steps
    context = prompt + args.warmup + args.steps // 2
    # what was decoded: every rank count must give the same stream (greedy, same weights)
    produced = dec.history[:, prompt:prompt + args.warmup + args.steps + 1].cpu()
    checksum = 0
    for t in produced.flatten().tolist():
        checksum = (checksum * 1000003 + int(t) + 1) % 2305843009213693951

    # ---- spread: the same K steps from the same cursor, five more times
    repeats = []
    for _ in range(5):
        dec.pos.copy_(cursor)
        barrier()
        r0, r1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        r0.record()
        for _ in range(args.steps):
            dec.step()
        r1.record()
        barrier()
        repeats.append(r0.elapsed_time(r1) / args.steps)

    # ---- e2e: every step feeds the token from pinned host memory and reads the new one back
    host_tok = dec.tokens.cpu().pin_memory()
    for _ in range(3):
        dec.tokens.copy_(host_tok, non_blocking=True)
        dec.step()
        host_tok.copy_(dec.tokens, non_blocking=True)
        torch.cuda.synchronize()
    barrier()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        dec.tokens.copy_(host_tok, non_blocking=True)
        dec.step()
        host_tok.copy_(dec.tokens, non_blocking=True)
        torch.cuda.synchronize()
    barrier()
    e2e_s = (time.perf_counter() - t0) / args.steps

    # ---- the dominant kernel by itself: every GEMV launch of a step (4 per layer + lm_head),
    # same fusions and buffers, captured as one graph and timed with CUDA events
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        dec.gemv_launches()
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()
    gemv_graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(gemv_graph):
        dec.gemv_launches()
    for _ in range(3):
        gemv_graph.replay()
    barrier()
    g0, g1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    g0.record()
    for _ in range(args.steps):
        gemv_graph.replay()
    g1.record()
    barrier()
    gemv_ms = g0.elapsed_time(g1) / args.steps
    gemv_launches = 4 * len(dec.layers) + 1

    times = torch.tensor([step_ms, e2e_s, gemv_ms] + repeats, dtype=torch.float64, device=device)
    if world > 1:
        dist.all_reduce(times, op=dist.ReduceOp.MAX)
    step_ms, e2e_s, gemv_ms, *repeats = times.tolist()
    repeats.sort()
    peaks, peak_kind = measured_peaks()
    step_bytes = decode_step_bytes(dec, context)
    step_achieved = step_bytes / (step_ms * 1e-3) / 1e9
    gemv_bytes = dec.gemv_bytes()
    achieved = gemv_bytes / (gemv_ms * 1e-3) / 1e9
    line = {
        "metric": "decode_tokens_per_s", "value": round(batch / (step_ms * 1e-3), 1),
        "unit": "tok/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": round(step_ms, 4), "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "int4/int8 codes x bf16, fp32 accumulate", "data": "synthetic",
        "config": {"workload": f"{args.workload} ({spec['label']}, attn int8 / mlp int4 g128 / "
                               f"lm_head int8 / int8 KV, greedy)",
                   "batch": batch, "prompt_tokens": prompt, "context_at_timing": context,
                   "first_tokens": produced[0, :8].tolist(), "token_checksum": checksum,
                   "tokens_checked": int(produced.numel()),
                   "l2_policy": f"{step_bytes / 1e6:.0f} MB of weights and KV streamed per step, larger than L2",
                   "parallelism": (f"tp{world}: column-parallel q/k/v, gate/up, lm_head; row-parallel "
                                   f"o_proj, down_proj, all-reduce = {dec.allreduce}") if world > 1 else "single"},
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": peaks["hbm_gbs"],
                     "unit": "GB/s", "frac": round(achieved / peaks["hbm_gbs"], 4),
                     "frac_of_nominal_8TBs": round(achieved / 8000.0, 4), "peak_kind": peak_kind,
                     # DRAM bytes per launch as one ncu capture of two shapes gave them: 1.006x
                     # (lm_head, int8) and 1.03x (gate|up, int4) the algorithmic bytes
                     "traffic": int(gemv_bytes * 1.02) // gemv_launches,
                     "traffic_source": "ncu captures of two shapes (1.006x and 1.03x algorithmic), scaled",
                     "kernel": (f"{'decode_gemm_kernel (with its planes and finish launches)' if dec.decode_gemm else 'gemv_stream_kernel'}"
                                f", the {gemv_launches} linears of one step timed alone as a graph (per GPU); "
                                f"achieved / traffic are per linear on average"),
                     "algorithmic_bytes_per_launch": gemv_bytes // gemv_launches,
                     "us_per_launch": round(gemv_ms * 1e3 / gemv_launches, 2),
                     "share_of_step": round(gemv_ms / step_ms, 3),
                     "whole_step": {"bytes": step_bytes, "achieved": round(step_achieved, 1),
                                    "frac": round(step_achieved / peaks["hbm_gbs"], 4)}},
        "e2e": {"value": round(batch / e2e_s, 1), "unit": "tok/s",
                "h2d_bytes_per_step": batch * 8, "d2h_bytes_per_step": batch * 8},
        "spread": {"repeats": len(repeats), "ms_per_step_median": round(repeats[len(repeats) // 2], 4),
                   "ms_per_step_min": round(repeats[0], 4), "ms_per_step_max": round(repeats[-1], 4)},
        "gpu_launches": dec.launches_per_step * args.steps,
        "clocks": clocks.summary(),
    }
    dec.check_device_errors()  # a bounded wait that ran out anywhere in the step voids the run
    # the same stream once more with the full logits at hand (gathered over the ranks): the
    # top-2 margin of every step, so that streams decoded on different numbers of GPUs can be
    # compared -- where they part, the margin says whether a near-tie decided it
    line["config"]["tokens"] = produced[0].tolist()
    line["config"]["top2_margin"] = decode_margins(dec, host_ids.to(device), produced.shape[1])
    if world == 1 and batch == 1 and args.workload == "decode_8b" and not args.no_batch_sweep:
        # the workload's other batch sizes (BASELINE config 5: batch 1, 8, 32), same prompt length,
        # a short timed loop each: whole-batch tokens per second, device-timed
        del dec
        torch.cuda.empty_cache()
        line["batch_sweep"] = {str(b): decode_at_batch(model, b, prompt, host_ids, device) for b in (8, 32)}
    if rank == 0:
        if world == 1 and not args.skip_cpu_baseline:  # (the host cores are busy with the other ranks otherwise)
            line["cpu_baseline"] = cpu_reference_decode(spec["shape"], steps=2, warmup=1)
        print(json.dumps(line), flush=True)


def cpu_reference_decode(shape_name, steps, warmup, sample_layers=2, prompt=64):
    """Decode steps of the reference's `real` mode on the host cores, run for real: a random-init
    Llama of the workload's width, cut to `sample_layers` decoder layers (the full depth does
    not fit a benchmark run on a CPU), quantized by the reference's own
    `oneshot(model, QuantConfig(...).to_modifier(mode="real"))` with its FakeQuantCache(8), a
    short prompt, then `warmup + steps` greedy tokens through the transformers model, each
    timed. The staged reference package is used when present (kind "reference"), else the
    oracle's restatement of the same modules (kind "port"). The per-token time of the full
    model = time outside the decoder layers + (full depth) x mean time of one layer, both
    measured in the same steps with forward hooks."""
    from transformers import LlamaForCausalLM

    from llmquant_b200.runtime.random_init import SHAPES, llama_config
    from oracle import make_ref

    torch.set_num_threads(os.cpu_count() or 1)  # torchrun pins OMP_NUM_THREADS=1
    full_layers = SHAPES[shape_name]["num_hidden_layers"]
    config = llama_config(shape_name, num_hidden_layers=sample_layers)
    with torch.device("meta"):
        model = LlamaForCausalLM(config)
    model = model.to_empty(device="cpu")
    g = torch.Generator().manual_seed(0)
    with torch.no_grad():
        for _, p in sorted(model.named_parameters()):
            if p.dim() >= 2:
                p.copy_(torch.randn(p.shape, generator=g) * 0.02)
            else:
                p.fill_(1.0)
    model.model.rotary_emb = type(model.model.rotary_emb)(config)
    model = model.to(torch.bfloat16).eval()
    if make_ref.available():
        make_ref.import_reference()
        from llmquant.core import QuantConfig, oneshot
        from llmquant.quantizers import make_cache_factory

        kind = "reference"
        cfg = QuantConfig(attn_weight="int8", mlp_weight="int4", head_weight="int8", kv_cache="int8")
        oneshot(model, cfg.to_modifier(mode="real"))
        cache = make_cache_factory(8)()
    else:
        from oracle.real_mode import FakeQuantKV, apply_real_mode

        kind = "port"
        apply_real_mode(model, attn_bits=8, mlp_bits=4, head_bits=8)
        cache = FakeQuantKV(8)
    in_layers = [0.0]

    def before(_m, _a, _k=None):
        in_layers.append(time.perf_counter())

    def after(_m, _a, _o):
        in_layers[0] += time.perf_counter() - in_layers.pop()

    for layer in model.model.layers:
        layer.register_forward_pre_hook(before)
        layer.register_forward_hook(after)
    ids = torch.randint(0, config.vocab_size, (1, prompt), generator=g)
    with torch.no_grad():
        out = model(ids, past_key_values=cache, use_cache=True, logits_to_keep=1)
        tok = out.logits[:, -1].argmax(-1)
        step_s, layer_s = [], []
        for i in range(warmup + steps):
            in_layers[0] = 0.0
            t0 = time.perf_counter()
            out = model(tok[:, None], past_key_values=cache, use_cache=True)
            tok = out.logits[:, -1].argmax(-1)
            if i >= warmup:
                step_s.append(time.perf_counter() - t0)
                layer_s.append(in_layers[0])
    sample_s = sum(step_s) / len(step_s)
    per_layer = sum(layer_s) / len(layer_s) / sample_layers
    token_s = (sample_s - per_layer * sample_layers) + full_layers * per_layer
    return {"value": round(1.0 / token_s, 4), "unit": "tok/s", "cores": torch.get_num_threads(),
            "kind": kind, "sample_ms_per_step": round(sample_s * 1e3, 2), "steps_timed": len(step_s),
            "sample": f"{kind} real mode (attn int8 / mlp int4 / lm_head int8 / FakeQuantCache(8)) of a "
                      f"random-init {shape_name} cut to {sample_layers} of {full_layers} decoder layers, "
                      f"{prompt}-token prompt, batch 1, {len(step_s)} greedy tokens timed one by one; token "
                      f"time of the full depth = time outside the layers + {full_layers} x mean layer time "
                      f"({per_layer * 1e3:.1f} ms)"}


# --------------------------------------------------------------------------- CPU arm
def cpu_baseline(sample_seconds=15.0, steps=None):
    """The reference's real-mode linear (quantizers/real.py:76-103) on the sweep shapes, M=1, on
    all host threads, bounded in time: `RealQuantLinear` of the staged reference package when it
    is there, else the oracle's numpy restatement."""
    import numpy as np

    import oracle
    from oracle import make_ref

    torch.set_num_threads(os.cpu_count() or 1)
    staged = make_ref.available()
    if staged:
        make_ref.import_reference()
        from llmquant.core.scheme import QuantizationArgs as RefArgs
        from llmquant.core.scheme import QuantizationScheme as RefScheme
        from llmquant.quantizers.real import RealQuantLinear
    rng = np.random.default_rng(0)
    done_bytes, spent, used = 0, 0.0, []
    budget = sample_seconds
    for name, n, k, bits in SWEEP_1B:
        if name.startswith("lm_head"):
            n = 16032  # one eighth of the vocabulary keeps the sample bounded
        w = oracle.round_to_dtype((rng.standard_normal((n, k)) * 0.02).astype(np.float32), "bf16")
        x = oracle.round_to_dtype(rng.standard_normal((1, k)).astype(np.float32), "bf16")
        if staged:
            lin = torch.nn.Linear(k, n, bias=False)
            lin.weight.data = torch.from_numpy(w).bfloat16()
            scheme = RefScheme(weights=RefArgs(num_bits=bits, strategy="group", group_size=128),
                               input_activations=None)
            mod = RealQuantLinear.from_linear(lin, scheme)
            xt = torch.from_numpy(x).bfloat16()
            run = lambda: mod(xt)  # noqa: E731
        else:
            q, scale = oracle.quantize_weight(w, bits, 128)
            run = lambda: oracle.real_linear(x, q, scale, bits, 128, out_dtype="bf16")  # noqa: E731
        with torch.no_grad():
            run()  # warm-up
            reps = steps or 3
            t0 = time.perf_counter()
            for _ in range(reps):
                run()
            dt = (time.perf_counter() - t0) / reps
        done_bytes += algorithmic_bytes(n, k, bits)
        spent += dt
        used.append(name if n != 16032 else name + "[16032 rows]")
        if spent * 3 > budget:
            break
    return {"value": round(done_bytes / spent / 1e9, 3), "unit": "GB/s",
            "cores": torch.get_num_threads(), "kind": "reference" if staged else "port",
            "sample": "one M=1 real-mode forward per shape (mean of the repetitions) over: " + ", ".join(used)}


def run_reference(args, rank):
    if rank != 0:
        return
    if args.workload in DECODE:
        spec = DECODE[args.workload]
        base = cpu_reference_decode(spec["shape"], steps=args.steps, warmup=args.warmup)
        line = {
            "impl": "reference", "metric": "decode_tokens_per_s", "value": base["value"], "unit": "tok/s",
            "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
            # the time of a step as it was run (the bounded sample); `value` is the full depth
            "ms_per_step": base["sample_ms_per_step"],
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "int codes x fp32 (torch CPU)", "data": "synthetic",
            "config": {"workload": f"{args.workload} ({spec['label']}, attn int8 / mlp int4 g128 / "
                                   f"lm_head int8 / int8 KV, greedy)", "batch": 1,
                       "sample": base["sample"]},
            "cpu_baseline": base,
            "e2e": {"value": base["value"], "unit": "tok/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        }
        print(json.dumps(line), flush=True)
        return
    base = cpu_baseline(sample_seconds=60.0, steps=max(1, args.steps))
    line = {
        "impl": "reference", "metric": "quant_gemv_hbm_gbs", "value": base["value"], "unit": "GB/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": None, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "int codes x fp32 (numpy)", "data": "synthetic",
        "config": {"workload": "gemv_sweep_1b (BASELINE config 2: Llama-3.2-1B linear shapes, M=1)",
                   "group_size": 128},
        "cpu_baseline": base,
        "e2e": {"value": base["value"], "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--workload", default="decode_8b",
                    choices=["decode_8b", "decode_1b", "gemv_sweep_1b", "gemv_one", "attn_one", "prefill_gemm"])
    ap.add_argument("--heads", type=int, default=32, help="attn_one: query heads")
    ap.add_argument("--kv-heads", type=int, default=8, help="attn_one: KV heads")
    ap.add_argument("--head-dim", type=int, default=128, help="attn_one: head width")
    ap.add_argument("--splits", type=int, default=0, help="attn_one: context slices per KV head (0 = the decoder's choice)")
    ap.add_argument("--attn-impl", type=int, default=0, help="attn_one: 0 library's choice, 1 SIMT, 2 mma, 3 cluster")
    ap.add_argument("--n", type=int, default=28672)
    ap.add_argument("--k", type=int, default=4096)
    ap.add_argument("--bits", type=int, default=4)
    ap.add_argument("--epilogue", type=int, default=0)
    ap.add_argument("--norm", type=int, default=0)
    ap.add_argument("--rows", default="", help="prefill_gemm: comma-separated token counts (default 16,128,512,2048)")
    ap.add_argument("--no-batch-sweep", action="store_true",
                    help="decode_8b: leave out the short batch-8 / batch-32 measurements")
    ap.add_argument("--skip-cpu-baseline", action="store_true",
                    help="leave the CPU reference sample out of the line (profiling runs)")
    ap.add_argument("--batch", type=int, default=1)
    ap.add_argument("--prompt", type=int, default=0, help="prompt tokens (0 = the workload's own)")
    ap.add_argument("--allreduce", default="peer", choices=["peer", "nccl"])
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        run_reference(args, rank)
        return
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the kernel path has no CPU fallback")
    torch.cuda.set_device(local)
    device = torch.device("cuda", local)
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=device)
    try:
        if args.workload == "gemv_one":
            run_gemv_one(args, device)
        elif args.workload == "attn_one":
            run_attn_one(args, device)
        elif args.workload == "prefill_gemm":
            run_gemm_sweep(args, device)
        elif args.workload in DECODE:
            run_decode(args, rank, world, device)
        else:
            run_gpu(args, rank, world, device)
    finally:
        if world > 1:
            import torch.distributed as dist
            dist.destroy_process_group()


if __name__ == "__main__":
    main()
