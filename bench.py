#!/usr/bin/env python3
"""Benchmark of the quantized projection path on B200.

Workload (N = 1 and per rank for N > 1): one decode step (B = 1) through the quantized projections of all
32 layers of RWKV-7 7.2B with FP8 W8A8 weights -- per layer the fused r/k/v launch (3 x [4096,4096]), the
attention output [4096,4096], the FFN key [16384,4096] and the FFN value [4096,16384] -- 128 launches that
stream 6.44 GB of distinct weights (>> the 126 MB L2, so every byte comes from HBM).  The metric is the HBM
rate of that step: algorithmic bytes (weights + scales + activations in + fp16 results out) per second.
Data is synthetic: seeded N(0,1/K) weights quantized like schemes._q_fp8, N(0,1) bf16 activations.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--extra]

For N > 1 launch with torch.distributed.run; ranks hold replicas and independent token streams (sequence
sharding, no collective on the data path).  `--impl reference` times the reference's CPU route (dequantize with
the stored scale, then a torch CPU matmul) on the host cores on a bounded sample of the same workload.
"""
import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
PKG = os.path.join(ROOT, "rwkv7-quantization_b200")
for _p in (ROOT, PKG):
    if _p not in sys.path:
        sys.path.insert(0, _p)

import torch  # noqa: E402

C, F, LAYERS = 4096, 16384, 32
PREFILL_T = 2048          # tokens per sequence of the prefill leg (the reference quotes its prefill figures at T = 2048)
METRIC = "B=1 quantized GEMV HBM GB/s + prefill GEMM TFLOPS, RWKV-7 7.2B shapes, 1-8 GPU"
WORKLOAD = "rwkv7-7.2B fp8 w8a8 decode B=1: 32 layers x (rkv-fused 3x[4096,4096] + att_out [4096,4096] + ffn_key [16384,4096] + ffn_value [4096,16384])"


def peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return {"hbm_gbs": d["hbm_gbs"], "bf16_tflops": d["bf16_tflops"], "bf16_tflops_sustained": d.get("bf16_tflops_sustained", d["bf16_tflops"]),
                "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


def gemv_bytes(m, n, k, in_bytes=2):
    """Algorithmic bytes of one W8A8 projection: weights + scale + activations in + fp16 out."""
    return n * k + 4 + m * k * in_bytes + m * n * 2


def step_bytes(m=1):
    per_layer = 3 * gemv_bytes(m, C, C) + gemv_bytes(m, C, C) + gemv_bytes(m, F, C) + gemv_bytes(m, C, F)
    return per_layer * LAYERS


class ClockSampler:
    """Samples SM clock and throttle reasons of one GPU with nvidia-smi while the timed region runs."""

    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index, self.rows, self.proc = index, [], None

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.index), f"--query-gpu={self.FIELDS}",
                                          "--format=csv,noheader,nounits", "-lms", "100"], stdout=subprocess.PIPE,
                                         stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None
        return self

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def __exit__(self, *exc):
        if self.proc:
            time.sleep(0.15)
            self.proc.terminate()
            self.thread.join(timeout=2)

    def summary(self):
        sm = sorted(int(r[0]) for r in self.rows if r and r[0].isdigit())
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["unsampled"]}
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        reasons = [n for i, n in enumerate(names) if any(len(r) > 2 + i and r[2 + i] == "Active" for r in self.rows)]
        mx = [int(r[1]) for r in self.rows if len(r) > 1 and r[1].isdigit()]
        return {"sm_mhz": sm[len(sm) // 2], "sm_max_mhz": max(mx) if mx else None, "reasons": reasons,
                "samples": len(sm)}


# ------------------------------------------------------------------------------------------ model data
def make_fp8_weight(n, k, gen, dev):
    """N(0,1/K) weights quantized per tensor to e4m3 the way schemes._q_fp8 does, on the device."""
    w = torch.randn((n, k), generator=gen, device=dev, dtype=torch.float32) * (1.0 / k) ** 0.5
    amax = w.abs().max().clamp(min=1e-12)
    scale = (amax / 448.0).float()
    q = (w / scale).clamp(-448.0, 448.0).round().to(torch.float8_e4m3fn)
    return {"weight": q, "tensor_scale": scale, "qtype": "fp8"}


def make_model(dev, seed, nlayers=LAYERS):
    gen = torch.Generator(device=dev).manual_seed(seed)
    layers = []
    for _ in range(nlayers):
        layers.append({
            "r": make_fp8_weight(C, C, gen, dev), "k": make_fp8_weight(C, C, gen, dev), "v": make_fp8_weight(C, C, gen, dev),
            "o": make_fp8_weight(C, C, gen, dev), "ffn_k": make_fp8_weight(F, C, gen, dev),
            "ffn_v": make_fp8_weight(C, F, gen, dev),
        })
    return layers


def make_inputs(dev, seed, m=1, pinned_host=False):
    """Six activation tensors of one decode step: xr, xk, xv, the WKV result, the FFN input, the FFN hidden."""
    gen = torch.Generator().manual_seed(seed)
    shapes = (("xr", C), ("xk", C), ("xv", C), ("xo", C), ("xf", C), ("xg", F))
    host = {name: torch.randn((m, k), generator=gen).to(torch.bfloat16) for name, k in shapes}
    if not pinned_host:
        return host, {k: v.to(dev) for k, v in host.items()}
    # one pinned staging buffer on the host and one buffer on the device, the six tensors as views of them: a step's
    # inputs then cross in ONE host -> device copy
    total = sum(m * k for _, k in shapes)
    flat_h = torch.empty(total, dtype=torch.bfloat16).pin_memory()
    flat_d = torch.empty(total, dtype=torch.bfloat16, device=dev)
    hv, dv, off = {}, {}, 0
    for name, k in shapes:
        hv[name] = flat_h[off:off + m * k].view(m, k)
        hv[name].copy_(host[name])
        dv[name] = flat_d[off:off + m * k].view(m, k)
        off += m * k
    flat_d.copy_(flat_h)
    hv["_flat"], dv["_flat"] = flat_h, flat_d
    return hv, dv


def decode_step(layers, x):
    """One token through the six quantized projections of every layer, by the public drop-in calls."""
    import fused_fp8_gemm as f
    y = None
    for L in layers:
        f.linear_rkv_fused(x["xr"], x["xk"], x["xv"], L["r"], L["k"], L["v"])
        f.linear_quantized_fused(x["xo"], L["o"])
        f.linear_quantized_fused(x["xf"], L["ffn_k"])
        y = f.linear_quantized_fused(x["xg"], L["ffn_v"])
    return y


LAUNCHES_PER_STEP = 4 * LAYERS
# dram__bytes_read.sum + dram__bytes_write.sum per gemv_w8a8_kernel launch of this workload, from an ncu launch list
# of `bench.py --layers 4` (traffic per launch does not depend on the number of layers): 44.70 MB for the r/k/v, att
# output and FFN key launches on average, 67.21 MB for the FFN value.  Algorithmic bytes per launch: 50 368 518.
DRAM_TRAFFIC_PER_LAUNCH = 50_330_000


def prefill_pass(layers, x, fused_rkv=True):
    """One sequence of PREFILL_T tokens through the six projections of every layer.  fused_rkv: r, k and v through
    linear_rkv_fused (one quantizer launch for the three activations, one GEMM launch over the three matrices), the
    call the engine makes for rows <= FUSED_M_MAX (rwkv7_fast_v3a.py:980-985); this build serves it at every row
    count (RWKVQ_FUSED_M_MAX raises the threshold the engine imports).  False: three linear_quantized_fused calls,
    what the engine does above the reference's threshold of 512 rows."""
    import fused_fp8_gemm as f
    y = None
    for L in layers:
        if fused_rkv:
            f.linear_rkv_fused(x["xr"], x["xk"], x["xv"], L["r"], L["k"], L["v"])
            rest = (("o", "xo"), ("ffn_k", "xf"), ("ffn_v", "xg"))
        else:
            rest = (("r", "xr"), ("k", "xk"), ("v", "xv"), ("o", "xo"), ("ffn_k", "xf"), ("ffn_v", "xg"))
        for name, inp in rest:
            y = f.linear_quantized_fused(x[inp], L[name])
    return y


def prefill_flops(nlayers):
    return 2 * PREFILL_T * (4 * C * C + 2 * C * F) * nlayers


# ------------------------------------------------------------------------------------------ CPU arm
_CPU_LAYER = []   # one layer of (weight-info, activation) pairs, built once

def cpu_reference_sample(threads, repeats=3):
    """The reference's CPU route on ONE layer of the workload (1/32 of a step): weights quantized like
    schemes._q_fp8, then per projection w.float()*scale and a torch CPU matmul.  Returns (GB/s, seconds/sample)."""
    from oracle import rwkvq_oracle as O
    torch.set_num_threads(threads)
    if not _CPU_LAYER:
        gen = torch.Generator().manual_seed(1)
        for n, k in [(C, C)] * 4 + [(F, C), (C, F)]:
            q, s = O.q_fp8(torch.randn((n, k), generator=gen) * (1.0 / k) ** 0.5)
            _CPU_LAYER.append(({"weight": q, "tensor_scale": s}, torch.randn((1, k), generator=gen).to(torch.bfloat16)))
    infos, xs = [p[0] for p in _CPU_LAYER], [p[1] for p in _CPU_LAYER]
    best = float("inf")
    for _ in range(repeats):
        t0 = time.perf_counter()
        for info, x in zip(infos, xs):
            O.cpu_dequant_matmul_fp8(x, info)
        best = min(best, time.perf_counter() - t0)
    layer_bytes = step_bytes(1) / LAYERS
    return layer_bytes / best / 1e9, best


def run_reference(args, rank, world):
    if rank != 0:
        return
    threads = os.cpu_count() or 1
    cpu_reference_sample(threads, repeats=max(1, args.warmup))
    t = []
    for _ in range(args.steps):
        gbs, sec = cpu_reference_sample(threads, repeats=1)
        t.append(sec)
    sec = sum(t) / len(t)
    gbs = step_bytes(1) / LAYERS / sec / 1e9
    sample = "one of the 32 layers (6 projections, 201 MB of e4m3 weights) per step; GB/s needs no scaling"
    print(json.dumps({
        "impl": "reference", "metric": METRIC, "value": round(gbs, 3), "unit": "GB/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(sec * 1e3 * LAYERS, 3), "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "fp8_e4m3", "data": "synthetic",
        "config": {"workload": WORKLOAD, "timed": "CPU; ms_per_step is the one-layer sample x 32"},
        "cpu_baseline": {"value": round(gbs, 3), "unit": "GB/s", "cores": threads, "kind": "port", "sample": sample},
        "e2e": {"value": round(gbs, 3), "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }))


# ------------------------------------------------------------------------------------------ GPU arm
def timed(fn, steps, dist_on):
    """Time `steps` calls of fn with CUDA events on the current stream; barrier + synchronize on both sides."""
    import torch.distributed as dist
    torch.cuda.synchronize()
    if dist_on:
        dist.barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        fn()
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1)
    if dist_on:
        t = torch.tensor([ms], device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        dist.barrier()
        ms = t.item()
    return ms


def run_ours(args, rank, world, local_rank):
    import torch.distributed as dist
    import rwkvq_abi as abi
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    abi.require_device()
    dist_on = world > 1
    if dist_on:
        os.environ.setdefault("NCCL_DEBUG_FILE", "/dev/stderr")      # stdout carries the one JSON line only
        dist.init_process_group("nccl", device_id=dev)

    layers = make_model(dev, seed=100 + rank, nlayers=args.layers)
    scale_l = args.layers / LAYERS
    host, x = make_inputs(dev, seed=7 + rank, m=args.tokens, pinned_host=True)
    stream = torch.cuda.Stream()
    with torch.cuda.stream(stream):
        for _ in range(max(3, args.warmup)):
            y = decode_step(layers, x)
        stream.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=stream):
            y = decode_step(layers, x)
        y_host = torch.empty(y.shape, dtype=y.dtype).pin_memory()

        def step_resident():
            graph.replay()

        def step_e2e():
            x["_flat"].copy_(host["_flat"], non_blocking=True)      # the step's six input tensors, one copy
            graph.replay()
            y_host.copy_(y, non_blocking=True)
            torch.cuda.current_stream().synchronize()

        def step_eager():
            x["_flat"].copy_(host["_flat"], non_blocking=True)
            out = decode_step(layers, x)
            y_host.copy_(out, non_blocking=True)
            torch.cuda.current_stream().synchronize()

        for _ in range(max(3, args.warmup)):
            step_resident()
        l0 = abi.launch_count()
        with ClockSampler(local_rank) as clocks:
            ms = timed(step_resident, args.steps, dist_on)
        for _ in range(3):
            step_e2e()
        ms_e2e = timed(step_e2e, args.steps, dist_on)
        for _ in range(3):
            step_eager()
        ms_eager = timed(step_eager, max(1, args.steps // 4), dist_on) / max(1, args.steps // 4) * args.steps
        eager_launches = abi.launch_count() - l0

        # the same step through the per-layer helper of the package (weights, shapes and outputs bound once; one
        # boundary crossing per layer): what an engine's Python decode loop can use instead of four drop-in calls
        from rwkvq_layer import DecodeLayer, MAX_ROWS
        try:
            dl = [DecodeLayer(L["r"], L["k"], L["v"], L["o"], L["ffn_k"], L["ffn_v"], rows=args.tokens) for L in layers] if args.tokens <= MAX_ROWS else []
        except ValueError:      # more rows than the one-launch kernel holds at K = 16384: no per-layer helper for this batch
            dl = []

        def step_layers():
            x["_flat"].copy_(host["_flat"], non_blocking=True)
            for d in dl:
                out = d.all(x["xr"], x["xk"], x["xv"], x["xo"], x["xf"], x["xg"])
            y_host.copy_(out[5], non_blocking=True)
            torch.cuda.current_stream().synchronize()

        if dl:
            for _ in range(3):
                step_layers()
            ms_layers = timed(step_layers, args.steps, dist_on)
        else:
            ms_layers = float("nan")

    prefill = None
    if not args.no_prefill:
        with torch.cuda.stream(stream):
            gen = torch.Generator(device=dev).manual_seed(5 + rank)
            xp = {name: torch.randn((PREFILL_T, k), generator=gen, device=dev).to(torch.bfloat16)
                  for name, k in (("xr", C), ("xk", C), ("xv", C), ("xo", C), ("xf", C), ("xg", F))}
            for _ in range(2):
                prefill_pass(layers, xp)
            reps = 3
            ms_p_eager = timed(lambda: prefill_pass(layers, xp), reps, dist_on) / reps
            stream.synchronize()
            ms_g = {}
            for fused_rkv in (True, False):                  # the same public-API calls, replayed from a CUDA graph
                prefill_pass(layers, xp, fused_rkv)
                stream.synchronize()
                gp = torch.cuda.CUDAGraph()
                with torch.cuda.graph(gp, stream=stream):
                    prefill_pass(layers, xp, fused_rkv)
                gp.replay()
                ms_g[fused_rkv] = timed(gp.replay, reps, dist_on) / reps
                del gp
            ms_p = ms_g[True]
        tfl = prefill_flops(args.layers) * world / (ms_p * 1e-3) / 1e12
        prefill = {"metric": "prefill GEMM TFLOPS (FP8 W8A8, T=2048 tokens, all projections incl. activation quantization)",
                   "value": round(tfl, 1), "unit": "TFLOP/s", "ms_per_sequence": round(ms_p, 3),
                   "launch": "CUDA graph of the %d public-API calls (r/k/v in one linear_rkv_fused call per layer); the same "
                             "calls eager from Python: %.3f ms per sequence" % (4 * args.layers, ms_p_eager),
                   "separate_rkv": {"ms_per_sequence": round(ms_g[False], 3),
                                    "tflops": round(prefill_flops(args.layers) * world / (ms_g[False] * 1e-3) / 1e12, 1),
                                    "note": "r, k and v as three linear_quantized_fused calls (%d calls per sequence), what the "
                                            "reference engine does above its FUSED_M_MAX of 512 rows" % (6 * args.layers)},
                   "roofline": {"bound": "tensor", "achieved": round(tfl / world, 1), "peak": round(2 * peaks()["bf16_tflops_sustained"], 1),
                                "unit": "TFLOP/s", "frac": round(tfl / world / (2 * peaks()["bf16_tflops_sustained"]), 4),
                                "frac_of_burst": round(tfl / world / (2 * peaks()["bf16_tflops"]), 4),
                                "peak_note": "2 x the measured dense bf16 cuBLAS rate (fp8 runs at twice the bf16 rate); the prefill leg is a "
                                             "seconds-long sequence of GEMMs under the power cap, so `peak` is the SUSTAINED measurement "
                                             "(bf16_tflops_sustained); frac_of_burst divides by the burst figure instead"}}
        del xp
    # per-shape breakdown: each of the four launch kinds of the step alone, graph replay over the 32 layers' weights
    per_shape = {}
    with torch.cuda.stream(stream):
        import fused_fp8_gemm as f
        m = args.tokens
        kinds = {
            "att_rkv": (lambda L: f.linear_rkv_fused(x["xr"], x["xk"], x["xv"], L["r"], L["k"], L["v"]), 3 * gemv_bytes(m, C, C)),
            "att_out": (lambda L: f.linear_quantized_fused(x["xo"], L["o"]), gemv_bytes(m, C, C)),
            "ffn_key": (lambda L: f.linear_quantized_fused(x["xf"], L["ffn_k"]), gemv_bytes(m, F, C)),
            "ffn_value": (lambda L: f.linear_quantized_fused(x["xg"], L["ffn_v"]), gemv_bytes(m, C, F)),
        }
        for name, (fn, nb) in kinds.items():
            for L in layers:
                fn(L)
            stream.synchronize()
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, stream=stream):
                for L in layers:
                    fn(L)
            for _ in range(3):
                g.replay()
            us = timed(g.replay, args.steps, dist_on) / args.steps * 1e3 / args.layers
            per_shape[name] = {"us": round(us, 2), "bytes": nb, "frac": round(nb / us / 1e3 / peaks()["hbm_gbs"], 4)}
    # FFN pair (key -> relu_square -> value) at one token: three separate steps against the fused pair, CUDA-graph replay over
    # all layers' FFN weights (4.3 GB of distinct weights per pass)
    ffn_pair = None
    if args.tokens == 1:
        import fused_fp8_gemm as f
        with torch.cuda.stream(stream):
            xf = x["xf"]

            def three_steps():
                for L in layers:
                    h = f.linear_quantized_fused(xf, L["ffn_k"])
                    h = (h.float().clamp_(min=0.0) ** 2).to(torch.float16)      # stand-in for the engine's relu_square kernel
                    f.linear_quantized_fused(h, L["ffn_v"])

            def fused_pair():
                for L in layers:
                    f.ffn_relu2_fp8(xf, L["ffn_k"], L["ffn_v"])
            res = {}
            for name, fn in (("three_steps", three_steps), ("fused_pair", fused_pair)):
                fn()
                stream.synchronize()
                g = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g, stream=stream):
                    fn()
                for _ in range(3):
                    g.replay()
                res[name] = timed(g.replay, args.steps, dist_on) / args.steps * 1e3 / args.layers
            pair_bytes = gemv_bytes(1, F, C) + gemv_bytes(1, C, F)
            ffn_pair = {"M": 1, "three_steps_us_per_layer": round(res["three_steps"], 2), "fused_pair_us_per_layer": round(res["fused_pair"], 2),
                        "fused_pair_frac_hbm": round(pair_bytes / res["fused_pair"] / 1e3 / peaks()["hbm_gbs"], 4),
                        "note": "three steps = key projection, relu_square (torch ops standing in for the engine's kernel), value projection"}
            if not args.no_prefill:
                # the same pair for one 2048-token sequence (eager calls, four layers' weights in turn)
                xp = torch.randn((PREFILL_T, C), device=dev).to(torch.bfloat16)
                some = layers[:4]

                def three_steps_p():
                    for L in some:
                        h = f.linear_quantized_fused(xp, L["ffn_k"])
                        h = (h.float().clamp_(min=0.0) ** 2).to(torch.float16)
                        f.linear_quantized_fused(h, L["ffn_v"])

                def relu_only():
                    for L in some:
                        (hbuf.float().clamp_(min=0.0) ** 2).to(torch.float16)

                def fused_pair_p():
                    for L in some:
                        f.ffn_relu2_fp8(xp, L["ffn_k"], L["ffn_v"])
                hbuf = torch.randn((PREFILL_T, F), device=dev).half()
                resp = {}
                for name, fn in (("three_steps", three_steps_p), ("relu_only", relu_only), ("fused_pair", fused_pair_p)):
                    for _ in range(2):
                        fn()
                    resp[name] = timed(fn, 3, dist_on) / 3 * 1e3 / len(some)
                fl = 2 * PREFILL_T * 2 * C * F
                ffn_pair["prefill_2048"] = {
                    "three_steps_us_per_layer": round(resp["three_steps"], 1), "of_which_relu_square_torch_us": round(resp["relu_only"], 1),
                    "fused_pair_us_per_layer": round(resp["fused_pair"], 1), "fused_pair_TFLOPs": round(fl / resp["fused_pair"] / 1e6, 1),
                    "note": "the engine's relu_square is ONE kernel (one read and one write of [2048, 16384] fp16); the torch stand-in "
                            "timed here takes several passes, so compare the fused pair with three_steps minus relu_square plus one pass"}
                del xp, hbuf
    colsplit = None
    if dist_on and not args.no_colsplit:
        with torch.cuda.stream(stream):
            try:
                colsplit = colsplit_leg(world, dev, dist_on)
            except Exception as e:          # the step's own numbers above stand; say what happened to this leg
                colsplit = {"error": f"{type(e).__name__}: {e}"[:400]}
    nbytes = int(step_bytes(args.tokens) * scale_l)
    per_step = ms / args.steps
    gbs = nbytes * world / (per_step * 1e-3) / 1e9
    gbs_e2e = nbytes * world / (ms_e2e / args.steps * 1e-3) / 1e9
    gbs_eager = nbytes * world / (ms_eager / args.steps * 1e-3) / 1e9
    gbs_layers = nbytes * world / (ms_layers / args.steps * 1e-3) / 1e9
    pk = peaks()
    per_gpu = gbs / world
    line = {
        "metric": METRIC, "value": round(gbs, 2), "unit": "GB/s", "n_gpus": world, "steps": args.steps,
        "warmup": max(3, args.warmup), "ms_per_step": round(per_step, 4), "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "fp8_e4m3", "data": "synthetic",
        "config": {"workload": WORKLOAD if args.tokens == 1 else WORKLOAD.replace("B=1", f"B={args.tokens}"), "tokens_per_step_per_gpu": args.tokens, "parallelism": f"sequence-sharded x{world}",
                   "l2": "6.44 GB of distinct weights per step (inputs larger than L2)",
                   "launch": "CUDA graph of the 128 public-API calls"},
        "roofline": {"bound": "hbm", "achieved": round(per_gpu, 2), "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": round(per_gpu / pk["hbm_gbs"], 4), "traffic": DRAM_TRAFFIC_PER_LAUNCH if args.layers == LAYERS else None,
                     "peak_source": pk["source"],
                     "kernel": "gemv_w8a8_kernel<fp8>", "bytes_per_launch": nbytes // (4 * args.layers),
                     "us_per_launch": round(per_step * 1e3 / (4 * args.layers), 3),
                     "launch_note": "bytes_per_launch / us_per_launch are averages over the four launch kinds of a layer; per_shape "
                                    "times each kind alone (same kernel, graph replay over the 32 layers' weights)",
                     "per_shape": per_shape},
        "e2e": {"value": round(gbs_e2e, 2), "unit": "GB/s",
                "h2d_bytes_per_step": host["_flat"].numel() * host["_flat"].element_size(),
                "d2h_bytes_per_step": y_host.numel() * y_host.element_size(),
                "mode": "one pinned host -> device copy of the step's six input tensors, graph replay of the public API calls, device -> host result",
                "eager_python_calls_gbs": round(gbs_eager, 2),
                "eager_layer_calls_gbs": round(gbs_layers, 2),
                "eager_note": "no CUDA graph: eager_python_calls = the 128 drop-in calls per step; eager_layer_calls = 32 "
                              "rwkvq_layer.DecodeLayer.all calls per step (descriptors bound once, one boundary crossing per layer)"},
        "gpu_launches": int(round(eager_launches / (3 + max(1, args.steps // 4)))) * args.steps,   # counted per eager step, x timed steps
        "launches_counted_eager": int(eager_launches),
        "clocks": clocks.summary(),
        "prefill": prefill,
        "colsplit": colsplit,
        "ffn_pair": ffn_pair,
    }
    if rank == 0:
        if world == 1 and not args.no_cpu:
            threads = os.cpu_count() or 1
            gbs_cpu, sec = cpu_reference_sample(threads, repeats=3)
            line["cpu_baseline"] = {"value": round(gbs_cpu, 3), "unit": "GB/s", "cores": threads, "kind": "port",
                                    "sample": "one of the 32 layers (6 projections, 201 MB of e4m3 weights), best of 3"}
        print(json.dumps(line))
    if dist_on:
        dist.destroy_process_group()


# ------------------------------------------------------------------------------------------ column-split FFN key (N > 1)
def colsplit_leg(world, dev, dist_on):
    """NVFP4 FFN key [16384, 4096] split by output rows over the ranks, activations replicated, slices gathered along
    the features: per M the local GEMM, the gather alone (NCCL all-gather + layout copy vs the library's peer-memory
    pull), both end to end, and the fused form (push: the GEMM's epilogue stores its tiles into every rank's buffer and
    the receivers wait for a flag); microseconds are maxima over ranks, GB/s counts the bytes a rank RECEIVES over NVLink."""
    import fp8_ops
    import nvfp4_ops
    import rwkvq_dist as D
    gen = torch.Generator(device=dev).manual_seed(11)                    # same weights on every rank
    w = torch.randn((F, C), generator=gen, device=dev) * C ** -0.5
    info = nvfp4_ops.quantize_to_nvfp4(w)
    del w
    lin = fp8_ops.linear_quantized
    rows = []
    splits = {"nccl": D.ColumnSplitLinear(info, lin, gather="nccl"), "peer": D.ColumnSplitLinear(info, lin, gather="peer", max_rows=4096),
              "push": D.ColumnSplitLinear(info, lin, gather="push", max_rows=4096)}
    local = splits["nccl"].local
    nl = F // world
    for m in (1, 256, 4096):
        x = torch.randn((m, C), generator=gen, device=dev).to(torch.bfloat16)
        reps = 20 if m <= 256 else 8
        flat = lin(x, local)
        gathered = torch.empty((world * m, nl), dtype=torch.float16, device=dev)
        full = torch.empty((m, world, nl), dtype=torch.float16, device=dev)

        def nccl_gather():
            torch.distributed.all_gather_into_tensor(gathered, flat)
            if m > 1:
                full.copy_(gathered.view(world, m, nl).permute(1, 0, 2))

        def peer_gather():
            splits["peer"].peer.next_buffer(m)
            splits["peer"].peer.gather()
        legs = {"local_gemm": lambda: lin(x, local), "nccl_gather": nccl_gather, "peer_gather": peer_gather,
                "nccl_e2e": lambda: splits["nccl"](x), "peer_e2e": lambda: splits["peer"](x), "push_e2e": lambda: splits["push"](x)}
        row = {"M": m, "bytes_received_per_rank": m * (F - nl) * 2}
        for name, fn in legs.items():
            for _ in range(3):
                fn()
            row[name + "_us"] = round(timed(fn, reps, dist_on) * 1e3 / reps, 2)
        for mode in ("nccl", "peer"):
            row[mode + "_gather_GBps"] = round(row["bytes_received_per_rank"] / row[mode + "_gather_us"] / 1e3, 1)
        row["peer_vs_nccl_e2e"] = round(row["nccl_e2e_us"] / row["peer_e2e_us"], 2)
        row["push_vs_nccl_e2e"] = round(row["nccl_e2e_us"] / row["push_e2e_us"], 2)
        row["push_fused"] = bool(nvfp4_ops.can_push(m, C))     # False: few rows take the decode GEMV and the pull form
        # what gather="auto" runs for this rank count and row count (the same code path as the mode it picks)
        row["auto_gather"] = "push" if (row["push_fused"] and D.ColumnSplitLinear.auto_pushes(world, m)) else "peer"
        row["auto_e2e_us"] = row[row["auto_gather"] + "_e2e_us"]
        row["auto_vs_nccl_e2e"] = round(row["nccl_e2e_us"] / row["auto_e2e_us"], 2)
        rows.append(row)
    for mode in ("peer", "push"):
        splits[mode].peer.check()
        splits[mode].peer.close()
    return {"workload": "NVFP4 FFN key [16384,4096] column-split over the ranks, bf16 activations replicated, fp16 [M,16384] gathered on every rank",
            "timing": "CUDA events on the launching stream, eager calls, max over ranks", "nvlink_peak_GBps_per_direction": 770.0, "rows": rows}


# ------------------------------------------------------------------------------------------ per-shape mode
SHAPES = {"att": (C, C), "ffn_key": (F, C), "ffn_value": (C, F), "c2": (2560, 2560), "c1": (768, 768),
          "att_rkv": (C, C), "c2_rkv": (2560, 2560)}      # *_rkv: three matrices of that shape in one r/k/v call


def _rand_weight(scheme, n, k, dev):
    """Random codes with valid scales: enough for timing (values do not change the work)."""
    if scheme == "fp8":
        return {"weight": torch.randint(0, 120, (n, k), dtype=torch.uint8, device=dev).view(torch.float8_e4m3fn),
                "tensor_scale": torch.tensor(0.01, device=dev), "qtype": "fp8"}
    if scheme == "int8":
        return {"weight": torch.randint(-127, 127, (n, k), dtype=torch.int8, device=dev),
                "tensor_scale": torch.tensor(0.01, device=dev), "qtype": "int8"}
    if scheme == "int4":
        return {"packed": torch.randint(0, 255, (n, k // 2), dtype=torch.uint8, device=dev),
                "scales": torch.rand(n, k // 128, device=dev) * 0.01, "zeros": -torch.rand(n, k // 128, device=dev) * 0.05,
                "group_size": 128, "qtype": "int4_groupwise"}
    if scheme == "nvfp4":
        return {"weight": torch.randint(0, 255, (n, k // 2), dtype=torch.uint8, device=dev),
                "block_scale": torch.randint(40, 100, (n, k // 16), dtype=torch.uint8, device=dev).view(torch.float8_e4m3fn),
                "tensor_scale": torch.tensor(0.001, device=dev), "qtype": "nvfp4"}
    raise ValueError(scheme)


def _weight_bytes(scheme, n, k):
    return {"fp8": n * k + 4, "int8": n * k + 4, "int4": n * k // 2 + n * (k // 128) * 8,
            "nvfp4": n * k // 2 + n * k // 16 + 4}[scheme]


def _linear(scheme):
    import fp8_ops
    if scheme == "int4":
        from int4 import int4_ops
        return int4_ops.linear_int4
    return fp8_ops.linear_quantized_fused if scheme in ("fp8", "int8") else fp8_ops.linear_quantized


def run_shape(args):
    """One projection shape, one scheme, one M: rotates over enough distinct weight buffers to exceed L2, replays a
    CUDA graph of the public calls, prints one JSON line (GB/s for M <= 128, TFLOP/s above)."""
    import rwkvq_abi as abi
    abi.require_device()
    dev = torch.device("cuda", 0)
    n, k = SHAPES[args.shape]
    nmat = 3 if args.shape.endswith("_rkv") else 1
    wb = _weight_bytes(args.scheme, n, k) * nmat
    nbuf = max(2, int(400e6 / wb) + 1)
    ws = [[_rand_weight(args.scheme, n, k, dev) for _ in range(nmat)] for _ in range(nbuf)]
    xs = [torch.randn(args.m, k, device=dev).to(torch.float16 if args.scheme == "int4" else torch.bfloat16) for _ in range(nmat)]
    x = xs[0]
    lin = _linear(args.scheme)
    if nmat == 3:
        import fused_fp8_gemm as f
        rkv = {"fp8": f.linear_rkv_fused, "int8": f.linear_rkv_int8_fused}[args.scheme]

    def fn():
        for w in ws:
            if nmat == 3:
                rkv(xs[0], xs[1], xs[2], w[0], w[1], w[2])
            else:
                lin(x, w[0])
    st = torch.cuda.Stream()
    with torch.cuda.stream(st):
        for _ in range(max(1, args.warmup)):
            fn()
        st.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=st):
            fn()
        for _ in range(max(1, args.warmup)):
            g.replay()
        ms = timed(g.replay, args.steps, False)
    us = ms * 1e3 / (args.steps * nbuf)
    nbytes = wb + nmat * (args.m * k * 2 + args.m * n * 2)
    line = {"case": "shape", "scheme": args.scheme, "shape": args.shape, "M": args.m, "N": n, "K": k, "us_per_call": round(us, 3),
            "algorithmic_bytes": nbytes, "GBps": round(nbytes / us / 1e3, 1), "frac_hbm": round(nbytes / us / 1e3 / peaks()["hbm_gbs"], 4),
            "TFLOPs": round(2 * nmat * args.m * n * k / us / 1e6, 1), "distinct_weight_buffers": nbuf}
    print(json.dumps(line))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-cpu", action="store_true", help="skip the cpu_baseline leg")
    ap.add_argument("--layers", type=int, default=LAYERS, help="layers of the stack (32 = the benchmark; fewer only for profiler captures)")
    ap.add_argument("--no-prefill", action="store_true", help="skip the secondary prefill measurement")
    ap.add_argument("--no-colsplit", action="store_true", help="N > 1: skip the column-split FFN key measurement")
    ap.add_argument("--case", default="decode", choices=["decode", "shape"], help="decode = the benchmark; shape = one projection")
    ap.add_argument("--scheme", default="fp8", choices=["fp8", "int8", "int4", "nvfp4"])
    ap.add_argument("--shape", default="ffn_key", choices=sorted(SHAPES))
    ap.add_argument("--m", type=int, default=1, help="rows of activations in --case shape")
    ap.add_argument("--tokens", type=int, default=1, help="rows per projection in the decode step (1 = the benchmark; more = batched decode)")
    args = ap.parse_args()
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    # stdout carries the result line(s) only: whatever libraries write to file descriptor 1 on the way (NCCL prints its
    # version there) goes to stderr, and print() below reaches the original stdout through sys.stdout
    sys.stdout.flush()
    sys.stdout = os.fdopen(os.dup(1), "w", buffering=1)
    os.dup2(2, 1)
    if args.case == "shape":
        if rank == 0:
            run_shape(args)
    elif args.impl == "reference":
        run_reference(args, rank, world)
    else:
        run_ours(args, rank, world, local_rank)


if __name__ == "__main__":
    main()
