#!/usr/bin/env python3
"""Record what the REFERENCE's own GPU kernels compute on a B200, as golden vectors for the FP8 / INT8 W8A8 path.

Run on a machine with a B200 and Triton, with a checkout (or a pip --target install) of AUXStar/rwkv7-quantization:

    python tests/golden/make_golden_b200.py --reference /path/to/rwkv7-quantization [--out FILE.npz] [--timing FILE.json]

The reference modules (fused_fp8_gemm.py, fp8_ops.py) are imported unmodified and called through their public
functions on the seeded inputs of fp8_b200_cases.py:

  prep_x_fp8                      e4m3 codes + scale                      (fused_fp8_gemm.py:363-390)
  prep_x / prep3_x with AWQ       bf16 copies + amax (div.full division)  (fused_fp8_gemm.py:30-150)
  linear_fp8_m1_fused             M = 1 Triton kernel                     (fused_fp8_gemm.py:600-679)
  linear_fp8_fused                prep_x + tl.dot(e4m3, e4m3) kernel      (fused_fp8_gemm.py:219-257, 1020-1077)
  linear_rkv_fused                r, k, v in one kernel                   (fused_fp8_gemm.py:264-334, 944-1017)
  linear_fp8                      prep_x_fp8 + torch._scaled_mm           (fp8_ops.py:58-86)
  prep_x_int8, linear_int8_fused  INT8 codes / scales / outputs           (fused_fp8_gemm.py:687-818)

--timing also measures the reference's kernels on the RWKV-7 7.2B projection shapes (CUDA events; eager calls, and
the same calls replayed from a CUDA graph) so that both implementations can be compared on the same GPU.
The committed fp8_triton_b200.npz was produced by exactly this script.
"""
import argparse
import json
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
DEV = "cuda" if torch.cuda.is_available() else "cpu"   # "cpu" only to dry-run the script under TRITON_INTERPRET=1
sys.path.insert(0, HERE)
import fp8_b200_cases as cases  # noqa: E402


def bits(t):
    t = t.detach().contiguous().cpu()
    if t.dtype in (torch.bfloat16, torch.float16):
        return t.view(torch.int16).numpy().view(np.uint16)
    if t.dtype == torch.float8_e4m3fn:
        return t.view(torch.uint8).numpy()
    return t.numpy()


def to_dev(info):
    return {k: (v.to(DEV) if torch.is_tensor(v) else v) for k, v in info.items()}


def record(ref_f, ref_ops):
    out = {}

    def put(tag, t, inputs):
        out[tag] = bits(t)
        out[tag + ".insum"] = np.array([cases.checksum(i) for i in inputs], dtype=np.int64)

    for tag, k, n, m, dt, outl in cases.SINGLE:
        s = cases.seed_of(tag)
        info, x = cases.q_fp8_weight(s, n, k), cases.act(s + 1, m, k, dt, outl)
        put(tag, ref_f.linear_fp8_fused(x.to(DEV), to_dev(info)), [info["weight"], x])
    for tag, k, n, m, dt, outl, awq in cases.RKV:
        s = cases.seed_of(tag)
        infos = [cases.q_fp8_weight(s + i, n, k) for i in range(3)]
        xs = [cases.act(s + 10 + i, m, k, dt, outl) for i in range(3)]
        dinfos = [to_dev(i) for i in infos]
        if awq:
            dinfos[0]["awq_scale"] = cases.awq_vec(k).to(DEV)
            dinfos[1]["awq_scale"] = (cases.awq_vec(k) * 1.25).to(DEV)
        r, kk, v = ref_f.linear_rkv_fused(*[x.to(DEV) for x in xs], *dinfos)
        ins = [i["weight"] for i in infos] + xs
        put(tag + ".r", r, ins)
        put(tag + ".k", kk, ins)
        put(tag + ".v", v, ins)
    for tag, k, n, m, dt, outl in cases.SCALED_MM:
        s = cases.seed_of(tag)
        info, x = cases.q_fp8_weight(s, n, k), cases.act(s + 1, m, k, dt, outl)
        put(tag, ref_ops.linear_fp8(x.to(DEV), to_dev(info)), [info["weight"], x])
    for tag, k, m, dt in cases.IDENTITY:
        s = cases.seed_of(tag)
        info, x = cases.identity_weight(k), cases.act(s, m, k, dt, True)
        put(tag, ref_f.linear_fp8_fused(x.to(DEV), to_dev(info)), [x])
    for tag, m, k, dt in cases.PREP_FP8:
        x = cases.act(cases.seed_of(tag), m, k, dt, True)
        codes, scale = ref_f.prep_x_fp8(x.to(DEV))
        if m > 64:                      # large cases: first and last rows only
            codes = torch.cat([codes[:4], codes[-4:]])
        put(tag + ".codes", codes, [x])
        put(tag + ".scale", scale, [x])
    for tag, m, k, dt in cases.PREP_X:
        s = cases.seed_of(tag)
        xs = [cases.act(s + i, m, k, dt, True) for i in range(3)]
        awq = cases.awq_vec(k)
        o, amax = ref_f.prep_x(xs[0].to(DEV), awq.to(DEV))
        put(tag + ".awq.bf16", o, xs[:1])
        put(tag + ".awq.amax", amax, xs[:1])
        o, amax = ref_f.prep_x(xs[0].to(DEV))
        put(tag + ".bf16", o, xs[:1])
        put(tag + ".amax", amax, xs[:1])
        p3 = ref_f.prep3_x(*[x.to(DEV) for x in xs], awq.to(DEV), (awq * 1.25).to(DEV))
        for name, t in zip(("or", "ok", "ov", "ar", "ak", "av"), p3):
            put(f"{tag}.p3.{name}", t, xs)
    for tag, m, k, dt in cases.PREP_INT8:
        x = cases.act(cases.seed_of(tag), m, k, dt, True)
        codes, scale = ref_f.prep_x_int8(x.to(DEV))
        put(tag + ".codes", codes, [x])
        put(tag + ".scale", scale, [x])
    for tag, k, n, m, dt in cases.INT8_LIN:
        s = cases.seed_of(tag)
        info, x = cases.q_int8_weight(s, n, k), cases.act(s + 1, m, k, dt, False)
        put(tag, ref_f.linear_int8_fused(x.to(DEV), to_dev(info)), [info["weight"], x])
    if DEV == "cuda":
        torch.cuda.synchronize()
    return out


# ------------------------------------------------------------------------------------------------- timing
def _time(fn, nbuf, reps=20):
    """Average microseconds per call: eager calls and a CUDA-graph replay of the same calls over `nbuf` weight sets."""
    for i in range(nbuf):
        fn(i)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(reps):
        for i in range(nbuf):
            fn(i)
    e1.record()
    torch.cuda.synchronize()
    eager = e0.elapsed_time(e1) * 1e3 / (reps * nbuf)
    graph_us = None
    try:
        st = torch.cuda.Stream()
        with torch.cuda.stream(st):
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, stream=st):
                for i in range(nbuf):
                    fn(i)
            g.replay()
            st.synchronize()
            e0.record()
            for _ in range(reps):
                g.replay()
            e1.record()
            st.synchronize()
            graph_us = e0.elapsed_time(e1) * 1e3 / (reps * nbuf)
    except Exception as exc:  # a kernel that cannot be captured is reported, not fatal
        graph_us = f"not captured: {type(exc).__name__}"
        torch.cuda.synchronize()
    return round(eager, 2), graph_us if isinstance(graph_us, str) else round(graph_us, 2)


def timing(ref_f, ref_ops):
    C, F = 4096, 16384
    shapes = {"att": (C, C), "ffn_key": (F, C), "ffn_value": (C, F)}
    dev = torch.device("cuda")
    rows = []

    def weights(n, k, count):
        return [{"weight": torch.randint(0, 120, (n, k), dtype=torch.uint8, device=dev).view(torch.float8_e4m3fn),
                 "tensor_scale": torch.tensor(0.01, device=dev), "qtype": "fp8"} for _ in range(count)]

    def add(name, shape, m, n, k, nmat, fn, nbuf):
        eager, graph = _time(fn, nbuf)
        wbytes = nmat * (n * k + 4) + nmat * m * (k * 2 + n * 2)
        best = min(eager, graph) if not isinstance(graph, str) else eager
        rows.append({"call": name, "shape": shape, "M": m, "N": n, "K": k, "us_eager": eager, "us_graph": graph,
                     "GBps_best": round(wbytes / best / 1e3, 1), "TFLOPs_best": round(2 * nmat * m * n * k / best / 1e6, 1)})
        print(json.dumps(rows[-1]), flush=True)

    for shape, (n, k) in shapes.items():
        nbuf = max(2, int(400e6 / (n * k)) + 1)
        ws = weights(n, k, nbuf)
        for m in (1, 16, 64, 256, 512):
            x = torch.randn(m, k, device=dev).to(torch.bfloat16)
            add("linear_fp8_fused", shape, m, n, k, 1, lambda i: ref_f.linear_fp8_fused(x, ws[i]), nbuf)
        for m in (2048, 8192):
            x = torch.randn(m, k, device=dev).to(torch.bfloat16)
            add("linear_fp8(_scaled_mm)", shape, m, n, k, 1, lambda i: ref_ops.linear_fp8(x, ws[i]), min(nbuf, 4))
        del ws
    for c in (2560, 4096):
        nbuf = max(2, int(400e6 / (3 * c * c)) + 1)
        ws = weights(c, c, 3 * nbuf)
        for m in (1, 8, 32, 256):
            xs = [torch.randn(m, c, device=dev).to(torch.bfloat16) for _ in range(3)]
            add("linear_rkv_fused", f"rkv{c}", m, c, c, 3,
                lambda i: ref_f.linear_rkv_fused(xs[0], xs[1], xs[2], ws[3 * i], ws[3 * i + 1], ws[3 * i + 2]), nbuf)
        del ws
    return rows


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True, help="directory holding the reference's fused_fp8_gemm.py and fp8_ops.py")
    ap.add_argument("--out", default=os.path.join(HERE, "fp8_triton_b200.npz"))
    ap.add_argument("--timing", default=None, help="also time the reference on the 7.2B shapes and write this JSON file")
    args = ap.parse_args()
    ref = os.path.abspath(args.reference)
    sys.path[:] = [p for p in sys.path if "rwkv7-quantization_b200" not in p]   # never the drop-in modules
    sys.path.insert(0, ref)
    import fused_fp8_gemm as ref_f
    import fp8_ops as ref_ops
    assert os.path.abspath(ref_f.__file__).startswith(ref), ref_f.__file__
    assert hasattr(ref_f, "fused_fp8_hwdot_gemm_kernel"), "this is not the reference module"
    import triton
    meta = {"gpu": torch.cuda.get_device_name(0) if DEV == "cuda" else "none (interpreter dry run)", "torch": torch.__version__,
            "triton": triton.__version__, "capability": list(torch.cuda.get_device_capability(0)) if DEV == "cuda" else []}
    print(json.dumps(meta), flush=True)
    out = record(ref_f, ref_ops)
    out["meta"] = np.frombuffer(json.dumps(meta).encode(), dtype=np.uint8)
    np.savez_compressed(args.out, **out)
    print(f"{args.out}: {len(out)} arrays, {os.path.getsize(args.out)} bytes", flush=True)
    if args.timing:
        rows = timing(ref_f, ref_ops)
        with open(args.timing, "w") as fh:
            json.dump({"meta": meta, "rows": rows}, fh, indent=1)


if __name__ == "__main__":
    main()
