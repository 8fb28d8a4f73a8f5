#!/usr/bin/env python3
"""Generate the golden vectors under tests/golden/ by IMPORTING THE REFERENCE ITSELF.

Run where a checkout of AUXStar/rwkv7-quantization is available:

    TRITON_INTERPRET=1 python tests/golden/make_golden.py --reference /path/to/rwkv7-quantization

What is recorded (all seeded, small):
  weights.npz    outputs of the reference's CPU quantizers (schemes.py, int4/quantize_int4.py,
                 int8/quantize_int8.py) and of its CPU dequant-matmul routes (int4_ops.py, int8_ops.py)
  int8_triton.npz outputs of the reference's INT8 Triton kernels (prep_x_int8, linear_int8_fused,
                 linear_rkv_int8_fused in fused_fp8_gemm.py) and of prep_x / prep3_x, executed by the
                 Triton CPU interpreter (IEEE division).  The interpreter's fp32->e4m3 cast is wrong
                 and its fp32->bf16 cast truncates (the GPU rounds to nearest even), so no FP8 code,
                 no FP8 GEMM output and no inexact bf16 copy is recorded from it: the bf16 copy of
                 prep_x / prep3_x is kept only where the conversion is exact (bf16 input, no AWQ).
The committed .npz files were produced by exactly this script.
"""
import argparse
import os
import sys

os.environ.setdefault("TRITON_INTERPRET", "1")

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))


def gen(seed, shape, std=1.0, dtype=torch.float32):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(shape, generator=g) * std).to(dtype)


def bits(t: torch.Tensor) -> np.ndarray:
    """Bit-preserving numpy view (bf16/fp16/fp8 -> unsigned ints)."""
    t = t.detach().contiguous().cpu()
    if t.dtype == torch.bfloat16 or t.dtype == torch.float16:
        return t.view(torch.int16).numpy().view(np.uint16)
    if t.dtype == torch.float8_e4m3fn:
        return t.view(torch.uint8).numpy()
    return t.numpy()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True, help="checkout of the reference repository")
    args = ap.parse_args()
    sys.path.insert(0, args.reference)
    import schemes as ref_schemes
    from int4 import quantize_int4 as ref_q4, int4_ops as ref_i4
    from int8 import quantize_int8 as ref_q8, int8_ops as ref_i8

    out = {}
    # ---- weight quantizers ------------------------------------------------------------
    w = gen(0, (48, 256), 0.02)                       # N(0, 0.02^2), as the reference's CPU-runnable 0.1B case
    w16 = w.to(torch.float16)
    out["w"] = w.numpy()
    for name in ("_q_fp8", "_q_fp8_perchannel", "_q_int8_sym"):
        q, s = getattr(ref_schemes, name)(w)
        out[name + ".q"] = bits(q)
        out[name + ".s"] = s.numpy()
    out["_q_int8_sym.fp16in.q"] = bits(ref_schemes._q_int8_sym(w16)[0])
    out["_q_int8_sym.fp16in.s"] = ref_schemes._q_int8_sym(w16)[1].numpy()
    out["_q_int8_affine"] = ref_schemes._q_int8_affine(w).numpy()
    out["_q_int4_sym"] = ref_schemes._q_int4_sym(w).numpy()
    out["_q_int4_gw.128"] = ref_schemes._q_int4_gw(w, group_size=128).numpy()
    w_odd = gen(1, (8, 200), 0.02)
    out["w_odd"] = w_odd.numpy()
    out["_q_int4_gw.128.padded"] = ref_schemes._q_int4_gw(w_odd, group_size=128).numpy()

    p, s = ref_q4.quantize_to_int4_per_tensor(w)
    out["q4pt.packed"], out["q4pt.scale"] = p.numpy(), s.numpy()
    a = ref_q4.quantize_to_int4_affine(w)
    for k in ("packed", "mx", "rx", "my", "ry"):
        out["q4af." + k] = a[k].numpy()
    gq = ref_q4.quantize_to_int4_groupwise(w, 128)
    for k in ("packed", "scales", "zeros"):
        out["q4gw." + k] = gq[k].numpy()
    q, s = ref_q8.quantize_to_int8_per_tensor(w)
    out["q8pt.q"], out["q8pt.s"] = q.numpy(), s.numpy()
    a8 = ref_q8.quantize_to_int8_affine(w)
    for k in ("w_u8", "mx", "rx", "my", "ry"):
        out["q8af." + k] = a8[k].numpy()

    # ---- reference CPU dequant-matmul routes ---------------------------------------------
    x = gen(2, (3, 256), 1.0, torch.float16)
    out["x"] = bits(x)
    out["unpack_int4"] = ref_i4.unpack_int4(gq["packed"]).numpy()
    out["lin4pt"] = bits(ref_i4.linear_int4_per_tensor(x, {"packed": p, "scale": out_t(out["q4pt.scale"])}))
    out["lin4af"] = bits(ref_i4.linear_int4_affine(x, dict(a)))
    out["lin4gw"] = bits(ref_i4.linear_int4_groupwise(x, dict(gq)))
    out["lin8pt"] = bits(ref_i8.linear_int8_per_tensor(x, {"weight": q, "tensor_scale": s}))
    out["lin8af"] = bits(ref_i8.linear_int8_affine(
        x, {"weight": a8["w_u8"], "mx": a8["mx"], "rx": a8["rx"], "my": a8["my"], "ry": a8["ry"]}))
    np.savez_compressed(os.path.join(HERE, "weights.npz"), **out)
    print("weights.npz:", len(out), "arrays")

    # ---- INT8 Triton kernels + prep_x under the interpreter -------------------------------
    import fused_fp8_gemm as ref_f
    t = {}
    C = 768                                             # RWKV-7 0.1B
    ws = [gen(10 + i, (96, C), 0.02, torch.float16) for i in range(3)]
    infos = []
    for i, wi in enumerate(ws):
        wq, sc = ref_schemes._q_int8_sym(wi)
        infos.append({"weight": wq, "tensor_scale": sc, "qtype": "int8"})
        t[f"w{i}.q"], t[f"w{i}.s"] = wq.numpy(), sc.numpy()
    for tag, m, dt in (("m1", 1, torch.float16), ("m16", 16, torch.float16), ("m5bf", 5, torch.bfloat16)):
        xs = [gen(20 + 7 * m + i, (m, C), 1.0, dt) for i in range(3)]
        if m == 5:
            xs[0][2].zero_()                            # an all-zero row: amax floor 1e-12
        for i, xi in enumerate(xs):
            t[f"{tag}.x{i}"] = bits(xi)
        codes, scale = ref_f.prep_x_int8(xs[0])
        t[f"{tag}.codes"], t[f"{tag}.scale"] = codes.numpy(), scale.numpy()
        t[f"{tag}.lin"] = bits(ref_f.linear_int8_fused(xs[0], infos[0]))
        r, k, v = ref_f.linear_rkv_int8_fused(xs[0], xs[1], xs[2], *infos)
        t[f"{tag}.r"], t[f"{tag}.k"], t[f"{tag}.v"] = bits(r), bits(k), bits(v)
        xb, amax = ref_f.prep_x(xs[0])
        t[f"{tag}.prep.amax"] = amax.numpy()
        exact = dt == torch.bfloat16
        if exact:
            t[f"{tag}.prep.bf16"] = bits(xb)
        awq = gen(99, (C,), 0.2).abs() + 0.5
        t["awq"] = awq.numpy()
        o = ref_f.prep3_x(xs[0], xs[1], xs[2], awq, None)
        if exact:
            t[f"{tag}.prep3.ov"] = bits(o[2])             # v carries no AWQ division
        t[f"{tag}.prep3.amax"] = np.concatenate([o[3].numpy(), o[4].numpy(), o[5].numpy()])
    np.savez_compressed(os.path.join(HERE, "int8_triton.npz"), **t)
    print("int8_triton.npz:", len(t), "arrays")


def out_t(a):
    return torch.from_numpy(np.asarray(a))


if __name__ == "__main__":
    main()
