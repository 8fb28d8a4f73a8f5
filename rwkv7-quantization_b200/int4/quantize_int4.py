#!/usr/bin/env python3
"""Offline INT4 quantizers with the storage layouts of the reference's int4/quantize_int4.py.

    per_tensor : signed nibbles (two per byte, even k in the low nibble) + one fp32 scale = max|w| / 7
    affine     : MM4 -- row offset my, column offset mx, column range rx, row range ry (ranges stored / 4),
                 u4 = floor(w_normalised * 16)
    groupwise  : unsigned nibbles per group of `group_size` along K, fp32 scale = (max - min) / 15, zero = min

Keys written into a checkpoint: <key>.int4_packed plus .int4_scale | .int4_{mx,rx,my,ry,m_orig} |
.int4_{scales,zeros,group_size}; the original <key> is removed (int4/quantize_int4.py:192-263).
"""
from __future__ import annotations

import argparse
import os

import torch

QUANTIZED_COMPONENTS = {"att_r", "att_k", "att_v", "att_o", "ffn_k", "ffn_v"}
INT4_MAX = 7.0


def _div(t: torch.Tensor, value: float) -> torch.Tensor:
    """t / value as an IEEE division on every device (the divisor is a tensor on t's device; torch's CUDA kernel would
    multiply by the rounded reciprocal of a Python scalar): the quantizers give the same bits on the CPU and on a GPU."""
    return t / torch.full((), value, dtype=t.dtype if t.is_floating_point() else torch.float32, device=t.device)
_NAMES = {("att", "receptance"): "att_r", ("att", "key"): "att_k", ("att", "value"): "att_v",
          ("att", "output"): "att_o", ("ffn", "key"): "ffn_k", ("ffn", "value"): "ffn_v"}


def classify_weight(key: str, num_layers: int):
    """`blocks.<l>.<att|ffn>.<name>.weight` -> (layer, component) for the six projections, else None."""
    parts = key.split(".")
    if len(parts) < 4 or parts[0] != "blocks":
        return None
    layer = int(parts[1])
    comp = _NAMES.get((parts[2], parts[3]))
    if comp is None or not 0 <= layer < num_layers:
        return None
    return layer, comp


def _pack_pairs(q: torch.Tensor) -> torch.Tensor:
    """[N, K] values in 0..15 -> [N, K/2] bytes, even k in the low nibble."""
    q = q.to(torch.uint8)
    return q[:, 0::2] | (q[:, 1::2] << 4)


def quantize_to_int4_per_tensor(w: torch.Tensor):
    """(packed uint8 [N, K/2], scale fp32 scalar); W ~ signed_nibble * scale (int4/quantize_int4.py:51-71)."""
    w = w.float()
    assert w.shape[1] % 2 == 0, f"Output dim must be even, got {w.shape[1]}"
    scale = _div(w.abs().max(), INT4_MAX).clamp(min=1e-12)
    q = (w / scale).round().clamp(-8, 7).to(torch.int8) & 0xF
    return _pack_pairs(q), scale.to(torch.float32)


def quantize_to_int4_affine(w: torch.Tensor):
    """MM4 dual affine (int4/quantize_int4.py:78-135); returns packed, mx, rx, my, ry, m_orig."""
    w = w.float()
    m_orig = w.shape[1]
    if m_orig % 2:
        w = torch.nn.functional.pad(w, (0, 1))
    my = w.amin(dim=1, keepdim=True)
    w = w - my
    mx = w.amin(dim=0, keepdim=True)
    w = w - mx
    rx = w.amax(dim=0, keepdim=True).clamp(min=1e-12)
    w = w / rx
    ry = w.amax(dim=1, keepdim=True).clamp(min=1e-12)
    w = w / ry
    u4 = (w * 16.0).floor().clamp(0, 15)
    return {"packed": _pack_pairs(u4), "mx": mx.squeeze(0).float(), "rx": (rx / 4.0).squeeze(0).float(),
            "my": my.squeeze(1).float(), "ry": (ry / 4.0).squeeze(1).float(), "m_orig": m_orig}


def quantize_to_int4_groupwise(w: torch.Tensor, group_size: int = 128):
    """Asymmetric group-wise uint4 (int4/quantize_int4.py:142-185); returns packed, scales, zeros, group_size."""
    w = w.float()
    n, k = w.shape
    assert k % group_size == 0, f"Input dim {k} not divisible by group_size {group_size}"
    assert k % 2 == 0, f"Output dim must be even, got {k}"
    g = w.reshape(n, k // group_size, group_size)
    lo = g.amin(dim=2, keepdim=True)
    step = _div(g.amax(dim=2, keepdim=True) - lo, 15.0).clamp(min=1e-12)
    q = ((g - lo) / step).round().clamp(0, 15).reshape(n, k)
    return {"packed": _pack_pairs(q), "scales": step.squeeze(2).float(), "zeros": lo.squeeze(2).float(),
            "group_size": group_size}


def quantize_model(model_path: str, output_path: str, scheme: str = "per_tensor", group_size: int = 128):
    """Quantize the six projections of every layer of a .pth checkpoint and save it (int4/quantize_int4.py:192-263)."""
    z = torch.load(model_path, map_location="cpu", weights_only=True)
    num_layers = 1 + max((int(k.split(".")[1]) for k in z if k.startswith("blocks.")), default=-1)
    untouched = [k for k in z if classify_weight(k, num_layers) is None]
    done = []
    for key in list(z):
        if classify_weight(key, num_layers) is None:
            continue
        w = z[key].float()
        if scheme == "per_tensor":
            fields = dict(zip(("packed", "scale"), quantize_to_int4_per_tensor(w)))
        elif scheme == "affine":
            fields = quantize_to_int4_affine(w)
        elif scheme == "groupwise":
            fields = quantize_to_int4_groupwise(w, group_size)
        else:
            raise ValueError(f"Unknown scheme: {scheme}")
        for suffix, value in fields.items():
            z[f"{key}.int4_{suffix}"] = value
        done.append(key)
    for key in done:
        del z[key]
    z["meta"] = {"quantization": f"int4_{scheme}", "scheme": scheme, "group_size": group_size if scheme == "groupwise" else 0,
                 "components": list(QUANTIZED_COMPONENTS), "non_quant_prefixes": untouched, "num_layers": num_layers,
                 "dtype": "int4"}
    torch.save(z, output_path)
    print(f"Quantized {len(done)} weights to INT4 ({scheme}): "
          f"{os.path.getsize(model_path) / 1e9:.2f} GB -> {os.path.getsize(output_path) / 1e9:.2f} GB")


if __name__ == "__main__":
    ap = argparse.ArgumentParser(description="Quantize RWKV-7 model to INT4")
    ap.add_argument("--model", required=True)
    ap.add_argument("--output", required=True)
    ap.add_argument("--scheme", default="per_tensor", choices=["per_tensor", "affine", "groupwise"])
    ap.add_argument("--group-size", type=int, default=128)
    a = ap.parse_args()
    quantize_model(a.model, a.output, a.scheme, a.group_size)
