#!/usr/bin/env python3
"""Offline INT8 quantizers with the storage layouts of the reference's int8/quantize_int8.py.

    per_tensor : int8 codes + one fp32 scale = max|w| / 127          keys .int8_weight, .int8_scale
    affine     : MM8 -- u8 = floor(w_normalised * 256), ranges / 16  keys .int8_w_u8, .int8_{mx,rx,my,ry}
"""
from __future__ import annotations

import argparse
import os

import torch

from int4.quantize_int4 import QUANTIZED_COMPONENTS, _div, classify_weight  # same six projections  # noqa: F401

INT8_MAX = 127.0


def quantize_to_int8_per_tensor(w: torch.Tensor):
    """(int8 codes, fp32 scale); W ~ codes * scale (int8/quantize_int8.py:51-62)."""
    w = w.float()
    scale = _div(w.abs().max(), INT8_MAX).clamp(min=1e-12)
    return (w / scale).round().clamp(-128, 127).to(torch.int8), scale.to(torch.float32)


def quantize_to_int8_affine(w: torch.Tensor):
    """MM8 dual affine (int8/quantize_int8.py:69-114); returns w_u8, mx, rx, my, ry."""
    w = w.float()
    my = w.amin(dim=1, keepdim=True)
    w = w - my
    mx = w.amin(dim=0, keepdim=True)
    w = w - mx
    rx = w.amax(dim=0, keepdim=True).clamp(min=1e-12)
    w = w / rx
    ry = w.amax(dim=1, keepdim=True).clamp(min=1e-12)
    w = w / ry
    return {"w_u8": (w * 256.0).floor().clamp(0, 255).to(torch.uint8), "mx": mx.squeeze(0).float(),
            "rx": (rx / 16.0).squeeze(0).float(), "my": my.squeeze(1).float(), "ry": (ry / 16.0).squeeze(1).float()}


def quantize_model(model_path: str, output_path: str, scheme: str = "per_tensor"):
    """Quantize the six projections of every layer of a .pth checkpoint and save it (int8/quantize_int8.py:121-185)."""
    z = torch.load(model_path, map_location="cpu", weights_only=True)
    num_layers = 1 + max((int(k.split(".")[1]) for k in z if k.startswith("blocks.")), default=-1)
    untouched = [k for k in z if classify_weight(k, num_layers) is None]
    done = []
    for key in list(z):
        if classify_weight(key, num_layers) is None:
            continue
        w = z[key].float()
        if scheme == "per_tensor":
            z[key + ".int8_weight"], z[key + ".int8_scale"] = quantize_to_int8_per_tensor(w)
        elif scheme == "affine":
            for suffix, value in quantize_to_int8_affine(w).items():
                z[f"{key}.int8_{suffix}"] = value
        else:
            raise ValueError(f"Unknown scheme: {scheme}")
        done.append(key)
    for key in done:
        del z[key]
    z["meta"] = {"quantization": f"int8_{scheme}", "scheme": scheme, "components": list(QUANTIZED_COMPONENTS),
                 "non_quant_prefixes": untouched, "num_layers": num_layers, "dtype": "int8"}
    torch.save(z, output_path)
    print(f"Quantized {len(done)} weights to INT8 ({scheme}): "
          f"{os.path.getsize(model_path) / 1e9:.2f} GB -> {os.path.getsize(output_path) / 1e9:.2f} GB")


if __name__ == "__main__":
    ap = argparse.ArgumentParser(description="Quantize RWKV-7 model to INT8")
    ap.add_argument("--model", required=True)
    ap.add_argument("--output", required=True)
    ap.add_argument("--scheme", default="per_tensor", choices=["per_tensor", "affine"])
    a = ap.parse_args()
    quantize_model(a.model, a.output, a.scheme)
