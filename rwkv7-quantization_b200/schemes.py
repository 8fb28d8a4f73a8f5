"""Drop-in for the reference's root `schemes.py`: the scheme registry and the offline (CPU, torch) weight
quantizers whose outputs define the on-disk weight and scale layouts.  The registry keys, the entry fields and
the quantizer results are the reference's (schemes.py:18-195); "nvfp4" is an added scheme.

A quantizer returns either (codes, scale) -- stored as `<key>` and `<key>.fp8_scale` -- or a float tensor of the
original shape holding the quantize->dequantize round trip (simulated quantization).
"""
from __future__ import annotations

from typing import Any

import torch

_TINY = 1e-12


def _div(t: torch.Tensor, value: float) -> torch.Tensor:
    """t / value with the divisor as a tensor on t's device: an IEEE division on the CPU and on a GPU alike (torch's CUDA
    kernel turns a division by a Python scalar into a product with the rounded reciprocal, one ulp off now and then), so
    the quantizers give the same bits wherever they run."""
    return t / torch.full((), value, dtype=t.dtype if t.is_floating_point() else torch.float32, device=t.device)


def _absmax_scale(w: torch.Tensor, qmax: float, dim=None) -> torch.Tensor:
    a = w.abs().max() if dim is None else w.abs().amax(dim=dim, keepdim=True)
    return _div(a.clamp(min=_TINY), qmax).float()


def _q_fp8(w: torch.Tensor, **kw):
    """Per-tensor e4m3: scale = amax/448; codes = e4m3(round(clamp(w/scale))) (schemes.py:18-24)."""
    s = _absmax_scale(w, 448.0)
    return (w.float() / s).clamp(-448.0, 448.0).round().to(torch.float8_e4m3fn), s


def _q_fp8_perchannel(w: torch.Tensor, **kw):
    """One e4m3 scale per output row (schemes.py:26-34)."""
    if w.dim() == 1:
        return _q_fp8(w)
    s = _absmax_scale(w, 448.0, dim=1)
    return (w.float() / s).clamp(-448.0, 448.0).round().to(torch.float8_e4m3fn), s.squeeze(1)


def _q_int8_sym(w: torch.Tensor, **kw):
    """Per-tensor symmetric int8, scale = amax/127 (schemes.py:36-42)."""
    s = _absmax_scale(w, 127.0)
    return (w.float() / s).round().clamp(-128, 127).to(torch.int8), s


def _mm_affine_sim(w: torch.Tensor, levels: float, stored_div: float) -> torch.Tensor:
    """Row/column dual affine round trip shared by the MM8-style scheme."""
    f = w.float() if w.dim() == 2 else w.float().reshape(1, -1)
    my = f.amin(dim=1, keepdim=True)
    f = f - my
    mx = f.amin(dim=0, keepdim=True)
    f = f - mx
    rx = f.amax(dim=0, keepdim=True).clamp(min=_TINY)
    f = f / rx
    ry = f.amax(dim=1, keepdim=True).clamp(min=_TINY)
    f = f / ry
    q = (f * levels).floor().clamp(0, levels - 1)
    back = (q + 0.5) * (ry * stored_div) * (rx * stored_div) + my + mx
    return back.reshape(w.shape).to(w.dtype)


def _q_int8_affine(w: torch.Tensor, **kw):
    """MM8 simulated quantization (schemes.py:44-62)."""
    return _mm_affine_sim(w, 256.0, 16.0)


def _q_int4_sym(w: torch.Tensor, **kw):
    """Per-tensor symmetric int4 round trip, scale = amax/7 (schemes.py:64-70)."""
    s = _absmax_scale(w, 7.0)
    return ((w.float() / s).round().clamp(-8, 7) * s).to(w.dtype)


def _q_int4_gw(w: torch.Tensor, group_size: int = 128, **kw):
    """Asymmetric uint4 per group of `group_size` along the input dim, round trip; the last group is padded
    with zeros (schemes.py:72-94)."""
    f = w.float() if w.dim() == 2 else w.float().reshape(1, -1)
    rows, cols = f.shape
    short = -cols % group_size
    if short:
        f = torch.nn.functional.pad(f, (0, short))
    g = f.reshape(rows, -1, group_size)
    lo, hi = g.amin(dim=2, keepdim=True), g.amax(dim=2, keepdim=True)
    step = _div(hi - lo, 15.0).clamp(min=_TINY)
    back = (((g - lo) / step).round().clamp(0, 15) * step + lo).reshape(rows, -1)[:, :cols]
    if back.numel() == w.numel():
        back = back.reshape(w.shape)
    return back.to(w.dtype)


def _q_nvfp4(w: torch.Tensor, **kw):
    """NVFP4 round trip: e2m1 values, one e4m3 scale per 16 along K, fp32 tensor scale amax/2688."""
    from nvfp4_ops import quantize_to_nvfp4, dequantize_nvfp4
    return dequantize_nvfp4(quantize_to_nvfp4(w)).reshape(w.shape).to(w.dtype)


def _entry(name, fmt, wbits, abits, comp, fn, hw, accel, **kwargs) -> dict[str, Any]:
    e = {"name": name, "format": fmt, "bits_per_weight": wbits, "activation_bits": abits, "compression": comp,
         "quantize": fn, "hardware_req": hw, "has_hardware_accel": accel}
    if kwargs:
        e["quantize_kwargs"] = kwargs
    return e


SCHEMES: dict[str, dict[str, Any]] = {
    "fp8": _entry("FP8 E4M3 (W8A8)", "float8_e4m3fn", 8, 8, 2.0, _q_fp8, "SM >= 8.9 (Ada/Hopper/Blackwell)", True),
    "fp8_perchannel": _entry("FP8 E4M3 per-channel (W8A8)", "float8_e4m3fn", 8, 8, 2.0, _q_fp8_perchannel, "SM >= 8.9", True),
    "int8_symmetric": _entry("INT8 Per-tensor Symmetric (W8A8)", "int8", 8, 8, 2.0, _q_int8_sym, "Any CUDA GPU", False),
    "int8_affine": _entry("INT8 Affine MM8-style (W8A8)", "uint8 + affine", 8, 8, 2.0, _q_int8_affine, "Any CUDA GPU", False),
    "int4_symmetric": _entry("INT4 Per-tensor Symmetric (W4A16)", "int4 packed", 4, 16, 4.0, _q_int4_sym, "Any CUDA GPU", False),
    "int4_groupwise_128": _entry("INT4 Group-wise (group=128, W4A16)", "int4 packed + per-group scale", 4, 16, 3.5,
                                 _q_int4_gw, "Any CUDA GPU", False, group_size=128),
    "int4_groupwise_256": _entry("INT4 Group-wise (group=256, W4A16)", "int4 packed + per-group scale", 4, 16, 3.7,
                                 _q_int4_gw, "Any CUDA GPU", False, group_size=256),
    "nvfp4": _entry("NVFP4 E2M1 block-16 (W4A4)", "e2m1 packed + e4m3 block scale", 4, 4, 3.5, _q_nvfp4,
                    "SM 10.x (Blackwell)", True),
}


def get_scheme(name: str) -> dict:
    if name not in SCHEMES:
        raise ValueError(f"Unknown scheme: {name!r}. Available: {list_schemes()}")
    return SCHEMES[name]


def list_schemes() -> list[str]:
    return list(SCHEMES)


def print_scheme_table():
    print(f"{'Name':20s} {'Bits':>4s} {'Act':>3s} {'Comp':>4s} {'HW Accel':>8s}  Description")
    print("-" * 72)
    for key, s in SCHEMES.items():
        print(f"{key:20s} {s['bits_per_weight']:4d} {s['activation_bits']:3d} {s['compression']:4.1f}x "
              f"{'Yes' if s['has_hardware_accel'] else 'No':>8s}  {s['name']}")
