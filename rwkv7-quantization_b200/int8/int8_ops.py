"""Stand-alone INT8 weight detection, loading and W8A16 projections (drop-in for the reference's int8/int8_ops.py).

Weight-info dicts (int8/int8_ops.py:22-41):
    per_tensor : {"weight" int8 [N,K], "tensor_scale", "qtype": "int8_per_tensor"}
    affine     : {"weight" uint8 [N,K], "mx", "rx", "my", "ry", "qtype": "int8_affine"}
"""
from __future__ import annotations

import torch

import rwkvq_abi as abi
from int4.int4_ops import _rows_f16, _run_rows, _f32


def is_int8_weight(z: dict, key: str) -> bool:
    return (key + ".int8_weight" in z) or (key + ".int8_w_u8" in z)


def load_int8_weight(z: dict, key: str, dev: str = "cuda"):
    if key + ".int8_weight" in z:
        return {"weight": z[key + ".int8_weight"].to(dev), "tensor_scale": z[key + ".int8_scale"].to(dev),
                "qtype": "int8_per_tensor"}
    if key + ".int8_w_u8" in z:
        info = {"weight": z[key + ".int8_w_u8"].to(dev), "qtype": "int8_affine"}
        info.update({n: z[f"{key}.int8_{n}"].to(dev) for n in ("mx", "rx", "my", "ry")})
        return info
    raise KeyError(f"No INT8 weight found for key: {key}")


def linear_int8_per_tensor(x, weight_info, out_dtype=torch.float16):
    """W8A16 projection: fp16 activations times int8 weights times the scale (int8/int8_ops.py:48-78)."""
    w = weight_info["weight"].contiguous()
    n, k = w.shape
    x2 = _rows_f16(x, k)
    scale = _f32(weight_info["tensor_scale"].reshape(1), x2.device)
    out = _run_rows(x2, n, lambda xc, oc, m: abi.call(
        "rwkvq_gemv_int8_w8a16", xc.data_ptr(), k, w.data_ptr(), w.stride(0), scale.data_ptr(), oc.data_ptr(), n, m, n, k,
        abi.stream_ptr()))
    return out.to(out_dtype).reshape(*x.shape[:-1], n)


def linear_int8_affine(x, weight_info, out_dtype=torch.float16):
    """MM8 projection (int8/int8_ops.py:81-110)."""
    w = weight_info["weight"].contiguous()
    n, k = w.shape
    x2 = _rows_f16(x, k)
    mx, rx, my, ry = (_f32(weight_info[v], x2.device) for v in ("mx", "rx", "my", "ry"))
    out = _run_rows(x2, n, lambda xc, oc, m: abi.call(
        "rwkvq_gemv_int8_affine", xc.data_ptr(), k, w.data_ptr(), w.stride(0), mx.data_ptr(), rx.data_ptr(), my.data_ptr(),
        ry.data_ptr(), oc.data_ptr(), n, m, n, k, abi.stream_ptr()))
    return out.to(out_dtype).reshape(*x.shape[:-1], n)


def linear_int8(x, weight_info, out_dtype=torch.float16):
    qtype = weight_info["qtype"]
    if qtype == "int8_per_tensor":
        return linear_int8_per_tensor(x, weight_info, out_dtype)
    if qtype == "int8_affine":
        return linear_int8_affine(x, weight_info, out_dtype)
    raise ValueError(f"Unknown INT8 qtype: {qtype}")
