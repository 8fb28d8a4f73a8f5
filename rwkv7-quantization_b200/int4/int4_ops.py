"""INT4 weight detection, loading and projections (drop-in for the reference's int4/int4_ops.py).

Weight-info dicts are the reference's (int4/int4_ops.py:43-72):
    per_tensor : {"packed", "scale", "qtype": "int4_per_tensor"}
    affine     : {"packed", "mx", "rx", "my", "ry", "m_orig", "qtype": "int4_affine"}
    groupwise  : {"packed", "scales", "zeros", "group_size", "qtype": "int4_groupwise"}
The projections run on the device through librwkvq.so: weights stay packed in HBM and are dequantized in
registers (the reference materialises an fp16 copy of the whole matrix and calls an fp16 matmul).
"""
from __future__ import annotations

import torch

import rwkvq_abi as abi

GEMV_ROWS = 16      # rows of activations per kernel launch


def unpack_int4(packed: torch.Tensor) -> torch.Tensor:
    """[N, K/2] bytes -> [N, K] int8 values 0..15, low nibble first (int4/int4_ops.py:18-31)."""
    pair = torch.stack((packed & 0x0F, (packed >> 4) & 0x0F), dim=-1)
    return pair.reshape(packed.shape[0], -1).to(torch.int8)


def is_int4_weight(z: dict, key: str) -> bool:
    return key + ".int4_packed" in z


def load_int4_weight(z: dict, key: str, dev: str = "cuda"):
    """Collect the tensors stored beside `key` into a weight-info dict on `dev` (int4/int4_ops.py:43-72)."""
    if key + ".int4_packed" not in z:
        raise KeyError(f"No INT4 weight found for key: {key}")
    info = {"packed": z[key + ".int4_packed"].to(dev)}
    get = lambda suffix: z[key + ".int4_" + suffix]
    if key + ".int4_scale" in z:
        info.update(scale=get("scale").to(dev), qtype="int4_per_tensor")
    elif key + ".int4_rx" in z:
        info.update({n: get(n).to(dev) for n in ("mx", "rx", "my", "ry")}, m_orig=get("m_orig"), qtype="int4_affine")
    elif key + ".int4_scales" in z:
        info.update(scales=get("scales").to(dev), zeros=get("zeros").to(dev), group_size=get("group_size"),
                    qtype="int4_groupwise")
    else:
        raise KeyError(f"Incomplete INT4 metadata for key: {key}")
    return info


# --------------------------------------------------------------------------- device projections
def _rows_f16(x: torch.Tensor, k: int) -> torch.Tensor:
    x2 = x.reshape(-1, x.shape[-1]).to(torch.float16)
    if x2.shape[1] < k:                                   # MM4 pads odd K with one zero column
        x2 = torch.nn.functional.pad(x2, (0, k - x2.shape[1]))
    x2 = x2.contiguous()
    return x2 if x2.data_ptr() % 16 == 0 else x2.clone()


def _run_rows(x2: torch.Tensor, n: int, launch, block: int = GEMV_ROWS) -> torch.Tensor:
    """Call `launch(x_chunk, out_chunk, rows)` for blocks of `block` rows."""
    abi.require_device()
    if not x2.is_cuda:
        raise RuntimeError("rwkvq: INT4 / INT8 projections run on the GPU only (no CPU fallback)")
    out = torch.empty((x2.shape[0], n), dtype=torch.float16, device=x2.device)
    for r0 in range(0, x2.shape[0], block):
        rows = min(block, x2.shape[0] - r0)
        launch(x2[r0:r0 + rows], out[r0:r0 + rows], rows)
    return out


def _f32(t: torch.Tensor, dev) -> torch.Tensor:
    return t.to(device=dev, dtype=torch.float32).contiguous()


def linear_int4_per_tensor(x, weight_info, out_dtype=torch.float16):
    """W4A16 projection, per-tensor symmetric (int4/int4_ops.py:79-101)."""
    packed, scale = weight_info["packed"], weight_info["scale"]
    n, k = packed.shape[0], packed.shape[1] * 2
    x2 = _rows_f16(x, k)
    scale = _f32(scale.reshape(1), x2.device)
    out = _run_rows(x2, n, lambda xc, oc, m: abi.call(
        "rwkvq_gemv_int4_tensor", xc.data_ptr(), k, packed.data_ptr(), packed.stride(0), scale.data_ptr(), oc.data_ptr(),
        n, m, n, k, abi.stream_ptr()))
    return out.to(out_dtype).reshape(*x.shape[:-1], n)


def linear_int4_affine(x, weight_info, out_dtype=torch.float16):
    """MM4 projection (int4/int4_ops.py:104-130)."""
    packed = weight_info["packed"]
    n, k = packed.shape[0], packed.shape[1] * 2
    x2 = _rows_f16(x, k)
    mx, rx, my, ry = (_f32(weight_info[v], x2.device) for v in ("mx", "rx", "my", "ry"))
    out = _run_rows(x2, n, lambda xc, oc, m: abi.call(
        "rwkvq_gemv_int4_affine", xc.data_ptr(), k, packed.data_ptr(), packed.stride(0), mx.data_ptr(), rx.data_ptr(),
        my.data_ptr(), ry.data_ptr(), oc.data_ptr(), n, m, n, k, abi.stream_ptr()))
    return out.to(out_dtype).reshape(*x.shape[:-1], n)


def linear_int4_groupwise(x, weight_info, out_dtype=torch.float16):
    """Group-wise projection (int4/int4_ops.py:133-157): scales fp32 (reference layout) or fp16, zeros optional
    (absent = symmetric, zero = -8 * scale)."""
    from int4.fused_int4_gemm import _groupwise_rows
    packed = weight_info["packed"]
    n = packed.shape[0]
    out = _groupwise_rows(x, packed, weight_info["scales"], weight_info.get("zeros"), int(weight_info["group_size"]))
    return out.to(out_dtype).reshape(*x.shape[:-1], n)


def linear_int4(x, weight_info, out_dtype=torch.float16):
    """Dispatch on `qtype` (int4/int4_ops.py:160-172)."""
    qtype = weight_info["qtype"]
    if qtype == "int4_per_tensor":
        return linear_int4_per_tensor(x, weight_info, out_dtype)
    if qtype == "int4_affine":
        return linear_int4_affine(x, weight_info, out_dtype)
    if qtype == "int4_groupwise":
        return linear_int4_groupwise(x, weight_info, out_dtype)
    raise ValueError(f"Unknown INT4 qtype: {qtype}")
