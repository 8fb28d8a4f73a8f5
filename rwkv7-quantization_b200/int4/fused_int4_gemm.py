"""INT4 GEMV entry points with the names of the reference's int4/fused_int4_gemm.py.  The reference's Triton
kernels take one activation vector [K]; these also take [M, K] (any M, processed 16 rows per launch)."""
from __future__ import annotations

import os

import torch

import rwkvq_abi as abi
from int4.int4_ops import _rows_f16, _run_rows, _f32

TRITON_AVAILABLE = False      # kept for importers; nothing here uses Triton


def _squeeze(out: torch.Tensor, x: torch.Tensor) -> torch.Tensor:
    return out.reshape(-1) if x.dim() == 1 else out.reshape(*x.shape[:-1], out.shape[-1])


def linear_int4_gemv_triton(x: torch.Tensor, packed: torch.Tensor, scale: torch.Tensor) -> torch.Tensor:
    """Per-tensor INT4 GEMV (int4/fused_int4_gemm.py:174-182)."""
    from int4.int4_ops import linear_int4_per_tensor
    return _squeeze(linear_int4_per_tensor(x.reshape(-1, x.shape[-1]), {"packed": packed, "scale": scale}), x)


def linear_int4_affine_gemv_triton(x, packed, mx, rx, my, ry) -> torch.Tensor:
    """MM4 GEMV (int4/fused_int4_gemm.py:185-194)."""
    from int4.int4_ops import linear_int4_affine
    info = {"packed": packed, "mx": mx, "rx": rx, "my": my, "ry": ry, "m_orig": x.shape[-1]}
    return _squeeze(linear_int4_affine(x.reshape(-1, x.shape[-1]), info), x)


_slices_cache: dict = {}


def _ksplit_slices(m: int, n: int, k: int) -> int:
    sl = _slices_cache.get((m, n, k))
    if sl is None:
        sl = _slices_cache[(m, n, k)] = int(abi.lib().rwkvq_gemv_int4_ksplit_slices(m, n, k))
    return sl


def _groupwise_rows(x, packed, scales, zeros, group_size: int) -> torch.Tensor:
    n, k = packed.shape[0], packed.shape[1] * 2
    x2 = _rows_f16(x, k)
    dev = x2.device
    scale_f16 = scales.dtype == torch.float16
    scales = scales.to(dev).contiguous() if scale_f16 else _f32(scales, dev)
    zeros = None if zeros is None else _f32(zeros, dev)
    generic = lambda xc, oc, m: abi.call(
        "rwkvq_gemv_int4_group_generic", xc.data_ptr(), k, packed.data_ptr(), packed.stride(0), scales.data_ptr(),
        abi.ptr(zeros), int(scale_f16), group_size, oc.data_ptr(), n, m, n, k, abi.stream_ptr())
    if os.environ.get("RWKVQ_INT4", "fast") == "generic" or group_size not in (128, 256) or k % 128:
        return _run_rows(x2, n, generic)
    if (group_size == 128 and not scale_f16 and k % 512 == 0 and scales.data_ptr() % 16 == 0
            and (zeros is None or zeros.data_ptr() % 16 == 0) and os.environ.get("RWKVQ_INT4_KSPLIT", "1") != "0"):
        # blocks too large to sit beside a deep weight ring (many rows, long rows): K in slices, fp32 partial sums, one
        # pass over the weights instead of one per block of rows
        def split(xc, oc, m):
            sl = _ksplit_slices(m, n, k)
            if sl > 1:
                ws = abi.plain_scratch(sl * m * n * 4, dev)
                abi.call("rwkvq_gemv_int4_group_ksplit", xc.data_ptr(), k, packed.data_ptr(), packed.stride(0), scales.data_ptr(),
                         abi.ptr(zeros), oc.data_ptr(), n, m, n, k, ws.data_ptr(), ws.numel(), abi.stream_ptr())
            else:
                abi.call("rwkvq_gemv_int4_group", xc.data_ptr(), k, packed.data_ptr(), packed.stride(0), scales.data_ptr(),
                         abi.ptr(zeros), 0, group_size, oc.data_ptr(), n, m, n, k, abi.stream_ptr())
        if _ksplit_slices(min(16, x2.shape[0]), n, k) >= 1:
            return _run_rows(x2, n, split, 16)
    # the streaming kernel keeps its rows of activations in shared memory: as many rows per launch as fit
    rows = 16
    while rows > 1 and abi.lib().rwkvq_gemv_int4_group_smem_bytes(rows, k) > 200 * 1024:
        rows //= 2
    if abi.lib().rwkvq_gemv_int4_group_smem_bytes(rows, k) > 200 * 1024:
        return _run_rows(x2, n, generic)
    return _run_rows(x2, n, lambda xc, oc, m: abi.call(
        "rwkvq_gemv_int4_group", xc.data_ptr(), k, packed.data_ptr(), packed.stride(0), scales.data_ptr(),
        abi.ptr(zeros), int(scale_f16), group_size, oc.data_ptr(), n, m, n, k, abi.stream_ptr()), rows)


def linear_int4_groupwise_gemv_triton(x, packed, scales, zeros, group_size: int) -> torch.Tensor:
    """Group-wise INT4 GEMV (int4/fused_int4_gemm.py:197-207)."""
    return _squeeze(_groupwise_rows(x.reshape(-1, x.shape[-1]), packed, scales, zeros, group_size), x)
