"""INT8 W8A16 GEMV entry points with the names of the reference's int8/fused_int8_gemm.py ([K] or [M, K] input)."""
from __future__ import annotations

import torch

TRITON_AVAILABLE = False      # kept for importers; nothing here uses Triton


def _squeeze(out, x):
    return out.reshape(-1) if x.dim() == 1 else out.reshape(*x.shape[:-1], out.shape[-1])


def linear_int8_gemv_triton(x: torch.Tensor, w_int8: torch.Tensor, scale: torch.Tensor) -> torch.Tensor:
    """Per-tensor W8A16 GEMV (int8/fused_int8_gemm.py:106-120)."""
    from int8.int8_ops import linear_int8_per_tensor
    return _squeeze(linear_int8_per_tensor(x.reshape(-1, x.shape[-1]), {"weight": w_int8, "tensor_scale": scale}), x)


def linear_int8_affine_gemv_triton(x, w_u8, mx, rx, my, ry) -> torch.Tensor:
    """MM8 GEMV (int8/fused_int8_gemm.py:123-139)."""
    from int8.int8_ops import linear_int8_affine
    return _squeeze(linear_int8_affine(x.reshape(-1, x.shape[-1]), {"weight": w_u8, "mx": mx, "rx": rx, "my": my, "ry": ry}), x)
