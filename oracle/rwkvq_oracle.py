"""CPU restatement of the quantized-projection path of AUXStar/rwkv7-quantization.

THIS IS TEST INFRASTRUCTURE, NOT PRODUCT CODE.  Only the test-suite, the smoke
check and the CPU-baseline leg of the benchmark may import it; the shipped
path (the C-ABI library and the Python modules that wrap it) never does.

Every function follows the reference operation for operation and cites the
reference file:line it restates.  Tensors are torch CPU tensors (the reference
is torch/Triton code, so torch's own rounding primitives -- `round()` =
half-to-even, fp32 -> bf16 / fp16 / e4m3 round-to-nearest-even -- are the
ones that define the result); `e4m3_encode` / `e2m1_encode` are independent
numpy encoders used to cross-check torch's casts and to build NVFP4, for which
torch has no CPU cast.

Parity status
  * weight quantizers (schemes.py, int4/quantize_int4.py, int8/quantize_int8.py),
    INT4 / INT8 dequant-matmul (int4_ops.py, int8_ops.py) and the INT8 W8A8
    kernels (fused_fp8_gemm.py, run under the Triton CPU interpreter) are PINNED
    by golden vectors produced by importing the reference itself
    (tests/golden/make_golden.py).
  * the FP8 kernels are pinned for their activation-preparation outputs
    (bf16 copy, amax); the e4m3 cast of the Triton interpreter is wrong, so
    FP8 codes/outputs are pinned against torch's e4m3 cast only.
  * NVFP4 has no code in the reference (only prose): PARITY UNPINNED.

Division: the reference's Triton kernels divide with PTX `div.full.f32`
(<= 2 ulp, hardware defined) when they run on a GPU, and with IEEE division
under the interpreter.  Every function that divides takes `div=`; the default
is IEEE.  GPU tests pass a `div` that evaluates the handful of scalar
divisions on the device, so codes and scales can be compared bit for bit.
"""
from __future__ import annotations

import numpy as np
import torch

F8_MAX = 448.0
E2M1_MAX = 6.0
NVFP4_BLOCK = 16


# --------------------------------------------------------------------------- #
# scalar formats
# --------------------------------------------------------------------------- #
def ieee_div(a: torch.Tensor, b) -> torch.Tensor:
    """fp32 IEEE round-to-nearest division (torch CPU)."""
    a = torch.as_tensor(a, dtype=torch.float32)
    b = torch.as_tensor(b, dtype=torch.float32)
    return a / b


def e4m3_decode(code: np.ndarray) -> np.ndarray:
    """uint8 e4m3fn bit pattern -> float32 value (0x7f / 0xff are NaN)."""
    c = np.asarray(code, dtype=np.uint8).astype(np.int32)
    s = (c >> 7) & 1
    e = (c >> 3) & 0xF
    m = c & 7
    mag = np.where(e == 0, m * 2.0 ** -9, (1.0 + m / 8.0) * np.exp2(e.astype(np.float64) - 7.0))
    mag = np.where((e == 15) & (m == 7), np.nan, mag)
    return np.where(s == 1, -mag, mag).astype(np.float32)


_E4M3_POS = e4m3_decode(np.arange(0, 127, dtype=np.uint8)).astype(np.float64)  # 0 .. 448, ascending


def e4m3_encode(x: np.ndarray) -> np.ndarray:
    """float32 -> e4m3fn bit pattern, round-to-nearest-even, saturating to +-448
    (the behaviour of `cvt.rn.satfinite.e4m3x2.f32`, which the reference's
    `.to(tl.float8e4nv)` lowers to on sm_100; fused_fp8_gemm.py:250,359)."""
    x = np.asarray(x, dtype=np.float32)
    a = np.minimum(np.abs(x).astype(np.float64), 448.0)
    hi = np.searchsorted(_E4M3_POS, a, side="left")          # first code with value >= a
    hi = np.clip(hi, 0, 126)
    lo = np.clip(hi - 1, 0, 126)
    dlo = a - _E4M3_POS[lo]
    dhi = _E4M3_POS[hi] - a
    pick_lo = (dlo < dhi) | ((dlo == dhi) & (lo % 2 == 0))
    code = np.where(pick_lo, lo, hi).astype(np.uint8)
    code = np.where(np.isnan(x), np.uint8(0x7F), code)
    sign = (np.signbit(x).astype(np.uint8) << 7).astype(np.uint8)
    return (code | sign).astype(np.uint8)


_E2M1_POS = np.array([0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0])


def e2m1_decode(code: np.ndarray) -> np.ndarray:
    c = np.asarray(code, dtype=np.uint8).astype(np.int32)
    mag = _E2M1_POS[c & 7]
    return np.where((c >> 3) & 1, -mag, mag).astype(np.float32)


def e2m1_encode(x: np.ndarray) -> np.ndarray:
    """float32 -> 4-bit e2m1 code (sign<<3 | index), round-to-nearest-even on the
    value grid {0,.5,1,1.5,2,3,4,6}, saturating (behaviour of
    `cvt.rn.satfinite.e2m1x2.f32`)."""
    x = np.asarray(x, dtype=np.float32)
    a = np.minimum(np.abs(x).astype(np.float64), 6.0)
    hi = np.clip(np.searchsorted(_E2M1_POS, a, side="left"), 0, 7)
    lo = np.clip(hi - 1, 0, 7)
    dlo = a - _E2M1_POS[lo]
    dhi = _E2M1_POS[hi] - a
    pick_lo = (dlo < dhi) | ((dlo == dhi) & (lo % 2 == 0))
    code = np.where(pick_lo, lo, hi).astype(np.uint8)
    sign = (np.signbit(x).astype(np.uint8) << 3).astype(np.uint8)
    return (code | sign).astype(np.uint8)


def _to_e4m3(t: torch.Tensor) -> torch.Tensor:
    """fp32 tensor (already clamped to +-448) -> torch.float8_e4m3fn, RNE."""
    return t.to(torch.float8_e4m3fn)


# --------------------------------------------------------------------------- #
# offline weight quantizers -- schemes.py
# --------------------------------------------------------------------------- #
def q_fp8(w: torch.Tensor):
    """schemes.py:18-24 -- per-tensor e4m3; note the integer round() before the cast."""
    amax = w.abs().max().clamp(min=1e-12)
    scale = (amax / F8_MAX).float()
    w_q = (w.float() / scale).clamp(-F8_MAX, F8_MAX).round().to(torch.float8_e4m3fn)
    return w_q, scale


def q_fp8_perchannel(w: torch.Tensor):
    """schemes.py:26-34 -- per-output-row e4m3."""
    if w.dim() == 1:
        return q_fp8(w)
    amax = w.abs().amax(dim=1, keepdim=True).clamp(min=1e-12)
    scale = (amax / F8_MAX).float()
    w_q = (w.float() / scale).clamp(-F8_MAX, F8_MAX).round().to(torch.float8_e4m3fn)
    return w_q, scale.squeeze(1)


def q_int8_sym(w: torch.Tensor):
    """schemes.py:36-42 -- per-tensor symmetric int8."""
    amax = w.abs().max().clamp(min=1e-12)
    scale = (amax / 127.0).float()
    w_q = (w.float() / scale).round().clamp(-128, 127).to(torch.int8)
    return w_q, scale


def q_int8_affine(w: torch.Tensor):
    """schemes.py:44-62 -- MM8 simulated quantization (returns a float tensor)."""
    wf = w.float()
    if wf.dim() != 2:
        wf = wf.reshape(1, -1)
    my = wf.amin(dim=1, keepdim=True)
    w2 = wf - my
    mx = w2.amin(dim=0, keepdim=True)
    w2 = w2 - mx
    rx = w2.amax(dim=0, keepdim=True).clamp(min=1e-12)
    w2 = w2 / rx
    ry = w2.amax(dim=1, keepdim=True).clamp(min=1e-12)
    w2 = w2 / ry
    wq = (w2 * 256.0).floor().clamp(0, 255)
    approx = (wq + 0.5) * (ry * 16.0) * (rx * 16.0) + my + mx
    if w.dim() != 2:
        approx = approx.reshape(w.shape)
    return approx.to(w.dtype)


def q_int4_sym(w: torch.Tensor):
    """schemes.py:64-70 -- per-tensor symmetric int4, simulated."""
    amax = w.abs().max().clamp(min=1e-12)
    scale = (amax / 7.0).float()
    w_q = (w.float() / scale).round().clamp(-8, 7)
    return (w_q * scale).to(w.dtype)


def q_int4_gw(w: torch.Tensor, group_size: int = 128):
    """schemes.py:72-94 -- group-wise asymmetric int4, simulated, K padded to the group."""
    wf = w.float()
    shape = wf.shape
    if wf.dim() != 2:
        wf = wf.reshape(1, -1)
    n, m = wf.shape
    pad = (group_size - m % group_size) % group_size
    if pad:
        wf = torch.nn.functional.pad(wf, (0, pad))
        m = wf.shape[1]
    wg = wf.reshape(n, m // group_size, group_size)
    wmin = wg.amin(dim=2, keepdim=True)
    wmax = wg.amax(dim=2, keepdim=True)
    scale = ((wmax - wmin) / 15.0).clamp(min=1e-12)
    wq = ((wg - wmin) / scale).round().clamp(0, 15)
    approx = (wq * scale + wmin).reshape(n, m)[:, : shape[-1]]
    if approx.numel() == torch.Size(shape).numel():
        approx = approx.reshape(shape)
    return approx.to(w.dtype)


# --------------------------------------------------------------------------- #
# stand-alone INT4 / INT8 tools -- int4/quantize_int4.py, int8/quantize_int8.py
# --------------------------------------------------------------------------- #
def quantize_to_int4_per_tensor(w: torch.Tensor):
    """int4/quantize_int4.py:51-71 -- signed nibble, scale=max/7, two per byte along K."""
    w = w.float()
    assert w.shape[1] % 2 == 0
    scale = (w.abs().max() / 7.0).clamp(min=1e-12)
    w_q = (w / scale).round().clamp(-8, 7).to(torch.int8)
    lo = (w_q[:, 0::2] & 0xF).to(torch.uint8)
    hi = (w_q[:, 1::2] & 0xF).to(torch.uint8)
    return lo | (hi << 4), scale.to(torch.float32)


def quantize_to_int4_affine(w: torch.Tensor):
    """int4/quantize_int4.py:78-135 -- MM4: row/col offsets and ranges, floor(w*16)."""
    w = w.float()
    n, m = w.shape
    if m % 2:
        w = torch.nn.functional.pad(w, (0, 1))
    my = w.amin(dim=1, keepdim=True)
    w = w - my
    mx = w.amin(dim=0, keepdim=True)
    w = w - mx
    rx = w.amax(dim=0, keepdim=True).clamp(min=1e-12)
    w = w / rx
    ry = w.amax(dim=1, keepdim=True).clamp(min=1e-12)
    w = w / ry
    u4 = (w * 16.0).floor().clamp(0, 15).to(torch.uint8)
    packed = u4[:, 0::2] | (u4[:, 1::2] << 4)
    return {
        "packed": packed,
        "mx": mx.squeeze(0).float(),
        "rx": (rx / 4.0).squeeze(0).float(),
        "my": my.squeeze(1).float(),
        "ry": (ry / 4.0).squeeze(1).float(),
        "m_orig": m,
    }


def quantize_to_int4_groupwise(w: torch.Tensor, group_size: int = 128):
    """int4/quantize_int4.py:142-185 -- asymmetric uint4 per group of K, fp32 scale+zero."""
    w = w.float()
    n, k = w.shape
    assert k % group_size == 0 and k % 2 == 0
    g = w.reshape(n, k // group_size, group_size)
    wmin = g.amin(dim=2, keepdim=True)
    wmax = g.amax(dim=2, keepdim=True)
    scale = ((wmax - wmin) / 15.0).clamp(min=1e-12)
    q = ((g - wmin) / scale).round().clamp(0, 15).to(torch.uint8).reshape(n, k)
    packed = q[:, 0::2] | (q[:, 1::2] << 4)
    return {
        "packed": packed,
        "scales": scale.squeeze(2).float(),
        "zeros": wmin.squeeze(2).float(),
        "group_size": group_size,
    }


def quantize_to_int8_per_tensor(w: torch.Tensor):
    """int8/quantize_int8.py:51-62."""
    w = w.float()
    scale = (w.abs().max() / 127.0).clamp(min=1e-12)
    return (w / scale).round().clamp(-128, 127).to(torch.int8), scale.to(torch.float32)


def quantize_to_int8_affine(w: torch.Tensor):
    """int8/quantize_int8.py:69-114 -- MM8, floor(w*256), ranges stored /16."""
    w = w.float()
    my = w.amin(dim=1, keepdim=True)
    w = w - my
    mx = w.amin(dim=0, keepdim=True)
    w = w - mx
    rx = w.amax(dim=0, keepdim=True).clamp(min=1e-12)
    w = w / rx
    ry = w.amax(dim=1, keepdim=True).clamp(min=1e-12)
    w = w / ry
    u8 = (w * 256.0).floor().clamp(0, 255).to(torch.uint8)
    return {
        "w_u8": u8,
        "mx": mx.squeeze(0).float(),
        "rx": (rx / 16.0).squeeze(0).float(),
        "my": my.squeeze(1).float(),
        "ry": (ry / 16.0).squeeze(1).float(),
    }


def unpack_int4(packed: torch.Tensor) -> torch.Tensor:
    """int4/int4_ops.py:18-31 -- low nibble is the even K index."""
    lo = packed & 0x0F
    hi = (packed >> 4) & 0x0F
    return torch.stack([lo, hi], dim=-1).reshape(packed.shape[0], -1).to(torch.int8)


# dequantized weights, fp32 (the value every W4A16 / W8A16 kernel multiplies by)
def dequant_int4_per_tensor(info) -> torch.Tensor:
    """int4/int4_ops.py:79-101 (weight part): signed nibble * scale."""
    u = unpack_int4(info["packed"]).float()
    return torch.where(u > 7, u - 16, u) * info["scale"]


def dequant_int4_affine(info) -> torch.Tensor:
    """int4/int4_ops.py:104-130 (weight part): (u4+.5)*ry*rx*16 + my + mx, trimmed to m_orig."""
    u = unpack_int4(info["packed"]).float()
    n, mp = u.shape
    w = (u + 0.5) * info["ry"].reshape(n, 1) * info["rx"].reshape(1, mp) * 16.0 \
        + info["my"].reshape(n, 1) + info["mx"].reshape(1, mp)
    return w[:, : info["m_orig"]]


def dequant_int4_groupwise(info) -> torch.Tensor:
    """int4/int4_ops.py:133-151 (weight part): u4*scale[g] + zero[g]."""
    u = unpack_int4(info["packed"]).float()
    n, k = u.shape
    g = info["group_size"]
    w = u.reshape(n, k // g, g) * info["scales"].reshape(n, k // g, 1).float() \
        + info["zeros"].reshape(n, k // g, 1).float()
    return w.reshape(n, k)


def dequant_int8_per_tensor(info) -> torch.Tensor:
    """int8/int8_ops.py:48-78 (weight part), fp32 form."""
    return info["weight"].float() * info["tensor_scale"].float()


def dequant_int8_affine(info) -> torch.Tensor:
    """int8/int8_ops.py:81-110 (weight part): (u8+.5)*ry*rx*256 + my + mx."""
    u = info["weight"].float()
    n, m = u.shape
    return (u + 0.5) * info["ry"].reshape(n, 1) * info["rx"].reshape(1, m) * 256.0 \
        + info["my"].reshape(n, 1) + info["mx"].reshape(1, m)


def linear_ref_fp16_dequant(x: torch.Tensor, w_fp32: torch.Tensor, out_dtype=torch.float16):
    """The reference's executable CPU path for every INT4 / stand-alone INT8 scheme
    (int4_ops.py:99-101,127-130,153-157; int8_ops.py:72-78,104-110): dequantize the
    whole weight to fp16, then an fp16 matmul."""
    w16 = w_fp32.to(torch.float16)
    x2 = x.reshape(-1, x.shape[-1]).to(torch.float16)
    out = x2 @ w16.t()
    return out.to(out_dtype).reshape(*x.shape[:-1], w16.shape[0])


def linear_w4a16_kernel_semantics(x: torch.Tensor, w_fp32: torch.Tensor):
    """What the reference's W4A16 / W8A16 GEMV kernels are written to compute
    (int4/fused_int4_gemm.py:120-171, int8/fused_int8_gemm.py:32-103): x and the
    dequantized weight both in fp32, fp32 accumulation, fp16 result."""
    x2 = x.reshape(-1, x.shape[-1]).float()
    out = (x2.double() @ w_fp32.double().t()).float()
    return out.to(torch.float16).reshape(*x.shape[:-1], w_fp32.shape[0])


# --------------------------------------------------------------------------- #
# activation preparation -- fused_fp8_gemm.py
# --------------------------------------------------------------------------- #
def _as_2d_16bit(x: torch.Tensor) -> torch.Tensor:
    x2 = x.reshape(-1, x.shape[-1])
    if x2.dtype not in (torch.float16, torch.bfloat16):
        x2 = x2.to(torch.bfloat16)
    return x2.contiguous()


def prep_x(x: torch.Tensor, awq_scale=None, div=ieee_div):
    """fused_fp8_gemm.py:30-79 -- bf16 copy of fp32(x)[/awq] and ONE amax for the whole call
    (taken before the bf16 rounding, accumulated from zero)."""
    x2 = _as_2d_16bit(x)
    xf = x2.float()
    if awq_scale is not None:
        xf = div(xf, awq_scale.float().reshape(1, -1))
    amax = xf.abs().max().reshape(1) if xf.numel() else torch.zeros(1)
    amax = torch.maximum(amax, torch.zeros(1))
    return xf.to(torch.bfloat16), amax.float()


def prep3_x(xr, xk, xv, awq_r=None, awq_k=None, div=ieee_div):
    """fused_fp8_gemm.py:86-150 -- prep_x for r, k, v; AWQ only on r and k."""
    o_r, a_r = prep_x(xr, awq_r, div)
    o_k, a_k = prep_x(xk, awq_k, div)
    o_v, a_v = prep_x(xv, None, div)
    return o_r, o_k, o_v, a_r, a_k, a_v


def prep_x_fp8(x: torch.Tensor):
    """fused_fp8_gemm.py:341-390 -- per-call amax; inv = 448/clamp(amax,1e-12) and x_scale = amax/448 as torch
    evaluates them ON A GPU, which is where the reference runs: `scalar / tensor` is reciprocal-then-multiply
    (Tensor.__rtruediv__), `tensor / python scalar` multiplies by the fp32-rounded reciprocal of the scalar (the CUDA
    true-division kernel's scalar fast path).  Both checked bit for bit against the reference's outputs recorded on a
    B200 (tests/golden/fp8_triton_b200.npz).  codes = RNE(clamp(x*inv, +-448))."""
    x2 = _as_2d_16bit(x)
    xf = x2.float()
    amax = torch.maximum(xf.abs().max().reshape(1), torch.zeros(1)).float()
    inv = amax.clamp(min=1e-12).reciprocal() * torch.tensor(F8_MAX, dtype=torch.float32)
    codes = _to_e4m3((xf * inv).clamp(-F8_MAX, F8_MAX))
    return codes, amax * (torch.tensor(1.0, dtype=torch.float32) / torch.tensor(F8_MAX, dtype=torch.float32))


def prep_x_int8(x: torch.Tensor, div=ieee_div):
    """fused_fp8_gemm.py:687-731 -- per-ROW amax (floor 1e-12), s = 127/amax,
    code = trunc(clamp(x*s, -128, 127)), stored scale = amax/127."""
    x2 = _as_2d_16bit(x)
    xf = x2.float()
    amax = xf.abs().amax(dim=1).clamp(min=1e-12)
    s = div(torch.full_like(amax, 127.0), amax)
    codes = (xf * s[:, None]).clamp(-128.0, 127.0).trunc().to(torch.int8)
    return codes, div(amax, torch.full_like(amax, 127.0))


# --------------------------------------------------------------------------- #
# FP8 W8A8 linears -- fused_fp8_gemm.py, fp8_ops.py
# --------------------------------------------------------------------------- #
def _fp8_codes_from_bf16(x_bf16: torch.Tensor, amax: torch.Tensor, div):
    """In-kernel activation quantization (fused_fp8_gemm.py:240-250, 292-325, 626-634)."""
    amax_v = amax.float().clamp(min=1e-12)
    inv = div(torch.full_like(amax_v, F8_MAX), amax_v)
    a = _to_e4m3((x_bf16.float() * inv).clamp(-F8_MAX, F8_MAX))
    return a, amax_v


def _fp8_scaled_out(a_codes, w_codes, amax_v, w_ts, div):
    """acc = sum_k a*w in fp32 (here: float64 then rounded, the order-independent limit);
    out = fp16(acc * (amax/448 * w_ts))  (fused_fp8_gemm.py:253-257).  A weight scale of N values (the
    "fp8_perchannel" scheme, schemes.py:26-34; no reference kernel consumes it) scales output column n by w_ts[n]."""
    acc = (a_codes.float().double() @ w_codes.float().double().t()).float()
    wv = w_ts.float().reshape(-1)
    s = div(amax_v, torch.full_like(amax_v, F8_MAX)) * (wv[0] if wv.numel() == 1 else wv.reshape(1, -1))
    return (acc * s).to(torch.float16)


def linear_fp8_m1_fused(x, weight_info, div=ieee_div):
    """fused_fp8_gemm.py:600-679 -- M == 1: x -> bf16 FIRST (:662), amax over the bf16 values."""
    w, w_ts = weight_info["weight"], weight_info["tensor_scale"]
    x1 = x.reshape(1, -1).contiguous()
    if x1.dtype == torch.float16:
        x1 = x1.to(torch.bfloat16)
    amax = x1.float().abs().max().reshape(1)
    a, amax_v = _fp8_codes_from_bf16(x1, amax, div)
    out = _fp8_scaled_out(a, w, amax_v, w_ts, div)
    return out.reshape(*x.shape[:-1], w.shape[0])


def linear_fp8_fused(x, weight_info, div=ieee_div):
    """fused_fp8_gemm.py:1020-1077 -- M == 1 -> m1 kernel; else prep_x (amax on the input
    dtype, bf16 copy) + hardware-dot GEMM quantizing the bf16 copy."""
    m = x.numel() // x.shape[-1]
    if m == 1:
        return linear_fp8_m1_fused(x, weight_info, div)
    w, w_ts = weight_info["weight"], weight_info["tensor_scale"]
    xb, amax = prep_x(x, None, div)
    a, amax_v = _fp8_codes_from_bf16(xb, amax, div)
    out = _fp8_scaled_out(a, w, amax_v, w_ts, div)
    return out.reshape(*x.shape[:-1], w.shape[0])


def linear_rkv_fused(xr, xk, xv, wr, wk, wv, div=ieee_div):
    """fused_fp8_gemm.py:944-1017, 264-334 -- three GEMMs, three amax, three weight scales."""
    outs = []
    prepped = prep3_x(xr, xk, xv, wr.get("awq_scale"), wk.get("awq_scale"), div)
    for xb, amax, info in zip(prepped[:3], prepped[3:], (wr, wk, wv)):
        a, amax_v = _fp8_codes_from_bf16(xb, amax, div)
        o = _fp8_scaled_out(a, info["weight"], amax_v, info["tensor_scale"], div)
        outs.append(o.reshape(*xr.shape[:-1], info["weight"].shape[0]))
    return tuple(outs)


def relu_square(x: torch.Tensor) -> torch.Tensor:
    """The engine's relu_square on fp16 (cuda/rwkv7_fast_ops_fp16.cu:787-799): fp16(max(float(x), 0)^2)."""
    v = x.to(torch.float16).float().clamp(min=0.0)
    return (v * v).to(torch.float16)


def ffn_relu2_fp8(x, key_info, value_info, div=ieee_div):
    """key projection -> relu_square -> value projection as the engine chains them (rwkv7_fast_v3a.py:1109, 1136-1144)."""
    hid = relu_square(linear_fp8_fused(x, key_info, div))
    return linear_fp8_fused(hid, value_info, div), hid


def ffn_relu2_int8(x, key_info, value_info, div=ieee_div):
    """The same chain on INT8 weights: each projection quantizes its input per row (fused_fp8_gemm.py:785-818)."""
    hid = relu_square(linear_int8_fused(x, key_info, div))
    return linear_int8_fused(hid, value_info, div), hid


def linear_fp8(x, weight_info, out_dtype=torch.float16):
    """fp8_ops.py:58-86 -- M > 512: fp16 -> bf16, prep_x_fp8, scaled matmul with a
    bf16 result, then the cast to fp16 (the result passes through bf16)."""
    w, w_ts = weight_info["weight"], weight_info["tensor_scale"]
    x2 = x.reshape(-1, x.shape[-1]).contiguous()
    if x2.dtype == torch.float16:
        x2 = x2.to(torch.bfloat16)
    codes, xs = prep_x_fp8(x2)
    acc = (codes.float().double() @ w.float().double().t()).float()
    wv = w_ts.float().reshape(-1)
    out = (acc * (xs.float() * (wv[0] if wv.numel() == 1 else wv.reshape(1, -1)))).to(torch.bfloat16)
    return out.reshape(*x.shape[:-1], w.shape[0]).to(out_dtype)


# --------------------------------------------------------------------------- #
# INT8 W8A8 linears -- fused_fp8_gemm.py
# --------------------------------------------------------------------------- #
def int8_acc(x_codes: torch.Tensor, w_codes: torch.Tensor) -> torch.Tensor:
    """int32 accumulators of fused_int8_gemm_kernel (fused_fp8_gemm.py:767-776); exact."""
    return (x_codes.to(torch.int32) @ w_codes.to(torch.int32).t()).to(torch.int32)


def linear_int8_fused(x, weight_info, div=ieee_div, return_acc=False):
    """fused_fp8_gemm.py:734-818 -- out = fp16(float(acc) * (x_scale[m] * w_scale))."""
    w, w_s = weight_info["weight"], weight_info["tensor_scale"]
    codes, xs = prep_x_int8(x, div)
    acc = int8_acc(codes, w)
    out = (acc.float() * (xs[:, None] * w_s.float().reshape(-1)[0])).to(torch.float16)
    out = out.reshape(*x.shape[:-1], w.shape[0])
    return (out, acc) if return_acc else out


def linear_rkv_int8_fused(xr, xk, xv, wr, wk, wv, div=ieee_div, shared_scale=True):
    """fused_fp8_gemm.py:825-934 -- the reference multiplies k and v by r's weight scale
    (:855-857, :906); `shared_scale=False` gives each its own."""
    outs = []
    for x, info in ((xr, wr), (xk, wk), (xv, wv)):
        eff = dict(info)
        if shared_scale:
            eff["tensor_scale"] = wr["tensor_scale"]
        outs.append(linear_int8_fused(x, eff, div))
    return tuple(outs)


# --------------------------------------------------------------------------- #
# NVFP4 W4A4 (no code in the reference: restated from its reports; parity unpinned)
# --------------------------------------------------------------------------- #
def _nvfp4_quantize_rows(xf: torch.Tensor, amax: torch.Tensor, div=ieee_div):
    """Block-scaled e2m1 quantization of rows of fp32 values.

    iterations/phase1_nvfp4_exploration/reports/03_fused_kernel_en.md:22-34 and
    iterations/phase3_x5_residual_scheme/reports/11_fused_gemm_ops_en.md:20-26:
      pts        = amax / 2688                      (2688 = 448 * 6)
      block scale= e4m3( clamp(max_abs_16 * 448 / amax, 2^-6, 448) )
      code       = e2m1_RNE( x * (1/pts) / block_scale )
    Returns (packed uint8 [M,K/2] low nibble = even k, block scales e4m3 bits uint8 [M,K/16], pts fp32[1]).
    """
    m, k = xf.shape
    assert k % NVFP4_BLOCK == 0
    amax_v = amax.float().reshape(1).clamp(min=1e-12)
    pts = div(amax_v, torch.full_like(amax_v, 2688.0))
    blk = xf.reshape(m, k // NVFP4_BLOCK, NVFP4_BLOCK)
    bmax = blk.abs().amax(dim=2)
    sb = (bmax * div(torch.full_like(amax_v, F8_MAX), amax_v)).clamp(2.0 ** -6, F8_MAX)
    bs_bits = e4m3_encode(sb.numpy())
    bs_val = torch.from_numpy(e4m3_decode(bs_bits))
    inv_pts = div(torch.ones_like(pts), pts)
    scaled = blk * inv_pts / bs_val[:, :, None]
    codes = e2m1_encode(scaled.reshape(m, k).numpy())
    packed = (codes[:, 0::2] | (codes[:, 1::2] << 4)).astype(np.uint8)
    return torch.from_numpy(packed), torch.from_numpy(bs_bits), pts


def nvfp4_quantize_weight(w: torch.Tensor):
    """Offline NVFP4 weight quantization in the storage layout of
    iterations/phase1_nvfp4_exploration/reports/07_quantization_toolchain_v2_en.md:18-25:
    packed e2m1 [N,K/2], `.nf4_b_scale` e4m3 [N,K/16], `.nvfp4_t_scale` fp32 scalar."""
    wf = w.float()
    amax = wf.abs().max().reshape(1)
    packed, bs, pts = _nvfp4_quantize_rows(wf, amax)
    return {"weight": packed, "block_scale": bs, "tensor_scale": pts.reshape(()), "qtype": "nvfp4"}


def nvfp4_actq(x: torch.Tensor, div=ieee_div):
    """On-the-fly activation quantization (per-call amax, like prep_x)."""
    x2 = _as_2d_16bit(x)
    xf = x2.float()
    amax = torch.maximum(xf.abs().max().reshape(1), torch.zeros(1))
    return _nvfp4_quantize_rows(xf, amax, div)


def nvfp4_dequant(packed: torch.Tensor, bs_bits: torch.Tensor) -> torch.Tensor:
    """code * block_scale (without the per-tensor scale), fp32 [rows, K]."""
    p = packed.numpy()
    codes = np.empty((p.shape[0], p.shape[1] * 2), dtype=np.uint8)
    codes[:, 0::2] = p & 0xF
    codes[:, 1::2] = p >> 4
    v = e2m1_decode(codes)
    s = e4m3_decode(bs_bits.numpy())
    return torch.from_numpy(v * np.repeat(s, NVFP4_BLOCK, axis=1))


def linear_nvfp4(x, weight_info, div=ieee_div):
    """out = fp16( (sum codeA*codeB*bsA*bsB) * ptsA * ptsB )   (11_fused_gemm_ops_en.md:20-26)."""
    pa, ba, pts_a = nvfp4_actq(x, div)
    a = nvfp4_dequant(pa, ba)
    w = nvfp4_dequant(weight_info["weight"], weight_info["block_scale"])
    acc = (a.double() @ w.double().t()).float()
    out = (acc * (pts_a * weight_info["tensor_scale"].float().reshape(1))).to(torch.float16)
    return out.reshape(*x.shape[:-1], w.shape[0])


# --------------------------------------------------------------------------- #
# CPU baseline: the reference's own CPU route (quantize with schemes.py, then a torch
# CPU dequant-matmul), used by the benchmark's cpu_baseline leg.
# --------------------------------------------------------------------------- #
def cpu_dequant_matmul_fp8(x: torch.Tensor, weight_info) -> torch.Tensor:
    """fp8: w.float()*scale then a float matmul."""
    w = weight_info["weight"].float() * weight_info["tensor_scale"].float()
    return (x.reshape(-1, x.shape[-1]).float() @ w.t()).to(torch.float16)
