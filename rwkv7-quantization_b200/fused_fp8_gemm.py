"""Drop-in for the reference module `fused_fp8_gemm.py`: same public names, argument meaning and return
shapes, with every device kernel replaced by librwkvq.so (hand-written CUDA for sm_100a, see include/rwkvq.h).

    prep_x / prep3_x / prep_x_fp8 / prep_x_int8 / prep3_x_int8     activation preparation
    linear_fp8_m1_fused / linear_fp8_fused / linear_rkv_fused       FP8 W8A8 projections
    linear_int8_fused / linear_rkv_int8_fused                       INT8 W8A8 projections
    linear_quantized_fused                                          dispatcher used by the engine

Outputs are freshly allocated tensors owned by the caller; weights are borrowed; launches go to torch's current
CUDA stream without host synchronisation -- the conventions of the reference wrappers
(fused_fp8_gemm.py:55-79, 645-679, 785-818, 944-1098).

Routing by M = rows of the flattened activation:
    M <= 8      ONE fused launch of the weight-streaming GEMV (activation quantization in its prologue, weights
                streamed once from HBM through per-warp cp.async rings into mma.sync fragments) -- the decode path
    9 .. 32     (and from 3 rows on when K is long) the same weight-streaming kernel on PRE-QUANTIZED codes: one small
                quantization launch (r, k, v together; a cluster of CTAs per tensor, launched with programmatic
                dependent launch), then every CTA copies the M*K bytes of codes instead of re-quantizing the whole
                block -- with many rows the per-CTA quantization (bound by the SMs' conversion throughput) costs more
                than the weight stream it precedes.  RWKVQ_CODES_M_MIN moves the boundary; shapes whose code tile
                does not fit shared memory fall to the routes around
    larger M    activation-quantization kernel, then the tcgen05 GEMM on the codes: tokens as the 128-row operand,
                128 x 256 tiles (narrower while there are fewer tiles than SMs); only a long K against few weight rows
                (FFN value) with at most 48 tokens, or a call whose activations do not fit the GEMV's shared memory,
                takes the weight-streaming form (weights as the 128-row operand, stream-K over the SMs)
RWKVQ_ROUTE=tc  sends M <= 4 to the tensor-memory kernel with the quantization fused into it as well;
RWKVQ_ROUTE=mma keeps everything on the mma.sync kernels (M <= 32 fused, codes GEMM above).  All routes compute the
same results (INT8 bit for bit) and cross-check each other in the tests.
"""
from __future__ import annotations

import os

import torch

import rwkvq_abi as abi

F8E4M3_MAX = 448.0
FUSED_M_MAX = int(os.environ.get("RWKVQ_FUSED_M_MAX", "512"))   # kept for importers (fused_fp8_gemm.py:1101); this build has no cuBLASLt route to switch to
USE_CUDA_GRAPH = False  # kept for importers (fused_fp8_gemm.py:941); graphs are the caller's business here

GEMV_M_MAX = 32
_GEMV_SMEM_BUDGET = 200 * 1024 - 70 * 1024     # what the activation tile may take beside the weight ring
TC_FUSED_M_MAX = 4                 # rows up to which the activation quantization rides inside the streaming kernel
_TC_CACHE_MAX = 100 * 1024        # shared memory for the activations (2 B) and their codes (1 B) in the fused kernel
ROUTE = os.environ.get("RWKVQ_ROUTE", "auto").lower()   # auto | tc | mma
GEMV_AUTO_M_MAX = 32
_ACTQ_FUSED = os.environ.get("RWKVQ_ACTQ", "fused") == "fused"   # one cooperative launch; else memset + two kernels
CODES_M_MIN = int(os.environ.get("RWKVQ_CODES_M_MIN", "9"))      # rows from which the decode GEMV runs on pre-quantized codes
TC_M_MIN = int(os.environ.get("RWKVQ_TC_M_MIN", "33"))          # rows from which the tensor-memory kernels take over from the decode GEMVs (never below 9)
CODES_MK_MIN = 49152       # ... and already from 3 rows when the block is this large (long rows: K = 16384); measured
# FP8, rows from which the cluster split-K tensor-core kernel takes over from the codes GEMV where it applies (matrices
# with few 128-row tiles, e.g. N = 4096).  Measured on [4096, 4096]: 16 rows 8.7 (GEMV) against 9.2 us, 20 rows 10.4 against
# 9.3, 28 rows 10.8 against 9.3; r/k/v: 16 rows 15.5 against 17.9, 20 rows 21.1 against 18.0, 28 rows 22.2 against 19.0
# (from 17 rows the GEMV works on three token tiles).  With many row tiles (N = 16384) the GEMV stays ahead up to 32 rows.
CLUSTER_FROM_M = int(os.environ.get("RWKVQ_CLUSTER_FROM_M", "17"))
_decode_route_cache: dict = {}
_tc_route_cache: dict = {}


def _takes_tc(m: int, k: int, n=None) -> bool:
    """Do `m` rows go to the tensor-memory kernels instead of the decode GEMVs?  Always from TC_M_MIN rows; FP8 callers
    that pass the matrix's row count `n` also from CLUSTER_FROM_M rows where the cluster split-K kernel applies."""
    if m >= TC_M_MIN and m > 8:
        return True
    if n is None or m < max(CLUSTER_FROM_M, 9) or m > GEMV_M_MAX or ROUTE != "auto" or k % 16 or not _ACTQ_FUSED:
        return False
    hit = _tc_route_cache.get((m, n, k))
    if hit is None:
        hit = _tc_route_cache[(m, n, k)] = bool(abi.lib().rwkvq_tc_cluster_gemv_route(m, n, k))
    return hit


def _codes_gemv_fits(m: int, k: int, n=None) -> bool:
    """The decode GEMV on pre-quantized codes: CODES_M_MIN..32 rows whose 1-byte code tile fits shared memory."""
    if not (m >= CODES_M_MIN or (m >= 3 and m * k >= CODES_MK_MIN and CODES_M_MIN <= GEMV_M_MAX)) or m > GEMV_M_MAX or ROUTE != "auto" or k % 16 or _takes_tc(m, k, n):
        return False
    fits = _decode_route_cache.get((m, k))
    if fits is None:
        fits = _decode_route_cache[(m, k)] = bool(abi.lib().rwkvq_gemm_decode_route(m, k))
    return fits


# --------------------------------------------------------------------------- helpers
def _rows16(x: torch.Tensor) -> torch.Tensor:
    """[..., K] -> contiguous [M, K] in fp16/bf16 (other dtypes become bf16), as the reference wrappers do."""
    x2 = x.reshape(-1, x.shape[-1])
    if x2.dtype not in (torch.float16, torch.bfloat16):
        x2 = x2.to(torch.bfloat16)
    if x2.stride(-1) != 1 or (x2.shape[0] > 1 and x2.stride(0) != x2.shape[1]) or x2.data_ptr() % 16:
        x2 = x2.contiguous()
        if x2.data_ptr() % 16:
            x2 = x2.clone()
    return x2


def _unpack(weight_info_or_w, res_scale=None):
    if isinstance(weight_info_or_w, dict):
        return weight_info_or_w["weight"], weight_info_or_w["tensor_scale"]
    return weight_info_or_w, res_scale


def _gemv_fits(m: int, k: int, fp8: bool = True, n=None) -> bool:
    """The fused mma.sync GEMV keeps the quantized activations in shared memory (FP8: 2 bytes each, INT8: 1)."""
    pitch = (2 * k + 127) // 128 * 128 + 16 if fp8 else (k + 127) // 128 * 128 + 64
    if not (0 < m <= GEMV_M_MAX and m * pitch <= _GEMV_SMEM_BUDGET and k % 16 == 0) or (ROUTE == "auto" and _takes_tc(m, k, n)):
        return False
    return ROUTE == "mma" or (ROUTE == "auto" and m <= GEMV_AUTO_M_MAX)


def _tc_fused_fits(m: int, k: int, nmat: int = 1) -> bool:
    return ROUTE == "tc" and 0 < m <= TC_FUSED_M_MAX and k % 16 == 0 and nmat * m * ((k + 127) // 128 * 128 + 2 * k) <= _TC_CACHE_MAX


def _finish(out2d: torch.Tensor, lead, n: int, out_dtype):
    out = out2d if len(lead) == 1 else out2d.reshape(*lead, n)
    return out if out_dtype in (None, out.dtype) else out.to(out_dtype)


def _u8(t: torch.Tensor) -> torch.Tensor:
    return t if t.dtype in (torch.uint8, torch.int8) else t.view(torch.uint8)


def _wscale_flag(w_ts: torch.Tensor, n: int) -> int:
    """A weight scale of N values (scheme "fp8_perchannel", schemes.py:26-34) is applied per output row; the reference
    kernels load one scalar (fused_fp8_gemm.py:242) and so cannot run such weights."""
    cnt = w_ts.numel()
    if cnt == 1:
        return 0
    if cnt != n or w_ts.dtype != torch.float32 or not w_ts.is_contiguous():
        raise ValueError(f"rwkvq: tensor_scale must hold 1 or N={n} contiguous fp32 values, got {tuple(w_ts.shape)} {w_ts.dtype}")
    return abi.FLAG_WSCALE_PER_ROW


# --------------------------------------------------------------------------- activation preparation
def prep_x(x, awq_scale=None, out=None):
    """bf16(AWQ(x)) and the per-call amax as a GPU scalar, one launch (fused_fp8_gemm.py:55-79)."""
    x2 = _rows16(x)
    m, k = x2.shape
    if out is None or out.shape != x2.shape or out.dtype != torch.bfloat16 or not out.is_contiguous():
        out = torch.empty((m, k), dtype=torch.bfloat16, device=x2.device)
    amax = torch.empty(1, dtype=torch.float32, device=x2.device)
    awq = None if awq_scale is None else awq_scale.to(device=x2.device, dtype=torch.float32).contiguous()
    abi.call("rwkvq_prep_x", x2.data_ptr(), abi.dtype_code(x2), m, k, x2.stride(0) if m > 1 else k, abi.ptr(awq),
             out.data_ptr(), k, amax.data_ptr(), abi.DEFAULT_DIV, abi.stream_ptr())
    return out, amax


def prep3_x(xr, xk, xv, awq_r=None, awq_k=None):
    """prep_x for the three attention inputs in one launch (fused_fp8_gemm.py:121-150)."""
    xs = [_rows16(t) for t in (xr, xk, xv)]
    if len({t.dtype for t in xs}) != 1:
        xs = [t.to(torch.bfloat16) for t in xs]
    xs = [t.contiguous() for t in xs]
    m, k = xs[0].shape
    outs = [torch.empty((m, k), dtype=torch.bfloat16, device=xs[0].device) for _ in range(3)]
    amax = torch.empty(3, dtype=torch.float32, device=xs[0].device)
    f32 = lambda a: None if a is None else a.to(device=xs[0].device, dtype=torch.float32).contiguous()
    awq_r, awq_k = f32(awq_r), f32(awq_k)
    abi.call("rwkvq_prep3_x", xs[0].data_ptr(), xs[1].data_ptr(), xs[2].data_ptr(), abi.dtype_code(xs[0]), m, k, k,
             abi.ptr(awq_r), abi.ptr(awq_k), outs[0].data_ptr(), outs[1].data_ptr(), outs[2].data_ptr(), k,
             amax.data_ptr(), abi.DEFAULT_DIV, abi.stream_ptr())
    return outs[0], outs[1], outs[2], amax[0:1], amax[1:2], amax[2:3]


def prep_x_fp8(x):
    """e4m3 codes and the GPU-resident scale amax/448 for a scaled matmul (fused_fp8_gemm.py:363-390)."""
    x2 = _rows16(x).contiguous()
    m, k = x2.shape
    codes = torch.empty((m, k), dtype=torch.float8_e4m3fn, device=x2.device)
    scale = torch.empty(1, dtype=torch.float32, device=x2.device)
    amax = torch.empty(1, dtype=torch.float32, device=x2.device)
    abi.call("rwkvq_prep_x_fp8", x2.data_ptr(), abi.dtype_code(x2), m, k, k, codes.data_ptr(), k, scale.data_ptr(),
             amax.data_ptr(), abi.stream_ptr())
    return codes, scale


def prep_x_int8(x):
    """int8 codes with one scale per row (fused_fp8_gemm.py:712-731)."""
    x2 = _rows16(x).contiguous()
    m, k = x2.shape
    codes = torch.empty((m, k), dtype=torch.int8, device=x2.device)
    scale = torch.empty(m, dtype=torch.float32, device=x2.device)
    abi.call("rwkvq_prep_x_int8", x2.data_ptr(), abi.dtype_code(x2), m, k, k, codes.data_ptr(), k, scale.data_ptr(),
             abi.DEFAULT_DIV, abi.stream_ptr())
    return codes, scale


def prep3_x_int8(xr, xk, xv):
    """Three prep_x_int8 calls; returns (codes_r, codes_k, codes_v, scale_r, scale_k, scale_v) (fused_fp8_gemm.py:889-894)."""
    (cr, sr), (ck, sk), (cv, sv) = prep_x_int8(xr), prep_x_int8(xk), prep_x_int8(xv)
    return cr, ck, cv, sr, sk, sv


# --------------------------------------------------------------------------- tile configuration (informational)
def _cfg_for(M, N=None, K=None):
    """(rows of activations, weight rows, K bytes per step, warps) of the kernel a shape is routed to."""
    if K is not None and _gemv_fits(M, K):
        return (16 if M <= 16 else 32, 8, 64, 8)       # mma.sync GEMV: 8 weight rows per CTA, 8 warps split K
    if M <= 128:
        return (16 if M <= 16 else 128, 128, 128, 10)  # tcgen05, weights as the 128-row operand
    return (128, 256, 128, 10)                         # tcgen05 prefill tile


def _cfg_for_rkv(M, N=None, K=None):
    """The r/k/v launch uses the single-matrix tile; the three matrices share the CTA schedule, not a tile."""
    return _cfg_for(M, N, K)


def _best_method(M, N, K):
    return "gemv_fused" if _gemv_fits(M, K) else ("actq+tcgen05_stream" if M <= 128 else "actq+tcgen05_gemm")


# --------------------------------------------------------------------------- FP8
def _fp8_gemv(x2, w, w_ts, awq, flags):
    m, k = x2.shape
    n = w.shape[0]
    flags |= _wscale_flag(w_ts, n)
    out = abi.new_out(m, n, x2.device)
    if _tc_fused_fits(m, k):
        ws = abi.workspace(m, n, k, 1, x2.device)
        abi.call("rwkvq_tc_gemv_fp8", x2.data_ptr(), abi.dtype_code(x2), abi.ptr(awq), w.data_ptr(), w.stride(0),
                 w_ts.data_ptr(), out.data_ptr(), out.stride(0), m, n, k, x2.stride(0) if m > 1 else k, abi.DEFAULT_DIV, flags,
                 ws.data_ptr(), ws.numel(), abi.stream_ptr())
        abi.after_call(ws)
        return out
    abi.call("rwkvq_gemv_fp8", x2.data_ptr(), abi.dtype_code(x2), abi.ptr(awq), w.data_ptr(), w.stride(0),
             w_ts.data_ptr(), out.data_ptr(), out.stride(0), m, n, k, x2.stride(0) if m > 1 else k, abi.DEFAULT_DIV, flags,
             abi.stream_ptr())
    abi.after_call()
    return out


def _actq_fp8(x2, codes, amax, scale, div, flags, st):
    """FP8 activation codes + per-call amax: one cooperative launch (K a multiple of 8), else memset + two kernels."""
    m, k = x2.shape
    ldx = x2.stride(0) if m > 1 else k
    if k % 8 == 0 and m > 0 and _ACTQ_FUSED:
        scratch = abi.actq_scratch(x2.device)
        abi.call("rwkvq_actq_fp8_fused", x2.data_ptr(), abi.dtype_code(x2), m, k, ldx, codes.data_ptr(), k, amax.data_ptr(),
                 abi.ptr(scale), scratch.data_ptr(), scratch.numel() * 4, None, div, flags, st)
    else:
        abi.call("rwkvq_actq_fp8", x2.data_ptr(), abi.dtype_code(x2), m, k, ldx, codes.data_ptr(), k, amax.data_ptr(),
                 abi.ptr(scale), div, flags, st)


def can_push(m: int, n: int, k: int) -> bool:
    """True if an FP8 projection of m rows runs the GEMM that can carry the all-gather of a column-split projection."""
    return ROUTE != "mma" and _ACTQ_FUSED and m > 0 and k % 16 == 0 and bool(abi.lib().rwkvq_tc_gemm_can_push(m, n, k))


def _fp8_codes_gemm(x2, w, w_ts, act_flags, gemm_flags=0, push=None):
    """Activation quantization kernels, then the GEMM on codes (any M).  push = (peer_out, peer_flag, npeers, epoch): the
    GEMM also stores its result into the peers' buffers and signals them (rwkvq_dist.PeerGather.push_targets)."""
    m, k = x2.shape
    n = w.shape[0]
    codes = torch.empty((m, k), dtype=torch.uint8, device=x2.device)
    amax = torch.empty(1, dtype=torch.float32, device=x2.device)
    out = abi.new_out(m, n, x2.device)
    st = abi.stream_ptr()
    gemm_flags |= _wscale_flag(w_ts, n)
    _actq_fp8(x2, codes, amax, None, abi.DEFAULT_DIV, act_flags, st)
    if push is not None:
        ws = abi.workspace(min(m, 128), n, k, 1, x2.device)
        abi.call("rwkvq_tc_gemm_fp8_push", codes.data_ptr(), k, amax.data_ptr(), 1, w.data_ptr(), w.stride(0),
                 w_ts.data_ptr(), out.data_ptr(), out.stride(0), m, n, k, abi.DEFAULT_DIV, gemm_flags, ws.data_ptr(), ws.numel(),
                 push[0], push[1], push[2], push[3], st)
        abi.after_call(ws)
    elif ROUTE != "mma":
        ws = abi.workspace(min(m, 128), n, k, 1, x2.device)
        abi.call("rwkvq_tc_gemm_fp8", codes.data_ptr(), k, amax.data_ptr(), 1, w.data_ptr(), w.stride(0),
                 w_ts.data_ptr(), out.data_ptr(), out.stride(0), m, n, k, abi.DEFAULT_DIV, gemm_flags, ws.data_ptr(), ws.numel(), st)
        abi.after_call(ws)
    else:
        abi.call("rwkvq_gemm_fp8", codes.data_ptr(), k, amax.data_ptr(), 1, w.data_ptr(), w.stride(0), w_ts.data_ptr(),
                 out.data_ptr(), out.stride(0), m, n, k, abi.DEFAULT_DIV, gemm_flags, st)
    return out


# The cluster split-K kernel with the activation quantization inside (rwkvq_tc_cluster_gemv_fp8, one launch) is OFF by
# default: measured on the FFN value shape it is slower than the quantizer kernel + the same GEMM on codes (16 rows:
# 23.2 against 18.7 us, 32 rows: 28.8 against 21.4) -- every one of the 32 clusters re-reads and re-quantizes the whole
# block, while the separate quantizer runs once, in parallel with the GEMM's weight prefetch.  RWKVQ_CLUSTER_ONE_LAUNCH=1
# routes 9..32 rows to it where it applies; =first also ahead of the decode GEMV on codes.
_CLUSTER_ONE_LAUNCH = os.environ.get("RWKVQ_CLUSTER_ONE_LAUNCH", "0").lower()
CLUSTER_M_MIN = 9
_CLUSTER_FIRST = _CLUSTER_ONE_LAUNCH == "first"
_cluster_route_cache: dict = {}


def _cluster_one_launch(m: int, n: int, k: int) -> bool:
    """9..32 rows against a matrix with few 128-row tiles: one launch, activation quantization inside the cluster
    split-K kernel (rwkvq_tc_cluster_gemv_fp8); opt-in, see above."""
    if _CLUSTER_ONE_LAUNCH not in ("1", "first") or m < CLUSTER_M_MIN or m > 32 or ROUTE != "auto" or not _ACTQ_FUSED or k % 16:
        return False
    fits = _cluster_route_cache.get((m, n, k))
    if fits is None:
        fits = _cluster_route_cache[(m, n, k)] = bool(abi.lib().rwkvq_tc_cluster_gemv_route(m, n, k))
    return fits


def _fp8_cluster_gemv(x2, w, w_ts):
    m, k = x2.shape
    n = w.shape[0]
    out = abi.new_out(m, n, x2.device)
    abi.call("rwkvq_tc_cluster_gemv_fp8", x2.data_ptr(), abi.dtype_code(x2), x2.stride(0), w.data_ptr(), w.stride(0), w_ts.data_ptr(),
             out.data_ptr(), out.stride(0), m, n, k, abi.DEFAULT_DIV, abi.FLAG_QUANT_FROM_BF16 | _wscale_flag(w_ts, n), abi.stream_ptr())
    abi.after_call()
    return out


def _fp8_codes_gemv(x2, w, w_ts):
    """9..32 rows: quantize once (one cooperative launch), then the weight-streaming decode kernel on the codes."""
    m, k = x2.shape
    n = w.shape[0]
    dev = x2.device
    codes = torch.empty((m, k), dtype=torch.uint8, device=dev)
    amax = torch.empty(1, dtype=torch.float32, device=dev)
    out = abi.new_out(m, n, dev)
    st = abi.stream_ptr()
    _actq_fp8(x2, codes, amax, None, abi.DEFAULT_DIV, abi.FLAG_QUANT_FROM_BF16, st)
    abi.call("rwkvq_gemm_fp8", codes.data_ptr(), k, amax.data_ptr(), 1, w.data_ptr(), w.stride(0), w_ts.data_ptr(),
             out.data_ptr(), out.stride(0), m, n, k, abi.DEFAULT_DIV, _wscale_flag(w_ts, n), st)
    abi.after_call()
    return out


def _fp8_codes_gemv_rkv(xs, ws_, scales):
    """r, k, v with 9..32 rows: ONE quantization launch for the three inputs, ONE weight-streaming launch on the codes."""
    m, k = xs[0].shape
    n = ws_[0].shape[0]
    dev = xs[0].device
    codes = torch.empty((3, m, k), dtype=torch.uint8, device=dev)
    amax = torch.empty(3, dtype=torch.float32, device=dev)
    outs = torch.empty((3, m, n), dtype=torch.float16, device=dev)
    st = abi.stream_ptr()
    scratch = abi.actq_scratch(dev)
    abi.call("rwkvq_actq_fp8_fused3", xs[0].data_ptr(), xs[1].data_ptr(), xs[2].data_ptr(), abi.dtype_code(xs[0]), m, k, k,
             codes[0].data_ptr(), codes[1].data_ptr(), codes[2].data_ptr(), k, amax.data_ptr(), scratch.data_ptr(),
             scratch.numel() * 4, None, abi.DEFAULT_DIV, abi.FLAG_QUANT_FROM_BF16, st)
    abi.call("rwkvq_gemm_fp8_rkv", codes[0].data_ptr(), codes[1].data_ptr(), codes[2].data_ptr(), k, amax.data_ptr(), 1,
             ws_[0].data_ptr(), ws_[1].data_ptr(), ws_[2].data_ptr(), ws_[0].stride(0), scales[0].data_ptr(),
             scales[1].data_ptr(), scales[2].data_ptr(), outs[0].data_ptr(), outs[1].data_ptr(), outs[2].data_ptr(), n,
             m, n, k, abi.DEFAULT_DIV, _wscale_flag(scales[0], n), st)
    abi.after_call()
    return [outs[0], outs[1], outs[2]]


def _fp8_codes_gemm_rkv(xs, ws_, scales):
    """r, k, v above the decode kernel's range: ONE activation-quantization launch for the three inputs and ONE
    tensor-core GEMM launch for the three projections (the reference: prep3_x + fused_rkv_fp8_kernel)."""
    m, k = xs[0].shape
    n = ws_[0].shape[0]
    dev = xs[0].device
    codes = torch.empty((3, m, k), dtype=torch.uint8, device=dev)
    amax = torch.empty(3, dtype=torch.float32, device=dev)
    outs = torch.empty((3, m, n), dtype=torch.float16, device=dev)
    st = abi.stream_ptr()
    scratch = abi.actq_scratch(dev)
    flags = _wscale_flag(scales[0], n)
    abi.call("rwkvq_actq_fp8_fused3", xs[0].data_ptr(), xs[1].data_ptr(), xs[2].data_ptr(), abi.dtype_code(xs[0]), m, k, k,
             codes[0].data_ptr(), codes[1].data_ptr(), codes[2].data_ptr(), k, amax.data_ptr(), scratch.data_ptr(),
             scratch.numel() * 4, None, abi.DEFAULT_DIV, abi.FLAG_QUANT_FROM_BF16, st)
    ws = abi.workspace(min(m, 128), n, k, 3, dev)
    abi.call("rwkvq_tc_gemm_fp8_rkv", codes[0].data_ptr(), codes[1].data_ptr(), codes[2].data_ptr(), k, amax.data_ptr(), 1,
             ws_[0].data_ptr(), ws_[1].data_ptr(), ws_[2].data_ptr(), ws_[0].stride(0), scales[0].data_ptr(),
             scales[1].data_ptr(), scales[2].data_ptr(), outs[0].data_ptr(), outs[1].data_ptr(), outs[2].data_ptr(), n,
             m, n, k, abi.DEFAULT_DIV, flags, ws.data_ptr(), ws.numel(), st)
    abi.after_call(ws)
    return [outs[0], outs[1], outs[2]]


def linear_fp8_m1_fused(x, weight_info, out_dtype=torch.float16):
    """M == 1 FP8 projection in a single launch (fused_fp8_gemm.py:645-679).  fp16 input is rounded to bf16
    before the amax, as there (:662)."""
    w, w_ts = _unpack(weight_info)
    n, k = w.shape
    dt = x.dtype
    if ((dt is torch.bfloat16 or dt is torch.float16) and ROUTE == "auto" and x.numel() == k and x.is_contiguous()
            and x.data_ptr() % 16 == 0 and _gemv_fits(1, k)):
        # the decode call itself, without the general path's reshapes and views: one allocation, one boundary crossing
        out = abi.new_out(1, n, x.device)
        abi.call("rwkvq_gemv_fp8", x.data_ptr(), abi.BF16 if dt is torch.bfloat16 else abi.F16, None, w.data_ptr(), w.stride(0),
                 w_ts.data_ptr(), out.data_ptr(), out.stride(0), 1, n, k, k, abi.DEFAULT_DIV,
                 abi.FLAG_AMAX_AFTER_BF16 | _wscale_flag(w_ts, n), abi.stream_ptr())
        abi.after_call()
        return _finish(out, x.shape[:-1], n, out_dtype)
    x2 = _rows16(x.reshape(1, -1))
    out = _fp8_gemv(x2, _u8(w), w_ts, None, abi.FLAG_AMAX_AFTER_BF16)
    return _finish(out, x.shape[:-1], n, out_dtype)


def linear_fp8_fused(x, weight_info_or_w, res_scale=None, out_dtype=torch.float16, push=None):
    """FP8 W8A8 projection with on-the-fly activation quantization (fused_fp8_gemm.py:1020-1077).  push: see
    _fp8_codes_gemm (only for row counts with can_push())."""
    w, w_ts = _unpack(weight_info_or_w, res_scale)
    k = x.shape[-1]
    m = x.numel() // k if k else 0
    if push is not None:
        if not can_push(m, w.shape[0], k):
            raise RuntimeError("rwkvq: the pushed all-gather rides in the tiled tensor-core GEMM only (see can_push)")
        out = _fp8_codes_gemm(_rows16(x), _u8(w), w_ts, abi.FLAG_QUANT_FROM_BF16, push=push)
        return _finish(out, x.shape[:-1], w.shape[0], out_dtype)
    if m == 1:
        return linear_fp8_m1_fused(x, {"weight": w, "tensor_scale": w_ts}, out_dtype)
    x2 = _rows16(x)
    if _CLUSTER_FIRST and _cluster_one_launch(m, w.shape[0], k):
        out = _fp8_cluster_gemv(x2, _u8(w), w_ts)
    elif _codes_gemv_fits(m, k, w.shape[0]) and _ACTQ_FUSED and k % 8 == 0:
        out = _fp8_codes_gemv(x2, _u8(w), w_ts)
    elif _tc_fused_fits(m, k) or _gemv_fits(m, k, n=w.shape[0]):
        out = _fp8_gemv(x2, _u8(w), w_ts, None, 0)
    elif _cluster_one_launch(m, w.shape[0], k):
        # where the two-launch route would run the cluster split-K kernel anyway: the same kernel with the activation
        # quantization inside (same codes, same K split: same bits, also as the r/k/v form on such shapes)
        out = _fp8_cluster_gemv(x2, _u8(w), w_ts)
    else:
        out = _fp8_codes_gemm(x2, _u8(w), w_ts, abi.FLAG_QUANT_FROM_BF16)
    return _finish(out, x.shape[:-1], w.shape[0], out_dtype)


def _rkv_decode_fast(xr, xk, xv, wr_info, wk_info, wv_info):
    """The decode call of linear_rkv_fused (up to 8 rows, plain contiguous inputs, no AWQ divisors) without the general
    path's per-tensor views and checks; None = take the general path."""
    dt = xr.dtype
    k = xr.shape[-1]
    m = xr.numel() // k if k else 0
    wr, wk, wv = wr_info["weight"], wk_info["weight"], wv_info["weight"]
    if not (0 < m <= 8 and ROUTE == "auto" and m < CODES_M_MIN and (dt is torch.bfloat16 or dt is torch.float16) and xk.dtype is dt and xv.dtype is dt
            and xr.is_contiguous() and xk.is_contiguous() and xv.is_contiguous() and xk.shape == xr.shape and xv.shape == xr.shape
            and wr.shape == wk.shape == wv.shape and wr.stride(0) == wk.stride(0) == wv.stride(0)
            and "awq_scale" not in wr_info and "awq_scale" not in wk_info and not abi._out_override):
        return None
    n = wr.shape[0]
    if wr.shape[1] != k or not _gemv_fits(m, k) or _codes_gemv_fits(m, k):
        return None
    if (xr.data_ptr() | xk.data_ptr() | xv.data_ptr()) % 16:
        return None
    sr, sk, sv = wr_info["tensor_scale"], wk_info["tensor_scale"], wv_info["tensor_scale"]
    wflag = _wscale_flag(sr, n)
    if _wscale_flag(sk, n) != wflag or _wscale_flag(sv, n) != wflag:
        return None
    outs = torch.empty((3, m, n), dtype=torch.float16, device=xr.device)
    o0 = outs.data_ptr()
    step = m * n * 2
    abi.call("rwkvq_gemv_fp8_rkv", xr.data_ptr(), xk.data_ptr(), xv.data_ptr(), abi.BF16 if dt is torch.bfloat16 else abi.F16,
             None, None, wr.data_ptr(), wk.data_ptr(), wv.data_ptr(), wr.stride(0), sr.data_ptr(), sk.data_ptr(), sv.data_ptr(),
             o0, o0 + step, o0 + 2 * step, n, m, n, k, k, abi.DEFAULT_DIV, wflag, abi.stream_ptr())
    abi.after_call()
    return outs.unbind(0)


def linear_rkv_fused(xr, xk, xv, wr_info, wk_info, wv_info, out_dtype=torch.float16):
    """r, k, v projections (fused_fp8_gemm.py:944-1017): one launch for decode-sized M."""
    lead = xr.shape[:-1]
    fast = _rkv_decode_fast(xr, xk, xv, wr_info, wk_info, wv_info)
    if fast is not None:
        return tuple(_finish(o, lead, o.shape[-1], out_dtype) for o in fast)
    xs = [_rows16(t) for t in (xr, xk, xv)]
    if len({t.dtype for t in xs}) != 1:
        xs = [t.to(torch.bfloat16) for t in xs]
    m, k = xs[0].shape
    ws_ = [_u8(i["weight"]) for i in (wr_info, wk_info, wv_info)]
    n = ws_[0].shape[0]
    dev = xs[0].device
    awq_r, awq_k = wr_info.get("awq_scale"), wk_info.get("awq_scale")
    wflags = {_wscale_flag(i["tensor_scale"], n) for i in (wr_info, wk_info, wv_info)}
    same_ld = len({w.stride(0) for w in ws_}) == 1 and all(w.shape == ws_[0].shape for w in ws_) and len(wflags) == 1
    wflag = next(iter(wflags)) if len(wflags) == 1 else 0
    f32 = lambda a: None if a is None else a.to(device=dev, dtype=torch.float32).contiguous()
    n_route = n if (awq_r is None and awq_k is None and same_ld) else None      # the cluster kernel runs on plain codes of like matrices
    if (_codes_gemv_fits(m, k, n_route) and _ACTQ_FUSED and same_ld and awq_r is None and awq_k is None and k % 8 == 0):
        outs = _fp8_codes_gemv_rkv([t.contiguous() for t in xs], ws_, [i["tensor_scale"] for i in (wr_info, wk_info, wv_info)])
    elif _tc_fused_fits(m, k, 3) and same_ld:
        xs = [t.contiguous() for t in xs]
        outs = [torch.empty((m, n), dtype=torch.float16, device=dev) for _ in range(3)]
        awq_r, awq_k = f32(awq_r), f32(awq_k)
        ws = abi.workspace(m, n, k, 3, dev)
        abi.call("rwkvq_tc_gemv_fp8_rkv", xs[0].data_ptr(), xs[1].data_ptr(), xs[2].data_ptr(), abi.dtype_code(xs[0]),
                 abi.ptr(awq_r), abi.ptr(awq_k), ws_[0].data_ptr(), ws_[1].data_ptr(), ws_[2].data_ptr(), ws_[0].stride(0),
                 wr_info["tensor_scale"].data_ptr(), wk_info["tensor_scale"].data_ptr(),
                 wv_info["tensor_scale"].data_ptr(), outs[0].data_ptr(), outs[1].data_ptr(), outs[2].data_ptr(), n,
                 m, n, k, k, abi.DEFAULT_DIV, wflag, ws.data_ptr(), ws.numel(), abi.stream_ptr())
        abi.after_call(ws)
    elif _gemv_fits(m, k, n=n_route) and same_ld:
        xs = [t.contiguous() for t in xs]
        outs = [torch.empty((m, n), dtype=torch.float16, device=dev) for _ in range(3)]
        awq_r, awq_k = f32(awq_r), f32(awq_k)
        abi.call("rwkvq_gemv_fp8_rkv", xs[0].data_ptr(), xs[1].data_ptr(), xs[2].data_ptr(), abi.dtype_code(xs[0]),
                 abi.ptr(awq_r), abi.ptr(awq_k), ws_[0].data_ptr(), ws_[1].data_ptr(), ws_[2].data_ptr(), ws_[0].stride(0),
                 wr_info["tensor_scale"].data_ptr(), wk_info["tensor_scale"].data_ptr(),
                 wv_info["tensor_scale"].data_ptr(), outs[0].data_ptr(), outs[1].data_ptr(), outs[2].data_ptr(), n,
                 m, n, k, k, abi.DEFAULT_DIV, wflag, abi.stream_ptr())
        abi.after_call()
    elif ROUTE != "mma" and _ACTQ_FUSED and same_ld and awq_r is None and awq_k is None and k % 8 == 0 and m > 0:
        outs = _fp8_codes_gemm_rkv([t.contiguous() for t in xs], ws_, [i["tensor_scale"] for i in (wr_info, wk_info, wv_info)])
    else:
        outs = []
        for x2, w, info, awq in zip(xs, ws_, (wr_info, wk_info, wv_info), (awq_r, awq_k, None)):
            if _tc_fused_fits(m, k) or _gemv_fits(m, k):   # three fused launches when one for all three does not fit
                outs.append(_fp8_gemv(x2.contiguous(), w, info["tensor_scale"], f32(awq), 0))
                continue
            if awq is not None:                      # AWQ division, then the plain route on the bf16 copy
                x2, _ = prep_x(x2, awq)
            outs.append(_fp8_codes_gemm(x2, w, info["tensor_scale"], abi.FLAG_QUANT_FROM_BF16))
    return tuple(_finish(o, lead, n, out_dtype) for o in outs)


_ffn_scratch: dict = {}


def ffn_scratch(device) -> torch.Tensor:
    """64 zeroed bytes per (device, stream) through which the key projection hands max|relu^2| (FP8: one value; INT8: one
    per token row) to the value projection."""
    key = (torch.device(device).index or 0, torch.cuda.current_stream().cuda_stream)
    sc = _ffn_scratch.get(key)
    if sc is None:
        sc = _ffn_scratch[key] = torch.zeros(16, dtype=torch.int32, device=device)
    return sc


def ffn_relu2_fp8(x, key_info, value_info, out_dtype=torch.float16, return_hidden=False):
    """The FFN of a layer on FP8 weights: value( relu_square( key(x) ) ), the chain the engine runs as three steps
    (rwkv7_fast_v3a.py:1109, 1136-1144).  For decode-sized calls (rows that fit the one-launch kernel) relu_square is
    folded into the key projection's epilogue and the value projection quantizes with the amax that epilogue publishes:
    two launches, no separate relu kernel, no abs-max pass over the [M, F] hidden activations.  Other sizes run the
    three steps.  Results equal the three-step chain bit for bit."""
    wk, sk = _unpack(key_info)
    wv, sv = _unpack(value_info)
    x2 = _rows16(x)
    m, k = x2.shape
    f_dim, n = wk.shape[0], wv.shape[0]
    if ROUTE == "auto" and 0 < m <= 8 and _gemv_fits(m, k) and _gemv_fits(m, f_dim) and not _codes_gemv_fits(m, k) and not _codes_gemv_fits(m, f_dim):
        flags = abi.FLAG_AMAX_AFTER_BF16 if m == 1 else 0           # the M == 1 kernel takes its amax after the bf16 rounding
        hid = torch.empty((m, f_dim), dtype=torch.float16, device=x2.device)
        out = abi.new_out(m, n, x2.device)
        sc = ffn_scratch(x2.device)
        st = abi.stream_ptr()
        abi.call("rwkvq_gemv_fp8_relu2", x2.data_ptr(), abi.dtype_code(x2), _u8(wk).data_ptr(), wk.stride(0), sk.data_ptr(),
                 hid.data_ptr(), f_dim, m, f_dim, k, x2.stride(0) if m > 1 else k, abi.DEFAULT_DIV, flags | _wscale_flag(sk, f_dim),
                 sc.data_ptr(), st)
        abi.call("rwkvq_gemv_fp8_preamax", hid.data_ptr(), abi.F16, _u8(wv).data_ptr(), wv.stride(0), sv.data_ptr(),
                 out.data_ptr(), out.stride(0), m, n, f_dim, f_dim, abi.DEFAULT_DIV, flags | _wscale_flag(sv, n), sc.data_ptr(), st)
        abi.after_call()
    elif ROUTE == "auto" and m > GEMV_M_MAX and _ACTQ_FUSED and k % 8 == 0 and f_dim % 8 == 0:
        # many rows: relu_square and the amax of its result come out of the key GEMM's epilogue; the hidden activations
        # are then quantized by a purely elementwise kernel (no abs-max pass, no grid rendezvous).  Up to FUSED_M_MAX
        # rows the two projections have the semantics of linear_fp8_fused, above those of fp8_ops.linear_fp8 (bf16
        # first, torch's scale arithmetic, results through bf16), as the engine's dispatch has them.
        big = m > FUSED_M_MAX
        dev_, st = x2.device, abi.stream_ptr()
        div = abi.DIV_TORCH if big else abi.DEFAULT_DIV
        aflags = abi.FLAG_QUANT_FROM_BF16 | (abi.FLAG_AMAX_AFTER_BF16 if big else 0)
        gflags = (abi.FLAG_OUT_VIA_BF16 | abi.FLAG_AMAX_AFTER_BF16) if big else 0
        codes = torch.empty((m, k), dtype=torch.uint8, device=dev_)
        sc4 = torch.empty(4, dtype=torch.float32, device=dev_)           # amax / scale of x, amax / scale of the hidden
        hid = torch.empty((m, f_dim), dtype=torch.float16, device=dev_)
        hcodes = torch.empty((m, f_dim), dtype=torch.uint8, device=dev_)
        out = abi.new_out(m, n, dev_)
        ffn = ffn_scratch(dev_)
        _actq_fp8(x2, codes, sc4[0:1], sc4[1:2], div, aflags, st)
        ws = abi.workspace(min(m, 128), max(f_dim, n), max(k, f_dim), 1, dev_)
        a_ptr, is_amax = (sc4[1:2].data_ptr(), 0) if big else (sc4[0:1].data_ptr(), 1)
        abi.call("rwkvq_tc_gemm_fp8_relu2", codes.data_ptr(), k, a_ptr, is_amax, _u8(wk).data_ptr(), wk.stride(0), sk.data_ptr(),
                 hid.data_ptr(), f_dim, m, f_dim, k, abi.DIV_IEEE if big else abi.DEFAULT_DIV, gflags | _wscale_flag(sk, f_dim),
                 ffn.data_ptr(), ws.data_ptr(), ws.numel(), st)
        abi.call("rwkvq_actq_fp8_given", hid.data_ptr(), abi.F16, m, f_dim, f_dim, hcodes.data_ptr(), f_dim, sc4[2:3].data_ptr(),
                 sc4[3:4].data_ptr(), ffn.data_ptr(), div, abi.FLAG_QUANT_FROM_BF16, st)
        h_ptr = sc4[3:4].data_ptr() if big else sc4[2:3].data_ptr()
        abi.call("rwkvq_tc_gemm_fp8", hcodes.data_ptr(), f_dim, h_ptr, is_amax, _u8(wv).data_ptr(), wv.stride(0), sv.data_ptr(),
                 out.data_ptr(), out.stride(0), m, n, f_dim, abi.DIV_IEEE if big else abi.DEFAULT_DIV,
                 (abi.FLAG_OUT_VIA_BF16 if big else 0) | _wscale_flag(sv, n), ws.data_ptr(), ws.numel(), st)
        abi.after_call(ws)
    else:
        hid = linear_quantized_fused(x2, {"weight": wk, "tensor_scale": sk, "qtype": "fp8"})
        hid = (hid.float().clamp_(min=0.0) ** 2).to(torch.float16)       # relu_square: fp16(max(y, 0)^2), fp32 arithmetic
        out = linear_quantized_fused(hid, {"weight": wv, "tensor_scale": sv, "qtype": "fp8"})
    out = _finish(out.reshape(m, n), x.shape[:-1], n, out_dtype)
    return (out, hid.reshape(*x.shape[:-1], f_dim)) if return_hidden else out


_row_max = {}


def _row_max_scratch(device, rows: int) -> torch.Tensor:
    """Zeroed floats, one per token row, per (device, stream): the key GEMM of the INT8 FFN pair folds the rows' maxima
    into them and the quantizer behind it clears them again."""
    key = (torch.device(device).index or 0, torch.cuda.current_stream().cuda_stream)
    buf = _row_max.get(key)
    if buf is None or buf.numel() < rows:
        buf = _row_max[key] = torch.zeros(max(rows, 4096), dtype=torch.float32, device=device)
    return buf


def ffn_relu2_int8(x, key_info, value_info, out_dtype=torch.float16, return_hidden=False):
    """ffn_relu2_fp8 for INT8 weights.  Up to 8 rows: two launches, relu_square in the key projection's epilogue, which
    publishes the maximum of its result per token row (INT8 activations are scaled per row), and a value projection
    that quantizes with those maxima instead of reducing the hidden activations again.  Row counts that run the tiled
    tensor-core GEMM: four launches (quantizer, key GEMM with relu_square and the row maxima in its epilogue, an
    elementwise given-maxima quantizer, value GEMM).  Other row counts: the three steps.  Results equal the three-step
    chain bit for bit."""
    wk, sk = key_info["weight"], key_info["tensor_scale"]
    wv, sv = value_info["weight"], value_info["tensor_scale"]
    x2 = _rows16(x)
    m, k = x2.shape
    f_dim, n = wk.shape[0], wv.shape[0]
    if (ROUTE == "auto" and 0 < m <= 8 and _gemv_fits(m, k, fp8=False) and _gemv_fits(m, f_dim, fp8=False)
            and not _codes_gemv_fits(m, k) and not _codes_gemv_fits(m, f_dim)):
        hid = torch.empty((m, f_dim), dtype=torch.float16, device=x2.device)
        out = abi.new_out(m, n, x2.device)
        sc = ffn_scratch(x2.device)
        st = abi.stream_ptr()
        abi.call("rwkvq_gemv_int8_relu2", x2.data_ptr(), abi.dtype_code(x2), wk.data_ptr(), wk.stride(0), sk.data_ptr(),
                 hid.data_ptr(), f_dim, m, f_dim, k, x2.stride(0) if m > 1 else k, abi.DEFAULT_DIV, 0, sc.data_ptr(), st)
        abi.call("rwkvq_gemv_int8_preamax", hid.data_ptr(), abi.F16, wv.data_ptr(), wv.stride(0), sv.data_ptr(),
                 out.data_ptr(), out.stride(0), m, n, f_dim, f_dim, abi.DEFAULT_DIV, 0, sc.data_ptr(), st)
        abi.after_call()
    elif ROUTE == "auto" and m > GEMV_M_MAX and k % 16 == 0 and f_dim % 16 == 0 and can_push(m, f_dim, k):
        # many rows on the tiled GEMM (can_push: neither the weight-streaming nor the cluster form takes these sizes)
        dev_, st = x2.device, abi.stream_ptr()
        codes = torch.empty((m, k), dtype=torch.int8, device=dev_)
        xs = torch.empty(m, dtype=torch.float32, device=dev_)
        hid = torch.empty((m, f_dim), dtype=torch.float16, device=dev_)
        hcodes = torch.empty((m, f_dim), dtype=torch.int8, device=dev_)
        hs = torch.empty(m, dtype=torch.float32, device=dev_)
        out = abi.new_out(m, n, dev_)
        rowmax = _row_max_scratch(dev_, m)
        abi.call("rwkvq_prep_x_int8", x2.data_ptr(), abi.dtype_code(x2), m, k, x2.stride(0), codes.data_ptr(), k, xs.data_ptr(), abi.DEFAULT_DIV, st)
        ws = abi.workspace(min(m, 128), max(f_dim, n), max(k, f_dim), 1, dev_)
        abi.call("rwkvq_tc_gemm_int8_relu2", codes.data_ptr(), k, xs.data_ptr(), wk.data_ptr(), wk.stride(0), sk.data_ptr(), hid.data_ptr(), f_dim,
                 m, f_dim, k, 0, rowmax.data_ptr(), ws.data_ptr(), ws.numel(), st)
        abi.call("rwkvq_actq_int8_given", hid.data_ptr(), abi.F16, m, f_dim, f_dim, hcodes.data_ptr(), f_dim, hs.data_ptr(), rowmax.data_ptr(),
                 abi.DEFAULT_DIV, st)
        abi.call("rwkvq_tc_gemm_int8", hcodes.data_ptr(), f_dim, hs.data_ptr(), wv.data_ptr(), wv.stride(0), sv.data_ptr(), out.data_ptr(),
                 out.stride(0), None, 0, m, n, f_dim, 0, ws.data_ptr(), ws.numel(), st)
        abi.after_call(ws)
    else:
        hid = linear_int8_fused(x2, key_info)
        hid = (hid.float().clamp_(min=0.0) ** 2).to(torch.float16)       # relu_square: fp16(max(y, 0)^2), fp32 arithmetic
        out = linear_int8_fused(hid, value_info)
    out = _finish(out.reshape(m, n), x.shape[:-1], n, out_dtype)
    return (out, hid.reshape(*x.shape[:-1], f_dim)) if return_hidden else out


# --------------------------------------------------------------------------- INT8
def _int8_any(x2, w, w_scale, acc_out=None, push=None):
    m, k = x2.shape
    n = w.shape[0]
    out = abi.new_out(m, n, x2.device)
    st = abi.stream_ptr()
    if push is not None:
        # column-split projection: the GEMM also delivers its result to the other ranks (see _fp8_codes_gemm)
        if acc_out is not None or not can_push(m, n, k):
            raise RuntimeError("rwkvq: the pushed all-gather rides in the tiled tensor-core GEMM only (see can_push), without acc_out")
        codes = torch.empty((m, k), dtype=torch.int8, device=x2.device)
        xs = torch.empty(m, dtype=torch.float32, device=x2.device)
        abi.call("rwkvq_prep_x_int8", x2.data_ptr(), abi.dtype_code(x2), m, k, x2.stride(0) if m > 1 else k,
                 codes.data_ptr(), k, xs.data_ptr(), abi.DEFAULT_DIV, st)
        ws = abi.workspace(min(m, 128), n, k, 1, x2.device)
        abi.call("rwkvq_tc_gemm_int8_push", codes.data_ptr(), k, xs.data_ptr(), w.data_ptr(), w.stride(0), w_scale.data_ptr(),
                 out.data_ptr(), out.stride(0), m, n, k, 0, ws.data_ptr(), ws.numel(), push[0], push[1], push[2], push[3], st)
        abi.after_call(ws)
        return out
    if _codes_gemv_fits(m, k):
        # 9..32 rows: quantize the rows once, then the weight-streaming decode kernel on the codes
        codes = torch.empty((m, k), dtype=torch.int8, device=x2.device)
        xs = torch.empty(m, dtype=torch.float32, device=x2.device)
        abi.call("rwkvq_prep_x_int8", x2.data_ptr(), abi.dtype_code(x2), m, k, x2.stride(0) if m > 1 else k,
                 codes.data_ptr(), k, xs.data_ptr(), abi.DEFAULT_DIV, st)
        abi.call("rwkvq_gemm_int8", codes.data_ptr(), k, xs.data_ptr(), w.data_ptr(), w.stride(0), w_scale.data_ptr(),
                 out.data_ptr(), out.stride(0), abi.ptr(acc_out), n, m, n, k, 0, st)
        abi.after_call()
    elif _tc_fused_fits(m, k):
        ws = abi.workspace(m, n, k, 1, x2.device)
        abi.call("rwkvq_tc_gemv_int8", x2.data_ptr(), abi.dtype_code(x2), w.data_ptr(), w.stride(0), w_scale.data_ptr(),
                 out.data_ptr(), out.stride(0), abi.ptr(acc_out), n, m, n, k, x2.stride(0) if m > 1 else k, abi.DEFAULT_DIV, 0,
                 ws.data_ptr(), ws.numel(), st)
    elif _gemv_fits(m, k, fp8=False):
        abi.call("rwkvq_gemv_int8", x2.data_ptr(), abi.dtype_code(x2), w.data_ptr(), w.stride(0), w_scale.data_ptr(),
                 out.data_ptr(), out.stride(0), abi.ptr(acc_out), n, m, n, k, x2.stride(0) if m > 1 else k, abi.DEFAULT_DIV, 0, st)
    else:
        codes = torch.empty((m, k), dtype=torch.int8, device=x2.device)
        xs = torch.empty(m, dtype=torch.float32, device=x2.device)
        abi.call("rwkvq_prep_x_int8", x2.data_ptr(), abi.dtype_code(x2), m, k, x2.stride(0) if m > 1 else k,
                 codes.data_ptr(), k, xs.data_ptr(), abi.DEFAULT_DIV, st)
        if ROUTE != "mma":
            ws = abi.workspace(min(m, 128), n, k, 1, x2.device)
            abi.call("rwkvq_tc_gemm_int8", codes.data_ptr(), k, xs.data_ptr(), w.data_ptr(), w.stride(0),
                     w_scale.data_ptr(), out.data_ptr(), out.stride(0), abi.ptr(acc_out), n, m, n, k, 0, ws.data_ptr(), ws.numel(), st)
        else:
            abi.call("rwkvq_gemm_int8", codes.data_ptr(), k, xs.data_ptr(), w.data_ptr(), w.stride(0), w_scale.data_ptr(),
                     out.data_ptr(), out.stride(0), abi.ptr(acc_out), n, m, n, k, 0, st)
    return out


def linear_int8_fused(x, weight_info, out_dtype=torch.float16, acc_out=None, push=None):
    """INT8 W8A8 projection, exact int32 accumulation (fused_fp8_gemm.py:785-818).  `acc_out` (optional int32
    [M, N]) receives the raw accumulators.  push: see _fp8_codes_gemm."""
    w, w_scale = weight_info["weight"], weight_info["tensor_scale"]
    out = _int8_any(_rows16(x), w, w_scale, acc_out, push)
    return _finish(out, x.shape[:-1], w.shape[0], out_dtype)


def linear_rkv_int8_fused(xr, xk, xv, wr_info, wk_info, wv_info, out_dtype=torch.float16, compat_shared_scale=True):
    """r, k, v INT8 projections (fused_fp8_gemm.py:897-934).  The reference scales all three results by r's
    weight scale (:855-857, :906); `compat_shared_scale=False` uses each matrix's own scale instead."""
    lead = xr.shape[:-1]
    xs = [_rows16(t) for t in (xr, xk, xv)]
    if len({t.dtype for t in xs}) != 1:
        xs = [t.to(torch.bfloat16) for t in xs]
    m, k = xs[0].shape
    infos = (wr_info, wk_info, wv_info)
    ws = [i["weight"] for i in infos]
    n = ws[0].shape[0]
    scales = [wr_info["tensor_scale"]] * 3 if compat_shared_scale else [i["tensor_scale"] for i in infos]
    same_ld = len({w.stride(0) for w in ws}) == 1 and all(w.shape == ws[0].shape for w in ws)
    if _codes_gemv_fits(m, k) and same_ld:
        dev = xs[0].device
        st = abi.stream_ptr()
        xs = [t.contiguous() for t in xs]
        codes = torch.empty((3, m, k), dtype=torch.int8, device=dev)
        xsc = torch.empty((3, m), dtype=torch.float32, device=dev)
        outs3 = torch.empty((3, m, n), dtype=torch.float16, device=dev)
        abi.call("rwkvq_prep3_x_int8", xs[0].data_ptr(), xs[1].data_ptr(), xs[2].data_ptr(), abi.dtype_code(xs[0]), m, k, k,
                 codes[0].data_ptr(), codes[1].data_ptr(), codes[2].data_ptr(), k, xsc[0].data_ptr(), xsc[1].data_ptr(),
                 xsc[2].data_ptr(), abi.DEFAULT_DIV, st)
        abi.call("rwkvq_gemm_int8_rkv", codes[0].data_ptr(), codes[1].data_ptr(), codes[2].data_ptr(), k, xsc[0].data_ptr(),
                 xsc[1].data_ptr(), xsc[2].data_ptr(), ws[0].data_ptr(), ws[1].data_ptr(), ws[2].data_ptr(), ws[0].stride(0),
                 scales[0].data_ptr(), scales[1].data_ptr(), scales[2].data_ptr(), outs3[0].data_ptr(), outs3[1].data_ptr(),
                 outs3[2].data_ptr(), n, m, n, k, 0, st)
        abi.after_call()
        outs = [outs3[0], outs3[1], outs3[2]]
    elif _tc_fused_fits(m, k, 3) and same_ld:
        xs = [t.contiguous() for t in xs]
        outs = [torch.empty((m, n), dtype=torch.float16, device=xs[0].device) for _ in range(3)]
        wsp = abi.workspace(m, n, k, 3, xs[0].device)
        abi.call("rwkvq_tc_gemv_int8_rkv", xs[0].data_ptr(), xs[1].data_ptr(), xs[2].data_ptr(), abi.dtype_code(xs[0]),
                 ws[0].data_ptr(), ws[1].data_ptr(), ws[2].data_ptr(), ws[0].stride(0), scales[0].data_ptr(),
                 scales[1].data_ptr(), scales[2].data_ptr(), outs[0].data_ptr(), outs[1].data_ptr(),
                 outs[2].data_ptr(), n, m, n, k, k, abi.DEFAULT_DIV, 0, wsp.data_ptr(), wsp.numel(), abi.stream_ptr())
    elif _gemv_fits(m, k, fp8=False) and same_ld:
        xs = [t.contiguous() for t in xs]
        outs = [torch.empty((m, n), dtype=torch.float16, device=xs[0].device) for _ in range(3)]
        abi.call("rwkvq_gemv_int8_rkv", xs[0].data_ptr(), xs[1].data_ptr(), xs[2].data_ptr(), abi.dtype_code(xs[0]),
                 ws[0].data_ptr(), ws[1].data_ptr(), ws[2].data_ptr(), ws[0].stride(0), scales[0].data_ptr(),
                 scales[1].data_ptr(), scales[2].data_ptr(), outs[0].data_ptr(), outs[1].data_ptr(),
                 outs[2].data_ptr(), n, m, n, k, k, abi.DEFAULT_DIV, 0, abi.stream_ptr())
    elif ROUTE != "mma" and same_ld and m > 0:
        # above the decode kernel's range: ONE row-quantization launch and ONE tensor-core GEMM launch for r, k, v
        # (the reference: 3 x _prep_x_int8_kernel + fused_rkv_int8_kernel)
        dev = xs[0].device
        st = abi.stream_ptr()
        xs = [t.contiguous() for t in xs]
        codes = torch.empty((3, m, k), dtype=torch.int8, device=dev)
        xsc = torch.empty((3, m), dtype=torch.float32, device=dev)
        outs3 = torch.empty((3, m, n), dtype=torch.float16, device=dev)
        abi.call("rwkvq_prep3_x_int8", xs[0].data_ptr(), xs[1].data_ptr(), xs[2].data_ptr(), abi.dtype_code(xs[0]), m, k, k,
                 codes[0].data_ptr(), codes[1].data_ptr(), codes[2].data_ptr(), k, xsc[0].data_ptr(), xsc[1].data_ptr(),
                 xsc[2].data_ptr(), abi.DEFAULT_DIV, st)
        wsp = abi.workspace(min(m, 128), n, k, 3, dev)
        abi.call("rwkvq_tc_gemm_int8_rkv", codes[0].data_ptr(), codes[1].data_ptr(), codes[2].data_ptr(), k, xsc[0].data_ptr(),
                 xsc[1].data_ptr(), xsc[2].data_ptr(), ws[0].data_ptr(), ws[1].data_ptr(), ws[2].data_ptr(), ws[0].stride(0),
                 scales[0].data_ptr(), scales[1].data_ptr(), scales[2].data_ptr(), outs3[0].data_ptr(), outs3[1].data_ptr(),
                 outs3[2].data_ptr(), n, m, n, k, 0, wsp.data_ptr(), wsp.numel(), st)
        abi.after_call(wsp)
        outs = [outs3[0], outs3[1], outs3[2]]
    else:
        outs = [_int8_any(x2, w, s) for x2, w, s in zip(xs, ws, scales)]
    return tuple(_finish(o, lead, n, out_dtype) for o in outs)


# --------------------------------------------------------------------------- dispatcher
def linear_quantized_fused(x, weight_info, out_dtype=torch.float16, push=None):
    """Engine-facing dispatcher (fused_fp8_gemm.py:1080-1098): qtype "int8" -> INT8 path; otherwise FP8, with the
    fused semantics up to FUSED_M_MAX rows and the linear_fp8 semantics (bf16 first, result through bf16) above.
    push (FP8, INT8 and NVFP4): the GEMM also delivers its result to the other ranks of a column-split projection."""
    qtype = weight_info.get("qtype", "fp8")
    m = x.numel() // x.size(-1)
    if m == 1 and qtype == "fp8" and push is None:          # the decode call: straight to the one-launch kernel
        return linear_fp8_m1_fused(x, weight_info, out_dtype)
    if push is not None and qtype not in ("fp8", "int8", "nvfp4"):
        raise RuntimeError(f"rwkvq: no pushing GEMM for qtype {qtype!r}")
    if qtype == "int8":
        return linear_int8_fused(x, weight_info, out_dtype, push=push)
    if qtype == "nvfp4":
        from nvfp4_ops import linear_nvfp4
        return linear_nvfp4(x, weight_info, out_dtype, push=push)
    if qtype.startswith("int4_"):          # weight-info dicts of int4/int4_ops.load_int4_weight
        from int4.int4_ops import linear_int4
        return linear_int4(x, weight_info, out_dtype)
    if m <= FUSED_M_MAX:
        return linear_fp8_fused(x, weight_info, out_dtype=out_dtype, push=push)
    from fp8_ops import linear_fp8
    return linear_fp8(x, weight_info, out_dtype, push=push)
