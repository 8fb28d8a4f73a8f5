"""ctypes binding of librwkvq.so (C ABI declared in include/rwkvq.h).

There is no fallback: if the library is missing, was built for another architecture, or the device is not
compute capability 10.x, the first call raises.  Tensors cross the boundary as raw device pointers
(`tensor.data_ptr()`), sizes and leading dimensions; the stream is torch's current CUDA stream.
"""
from __future__ import annotations

import ctypes
import os

import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.environ.get("RWKVQ_LIB") or os.path.join(_HERE, "librwkvq.so")   # RWKVQ_LIB: another build of the library

OK = 0
F16, BF16 = 0, 1
DIV_IEEE, DIV_FULL, DIV_TORCH = 0, 1, 2
FLAG_AMAX_AFTER_BF16 = 1
FLAG_INT8_SHARED_WSCALE = 2
FLAG_OUT_VIA_BF16 = 4
FLAG_QUANT_FROM_BF16 = 8
FLAG_WSCALE_PER_ROW = 16

# The reference's Triton kernels divide with div.full.f32 on a GPU; RWKVQ_DIV=ieee switches every wrapper
# to IEEE division (what torch and the Triton CPU interpreter compute).
DEFAULT_DIV = DIV_IEEE if os.environ.get("RWKVQ_DIV", "full").lower() == "ieee" else DIV_FULL

_p, _i32, _i64, _u32 = ctypes.c_void_p, ctypes.c_int32, ctypes.c_int64, ctypes.c_uint32

# name -> argtypes (restype is int32 unless listed in _RESTYPES)
SIGNATURES = {
    "rwkvq_version": [],
    "rwkvq_last_error_string": [],
    "rwkvq_device_ok": [],
    "rwkvq_launch_count": [],
    "rwkvq_div_f32": [_p, _p, _p, _i64, _i32, _p],
    "rwkvq_prep_x": [_p, _i32, _i64, _i64, _i64, _p, _p, _i64, _p, _i32, _p],
    "rwkvq_prep3_x": [_p, _p, _p, _i32, _i64, _i64, _i64, _p, _p, _p, _p, _p, _i64, _p, _i32, _p],
    "rwkvq_prep_x_fp8": [_p, _i32, _i64, _i64, _i64, _p, _i64, _p, _p, _p],
    "rwkvq_actq_fp8": [_p, _i32, _i64, _i64, _i64, _p, _i64, _p, _p, _i32, _u32, _p],
    "rwkvq_prep_x_int8": [_p, _i32, _i64, _i64, _i64, _p, _i64, _p, _i32, _p],
    "rwkvq_gemv_fp8": [_p, _i32, _p, _p, _i64, _p, _p, _i64, _i64, _i64, _i64, _i64, _i32, _u32, _p],
    "rwkvq_gemv_fp8_rkv": [_p, _p, _p, _i32, _p, _p, _p, _p, _p, _i64, _p, _p, _p, _p, _p, _p, _i64, _i64, _i64, _i64,
                           _i64, _i32, _u32, _p],
    "rwkvq_gemv_int8": [_p, _i32, _p, _i64, _p, _p, _i64, _p, _i64, _i64, _i64, _i64, _i64, _i32, _u32, _p],
    "rwkvq_gemv_int8_rkv": [_p, _p, _p, _i32, _p, _p, _p, _i64, _p, _p, _p, _p, _p, _p, _i64, _i64, _i64, _i64, _i64,
                            _i32, _u32, _p],
    "rwkvq_gemm_fp8": [_p, _i64, _p, _i32, _p, _i64, _p, _p, _i64, _i64, _i64, _i64, _i32, _u32, _p],
    "rwkvq_gemm_int8": [_p, _i64, _p, _p, _i64, _p, _p, _i64, _p, _i64, _i64, _i64, _i64, _u32, _p],
    "rwkvq_workspace_bytes": [_i64, _i64, _i64, _i32],
    "rwkvq_workspace_status": [_p, _p],
    "rwkvq_tc_gemv_fp8": [_p, _i32, _p, _p, _i64, _p, _p, _i64, _i64, _i64, _i64, _i64, _i32, _u32, _p, _i64, _p],
    "rwkvq_tc_gemv_fp8_rkv": [_p, _p, _p, _i32, _p, _p, _p, _p, _p, _i64, _p, _p, _p, _p, _p, _p, _i64, _i64, _i64,
                              _i64, _i64, _i32, _u32, _p, _i64, _p],
    "rwkvq_tc_gemv_int8": [_p, _i32, _p, _i64, _p, _p, _i64, _p, _i64, _i64, _i64, _i64, _i64, _i32, _u32, _p, _i64, _p],
    "rwkvq_tc_gemv_int8_rkv": [_p, _p, _p, _i32, _p, _p, _p, _i64, _p, _p, _p, _p, _p, _p, _i64, _i64, _i64, _i64,
                               _i64, _i32, _u32, _p, _i64, _p],
    "rwkvq_tc_gemm_fp8": [_p, _i64, _p, _i32, _p, _i64, _p, _p, _i64, _i64, _i64, _i64, _i32, _u32, _p, _i64, _p],
    "rwkvq_tc_gemm_can_push": [_i64, _i64, _i64],
    "rwkvq_tc_gemm_int8_push": [_p, _i64, _p, _p, _i64, _p, _p, _i64, _i64, _i64, _i64, _u32, _p, _i64, _p, _p, _i32, _u32, _p],
    "rwkvq_tc_cluster_gemv_route": [_i64, _i64, _i64],
    "rwkvq_tc_gemm_nvfp4_cluster_route": [_i64, _i64, _i64],
    "rwkvq_tc_gemv_nvfp4_fused_route": [_i64, _i64, _i64],
    "rwkvq_tc_gemv_nvfp4_fused": [_p, _i32, _i64, _p, _i64, _p, _p, _p, _i64, _i64, _i64, _i64, _p],
    "rwkvq_tc_cluster_gemv_fp8": [_p, _i32, _i64, _p, _i64, _p, _p, _i64, _i64, _i64, _i64, _i32, _u32, _p],
    "rwkvq_tc_gemm_fp8_push": [_p, _i64, _p, _i32, _p, _i64, _p, _p, _i64, _i64, _i64, _i64, _i32, _u32, _p, _i64, _p, _p, _i32, _u32, _p],
    "rwkvq_tc_gemm_int8": [_p, _i64, _p, _p, _i64, _p, _p, _i64, _p, _i64, _i64, _i64, _i64, _u32, _p, _i64, _p],
    "rwkvq_gemv_int4_tensor": [_p, _i64, _p, _i64, _p, _p, _i64, _i64, _i64, _i64, _p],
    "rwkvq_gemv_int4_affine": [_p, _i64, _p, _i64, _p, _p, _p, _p, _p, _i64, _i64, _i64, _i64, _p],
    "rwkvq_gemv_int4_group_generic": [_p, _i64, _p, _i64, _p, _p, _i32, _i32, _p, _i64, _i64, _i64, _i64, _p],
    "rwkvq_gemv_int8_w8a16": [_p, _i64, _p, _i64, _p, _p, _i64, _i64, _i64, _i64, _p],
    "rwkvq_gemv_int8_affine": [_p, _i64, _p, _i64, _p, _p, _p, _p, _p, _i64, _i64, _i64, _i64, _p],
    "rwkvq_gemv_int4_group_smem_bytes": [_i64, _i64],
    "rwkvq_gemv_int4_group": [_p, _i64, _p, _i64, _p, _p, _i32, _i32, _p, _i64, _i64, _i64, _i64, _p],
    "rwkvq_gemv_int4_ksplit_slices": [_i64, _i64, _i64],
    "rwkvq_gemv_int4_group_ksplit": [_p, _i64, _p, _i64, _p, _p, _p, _i64, _i64, _i64, _i64, _p, _i64, _p],
    "rwkvq_actq_nvfp4": [_p, _i32, _i64, _i64, _i64, _p, _i64, _p, _i64, _p, _p, _p],
    "rwkvq_gemv_nvfp4_smem_bytes": [_i64, _i64],
    "rwkvq_gemv_nvfp4": [_p, _i64, _p, _i64, _p, _p, _i64, _p, _i64, _p, _p, _i64, _i64, _i64, _i64, _p],
    "rwkvq_actq_nvfp4_fused_scratch_bytes": [],
    "rwkvq_actq_nvfp4_fused": [_p, _i32, _i64, _i64, _i64, _p, _i64, _p, _i64, _p, _p, _p, _i64, _p, _p],
    "rwkvq_gemv_nvfp4_fused_smem_bytes": [_i64, _i64],
    "rwkvq_gemv_nvfp4_fused": [_p, _i32, _i64, _p, _i64, _p, _i64, _p, _p, _i64, _i64, _i64, _i64, _p],
    "rwkvq_nvfp4_blocked_scale_bytes": [_i64, _i64],
    "rwkvq_nvfp4_pack_scales": [_p, _i64, _i64, _i64, _p, _p],
    "rwkvq_tc_gemm_nvfp4": [_p, _i64, _p, _p, _p, _i64, _p, _p, _p, _i64, _i64, _i64, _i64, _p, _i64, _p],
    "rwkvq_tc_gemm_nvfp4_push": [_p, _i64, _p, _p, _p, _i64, _p, _p, _p, _i64, _i64, _i64, _i64, _p, _i64, _p, _p, _i32, _u32, _p],
    "rwkvq_tc_gemm_fp8_static": [_p, _i64, _p, _i32, _p, _i64, _p, _p, _i64, _i64, _i64, _i64, _i32, _u32, _p],
    "rwkvq_actq_fp8_fused_scratch_bytes": [],
    "rwkvq_actq_fp8_fused": [_p, _i32, _i64, _i64, _i64, _p, _i64, _p, _p, _p, _i64, _p, _i32, _u32, _p],
    "rwkvq_actq_fp8_fused3": [_p, _p, _p, _i32, _i64, _i64, _i64, _p, _p, _p, _i64, _p, _p, _i64, _p, _i32, _u32, _p],
    "rwkvq_tc_gemm_fp8_rkv": [_p, _p, _p, _i64, _p, _i32, _p, _p, _p, _i64, _p, _p, _p, _p, _p, _p, _i64, _i64, _i64, _i64,
                              _i32, _u32, _p, _i64, _p],
    "rwkvq_tc_gemm_int8_rkv": [_p, _p, _p, _i64, _p, _p, _p, _p, _p, _p, _i64, _p, _p, _p, _p, _p, _p, _i64, _i64, _i64, _i64,
                               _u32, _p, _i64, _p],
    "rwkvq_tc_static_status": [_p],
    "rwkvq_gemv_batch": [_p, _i32, _p],
    "rwkvq_tc_gemm_fp8_relu2": [_p, _i64, _p, _i32, _p, _i64, _p, _p, _i64, _i64, _i64, _i64, _i32, _u32, _p, _p, _i64, _p],
    "rwkvq_actq_fp8_given": [_p, _i32, _i64, _i64, _i64, _p, _i64, _p, _p, _p, _i32, _u32, _p],
    "rwkvq_actq_int8_given": [_p, _i32, _i64, _i64, _i64, _p, _i64, _p, _p, _i32, _p],
    "rwkvq_tc_gemm_int8_relu2": [_p, _i64, _p, _p, _i64, _p, _p, _i64, _i64, _i64, _i64, _u32, _p, _p, _i64, _p],
    "rwkvq_gemv_fp8_relu2": [_p, _i32, _p, _i64, _p, _p, _i64, _i64, _i64, _i64, _i64, _i32, _u32, _p, _p],
    "rwkvq_gemv_fp8_preamax": [_p, _i32, _p, _i64, _p, _p, _i64, _i64, _i64, _i64, _i64, _i32, _u32, _p, _p],
    "rwkvq_gemv_int8_relu2": [_p, _i32, _p, _i64, _p, _p, _i64, _i64, _i64, _i64, _i64, _i32, _u32, _p, _p],
    "rwkvq_gemv_int8_preamax": [_p, _i32, _p, _i64, _p, _p, _i64, _i64, _i64, _i64, _i64, _i32, _u32, _p, _p],
    "rwkvq_enable_peer_access": [_i32],
    "rwkvq_peer_alloc": [_i64, _p, _p],
    "rwkvq_peer_open": [_p, _p],
    "rwkvq_peer_close": [_p],
    "rwkvq_peer_free": [_p],
    "rwkvq_peer_signal": [_p, _i32, _i32, _u32, _p],
    "rwkvq_allgather_cols_pull": [_p, _p, _u32, _i32, _i32, _i64, _i64, _i64, _p, _p],
    "rwkvq_peer_wait": [_p, _u32, _i32, _i32, _p, _p],
    "rwkvq_prep3_x_int8": [_p, _p, _p, _i32, _i64, _i64, _i64, _p, _p, _p, _i64, _p, _p, _p, _i32, _p],
    "rwkvq_gemm_decode_route": [_i64, _i64],
    "rwkvq_gemm_fp8_rkv": [_p, _p, _p, _i64, _p, _i32, _p, _p, _p, _i64, _p, _p, _p, _p, _p, _p, _i64, _i64, _i64, _i64, _i32, _u32, _p],
    "rwkvq_gemm_int8_rkv": [_p, _p, _p, _i64, _p, _p, _p, _p, _p, _p, _i64, _p, _p, _p, _p, _p, _p, _i64, _i64, _i64, _i64, _u32, _p],
    "rwkvq_set_wait_limit_us": [_i64],
    "rwkvq_device_status": [_p, _i32],
    "rwkvq_selftest_timeout": [_p, _p, _i64, _i32, _p],
    "rwkvq_gemv_set_trace": [_p],
    "rwkvq_tc_set_trace": [_p],
}
_RESTYPES = {"rwkvq_actq_nvfp4_fused_scratch_bytes": ctypes.c_int64, "rwkvq_gemv_nvfp4_fused_smem_bytes": ctypes.c_int64, "rwkvq_nvfp4_blocked_scale_bytes": ctypes.c_int64, "rwkvq_actq_fp8_fused_scratch_bytes": ctypes.c_int64, "rwkvq_gemv_nvfp4_smem_bytes": ctypes.c_int64, "rwkvq_gemv_int4_group_smem_bytes": ctypes.c_int64, "rwkvq_workspace_bytes": ctypes.c_int64, "rwkvq_last_error_string": ctypes.c_char_p, "rwkvq_launch_count": ctypes.c_int64,
             "rwkvq_set_wait_limit_us": None, "rwkvq_gemv_set_trace": None, "rwkvq_tc_set_trace": None}



class ProjDesc(ctypes.Structure):
    """rwkvq_proj_desc of include/rwkvq.h."""
    _fields_ = [("kind", _i32), ("x_dtype", _i32), ("x", _p * 3), ("awq", _p * 2), ("w", _p * 3), ("w_scale", _p * 3),
                ("out", _p * 3), ("ldw", _i64), ("ldo", _i64), ("ldx", _i64), ("M", _i64), ("N", _i64), ("K", _i64),
                ("div_mode", _i32), ("flags", _u32)]


PROJ_FP8, PROJ_FP8_RKV, PROJ_INT8, PROJ_INT8_RKV = 0, 1, 2, 3

_lib = None
_device_checked = False


def lib() -> ctypes.CDLL:
    """The loaded library; raises if it has not been built (python build_ext.py)."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(f"{LIB_PATH} is missing: build it with `python build_ext.py` (nvcc, sm_100a). "
                               "There is no CPU or Triton fallback.")
        L = ctypes.CDLL(LIB_PATH)
        for name, args in SIGNATURES.items():
            fn = getattr(L, name)          # AttributeError here = header and library out of step
            fn.argtypes = args
            fn.restype = _RESTYPES.get(name, _i32)
        _lib = L
    return _lib


def last_error() -> str:
    return lib().rwkvq_last_error_string().decode("utf-8", "replace")


def require_device() -> None:
    global _device_checked
    if _device_checked:
        return
    if not torch.cuda.is_available():
        raise RuntimeError("rwkvq: no CUDA device; this library runs on sm_100a only and has no CPU path")
    rc = lib().rwkvq_device_ok()
    if rc != OK:
        raise RuntimeError(f"rwkvq: {last_error()}")
    _device_checked = True


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)
_raw_device = getattr(torch._C, "_cuda_getDevice", None)


def stream_ptr() -> int:
    """cudaStream_t of torch's current stream on the current device (the raw getters: the Stream object costs 3 us)."""
    if _raw_stream is not None and _raw_device is not None:
        return _raw_stream(_raw_device())
    return torch.cuda.current_stream().cuda_stream


_fn_cache: dict = {}


def call(name: str, *args) -> None:
    """Invoke an entry point; a non-zero status becomes RuntimeError carrying the library's message."""
    fn = _fn_cache.get(name)
    if fn is None:
        require_device()
        fn = _fn_cache[name] = getattr(lib(), name)
    rc = fn(*args)
    if rc != OK:
        raise RuntimeError(f"{name} failed with status {rc}: {last_error()}")


def ptr(t) -> int | None:
    return None if t is None else t.data_ptr()


def dtype_code(t: torch.Tensor) -> int:
    if t.dtype == torch.float16:
        return F16
    if t.dtype == torch.bfloat16:
        return BF16
    raise TypeError(f"rwkvq: activations must be float16 or bfloat16, got {t.dtype}")


def launch_count() -> int:
    return int(lib().rwkvq_launch_count())


def div_on_device(a: torch.Tensor, b: torch.Tensor, mode: int = DIV_FULL) -> torch.Tensor:
    """Element-wise a / b evaluated by the GPU with the chosen division mode (for checkers)."""
    a32 = a.to(device="cuda", dtype=torch.float32).contiguous()
    b32 = torch.broadcast_to(torch.as_tensor(b, dtype=torch.float32).to("cuda"), a32.shape).contiguous()
    out = torch.empty_like(a32)
    call("rwkvq_div_f32", a32.data_ptr(), b32.data_ptr(), out.data_ptr(), a32.numel(), mode, stream_ptr())
    return out


# ---------------------------------------------------------------------------- where a projection writes its result
_out_override: list = []


class output_into:
    """`with output_into(view):` the next single-matrix projection writes its fp16 [M, N] result into `view` (rows may
    be strided: a column range of a wider buffer) instead of a fresh tensor -- the kernels take a leading dimension."""

    def __init__(self, view: torch.Tensor):
        assert view.dim() == 2 and view.dtype == torch.float16 and view.stride(1) == 1 and view.data_ptr() % 16 == 0
        self.view = view

    def __enter__(self):
        _out_override.append(self.view)
        return self.view

    def __exit__(self, *exc):
        _out_override.pop()


def new_out(m: int, n: int, device) -> torch.Tensor:
    if _out_override:
        v = _out_override[-1]
        if tuple(v.shape) != (m, n) or v.device != torch.device(device):
            raise ValueError(f"rwkvq: output view {tuple(v.shape)} on {v.device} does not match the result [{m}, {n}] on {device}")
        return v
    return torch.empty((m, n), dtype=torch.float16, device=device)


# ---------------------------------------------------------------------------- status of the bounded device-side waits
# RWKVQ_CHECK_STATUS=1: every wrapper call that can time out on the device is followed by a read of the status words
# (this synchronizes, so it is a debugging mode); a timeout then raises instead of leaving undefined results behind.
CHECK_STATUS = os.environ.get("RWKVQ_CHECK_STATUS", "0") == "1"
E_TIMEOUT = -6


def device_status(clear: bool = True) -> int:
    """The library's per-device status word (set by kernels whose entry points take no status pointer)."""
    out = ctypes.c_int32(0)
    call("rwkvq_device_status", ctypes.addressof(out), 1 if clear else 0)
    return out.value


def check_status(ws: "torch.Tensor | None" = None) -> None:
    """Raise if a bounded wait gave up since the last check: the per-device word and, if given, a workspace's word.
    A workspace that reported a timeout is cleared again (its arrival counters may be left non-zero)."""
    st = device_status()
    if ws is not None:
        st = st or workspace_status(ws)
        if st:
            ws.zero_()
    if st:
        raise RuntimeError(f"rwkvq: a device-side wait gave up (status {st}); results of the last calls are undefined")


def after_call(ws: "torch.Tensor | None" = None) -> None:
    if CHECK_STATUS:
        check_status(ws)


# ---------------------------------------------------------------------------- scratch of the one-launch quantizers
_scratch: dict = {}


def actq_scratch(device) -> torch.Tensor:
    """Zero-initialised rendezvous scratch of the one-launch activation quantizers, one per (device, stream): calls on
    a stream are ordered, so they share it; the kernels advance its epoch word themselves."""
    key = (torch.device(device).index or 0, torch.cuda.current_stream().cuda_stream)
    sc = _scratch.get(key)
    if sc is None:
        need = max(int(lib().rwkvq_actq_fp8_fused_scratch_bytes()), int(lib().rwkvq_actq_nvfp4_fused_scratch_bytes()))
        sc = torch.zeros(need // 4 + 16, dtype=torch.int32, device=device)
        _scratch[key] = sc
    return sc


# ---------------------------------------------------------------------------- workspace of the tensor-memory kernels
_workspaces: dict = {}


_ws_need: dict = {}


def workspace(m: int, n: int, k: int, nmat: int, device) -> torch.Tensor:
    """Zero-initialised scratch for the tcgen05 kernels, one per (device, stream), grown on demand.
    Launches on one stream are ordered, so they can share it; the kernels leave its counters zero."""
    need = _ws_need.get((m, n, k, nmat))
    if need is None:
        need = _ws_need[(m, n, k, nmat)] = int(lib().rwkvq_workspace_bytes(m, n, k, nmat))
    key = (torch.device(device).index or 0, torch.cuda.current_stream().cuda_stream)
    ws = _workspaces.get(key)
    if ws is None or ws.numel() < need:
        ws = torch.zeros(max(need, 1 << 20), dtype=torch.uint8, device=device)
        _workspaces[key] = ws
    return ws


_plain: dict = {}


def plain_scratch(nbytes: int, device) -> torch.Tensor:
    """Uninitialised scratch (partial sums that a kernel writes before another reads them), one per (device, stream),
    grown on demand.  Separate from workspace(): that one must stay zero between launches."""
    key = (torch.device(device).index or 0, torch.cuda.current_stream().cuda_stream)
    buf = _plain.get(key)
    if buf is None or buf.numel() < nbytes:
        buf = torch.empty(max(int(nbytes), 1 << 20), dtype=torch.uint8, device=device)
        _plain[key] = buf
    return buf


def workspace_status(ws: torch.Tensor) -> int:
    out = ctypes.c_int32(0)
    call("rwkvq_workspace_status", ws.data_ptr(), ctypes.addressof(out))
    return out.value
