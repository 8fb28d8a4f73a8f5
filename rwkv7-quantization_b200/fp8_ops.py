"""Drop-in for the reference module `fp8_ops.py` (quantized-weight detection, loading and the engine-facing
linear dispatchers) on top of librwkvq.so.  Names, arguments and the weight-info dict are the reference's:

    {"weight": [N, K] float8_e4m3fn | int8 (contiguous, on the device),
     "tensor_scale": fp32 scalar on the device, "qtype": "fp8" | "int8"}          (fp8_ops.py:26-49)
"""
import os

import torch

import rwkvq_abi as abi

FP8_E4M3_MAX = 448.0
FUSED_M_MAX = int(os.environ.get("RWKVQ_FUSED_M_MAX", "512"))   # rows up to which the engine takes the fused r/k/v route (fp8_ops.py:118); the fused calls here serve any row count


def is_fp8_weight(z, key):
    """True when `key` has a quantization scale stored beside it (fp8_ops.py:17-19)."""
    return (key + ".fp8_scale") in z


def load_fp8_weight(z, key, dev):
    """Move a quantized weight and its per-tensor scale to `dev`, drop the scale key from `z`, and describe the
    pair as a weight-info dict (fp8_ops.py:26-49).  The quantized type follows from the storage dtype."""
    weight = z[key].to(device=dev).contiguous()
    scale = z.pop(key + ".fp8_scale").to(device=dev)
    return {
        "weight": weight,
        "tensor_scale": scale,
        "qtype": "fp8" if weight.dtype == torch.float8_e4m3fn else "int8",
    }


def linear_fp8(x, weight_info, out_dtype=torch.float16, push=None):
    """The large-M FP8 route (fp8_ops.py:58-86): fp16 activations are taken as bf16, quantized per call with torch's
    scale arithmetic, multiplied on the tensor cores, and the result is rounded to bf16 before `out_dtype`.
    push = (peer_out, peer_flag, npeers, epoch): the GEMM also stores its result into the other ranks' buffers and signals
    them (column-split projection, rwkvq_dist.PeerGather.push_targets; only row counts with fused_fp8_gemm.can_push)."""
    import fused_fp8_gemm as f
    w, w_ts = weight_info["weight"], weight_info["tensor_scale"]
    x2 = f._rows16(x)
    m, k = x2.shape
    n = w.shape[0]
    dev = x2.device
    codes = torch.empty((m, k), dtype=torch.uint8, device=dev)
    amax = torch.empty(1, dtype=torch.float32, device=dev)
    scale = torch.empty(1, dtype=torch.float32, device=dev)
    out = abi.new_out(m, n, dev)
    st = abi.stream_ptr()
    # inv = 448/amax and scale = amax/448 the way torch evaluates them on a GPU in prep_x_fp8 (DIV_TORCH)
    f._actq_fp8(x2, codes, amax, scale, abi.DIV_TORCH, abi.FLAG_AMAX_AFTER_BF16 | abi.FLAG_QUANT_FROM_BF16, st)
    gflags = abi.FLAG_OUT_VIA_BF16 | f._wscale_flag(w_ts, n)
    if push is not None:
        if not f.can_push(m, n, k):
            raise RuntimeError("rwkvq: the pushed all-gather rides in the tiled tensor-core GEMM only (see can_push)")
        ws = abi.workspace(min(m, 128), n, k, 1, dev)
        abi.call("rwkvq_tc_gemm_fp8_push", codes.data_ptr(), k, scale.data_ptr(), 0, f._u8(w).data_ptr(), w.stride(0),
                 w_ts.data_ptr(), out.data_ptr(), out.stride(0), m, n, k, abi.DIV_IEEE, gflags, ws.data_ptr(), ws.numel(),
                 push[0], push[1], push[2], push[3], st)
        abi.after_call(ws)
    elif f.ROUTE != "mma":
        ws = abi.workspace(min(m, 128), n, k, 1, dev)
        abi.call("rwkvq_tc_gemm_fp8", codes.data_ptr(), k, scale.data_ptr(), 0, f._u8(w).data_ptr(), w.stride(0),
                 w_ts.data_ptr(), out.data_ptr(), out.stride(0), m, n, k, abi.DIV_IEEE, gflags, ws.data_ptr(), ws.numel(), st)
        abi.after_call(ws)
    else:
        abi.call("rwkvq_gemm_fp8", codes.data_ptr(), k, scale.data_ptr(), 0, f._u8(w).data_ptr(), w.stride(0),
                 w_ts.data_ptr(), out.data_ptr(), out.stride(0), m, n, k, abi.DIV_IEEE, gflags, st)
    return f._finish(out, x.shape[:-1], n, out_dtype)


def linear_int8(x, weight_info, out_dtype=torch.float16):
    """INT8 W8A8 projection (fp8_ops.py:90-97)."""
    from fused_fp8_gemm import linear_int8_fused
    return linear_int8_fused(x, weight_info, out_dtype)


def linear_quantized(x, weight_info, out_dtype=torch.float16):
    """Pick the projection by `qtype` (fp8_ops.py:100-106)."""
    qtype = weight_info.get("qtype", "fp8")
    if qtype == "int8":
        return linear_int8(x, weight_info, out_dtype)
    if qtype == "nvfp4":
        from nvfp4_ops import linear_nvfp4
        return linear_nvfp4(x, weight_info, out_dtype)
    if qtype.startswith("int4_"):          # weight-info dicts of int4/int4_ops.load_int4_weight
        from int4.int4_ops import linear_int4
        return linear_int4(x, weight_info, out_dtype)
    return linear_fp8(x, weight_info, out_dtype)


def linear_quantized_fused(x, weight_info, out_dtype=torch.float16, push=None):
    """Forward to the dispatcher of fused_fp8_gemm (fp8_ops.py:109-115)."""
    from fused_fp8_gemm import linear_quantized_fused as dispatch
    return dispatch(x, weight_info, out_dtype, push=push) if push is not None else dispatch(x, weight_info, out_dtype)
