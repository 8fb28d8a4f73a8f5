"""NVFP4 (W4A4) scheme: offline weight quantizer, loader and projection.

The reference repository describes this format in its reports but ships no code for it any more, so this module is
an addition behind the same conventions as fp8_ops.py:

    storage (07_quantization_toolchain_v2_en.md:18-25)
        <key>                 uint8 [N, K/2]   two e2m1 codes per byte, even k in the low nibble
        <key>.nf4_b_scale     float8_e4m3fn [N, K/16]   one scale per 16 consecutive k
        <key>.nvfp4_t_scale   float32 scalar            amax / 2688  (2688 = 448 * 6)
    weight-info dict   {"weight", "block_scale", "tensor_scale", "qtype": "nvfp4"}
    arithmetic (03_fused_kernel_en.md:22-34, 11_fused_gemm_ops_en.md:20-26)
        block scale = e4m3(clamp(max|x|_16 * 448 / amax, 2^-6, 448));  code = e2m1_rn(x / pts / block scale)
        out = (sum codeA*bsA * codeB*bsB) * ptsA * ptsW
"""
from __future__ import annotations

import os

import torch

import rwkvq_abi as abi

E2M1_VALUES = (0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0)
BLOCK = 16
GEMV_ROWS = 16
ONE_LAUNCH = os.environ.get("RWKVQ_NVFP4_ONE_LAUNCH", "0") == "1"   # 1-4 tokens: quantization inside the cluster kernel (see linear_nvfp4)
TC_LONG_K = int(os.environ.get("RWKVQ_NVFP4_TC_LONG_K", "8192"))   # rows this long go to the tensor-core route at every token count
TC_WIDE_N = int(os.environ.get("RWKVQ_NVFP4_TC_WIDE_N", "8192"))   # this many weight rows: from 3 tokens on
TC_MIN_M = int(os.environ.get("RWKVQ_NVFP4_TC_MIN_M", "8"))   # more tokens than this go to the tensor-core GEMM (measured: from 9 rows it is as fast or faster on the 7.2B shapes)


def _e2m1_codes(v: torch.Tensor) -> torch.Tensor:
    """fp32 -> 4-bit e2m1 codes (sign << 3 | index), round-to-nearest-even on the value grid, saturating."""
    a = v.abs().clamp(max=6.0)
    # thresholds are the midpoints; a tie goes to the neighbour with an even index
    idx = ((a > 0.25).to(torch.uint8) + (a >= 0.75) + (a > 1.25) + (a >= 1.75) + (a > 2.5) + (a >= 3.5) + (a > 5.0))
    return (idx | (torch.signbit(v).to(torch.uint8) << 3)).to(torch.uint8)


def quantize_to_nvfp4(w: torch.Tensor):
    """Offline weight quantization (any device).  Returns the weight-info dict; store it with `to_state`."""
    wf = w.float()
    n, k = wf.shape
    assert k % BLOCK == 0, f"K={k} must be a multiple of {BLOCK}"
    amax = wf.abs().max().clamp(min=1e-12)
    pts = amax / 2688.0
    blk = wf.reshape(n, k // BLOCK, BLOCK)
    sb = (blk.abs().amax(dim=2) * (448.0 / amax)).clamp(2.0 ** -6, 448.0)
    bs = sb.to(torch.float8_e4m3fn)
    codes = _e2m1_codes((blk * (1.0 / pts) / bs.float().unsqueeze(2)).reshape(n, k))
    packed = codes[:, 0::2] | (codes[:, 1::2] << 4)
    return {"weight": packed.contiguous(), "block_scale": bs.contiguous(), "tensor_scale": pts.reshape(()).float(), "qtype": "nvfp4"}


def dequantize_nvfp4(info) -> torch.Tensor:
    """code * block scale * tensor scale as fp32 [N, K]."""
    p = info["weight"]
    codes = torch.stack((p & 0xF, p >> 4), dim=-1).reshape(p.shape[0], -1).long()
    table = torch.tensor(E2M1_VALUES + tuple(-x for x in E2M1_VALUES), dtype=torch.float32, device=p.device)
    vals = table[codes]
    return vals * info["block_scale"].float().repeat_interleave(BLOCK, dim=1) * info["tensor_scale"].float()


def to_state(key: str, info) -> dict:
    return {key: info["weight"], key + ".nf4_b_scale": info["block_scale"], key + ".nvfp4_t_scale": info["tensor_scale"]}


def is_nvfp4_weight(z, key) -> bool:
    return (key + ".nf4_b_scale") in z


def load_nvfp4_weight(z, key, dev):
    """Move an NVFP4 weight to `dev`, drop its side keys from `z` (as load_fp8_weight does) and describe it."""
    return {"weight": z[key].to(dev).contiguous(), "block_scale": z.pop(key + ".nf4_b_scale").to(dev).contiguous(),
            "tensor_scale": z.pop(key + ".nvfp4_t_scale").to(dev).float(), "qtype": "nvfp4"}


def quantize_activations_nvfp4(x: torch.Tensor, blocked: bool = False):
    """On-the-fly activation quantization on the device (one cluster launch, two chained launches or one cooperative
    launch by block size: rwkvq_actq_nvfp4_fused picks):
    (packed codes [M,K/2], block scales [M,K/16] e4m3, pts [1]); with blocked=True the scales come in the blocked
    order of the tensor-core GEMM (a flat uint8 buffer) instead of row-major."""
    from fused_fp8_gemm import _rows16
    x2 = _rows16(x).contiguous()
    m, k = x2.shape
    dev = x2.device
    codes = torch.empty((m, k // 2), dtype=torch.uint8, device=dev)
    pts = torch.empty(1, dtype=torch.float32, device=dev)
    if os.environ.get("RWKVQ_NVFP4_ACTQ", "fused") != "fused" or m == 0 or (blocked and k % 64):
        bs = torch.empty((m, k // BLOCK), dtype=torch.float8_e4m3fn, device=dev)
        amax = torch.empty(1, dtype=torch.float32, device=dev)
        abi.call("rwkvq_actq_nvfp4", x2.data_ptr(), abi.dtype_code(x2), m, k, k, codes.data_ptr(), k // 2, bs.data_ptr(),
                 k // BLOCK, pts.data_ptr(), amax.data_ptr(), abi.stream_ptr())
        return codes, (pack_scales(bs, k) if blocked else bs), pts
    scratch = abi.actq_scratch(dev)
    if blocked:
        bs = torch.empty(int(abi.lib().rwkvq_nvfp4_blocked_scale_bytes(m, k)), dtype=torch.uint8, device=dev)
        rows_ptr, blk_ptr = None, bs.data_ptr()
    else:
        bs = torch.empty((m, k // BLOCK), dtype=torch.float8_e4m3fn, device=dev)
        rows_ptr, blk_ptr = bs.data_ptr(), None
    abi.call("rwkvq_actq_nvfp4_fused", x2.data_ptr(), abi.dtype_code(x2), m, k, k, codes.data_ptr(), k // 2, rows_ptr, k // BLOCK,
             blk_ptr, pts.data_ptr(), scratch.data_ptr(), scratch.numel() * 4, None, abi.stream_ptr())
    return codes, bs, pts


def pack_scales(block_scales: torch.Tensor, k: int) -> torch.Tensor:
    """Row-major scales [rows, K/16] -> the blocked order the tensor core reads (512-byte chunks per 128 rows x 64 k)."""
    rows = block_scales.shape[0]
    out = torch.empty(int(abi.lib().rwkvq_nvfp4_blocked_scale_bytes(rows, k)), dtype=torch.uint8, device=block_scales.device)
    abi.call("rwkvq_nvfp4_pack_scales", block_scales.data_ptr(), block_scales.stride(0), rows, k, out.data_ptr(), abi.stream_ptr())
    return out


def _blocked_weight_scales(weight_info, k: int) -> torch.Tensor:
    """The weight's scales in blocked order, packed on first use and kept in the weight-info dict."""
    blk = weight_info.get("block_scale_blocked")
    if blk is None or blk.device != weight_info["block_scale"].device:
        blk = pack_scales(weight_info["block_scale"], k)
        weight_info["block_scale_blocked"] = blk
    return blk


def _route(m: int, k: int, n: int = 0) -> str:
    """'fused' = one launch, activation quantization in the GEMV's prologue (up to TC_MIN_M tokens, K a multiple of 512);
    'tc' = block-scaled tensor-core GEMM (more tokens, K a multiple of 256); 'gemv' = quantization kernels + the
    16-row GEMV (any K that is a multiple of 128).
    The fused GEMV quantizes the whole block in every CTA and converts every weight code in registers; the tensor-core
    route quantizes once and streams the codes into block-scaled MMAs (K split across a cluster), so it takes over where
    the prologue or the conversions weigh: measured at K = 16384 from one token on (13.2 against 16.3 us; 4 tokens 17.4
    against 25.2), and at K = 4096 against many weight rows from 3 tokens on (N = 16384, 4 tokens: 13.9 against 16.0 us;
    8 tokens: 14.3 against 19.7)."""
    forced = os.environ.get("RWKVQ_NVFP4_ROUTE", "auto")
    if forced == "gemv" or k % 256 != 0:
        return "gemv"
    if forced == "tc" or m > TC_MIN_M:
        return "tc"
    if forced == "auto" and (k >= TC_LONG_K or (m >= 3 and n >= TC_WIDE_N)) and abi.lib().rwkvq_tc_gemm_nvfp4_cluster_route(m, n, k):
        return "tc"
    # the tensor scale is per call: all rows must go into one launch
    if k % 512 == 0 and abi.lib().rwkvq_gemv_nvfp4_fused_smem_bytes(m, k) <= 224 * 1024:
        return "fused"
    # rows that do not fit one fused launch (long rows): the GEMM streams the weights once, row blocks would re-read them
    return "tc" if m > 4 else "gemv"


def can_push(m: int, k: int) -> bool:
    """True if linear_nvfp4 with these rows runs the kernel that can carry the all-gather of a column-split projection."""
    return m > 0 and _route(m, k) == "tc"


def linear_nvfp4(x, weight_info, out_dtype=torch.float16, push=None):
    """W4A4 projection: activations quantized per call, weights streamed in packed form.  Few tokens run the
    weight-streaming GEMV; more than TC_MIN_M tokens run the tcgen05 block-scaled GEMM.
    push = (peer_out_array, peer_flag_array, npeers, epoch) from rwkvq_dist.PeerGather.push_targets(): the GEMM also
    stores its result into the peers' buffers and signals them (only on the GEMM route: check can_push first)."""
    w, wbs, wts = weight_info["weight"], weight_info["block_scale"], weight_info["tensor_scale"]
    n, k = w.shape[0], w.shape[1] * 2
    wts = wts.reshape(1)
    from fused_fp8_gemm import _rows16
    x2 = _rows16(x).contiguous()
    m = x2.shape[0]
    route = _route(m, k, n)
    if push is not None and route != "tc":
        raise RuntimeError("rwkvq: the pushed all-gather rides in the tensor-core GEMM only (see can_push)")
    if route == "fused" and wbs.stride(0) % 16 == 0 and wbs.data_ptr() % 16 == 0:
        out = abi.new_out(m, n, x2.device)
        abi.call("rwkvq_gemv_nvfp4_fused", x2.data_ptr(), abi.dtype_code(x2), k, w.data_ptr(), w.stride(0), wbs.data_ptr(),
                 wbs.stride(0), wts.data_ptr(), out.data_ptr(), out.stride(0), m, n, k, abi.stream_ptr())
        out = out.reshape(*x.shape[:-1], n)
        return out if out_dtype in (None, out.dtype) else out.to(out_dtype)
    if (ONE_LAUNCH and route == "tc" and push is None and 0 < m <= 4 and os.environ.get("RWKVQ_NVFP4_ROUTE", "auto") == "auto"
            and abi.lib().rwkvq_tc_gemv_nvfp4_fused_route(m, n, k)):
        # one to four tokens in ONE launch: the activation quantization runs inside the cluster split-K kernel (same bits as
        # the quantizer launch followed by the GEMM).  Opt-in: measured as fast or slower than the two launches (FFN value,
        # one token: 14.0 against 12.8 us; FFN key: 12.2 against 12.0) -- the quantizer launch already runs under the
        # GEMM's weight prefetch, and inside the kernel the MMAs wait for the same abs-max exchange.
        out = abi.new_out(m, n, x2.device)
        w_blk = _blocked_weight_scales(weight_info, k)
        abi.call("rwkvq_tc_gemv_nvfp4_fused", x2.data_ptr(), abi.dtype_code(x2), k, w.data_ptr(), w.stride(0), w_blk.data_ptr(),
                 wts.data_ptr(), out.data_ptr(), out.stride(0), m, n, k, abi.stream_ptr())
        out = out.reshape(*x.shape[:-1], n)
        return out if out_dtype in (None, out.dtype) else out.to(out_dtype)
    codes, bs, pts = quantize_activations_nvfp4(x, blocked=(route == "tc"))
    out = abi.new_out(m, n, codes.device)
    if route == "tc":
        ws = abi.workspace(1, 1, 1, 1, codes.device)
        a_blk, w_blk = bs, _blocked_weight_scales(weight_info, k)     # both alive until the launch
        if push is not None:
            abi.call("rwkvq_tc_gemm_nvfp4_push", codes.data_ptr(), k // 2, a_blk.data_ptr(), pts.data_ptr(), w.data_ptr(), w.stride(0),
                     w_blk.data_ptr(), wts.data_ptr(), out.data_ptr(), out.stride(0), m, n, k, ws.data_ptr(), ws.numel(),
                     push[0], push[1], push[2], push[3], abi.stream_ptr())
        else:
            abi.call("rwkvq_tc_gemm_nvfp4", codes.data_ptr(), k // 2, a_blk.data_ptr(), pts.data_ptr(), w.data_ptr(), w.stride(0),
                     w_blk.data_ptr(), wts.data_ptr(), out.data_ptr(), out.stride(0), m, n, k, ws.data_ptr(), ws.numel(), abi.stream_ptr())
    else:
        rows = GEMV_ROWS
        while rows > 1 and abi.lib().rwkvq_gemv_nvfp4_smem_bytes(rows, k) > 200 * 1024:
            rows //= 2
        for r0 in range(0, m, rows):
            r = min(rows, m - r0)
            abi.call("rwkvq_gemv_nvfp4", codes[r0:].data_ptr(), k // 2, bs[r0:].data_ptr(), k // BLOCK, pts.data_ptr(),
                     w.data_ptr(), w.stride(0), wbs.data_ptr(), wbs.stride(0), wts.data_ptr(), out[r0:].data_ptr(), out.stride(0), r, n, k,
                     abi.stream_ptr())
    out = out.reshape(*x.shape[:-1], n)
    return out if out_dtype in (None, out.dtype) else out.to(out_dtype)
