"""The six quantized projections of one RWKV-7 layer for decode-sized batches, with the host-side work done once.

The reference engine walks its layers in Python (rwkv7_fast_v3a.py:819) and calls the projection API four times per
layer (r/k/v fused, attention output, FFN key, FFN value: rwkv7_fast_v3a.py:982, 1109, 1143-1144).  At batch 1 a
projection kernel runs for 5 to 15 microseconds on a B200, less than the Python work of one drop-in call (argument
checks, output allocation, ctypes marshalling), so a decode loop written that way is bound by the host.  `DecodeLayer`
binds everything that does not change between tokens -- weight pointers, scales, shapes, flags, output buffers --
into C descriptors once; a call fills in the activation pointers and crosses the boundary once (rwkvq_gemv_batch),
either per projection (`rkv`, `att_out`, `ffn_key`, `ffn_value`: for an engine that runs its own kernels in between)
or for all four (`all`).  `capture` records the four launches in a CUDA graph.  The kernels, and therefore the results,
are those of fused_fp8_gemm.linear_rkv_fused / linear_quantized_fused (INT8: linear_rkv_int8_fused / linear_int8_fused)
bit for bit.  Outputs are owned by the object and overwritten by the next call.
"""
from __future__ import annotations

import ctypes

import torch

import rwkvq_abi as abi

MAX_ROWS = 8        # rows the one-launch decode kernel takes (more rows: use the drop-in calls, which quantize once)


class DecodeLayer:
    def __init__(self, r: dict, k: dict, v: dict, o: dict, ffn_key: dict, ffn_value: dict, rows: int = 1,
                 x_dtype: torch.dtype = torch.bfloat16, compat_shared_scale: bool = True):
        """Weight-info dicts as fp8_ops.load_fp8_weight returns them (qtype "fp8" or "int8", all six alike)."""
        abi.require_device()
        infos = (r, k, v, o, ffn_key, ffn_value)
        qtypes = {i.get("qtype", "fp8") for i in infos}
        if len(qtypes) != 1 or next(iter(qtypes)) not in ("fp8", "int8"):
            raise ValueError(f"DecodeLayer takes six FP8 or six INT8 weight-info dicts, got {sorted(qtypes)}")
        if not 1 <= rows <= MAX_ROWS:
            raise ValueError(f"DecodeLayer serves 1..{MAX_ROWS} rows, got {rows}")
        self.int8 = next(iter(qtypes)) == "int8"
        self.rows, self.x_dtype = rows, x_dtype
        self.device = r["weight"].device
        self._keep = infos                                   # the descriptors point into these tensors
        dt = abi.F16 if x_dtype == torch.float16 else abi.BF16
        if x_dtype not in (torch.float16, torch.bfloat16):
            raise TypeError("activations must be float16 or bfloat16")
        for i in (r, k, v):
            if i["weight"].shape != r["weight"].shape or i["weight"].stride(0) != r["weight"].stride(0) or "awq_scale" in i:
                raise ValueError("r, k, v must have one shape and no AWQ divisors (use fused_fp8_gemm.linear_rkv_fused otherwise)")
        self._descs = (abi.ProjDesc * 4)()
        self.outs = []
        # the M == 1 kernel of the reference rounds fp16 input to bf16 before the amax (fused_fp8_gemm.py:662)
        single_flags = abi.FLAG_AMAX_AFTER_BF16 if (rows == 1 and not self.int8) else 0
        plan = ((abi.PROJ_INT8_RKV if self.int8 else abi.PROJ_FP8_RKV, (r, k, v),
                 abi.FLAG_INT8_SHARED_WSCALE if (self.int8 and compat_shared_scale) else 0),
                (abi.PROJ_INT8 if self.int8 else abi.PROJ_FP8, (o,), single_flags),
                (abi.PROJ_INT8 if self.int8 else abi.PROJ_FP8, (ffn_key,), single_flags),
                (abi.PROJ_INT8 if self.int8 else abi.PROJ_FP8, (ffn_value,), single_flags))
        from fused_fp8_gemm import _gemv_fits
        for d, (kind, ws, flags) in zip(self._descs, plan):
            n, kk = ws[0]["weight"].shape
            if kk % 16 or ws[0]["weight"].stride(0) % 16:
                raise ValueError("K and the weight row pitch must be multiples of 16")
            if not _gemv_fits(rows, kk, fp8=not self.int8):
                raise ValueError(f"{rows} rows of K = {kk} do not fit the one-launch decode kernel's shared memory; "
                                 "use the drop-in calls (they quantize once and run the kernel on the codes)")
            outs = torch.empty((len(ws), rows, n), dtype=torch.float16, device=self.device)
            self.outs.append(outs)
            d.kind, d.x_dtype = kind, dt
            for j, info in enumerate(ws):
                w, s = info["weight"], info["tensor_scale"]
                if s.numel() == n and n > 1:
                    flags |= abi.FLAG_WSCALE_PER_ROW
                elif s.numel() != 1:
                    raise ValueError("tensor_scale must hold 1 or N values")
                d.w[j], d.w_scale[j], d.out[j] = w.data_ptr(), s.data_ptr(), outs[j].data_ptr()
            d.ldw, d.ldo, d.ldx, d.M, d.N, d.K = ws[0]["weight"].stride(0), n, kk, rows, n, kk
            d.div_mode, d.flags = abi.DEFAULT_DIV, flags
        self._one = [ctypes.byref(self._descs, i * ctypes.sizeof(abi.ProjDesc)) for i in range(4)]
        self._batch = abi.lib().rwkvq_gemv_batch
        self._k = [int(d.K) for d in self._descs]
        self._ffn_scratch = None

    # ------------------------------------------------------------------ helpers
    def _bind(self, d, j: int, x: torch.Tensor, k: int) -> None:
        if x.dtype != self.x_dtype or x.numel() != self.rows * k or not x.is_contiguous() or x.data_ptr() % 16:
            raise ValueError(f"expected a contiguous, 16-byte aligned {self.x_dtype} tensor of {self.rows} x {k}")
        d.x[j] = x.data_ptr()

    def _launch(self, first: int, count: int) -> None:
        rc = self._batch(self._one[first], count, torch.cuda.current_stream().cuda_stream)
        if rc != abi.OK:
            raise RuntimeError(f"rwkvq_gemv_batch failed with status {rc}: {abi.last_error()}")

    # ------------------------------------------------------------------ one projection per boundary crossing
    def rkv(self, xr, xk, xv):
        d = self._descs[0]
        self._bind(d, 0, xr, self._k[0]); self._bind(d, 1, xk, self._k[0]); self._bind(d, 2, xv, self._k[0])
        self._launch(0, 1)
        o = self.outs[0]
        return o[0], o[1], o[2]

    def att_out(self, x):
        self._bind(self._descs[1], 0, x, self._k[1])
        self._launch(1, 1)
        return self.outs[1][0]

    def ffn_key(self, x):
        self._bind(self._descs[2], 0, x, self._k[2])
        self._launch(2, 1)
        return self.outs[2][0]

    def ffn_value(self, x):
        self._bind(self._descs[3], 0, x, self._k[3])
        self._launch(3, 1)
        return self.outs[3][0]

    def ffn(self, x):
        """value( relu_square( key(x) ) ) in two launches: relu_square runs in the key projection's epilogue, the value
        projection quantizes with the maximum (FP8: of the block; INT8: per token row) that epilogue publishes.
        Returns (ffn output, relu^2 hidden)."""
        dk, dv = self._descs[2], self._descs[3]
        self._bind(dk, 0, x, self._k[2])
        if self._ffn_scratch is None:
            self._ffn_scratch = torch.zeros(16, dtype=torch.int32, device=self.device)
        st, sc = torch.cuda.current_stream().cuda_stream, self._ffn_scratch.data_ptr()
        hid, out = self.outs[2][0], self.outs[3][0]
        if self.int8:
            abi.call("rwkvq_gemv_int8_relu2", dk.x[0], dk.x_dtype, dk.w[0], dk.ldw, dk.w_scale[0], hid.data_ptr(), dk.ldo, dk.M, dk.N, dk.K,
                     dk.ldx, dk.div_mode, dk.flags, sc, st)
            abi.call("rwkvq_gemv_int8_preamax", hid.data_ptr(), abi.F16, dv.w[0], dv.ldw, dv.w_scale[0], out.data_ptr(), dv.ldo, dv.M, dv.N,
                     dv.K, dv.ldx, dv.div_mode, dv.flags, sc, st)
            return out, hid
        abi.call("rwkvq_gemv_fp8_relu2", dk.x[0], dk.x_dtype, dk.w[0], dk.ldw, dk.w_scale[0], hid.data_ptr(), dk.ldo, dk.M, dk.N, dk.K,
                 dk.ldx, dk.div_mode, dk.flags, sc, st)
        abi.call("rwkvq_gemv_fp8_preamax", hid.data_ptr(), abi.F16, dv.w[0], dv.ldw, dv.w_scale[0], out.data_ptr(), dv.ldo, dv.M, dv.N,
                 dv.K, dv.ldx, dv.div_mode, dv.flags, sc, st)
        return out, hid

    # ------------------------------------------------------------------ the whole layer
    def all(self, xr, xk, xv, xo, xf, xg):
        """The four launches of the layer with one boundary crossing; returns (r, k, v, att_out, ffn_key, ffn_value)."""
        d = self._descs
        self._bind(d[0], 0, xr, self._k[0]); self._bind(d[0], 1, xk, self._k[0]); self._bind(d[0], 2, xv, self._k[0])
        self._bind(d[1], 0, xo, self._k[1]); self._bind(d[2], 0, xf, self._k[2]); self._bind(d[3], 0, xg, self._k[3])
        self._launch(0, 4)
        o = self.outs
        return o[0][0], o[0][1], o[0][2], o[1][0], o[2][0], o[3][0]

    def capture(self, xr, xk, xv, xo, xf, xg, stream=None):
        """A CUDA graph of the four launches reading these (static) input tensors; replay() refreshes the outputs."""
        stream = stream or torch.cuda.Stream()
        with torch.cuda.stream(stream):
            self.all(xr, xk, xv, xo, xf, xg)                 # warm-up: per-device kernel attributes are set outside capture
            stream.synchronize()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=stream):
                outs = self.all(xr, xk, xv, xo, xf, xg)
        return graph, outs
