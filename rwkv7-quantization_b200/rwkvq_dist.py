"""Multi-GPU use of the quantized projections: one process per GPU (torch.distributed, NCCL over NVLink).

Two patterns, both outside the reference (which is single-process):

  * rows of activations (sequences in prefill, batch rows in decode) are independent in every projection, so they
    are SHARDED across ranks with replicated weights and no communication: `shard_sequences`, `shard_rows`.
    The FP8 activation scale is per call, so a rank's scale covers its own rows -- exactly what the reference
    computes when it is called on those rows.
  * the FFN key projection [F, C] is COLUMN-SPLIT: every rank keeps F/world output rows of the weight (and of its
    block scales), computes [M, F/world] from the full activations, and the slices are all-gathered along the
    feature dimension: `slice_weight_info`, `ColumnSplitLinear`.
"""
from __future__ import annotations

import torch
import torch.distributed as dist


def shard_rows(m: int, rank: int, world: int) -> tuple[int, int]:
    """Contiguous, balanced split of m rows: rank r gets [start, end)."""
    base, extra = divmod(m, world)
    start = rank * base + min(rank, extra)
    return start, start + base + (1 if rank < extra else 0)


def shard_sequences(num_sequences: int, rank: int, world: int) -> list[int]:
    """Sequence s runs on rank s mod world."""
    return list(range(rank, num_sequences, world))


# weight-info entries with one row per OUTPUT feature (sliced) -- everything else is per input channel or per tensor
_ROW_KEYS = ("weight", "packed", "block_scale", "scales", "zeros", "my", "ry")
# entries derived from the full matrix and cached in the dict by the wrappers: a slice must rebuild its own
_DERIVED_KEYS = ("block_scale_blocked",)


def slice_weight_info(info: dict, rank: int, world: int, align: int = 128) -> dict:
    """Rows [start, end) of a quantized weight (output features) for a column-split projection.  Per-row tensors
    (weight codes, block scales, group scales / zeros, MM4 / MM8 row vectors, a per-row `tensor_scale`) are sliced;
    per-tensor scalars and per-input-channel vectors (`awq_scale`, `mx`, `rx`) are shared; derived caches are dropped.
    Slice boundaries fall on multiples of `align` rows (the kernels' row tile)."""
    n = info["weight" if "weight" in info else "packed"].shape[0]
    if n % (world * align):
        raise ValueError(f"{n} output rows cannot be split into {world} slices of a multiple of {align} rows")
    start, end = rank * (n // world), (rank + 1) * (n // world)
    out = {}
    for key, value in info.items():
        if key in _DERIVED_KEYS:
            continue
        per_row = key in _ROW_KEYS or (key == "tensor_scale" and torch.is_tensor(value) and value.dim() == 1 and value.numel() == n and n > 1)
        out[key] = value[start:end].contiguous() if per_row else value
    return out


class PeerGather:
    """The all-gather of a column-split projection over NVLink peer memory, by this library's own kernels.

    Every rank allocates two result buffers [max_rows, N] fp16 and a flag array, exports them to the other ranks of
    the group as CUDA IPC handles (exchanged once through the process group) and maps theirs.  Per call the local
    projection writes its columns straight into the current buffer, `rwkvq_peer_signal` publishes that on every rank,
    and `rwkvq_allgather_cols_pull` copies the other ranks' columns in with peer loads behind bounded flag waits: the
    result is assembled in its final [M, N] layout, without NCCL, staging or a transposing copy.  The two buffers are
    used in turn, so a rank may compute call i+1 while a peer still reads its columns of call i."""

    def __init__(self, max_rows: int, n_total: int, group=None, device=None):
        import ctypes
        import rwkvq_abi as abi
        self.abi, self.ctypes = abi, ctypes
        self.group = group
        self.world, self.rank = dist.get_world_size(group), dist.get_rank(group)
        if n_total % (8 * self.world):
            raise ValueError(f"{n_total} columns cannot be split into {self.world} slices of a multiple of 8")
        self.n, self.nl, self.max_rows = n_total, n_total // self.world, max_rows
        self.device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
        abi.require_device()
        buf_bytes = max_rows * n_total * 2
        total = 2 * buf_bytes + 512                      # two result buffers, the flag array, the status word
        with torch.cuda.device(self.device):
            ptr, handle = ctypes.c_void_p(), ctypes.create_string_buffer(64)
            abi.call("rwkvq_peer_alloc", total, ctypes.byref(ptr), handle)
            self._base = ptr.value
            everyone = [None] * self.world
            dist.all_gather_object(everyone, bytes(handle.raw), group=group)
            bases, self._opened = [], []
            for r, h in enumerate(everyone):
                if r == self.rank:
                    bases.append(self._base)
                    continue
                p = ctypes.c_void_p()
                abi.call("rwkvq_peer_open", ctypes.create_string_buffer(h, 64), ctypes.byref(p))   # this rank's device is current
                self._opened.append(p.value)
                bases.append(p.value)

        class _Raw:                                       # the library's allocation as a torch tensor (zero copy)
            def __init__(self, address, nbytes):
                self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (address, False), "version": 3}
        raw = torch.as_tensor(_Raw(self._base, total), device=self.device)
        self.bufs = [raw[i * buf_bytes:(i + 1) * buf_bytes].view(torch.float16).view(max_rows, n_total) for i in range(2)]
        self.flags = raw[2 * buf_bytes:2 * buf_bytes + 256].view(torch.int32)
        self.status = raw[2 * buf_bytes + 256:2 * buf_bytes + 260].view(torch.int32)
        arr = ctypes.c_void_p * self.world
        self._out_arrays = [arr(*[b + i * buf_bytes for b in bases]) for i in range(2)]
        self._flag_array = arr(*[b + 2 * buf_bytes for b in bases])
        # push form: this rank's column range in every OTHER rank's buffers, and its slot in their flag arrays
        peers = [r for r in range(self.world) if r != self.rank]
        parr = ctypes.c_void_p * max(len(peers), 1)
        col0 = self.rank * self.nl * 2
        self._push_out = [parr(*[bases[r] + i * buf_bytes + col0 for r in peers]) if peers else parr() for i in range(2)]
        self._push_flag = parr(*[bases[r] + 2 * buf_bytes + 4 * self.rank for r in peers]) if peers else parr()
        self._npeers = len(peers)
        self.epoch = 0
        dist.barrier(group=group)      # every rank has mapped every buffer before anyone signals

    def close(self) -> None:
        """Unmap the peers' buffers and free this rank's (after a barrier: nobody may still be reading it)."""
        if self._base is None:
            return
        torch.cuda.synchronize(self.device)
        dist.barrier(group=self.group)
        with torch.cuda.device(self.device):
            for p in self._opened:
                self.abi.call("rwkvq_peer_close", p)
            dist.barrier(group=self.group)
            self.bufs, self.flags, self.status = [], None, None
            self.abi.call("rwkvq_peer_free", self._base)
        self._base = None

    def next_buffer(self, m: int) -> torch.Tensor:
        """Advance to the next call; returns this rank's column view [m, N/world] of the buffer to write into."""
        if m > self.max_rows:
            raise ValueError(f"{m} rows exceed the {self.max_rows} the peer buffers were sized for")
        self.epoch += 1
        self.m = m
        buf = self.bufs[self.epoch & 1]
        return buf[:m, self.rank * self.nl:(self.rank + 1) * self.nl]

    def gather(self) -> torch.Tensor:
        """Signal this rank's columns, pull everybody else's; returns the assembled [m, N] (a view of the buffer, valid
        until the call after next)."""
        abi, b = self.abi, self.epoch & 1
        st = abi.stream_ptr()
        abi.call("rwkvq_peer_signal", self._flag_array, self.rank, self.world, self.epoch, st)
        abi.call("rwkvq_allgather_cols_pull", self._out_arrays[b], self.flags.data_ptr(), self.epoch, self.rank, self.world,
                 self.m, self.nl, self.n, self.status.data_ptr(), st)
        return self.bufs[b][:self.m]

    def push_targets(self):
        """What a pushing GEMM needs for the current call (after next_buffer): (peer_out, peer_flag, npeers, epoch)."""
        return self._push_out[self.epoch & 1], self._push_flag, self._npeers, self.epoch

    def wait(self) -> torch.Tensor:
        """Receiver side of a pushed call: wait (on the stream, bounded) for every other rank's signal; returns [m, N]."""
        abi = self.abi
        abi.call("rwkvq_peer_wait", self.flags.data_ptr(), self.epoch, self.rank, self.world, self.status.data_ptr(), abi.stream_ptr())
        return self.bufs[self.epoch & 1][:self.m]

    def check(self) -> None:
        """Raise if a pull gave up waiting for a peer (synchronizes)."""
        if int(self.status.item()) != 0:
            self.status.zero_()
            raise RuntimeError("rwkvq: a rank did not deliver its columns within the wait limit")


class ColumnSplitLinear:
    """y = x @ W^T with W split by output rows across the ranks of `group`, slices gathered along the features.

    `linear_fn(x, weight_info, out_dtype)` is the projection to run on the local slice (fp8_ops.linear_quantized for
    FP8 / INT8 / NVFP4 weight-info dicts, int4.int4_ops.linear_int4 for INT4 ones).  gather="nccl": an NCCL all-gather
    (rank-major) followed by one copy into the [M, N] layout; gather="peer": PeerGather above (GPU only, fp16 results;
    `max_rows` sizes its buffers); gather="push": the projection's GEMM stores its result tiles into every rank's buffer
    itself and the receivers only wait for a flag (FP8, INT8 and NVFP4 weights, row counts that run the tiled tensor-core
    GEMM; other calls fall back to "peer").  The pushed FP8 result follows linear_quantized_fused's semantics.
    gather="auto": "push" where it was measured faster than "peer" -- up to 4 ranks at every row count (4096 rows:
    194 against 266 us on 2 GPUs, 232 against 279 us on 4), on more ranks up to PUSH_MAX_ROWS_WIDE rows (8 GPUs: 78
    against 80 us at 256 rows, but 548 against 284 us at 4096, where every epilogue warp stores each tile to seven
    peers) -- else "peer".  The choice depends on sizes only, so every rank makes the same one."""

    PUSH_MAX_ROWS_WIDE = 512

    @classmethod
    def auto_pushes(cls, world: int, rows: int) -> bool:
        """gather="auto": does a call of `rows` rows on `world` ranks push (True) or pull (False)?"""
        return world <= 4 or rows <= cls.PUSH_MAX_ROWS_WIDE

    def __init__(self, weight_info: dict, linear_fn, group=None, already_sliced: bool = False, gather: str = "nccl", max_rows: int = 4096):
        if gather not in ("nccl", "peer", "push", "auto"):
            raise ValueError(f"gather must be 'nccl', 'peer', 'push' or 'auto', got {gather!r}")
        self.group = group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self.local = weight_info if already_sliced else slice_weight_info(weight_info, self.rank, self.world)
        self.linear_fn = linear_fn
        self.n_local = self.local["weight" if "weight" in self.local else "packed"].shape[0]
        self.peer = PeerGather(max_rows, self.n_local * self.world, group) if gather in ("peer", "push", "auto") else None
        self.auto = gather == "auto"
        # "push": the GEMM itself stores its tiles into every rank's buffer (one kernel computes and gathers); taken where
        # the projection runs the kernel that can do it (NVFP4 weights on the tensor-core route), else the pull form
        self.push = gather in ("push", "auto") and self.local.get("qtype", "fp8") in ("nvfp4", "fp8", "int8")

    def __call__(self, x: torch.Tensor, out_dtype=torch.float16) -> torch.Tensor:
        if self.peer is not None:
            import rwkvq_abi as abi
            x2 = x.reshape(-1, x.shape[-1])
            pushing = False
            if self.push and (not self.auto or self.auto_pushes(self.world, x2.shape[0])):
                if self.local.get("qtype") == "nvfp4":
                    import nvfp4_ops
                    pushing = nvfp4_ops.can_push(x2.shape[0], x2.shape[1])
                else:
                    import fused_fp8_gemm
                    pushing = fused_fp8_gemm.can_push(x2.shape[0], self.n_local, x2.shape[1])
            with abi.output_into(self.peer.next_buffer(x2.shape[0])):
                if pushing:
                    import fused_fp8_gemm
                    fused_fp8_gemm.linear_quantized_fused(x2, self.local, torch.float16, push=self.peer.push_targets())
                else:
                    self.linear_fn(x2, self.local, torch.float16)         # writes this rank's columns in place
            y = (self.peer.wait() if pushing else self.peer.gather()).reshape(*x.shape[:-1], self.n_local * self.world)
            return y if out_dtype in (None, torch.float16) else y.to(out_dtype)
        local = self.linear_fn(x, self.local, out_dtype)                  # [..., N/world]
        lead, nl = local.shape[:-1], local.shape[-1]
        flat = local.reshape(-1, nl).contiguous()
        gathered = torch.empty((self.world * flat.shape[0], nl), dtype=flat.dtype, device=flat.device)
        dist.all_gather_into_tensor(gathered, flat, group=self.group)    # NCCL all-gather over NVLink; rank-major
        gathered = gathered.view(self.world, flat.shape[0], nl)
        if flat.shape[0] == 1:
            return gathered.reshape(*lead, nl * self.world)               # one row: rank-major IS the feature order
        out = torch.empty((flat.shape[0], self.world, nl), dtype=flat.dtype, device=flat.device)
        out.copy_(gathered.permute(1, 0, 2))                              # one strided copy into the [M, N] layout
        return out.reshape(*lead, nl * self.world)
