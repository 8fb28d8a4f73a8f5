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


class ColumnSplitLinear:
    """y = x @ W^T with W split by output rows across the ranks of `group`, slices all-gathered along the features.

    `linear_fn(x, weight_info, out_dtype)` is the projection to run on the local slice (fp8_ops.linear_quantized for
    FP8 / INT8 / NVFP4 weight-info dicts, int4.int4_ops.linear_int4 for INT4 ones)."""

    def __init__(self, weight_info: dict, linear_fn, group=None, already_sliced: bool = False):
        self.group = group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self.local = weight_info if already_sliced else slice_weight_info(weight_info, self.rank, self.world)
        self.linear_fn = linear_fn

    def __call__(self, x: torch.Tensor, out_dtype=torch.float16) -> torch.Tensor:
        local = self.linear_fn(x, self.local, out_dtype)                  # [..., N/world]
        lead, nl = local.shape[:-1], local.shape[-1]
        flat = local.reshape(-1, nl).contiguous()
        gathered = torch.empty((self.world * flat.shape[0], nl), dtype=flat.dtype, device=flat.device)
        dist.all_gather_into_tensor(gathered, flat, group=self.group)    # NCCL all-gather over NVLink; rank-major rows
        return gathered.reshape(self.world, flat.shape[0], nl).permute(1, 0, 2).reshape(*lead, nl * self.world)
