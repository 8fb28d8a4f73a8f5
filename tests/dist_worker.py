"""One gloo rank of the CPU multi-process test: python dist_worker.py RANK WORLD PORT."""
import os
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path[:0] = [ROOT, os.path.join(ROOT, "rwkv7-quantization_b200")]

import torch
import torch.distributed as dist

import rwkvq_dist as D
from oracle import rwkvq_oracle as O


def cpu_linear(x, info, out_dtype=torch.float16):
    """Stand-in for the GPU projection in this host-logic test."""
    return O.cpu_dequant_matmul_fp8(x, info).to(out_dtype).reshape(*x.shape[:-1], info["weight"].shape[0])


def main():
    rank, world, port = int(sys.argv[1]), int(sys.argv[2]), sys.argv[3]
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    g = torch.Generator().manual_seed(0)
    q, s = O.q_fp8(torch.randn(256, 64, generator=g) / 8)
    info = {"weight": q, "tensor_scale": s, "qtype": "fp8"}
    x = torch.randn(2, 3, 64, generator=g).to(torch.bfloat16)
    y = D.ColumnSplitLinear(info, cpu_linear)(x)
    ok_split = torch.equal(y, cpu_linear(x, info)) and y.shape == (2, 3, 256)
    rows = x.reshape(-1, 64)
    s0, s1 = D.shard_rows(rows.shape[0], rank, world)
    parts = [None] * world
    dist.all_gather_object(parts, cpu_linear(rows[s0:s1], info))
    ok_rows = torch.equal(torch.cat(parts), cpu_linear(rows, info))
    print(f"rank {rank} split={ok_split} rows={ok_rows}")
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
