"""One NCCL rank of the multi-GPU column-split test: python dist_gpu_worker.py RANK WORLD PORT.

The FFN key projection [16384, 4096] of RWKV-7 7.2B is split by output rows over the ranks; every rank computes its
slice on its own GPU and the slices are gathered -- through NCCL, through the library's peer-memory pull, and (NVFP4,
256 rows) by the GEMM itself storing its tiles into every rank's buffer.
Checked per rank: both gathers equal the concatenation of the per-slice projections computed locally (bit for bit)
and the unsplit projection within 1e-2 (INT8: bit for bit; FP8 decode splits K by the slice's tile count, so the
order of its fp32 additions may differ from the unsplit run)."""
import os
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path[:0] = [ROOT, os.path.join(ROOT, "rwkv7-quantization_b200")]

import torch
import torch.distributed as dist


def rel_err(out, ref):
    out, ref = out.float(), ref.float()
    floor = 0.02 * ref.pow(2).mean().sqrt().item() + 1e-30
    return ((out - ref).abs() / ref.abs().clamp(min=floor)).max().item()


def main():
    rank, world, port = int(sys.argv[1]), int(sys.argv[2]), sys.argv[3]
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=port, NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    import fp8_ops
    import nvfp4_ops
    import rwkvq_dist as D
    from oracle import rwkvq_oracle as O

    n, k = 16384, 4096
    g = torch.Generator().manual_seed(0)                      # the same weights and activations on every rank
    w = torch.randn(n, k, generator=g) * k ** -0.5
    q, s = O.q_fp8(w)
    infos = {
        "fp8": {"weight": q.to(dev), "tensor_scale": s.to(dev), "qtype": "fp8"},
        "int8": dict(zip(("weight", "tensor_scale"), (t.to(dev) for t in O.q_int8_sym(w.half()))), qtype="int8"),
        "nvfp4": {kk: (v.to(dev) if torch.is_tensor(v) else v) for kk, v in nvfp4_ops.quantize_to_nvfp4(w.to(dev)).items()},
    }
    verdict = []
    for scheme, info in infos.items():
        lin = fp8_ops.linear_quantized_fused if scheme != "nvfp4" else fp8_ops.linear_quantized
        modes = ("nccl", "peer", "push")                          # push: the GEMM stores its tiles into the peers itself
        if scheme == "nvfp4":
            modes += ("auto",)                                    # push or peer by rank count and rows
        splits = {mode: D.ColumnSplitLinear(info, lin, gather=mode, max_rows=256) for mode in modes}
        for m in (1, 256):
            x = (torch.randn(m, k, generator=g)).to(torch.bfloat16).to(dev)
            full = lin(x, info)
            parts = torch.cat([lin(x, D.slice_weight_info(info, r, world)) for r in range(world)], dim=-1)
            for mode, split in splits.items():
                y = split(x)
                torch.cuda.synchronize()
                if mode != "nccl":
                    split.peer.check()
                ok = y.shape == full.shape and torch.equal(y, parts) and rel_err(y, full) <= 1e-2
                if scheme == "int8":
                    ok = ok and torch.equal(y, full)
                verdict.append(f"{scheme}.m{m}.{mode}={ok}")
                y2 = split(x)                                    # a second call: the other peer buffer, the next epoch
                torch.cuda.synchronize()
                verdict[-1] += f"/{torch.equal(y2, parts)}"
        for split in splits.values():
            if split.peer is not None:
                split.peer.close()
    dist.barrier()
    print(f"rank {rank} " + " ".join(verdict), flush=True)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
