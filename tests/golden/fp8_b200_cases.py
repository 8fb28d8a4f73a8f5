"""Seeded inputs of the golden vectors that the reference's own GPU kernels produced on a B200.

Shared by make_golden_b200.py (which runs the reference and records its outputs in fp8_triton_b200.npz) and by
tests/test_fp8_reference_b200_gpu.py (which rebuilds the same inputs and compares librwkvq with the recorded
outputs).  Inputs are not stored: they are regenerated from the seeds below, and the .npz holds a checksum of each
so that a different random generator is noticed instead of producing a misleading mismatch.
"""
import torch

DT = {"f16": torch.float16, "bf16": torch.bfloat16}


def gen(seed, shape, std=1.0, dtype=torch.float32):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(shape, generator=g) * std).to(dtype)


def outliers(x):
    """0.1 % of the channels scaled by 20: the activation distribution of the FP8 decode configuration."""
    k = x.shape[-1]
    n = max(1, -(-k // 1000))
    idx = torch.arange(n) * (k // n) + 7
    x = x.clone()
    x[..., idx] *= 20
    return x


def checksum(t):
    """Order-sensitive 64-bit checksum of a tensor's bytes."""
    b = t.detach().contiguous().cpu().view(torch.uint8).to(torch.int64)
    w = torch.arange(1, b.numel() + 1, dtype=torch.int64) % 65521
    return int((b.flatten() * w).sum().item())


def q_fp8_weight(seed, n, k):
    """Weights N(0, 1/K) quantized per tensor the way schemes._q_fp8 of the reference does (integer-valued codes)."""
    w = gen(seed, (n, k), (1.0 / k) ** 0.5)
    amax = w.abs().max().clamp(min=1e-12)
    scale = (amax / 448.0).float()
    q = (w / scale).clamp(-448.0, 448.0).round().to(torch.float8_e4m3fn)
    return {"weight": q, "tensor_scale": scale, "qtype": "fp8"}


def identity_weight(k):
    """e4m3 identity with scale 1: a projection through it returns fp16(code * amax/448), i.e. exposes the codes."""
    return {"weight": torch.eye(k).to(torch.float8_e4m3fn), "tensor_scale": torch.tensor(1.0), "qtype": "fp8"}


def q_int8_weight(seed, n, k):
    w = gen(seed, (n, k), 0.02, torch.float16)
    scale = (w.abs().max().float() / 127.0).float()
    q = (w.float() / scale).round().clamp(-128, 127).to(torch.int8)
    return {"weight": q, "tensor_scale": scale, "qtype": "int8"}


def act(seed, m, k, dt, with_outliers):
    x = gen(seed, (m, k), 1.0)
    if with_outliers:
        x = outliers(x)
    return x.to(DT[dt])


def awq_vec(k):
    return gen(99, (k,), 0.2).abs() + 0.5


# (tag, K, N, M, dtype, outliers)
SINGLE = (
    [(f"s768_m{m}_{dt}", 768, 768, m, dt, False) for m in (1, 2, 8, 32, 64) for dt in ("f16", "bf16")]
    + [(f"s2560_m{m}", 2560, 128, m, "bf16", True) for m in (1, 8, 32, 64, 300)]
    + [("s768_m600_bf16", 768, 128, 600, "bf16", True), ("s768_m600_f16", 768, 128, 600, "f16", False)]
)
# r/k/v in one call; AWQ divisors on r and k where `awq`
RKV = (
    [(f"r768_m{m}_{dt}", 768, 768, m, dt, False, True) for m in (1, 5, 16) for dt in ("f16", "bf16")]
    + [(f"r2560_b{m}", 2560, 2560, m, "bf16", True, False) for m in (1, 8, 32)]
    + [(f"r2560_m{m}", 2560, 128, m, "bf16", True, False) for m in (64, 200)]
)
# linear_fp8 (scaled matmul above 512 rows; also legal below)
SCALED_MM = [("mm768_m600_f16", 768, 128, 600, "f16", False), ("mm768_m2048_bf16", 768, 128, 2048, "bf16", True),
             ("mm2560_m520_bf16", 2560, 128, 520, "bf16", True)]
# projection through the identity: the outputs expose the activation codes and the result scale bit for bit
IDENTITY = [(f"id768_m{m}_{dt}", 768, m, dt) for m in (1, 8, 40) for dt in ("f16", "bf16")]
# activation preparation
PREP_FP8 = [(f"pf_{m}x{k}_{dt}", m, k, dt) for (m, k) in ((1, 768), (8, 768), (64, 2560), (600, 768)) for dt in ("f16", "bf16")]
PREP_X = [(f"px_{m}x{k}_{dt}", m, k, dt) for (m, k) in ((8, 768), (9, 2560)) for dt in ("f16", "bf16")]
PREP_INT8 = [(f"pi_{m}x{k}_{dt}", m, k, dt) for (m, k) in ((1, 768), (16, 768), (40, 2560)) for dt in ("f16", "bf16")]
INT8_LIN = [(f"i8_m{m}_{dt}", 768, 96, m, dt) for m in (1, 16, 70) for dt in ("f16", "bf16")]


def seed_of(tag):
    return sum((i + 1) * ord(c) for i, c in enumerate(tag)) % 100000 + 1000
