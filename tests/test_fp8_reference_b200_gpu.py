"""GPU parity against what the REFERENCE's own kernels computed on a B200.

tests/golden/fp8_triton_b200.npz holds the outputs of the unmodified reference (Triton kernels of fused_fp8_gemm.py and
torch._scaled_mm through fp8_ops.linear_fp8) on the seeded inputs of tests/golden/fp8_b200_cases.py, recorded by
tests/golden/make_golden_b200.py.  Here the same inputs go through librwkvq (C ABI, default division mode div.full,
which is what Triton emits for `/` on a GPU).

Bars: activation codes, scales, amax, bf16 copies, INT8 codes / scales / outputs and the projections through an identity
matrix (which expose the FP8 codes and the result scale) bit-exact; FP8 projection outputs within max-rel-err 1e-2,
an element's error measured against max(|ref|, 0.02*rms(ref)).
"""
import os
import sys

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu
G = os.path.join(os.path.dirname(__file__), "golden")
sys.path.insert(0, G)
import fp8_b200_cases as cases  # noqa: E402

NPZ = os.path.join(G, "fp8_triton_b200.npz")


@pytest.fixture(scope="module")
def T():
    assert os.path.exists(NPZ), "tests/golden/fp8_triton_b200.npz is missing (make_golden_b200.py writes it)"
    return dict(np.load(NPZ))


@pytest.fixture(scope="module")
def mods():
    import rwkvq_abi as abi
    import fused_fp8_gemm as f
    import fp8_ops
    abi.require_device()
    assert abi.DEFAULT_DIV == abi.DIV_FULL
    return abi, f, fp8_ops


def want(T, tag, dt, inputs):
    got = [cases.checksum(i) for i in inputs]
    assert got == list(T[tag + ".insum"]), f"{tag}: the regenerated inputs differ from the ones the reference was run on"
    a = T[tag]
    if dt in (torch.float16, torch.bfloat16):
        return torch.from_numpy(a.view(np.int16).copy()).view(dt)
    if dt == torch.float8_e4m3fn:
        return torch.from_numpy(a.copy()).view(dt)
    return torch.from_numpy(a.copy())


def bits_equal(a, b, what=""):
    a, b = a.detach().cpu().contiguous(), b.detach().cpu().contiguous()
    assert a.shape == b.shape and a.dtype == b.dtype, (what, a.shape, b.shape, a.dtype, b.dtype)
    view = {1: torch.uint8, 2: torch.int16, 4: torch.int32}[a.element_size()]
    ne = a.view(view) != b.view(view)
    assert not ne.any(), f"{what}: {int(ne.sum())} of {a.numel()} elements differ"


def rel_err(out, ref):
    out, ref = out.detach().cpu().float(), ref.detach().cpu().float()
    floor = 0.02 * ref.pow(2).mean().sqrt().item() + 1e-30
    return ((out - ref).abs() / ref.abs().clamp(min=floor)).max().item()


def dev(info):
    return {k: (v.cuda() if torch.is_tensor(v) else v) for k, v in info.items()}


@pytest.mark.parametrize("route", ["auto", "mma"])
@pytest.mark.parametrize("case", cases.SINGLE, ids=[c[0] for c in cases.SINGLE])
def test_linear_fp8_fused_vs_reference(T, mods, case, route, monkeypatch):
    _, f, _ = mods
    tag, k, n, m, dt, outl = case
    monkeypatch.setattr(f, "ROUTE", route)
    s = cases.seed_of(tag)
    info, x = cases.q_fp8_weight(s, n, k), cases.act(s + 1, m, k, dt, outl)
    ref = want(T, tag, torch.float16, [info["weight"], x])
    out = f.linear_fp8_fused(x.cuda(), dev(info))
    assert out.shape == ref.shape
    assert rel_err(out, ref) <= 1e-2


@pytest.mark.parametrize("case", cases.RKV, ids=[c[0] for c in cases.RKV])
def test_linear_rkv_fused_vs_reference(T, mods, case):
    _, f, _ = mods
    tag, k, n, m, dt, outl, awq = case
    s = cases.seed_of(tag)
    infos = [cases.q_fp8_weight(s + i, n, k) for i in range(3)]
    xs = [cases.act(s + 10 + i, m, k, dt, outl) for i in range(3)]
    d = [dev(i) for i in infos]
    if awq:
        d[0]["awq_scale"] = cases.awq_vec(k).cuda()
        d[1]["awq_scale"] = (cases.awq_vec(k) * 1.25).cuda()
    got = f.linear_rkv_fused(*[x.cuda() for x in xs], *d)
    ins = [i["weight"] for i in infos] + xs
    for g, nm in zip(got, "rkv"):
        assert rel_err(g, want(T, f"{tag}.{nm}", torch.float16, ins)) <= 1e-2, nm


@pytest.mark.parametrize("case", cases.SCALED_MM, ids=[c[0] for c in cases.SCALED_MM])
def test_linear_fp8_scaled_mm_vs_reference(T, mods, case):
    _, _, fp8_ops = mods
    tag, k, n, m, dt, outl = case
    s = cases.seed_of(tag)
    info, x = cases.q_fp8_weight(s, n, k), cases.act(s + 1, m, k, dt, outl)
    ref = want(T, tag, torch.float16, [info["weight"], x])
    out = fp8_ops.linear_fp8(x.cuda(), dev(info))
    assert out.dtype == torch.float16 and rel_err(out, ref) <= 1e-2


@pytest.mark.parametrize("route", ["auto", "mma"])
@pytest.mark.parametrize("case", cases.IDENTITY, ids=[c[0] for c in cases.IDENTITY])
def test_identity_projection_exposes_codes(T, mods, case, route, monkeypatch):
    """out = fp16(code * (amax/448 * 1)): one product per element, so equal codes and an equal scale give equal bits."""
    _, f, _ = mods
    tag, k, m, dt = case
    monkeypatch.setattr(f, "ROUTE", route)
    x = cases.act(cases.seed_of(tag), m, k, dt, True)
    out = f.linear_fp8_fused(x.cuda(), dev(cases.identity_weight(k)))
    bits_equal(out, want(T, tag, torch.float16, [x]), tag)


@pytest.mark.parametrize("case", cases.PREP_FP8, ids=[c[0] for c in cases.PREP_FP8])
def test_prep_x_fp8_vs_reference(T, mods, case):
    _, f, _ = mods
    tag, m, k, dt = case
    x = cases.act(cases.seed_of(tag), m, k, dt, True)
    codes, scale = f.prep_x_fp8(x.cuda())
    if m > 64:
        codes = torch.cat([codes[:4], codes[-4:]])
    bits_equal(codes, want(T, tag + ".codes", torch.float8_e4m3fn, [x]), "codes")
    bits_equal(scale, want(T, tag + ".scale", torch.float32, [x]), "scale")


@pytest.mark.parametrize("case", cases.PREP_X, ids=[c[0] for c in cases.PREP_X])
def test_prep_x_awq_vs_reference(T, mods, case):
    """bf16 copies after the AWQ division and the amax: the division is div.full.f32 in the reference's kernel."""
    _, f, _ = mods
    tag, m, k, dt = case
    s = cases.seed_of(tag)
    xs = [cases.act(s + i, m, k, dt, True) for i in range(3)]
    awq = cases.awq_vec(k)
    o, amax = f.prep_x(xs[0].cuda(), awq.cuda())
    bits_equal(o, want(T, tag + ".awq.bf16", torch.bfloat16, xs[:1]), "awq bf16")
    bits_equal(amax, want(T, tag + ".awq.amax", torch.float32, xs[:1]), "awq amax")
    o, amax = f.prep_x(xs[0].cuda())
    bits_equal(o, want(T, tag + ".bf16", torch.bfloat16, xs[:1]), "bf16")
    bits_equal(amax, want(T, tag + ".amax", torch.float32, xs[:1]), "amax")
    p3 = f.prep3_x(*[x.cuda() for x in xs], awq.cuda(), (awq * 1.25).cuda())
    for name, t in zip(("or", "ok", "ov", "ar", "ak", "av"), p3):
        bits_equal(t, want(T, f"{tag}.p3.{name}", torch.bfloat16 if name[0] == "o" else torch.float32, xs), name)


@pytest.mark.parametrize("case", cases.PREP_INT8, ids=[c[0] for c in cases.PREP_INT8])
def test_prep_x_int8_vs_reference(T, mods, case):
    _, f, _ = mods
    tag, m, k, dt = case
    x = cases.act(cases.seed_of(tag), m, k, dt, True)
    codes, scale = f.prep_x_int8(x.cuda())
    bits_equal(codes, want(T, tag + ".codes", torch.int8, [x]), "codes")
    bits_equal(scale, want(T, tag + ".scale", torch.float32, [x]), "scale")


@pytest.mark.parametrize("case", cases.INT8_LIN, ids=[c[0] for c in cases.INT8_LIN])
def test_linear_int8_fused_vs_reference(T, mods, case):
    _, f, _ = mods
    tag, k, n, m, dt = case
    s = cases.seed_of(tag)
    info, x = cases.q_int8_weight(s, n, k), cases.act(s + 1, m, k, dt, False)
    bits_equal(f.linear_int8_fused(x.cuda(), dev(info)), want(T, tag, torch.float16, [info["weight"], x]), tag)
