"""The CPU oracle against golden vectors produced by the reference itself
(tests/golden/make_golden.py).  Everything here is bit-exact."""
import os

import numpy as np
import pytest
import torch

from oracle import rwkvq_oracle as O

G = os.path.join(os.path.dirname(__file__), "golden")


def gen(seed, shape, std=1.0, dtype=torch.float32):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(shape, generator=g) * std).to(dtype)


def bits(t):
    t = t.detach().contiguous()
    if t.dtype in (torch.bfloat16, torch.float16):
        return t.view(torch.int16).numpy().view(np.uint16)
    if t.dtype == torch.float8_e4m3fn:
        return t.view(torch.uint8).numpy()
    return t.numpy()


def from_bits(a, dtype):
    return torch.from_numpy(a.view(np.int16).copy()).view(dtype)


@pytest.fixture(scope="module")
def W():
    return dict(np.load(os.path.join(G, "weights.npz")))


@pytest.fixture(scope="module")
def T():
    return dict(np.load(os.path.join(G, "int8_triton.npz")))


def eq(a, b):
    a, b = np.asarray(a), np.asarray(b)
    assert a.shape == b.shape and a.dtype == b.dtype, (a.shape, b.shape, a.dtype, b.dtype)
    if a.dtype.kind == "f":
        a, b = a.view(np.uint32), b.view(np.uint32)
    assert np.array_equal(a, b), f"{np.count_nonzero(a != b)} of {a.size} differ"


def test_inputs_are_regenerated_identically(W):
    eq(gen(0, (48, 256), 0.02).numpy(), W["w"])


def test_schemes_quantizers(W):
    w = torch.from_numpy(W["w"])
    for name, fn in (("_q_fp8", O.q_fp8), ("_q_fp8_perchannel", O.q_fp8_perchannel), ("_q_int8_sym", O.q_int8_sym)):
        q, s = fn(w)
        eq(bits(q), W[name + ".q"])
        eq(s.numpy(), W[name + ".s"])
    q, s = O.q_int8_sym(w.to(torch.float16))
    eq(bits(q), W["_q_int8_sym.fp16in.q"])
    eq(s.numpy(), W["_q_int8_sym.fp16in.s"])
    eq(O.q_int8_affine(w).numpy(), W["_q_int8_affine"])
    eq(O.q_int4_sym(w).numpy(), W["_q_int4_sym"])
    eq(O.q_int4_gw(w, 128).numpy(), W["_q_int4_gw.128"])
    eq(O.q_int4_gw(torch.from_numpy(W["w_odd"]), 128).numpy(), W["_q_int4_gw.128.padded"])


def test_int4_int8_tools(W):
    w = torch.from_numpy(W["w"])
    p, s = O.quantize_to_int4_per_tensor(w)
    eq(p.numpy(), W["q4pt.packed"]); eq(s.numpy(), W["q4pt.scale"])
    a = O.quantize_to_int4_affine(w)
    for k in ("packed", "mx", "rx", "my", "ry"):
        eq(a[k].numpy(), W["q4af." + k])
    g = O.quantize_to_int4_groupwise(w, 128)
    for k in ("packed", "scales", "zeros"):
        eq(g[k].numpy(), W["q4gw." + k])
    q, s = O.quantize_to_int8_per_tensor(w)
    eq(q.numpy(), W["q8pt.q"]); eq(s.numpy(), W["q8pt.s"])
    a8 = O.quantize_to_int8_affine(w)
    for k in ("w_u8", "mx", "rx", "my", "ry"):
        eq(a8[k].numpy(), W["q8af." + k])
    eq(O.unpack_int4(g["packed"]).numpy(), W["unpack_int4"])


def test_reference_cpu_dequant_matmul(W):
    w = torch.from_numpy(W["w"])
    x = from_bits(W["x"], torch.float16)
    p, s = O.quantize_to_int4_per_tensor(w)
    eq(bits(O.linear_ref_fp16_dequant(x, O.dequant_int4_per_tensor({"packed": p, "scale": s}))), W["lin4pt"])
    eq(bits(O.linear_ref_fp16_dequant(x, O.dequant_int4_affine(O.quantize_to_int4_affine(w)))), W["lin4af"])
    eq(bits(O.linear_ref_fp16_dequant(x, O.dequant_int4_groupwise(O.quantize_to_int4_groupwise(w)))), W["lin4gw"])
    a8 = O.quantize_to_int8_affine(w)
    a8["weight"] = a8["w_u8"]
    eq(bits(O.linear_ref_fp16_dequant(x, O.dequant_int8_affine(a8))), W["lin8af"])
    # int8 per-tensor: the reference multiplies in fp16 (int8_ops.py:72), so dequantize that way here
    q, s = O.quantize_to_int8_per_tensor(w)
    w16 = q.to(torch.float16) * s.to(torch.float16)
    eq(bits((x @ w16.t())), W["lin8pt"])


@pytest.mark.parametrize("tag,dt", [("m1", torch.float16), ("m16", torch.float16), ("m5bf", torch.bfloat16)])
def test_int8_triton_kernels_and_prep(T, tag, dt):
    xs = [from_bits(T[f"{tag}.x{i}"], dt) for i in range(3)]
    infos = [{"weight": torch.from_numpy(T[f"w{i}.q"]), "tensor_scale": torch.from_numpy(T[f"w{i}.s"])} for i in range(3)]
    codes, scale = O.prep_x_int8(xs[0])
    eq(codes.numpy(), T[f"{tag}.codes"])
    eq(scale.numpy(), T[f"{tag}.scale"])
    eq(bits(O.linear_int8_fused(xs[0], infos[0])), T[f"{tag}.lin"])
    r, k, v = O.linear_rkv_int8_fused(xs[0], xs[1], xs[2], *infos, shared_scale=True)
    eq(bits(r), T[f"{tag}.r"]); eq(bits(k), T[f"{tag}.k"]); eq(bits(v), T[f"{tag}.v"])
    xb, amax = O.prep_x(xs[0])
    eq(amax.numpy(), T[f"{tag}.prep.amax"])
    o = O.prep3_x(xs[0], xs[1], xs[2], torch.from_numpy(T["awq"]), None)
    if dt == torch.bfloat16:      # the interpreter truncates fp32->bf16; only exact copies are golden
        eq(bits(xb), T[f"{tag}.prep.bf16"])
        eq(bits(o[2]), T[f"{tag}.prep3.ov"])
    eq(torch.cat(o[3:]).numpy(), T[f"{tag}.prep3.amax"])


def test_numpy_e4m3_matches_torch_cast():
    v = torch.cat([torch.linspace(-460, 460, 200001), gen(5, (100000,), 3.0), gen(6, (100000,), 0.01),
                   torch.tensor([0.0, -0.0, 2.0 ** -10, 1.5 * 2.0 ** -9, 2.0 ** -9])]).clamp(-448, 448)
    want = v.to(torch.float8_e4m3fn).view(torch.uint8).numpy()
    got = O.e4m3_encode(v.numpy())
    nz = v.numpy() != 0          # torch keeps the sign of -0 as well; compare it too
    assert np.array_equal(got[nz], want[nz])
    assert np.array_equal(got & 0x7F, want & 0x7F)
    back = O.e4m3_decode(np.arange(256, dtype=np.uint8))
    ref = torch.arange(256, dtype=torch.uint8).view(torch.float8_e4m3fn).float().numpy()
    assert np.array_equal(np.nan_to_num(back, nan=7e7), np.nan_to_num(ref, nan=7e7))


def test_e2m1_grid_and_ties():
    x = np.array([0.0, 0.2, 0.25, 0.3, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0, 5.1, 7.0, -0.75, -6.5, -0.25], np.float32)
    want = np.array([0.0, 0.0, 0.0, 0.5, 1.0, 1.0, 2.0, 2.0, 4.0, 4.0, 6.0, 6.0, -1.0, -6.0, -0.0], np.float32)
    assert np.array_equal(O.e2m1_decode(O.e2m1_encode(x)), want)


def test_nvfp4_self_consistency():
    w = gen(7, (64, 256), 1.0 / 16)
    info = O.nvfp4_quantize_weight(w)
    deq = O.nvfp4_dequant(info["weight"], info["block_scale"]) * info["tensor_scale"]
    rel = ((deq - w).norm() / w.norm()).item()
    assert 0.04 < rel < 0.13          # the reference reports ~8.8 % weight error for NVFP4
    x = gen(8, (4, 256), 1.0, torch.bfloat16)
    out = O.linear_nvfp4(x, info).float()
    ref = x.float() @ w.t()
    assert ((out - ref).norm() / ref.norm()).item() < 0.2
