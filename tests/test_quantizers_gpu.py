"""The offline weight quantizers run ON THE DEVICE (the same functions given CUDA tensors) against the golden vectors the
reference produced on the CPU (tests/golden/weights.npz): codes, scales and round-trip weights bit for bit, so a model
can be quantized on the GPU it will run on and still load with the reference's layouts."""
import os

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu
G = os.path.join(os.path.dirname(__file__), "golden")


def bits(t):
    t = t.detach().contiguous().cpu()
    if t.dtype in (torch.bfloat16, torch.float16):
        return t.view(torch.int16).numpy().view(np.uint16)
    if t.dtype == torch.float8_e4m3fn:
        return t.view(torch.uint8).numpy()
    return t.numpy()


def eq(a, b, what=""):
    a, b = np.asarray(a), np.asarray(b)
    assert a.shape == b.shape and a.dtype == b.dtype, (what, a.shape, b.shape, a.dtype, b.dtype)
    if a.dtype.kind == "f":
        a, b = a.view(np.uint32), b.view(np.uint32)
    assert np.array_equal(a, b), f"{what}: {np.count_nonzero(a != b)} of {a.size} differ"


@pytest.fixture(scope="module")
def W():
    return dict(np.load(os.path.join(G, "weights.npz")))


def test_scheme_quantizers_on_device(W):
    import schemes
    w = torch.from_numpy(W["w"]).cuda()
    for name in ("_q_fp8", "_q_fp8_perchannel", "_q_int8_sym"):
        q, s = getattr(schemes, name)(w)
        assert q.is_cuda and s.is_cuda
        eq(bits(q), W[name + ".q"], name)
        eq(bits(s), W[name + ".s"], name + " scale")
    eq(bits(schemes._q_int8_affine(w)), W["_q_int8_affine"], "_q_int8_affine")
    eq(bits(schemes._q_int4_sym(w)), W["_q_int4_sym"], "_q_int4_sym")
    eq(bits(schemes._q_int4_gw(w, group_size=128)), W["_q_int4_gw.128"], "_q_int4_gw")
    eq(bits(schemes._q_int4_gw(torch.from_numpy(W["w_odd"]).cuda(), group_size=128)), W["_q_int4_gw.128.padded"], "_q_int4_gw padded")


def test_int4_int8_tool_quantizers_on_device(W):
    from int4 import quantize_int4 as q4
    from int8 import quantize_int8 as q8
    w = torch.from_numpy(W["w"]).cuda()
    p, s = q4.quantize_to_int4_per_tensor(w)
    eq(bits(p), W["q4pt.packed"]); eq(bits(s), W["q4pt.scale"])
    a = q4.quantize_to_int4_affine(w)
    for k in ("packed", "mx", "rx", "my", "ry"):
        eq(bits(a[k]), W["q4af." + k], "int4 affine " + k)
    g = q4.quantize_to_int4_groupwise(w, 128)
    for k in ("packed", "scales", "zeros"):
        eq(bits(g[k]), W["q4gw." + k], "int4 groupwise " + k)
    q, s = q8.quantize_to_int8_per_tensor(w)
    eq(bits(q), W["q8pt.q"]); eq(bits(s), W["q8pt.s"])
    a8 = q8.quantize_to_int8_affine(w)
    for k in ("w_u8", "mx", "rx", "my", "ry"):
        eq(bits(a8[k]), W["q8af." + k], "int8 affine " + k)
