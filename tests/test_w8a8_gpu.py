"""GPU parity of the W8A8 path (activation preparation, FP8 and INT8 projections) against the CPU oracle and
the golden vectors the reference produced.  Everything is called through the drop-in modules, i.e. through
the C ABI.

Bars: codes, scales, amax, bf16 copies and INT8 accumulators / outputs bit-exact; FP8 outputs within
max-rel-err 1e-2 of the oracle, the error of an element being measured against max(|ref|, 0.02*rms(ref)).
Division: the library divides the handful of fp32 scales either IEEE or with div.full.f32 (what the reference's
Triton kernels execute on a GPU).  IEEE mode is compared with the oracle as is; div.full mode is compared with the
oracle evaluating exactly those divisions on the device (rwkvq_div_f32), everything else on the CPU.
"""
import os

import numpy as np
import pytest
import torch

from oracle import rwkvq_oracle as O

pytestmark = pytest.mark.gpu
G = os.path.join(os.path.dirname(__file__), "golden")


def gen(seed, shape, std=1.0, dtype=torch.float32):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(shape, generator=g) * std).to(dtype)


@pytest.fixture(scope="module")
def mods():
    import rwkvq_abi as abi
    import fused_fp8_gemm as f
    import fp8_ops
    abi.require_device()
    return abi, f, fp8_ops


@pytest.fixture(params=["ieee", "full"])
def div(request, mods):
    """Sets the library's division mode and returns the matching division for the oracle."""
    abi = mods[0]
    old = abi.DEFAULT_DIV
    if request.param == "ieee":
        abi.DEFAULT_DIV = abi.DIV_IEEE
        yield O.ieee_div
    else:
        abi.DEFAULT_DIV = abi.DIV_FULL

        def dev_div(a, b):
            a = torch.as_tensor(a, dtype=torch.float32)
            b = torch.broadcast_to(torch.as_tensor(b, dtype=torch.float32), a.shape)
            return abi.div_on_device(a, b, abi.DIV_FULL).cpu()
        yield dev_div
    abi.DEFAULT_DIV = old


def bits_equal(a: torch.Tensor, b: torch.Tensor):
    a, b = a.detach().cpu().contiguous(), b.detach().cpu().contiguous()
    assert a.shape == b.shape and a.dtype == b.dtype, (a.shape, b.shape, a.dtype, b.dtype)
    size = a.element_size()
    view = {1: torch.uint8, 2: torch.int16, 4: torch.int32}[size]
    ne = (a.view(view) != b.view(view))
    assert not ne.any(), f"{int(ne.sum())} of {a.numel()} elements differ"


def rel_err(out: torch.Tensor, ref: torch.Tensor) -> float:
    out, ref = out.detach().cpu().float(), ref.detach().cpu().float()
    floor = 0.02 * ref.pow(2).mean().sqrt().item() + 1e-30
    return ((out - ref).abs() / ref.abs().clamp(min=floor)).max().item()


def outliers(x: torch.Tensor) -> torch.Tensor:
    """0.1 % of the channels scaled by 20, the activation distribution of the 2.9B r/k/v case."""
    k = x.shape[-1]
    n = max(1, -(-k // 1000))
    idx = torch.arange(n) * (k // n) + 7
    x = x.clone()
    x[..., idx] *= 20
    return x


# ------------------------------------------------------------------ activation preparation
@pytest.mark.parametrize("dt", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("m,k", [(1, 768), (16, 2560), (33, 4096), (3, 200), (2, 16384), (5, 40000)])
def test_prep_x(mods, div, dt, m, k):
    _, f, _ = mods
    x = outliers(gen(m * 131 + k, (m, k), 1.0)).to(dt)
    awq = gen(9, (k,), 0.2).abs() + 0.5
    for a in (None, awq):
        out, amax = f.prep_x(x.cuda(), None if a is None else a.cuda())
        want, want_amax = O.prep_x(x, a, div)
        bits_equal(out, want)
        bits_equal(amax, want_amax)


def test_prep_x_zero_and_leading_dims(mods):
    _, f, _ = mods
    x = torch.zeros(2, 3, 64, dtype=torch.float16)
    out, amax = f.prep_x(x.cuda())
    assert out.shape == (6, 64) and amax.item() == 0.0 and not out.float().any()


def test_prep3_x(mods, div):
    _, f, _ = mods
    xs = [gen(40 + i, (7, 768), 1.0, torch.float16) for i in range(3)]
    awq = gen(9, (768,), 0.2).abs() + 0.5
    got = f.prep3_x(*[t.cuda() for t in xs], awq.cuda(), None)
    want = O.prep3_x(*xs, awq, None, div)
    for g, w in zip(got, want):
        bits_equal(g, w)


def test_prep_noncontiguous_input(mods):
    """A strided view must give the result of its contiguous copy (the reference once produced NaN here)."""
    _, f, _ = mods
    base = gen(3, (8, 2, 768), 1.0, torch.float16).cuda()
    view = base[:, 1, :]
    a, amax_a = f.prep_x(view)
    b, amax_b = f.prep_x(view.contiguous())
    bits_equal(a, b)
    bits_equal(amax_a, amax_b)
    c, s = f.prep_x_int8(view)
    c2, s2 = f.prep_x_int8(view.contiguous())
    bits_equal(c, c2)
    bits_equal(s, s2)


@pytest.mark.parametrize("dt", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("m,k", [(1, 768), (32, 2560), (600, 4096), (3, 200), (2048, 4096)])
def test_prep_x_fp8(mods, dt, m, k):
    _, f, _ = mods
    x = outliers(gen(m + k, (m, k), 1.0)).to(dt)
    codes, scale = f.prep_x_fp8(x.cuda())
    want_codes, want_scale = O.prep_x_fp8(x)
    assert codes.dtype == torch.float8_e4m3fn
    bits_equal(codes, want_codes)
    bits_equal(scale, want_scale)


@pytest.mark.parametrize("dt", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("m,k", [(1, 768), (16, 3072), (32, 2560), (2048, 4096), (3, 200), (4, 16384)])
def test_prep_x_int8(mods, div, dt, m, k):
    _, f, _ = mods
    x = gen(m * 7 + k, (m, k), 1.0).to(dt)
    if m > 2:
        x[1].zero_()                      # amax floor 1e-12
    codes, scale = f.prep_x_int8(x.cuda())
    want_codes, want_scale = O.prep_x_int8(x, div)
    bits_equal(codes, want_codes)
    bits_equal(scale, want_scale)


# ------------------------------------------------------------------ golden vectors from the reference (IEEE division)
def _from_bits(a, dt):
    return torch.from_numpy(a.view(np.int16).copy()).view(dt)


@pytest.mark.parametrize("tag,dt", [("m1", torch.float16), ("m16", torch.float16), ("m5bf", torch.bfloat16)])
def test_golden_int8_reference_kernels(mods, tag, dt):
    abi, f, _ = mods
    T = dict(np.load(os.path.join(G, "int8_triton.npz")))
    old, abi.DEFAULT_DIV = abi.DEFAULT_DIV, abi.DIV_IEEE
    try:
        xs = [_from_bits(T[f"{tag}.x{i}"], dt).cuda() for i in range(3)]
        infos = [{"weight": torch.from_numpy(T[f"w{i}.q"]).cuda(), "tensor_scale": torch.from_numpy(T[f"w{i}.s"]).cuda(),
                  "qtype": "int8"} for i in range(3)]
        codes, scale = f.prep_x_int8(xs[0])
        bits_equal(codes, torch.from_numpy(T[f"{tag}.codes"]))
        bits_equal(scale, torch.from_numpy(T[f"{tag}.scale"]))
        bits_equal(f.linear_int8_fused(xs[0], infos[0]), _from_bits(T[f"{tag}.lin"], torch.float16))
        r, k, v = f.linear_rkv_int8_fused(xs[0], xs[1], xs[2], *infos)
        for got, nm in ((r, "r"), (k, "k"), (v, "v")):
            bits_equal(got, _from_bits(T[f"{tag}.{nm}"], torch.float16))
        _, amax = f.prep_x(xs[0])
        bits_equal(amax, torch.from_numpy(T[f"{tag}.prep.amax"]))
        o = f.prep3_x(xs[0], xs[1], xs[2], torch.from_numpy(T["awq"]).cuda(), None)
        bits_equal(torch.cat(o[3:]), torch.from_numpy(T[f"{tag}.prep3.amax"]))
        if dt == torch.bfloat16:
            bits_equal(o[2], _from_bits(T[f"{tag}.prep3.ov"], torch.bfloat16))
    finally:
        abi.DEFAULT_DIV = old


# ------------------------------------------------------------------ INT8 projections
def int8_weight(seed, n, k):
    w = gen(seed, (n, k), 0.02, torch.float16)
    q, s = O.q_int8_sym(w)
    return {"weight": q, "tensor_scale": s, "qtype": "int8"}


def to_dev(info):
    return {k: (v.cuda() if torch.is_tensor(v) else v) for k, v in info.items()}


@pytest.mark.parametrize("m", [1, 5, 16, 17, 32, 40, 600])
@pytest.mark.parametrize("n,k", [(768, 768), (3072, 768), (100, 3072), (768, 3072)])
def test_int8_linear_exact(mods, div, m, n, k):
    _, f, _ = mods
    info = int8_weight(n + k, n, k)
    x = gen(m * 3 + n, (m, k), 1.0, torch.float16)
    acc = torch.empty((m, n), dtype=torch.int32, device="cuda")
    out = f.linear_int8_fused(x.cuda(), to_dev(info), acc_out=acc)
    want, want_acc = O.linear_int8_fused(x, info, div, return_acc=True)
    bits_equal(acc, want_acc)
    bits_equal(out, want)


@pytest.mark.parametrize("m", [1, 16, 32, 48])
def test_int8_rkv(mods, div, m):
    _, f, _ = mods
    infos = [int8_weight(60 + i, 768, 768) for i in range(3)]
    xs = [gen(70 + i + m, (m, 768), 1.0, torch.bfloat16) for i in range(3)]
    d = [to_dev(i) for i in infos]
    for shared in (True, False):
        got = f.linear_rkv_int8_fused(*[t.cuda() for t in xs], *d, compat_shared_scale=shared)
        want = O.linear_rkv_int8_fused(*xs, *infos, div=div, shared_scale=shared)
        for g, w in zip(got, want):
            bits_equal(g, w)
    # the fused launch equals three single calls when every matrix keeps its own scale
    got = f.linear_rkv_int8_fused(*[t.cuda() for t in xs], *d, compat_shared_scale=False)
    for g, x, i in zip(got, xs, d):
        bits_equal(g, f.linear_int8_fused(x.cuda(), i))


def test_int8_leading_dims_and_dtype(mods):
    _, f, fp8_ops = mods
    info = int8_weight(5, 96, 768)
    x = gen(6, (2, 3, 768), 1.0, torch.float16)
    out = fp8_ops.linear_quantized(x.cuda(), to_dev(info), torch.float32)
    assert out.shape == (2, 3, 96) and out.dtype == torch.float32
    bits_equal(out.half(), O.linear_int8_fused(x, info, _lib_div(mods)))


def _lib_div(mods):
    abi = mods[0]
    if abi.DEFAULT_DIV == abi.DIV_IEEE:
        return O.ieee_div
    return lambda a, b: abi.div_on_device(torch.as_tensor(a, dtype=torch.float32),
                                          torch.broadcast_to(torch.as_tensor(b, dtype=torch.float32),
                                                             torch.as_tensor(a).shape), abi.DIV_FULL).cpu()


# ------------------------------------------------------------------ FP8 projections
def fp8_weight(seed, n, k):
    w = gen(seed, (n, k), (1.0 / k) ** 0.5)
    q, s = O.q_fp8(w)
    return {"weight": q, "tensor_scale": s, "qtype": "fp8"}


@pytest.mark.parametrize("dt", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("m", [1, 2, 8, 16, 32, 33, 600])
@pytest.mark.parametrize("n,k", [(2560, 2560), (104, 768), (512, 16384)])
def test_fp8_linear_fused(mods, m, n, k, dt):
    _, f, _ = mods
    info = fp8_weight(n * 3 + k, n, k)
    x = outliers(gen(m + n + k, (m, k), 1.0)).to(dt)
    out = f.linear_fp8_fused(x.cuda(), to_dev(info))
    want = O.linear_fp8_fused(x, info, _lib_div(mods))
    assert out.shape == want.shape and out.dtype == torch.float16
    assert rel_err(out, want) <= 1e-2


@pytest.mark.parametrize("scheme", ["fp8", "int8"])
@pytest.mark.parametrize("m", [9, 15, 16, 31])
def test_decode_width_4096_many_rows(mods, scheme, m):
    """K = 4096 with as many rows as the fused GEMV takes by itself: the activation tile is at its largest here
    (shared-memory sizing of the ring beside it)."""
    _, f, _ = mods
    n, k = 520, 4096
    x = outliers(gen(m + 5, (m, k), 1.0)).to(torch.bfloat16)
    if scheme == "fp8":
        info = fp8_weight(3, n, k)
        assert rel_err(f.linear_fp8_fused(x.cuda(), to_dev(info)), O.linear_fp8_fused(x, info, _lib_div(mods))) <= 1e-2
    else:
        info = int8_weight(4, n, k)
        bits_equal(f.linear_int8_fused(x.cuda(), to_dev(info)), O.linear_int8_fused(x, info, _lib_div(mods)))


@pytest.mark.parametrize("m", [1, 8, 32, 64])
def test_fp8_rkv_config2(mods, m):
    """The 2.9B r/k/v case: three [2560,2560] e4m3 matrices, bf16 activations with outlier channels."""
    _, f, _ = mods
    infos = [fp8_weight(80 + i, 2560, 2560) for i in range(3)]
    xs = [outliers(gen(90 + i + m, (m, 2560), 1.0)).to(torch.bfloat16) for i in range(3)]
    d = [to_dev(i) for i in infos]
    got = f.linear_rkv_fused(*[t.cuda() for t in xs], *d)
    want = O.linear_rkv_fused(*xs, *infos, div=_lib_div(mods))
    for g, w in zip(got, want):
        assert rel_err(g, w) <= 1e-2
    # the reference reports the fused launch bit-identical to separate calls
    for g, x, i in zip(got, xs, d):
        if m > 1:
            bits_equal(g, f.linear_fp8_fused(x.cuda(), i))


def test_fp8_rkv_with_awq(mods):
    _, f, _ = mods
    infos = [fp8_weight(100 + i, 256, 768) for i in range(3)]
    awq = gen(9, (768,), 0.2).abs() + 0.5
    infos[0]["awq_scale"] = awq
    xs = [gen(110 + i, (4, 768), 1.0, torch.float16) for i in range(3)]
    got = f.linear_rkv_fused(*[t.cuda() for t in xs], *[to_dev(i) for i in infos])
    want = O.linear_rkv_fused(*xs, *infos, div=_lib_div(mods))
    for g, w in zip(got, want):
        assert rel_err(g, w) <= 1e-2


@pytest.mark.parametrize("m", [513, 2048])
def test_fp8_large_m_route(mods, m):
    """linear_fp8 (M > 512): bf16 first, IEEE scales, result through bf16."""
    _, f, fp8_ops = mods
    info = fp8_weight(7, 768, 768)
    x = gen(m, (m, 768), 1.0, torch.float16)
    out = fp8_ops.linear_quantized_fused(x.cuda(), to_dev(info))
    want = O.linear_fp8(x, info)
    assert rel_err(out, want) <= 1e-2


# ------------------------------------------------------------------ argument checking through the raw C ABI
def test_status_codes(mods):
    abi, _, _ = mods
    L = abi.lib()
    x = torch.zeros(2, 64, dtype=torch.float16, device="cuda")
    w = torch.zeros(8, 64, dtype=torch.uint8, device="cuda")
    s = torch.ones(1, device="cuda")
    o = torch.zeros(2, 8, dtype=torch.float16, device="cuda")
    st = abi.stream_ptr()
    ok = L.rwkvq_gemv_fp8(x.data_ptr(), 0, None, w.data_ptr(), 64, s.data_ptr(), o.data_ptr(), 8, 2, 8, 64, 64, 1, 0, st)
    assert ok == 0
    assert L.rwkvq_gemv_fp8(None, 0, None, w.data_ptr(), 64, s.data_ptr(), o.data_ptr(), 8, 2, 8, 64, 64, 1, 0, st) == -1
    assert L.rwkvq_gemv_fp8(x.data_ptr(), 0, None, w.data_ptr(), 64, s.data_ptr(), o.data_ptr(), 8, 2, 8, 40, 64, 1, 0, st) == -3
    assert L.rwkvq_gemv_fp8(x.data_ptr(), 0, None, w.data_ptr(), 64, s.data_ptr(), o.data_ptr(), 8, 33, 8, 64, 64, 1, 0, st) == -3
    assert L.rwkvq_gemv_fp8(x.data_ptr() + 2, 0, None, w.data_ptr(), 64, s.data_ptr(), o.data_ptr(), 8, 2, 8, 64, 64, 1, 0, st) == -2
    assert L.rwkvq_gemv_fp8(x.data_ptr(), 7, None, w.data_ptr(), 64, s.data_ptr(), o.data_ptr(), 8, 2, 8, 64, 64, 1, 0, st) == -1
    assert b"x_dtype" in L.rwkvq_last_error_string()
    assert L.rwkvq_prep_x_int8(x.data_ptr(), 0, 2, 64, 32, w.data_ptr(), 64, s.data_ptr(), 1, st) == -3
    torch.cuda.synchronize()
