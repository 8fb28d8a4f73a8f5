"""GPU tests of the pieces around the kernels' waits: CUDA-graph replay of the one-launch activation quantizers (their
grid rendezvous must not depend on anything fixed at capture time), a bounded wait that is seen to run out and to
report RWKVQ_E_TIMEOUT without disturbing the context, the one-launch r/k/v GEMM route, and per-row weight scales.
Everything goes through the C ABI (ctypes)."""
import ctypes

import pytest
import torch

from oracle import rwkvq_oracle as O

pytestmark = pytest.mark.gpu


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


def bits_equal(a, b, what=""):
    a, b = a.detach().cpu().contiguous(), b.detach().cpu().contiguous()
    assert a.shape == b.shape and a.dtype == b.dtype, (what, a.shape, b.shape)
    view = {1: torch.uint8, 2: torch.int16, 4: torch.int32}[a.element_size()]
    ne = a.view(view) != b.view(view)
    assert not ne.any(), f"{what}: {int(ne.sum())} of {a.numel()} elements differ"


def rel_err(out, ref):
    out, ref = out.detach().cpu().float(), ref.detach().cpu().float()
    floor = 0.02 * ref.pow(2).mean().sqrt().item() + 1e-30
    return ((out - ref).abs() / ref.abs().clamp(min=floor)).max().item()


def fp8_weight(seed, n, k, perchannel=False):
    w = gen(seed, (n, k), (1.0 / k) ** 0.5)
    if perchannel:
        w = w * (0.25 + torch.arange(n).float().remainder(7).reshape(-1, 1))     # rows of very different magnitude
        q, s = O.q_fp8_perchannel(w)
    else:
        q, s = O.q_fp8(w)
    return {"weight": q, "tensor_scale": s, "qtype": "fp8"}


def dev(info):
    return {k: (v.cuda() if torch.is_tensor(v) else v) for k, v in info.items()}


def lib_div(abi):
    return lambda a, b: abi.div_on_device(torch.as_tensor(a, dtype=torch.float32),
                                          torch.broadcast_to(torch.as_tensor(b, dtype=torch.float32), torch.as_tensor(a).shape),
                                          abi.DEFAULT_DIV).cpu()


# ------------------------------------------------------------------------------------------------ graph replay
def test_captured_projection_replays_with_new_activations(mods):
    """ONE linear_fp8_fused call at M = 64 (activation-quantization launch + tensor-core GEMM) captured in a graph and
    replayed with different inputs -- a large amax first, then small ones -- equals the eager result bit for bit."""
    abi, f, _ = mods
    info = dev(fp8_weight(1, 256, 1024))
    xs = [gen(10 + i, (64, 1024), s).to(torch.bfloat16).cuda() for i, s in enumerate((50.0, 0.01, 1.0, 3.0))]
    eager = [f.linear_fp8_fused(x, info).clone() for x in xs]
    static_x = xs[0].clone()
    st = torch.cuda.Stream()
    with torch.cuda.stream(st):
        f.linear_fp8_fused(static_x, info)              # warm-up on the capture stream (allocates its scratch)
        st.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=st):
            out = f.linear_fp8_fused(static_x, info)
        for x, want in zip(xs, eager):
            static_x.copy_(x)
            g.replay()
            st.synchronize()
            bits_equal(out, want, "replay")


@pytest.mark.parametrize("form", ["auto", "two", "coop"])
@pytest.mark.parametrize("which", ["fp8", "nvfp4"])
def test_captured_quantizer_with_own_scratch_replays(mods, monkeypatch, which, form):
    """The raw fused quantizer with caller-owned scratch, captured alone and replayed with new inputs, in each of its
    forms: the cluster launch this size takes by default, the two chained launches (their scratch words must be zero
    again for every replay) and the cooperative launch (every replay must rendezvous afresh: nothing about the
    rendezvous is fixed at capture time)."""
    abi, f, _ = mods
    if form != "auto":
        monkeypatch.setenv("RWKVQ_ACTQ_SMALL_MAX", "0")
        monkeypatch.setenv("RWKVQ_NVFP4_ACTQ_SMALL_MAX", "0")
    if form == "coop":
        monkeypatch.setenv("RWKVQ_ACTQ_TWO_MAX", "0")
        monkeypatch.setenv("RWKVQ_NVFP4_ACTQ_TWO_MAX", "0")
    L = abi.lib()
    m, k = 96, 2048
    xs = [gen(20 + i, (m, k), s).to(torch.bfloat16).cuda() for i, s in enumerate((40.0, 0.02, 2.0))]
    x = xs[0].clone()
    amax = torch.zeros(1, device="cuda")
    if which == "fp8":
        codes = torch.empty((m, k), dtype=torch.uint8, device="cuda")
        scratch = torch.zeros(int(L.rwkvq_actq_fp8_fused_scratch_bytes()) // 4, dtype=torch.int32, device="cuda")

        def launch(stream):
            abi.call("rwkvq_actq_fp8_fused", x.data_ptr(), abi.BF16, m, k, k, codes.data_ptr(), k, amax.data_ptr(), None,
                     scratch.data_ptr(), scratch.numel() * 4, None, abi.DIV_FULL, 0, stream)
        results = lambda: (codes.clone(), amax.clone())
    else:
        codes = torch.empty((m, k // 2), dtype=torch.uint8, device="cuda")
        bs = torch.empty((m, k // 16), dtype=torch.uint8, device="cuda")
        scratch = torch.zeros(int(L.rwkvq_actq_nvfp4_fused_scratch_bytes()) // 4, dtype=torch.int32, device="cuda")

        def launch(stream):
            abi.call("rwkvq_actq_nvfp4_fused", x.data_ptr(), abi.BF16, m, k, k, codes.data_ptr(), k // 2, bs.data_ptr(), k // 16,
                     None, amax.data_ptr(), scratch.data_ptr(), scratch.numel() * 4, None, stream)
        results = lambda: (codes.clone(), bs.clone(), amax.clone())
    eager = []
    for xi in xs:
        x.copy_(xi)
        launch(abi.stream_ptr())
        torch.cuda.synchronize()
        eager.append(results())
    st = torch.cuda.Stream()
    with torch.cuda.stream(st):
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=st):
            launch(st.cuda_stream)
        for xi, want in zip(xs + xs[::-1], eager + eager[::-1]):
            x.copy_(xi)
            g.replay()
            st.synchronize()
            for got, w in zip(results(), want):
                bits_equal(got, w, which)


# ------------------------------------------------------------------------------------------------ bounded waits
@pytest.mark.parametrize("mode", [0, 1])
def test_bounded_wait_runs_out_and_reports(mods, mode):
    """A wait for something that never comes gives up after its limit, records RWKVQ_E_TIMEOUT and the kernel returns
    normally: the context stays usable (a projection right after it is correct)."""
    abi, f, _ = mods
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    word = torch.zeros(1, dtype=torch.int32, device="cuda")
    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0.record()
    abi.call("rwkvq_selftest_timeout", status.data_ptr(), word.data_ptr(), 200, mode, abi.stream_ptr())
    t1.record()
    torch.cuda.synchronize()
    assert status.item() == abi.E_TIMEOUT
    assert 0.15 <= t0.elapsed_time(t1) < 500.0, t0.elapsed_time(t1)       # waited at least the limit, not seconds
    info = fp8_weight(3, 128, 512)
    x = gen(4, (3, 512), 1.0, torch.bfloat16)
    assert rel_err(f.linear_fp8_fused(x.cuda(), dev(info)), O.linear_fp8_fused(x, info, lib_div(abi))) <= 1e-2


def test_peer_wait_gives_up_when_a_rank_never_signals(mods):
    """Receiver side of a pushed / pulled all-gather with a rank that never delivers: the flag wait runs out after the
    wait limit, the status word reads RWKVQ_E_TIMEOUT, the kernel returns and the context stays usable.  (The failure
    is made on the host: a flag array that nothing writes; no GPU fault is involved.)"""
    abi, f, _ = mods
    L = abi.lib()
    flags = torch.zeros(64, dtype=torch.int32, device="cuda")
    flags[0] = 7                                                          # this rank's own slot is never looked at
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    L.rwkvq_set_wait_limit_us(200_000)
    try:
        t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0.record()
        abi.call("rwkvq_peer_wait", flags.data_ptr(), 7, 0, 4, status.data_ptr(), abi.stream_ptr())     # ranks 1-3 stay silent
        t1.record()
        torch.cuda.synchronize()
        assert status.item() == abi.E_TIMEOUT
        assert 150.0 <= t0.elapsed_time(t1) < 5000.0, t0.elapsed_time(t1)
        status.zero_()
        flags[1:4] = 7                                                    # everybody has signalled epoch 7
        abi.call("rwkvq_peer_wait", flags.data_ptr(), 7, 0, 4, status.data_ptr(), abi.stream_ptr())
        torch.cuda.synchronize()
        assert status.item() == 0
    finally:
        L.rwkvq_set_wait_limit_us(0)
    info = fp8_weight(5, 128, 512)
    x = gen(6, (3, 512), 1.0, torch.bfloat16)
    assert rel_err(f.linear_fp8_fused(x.cuda(), dev(info)), O.linear_fp8_fused(x, info, lib_div(abi))) <= 1e-2


def test_device_status_word_reads_and_clears(mods):
    abi, _, _ = mods
    assert abi.device_status() == 0
    abi.check_status()                                                    # nothing pending: no exception
    L = abi.lib()
    assert L.rwkvq_selftest_timeout(None, None, 10, 0, abi.stream_ptr()) == -1
    L.rwkvq_set_wait_limit_us(2_000_000)
    L.rwkvq_set_wait_limit_us(0)                                          # back to the default


# ------------------------------------------------------------------------------------------------ r/k/v GEMM route
@pytest.mark.parametrize("m", [33, 64, 200, 600])
def test_fp8_rkv_gemm_route_equals_single_calls(mods, m):
    """Above the decode kernel's range r, k, v run as one quantization step for the three tensors (one launch, or an
    abs-max and a codes launch for mid-sized blocks) + one GEMM launch; results equal three single projections bit for
    bit and the oracle within 1e-2."""
    abi, f, _ = mods
    infos = [fp8_weight(30 + i, 384, 1024) for i in range(3)]
    xs = [gen(40 + i + m, (m, 1024), 1.0 + i).to(torch.bfloat16) for i in range(3)]
    d = [dev(i) for i in infos]
    before = abi.launch_count()
    got = f.linear_rkv_fused(*[x.cuda() for x in xs], *d)
    assert abi.launch_count() - before in (2, 3)
    want = O.linear_rkv_fused(*xs, *infos, div=lib_div(abi))
    for g, w, x, i in zip(got, want, xs, d):
        assert rel_err(g, w) <= 1e-2
        bits_equal(g, f.linear_fp8_fused(x.cuda(), i), "fused vs single")


@pytest.mark.parametrize("m", [40, 300])
def test_int8_rkv_gemm_route_exact(mods, m):
    abi, f, _ = mods
    infos = []
    for i in range(3):
        q, s = O.q_int8_sym(gen(50 + i, (256, 768), 0.02, torch.float16))
        infos.append({"weight": q, "tensor_scale": s, "qtype": "int8"})
    xs = [gen(60 + i + m, (m, 768), 1.0, torch.float16) for i in range(3)]
    d = [dev(i) for i in infos]
    for shared in (True, False):
        before = abi.launch_count()
        got = f.linear_rkv_int8_fused(*[x.cuda() for x in xs], *d, compat_shared_scale=shared)
        assert abi.launch_count() - before == 2
        want = O.linear_rkv_int8_fused(*xs, *infos, div=lib_div(abi), shared_scale=shared)
        for g, w in zip(got, want):
            bits_equal(g, w, f"int8 rkv shared={shared}")


# ------------------------------------------------------------------------------------------------ per-row weight scales
@pytest.mark.parametrize("m", [1, 8, 32, 48, 300, 600])
def test_fp8_perchannel_weight_scales(mods, m):
    """Weights of the "fp8_perchannel" scheme (one scale per output row): every route applies scale[n] to column n."""
    abi, f, fp8_ops = mods
    info = fp8_weight(70, 200, 768, perchannel=True)
    assert info["tensor_scale"].shape == (200,)
    x = gen(71 + m, (m, 768), 1.0, torch.bfloat16)
    want = O.linear_fp8_fused(x, info, lib_div(abi))
    for route in ("auto", "mma"):
        old, f.ROUTE = f.ROUTE, route
        try:
            assert rel_err(f.linear_fp8_fused(x.cuda(), dev(info)), want) <= 1e-2, route
        finally:
            f.ROUTE = old
    if m > 512:
        assert rel_err(fp8_ops.linear_quantized_fused(x.cuda(), dev(info)), O.linear_fp8(x, info)) <= 1e-2
    infos = [info, fp8_weight(72, 200, 768, perchannel=True), fp8_weight(73, 200, 768, perchannel=True)]
    xs = [x, gen(74, (m, 768), 2.0, torch.bfloat16), gen(75, (m, 768), 0.5, torch.bfloat16)]
    got = f.linear_rkv_fused(*[t.cuda() for t in xs], *[dev(i) for i in infos])
    for g, w in zip(got, O.linear_rkv_fused(*xs, *infos, div=lib_div(abi))):
        assert rel_err(g, w) <= 1e-2


@pytest.mark.parametrize("scheme", ["fp8", "int8"])
@pytest.mark.parametrize("m,n,k", [(9, 2560, 2560), (16, 520, 4096), (32, 2560, 2560), (32, 300, 4096), (12, 192, 8192)])
def test_decode_on_codes_route(mods, scheme, m, n, k):
    """9..32 rows: the activations are quantized once and the weight-streaming kernel copies the codes; two launches
    for a single projection and for r, k, v alike, r/k/v equal to single calls bit for bit."""
    abi, f, _ = mods
    assert f._codes_gemv_fits(m, k)
    xs = [gen(90 + i + m, (m, k), 1.0 + i).to(torch.bfloat16) for i in range(3)]
    if scheme == "fp8":
        infos = [fp8_weight(91 + i, n, k) for i in range(3)]
        d = [dev(i) for i in infos]
        before = abi.launch_count()
        got = f.linear_rkv_fused(*[x.cuda() for x in xs], *d)
        assert abi.launch_count() - before == 2
        for g, w, x, i in zip(got, O.linear_rkv_fused(*xs, *infos, div=lib_div(abi)), xs, d):
            assert rel_err(g, w) <= 1e-2
            before = abi.launch_count()
            single = f.linear_fp8_fused(x.cuda(), i)
            assert abi.launch_count() - before == 2
            bits_equal(g, single, "fused vs single")
    else:
        infos = []
        for i in range(3):
            q, s = O.q_int8_sym(gen(95 + i, (n, k), 0.02, torch.float16))
            infos.append({"weight": q, "tensor_scale": s, "qtype": "int8"})
        d = [dev(i) for i in infos]
        before = abi.launch_count()
        got = f.linear_rkv_int8_fused(*[x.cuda() for x in xs], *d, compat_shared_scale=False)
        assert abi.launch_count() - before == 2
        acc = torch.empty((m, n), dtype=torch.int32, device="cuda")
        for j, (g, w, x, i) in enumerate(zip(got, O.linear_rkv_int8_fused(*xs, *infos, div=lib_div(abi), shared_scale=False), xs, d)):
            bits_equal(g, w, "int8 rkv")
            bits_equal(f.linear_int8_fused(x.cuda(), i, acc_out=acc), w, "int8 single")
            bits_equal(acc, O.linear_int8_fused(x, infos[j], lib_div(abi), return_acc=True)[1], "int8 acc")


def test_quantized_dispatch_routes_int4(mods):
    """linear_quantized / linear_quantized_fused accept the INT4 weight-info dicts of int4_ops.load_int4_weight."""
    _, f, fp8_ops = mods
    from int4 import int4_ops, quantize_int4
    w = gen(80, (256, 512), 512 ** -0.5)
    q = quantize_int4.quantize_to_int4_groupwise(w, 128)
    info = {"packed": q["packed"].cuda(), "scales": q["scales"].cuda(), "zeros": q["zeros"].cuda(), "group_size": 128,
            "qtype": "int4_groupwise"}
    x = gen(81, (4, 512), 1.0, torch.float16).cuda()
    want = int4_ops.linear_int4(x, info)
    bits_equal(fp8_ops.linear_quantized(x, info), want)
    bits_equal(f.linear_quantized_fused(x, info), want)


# ------------------------------------------------------------------------------------------------ decode layer helper
@pytest.mark.parametrize("scheme", ["fp8", "int8"])
@pytest.mark.parametrize("rows,dt", [(1, torch.bfloat16), (1, torch.float16), (4, torch.bfloat16)])
def test_decode_layer_equals_dropin_calls(mods, scheme, rows, dt):
    """DecodeLayer (descriptors bound once, one boundary crossing) against the drop-in calls: same kernels, same bits."""
    abi, f, _ = mods
    from rwkvq_layer import DecodeLayer
    c, ff = 512, 1024
    shapes = [(c, c)] * 4 + [(ff, c), (c, ff)]
    infos = []
    for i, (n, k) in enumerate(shapes):
        if scheme == "fp8":
            infos.append(dev(fp8_weight(120 + i, n, k)))
        else:
            q, s = O.q_int8_sym(gen(130 + i, (n, k), 0.02, torch.float16))
            infos.append({"weight": q.cuda(), "tensor_scale": s.cuda(), "qtype": "int8"})
    xs = [gen(140 + i, (rows, k), 1.0).to(dt).cuda() for i, k in enumerate((c, c, c, c, c, ff))]
    layer = DecodeLayer(*infos, rows=rows, x_dtype=dt)
    before = abi.launch_count()
    got = [t.clone() for t in layer.all(*xs)]
    assert abi.launch_count() - before == 4
    if scheme == "fp8":
        want = list(f.linear_rkv_fused(xs[0], xs[1], xs[2], *infos[:3]))
    else:
        want = list(f.linear_rkv_int8_fused(xs[0], xs[1], xs[2], *infos[:3]))
    want += [f.linear_quantized_fused(x, i) for x, i in zip(xs[3:], infos[3:])]
    for g, w in zip(got, want):
        bits_equal(g, w.reshape(g.shape), "layer vs drop-in")
    per_op = [*layer.rkv(*xs[:3]), layer.att_out(xs[3]), layer.ffn_key(xs[4]), layer.ffn_value(xs[5])]
    for g, w in zip(per_op, want):
        bits_equal(g, w.reshape(g.shape), "per projection")
    graph, outs = layer.capture(*xs)
    for t in xs:
        t.mul_(0.5)
    graph.replay()
    torch.cuda.synchronize()
    want2 = list(f.linear_rkv_fused(*xs[:3], *infos[:3]) if scheme == "fp8" else f.linear_rkv_int8_fused(*xs[:3], *infos[:3]))
    want2 += [f.linear_quantized_fused(x, i) for x, i in zip(xs[3:], infos[3:])]
    for g, w in zip(outs, want2):
        bits_equal(g, w.reshape(g.shape), "graph replay")
    with pytest.raises(ValueError):
        layer.att_out(xs[3][:, :-16])


# ------------------------------------------------------------------------------------------------ FFN pair with relu^2 folded in
@pytest.mark.parametrize("m,dt", [(1, torch.bfloat16), (1, torch.float16), (3, torch.bfloat16), (8, torch.float16), (20, torch.bfloat16),
                                  (40, torch.bfloat16), (300, torch.float16), (600, torch.bfloat16)])
def test_ffn_relu2_pair_equals_three_step_chain(mods, m, dt):
    """key -> relu_square -> value: the fused pair (relu^2 in the key epilogue, published amax) equals the three steps
    run separately bit for bit, and the oracle's chain within 1e-2.  Twice in a row: the scratch is left clean."""
    abi, f, _ = mods
    c, ff = 768, 3072
    key, val = fp8_weight(150, ff, c), fp8_weight(151, c, ff)
    dk, dv = dev(key), dev(val)
    for rep in range(2):
        x = gen(152 + m + rep, (m, c), 1.0 + rep).to(dt)
        before = abi.launch_count()
        out, hid = f.ffn_relu2_fp8(x.cuda(), dk, dv, return_hidden=True)
        launches = abi.launch_count() - before
        y = f.linear_quantized_fused(x.cuda(), dk)
        h = (y.float().clamp(min=0) ** 2).half()
        bits_equal(hid, h, "hidden")
        bits_equal(out, f.linear_quantized_fused(h, dv), "ffn output")
        if m <= 512:
            want, want_h = O.ffn_relu2_fp8(x, key, val, lib_div(abi))
        else:
            want_h = O.relu_square(O.linear_fp8(x, key))
            want = O.linear_fp8(want_h, val)
        assert rel_err(hid, want_h) <= 2e-2 and rel_err(out, want) <= 2e-2      # the square doubles the relative error of y
        if m <= 8:
            assert launches == 2
        if m > 32:
            assert launches == 4                # quantize x, key GEMM (+relu^2, amax), quantize hidden (elementwise), value GEMM
        if m <= 8 or m > 32:
            assert int(f.ffn_scratch("cuda").abs().sum().item()) == 0
    if m <= 8:
        from rwkvq_layer import DecodeLayer
        sq = dev(fp8_weight(153, c, c))
        layer = DecodeLayer(sq, sq, sq, sq, dk, dv, rows=m, x_dtype=dt)
        out2, hid2 = layer.ffn(x.cuda())
        bits_equal(out2.reshape(out.shape), out, "DecodeLayer.ffn")


@pytest.mark.parametrize("m,dt", [(1, torch.bfloat16), (2, torch.float16), (3, torch.bfloat16), (5, torch.float16), (8, torch.bfloat16),
                                  (8, torch.float16), (20, torch.bfloat16), (40, torch.bfloat16), (300, torch.float16), (600, torch.bfloat16)])
def test_int8_ffn_relu2_pair_equals_three_step_chain(mods, m, dt):
    """The pair on INT8 weights (per-row maxima published by the key projection): bit-equal to the three steps run
    separately and to the oracle's chain; two launches up to 8 rows, four on the tiled GEMM (quantizer, key GEMM with
    relu_square and row maxima, given-maxima quantizer, value GEMM); the scratch is left clean; rows whose hidden
    activations are all zero (negative key results only) keep the quantizer's floor."""
    abi, f, _ = mods
    c, ff = 768, 3072
    qk, sk = O.q_int8_sym(gen(160, (ff, c), 0.02, torch.float16))
    qv, sv = O.q_int8_sym(gen(161, (c, ff), 0.02, torch.float16))
    key, val = {"weight": qk, "tensor_scale": sk, "qtype": "int8"}, {"weight": qv, "tensor_scale": sv, "qtype": "int8"}
    dk, dv = dev(key), dev(val)
    for rep in range(3):
        x = gen(162 + m + rep, (m, c), 1.0 + rep).to(dt)
        if rep == 2:
            x[m // 2] = 0                                        # a row of zeros: relu^2 of it is zero, its published maximum stays 0
        before = abi.launch_count()
        out, hid = f.ffn_relu2_int8(x.cuda(), dk, dv, return_hidden=True)
        launches = abi.launch_count() - before
        y = f.linear_int8_fused(x.cuda(), dk)
        h = (y.float().clamp(min=0) ** 2).half()
        bits_equal(hid, h, "hidden")
        bits_equal(out, f.linear_int8_fused(h, dv), "ffn output")
        want, want_h = O.ffn_relu2_int8(x, key, val, lib_div(abi))
        bits_equal(hid, want_h, "hidden against the oracle")
        bits_equal(out, want, "ffn output against the oracle")
        if m <= 8:
            assert launches == 2
            assert int(f.ffn_scratch("cuda").abs().sum().item()) == 0
        if m > 32:
            assert launches == 4
            assert float(f._row_max_scratch("cuda", m).abs().sum().item()) == 0.0
    if m <= 8:
        from rwkvq_layer import DecodeLayer
        qs, ss = O.q_int8_sym(gen(163, (c, c), 0.02, torch.float16))
        sq = dev({"weight": qs, "tensor_scale": ss, "qtype": "int8"})
        layer = DecodeLayer(sq, sq, sq, sq, dk, dv, rows=m, x_dtype=dt)
        xg = x.cuda()
        out2, hid2 = layer.ffn(xg)
        bits_equal(out2.reshape(out.shape), out, "DecodeLayer.ffn")
        graph = torch.cuda.CUDAGraph()                          # and under replay: the scratch returns to zero every time
        side = torch.cuda.Stream()
        with torch.cuda.stream(side):
            layer.ffn(xg)
            torch.cuda.synchronize()
            with torch.cuda.graph(graph, stream=side):
                out3, _ = layer.ffn(xg)
        for _ in range(3):
            graph.replay()
        torch.cuda.synchronize()
        bits_equal(out3.reshape(out.shape), out, "DecodeLayer.ffn under graph replay")


# ------------------------------------------------------------------------------------------------ CTA-pair GEMM (tcgen05 cta_group::2)
@pytest.mark.parametrize("scheme", ["fp8", "int8"])
@pytest.mark.parametrize("m,n,k", [(4096, 2560, 256), (4100, 2600, 272)])
def test_cta_pair_gemm_many_tokens(mods, scheme, m, n, k):
    """From 4096 tokens on the codes GEMM runs on CTA pairs (two SMs per 256 x 256 tile): INT8 accumulators and outputs
    exact, FP8 within 1e-2 of the oracle and of the mma.sync kernel."""
    abi, f, _ = mods
    x = gen(200 + m, (m, k), 1.0).to(torch.bfloat16)
    if scheme == "fp8":
        info = fp8_weight(201, n, k)
        out = f.linear_fp8_fused(x.cuda(), dev(info))
        assert rel_err(out, O.linear_fp8_fused(x, info, lib_div(abi))) <= 1e-2
        old, f.ROUTE = f.ROUTE, "mma"                                   # and against the mma.sync kernel on the same codes
        try:
            ref = f.linear_fp8_fused(x.cuda(), dev(info))
        finally:
            f.ROUTE = old
        assert rel_err(out, ref) <= 1e-2
    else:
        q, s = O.q_int8_sym(gen(202, (n, k), 0.02, torch.float16))
        info = {"weight": q, "tensor_scale": s, "qtype": "int8"}
        acc = torch.empty((m, n), dtype=torch.int32, device="cuda")
        out = f.linear_int8_fused(x.cuda(), dev(info), acc_out=acc)
        want, want_acc = O.linear_int8_fused(x, info, lib_div(abi), return_acc=True)
        bits_equal(acc, want_acc, "accumulators")
        bits_equal(out, want, "outputs")


# ------------------------------------------------------------------------------------------------ cluster split-K (few tokens)
@pytest.mark.parametrize("scheme", ["fp8", "int8"])
@pytest.mark.parametrize("m,n,k", [(33, 4096, 4096),      # 32 row tiles, cluster of 8 (attention shapes)
                                   (64, 4096, 4096),
                                   (48, 1000, 1040),      # ragged N and K: zero-filled tile edges; 9 K steps: cluster of 4
                                   (40, 5000, 2048),      # 40 row tiles: cluster of 4
                                   (12, 520, 16384),      # long K that the decode GEMV's code tile cannot hold
                                   (64, 4096, 16384),     # FFN value
                                   (128, 4096, 8192),     # one token tile of 128: cluster of 4, one CTA per SM
                                   (200, 1000, 8320),     # two token tiles (128 + 72), ragged N, 65 K steps
                                   (256, 4096, 16384)])   # FFN value, short prefill chunk: cluster of 2
def test_cluster_splitk_few_tokens(mods, scheme, m, n, k):
    """Up to 256 rows against a matrix with few 128-row tiles: K is split across a thread-block cluster and the partial
    sums travel through distributed shared memory.  INT8 accumulators and outputs exact; FP8 within 1e-2 of the oracle
    and of the mma.sync kernel on the same codes; two calls give the same bits."""
    abi, f, _ = mods
    x = gen(300 + m + n, (m, k), 1.0).to(torch.bfloat16)
    if scheme == "fp8":
        info = fp8_weight(301 + n, n, k, perchannel=(n == 1000))
        d = dev(info)
        out = f.linear_fp8_fused(x.cuda(), d)
        assert rel_err(out, O.linear_fp8_fused(x, info, lib_div(abi))) <= 1e-2
        bits_equal(out, f.linear_fp8_fused(x.cuda(), d), "run to run")
        old, f.ROUTE = f.ROUTE, "mma"
        try:
            ref = f.linear_fp8_fused(x.cuda(), d)
        finally:
            f.ROUTE = old
        assert rel_err(out, ref) <= 1e-2
    else:
        q, s = O.q_int8_sym(gen(302 + n, (n, k), 0.02, torch.float16))
        info = {"weight": q, "tensor_scale": s, "qtype": "int8"}
        acc = torch.empty((m, n), dtype=torch.int32, device="cuda")
        out = f.linear_int8_fused(x.cuda(), dev(info), acc_out=acc)
        want, want_acc = O.linear_int8_fused(x, info, lib_div(abi), return_acc=True)
        bits_equal(acc, want_acc, "accumulators")
        bits_equal(out, want, "outputs")
    assert abi.device_status() == 0


@pytest.mark.parametrize("dt", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("m,n,k", [(9, 4096, 16384), (16, 520, 16384), (32, 1000, 8320), (12, 4096, 4096), (32, 2560, 2560)])
def test_cluster_one_launch_equals_two_launch_route(mods, dt, m, n, k):
    """Up to 32 rows: the cluster split-K kernel with the activation quantization inside (one launch) gives the bits of
    the quantizer kernel followed by the same GEMM on codes, and the oracle's result within 1e-2."""
    abi, f, _ = mods
    assert abi.lib().rwkvq_tc_cluster_gemv_route(m, n, k) == 1
    info = fp8_weight(400 + n, n, k, perchannel=(n == 1000))
    d = dev(info)
    x = gen(401 + m, (m, k), 1.0).to(dt)
    x[m // 2, :64] *= 30.0                                            # the abs-max sits in one CTA's K slice
    w, w_ts = f._u8(d["weight"]), d["tensor_scale"]
    x2 = x.cuda()
    before = abi.launch_count()
    one = f._fp8_cluster_gemv(x2, w, w_ts)
    assert abi.launch_count() - before == 1
    two = f._fp8_codes_gemm(x2, w, w_ts, abi.FLAG_QUANT_FROM_BF16)
    bits_equal(one, two, "one launch vs quantizer + GEMM")
    bits_equal(one, f._fp8_cluster_gemv(x2, w, w_ts), "run to run")
    assert rel_err(one, O.linear_fp8_fused(x, info, lib_div(abi))) <= 1e-2
    assert abi.device_status() == 0


# ------------------------------------------------------------------------------------------------ GEMM + all-gather in one kernel
@pytest.mark.parametrize("scheme", ["fp8", "int8", "nvfp4"])
@pytest.mark.parametrize("m,n,k", [(300, 520, 1024), (96, 16384, 512)])
def test_pushing_epilogue_on_one_gpu(mods, scheme, m, n, k):
    """The GEMMs that carry a column-split projection's all-gather, exercised on ONE GPU: the "peers" are two more
    buffers on the same device.  Every buffer receives this rank's column range bit-equal to the plain GEMM's result, the
    columns of other ranks stay untouched, and both flag slots read the call's epoch; a second call (next epoch) works."""
    import ctypes
    import nvfp4_ops
    abi, f, fp8_ops = mods
    x = gen(500 + m, (m, k), 1.0).to(torch.bfloat16).cuda()
    if scheme == "fp8":
        info = dev(fp8_weight(501, n, k))
    elif scheme == "int8":
        q, s = O.q_int8_sym(gen(502, (n, k), 0.02, torch.float16))
        info = dev({"weight": q, "tensor_scale": s, "qtype": "int8"})
    else:
        info = {kk: (v.cuda() if torch.is_tensor(v) else v) for kk, v in nvfp4_ops.quantize_to_nvfp4(gen(503, (n, k), (1.0 / k) ** 0.5).cuda()).items()}
    assert nvfp4_ops.can_push(m, k) if scheme == "nvfp4" else f.can_push(m, n, k)
    plain = fp8_ops.linear_quantized_fused(x, info)
    n_total, col0 = 3 * n, n                                             # this "rank" owns the middle third of the columns
    bufs = [torch.full((m, n_total), -7.0, dtype=torch.float16, device="cuda") for _ in range(3)]
    flags = torch.zeros(64, dtype=torch.int32, device="cuda")
    arr = ctypes.c_void_p * 2
    peer_out = arr(bufs[1].data_ptr() + col0 * 2, bufs[2].data_ptr() + col0 * 2)
    for epoch in (5, 6):
        peer_flag = arr(flags.data_ptr() + 4 * 1, flags.data_ptr() + 4 * 2)
        with abi.output_into(bufs[0][:, col0:col0 + n]):
            fp8_ops.linear_quantized_fused(x, info, torch.float16, push=(peer_out, peer_flag, 2, epoch))
        torch.cuda.synchronize()
        for b in bufs:
            bits_equal(b[:, col0:col0 + n], plain, f"{scheme} pushed columns")
            assert bool((b[:, :col0] == -7.0).all()) and bool((b[:, col0 + n:] == -7.0).all())
        assert flags[1].item() == epoch and flags[2].item() == epoch and flags[0].item() == 0
    assert abi.device_status() == 0


# ------------------------------------------------------------------------------------------------ results into a column range
@pytest.mark.parametrize("scheme,m,n,k", [("fp8", 16, 256, 4096), ("fp8", 200, 384, 16384), ("int8", 40, 256, 4096),
                                           ("nvfp4", 16, 256, 16384), ("nvfp4", 200, 384, 16384), ("nvfp4", 256, 2048, 4096),
                                           ("nvfp4", 2, 256, 16384)])
def test_cluster_kernels_write_into_a_column_range(mods, monkeypatch, scheme, m, n, k):
    """What a column-split projection does on every rank: the projection writes its [M, N] result into a column range of
    a wider buffer (leading dimension 3 N).  Sizes that run the cluster split-K kernels (and, for two tokens of NVFP4,
    the one-launch form): the range equals the plain call bit for bit and the neighbouring columns stay untouched."""
    import nvfp4_ops
    abi, f, fp8_ops = mods
    x = gen(600 + m, (m, k), 1.0).to(torch.bfloat16).cuda()

    def takes_cluster_kernel(m, n, k):
        # up to 32 rows the one-launch route query covers the same sizes; above 48 rows (no weight-streaming form) a
        # tensor-core call that cannot carry a push is one the cluster kernel takes
        L = abi.lib()
        return L.rwkvq_tc_cluster_gemv_route(m, n, k) == 1 if m <= 32 else (m > 48 or k < 8192) and L.rwkvq_tc_gemm_can_push(m, n, k) == 0
    if scheme == "fp8":
        info = dev(fp8_weight(601, n, k))
        assert takes_cluster_kernel(m, n, k)
    elif scheme == "int8":
        q, s = O.q_int8_sym(gen(602, (n, k), 0.02, torch.float16))
        info = dev({"weight": q, "tensor_scale": s, "qtype": "int8"})
        assert takes_cluster_kernel(m, n, k)
    else:
        info = {kk: (v.cuda() if torch.is_tensor(v) else v) for kk, v in nvfp4_ops.quantize_to_nvfp4(gen(603, (n, k), (1.0 / k) ** 0.5).cuda()).items()}
        assert abi.lib().rwkvq_tc_gemm_nvfp4_cluster_route(m, n, k) == 1
        if m <= 4:
            monkeypatch.setattr(nvfp4_ops, "ONE_LAUNCH", True)
    lin = fp8_ops.linear_quantized if scheme == "nvfp4" else fp8_ops.linear_quantized_fused
    plain = lin(x, info)
    buf = torch.full((m, 3 * n), -7.0, dtype=torch.float16, device="cuda")
    with abi.output_into(buf[:, n:2 * n]):
        lin(x, info)
    torch.cuda.synchronize()
    bits_equal(buf[:, n:2 * n], plain, f"{scheme} column range")
    assert bool((buf[:, :n] == -7.0).all()) and bool((buf[:, 2 * n:] == -7.0).all())
    assert abi.device_status() == 0
