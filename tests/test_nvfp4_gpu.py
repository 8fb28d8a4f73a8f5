"""NVFP4 (W4A4) on the GPU against the CPU restatement of the format described in the reference's reports
(parity unpinned: the reference holds no NVFP4 code).  Activation codes, block scales and the tensor scale are
compared bit for bit (IEEE arithmetic on both sides); projections within max-rel-err 1e-2, an element's error
measured against max(|ref|, 0.02*rms(ref)) -- every product is exact in the kernel, only the summation order differs."""
import pytest
import torch

from oracle import rwkvq_oracle as O

pytestmark = pytest.mark.gpu


def gen(seed, shape, std=1.0, dtype=torch.float32):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(shape, generator=g) * std).to(dtype)


def rel_err(out, ref):
    out, ref = out.detach().cpu().float(), ref.detach().cpu().float()
    floor = 0.02 * ref.pow(2).mean().sqrt().item() + 1e-30
    return ((out - ref).abs() / ref.abs().clamp(min=floor)).max().item()


@pytest.fixture(scope="module")
def nf():
    import rwkvq_abi as abi
    abi.require_device()
    import nvfp4_ops
    return nvfp4_ops


def dev(info):
    return {k: (v.cuda() if torch.is_tensor(v) else v) for k, v in info.items()}


@pytest.mark.parametrize("dt", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("m,k", [(1, 4096), (7, 768), (256, 4096), (3, 16384)])
def test_activation_quantization_bit_exact(nf, dt, m, k):
    x = gen(m + k, (m, k), 1.0).to(dt)
    if m > 2:
        x[1].zero_()
    codes, bs, pts = nf.quantize_activations_nvfp4(x.cuda())
    want_codes, want_bs, want_pts = O.nvfp4_actq(x)
    assert torch.equal(codes.cpu(), want_codes)
    assert torch.equal(bs.cpu().view(torch.uint8), want_bs)
    assert torch.equal(pts.cpu(), want_pts)


def test_weight_quantizer_matches_oracle_and_runs_on_device(nf):
    w = gen(5, (96, 512), 1.0 / 16)
    a, b = nf.quantize_to_nvfp4(w), O.nvfp4_quantize_weight(w)
    assert torch.equal(a["weight"], b["weight"]) and torch.equal(a["block_scale"].view(torch.uint8), b["block_scale"])
    g = nf.quantize_to_nvfp4(w.cuda())
    assert torch.equal(g["weight"].cpu(), a["weight"]) and torch.equal(g["block_scale"].cpu().view(torch.uint8), b["block_scale"])
    z = nf.to_state("k", a)
    assert nf.is_nvfp4_weight(z, "k")
    info = nf.load_nvfp4_weight(z, "k", "cuda")
    assert info["qtype"] == "nvfp4" and "k.nf4_b_scale" not in z


@pytest.mark.parametrize("m", [1, 5, 16, 40])
@pytest.mark.parametrize("n,k", [(1000, 768), (512, 4096), (136, 16384)])
def test_linear_nvfp4(nf, m, n, k):
    w = gen(n + k, (n, k), (1.0 / k) ** 0.5)
    info = nf.quantize_to_nvfp4(w)
    x = gen(m, (m, k), 1.0, torch.bfloat16)
    out = nf.linear_nvfp4(x.cuda(), dev(info))
    oinfo = {"weight": info["weight"], "block_scale": info["block_scale"].view(torch.uint8), "tensor_scale": info["tensor_scale"]}
    want = O.linear_nvfp4(x, oinfo)
    assert out.shape == want.shape and out.dtype == torch.float16
    assert rel_err(out, want) <= 1e-2


def test_config5_ffn_shapes(nf):
    """NVFP4 at the 7.2B FFN shapes: key [16384,4096] and value [4096,16384], M in {1, 256}; M = 4096 on a slice of rows."""
    import fp8_ops
    for n, k in ((16384, 4096), (4096, 16384)):
        w = gen(n, (n, k), (1.0 / k) ** 0.5)
        info = nf.quantize_to_nvfp4(w.cuda())
        cpu = {"weight": info["weight"].cpu(), "block_scale": info["block_scale"].cpu().view(torch.uint8),
               "tensor_scale": info["tensor_scale"].cpu()}
        for m in (1, 256):
            x = gen(m + n, (m, k), 1.0, torch.bfloat16)
            out = fp8_ops.linear_quantized(x.cuda(), info)            # routed by qtype "nvfp4"
            cols = slice(0, 640)                                      # the oracle checks 640 of the output columns
            sub = {"weight": cpu["weight"][cols], "block_scale": cpu["block_scale"][cols], "tensor_scale": cpu["tensor_scale"]}
            assert rel_err(out[:, cols], O.linear_nvfp4(x, sub)) <= 1e-2
    w = gen(9, (256, 4096), 1.0 / 64)
    info = nf.quantize_to_nvfp4(w)
    x = gen(10, (4096, 4096), 1.0, torch.bfloat16)
    oinfo = {"weight": info["weight"], "block_scale": info["block_scale"].view(torch.uint8), "tensor_scale": info["tensor_scale"]}
    assert rel_err(nf.linear_nvfp4(x.cuda(), dev(info)), O.linear_nvfp4(x, oinfo)) <= 1e-2


def test_pack_scales_blocked_order(nf):
    """Blocked scale order: 512-byte chunks per (128-row tile, 64 k), byte (r%32)*16 + (r/32)*4 + (k/16)%4; row tiles
    padded to a multiple of 256 rows with zeros."""
    import numpy as np
    rows, k = 300, 512
    g = torch.Generator().manual_seed(3)
    sf = torch.randint(0, 256, (rows, k // 16), generator=g, dtype=torch.uint8)
    got = nf.pack_scales(sf.cuda(), k).cpu().numpy()
    tiles, k64 = ((rows + 255) // 256) * 2, k // 64
    want = np.zeros((tiles, k64, 512), dtype=np.uint8)
    src = sf.numpy()
    for r in range(rows):
        for b in range(k // 16):
            want[r // 128, b // 4, (r % 32) * 16 + ((r % 128) // 32) * 4 + b % 4] = src[r, b]
    assert got.shape[0] == want.size and (got == want.reshape(-1)).all()


@pytest.mark.parametrize("bn", ["128", "256"])
@pytest.mark.parametrize("m,n,k", [(17, 128, 256), (130, 520, 1024), (300, 384, 2048), (128, 2048, 4096), (513, 1000, 768)])
def test_tensor_core_route(nf, monkeypatch, bn, m, n, k):
    """The tcgen05 block-scaled GEMM (both tile widths) against the oracle and against the GEMV route; ragged M and N."""
    import rwkvq_abi as abi
    monkeypatch.setenv("RWKVQ_NF4_BN", bn)
    w = gen(n * 3 + k, (n, k), (1.0 / k) ** 0.5)
    info = dev(nf.quantize_to_nvfp4(w))
    x = gen(m + 11, (m, k), 1.0, torch.bfloat16)
    x[m // 2].zero_()
    monkeypatch.setenv("RWKVQ_NVFP4_ROUTE", "tc")
    out = nf.linear_nvfp4(x.cuda(), info)
    torch.cuda.synchronize()
    assert abi.workspace_status(abi.workspace(1, 1, 1, 1, out.device)) == 0
    monkeypatch.setenv("RWKVQ_NVFP4_ROUTE", "gemv")
    via_gemv = nf.linear_nvfp4(x.cuda(), info)
    assert rel_err(out, via_gemv) <= 2e-3
    oinfo = {"weight": info["weight"].cpu(), "block_scale": info["block_scale"].cpu().view(torch.uint8),
             "tensor_scale": info["tensor_scale"].cpu()}
    assert rel_err(out, O.linear_nvfp4(x, oinfo)) <= 1e-2


@pytest.mark.parametrize("dt", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("m,n,k", [(1, 4096, 4096), (3, 520, 1024), (8, 136, 512), (9, 1000, 2048), (16, 256, 4096), (2, 264, 16384)])
def test_fused_decode_route(nf, monkeypatch, dt, m, n, k):
    """One-launch decode GEMV (activation quantization in its prologue) against the oracle and against the
    quantize-then-GEMV route."""
    w = gen(n + k + 1, (n, k), (1.0 / k) ** 0.5)
    info = dev(nf.quantize_to_nvfp4(w))
    x = gen(m * 7 + 1, (m, k), 1.0).to(dt)
    if m > 2:
        x[1].zero_()
    monkeypatch.setenv("RWKVQ_NVFP4_ROUTE", "auto")
    monkeypatch.setattr(nf, "TC_MIN_M", 16)            # the kernel takes up to 16 rows; the dispatcher hands over to the GEMM earlier
    monkeypatch.setattr(nf, "TC_LONG_K", 1 << 30)      # ... and so it does for long rows and wide matrices
    monkeypatch.setattr(nf, "TC_WIDE_N", 1 << 30)
    assert nf._route(m, k, n) == "fused"
    out = nf.linear_nvfp4(x.cuda(), info)
    monkeypatch.setenv("RWKVQ_NVFP4_ROUTE", "gemv")
    via_gemv = nf.linear_nvfp4(x.cuda(), info)
    assert rel_err(out, via_gemv) <= 2e-3
    oinfo = {"weight": info["weight"].cpu(), "block_scale": info["block_scale"].cpu().view(torch.uint8),
             "tensor_scale": info["tensor_scale"].cpu()}
    assert rel_err(out, O.linear_nvfp4(x, oinfo)) <= 1e-2


def test_few_tokens_take_the_tensor_core_route_where_it_is_faster(nf, monkeypatch):
    """Dispatcher: long rows (K >= 8192) at every token count, wide matrices (N >= 8192) from 3 tokens on; the rest of
    the few-token calls stay on the one-launch GEMV."""
    monkeypatch.setenv("RWKVQ_NVFP4_ROUTE", "auto")
    assert nf._route(1, 16384, 4096) == "tc" and nf._route(4, 16384, 4096) == "tc"
    assert nf._route(1, 4096, 16384) == "fused" and nf._route(2, 4096, 16384) == "fused"
    assert nf._route(3, 4096, 16384) == "tc" and nf._route(8, 4096, 16384) == "tc"
    assert nf._route(1, 4096, 4096) == "fused" and nf._route(8, 4096, 4096) == "fused" and nf._route(9, 4096, 4096) == "tc"
    w = gen(77, (256, 16384), 1.0 / 128)
    info = dev(nf.quantize_to_nvfp4(w))
    for m in (1, 2, 5):
        x = gen(78 + m, (m, 16384), 1.0, torch.bfloat16)
        out = nf.linear_nvfp4(x.cuda(), info)
        oinfo = {"weight": info["weight"].cpu(), "block_scale": info["block_scale"].cpu().view(torch.uint8),
                 "tensor_scale": info["tensor_scale"].cpu()}
        assert rel_err(out, O.linear_nvfp4(x, oinfo)) <= 1e-2


@pytest.mark.parametrize("dt", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("m,n,k", [(1, 256, 16384), (2, 136, 16384), (4, 384, 16384), (3, 16384, 4096), (4, 4096, 8192), (1, 130, 2048)])
def test_one_launch_cluster_kernel_equals_quantizer_plus_gemm(nf, monkeypatch, dt, m, n, k):
    """One to four tokens against long rows or many weight rows: the activation quantization runs INSIDE the cluster
    split-K kernel (one launch).  Same bits as the quantizer launch followed by the cluster GEMM; within 1e-2 of the
    oracle; a zero row and a second call in a row."""
    import rwkvq_abi as abi
    w = gen(n * 5 + k, (n, k), (1.0 / k) ** 0.5)
    info = dev(nf.quantize_to_nvfp4(w))
    x = gen(m + 17, (m, k), 1.0).to(dt)
    if m > 1:
        x[m - 1].zero_()
    monkeypatch.setenv("RWKVQ_NVFP4_ROUTE", "auto")
    monkeypatch.setattr(nf, "TC_LONG_K", 0)                      # every size of this test takes the tensor-core route
    monkeypatch.setattr(nf, "ONE_LAUNCH", True)                  # opt-in form
    assert abi.lib().rwkvq_tc_gemv_nvfp4_fused_route(m, n, k) == 1
    out = nf.linear_nvfp4(x.cuda(), info)                        # the first call also packs the weight scales (cached)
    before = abi.launch_count()
    again = nf.linear_nvfp4(x.cuda(), info)
    assert abi.launch_count() - before == 1
    torch.cuda.synchronize()
    assert abi.device_status() == 0
    assert torch.equal(out, again)
    monkeypatch.setenv("RWKVQ_TCSN", "0")                        # quantizer launch + cluster GEMM
    assert abi.lib().rwkvq_tc_gemv_nvfp4_fused_route(m, n, k) == 0
    two = nf.linear_nvfp4(x.cuda(), info)
    assert torch.equal(out, two)
    oinfo = {"weight": info["weight"].cpu(), "block_scale": info["block_scale"].cpu().view(torch.uint8),
             "tensor_scale": info["tensor_scale"].cpu()}
    assert rel_err(out, O.linear_nvfp4(x, oinfo)) <= 1e-2


@pytest.mark.parametrize("m,n,k", [(16, 256, 4096), (9, 136, 16384), (64, 384, 8192), (200, 256, 16384), (256, 130, 16384), (33, 512, 2048)])
def test_cluster_splitk_route(nf, monkeypatch, m, n, k):
    """Few tokens against a long K: the weights become the 128-row operand and K is split across a thread-block cluster
    (partial sums through distributed shared memory).  Against the oracle, and against the tiled GEMM on the same codes."""
    import rwkvq_abi as abi
    w = gen(n * 7 + k, (n, k), (1.0 / k) ** 0.5)
    info = dev(nf.quantize_to_nvfp4(w))
    x = gen(m + 13, (m, k), 1.0, torch.bfloat16)
    x[m // 2].zero_()
    monkeypatch.setenv("RWKVQ_NVFP4_ROUTE", "tc")
    assert abi.lib().rwkvq_tc_gemm_nvfp4_cluster_route(m, n, k) == 1
    out = nf.linear_nvfp4(x.cuda(), info)
    again = nf.linear_nvfp4(x.cuda(), info)
    torch.cuda.synchronize()
    assert abi.workspace_status(abi.workspace(1, 1, 1, 1, out.device)) == 0
    assert torch.equal(out, again)                                      # rank-ordered sums: run-to-run identical
    monkeypatch.setenv("RWKVQ_TCS_NF4_MIN_C", "99")                     # the tiled form
    assert abi.lib().rwkvq_tc_gemm_nvfp4_cluster_route(m, n, k) == 0
    tiled = nf.linear_nvfp4(x.cuda(), info)
    assert rel_err(out, tiled) <= 2e-3
    oinfo = {"weight": info["weight"].cpu(), "block_scale": info["block_scale"].cpu().view(torch.uint8),
             "tensor_scale": info["tensor_scale"].cpu()}
    assert rel_err(out, O.linear_nvfp4(x, oinfo)) <= 1e-2


@pytest.mark.parametrize("form", ["auto", "two", "coop"])
@pytest.mark.parametrize("m,k", [(1, 512), (130, 1024), (300, 4096), (16, 16384), (5, 4096), (64, 4096), (3, 16448)])
def test_fused_activation_quantizer_routes_agree(nf, monkeypatch, m, k, form):
    """Fused quantizer -- one cluster launch up to 65536 vectors, two chained launches up to 2^19, one cooperative
    launch above ("two" and "coop" force the later forms with limits of 0) -- against the three-kernel route (codes,
    scales, tensor scale bit for bit), and its blocked scales against pack_scales of the row-major ones on every valid
    row.  The two-launch form leaves its scratch words zero."""
    import numpy as np
    import rwkvq_abi as abi
    monkeypatch.setenv("RWKVQ_NVFP4_ACTQ_SMALL_MAX", "16384" if form == "auto" else "0")      # "auto": the cluster kernel up to its own limit
    if form == "coop":
        monkeypatch.setenv("RWKVQ_NVFP4_ACTQ_TWO_MAX", "0")
    x = gen(m * 5 + k, (m, k), 1.0, torch.bfloat16).cuda()
    monkeypatch.setenv("RWKVQ_NVFP4_ACTQ", "split")
    c0, s0, p0 = nf.quantize_activations_nvfp4(x)
    monkeypatch.setenv("RWKVQ_NVFP4_ACTQ", "fused")
    c1, s1, p1 = nf.quantize_activations_nvfp4(x)
    assert torch.equal(c0, c1) and torch.equal(s0.view(torch.uint8), s1.view(torch.uint8)) and torch.equal(p0, p1)
    c2, blk, p2 = nf.quantize_activations_nvfp4(x, blocked=True)
    assert torch.equal(c0, c2) and torch.equal(p0, p2)
    got = blk.cpu().numpy().reshape(-1, k // 64, 512)
    src = s0.view(torch.uint8).cpu().numpy()
    r = np.arange(m)[:, None]
    b = np.arange(k // 16)[None, :]
    assert (got[r // 128, b // 4, (r % 32) * 16 + ((r % 128) // 32) * 4 + b % 4] == src).all()
    assert int(abi.actq_scratch(x.device)[1024 + 4:1024 + 8].abs().sum().item()) == 0
