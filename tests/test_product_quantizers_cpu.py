"""The PRODUCT's offline weight quantizers (schemes.py, int4/quantize_int4.py, int8/quantize_int8.py of the drop-in
package) against the golden vectors the reference produced (tests/golden/weights.npz), bit for bit, and the
reference's own `rwkv-quant q` step run once with its schemes module and once with the drop-in one.
"""
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
PKG = os.path.join(ROOT, "rwkv7-quantization_b200")
G = os.path.join(os.path.dirname(__file__), "golden")


def bits(t):
    t = t.detach().contiguous()
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


def test_scheme_quantizers_bit_exact(W):
    import schemes
    w = torch.from_numpy(W["w"])
    for name in ("_q_fp8", "_q_fp8_perchannel", "_q_int8_sym"):
        q, s = getattr(schemes, name)(w)
        eq(bits(q), W[name + ".q"], name)
        eq(s.numpy(), W[name + ".s"], name + " scale")
    q, s = schemes._q_int8_sym(w.to(torch.float16))
    eq(bits(q), W["_q_int8_sym.fp16in.q"])
    eq(s.numpy(), W["_q_int8_sym.fp16in.s"])
    eq(schemes._q_int8_affine(w).numpy(), W["_q_int8_affine"], "_q_int8_affine")
    eq(schemes._q_int4_sym(w).numpy(), W["_q_int4_sym"], "_q_int4_sym")
    eq(schemes._q_int4_gw(w, group_size=128).numpy(), W["_q_int4_gw.128"], "_q_int4_gw")
    eq(schemes._q_int4_gw(torch.from_numpy(W["w_odd"]), group_size=128).numpy(), W["_q_int4_gw.128.padded"], "_q_int4_gw padded")
    # the registry hands out the same functions with the reference's keyword arguments
    e = schemes.get_scheme("int4_groupwise_128")
    eq(e["quantize"](w, **e["quantize_kwargs"]).numpy(), W["_q_int4_gw.128"])
    q, s = schemes.get_scheme("fp8")["quantize"](w)
    eq(bits(q), W["_q_fp8.q"])


def test_int4_int8_tool_quantizers_bit_exact(W):
    from int4 import quantize_int4 as q4
    from int8 import quantize_int8 as q8
    w = torch.from_numpy(W["w"])
    p, s = q4.quantize_to_int4_per_tensor(w)
    eq(p.numpy(), W["q4pt.packed"]); eq(s.numpy(), W["q4pt.scale"])
    a = q4.quantize_to_int4_affine(w)
    for k in ("packed", "mx", "rx", "my", "ry"):
        eq(a[k].numpy(), W["q4af." + k], "int4 affine " + k)
    g = q4.quantize_to_int4_groupwise(w, 128)
    for k in ("packed", "scales", "zeros"):
        eq(g[k].numpy(), W["q4gw." + k], "int4 groupwise " + k)
    q, s = q8.quantize_to_int8_per_tensor(w)
    eq(q.numpy(), W["q8pt.q"]); eq(s.numpy(), W["q8pt.s"])
    a8 = q8.quantize_to_int8_affine(w)
    for k in ("w_u8", "mx", "rx", "my", "ry"):
        eq(a8[k].numpy(), W["q8af." + k], "int8 affine " + k)


# ------------------------------------------------------------------------------------------------ the CLI's quantize step
def _reference_dir():
    for cand in (os.environ.get("RWKVQ_REFERENCE"), os.path.join(ROOT, "baseline", "_ref")):
        if cand and os.path.exists(os.path.join(cand, "rwkv_quant", "commands.py")):
            return cand
    return None


_RUN = r"""
import sys, types
ref, pkg, model, outdir, schemes_csv, dropin = sys.argv[1:7]
if dropin == "1":
    sys.path.insert(0, pkg)
    import schemes                      # the drop-in module is the one `from schemes import get_scheme` finds
    assert schemes.__file__.startswith(pkg), schemes.__file__
sys.path.insert(0 if dropin != "1" else 1, ref)
from rwkv_quant import commands
for scheme in schemes_csv.split(","):
    rc = commands.cmd_quantize(types.SimpleNamespace(model=model, output=outdir + "/" + scheme + ".pth", scheme=scheme))
    assert not rc, (scheme, rc)
import schemes as used
print("USED", used.__file__)
"""


CLI_SCHEMES = ["fp8", "fp8_perchannel", "int8_symmetric", "int8_affine", "int4_symmetric", "int4_groupwise_128"]


def test_cli_quantize_step_with_dropin_schemes(tmp_path):
    """`rwkv-quant q` of the reference (rwkv_quant/commands.py:173-236) saves the same tensors whichever schemes module
    it resolves: its own or the drop-in."""
    ref = _reference_dir()
    if ref is None:
        pytest.skip("no reference checkout (set RWKVQ_REFERENCE or install it under baseline/_ref)")
    g = torch.Generator().manual_seed(3)
    state = {"emb.weight": torch.randn(16, 64, generator=g).bfloat16()}
    for layer in range(2):
        for name, shape in (("att.receptance", (64, 64)), ("att.key", (64, 64)), ("att.value", (64, 64)), ("att.output", (64, 64)),
                            ("ffn.key", (256, 64)), ("ffn.value", (64, 256))):
            state[f"blocks.{layer}.{name}.weight"] = (torch.randn(shape, generator=g) * 0.05).bfloat16()
        state[f"blocks.{layer}.ln1.weight"] = torch.ones(64).bfloat16()
    model = str(tmp_path / "tiny.pth")
    torch.save(state, model)
    for dropin in ("0", "1"):
        os.makedirs(tmp_path / dropin)
        p = subprocess.run([sys.executable, "-c", _RUN, ref, PKG, model, str(tmp_path / dropin), ",".join(CLI_SCHEMES), dropin],
                           capture_output=True, text=True, env={**os.environ, "NO_COLOR": "1"})
        assert p.returncode == 0, p.stdout + p.stderr
        used = [l for l in p.stdout.splitlines() if l.startswith("USED")][-1]
        assert (PKG in used) == (dropin == "1"), used
    for scheme in CLI_SCHEMES:
        a, b = (torch.load(str(tmp_path / d / f"{scheme}.pth"), map_location="cpu", weights_only=False) for d in ("0", "1"))
        assert set(a) == set(b), scheme
        changed = 0
        for k in a:
            if k == "quant_meta":
                continue
            assert a[k].dtype == b[k].dtype and a[k].shape == b[k].shape, (scheme, k)
            eq(bits(a[k]), bits(b[k]), f"{scheme} {k}")
            changed += k.endswith(".fp8_scale") or (k in state and not torch.equal(a[k].float(), state[k].float()))
        assert changed >= 12, scheme
