"""CPU-side checks of the boundary: the library loads, exports every symbol the header declares, and the
drop-in modules expose the reference's names with the reference's arguments.  No compute call is made."""
import ctypes
import inspect
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HEADER = os.path.join(ROOT, "include", "rwkvq.h")


def declared_symbols():
    text = open(HEADER).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(rwkvq_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    import rwkvq_abi as abi
    assert os.path.exists(abi.LIB_PATH), "librwkvq.so not built: python rwkv7-quantization_b200/build_ext.py"
    lib = ctypes.CDLL(abi.LIB_PATH)
    names = declared_symbols()
    assert len(names) >= 15
    for n in names:
        assert hasattr(lib, n), f"{n} declared in include/rwkvq.h but not exported"
    # and the binding table covers the header
    assert set(names) <= set(abi.SIGNATURES), set(names) - set(abi.SIGNATURES)
    assert abi.lib().rwkvq_version() >= 100


def test_binding_argument_counts_match_header():
    import rwkvq_abi as abi
    text = re.sub(r"/\*.*?\*/", "", open(HEADER).read(), flags=re.S)
    for name, args in abi.SIGNATURES.items():
        m = re.search(r"\b" + name + r"\s*\(([^;]*?)\)\s*;", text, flags=re.S)
        assert m, name
        params = m.group(1).strip()
        n = 0 if params in ("", "void") else params.count(",") + 1
        assert n == len(args), f"{name}: header has {n} parameters, binding has {len(args)}"


# public names of the reference modules and the parameter names their callers rely on
REFERENCE_API = {
    "fp8_ops": {
        "is_fp8_weight": ["z", "key"],
        "load_fp8_weight": ["z", "key", "dev"],
        "linear_fp8": ["x", "weight_info", "out_dtype"],
        "linear_int8": ["x", "weight_info", "out_dtype"],
        "linear_quantized": ["x", "weight_info", "out_dtype"],
        "linear_quantized_fused": ["x", "weight_info", "out_dtype"],
    },
    "fused_fp8_gemm": {
        "prep_x": ["x", "awq_scale", "out"],
        "prep3_x": ["xr", "xk", "xv", "awq_r", "awq_k"],
        "prep_x_fp8": ["x"],
        "prep_x_int8": ["x"],
        "prep3_x_int8": ["xr", "xk", "xv"],
        "linear_fp8_m1_fused": ["x", "weight_info", "out_dtype"],
        "linear_fp8_fused": ["x", "weight_info_or_w", "res_scale", "out_dtype"],
        "linear_rkv_fused": ["xr", "xk", "xv", "wr_info", "wk_info", "wv_info", "out_dtype"],
        "linear_int8_fused": ["x", "weight_info", "out_dtype"],
        "linear_rkv_int8_fused": ["xr", "xk", "xv", "wr_info", "wk_info", "wv_info", "out_dtype"],
        "linear_quantized_fused": ["x", "weight_info", "out_dtype"],
        "_cfg_for": ["M", "N", "K"],
        "_cfg_for_rkv": ["M", "N", "K"],
        "_best_method": ["M", "N", "K"],
    },
    "schemes": {
        "get_scheme": ["name"],
        "list_schemes": [],
        "print_scheme_table": [],
        "_q_fp8": ["w"], "_q_fp8_perchannel": ["w"], "_q_int8_sym": ["w"], "_q_int8_affine": ["w"],
        "_q_int4_sym": ["w"], "_q_int4_gw": ["w", "group_size"],
    },
}


@pytest.mark.parametrize("module", sorted(REFERENCE_API))
def test_dropin_modules_keep_reference_names(module):
    mod = __import__(module)
    for fn, params in REFERENCE_API[module].items():
        assert hasattr(mod, fn), f"{module}.{fn} missing"
        got = [p.name for p in inspect.signature(getattr(mod, fn)).parameters.values()
               if p.kind in (p.POSITIONAL_OR_KEYWORD,)]
        assert got[: len(params)] == params, (module, fn, got)


def test_engine_import_line_resolves():
    # the import line of the reference engine (rwkv7_fast_v3a.py:12-15)
    from fp8_ops import is_fp8_weight, load_fp8_weight, linear_quantized, linear_quantized_fused, FUSED_M_MAX  # noqa
    from fused_fp8_gemm import linear_rkv_fused, linear_rkv_int8_fused  # noqa
    import fused_fp8_gemm as f
    import fp8_ops
    assert FUSED_M_MAX == 512 and f.FUSED_M_MAX == 512 and f.USE_CUDA_GRAPH is False
    assert fp8_ops.FP8_E4M3_MAX == 448.0 and f.F8E4M3_MAX == 448.0


def test_scheme_registry_keys_and_fields():
    import schemes
    for key in ("fp8", "fp8_perchannel", "int8_symmetric", "int8_affine", "int4_symmetric", "int4_groupwise_128",
                "int4_groupwise_256"):
        s = schemes.get_scheme(key)
        for field in ("name", "format", "bits_per_weight", "activation_bits", "compression", "quantize",
                      "hardware_req", "has_hardware_accel"):
            assert field in s
    assert schemes.SCHEMES["int4_groupwise_256"]["quantize_kwargs"] == {"group_size": 256}
    with pytest.raises(ValueError):
        schemes.get_scheme("nope")


def test_load_fp8_weight_dict_layout():
    import torch
    import fp8_ops
    z = {"w": torch.zeros(4, 16, dtype=torch.int8), "w.fp8_scale": torch.tensor(0.5)}
    assert fp8_ops.is_fp8_weight(z, "w")
    info = fp8_ops.load_fp8_weight(z, "w", "cpu")
    assert info["qtype"] == "int8" and "w.fp8_scale" not in z and info["tensor_scale"].item() == 0.5
    z = {"w": torch.zeros(4, 16).to(torch.float8_e4m3fn), "w.fp8_scale": torch.tensor(0.5)}
    assert fp8_ops.load_fp8_weight(z, "w", "cpu")["qtype"] == "fp8"


def test_no_cpu_fallback_without_device():
    import torch
    if torch.cuda.is_available():
        pytest.skip("device present")
    import fused_fp8_gemm as f
    with pytest.raises(RuntimeError):
        f.prep_x_int8(torch.zeros(2, 64, dtype=torch.float16))


def test_int4_k_split_plan_is_host_arithmetic():
    """rwkvq_gemv_int4_ksplit_slices only does shared-memory arithmetic (no device needed): the slices the K-split
    form uses for the 7.2B shapes, 1 where one launch already holds the block, 0 for shapes it does not take."""
    import rwkvq_abi as abi
    sl = abi.lib().rwkvq_gemv_int4_ksplit_slices
    assert sl(16, 4096, 16384) == 8          # FFN value, 16 rows: 2048-k slices, 64 KB of activations each
    assert sl(8, 4096, 16384) == 4
    assert sl(4, 4096, 16384) == 2
    assert sl(1, 4096, 16384) == 1           # one row fits beside a deep ring
    assert sl(16, 4096, 4096) == 2           # attention output: few row tiles, the split pays
    assert sl(16, 16384, 4096) == 1          # FFN key: many row tiles, the block that fits is left whole
    assert sl(17, 4096, 4096) == 0 and sl(4, 4096, 1000) == 0 and sl(0, 4096, 4096) == 0


def test_column_split_auto_gather_rule():
    """gather="auto": push up to 4 ranks at every row count, on more ranks only up to 512 rows (measured basis in the
    class's docstring); the rule depends on sizes only, so all ranks agree."""
    import rwkvq_dist as D
    C = D.ColumnSplitLinear
    assert C.auto_pushes(2, 1) and C.auto_pushes(2, 4096) and C.auto_pushes(4, 100000)
    assert C.auto_pushes(8, 256) and C.auto_pushes(8, 512) and not C.auto_pushes(8, 513) and not C.auto_pushes(8, 4096)


def test_column_split_rejects_unknown_gather():
    import rwkvq_dist as D
    with pytest.raises(ValueError):
        D.ColumnSplitLinear({"weight": None}, lambda *a: None, gather="ring")
