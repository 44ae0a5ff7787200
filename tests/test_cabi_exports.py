"""The C-ABI library loads without a GPU and exports every symbol the header declares."""
import ctypes
import os
import re

from conftest import ROOT

REFERENCE_SYMBOLS = [
    "int64_32_bmm_broadcast_launcher", "int64_64_bmm_broadcast_launcher", "bf16_to_int32_2d",
    "wkv_b_bf16_to_int32", "float32_to_int64_2d", "complex_int64_mul", "rms_norm_32", "rms_norm_64",
    "einsum_bshd_hdc_bshc", "einsum_bshc_btc_bsht", "einsum_bsht_btc_bshc", "einsum_bshc_hdc_bshd",
    "softmax_q21", "softmax_q19", "softmax_init_q21", "softmax_init_q19", "silu_q25", "sigmoid_q25",
    "silu_q23", "sigmoid_q23", "silu_init_q25", "silu_init_q23",
]


def declared_functions():
    names = []
    for fn in sorted(os.listdir(os.path.join(ROOT, "include"))):
        if not fn.endswith(".h"):
            continue
        src = open(os.path.join(ROOT, "include", fn)).read()
        src = re.sub(r"/\*.*?\*/", "", src, flags=re.S)
        src = re.sub(r"^\s*#.*$", "", src, flags=re.M)
        names += re.findall(r"\b([A-Za-z_][A-Za-z0-9_]*)\s*\([^;{]*\)\s*;", src)
    return names


def test_header_declares_the_reference_symbols():
    decl = set(declared_functions())
    missing = [s for s in REFERENCE_SYMBOLS if s not in decl]
    assert not missing, missing


def test_library_exports_every_declared_symbol(libpath):
    lib = ctypes.CDLL(libpath)
    names = declared_functions()
    assert len(names) >= len(REFERENCE_SYMBOLS) + 10
    missing = [n for n in names if not hasattr(lib, n)]
    assert not missing, missing


def test_host_only_entry_points(libpath, orc):
    """The LUT generators run on the host: callable without a GPU."""
    import json
    lib = ctypes.CDLL(libpath)
    ts = json.load(open(os.path.join(ROOT, "tests/golden/ts_tables.json")))
    ref = json.load(open(os.path.join(ROOT, "tests/golden/ref_luts.json")))
    for name, want in (("softmax_init_q19", ts["q19Table"]), ("silu_init_q23", ts["q23Table"]),
                       ("softmax_init_q21", ref["softmax_init_q21"]),
                       ("silu_init_q25", ref["silu_init_q25"])):
        buf = (ctypes.c_int64 * 256)()
        getattr(lib, name)(buf)
        assert list(buf) == want, name
    lib.zkds_status_string.restype = ctypes.c_char_p
    assert lib.zkds_status_string(0) == b"ok"
    assert lib.zkds_last_status() == 0


def test_kernel_module_surface(kmod):
    """Every name the reference's model.py / generate.py import from `kernel` exists."""
    for name in ("act_quant", "weight_dequant", "fp8_gemm", "int64_bmm_broadcast",
                 "complex_int64_mul_broadcast", "einsum_bshd_hdc_bshc", "einsum_bshc_btc_bsht",
                 "softmax_init_q21", "softmax_q21", "einsum_bsht_btc_bshc", "einsum_bshc_hdc_bshd",
                 "silu_init_q25", "silu_q25", "sigmoid_q25", "softmax_init_q19", "softmax_q19",
                 "silu_init_q23", "silu_q23", "sigmoid_q23", "RMS_Norm_int64", "saveTensor"):
        assert callable(getattr(kmod, name)), name
