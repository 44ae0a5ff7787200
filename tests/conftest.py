import ctypes
import importlib
import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
PKG = "zk-deepseek_b200"
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


@pytest.fixture(scope="session")
def orc():
    from oracle import oracle
    oracle.build()
    return oracle


@pytest.fixture(scope="session")
def libpath():
    importlib.import_module(PKG + ".build").build()
    return os.path.join(ROOT, PKG, "libint64gemm.so")


@pytest.fixture(scope="session")
def kmod(libpath):
    """The drop-in kernel module (needs the built library; GPU needed only to call it)."""
    return importlib.import_module(PKG + ".kernel")


@pytest.fixture(scope="session")
def dev():
    import torch
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    return torch.device("cuda:0")


class RefLib:
    """ctypes view of the reference's own library (oracle/_ref), bound the way the
    reference's kernel.py binds it.  Usable only inside the reference's limits:
    rows of T, C, D, H <= 1024 threads per block and < 2^31 elements."""

    def __init__(self, path):
        self.lib = ctypes.CDLL(path)
        vp, ll, i = ctypes.c_void_p, ctypes.c_longlong, ctypes.c_int
        L = self.lib
        for n in ("int64_64_bmm_broadcast_launcher", "int64_32_bmm_broadcast_launcher"):
            getattr(L, n).argtypes = [vp, vp, vp, vp, ll, ll, ll, i, i, i, i]
        L.complex_int64_mul.argtypes = [vp, vp, vp, i, i, i, i]
        L.rms_norm_32.argtypes = [vp, vp, vp, vp, i, i]
        L.rms_norm_64.argtypes = [vp, vp, vp, vp, i, i]
        for n in ("einsum_bshd_hdc_bshc", "einsum_bshc_btc_bsht", "einsum_bsht_btc_bshc",
                  "einsum_bshc_hdc_bshd"):
            getattr(L, n).argtypes = [vp, vp, vp, ll, i, i, i, i, i]
        for n in ("softmax_q21", "softmax_q19"):
            getattr(L, n).argtypes = [vp, vp, vp, i, i, i, i]
        for n in ("silu_q25", "sigmoid_q25", "silu_q23", "sigmoid_q23"):
            getattr(L, n).argtypes = [vp, vp, vp, i, i, i]
        for n in ("softmax_init_q21", "softmax_init_q19", "silu_init_q25", "silu_init_q23"):
            getattr(L, n).argtypes = [vp]
        # exported by the reference, bound nowhere in its kernel.py (int64_gemm.cu:126,173,215)
        L.bf16_to_int32_2d.argtypes = [vp, vp, i, i, i]
        L.wkv_b_bf16_to_int32.argtypes = [vp, vp, i, i]
        L.float32_to_int64_2d.argtypes = [vp, vp, i, i, i]


@pytest.fixture(scope="session")
def reflib():
    path = os.path.join(ROOT, "oracle", "_ref", "libint64gemm_ref.so")
    if not os.path.exists(path):
        pytest.skip("reference library not built (oracle/_ref)")
    return RefLib(path)


def rand_i64(rng, shape, bits):
    """uniform signed integers of about `bits` magnitude bits"""
    lim = 1 << bits
    return rng.integers(-lim, lim, size=shape, dtype=np.int64)
