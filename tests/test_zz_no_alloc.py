"""zkds_gemm_noalloc: the GEMM entry point for hosts that cannot allocate inside a call.

Who needs it: a serving process whose own memory pool already holds the whole GPU (so a
cudaMalloc made by this library would fail or fragment the pool), or a latency-critical loop
that cannot take the device-wide synchronisation an allocation implies.  The entry point keeps
its limb planes and status words in a fixed 64 MiB device array inside the library instead.

This file is collected last on purpose: if it fails, every other test has already run.
Checked here, through the C ABI: two calls in a row give word-for-word the output of the
allocating entry point zkds_gemm and of the CPU oracle (the second call is smaller, so stale bytes of the first would
show), a shape beyond the fixed capacity is refused, and the second call changes the amount of
free device memory by nothing.
"""
import ctypes

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _bind(libpath):
    lib = ctypes.CDLL(libpath)
    vp, ll, i = ctypes.c_void_p, ctypes.c_longlong, ctypes.c_int
    sig = [vp, vp, i, vp, vp, ll, ll, ll, ll, ll, ll, ll, i, i, i, vp]
    lib.zkds_gemm.argtypes = sig
    lib.zkds_gemm_noalloc.argtypes = sig
    lib.zkds_gemm_noalloc_capacity.restype = ctypes.c_ulonglong
    lib.zkds_gemm_noalloc_bytes.restype = ctypes.c_ulonglong
    lib.zkds_gemm_noalloc_bytes.argtypes = [ll, ll, ll, ll, i, i]
    return lib


def _case(rng, dev, Bd, M, K, N, abits, bbits, b32):
    A = rng.integers(-(1 << abits), 1 << abits, (Bd, M, K), dtype=np.int64)
    B = rng.integers(-(1 << bbits), 1 << bbits, (N, K), dtype=np.int64)
    if b32:
        B = B.astype(np.int32)
    return torch.from_numpy(A).to(dev), torch.from_numpy(B).to(dev)


def _run(fn, A, B, s, a_limbs, b_limbs, flags):
    Bd, M, K = A.shape
    N = B.shape[0]
    C = torch.full((Bd, M, N), -7, dtype=torch.int64, device=A.device)
    R = torch.full((Bd, M, N), -7, dtype=torch.int64, device=A.device)
    rc = fn(A.data_ptr(), B.data_ptr(), 32 if B.dtype == torch.int32 else 64, C.data_ptr(),
            R.data_ptr(), 1, 1, s, Bd, M, K, N, a_limbs, b_limbs, flags,
            ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
    torch.cuda.synchronize()
    return rc, C.cpu().numpy(), R.cpu().numpy()


def test_noalloc_gemm_matches_the_allocating_entry_point_twice_in_a_row(libpath, dev, orc):
    lib = _bind(libpath)
    rng = np.random.default_rng(2025)
    LIMB = 2           # ZKDS_ALGO_LIMB: both entry points on the tensor-core kernel
    cases = [
        (1, 300, 2000, 520, 30, 31, True, 30, 0, 0),     # ranges measured on the device
        (2, 33, 700, 65, 20, 15, False, 16, 3, 3),       # smaller, caller-provided limb counts
    ]
    free_before = None
    for n, (Bd, M, K, N, ab, bb, b32, s, al, bl) in enumerate(cases):
        A, B = _case(rng, dev, Bd, M, K, N, ab, bb, b32)
        rc0, C0, R0 = _run(lib.zkds_gemm, A, B, s, al, bl, LIMB)
        assert rc0 == 0
        if n == 1:
            torch.cuda.synchronize()
            free_before = torch.cuda.mem_get_info(dev)[0]
        rc1, C1, R1 = _run(lib.zkds_gemm_noalloc, A, B, s, al, bl, LIMB)
        if n == 1:
            assert torch.cuda.mem_get_info(dev)[0] == free_before, "the call allocated device memory"
        assert rc1 == 0
        assert np.array_equal(C1, C0), "call %d: quotient differs" % n
        assert np.array_equal(R1, R0), "call %d: remainder differs" % n
        # and both are what the CPU oracle computes (flags = 2: remainder sum mod 2^s)
        Co, Ro = orc.gemm(A.cpu().numpy(), B.cpu().numpy(), 1, 1, s, orc.R_MATH)
        assert np.array_equal(C1, Co), "call %d: quotient differs from the oracle" % n
        assert np.array_equal(R1, Ro), "call %d: remainder differs from the oracle" % n


def test_noalloc_gemm_rejects_what_does_not_fit(libpath, dev):
    lib = _bind(libpath)
    cap = lib.zkds_gemm_noalloc_capacity()
    assert cap == (64 << 20) - 256
    # 4 limbs x 4096 x 8192 bytes of A planes alone exceed the fixed array
    assert lib.zkds_gemm_noalloc_bytes(1, 4096, 8192, 64, 4, 4) > cap
    A = torch.zeros((1, 4096, 8192), dtype=torch.int64, device=dev)
    B = torch.zeros((64, 8192), dtype=torch.int32, device=dev)
    rc, C, R = _run(lib.zkds_gemm_noalloc, A, B, 16, 4, 4, 2)
    assert rc == 2                       # ZKDS_ERR_RANGE
    assert (C == -7).all()               # nothing was written
    # a promised limb count that the data does not fit is reported, not silently wrong
    A = torch.full((1, 8, 64), 1 << 40, dtype=torch.int64, device=dev)
    B = torch.ones((16, 64), dtype=torch.int32, device=dev)
    rc, C, R = _run(lib.zkds_gemm_noalloc, A, B, 0, 2, 1, 2)
    assert rc == 2
