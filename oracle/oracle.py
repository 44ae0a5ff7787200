"""numpy front end of the CPU oracle (liboracle.so, built from oracle.c).

TEST INFRASTRUCTURE ONLY: imported by tests/, by the smoke test and by the
bench's cpu_baseline / reference legs as the checker.  The product path never
imports this module.

Every function takes and returns C-contiguous numpy arrays and follows the
reference kernel named in the matching function of oracle.c.
"""
import ctypes
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB = None

R_MATH = 0
R_LEGACY = 1


def build(force=False):
    """Compile liboracle.so (and oracle/_ref when the reference checkout exists)."""
    so = os.path.join(_HERE, "liboracle.so")
    if force or not os.path.exists(so) or os.path.getmtime(so) < os.path.getmtime(
            os.path.join(_HERE, "oracle.c")):
        subprocess.run(["make", "-C", _HERE, "-s", os.path.join(_HERE, "liboracle.so")],
                       check=True)
    return so


def lib():
    global _LIB
    if _LIB is None:
        _LIB = ctypes.CDLL(build())
        _LIB.orc_num_threads.restype = ctypes.c_int
    return _LIB


def num_threads():
    return int(lib().orc_num_threads())


def set_threads(n):
    lib().orc_set_threads(ctypes.c_int(int(n)))


def _p(a):
    return ctypes.c_void_p(a.ctypes.data) if a is not None else ctypes.c_void_p(0)


def _ll(v):
    return ctypes.c_longlong(int(v))


def _i64(a):
    a = np.ascontiguousarray(a)
    assert a.dtype == np.int64, a.dtype
    return a


def gemm(A, B, a_r=1, b_r=1, s=0, rmode=R_MATH):
    """(Bdim,M,K) int64 x (N,K) int32|int64 -> C, R (Bdim,M,N) int64."""
    A = _i64(A)
    B = np.ascontiguousarray(B)
    assert B.dtype in (np.int32, np.int64)
    Bd, M, K = A.shape
    N, K2 = B.shape
    assert K2 == K
    C = np.empty((Bd, M, N), np.int64)
    R = np.empty((Bd, M, N), np.int64)
    lib().orc_gemm(_p(A), _p(B), ctypes.c_int(B.dtype == np.int32), _p(C), _p(R), _ll(a_r),
                   _ll(b_r), _ll(s), _ll(Bd), _ll(M), _ll(K), _ll(N), ctypes.c_int(rmode))
    return C, R


def gemm_wrap64(A, B, s):
    """Wrapping-int64 (M,K)x(N,K) >> s: the reference's torch CPU path."""
    A = _i64(A)
    B = _i64(B)
    M, K = A.shape
    N = B.shape[0]
    C = np.empty((M, N), np.int64)
    lib().orc_gemm_wrap64(_p(A), _p(B), _p(C), _ll(s), _ll(M), _ll(K), _ll(N))
    return C


def rope(A, T, shift=42):
    """A (B,S,H,P,2) int64, T (..S..,P,2) int64 broadcast over B,H."""
    A = _i64(A)
    T = _i64(T)
    Bn, S, H, P, two = A.shape
    assert two == 2 and T.size == S * P * 2
    C = np.empty_like(A)
    lib().orc_rope(_p(A), _p(T), _p(C), _ll(Bn), _ll(S), _ll(H), _ll(P), ctypes.c_int(shift))
    return C


def rms_rows(A, eps, dim):
    A = _i64(A)
    M, N = A.shape
    rms = np.empty((M,), np.int64)
    lib().orc_rms_rows(_p(A), _ll(M), _ll(N), _ll(eps), _ll(dim), _p(rms))
    return rms


def rms_norm(A, W, eps=1, dim=None):
    """Full RMSNorm: returns (C, rms)."""
    A = _i64(A)
    W = np.ascontiguousarray(W)
    M, N = A.shape
    if dim is None:
        dim = N
    rms = rms_rows(A, eps, dim)
    C = np.empty_like(A)
    lib().orc_rms_norm(_p(A), _p(W), ctypes.c_int(W.dtype == np.int32), _p(rms), _p(C), _ll(M),
                       _ll(N))
    return C, rms


def rms_norm_given(A, W, rms):
    A = _i64(A)
    W = np.ascontiguousarray(W)
    rms = _i64(rms)
    M, N = A.shape
    C = np.empty_like(A)
    lib().orc_rms_norm(_p(A), _p(W), ctypes.c_int(W.dtype == np.int32), _p(rms), _p(C), _ll(M),
                       _ll(N))
    return C


def einsum_bshd_hdc_bshc(q, W, r):
    q = _i64(q)
    W = np.ascontiguousarray(W)
    assert W.dtype == np.int32
    B, S, H, D = q.shape
    C = W.shape[2]
    out = np.empty((B, S, H, C), np.int64)
    lib().orc_einsum_bshd_hdc_bshc(_p(q), _p(W), _p(out), _ll(r), _ll(B), _ll(S), _ll(H), _ll(D),
                                   _ll(C))
    return out


def einsum_bshc_btc_bsht(A, KV, r):
    A = _i64(A)
    KV = _i64(KV)
    B, S, H, C = A.shape
    T = KV.shape[1]
    out = np.empty((B, S, H, T), np.int64)
    lib().orc_einsum_bshc_btc_bsht(_p(A), _p(KV), _p(out), _ll(r), _ll(B), _ll(S), _ll(H), _ll(T),
                                   _ll(C))
    return out


def einsum_bsht_btc_bshc(P, KV, r):
    P = _i64(P)
    KV = _i64(KV)
    B, S, H, T = P.shape
    C = KV.shape[2]
    out = np.empty((B, S, H, C), np.int64)
    lib().orc_einsum_bsht_btc_bshc(_p(P), _p(KV), _p(out), _ll(r), _ll(B), _ll(S), _ll(H), _ll(T),
                                   _ll(C))
    return out


def einsum_bshc_hdc_bshd(A, W, r):
    A = _i64(A)
    W = np.ascontiguousarray(W)
    assert W.dtype == np.int32
    B, S, H, C = A.shape
    D = W.shape[1]
    out = np.empty((B, S, H, D), np.int64)
    lib().orc_einsum_bshc_hdc_bshd(_p(A), _p(W), _p(out), _ll(r), _ll(B), _ll(S), _ll(H), _ll(D),
                                   _ll(C))
    return out


def lut(name):
    """name in {'softmax_q19','softmax_q21','silu_q23','silu_q25'} -> int64[256]."""
    t = np.zeros((256,), np.int64)
    getattr(lib(), "orc_%s" % name.replace("softmax_", "softmax_init_").replace(
        "silu_", "silu_init_"))(_p(t))
    return t


def softmax(X, frac=19, want_weights=False):
    X = _i64(X)
    T = X.shape[-1]
    rows = X.size // T if T else 0
    C = np.empty_like(X)
    Rw = np.empty_like(X) if want_weights else None
    fn = lib().orc_softmax_q19 if frac == 19 else lib().orc_softmax_q21
    table = lut("softmax_q%d" % frac)  # keep alive across the call
    fn(_p(X), _p(Rw), _p(C), _p(table), _ll(rows), _ll(T))
    return (C, Rw) if want_weights else C


def act(X, kind="silu", frac=23):
    X = _i64(X)
    C = np.empty_like(X)
    fn = lib().orc_act_q23 if frac == 23 else lib().orc_act_q25
    table = lut("silu_q%d" % frac)  # keep alive across the call
    fn(_p(X), _p(C), _p(table), _ll(X.size), ctypes.c_int(kind == "silu"))
    return C
