"""Pins the CPU oracle: against the tables the reference's circuits hard-code, against
the tables the reference's own host functions produce, against an independent
Python big-integer restatement on small cases, and against outputs of the
reference's CUDA kernels captured on a B200 (tests/golden/ref_gpu_vectors.npz)."""
import json
import math
import os

import numpy as np
import pytest

from conftest import ROOT, rand_i64

GOLD = os.path.join(ROOT, "tests", "golden")


def test_luts_match_the_circuit_tables(orc):
    ts = json.load(open(os.path.join(GOLD, "ts_tables.json")))
    assert orc.lut("softmax_q19").tolist() == ts["q19Table"]      # zk/src/index.ts:2645-2681
    assert orc.lut("silu_q23").tolist() == ts["q23Table"]         # zk/src/index.ts:3382-3418
    assert ts["LOG2E_Q19"] == 756388 and ts["LOG2E_Q23"] == 12102203


def test_luts_match_the_reference_host_functions(orc):
    ref = json.load(open(os.path.join(GOLD, "ref_luts.json")))
    for ours, theirs in (("softmax_q19", "softmax_init_q19"), ("softmax_q21", "softmax_init_q21"),
                         ("silu_q23", "silu_init_q23"), ("silu_q25", "silu_init_q25")):
        assert orc.lut(ours).tolist() == ref[theirs], ours


# ---- independent big-integer restatements (small cases only) -----------------------------

def _wrap64(v):
    v &= (1 << 64) - 1
    return v - (1 << 64) if v >> 63 else v


def _tdiv(a, b):
    q = abs(a) // abs(b)
    return q if (a < 0) == (b < 0) else -q


def py_gemm(A, B, a_r, b_r, s, legacy):
    Bd, M, K = A.shape
    N = B.shape[0]
    C = np.zeros((Bd, M, N), np.int64)
    R = np.zeros((Bd, M, N), np.int64)
    for b in range(Bd):
        for m in range(M):
            for n in range(N):
                tot = sum(_tdiv(int(A[b, m, k]), a_r) * _tdiv(int(B[n, k]), b_r) for k in range(K))
                C[b, m, n] = _wrap64(tot >> s)
                if legacy:
                    mask = ((1 << s) - 1) if s <= 31 else 0xFFFFFFFF   # observed on a B200
                    R[b, m, n] = _wrap64(tot & mask)
                else:
                    R[b, m, n] = _wrap64(tot % (1 << s)) if s > 0 else 0
    return C, R


@pytest.mark.parametrize("b32", [True, False])
@pytest.mark.parametrize("s,a_r,b_r", [(0, 1, 1), (16, 1, 1), (30, 1, 1), (31, 3, 1), (33, 1, 256),
                                       (37, -5, 7), (64, 1, 1), (90, 1, 1)])
def test_gemm_against_bigint(orc, b32, s, a_r, b_r):
    rng = np.random.default_rng(s + 7)
    A = rand_i64(rng, (2, 3, 19), 62)
    B = rand_i64(rng, (4, 19), 31 if b32 else 62)
    if b32:
        B = B.astype(np.int32)
    for legacy in (0, 1):
        C, R = orc.gemm(A, B, a_r, b_r, s, legacy)
        Cp, Rp = py_gemm(A, B, a_r, b_r, s, legacy)
        assert (C == Cp).all()
        assert (R == Rp).all()


def test_gemm_sum_straddles_2_63(orc):
    """int128 accumulation differs from a wrapping int64 one once |sum| >= 2^63."""
    A = np.full((1, 1, 4), 2**40, np.int64)
    B = np.full((1, 4), 2**30, np.int64)
    C, R = orc.gemm(A, B, 1, 1, 16)
    assert int(C[0, 0, 0]) == (4 * 2**70) >> 16
    assert int(orc.gemm_wrap64(A[0], B, 16)[0, 0]) != int(C[0, 0, 0])


def test_gemm_empty_and_ragged(orc):
    A = np.zeros((1, 0, 5), np.int64)
    B = np.zeros((3, 5), np.int32)
    C, R = orc.gemm(A, B, 1, 1, 3)
    assert C.shape == (1, 0, 3)
    A = np.arange(6, dtype=np.int64).reshape(1, 2, 3) - 2
    B = np.array([[1, -1, 2]], np.int32)
    C, R = orc.gemm(A, B, 1, 1, 1)
    assert C.tolist() == [[[(-2 + 1 + 0) >> 1], [(1 - 2 + 6) >> 1]]]
    assert R.tolist() == [[[1], [1]]]


def test_rope_against_bigint(orc):
    rng = np.random.default_rng(3)
    A = rand_i64(rng, (2, 3, 2, 4, 2), 62)
    T = rand_i64(rng, (3, 4, 2), 43)
    for shift in (42, 16, 0, 63):
        C = orc.rope(A, T, shift)
        for idx in np.ndindex(2, 3, 2, 4):
            a0, a1 = (int(v) for v in A[idx])
            b0, b1 = (int(v) for v in T[idx[1], idx[3]])
            p = lambda x, y: _wrap64((x * y) >> shift)
            assert int(C[idx][0]) == _wrap64(p(a0, b0) - p(a1, b1))
            assert int(C[idx][1]) == _wrap64(p(a0, b1) + p(a1, b0))


def test_rms_norm_against_bigint(orc):
    rng = np.random.default_rng(4)
    for bits, wdt in ((37, np.int32), (60, np.int64), (5, np.int32)):
        A = rand_i64(rng, (5, 33), bits)
        W = rand_i64(rng, (33,), 20).astype(wdt)
        C, rms = orc.rms_norm(A, W, 1, 33)
        for m in range(5):
            acc = 1 + sum(int(v) * int(v) for v in A[m])
            r = math.isqrt(acc // 33)
            assert int(rms[m]) == r
            for i in range(33):
                want = (int(A[m, i]) * int(W[i])) // r if r else 0   # floor division
                assert int(C[m, i]) == _wrap64(want)
    # the circuit's constraint: x*w = q*rms + r with 0 <= r < rms (zk/src/index.ts:623-625)
    A = rand_i64(rng, (2, 64), 37)
    W = rand_i64(rng, (64,), 21).astype(np.int32)
    C, rms = orc.rms_norm(A, W, 1, 64)
    rem = A.astype(object) * W.astype(object) - C.astype(object) * rms.astype(object)[:, None]
    assert all(0 <= int(v) < int(rms[i]) for i in range(2) for v in rem[i])


def test_rms_zero_row_is_defined_as_zero(orc):
    A = np.zeros((1, 8), np.int64)
    C, rms = orc.rms_norm(A, np.ones(8, np.int32), 1, 8)
    assert rms.tolist() == [0] and not C.any()


def py_softmax_q19(x, lut):
    mx = max(x)
    w = []
    for v in x:
        d = (mx - v) & ((1 << 64) - 1)
        if d > (64 << 19):
            w.append(0)
            continue
        y = (d * 756388) >> 19
        k, f = y >> 19, y & 0x7FFFF
        t = int(lut[f >> 11])
        w.append(0 if k >= 64 else t >> k)
    s = sum(w)
    return [((wi << 19) // s) if s else 0 for wi in w], w


def test_softmax_q19_against_bigint(orc):
    rng = np.random.default_rng(5)
    lut = orc.lut("softmax_q19")
    X = np.rint(rng.standard_normal((3, 4, 37)) * 4 * 2**19).astype(np.int64)
    X[0, 0, 5:] += -(64 << 36)          # the causal mask value (model.py:1555)
    X[1, 2, :] = 7                      # constant row
    X[2, 3, 0] = 2**62
    X[2, 3, 1] = -2**62                 # difference wraps as uint64
    C, W = orc.softmax(X, 19, want_weights=True)
    for idx in np.ndindex(3, 4):
        c, w = py_softmax_q19([int(v) for v in X[idx]], lut)
        assert C[idx].tolist() == c
        assert W[idx].tolist() == w
    # circuit constraint: probabilities of a row sum to at most 2^19 (zk/src/index.ts:2727-2749)
    assert (C.sum(-1) <= 2**19).all() and (C >= 0).all()


def test_softmax_q21_properties(orc):
    rng = np.random.default_rng(6)
    X = np.rint(rng.standard_normal((8, 50)) * 2**21).astype(np.int64)
    C = orc.softmax(X, 21)
    ref = np.exp((X - X.max(-1, keepdims=True)) / 2.0**21)
    ref = ref / ref.sum(-1, keepdims=True)
    assert np.abs(C / 2.0**21 - ref).max() < 2e-3
    assert (C.argmax(-1) == X.argmax(-1)).all()


def py_act_q23(r, lut, silu):
    LIM = 64 << 23
    if r >= LIM:
        return r
    if r <= -LIM:
        return 0
    y = ((-r) * 12102203) >> 23
    k, f = y >> 23, y & 0x7FFFFF
    t = int(lut[f >> 15])
    u = 0
    if k > -63:
        if k < 0:
            u = t >> (-k)
        else:
            u = 0 if k >= 64 else _wrap64(t << k)     # GPU shift semantics
    den = _wrap64((1 << 23) + u)
    q = _tdiv(1 << 46, den) if den else 0
    return _wrap64(_wrap64(r * q) >> 23) if silu else q


def test_act_q23_against_bigint_including_the_wrapping_shift_range(orc):
    lut = orc.lut("silu_q23")
    LIM = 64 << 23
    rng = np.random.default_rng(7)
    r = np.concatenate([
        np.array([0, 1, -1, LIM - 1, LIM, LIM + 1, -LIM + 1, -LIM, -LIM - 1, 2**62, -2**62]),
        rng.integers(-LIM, LIM, 3000),
        rng.integers(-LIM, -20 * 2**23, 3000),        # k >= 28: u overflows 64 bits from k = 40
        np.rint(rng.standard_normal(2000) * 2**23).astype(np.int64),
    ]).astype(np.int64)
    for silu in (True, False):
        got = orc.act(r, "silu" if silu else "sigmoid", 23)
        want = [py_act_q23(int(v), lut, silu) for v in r]
        assert got.tolist() == want
    # sigmoid stays within [0, 2^23] wherever the shift does not wrap (r > -27 * 2^23)
    mid = r[(r > -27 * 2**23) & (r < LIM)]
    s = orc.act(mid, "sigmoid", 23)
    assert (s >= 0).all() and (s <= 2**23).all()


def test_act_q25_matches_float_sigmoid(orc):
    rng = np.random.default_rng(8)
    r = np.rint(rng.standard_normal(4000) * 3 * 2**25).astype(np.int64)
    s = orc.act(r, "sigmoid", 25) / 2.0**25
    assert np.abs(s - 1 / (1 + np.exp(-r / 2.0**25))).max() < 4e-3
    # Q25 negates after the floor shift, Q23 before: the two forms differ on non-multiples
    assert orc.act(np.array([5], np.int64), "silu", 25).tolist() != [None]


def test_einsums_against_numpy_object_math(orc):
    rng = np.random.default_rng(9)
    B, S, H, D, C, T = 2, 3, 2, 5, 7, 4
    q = rand_i64(rng, (B, S, H, D), 40)
    W1 = rand_i64(rng, (H, D, C), 31).astype(np.int32)
    r = 29
    out = orc.einsum_bshd_hdc_bshc(q, W1, r)
    want = (np.einsum("bshd,hdc->bshc", q.astype(object), W1.astype(object)) + r // 2) >> r
    assert (out.astype(object) == want).all()
    A = rand_i64(rng, (B, S, H, C), 40)
    KV = rand_i64(rng, (B, T, C), 40)
    out = orc.einsum_bshc_btc_bsht(A, KV, 23)
    want = (np.einsum("bshc,btc->bsht", A.astype(object), KV.astype(object)) + 11) >> 23
    assert (out.astype(object) == want).all()
    P = rand_i64(rng, (B, S, H, T), 19)
    out = orc.einsum_bsht_btc_bshc(P, KV, 23)
    want = (np.einsum("bsht,btc->bshc", P.astype(object), KV.astype(object)) + 11) >> 23
    assert (out.astype(object) == want).all()
    W2 = rand_i64(rng, (H, D, C), 31).astype(np.int32)
    out = orc.einsum_bshc_hdc_bshd(A, W2, 30)
    want = np.einsum("bshc,hdc->bshd", A.astype(object), W2.astype(object)) >> 30   # no rounding
    assert (out.astype(object) == want).all()


# ---- outputs of the reference's own CUDA kernels, captured on a B200 ----------------------

def _gpu_vectors():
    path = os.path.join(GOLD, "ref_gpu_vectors.npz")
    if not os.path.exists(path):
        pytest.skip("ref_gpu_vectors.npz not generated yet (tests/golden/make_gpu_golden.py)")
    return np.load(path)


def test_oracle_matches_reference_gpu_kernels(orc):
    v = _gpu_vectors()
    import sys
    sys.path.insert(0, GOLD)
    import make_gpu_golden as mk
    bad = mk.check_against(v, orc)
    assert not bad, bad
