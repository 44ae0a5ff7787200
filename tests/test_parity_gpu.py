"""GPU parity: the sm_100a library, called through its C ABI (the drop-in kernel
module and the reference's own symbol names), against the CPU oracle and against the
reference's CUDA kernels.  Bit-exact: 0 mismatched int64 words everywhere."""
import ctypes

import numpy as np
import pytest
import torch

from conftest import rand_i64

pytestmark = pytest.mark.gpu


def g(a, dev):
    return torch.from_numpy(np.ascontiguousarray(a)).to(dev)


def same(got, want, what=""):
    got = got.cpu().numpy() if isinstance(got, torch.Tensor) else got
    assert got.shape == want.shape, (what, got.shape, want.shape)
    bad = int((got != want).sum())
    assert bad == 0, "%s: %d of %d words differ" % (what, bad, got.size)


# ---- GEMM ---------------------------------------------------------------------------------

@pytest.mark.parametrize("algo", ["exact", "auto"])
@pytest.mark.parametrize("wdtype", [np.int64, np.int32])
def test_gemm_config1(kmod, orc, dev, algo, wdtype):
    """BASELINE config: X int64 [32,7168] in +-2^20, W [576,7168] in +-2^15, shift 16, seed 0."""
    rng = np.random.default_rng(0)
    X = rng.integers(-2**20, 2**20, (1, 32, 7168), dtype=np.int64)
    W = rng.integers(-2**15, 2**15, (576, 7168), dtype=np.int64).astype(wdtype)
    kmod.ALGO = kmod.ALGO_EXACT if algo == "exact" else kmod.ALGO_AUTO
    try:
        C, R = kmod.int64_bmm_broadcast(g(X, dev), g(W, dev), 1, 1, 16)
    finally:
        kmod.ALGO = kmod.ALGO_AUTO
    Co, Ro = orc.gemm(X, W, 1, 1, 16, orc.R_LEGACY)
    same(C, Co, "C")
    same(R, Ro, "R")
    # wrapping int64 equals the 128-bit sum here (|sum| < 2^63): the reference's torch CPU path
    same(C[0], orc.gemm_wrap64(X[0], W.astype(np.int64), 16), "wrap64")


@pytest.mark.parametrize("algo", ["exact", "auto"])
@pytest.mark.parametrize("shape", [(1, 1, 1, 1), (2, 5, 37, 7), (1, 130, 200, 70), (3, 64, 128, 64),
                                   (1, 257, 1000, 129), (1, 128, 4096, 256)])
@pytest.mark.parametrize("s,a_r,b_r,abits,bbits,b32", [
    (16, 1, 1, 20, 15, True), (30, 1, 1, 36, 31, True), (29, 1, 256, 30, 43, False),
    (33, 3, -7, 62, 62, False), (0, 1, 1, 8, 8, True), (64, 1, 1, 62, 31, True),
    (100, 1, 1, 62, 62, False)])
def test_gemm_shapes_ranges_shifts(kmod, orc, dev, algo, shape, s, a_r, b_r, abits, bbits, b32):
    Bd, M, K, N = shape
    rng = np.random.default_rng(M * 131 + K + s)
    A = rand_i64(rng, (Bd, M, K), abits)
    B = rand_i64(rng, (N, K), bbits)
    if b32:
        B = B.astype(np.int32)
    kmod.ALGO = kmod.ALGO_EXACT if algo == "exact" else kmod.ALGO_AUTO
    try:
        for legacy in (True, False):
            kmod.LEGACY_REMAINDER = legacy
            C, R = kmod.int64_bmm_broadcast(g(A, dev), g(B, dev), a_r, b_r, s)
            Co, Ro = orc.gemm(A, B, a_r, b_r, s, orc.R_LEGACY if legacy else orc.R_MATH)
            same(C, Co, "C")
            same(R, Ro, "R legacy=%s" % legacy)
    finally:
        kmod.ALGO = kmod.ALGO_AUTO
        kmod.LEGACY_REMAINDER = True


def test_gemm_extreme_values(kmod, orc, dev):
    """INT64_MIN / INT32_MIN operands and sums that straddle 2^63 and 2^127."""
    A = np.array([[[np.iinfo(np.int64).min, np.iinfo(np.int64).max, -1, 0, 1, 2**62, -2**62, 7]]],
                 np.int64).repeat(3, 1)
    B = np.array([[np.iinfo(np.int32).min] * 8, [np.iinfo(np.int32).max] * 8,
                  [1, -1, 1, -1, 1, -1, 1, -1]], np.int32)
    for s in (0, 1, 31, 63):
        C, R = kmod.int64_bmm_broadcast(g(A, dev), g(B, dev), 1, 1, s)
        Co, Ro = orc.gemm(A, B, 1, 1, s, orc.R_LEGACY)
        same(C, Co)
        same(R, Ro)


def test_gemm_empty(kmod, dev):
    A = torch.zeros((1, 0, 16), dtype=torch.int64, device=dev)
    B = torch.zeros((4, 16), dtype=torch.int32, device=dev)
    C, R = kmod.int64_bmm_broadcast(A, B, 1, 1, 3)
    assert C.shape == (1, 0, 4)
    A = torch.ones((1, 2, 0), dtype=torch.int64, device=dev)
    B = torch.zeros((4, 0), dtype=torch.int32, device=dev)
    C, R = kmod.int64_bmm_broadcast(A, B, 1, 1, 3)
    assert not C.any() and not R.any()


def test_gemm_rejects_bad_arguments(kmod, dev):
    A = torch.zeros((1, 2, 4), dtype=torch.int64, device=dev)
    B = torch.zeros((4, 4), dtype=torch.int32, device=dev)
    with pytest.raises(kmod.ZkdsError):
        kmod.int64_bmm_broadcast(A, B, 0, 1, 3)      # zero divisor
    with pytest.raises(kmod.ZkdsError):
        kmod.int64_bmm_broadcast(A, B, 1, 1, 200)    # shift out of range
    with pytest.raises(TypeError):
        kmod.int64_bmm_broadcast(A, B.to(torch.int16), 1, 1, 3)


# ---- the four MLA einsums ------------------------------------------------------------------

@pytest.mark.parametrize("algo", ["exact", "auto"])
@pytest.mark.parametrize("dims", [(1, 3, 2, 8, 16, 5), (2, 7, 3, 128, 512, 33),
                                  (1, 64, 16, 128, 512, 200)])
def test_einsums(kmod, orc, dev, algo, dims):
    Bn, S, H, D, C, T = dims
    rng = np.random.default_rng(S + H)
    q = rand_i64(rng, (Bn, S, H, D), 30)
    W1 = rand_i64(rng, (H, D, C), 31).astype(np.int32)
    A = rand_i64(rng, (Bn, S, H, C), 34)
    KV = rand_i64(rng, (Bn, T, C), 30)
    P = rng.integers(0, 2**19 + 1, (Bn, S, H, T), dtype=np.int64)
    W2 = rand_i64(rng, (H, D, C), 31).astype(np.int32)
    kmod.ALGO = kmod.ALGO_EXACT if algo == "exact" else kmod.ALGO_AUTO
    try:
        same(kmod.einsum_bshd_hdc_bshc(g(q, dev), g(W1, dev), 33),
             orc.einsum_bshd_hdc_bshc(q, W1, 33), "bshd,hdc->bshc")
        same(kmod.einsum_bshc_btc_bsht(g(A, dev), g(KV, dev), 23),
             orc.einsum_bshc_btc_bsht(A, KV, 23), "bshc,btc->bsht")
        same(kmod.einsum_bsht_btc_bshc(g(P, dev), g(KV, dev), 23),
             orc.einsum_bsht_btc_bshc(P, KV, 23), "bsht,btc->bshc")
        same(kmod.einsum_bshc_hdc_bshd(g(A, dev), g(W2, dev), 30),
             orc.einsum_bshc_hdc_bshd(A, W2, 30), "bshc,hdc->bshd")
    finally:
        kmod.ALGO = kmod.ALGO_AUTO


@pytest.mark.parametrize("dims,bits", [((1, 40, 4, 40, 128, 64), (20, 20)), ((2, 5, 3, 37, 512, 64), (30, 23)),
                                       ((1, 200, 16, 333, 512, 64), (34, 30)), ((1, 3, 2, 9, 256, 16), (16, 16))])
def test_mla_scores_in_one_pass(kmod, orc, dev, dims, bits):
    """(einsum(q_abs, kv) >> 23 + einsum(q_pe, pe) >> 21) * 94 // 695 + causal mask, fused
    (model.py:884-905), against the two oracle einsums and numpy's floor division"""
    Bn, S, H, T, C1, C2 = dims
    rng = np.random.default_rng(T)
    qa = rand_i64(rng, (Bn, S, H, C1), bits[0])
    kv = rand_i64(rng, (Bn, T, C1), bits[1])
    qp = rand_i64(rng, (Bn, S, H, C2), bits[0])
    pe = rand_i64(rng, (Bn, T, C2), bits[1])
    base = (orc.einsum_bshc_btc_bsht(qa, kv, 23) + orc.einsum_bshc_btc_bsht(qp, pe, 21)) * 94 // 695
    for causal in (False, True):
        want = base
        if causal:
            mask = np.where(np.arange(T)[None, :] > np.arange(S)[:, None], -(64 << 36), 0).astype(np.int64)
            want = base + mask[None, :, None, :]
        for (al, bl, dyn) in ((0, 0, False), (5, 5, True), (5, 4, False)):
            got = kmod.mla_scores_fused(g(qa, dev), g(kv, dev), g(qp, dev), g(pe, dev), causal=causal,
                                        a_limbs=al, b_limbs=bl, dynamic=dyn)
            assert got is not None, "the fused kernel should take this shape"
            same(got, want, "causal=%s limbs=%s" % (causal, (al, bl)))
    kmod.device_status()


@pytest.mark.parametrize("dims", [(1, 40, 4, 40, 128, 64), (2, 300, 2, 300, 256, 64), (1, 130, 16, 130, 512, 64)])
def test_causal_skip_pipeline(kmod, orc, dev, dims):
    """scores with masked tiles skipped -> causal softmax -> causal P.KV gives the same context
    tensor as the reference's fully materialised path; the unmasked scores and probabilities match"""
    Bn, S, H, T, C1, C2 = dims
    rng = np.random.default_rng(S + H)
    qa = rand_i64(rng, (Bn, S, H, C1), 22)
    kv = rand_i64(rng, (Bn, T, C1), 23)
    qp = rand_i64(rng, (Bn, S, H, C2), 21)
    pe = rand_i64(rng, (Bn, T, C2), 21)
    mask = np.where(np.arange(T)[None, :] > np.arange(S)[:, None], -(64 << 36), 0).astype(np.int64)
    scores = (orc.einsum_bshc_btc_bsht(qa, kv, 23) + orc.einsum_bshc_btc_bsht(qp, pe, 21)) * 94 // 695 \
        + mask[None, :, None, :]
    probs = orc.softmax(scores, 19)
    ctx = orc.einsum_bsht_btc_bshc(probs, kv, 23)
    keep = np.broadcast_to((mask == 0)[None, :, None, :], scores.shape)

    kmod.softmax_init_q19()
    kvd = g(kv, dev)
    got_s = kmod.mla_scores_fused(g(qa, dev), kvd, g(qp, dev), g(pe, dev), causal=True, a_limbs=4, b_limbs=4,
                                  dynamic=True, skip_masked=True)
    assert got_s is not None
    assert np.array_equal(got_s.cpu().numpy()[keep], scores[keep])
    got_p = torch.full_like(got_s, 77)
    assert kmod.softmax_q19_causal(got_s, got_p, 0)
    gp = got_p.cpu().numpy()
    assert np.array_equal(gp[keep], probs[keep])
    got_c = kmod.einsum_bsht_btc_bshc_causal(got_p, kvd, 23, 0, a_limbs=3, b_limbs=4)
    same(got_c, ctx, "context")
    # softmax and P.KV in one call, reading only the owned columns of the skipped scores
    if T % 4 == 0:
        fused = kmod.softmax_pv_fused(got_s, kvd, 23, causal_skip=True, start_pos=0, a_limbs=3, b_limbs=4)
        assert fused is not None
        same(fused, ctx, "context, fused softmax")
    kmod.device_status()


@pytest.mark.parametrize("dims", [(1, 5, 3, 4, 16), (2, 33, 4, 100, 128), (1, 64, 8, 1024, 512),
                                  (1, 3, 2, 4100, 64), (1, 2, 2, 8176, 32)])
def test_softmax_then_pv_in_one_call(kmod, orc, dev, dims):
    """softmax_q19 -> einsum_bsht_btc_bshc with the probabilities kept as int8 limb planes
    (model.py:911-926) against the two oracle steps"""
    Bn, S, H, T, C = dims
    rng = np.random.default_rng(T + C)
    scores = np.rint(rng.standard_normal((Bn, S, H, T)) * 2.0**21).astype(np.int64)
    scores[:, :, :, T // 2:] -= rng.integers(0, 70 << 19, (Bn, S, H, T - T // 2))
    scores[0, 0, 0, :] = -(64 << 36)              # a fully masked row: uniform weights
    if S > 1:
        scores[0, 1, 0, 1:] = -(64 << 36)         # one live column: probability 2^19
    kv = rand_i64(rng, (Bn, T, C), 24)
    want = orc.einsum_bsht_btc_bshc(orc.softmax(scores, 19), kv, 23)
    kmod.softmax_init_q19()
    sd = g(scores, dev)
    for al, bl in ((0, 0), (3, 4), (4, 5)):
        got = kmod.softmax_pv_fused(sd, g(kv, dev), 23, a_limbs=al, b_limbs=bl)
        assert got is not None
        same(got, want, "limbs %s" % ((al, bl),))
    same(sd, scores, "scores untouched")
    kmod.device_status()
    # shapes the fused kernel declines
    z = torch.zeros((1, 1, 1, 6), dtype=torch.int64, device=dev)
    assert kmod.softmax_pv_fused(z, torch.zeros((1, 6, 8), dtype=torch.int64, device=dev)) is None


def test_mla_scores_fused_declines_other_shapes(kmod, dev):
    z = lambda *s: torch.zeros(s, dtype=torch.int64, device=dev)
    assert kmod.mla_scores_fused(z(1, 2, 2, 64), z(1, 4, 64), z(1, 2, 2, 16), z(1, 4, 16)) is None


# ---- RoPE -------------------------------------------------------------------------------------

def rope_table(S, pairs, frac, base=10000.0):
    freqs = 1.0 / (base ** (np.arange(0, 2 * pairs, 2, dtype=np.float64) / (2 * pairs)))
    ang = np.outer(np.arange(S), freqs)
    return np.stack([np.rint(np.cos(ang) * 2.0**frac), np.rint(np.sin(ang) * 2.0**frac)],
                    -1).astype(np.int64)


@pytest.mark.parametrize("shape", [(1, 256, 128, 32), (2, 5, 1, 32), (1, 3, 7, 3), (1, 1, 1, 1)])
@pytest.mark.parametrize("shift", [42, 16])
def test_rope(kmod, orc, dev, shape, shift):
    Bn, S, H, P = shape
    rng = np.random.default_rng(S)
    A = np.rint(rng.standard_normal((Bn, S, H, P, 2)) * 2**16).astype(np.int64)
    A.flat[:7] = [2**62, -2**62, 2**63 - 1, -2**63, 0, 1, -1][:A.size][:min(7, A.size)]
    if A.size > 4000:       # magnitudes on both sides of the kernel's one-word multiply bound
        for k, bits in enumerate((18, 19, 20, 21, 22, 23, 30, 45)):
            A.flat[100 + 400 * k:500 + 400 * k] = rand_i64(rng, 400, bits)
    T = rope_table(S, P, shift)
    C = kmod.complex_int64_mul_broadcast(g(A, dev), g(T.reshape(1, S, 1, P, 2), dev), shift)
    same(C, orc.rope(A, T, shift))


# ---- RMSNorm ------------------------------------------------------------------------------------

@pytest.mark.parametrize("M,N,bits,wdt", [(64, 7168, 17, np.int32), (33, 1536, 37, np.int32),
                                          (5, 512, 50, np.int64), (3, 7, 3, np.int32), (1300, 1536, 20, np.int32),
                                          (700, 7168, 33, np.int64),
                                          (2, 30001, 31, np.int64)])
def test_rms_norm(kmod, orc, dev, M, N, bits, wdt):
    rng = np.random.default_rng(N)
    A = np.rint(rng.standard_normal((M, N)) * 2.0**bits).astype(np.int64)
    A[0, :] = 0                                    # all-zero row: rms 0, defined as zeros
    if M > 1:
        A[1, ::2] = -A[1, ::2]
    W = (2**16 + np.rint(rng.standard_normal(N) * 2**8)).astype(wdt)
    W[: min(4, N)] = [-3, 0, 2**30, -2**30][: min(4, N)]
    C, rms = kmod.RMS_Norm_int64(g(A, dev), g(W, dev), 1, N)
    Co, rmso = orc.rms_norm(A, W, 1, N)
    assert rms.device.type == "cpu" and rms.numel() >= 500
    same(rms[:M], rmso, "rms")
    same(C, Co, "C")
    # caller-provided rms (the reference's rms_norm_32/64 entry points)
    given = np.maximum(rmso, 1) + 3
    same(kmod.rms_norm_apply(g(A, dev), g(W, dev), g(given, dev)), orc.rms_norm_given(A, W, given))


# ---- softmax ------------------------------------------------------------------------------------

@pytest.mark.parametrize("frac", [19, 21])
@pytest.mark.parametrize("shape", [(1, 32, 8, 2048), (1, 3, 2, 37), (1, 2, 1, 1), (1, 1, 2, 30000)])
def test_softmax(kmod, orc, dev, frac, shape):
    rng = np.random.default_rng(shape[-1] + frac)
    X = np.rint(rng.standard_normal(shape) * 4 * 2.0**frac).astype(np.int64)
    T = shape[-1]
    if T > 8:
        S = shape[1]
        mask = np.triu(np.full((S, T), -(64 << 36), np.int64), T - S + 1)   # causal, model.py:1555
        X += mask[None, :, None, :]
        X[0, 0, 0, :] = 123                                                     # constant row
    (kmod.softmax_init_q19 if frac == 19 else kmod.softmax_init_q21)()
    fn = kmod.softmax_q19 if frac == 19 else kmod.softmax_q21
    Xd = g(X, dev)
    C = torch.empty_like(Xd)
    fn(Xd, C)
    Co, Wo = orc.softmax(X, frac, want_weights=True)
    same(C, Co, "probabilities")
    same(Xd, Wo, "input buffer holds the weights afterwards")
    kmod.SOFTMAX_WRITES_WEIGHTS = False
    try:
        Xd = g(X, dev)
        C = torch.empty_like(Xd)
        fn(Xd, C)
        same(C, Co)
        same(Xd, X, "input untouched")
    finally:
        kmod.SOFTMAX_WRITES_WEIGHTS = True


# ---- SiLU / sigmoid -------------------------------------------------------------------------------

@pytest.mark.parametrize("frac", [23, 25])
def test_activations(kmod, orc, dev, frac):
    LIM = 64 << frac
    rng = np.random.default_rng(frac)
    X = np.concatenate([
        np.array([0, 1, -1, LIM - 1, LIM, LIM + 1, -LIM + 1, -LIM, -LIM - 1, 2**62, -2**62,
                  np.iinfo(np.int64).min, np.iinfo(np.int64).max]),
        rng.integers(-LIM, LIM, 100000),
        rng.integers(-LIM, -20 * 2**frac, 100000),
        np.rint(rng.standard_normal(300001) * 2.0**frac).astype(np.int64),
        np.rint(rng.standard_normal(100000) * 2.0**16).astype(np.int64),
    ]).astype(np.int64)
    (kmod.silu_init_q23 if frac == 23 else kmod.silu_init_q25)()
    silu = kmod.silu_q23 if frac == 23 else kmod.silu_q25
    sigm = kmod.sigmoid_q23 if frac == 23 else kmod.sigmoid_q25
    for view in (X.reshape(1, 1, -1), X[:-2].reshape(1, 2, -1), X[1:]):
        Xd = g(view, dev)
        C = torch.empty_like(Xd)
        silu(Xd, C)
        same(C, orc.act(view, "silu", frac), "silu")
        sigm(Xd, C)
        same(C, orc.act(view, "sigmoid", frac), "sigmoid")


# ---- expert plumbing: gated product, row gather, weighted combine ---------------------------------

def test_glu_gather_combine(kmod, orc, dev):
    rng = np.random.default_rng(77)
    rows, n = 37, 258
    r12 = np.rint(rng.standard_normal((rows, 2 * n)) * 2.0**24).astype(np.int64)
    r12[0, :4] = [64 << 23, -(64 << 23), (64 << 23) - 1, 0]
    d = g(r12, dev)
    kmod.silu_init_q23()
    h, s1 = kmod.glu_q23(d[:, :n], d[:, n:], ld=2 * n, want_silu=True)
    want_s = orc.act(np.ascontiguousarray(r12[:, :n]), "silu", 23)
    same(s1, want_s, "silu part")
    same(h, (want_s * r12[:, n:]) >> 23, "gated product")

    src = rand_i64(rng, (19, 64), 62)
    index = rng.integers(-1, 19, 50).astype(np.int32)
    got = kmod.gather_rows(g(src, dev), torch.from_numpy(index).to(dev))
    same(got, np.where(index[:, None] >= 0, src[np.maximum(index, 0)], 0), "gather")
    # a source without rows (an expert-parallel rank that received nothing): all padding
    got = kmod.gather_rows(torch.empty((0, 64), dtype=torch.int64, device=dev),
                           torch.full((128,), -1, dtype=torch.int32, device=dev))
    assert got.shape == (128, 64) and int(got.abs().sum()) == 0

    tokens, slots, cols = 23, 8, 96
    out = rand_i64(rng, (tokens * slots + 5, cols), 38)
    pos = rng.permutation(tokens * slots + 5)[:tokens * slots].reshape(tokens, slots).astype(np.int32)
    w = rng.integers(0, 5 << 22, (tokens, slots)).astype(np.int64)
    base = rand_i64(rng, (tokens, cols), 40)
    y = kmod.moe_combine(g(out, dev), torch.from_numpy(pos).to(dev), g(w, dev), g(base, dev))
    want = base.copy()
    for t in range(tokens):
        for sl in range(slots):
            want[t] += out[pos[t, sl]] * w[t, sl] // (1 << 23)
    same(y, want, "combine")


@pytest.mark.parametrize("rows,n,N", [(37, 258, 70), (256, 2048, 96), (5, 16, 8)])
def test_gated_mlp_tail_in_one_call(kmod, orc, dev, rows, n, N):
    """(silu_q23(r1) * r2) >> 23 followed by w2 (model.py:1034-1049) with the gated product kept as limb
    planes, against the oracle's activation and GEMM; plain and grouped (expert) form"""
    rng = np.random.default_rng(rows + n)
    r12 = np.rint(rng.standard_normal((rows, 2 * n)) * 2.0**24).astype(np.int64)
    r12[0, :4] = [64 << 23, -(64 << 23), (64 << 23) - 1, 0]
    W2 = rand_i64(rng, (N, n), 30).astype(np.int32)
    h = (orc.act(np.ascontiguousarray(r12[:, :n]), "silu", 23) * r12[:, n:]) >> 23
    want, _ = orc.gemm(h[None], W2, 1, 1, 31)
    d = g(r12, dev)
    kmod.silu_init_q23()
    got = kmod.glu_prepared(d[:, :n], d[:, n:], kmod.WeightPlanes(g(W2, dev)), 31, ld=2 * n, a_limbs=5)
    assert got is not None
    same(got, want[0], "gate + down projection")
    if rows == 256:      # two expert tiles with their own weights and shifts, one unused tile in between
        W = np.stack([W2, rand_i64(rng, (N, n), 30).astype(np.int32)])
        tg = torch.tensor([1, -1, 0], dtype=torch.int32, device=dev)
        sh = g(np.array([[29, 29], [33, 33]], np.int32), dev)
        pad = np.concatenate([r12[:128], np.zeros((128, 2 * n), np.int64), r12[128:]])
        dp = g(pad, dev)
        got = kmod.glu_prepared(dp[:, :n], dp[:, n:], kmod.WeightPlanes(g(W, dev)), 0, ld=2 * n, a_limbs=5,
                                tile_group=tg, group_shift=sh, n_split=0)
        assert got is not None
        want_g = np.zeros((384, N), np.int64)
        want_g[:128] = orc.gemm(h[None, :128], W[1], 1, 1, 33)[0][0]
        want_g[256:] = orc.gemm(h[None, 128:], W[0], 1, 1, 29)[0][0]
        same(got, want_g, "grouped gate + down projection")
    torch.cuda.synchronize()
    kmod.device_status()


def test_grouped_expert_gemm_with_and_without_fused_gather(kmod, orc, dev):
    """all experts of a routed layer in one launch (model.py:1372-1378): rows grouped by expert in
    128-row tiles, per-expert shifts left / right of n_split; the row gather as a separate pass and
    folded into the limb split give the oracle's per-expert GEMMs"""
    rng = np.random.default_rng(5)
    E, N, Kd, T = 5, 96, 200, 300
    W = rand_i64(rng, (E, N, Kd), 30).astype(np.int32)
    x = rand_i64(rng, (T, Kd), 20)
    shifts = rng.integers(10, 34, (E, 2)).astype(np.int32)
    n_split = 40
    expert_of = rng.integers(0, E, T)
    expert_of[expert_of == 3] = 2                       # expert 3 gets no token
    row_src, tile_group = [], []
    for e in range(E):
        toks = np.nonzero(expert_of == e)[0]
        for t0 in range(0, len(toks), 128):
            part = toks[t0:t0 + 128]
            row_src += part.tolist() + [-1] * (128 - len(part))
            tile_group.append(e)
    tile_group.append(-1)                               # an unused tile: its output rows are zeros
    row_src += [-1] * 128
    row_src = np.array(row_src, np.int32)
    tile_group = np.array(tile_group, np.int32)
    want = np.zeros((len(row_src), N), np.int64)
    for i, e in enumerate(tile_group):
        if e < 0:
            continue
        rows = row_src[i * 128:(i + 1) * 128]
        xe = np.where(rows[:, None] >= 0, x[np.maximum(rows, 0)], 0)
        lo, _ = orc.gemm(xe[None], W[e, :n_split], 1, 1, int(shifts[e, 0]))
        hi, _ = orc.gemm(xe[None], W[e, n_split:], 1, 1, int(shifts[e, 1]))
        want[i * 128:(i + 1) * 128] = np.concatenate([lo[0], hi[0]], 1)
    planes = kmod.WeightPlanes(g(W, dev))
    xd, rs, tg, sh = g(x, dev), torch.from_numpy(row_src).to(dev), torch.from_numpy(tile_group).to(dev), g(shifts, dev)
    separate = kmod.grouped_prepared(kmod.gather_rows(xd, rs), planes, tg, 0, a_limbs=3, dynamic=True,
                                     group_shift=sh, n_split=n_split)
    same(separate, want, "gather pass + grouped GEMM")
    fused = kmod.grouped_prepared(xd, planes, tg, 0, a_limbs=3, dynamic=True, group_shift=sh, n_split=n_split,
                                  row_index=rs)
    same(fused, want, "gather folded into the split")
    torch.cuda.synchronize()
    kmod.device_status()


@pytest.mark.parametrize("T", [7, 32, 64])
def test_grouped_expert_gemm_with_few_rows_per_expert(kmod, orc, dev, T):
    """decode: every expert receives a handful of rows (at most one per token).  With the caller's bound on
    the rows of a group the kernel fetches only the first 32 / 64 rows of every 128-row tile; the result,
    padding rows included, is that of the launch without the bound and the oracle's, for the first expert GEMM
    (fused gather, deep K) and for the gated down projection (zkds_glu_prepared)."""
    rng = np.random.default_rng(50 + T)
    E, I, Kd, k = 12, 1040, 1100, 4        # both contractions deeper than the persistent kernel takes
    W13 = rand_i64(rng, (E, 2 * I, Kd), 15).astype(np.int32)
    W2 = rand_i64(rng, (E, 80, I), 15).astype(np.int32)
    x = rand_i64(rng, (T, Kd), 12)          # keeps the gated product within the three limbs promised below
    # every token names k distinct experts; expert E-1 stays empty
    choice = np.stack([rng.choice(E - 1, k, replace=False) for _ in range(T)])
    row_src, tile_group = [], []
    for e in range(E):
        toks = np.nonzero((choice == e).any(1))[0]
        if len(toks) == 0:
            continue
        assert len(toks) <= T
        row_src += toks.tolist() + [-1] * (128 - len(toks))
        tile_group.append(e)
    tile_group.append(-1)
    row_src += [-1] * 128
    row_src, tile_group = np.array(row_src, np.int32), np.array(tile_group, np.int32)
    sh13 = rng.integers(12, 20, (E, 2)).astype(np.int32)
    sh2 = np.repeat(rng.integers(10, 18, (E, 1)), 2, axis=1).astype(np.int32)
    want13 = np.zeros((len(row_src), 2 * I), np.int64)
    want2 = np.zeros((len(row_src), 80), np.int64)
    for i, e in enumerate(tile_group):
        if e < 0:
            continue
        rows = row_src[i * 128:(i + 1) * 128]
        xe = np.where(rows[:, None] >= 0, x[np.maximum(rows, 0)], 0)
        lo, _ = orc.gemm(xe[None], W13[e, :I], 1, 1, int(sh13[e, 0]))
        hi, _ = orc.gemm(xe[None], W13[e, I:], 1, 1, int(sh13[e, 1]))
        want13[i * 128:(i + 1) * 128] = np.concatenate([lo[0], hi[0]], 1)
        h = (orc.act(np.ascontiguousarray(lo), "silu", 23) * hi) >> 23
        want2[i * 128:(i + 1) * 128] = orc.gemm(h, W2[e], 1, 1, int(sh2[e, 0]))[0][0]
    p13, p2 = kmod.WeightPlanes(g(W13, dev)), kmod.WeightPlanes(g(W2, dev))
    xd, rs, tg = g(x, dev), torch.from_numpy(row_src).to(dev), torch.from_numpy(tile_group).to(dev)
    s13, s2 = g(sh13, dev), g(sh2, dev)
    kmod.silu_init_q23()
    for bound in (None, T):
        r13 = kmod.grouped_prepared(xd, p13, tg, 0, a_limbs=3, dynamic=True, group_shift=s13, n_split=I,
                                    row_index=rs, max_group_rows=bound)
        same(r13, want13, "w13, bound %s" % bound)
        out = kmod.glu_prepared(r13[:, :I], r13[:, I:], p2, 0, ld=2 * I, a_limbs=3, dynamic=True, tile_group=tg,
                                group_shift=s2, n_split=0, max_group_rows=bound)
        assert out is not None
        same(out, want2, "w2, bound %s" % bound)
    torch.cuda.synchronize()
    kmod.device_status()


# ---- the reference's own symbol names, and the reference's own kernels ------------------------------

def test_reference_symbols_against_reference_kernels(libpath, reflib, orc, dev):
    """Calls the 21-symbol ABI of both libraries with the same raw pointers, the way the
    reference's kernel.py does, inside the reference's limits."""
    ours = type(reflib)(libpath).lib
    ref = reflib.lib
    rng = np.random.default_rng(11)

    def z(shape):
        return torch.zeros(shape, dtype=torch.int64, device=dev)

    def both(name, args_fn, outs):
        res = []
        for L in (ours, ref):
            bufs = [z(o) for o in outs]
            getattr(L, name)(*args_fn(bufs))
            torch.cuda.synchronize()
            res.append([b.cpu().numpy() for b in bufs])
        for a, b in zip(*res):
            assert np.array_equal(a, b), name
        return res[0]

    A = g(rand_i64(rng, (2, 40, 300), 36), dev)
    B32 = g(rand_i64(rng, (50, 300), 31).astype(np.int32), dev)
    B64 = g(rand_i64(rng, (50, 300), 43), dev)
    for s in (16, 30, 31, 32, 33, 37):
        both("int64_32_bmm_broadcast_launcher",
             lambda o: (A.data_ptr(), B32.data_ptr(), o[0].data_ptr(), o[1].data_ptr(), 1, 1, s, 2, 40,
                        300, 50), [(2, 40, 50)] * 2)
    both("int64_64_bmm_broadcast_launcher",
         lambda o: (A.data_ptr(), B64.data_ptr(), o[0].data_ptr(), o[1].data_ptr(), 1, 256, 29, 2, 40,
                    300, 50), [(2, 40, 50)] * 2)

    q = g(rand_i64(rng, (1, 9, 4, 128), 30), dev)
    W1 = g(rand_i64(rng, (4, 128, 512), 31).astype(np.int32), dev)
    Ae = g(rand_i64(rng, (1, 9, 4, 512), 34), dev)
    KV = g(rand_i64(rng, (1, 100, 512), 30), dev)
    P = g(rng.integers(0, 2**19, (1, 9, 4, 100), dtype=np.int64), dev)
    both("einsum_bshd_hdc_bshc", lambda o: (q.data_ptr(), W1.data_ptr(), o[0].data_ptr(), 33, 1, 9, 4,
                                            128, 512), [(1, 9, 4, 512)])
    both("einsum_bshc_btc_bsht", lambda o: (Ae.data_ptr(), KV.data_ptr(), o[0].data_ptr(), 23, 1, 9, 4,
                                            100, 512), [(1, 9, 4, 100)])
    both("einsum_bsht_btc_bshc", lambda o: (P.data_ptr(), KV.data_ptr(), o[0].data_ptr(), 23, 1, 9, 4,
                                            100, 512), [(1, 9, 4, 512)])
    both("einsum_bshc_hdc_bshd", lambda o: (Ae.data_ptr(), W1.data_ptr(), o[0].data_ptr(), 30, 1, 9, 4,
                                            128, 512), [(1, 9, 4, 128)])

    Ar = g(rand_i64(rng, (1, 50, 16, 32, 2), 30), dev)
    Tr = g(rope_table(50, 32, 42), dev)
    both("complex_int64_mul", lambda o: (Ar.data_ptr(), Tr.data_ptr(), o[0].data_ptr(), 1, 50, 16, 32),
         [(1, 50, 16, 32, 2)])

    An = rand_i64(rng, (20, 1536), 37)
    Wn = (2**19 + rand_i64(rng, (1536,), 10)).astype(np.int32)
    rms = g(orc.rms_rows(An, 1, 1536), dev)
    And, Wnd = g(An, dev), g(Wn, dev)
    both("rms_norm_32", lambda o: (And.data_ptr(), Wnd.data_ptr(), rms.data_ptr(), o[0].data_ptr(), 20,
                                   1536), [(20, 1536)])
    Wn64 = g(Wn.astype(np.int64) << 12, dev)
    both("rms_norm_64", lambda o: (And.data_ptr(), Wn64.data_ptr(), rms.data_ptr(), o[0].data_ptr(), 20,
                                   1536), [(20, 1536)])

    for frac in (19, 21):
        lut = torch.zeros(256, dtype=torch.int64)
        getattr(ours, "softmax_init_q%d" % frac)(lut.data_ptr())
        lut = lut.to(dev)
        X = np.rint(rng.standard_normal((1, 6, 8, 333)) * 4 * 2.0**frac).astype(np.int64)
        outs = []
        for L in (ours, ref):
            Xd, C = g(X, dev), z(X.shape)
            getattr(L, "softmax_q%d" % frac)(Xd.data_ptr(), C.data_ptr(), lut.data_ptr(), 1, 6, 8, 333)
            torch.cuda.synchronize()
            outs.append((C.cpu().numpy(), Xd.cpu().numpy()))
        assert np.array_equal(outs[0][0], outs[1][0]) and np.array_equal(outs[0][1], outs[1][1])

    for frac in (23, 25):
        lut = torch.zeros(256, dtype=torch.int64)
        getattr(ours, "silu_init_q%d" % frac)(lut.data_ptr())
        lut = lut.to(dev)
        LIM = 64 << frac
        X = g(np.concatenate([rng.integers(-LIM + 1, LIM, 5000),
                              rng.integers(-LIM + 1, -20 * 2**frac, 5000)]).reshape(1, 2, 5000), dev)
        for name in ("silu_q%d" % frac, "sigmoid_q%d" % frac):
            both(name, lambda o: (X.data_ptr(), o[0].data_ptr(), lut.data_ptr(), 1, 2, 5000),
                 [(1, 2, 5000)])


def test_golden_vectors_from_the_reference_replay_on_the_gpu(kmod, orc, dev):
    """The committed reference-kernel outputs also hold for the CUDA path (via the oracle's
    replay helper, with the GPU library standing in for the oracle)."""
    import os
    import sys
    from conftest import ROOT
    path = os.path.join(ROOT, "tests", "golden", "ref_gpu_vectors.npz")
    if not os.path.exists(path):
        pytest.skip("ref_gpu_vectors.npz not generated yet")
    sys.path.insert(0, os.path.join(ROOT, "tests", "golden"))
    import make_gpu_golden as mk

    class GpuAsOracle:
        R_LEGACY, R_MATH = 1, 0

        def gemm(self, A, B, a_r, b_r, s, rmode):
            kmod.LEGACY_REMAINDER = bool(rmode)
            C, R = kmod.int64_bmm_broadcast(g(A, dev), g(B, dev), a_r, b_r, s)
            kmod.LEGACY_REMAINDER = True
            return C.cpu().numpy(), R.cpu().numpy()

        def rope(self, A, T, shift):
            S, P = T.shape[0], T.shape[1]
            return kmod.complex_int64_mul_broadcast(g(A, dev), g(T.reshape(1, S, 1, P, 2), dev),
                                                    shift).cpu().numpy()

        def rms_norm_given(self, A, W, rms):
            return kmod.rms_norm_apply(g(A, dev), g(W, dev), g(rms, dev)).cpu().numpy()

        def softmax(self, X, frac, want_weights=False):
            (kmod.softmax_init_q19 if frac == 19 else kmod.softmax_init_q21)()
            Xd = g(X, dev)
            C = torch.empty_like(Xd)
            (kmod.softmax_q19 if frac == 19 else kmod.softmax_q21)(Xd, C)
            return C.cpu().numpy(), Xd.cpu().numpy()

        def act(self, X, kind, frac):
            (kmod.silu_init_q23 if frac == 23 else kmod.silu_init_q25)()
            Xd = g(X, dev)
            C = torch.empty_like(Xd)
            getattr(kmod, "%s_q%d" % (kind, frac))(Xd, C)
            return C.cpu().numpy()

        def __getattr__(self, name):
            if name.startswith("einsum_"):
                return lambda A, B, r: getattr(kmod, name)(g(A, dev), g(B, dev), r).cpu().numpy()
            raise AttributeError(name)

    bad = mk.check_against(np.load(path), GpuAsOracle())
    assert not bad, bad


# ---- small M: the weight-streaming shapes (BASELINE config 1, decode) ----------------------------

@pytest.mark.parametrize("M", [1, 7, 32, 64])
@pytest.mark.parametrize("K,N", [(7168, 576), (2048, 1536), (1536, 200)])
@pytest.mark.parametrize("abits,bbits,s", [(20, 15, 16), (36, 31, 30), (47, 31, 33)])
def test_small_m_gemm_split_over_k(kmod, orc, dev, M, K, N, abits, bbits, s):
    """Few output tiles and a deep K: the K range is split over CTAs that add their int32 diagonals before
    the shift.  Sums reach 2^80 (beyond int64) in the wide ranges.  Through prepared planes (promised and
    measured limb counts) and through the reference symbol's wrapper, twice each: the second call finds the
    partial-sum scratch as the first one left it."""
    rng = np.random.default_rng(M * 7 + K + N + s)
    A = rand_i64(rng, (1, M, K), abits)
    B = rand_i64(rng, (N, K), bbits).astype(np.int32)
    Co, Ro = orc.gemm(A, B, 1, 1, s, orc.R_LEGACY)
    Ad, Bd = g(A, dev), g(B, dev)
    planes = kmod.WeightPlanes(Bd)
    la = (abits + 8) // 8                  # signed 8-bit limbs that cover |x| < 2^abits
    for rep in range(2):
        C, R = kmod.int64_bmm_broadcast(Ad, Bd, 1, 1, s)
        same(C, Co, "legacy C, call %d" % rep)
        same(R, Ro, "legacy R, call %d" % rep)
        if la <= 5:
            C, R = kmod.linear_prepared(Ad, planes, s, a_limbs=la, want_remainder=True, dynamic=True)
            same(C, Co, "prepared dynamic C, call %d" % rep)
            same(R, Ro, "prepared dynamic R, call %d" % rep)
            C = kmod.linear_prepared(Ad, planes, s, a_limbs=0)
            same(C, Co, "prepared measured C, call %d" % rep)
        # (wider activations do not fit the tensor-core kernel's shared memory; with prepared planes there is no
        # other kernel to fall back to, the reference-named wrapper above falls back to the exact one)
    kmod.device_status()


def test_small_m_gemm_batched_and_int64_weights(kmod, orc, dev):
    """batch > 1 with a shared int64 weight and divisors (the head projection's form, model.py:1517-1519),
    interleaved with a shape of another tile geometry so that the shared partial-sum scratch is reused
    under a different layout"""
    rng = np.random.default_rng(77)
    A = rand_i64(rng, (3, 9, 3000), 30)
    B = rand_i64(rng, (333, 3000), 43)
    A2 = rand_i64(rng, (1, 64, 7168), 21)
    B2 = rand_i64(rng, (1536, 7168), 17).astype(np.int32)
    want = orc.gemm(A, B, 1, 256, 29, orc.R_LEGACY)
    want2 = orc.gemm(A2, B2, 1, 1, 30, orc.R_LEGACY)
    for rep in range(3):
        C, R = kmod.int64_bmm_broadcast(g(A, dev), g(B, dev), 1, 256, 29)
        same(C, want[0], "batched C %d" % rep)
        same(R, want[1], "batched R %d" % rep)
        C, R = kmod.int64_bmm_broadcast(g(A2, dev), g(B2, dev), 1, 1, 30)
        same(C, want2[0], "wq_a-shaped C %d" % rep)
        same(R, want2[1], "wq_a-shaped R %d" % rep)
    kmod.device_status()


def test_small_m_against_the_reference_kernels(libpath, reflib, dev):
    """config 1 and a decode-shaped projection through the reference's symbols of both libraries"""
    ours, ref = type(reflib)(libpath).lib, reflib.lib
    rng = np.random.default_rng(0)
    for (M, K, N, ab, bb, s, w64) in ((32, 7168, 576, 20, 15, 16, True), (32, 7168, 576, 20, 15, 16, False),
                                      (64, 7168, 1536, 21, 30, 30, False), (7, 2048, 7168, 23, 29, 29, False),
                                      (1, 16384, 300, 36, 31, 31, False)):
        A = g(rand_i64(rng, (1, M, K), ab), dev)
        B = rand_i64(rng, (N, K), bb)
        B = g(B if w64 else B.astype(np.int32), dev)
        name = "int64_64_bmm_broadcast_launcher" if w64 else "int64_32_bmm_broadcast_launcher"
        res = []
        for L in (ours, ref):
            C = torch.zeros((1, M, N), dtype=torch.int64, device=dev)
            R = torch.zeros_like(C)
            getattr(L, name)(A.data_ptr(), B.data_ptr(), C.data_ptr(), R.data_ptr(), 1, 1, s, 1, M, K, N)
            torch.cuda.synchronize()
            res.append((C.cpu().numpy(), R.cpu().numpy()))
        assert np.array_equal(res[0][0], res[1][0]) and np.array_equal(res[0][1], res[1][1]), (M, K, N)


# ---- float -> fixed converters (exported by the reference, called by nothing in it) ------------------

def test_converters_against_the_reference_kernels(libpath, reflib, dev):
    """bf16_to_int32_2d, wkv_b_bf16_to_int32, float32_to_int64_2d (int64_gemm.cu:92-221) over every bf16 bit
    pattern and a sample of float32 patterns.  Compared wherever the reference is defined: it divides by
    `1 << -e` evaluated in 32-bit int, which is zero (a division by zero) from e <= -32 on."""
    ours, ref = type(reflib)(libpath).lib, reflib.lib
    bits = np.arange(65536, dtype=np.uint16)
    ex0 = ((bits.astype(np.int64) >> 7) & 0xFF) - 127
    src = torch.from_numpy(bits.view(np.int16).copy()).to(dev)
    for rescale in (0, 19, 31, 40):
        outs = []
        for L in (ours, ref):
            o = torch.zeros(65536, dtype=torch.int32, device=dev)
            L.bf16_to_int32_2d(src.data_ptr(), o.data_ptr(), 256, 256, rescale)
            torch.cuda.synchronize()
            outs.append(o.cpu().numpy())
        ok = ex0 + rescale > -32
        assert np.array_equal(outs[0][ok], outs[1][ok]), "bf16_to_int32_2d rescale %d" % rescale
    outs = []
    for L in (ours, ref):
        o = torch.zeros(65536, dtype=torch.int32, device=dev)
        L.wkv_b_bf16_to_int32(src.data_ptr(), o.data_ptr(), 64, 1024)
        torch.cuda.synchronize()
        outs.append(o.cpu().numpy())
    ok = (ex0 + 25 > -32) | (ex0 >= -1)
    assert np.array_equal(outs[0][ok], outs[1][ok]), "wkv_b_bf16_to_int32"

    rng = np.random.default_rng(5)
    f = np.concatenate([rng.integers(0, 2**32, 200000, dtype=np.uint64).astype(np.uint32),
                        np.array([0, 0x80000000, 1, 0x00800000, 0x3F800000, 0xBF800000, 0x7F7FFFFF, 0x7F800000,
                                  0xFFFFFFFF, 0x4B000000], np.uint32)])
    f = np.resize(f, (500, 420)).copy()
    exf = ((f.astype(np.int64) >> 23) & 0xFF) - 127
    srcf = torch.from_numpy(f.view(np.int32)).to(dev)
    for rescale in (0, 19, 31, 40):
        outs = []
        for L in (ours, ref):
            o = torch.zeros(f.shape, dtype=torch.int64, device=dev)
            L.float32_to_int64_2d(srcf.data_ptr(), o.data_ptr(), f.shape[0], f.shape[1], rescale)
            torch.cuda.synchronize()
            outs.append(o.cpu().numpy())
        ok = exf + rescale > -32
        assert np.array_equal(outs[0][ok], outs[1][ok]), "float32_to_int64_2d rescale %d" % rescale
