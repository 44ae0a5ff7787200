"""Circuit-acceptance checker for zkdata dumps: a Python stand-in for the constraints the
reference's o1js circuits (zk/src/index.ts) put on the files inference/model.py writes.
TEST INFRASTRUCTURE ONLY (node / o1js are not available here); nothing on the product path
imports it.

It restates, per dump family, the relation the circuit asserts between the dumped input and the
dumped output, in exact integer arithmetic (numpy int64 where the values provably fit, Python
integers otherwise), with the circuit's own lookup tables (tests/golden/ts_tables.json, extracted
from index.ts as text):

    norm      x * w = q * rms + r, 0 <= r < rms                                   ts:623-625
              rms^2 <= floor(sum x^2 / dim) + 1 < (rms + 1)^2                     ts:990-996
    gemm      y * 2^s + r = sum_k x * w, 0 <= r < 2^s                             ts:1698-1702, 1948
    rope      a*b = q * 2^42 + r (four products), y0 = q00 - q11, y1 = q01 + q10  ts:2089-2111
    softmax   d = max - x, y = (d * LOG2E_Q19) >> 19, k = y >> 19, table lookup,
              w = k >= 64 ? 0 : t >> k, out = (w << 19) / sum w                   ts:2727-2749
    sigmoid   y = (-x * LOG2E_Q23) >> 23, k, f, table, u, q = 2^46 / (2^23 + u)   ts:3504-3555
    silu      sigmoid q, then c = x * q / 2^23                                    ts:3652
    selector  scores = sigma + bias; chosen experts sorted by score, taken from the
              groups with the largest top-2 sums                                  ts:4041-4595

The reference is not self-consistent in two places: the norm circuit wants
isqrt(floor(sum x^2 / dim) + 1) where the host computes isqrt(floor((1 + sum x^2) / dim)), and the
SiLU circuit divides x * q by 2^23 truncating toward zero where the kernel shifts (floor).  Dumps
that follow the HOST (what "bit-identical dumps" means) are reported as WARNINGS there, with the
count of affected values, never as failures.
"""
import json
import math
import os

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_TABLES = None


def tables():
    global _TABLES
    if _TABLES is None:
        with open(os.path.join(os.path.dirname(_HERE), "tests", "golden", "ts_tables.json")) as f:
            t = json.load(f)
        _TABLES = {"q19": np.array(t["q19Table"], np.int64), "q23": np.array(t["q23Table"], np.int64),
                   "log2e19": int(t["LOG2E_Q19"]), "log2e23": int(t["LOG2E_Q23"])}
    return _TABLES


class Report:
    def __init__(self):
        self.failures, self.warnings, self.checked = [], [], {}

    def fail(self, what, n=1):
        self.failures.append("%s (%d values)" % (what, n))

    def warn(self, what, n=1):
        self.warnings.append("%s (%d values)" % (what, n))

    def count(self, family, n):
        self.checked[family] = self.checked.get(family, 0) + int(n)

    def ok(self):
        return not self.failures


def _obj(a):
    """int64 array -> array of Python integers (exact products of any size)"""
    return np.asarray(a).astype(object)


# ---- norm (ts:623-625, 990-996) ----------------------------------------------------------------
def check_norm(rep, name, x, w, y, rms):
    """x, y int64 [M, dim]; w int32/int64 [dim]; rms int64 [>= M]"""
    M, dim = x.shape
    rms = np.asarray(rms[:M], np.int64)
    xo, wo, yo, ro = _obj(x), _obj(w.astype(np.int64)), _obj(y), _obj(rms)[:, None]
    if (rms <= 0).any():
        rep.fail("%s: rms <= 0" % name, int((rms <= 0).sum()))
        return
    r = xo * wo[None, :] - yo * ro
    bad = (r < 0) | (r >= ro)
    if bad.any():
        rep.fail("%s: x*w != q*rms + r with 0 <= r < rms" % name, int(bad.sum()))
    sq = (xo * xo).sum(1)
    host, circuit = 0, 0
    for i in range(M):
        s, v = int(sq[i]), int(rms[i])
        host += v != math.isqrt((s + 1) // dim)                       # kernel.py:484-492
        q1 = s // dim + 1
        circuit += not (v * v <= q1 < (v + 1) * (v + 1))              # ts:990-994
    if host:
        rep.fail("%s: rms is not isqrt((1 + sum x^2) // dim), the host formula" % name, host)
    if circuit:
        rep.warn("%s: rms follows the host formula where the circuit's isqrt(sum x^2 // dim + 1) differs" % name,
                 circuit)
    rep.count("norm", x.size)


# ---- gemm (ts:1698-1702, 1948) -------------------------------------------------------------------
def check_gemm(rep, name, x, w, y, r, shift, legacy_remainder=True):
    """x int64 [M, K]; w int32/int64 [N, K]; y, r int64 [M, N]: y * 2^s + r = x . w^T.
    The equality is checked modulo 2^64 (wrapping int64 matmul) and in magnitude (float64), which
    together leave no room for an error below 2^64 * 2^-40 of the sum.  legacy_remainder: for
    s >= 32 the reference binary dumps the low 32 bits of the sum (int64_gemm.cu:22), which the
    circuit cannot accept; reported as a warning with the exact remainder recomputed."""
    x, w = np.asarray(x, np.int64), np.asarray(w).astype(np.int64)
    with np.errstate(over="ignore"):
        lo = x @ w.T                                                  # sum mod 2^64
        approx = x.astype(np.float64) @ w.T.astype(np.float64)
    if shift >= 32 and legacy_remainder:
        want_r = lo & np.int64(0xFFFFFFFF)
        if not np.array_equal(r, want_r):
            rep.fail("%s: remainder is not the low 32 bits of the sum (reference binary, s >= 32)" % name,
                     int((r != want_r).sum()))
        rep.warn("%s: s = %d >= 32, the dumped remainder is the reference binary's 32-bit mask, not sum mod 2^s"
                 % (name, shift), r.size)
        with np.errstate(over="ignore"):
            r = lo & np.int64((1 << shift) - 1) if shift < 63 else lo
    if ((r < 0) | (r >= (1 << min(shift, 62)))).any() and shift < 63:
        rep.fail("%s: remainder outside [0, 2^s)" % name, int(((r < 0) | (r >= (1 << shift))).sum()))
    with np.errstate(over="ignore"):
        back = (y << np.int64(shift)) + r if shift < 64 else r
    bad = back != lo
    if bad.any():
        rep.fail("%s: y * 2^s + r != sum x*w (mod 2^64)" % name, int(bad.sum()))
    mag = np.abs(y.astype(np.float64) * 2.0 ** shift - approx) > 1e-9 * np.abs(approx) + 2.0 ** (shift + 1)
    if mag.any():
        rep.fail("%s: y * 2^s is not the magnitude of sum x*w" % name, int(mag.sum()))
    rep.count("gemm", y.size)


# ---- rope (ts:2089-2111) ---------------------------------------------------------------------------
def check_rope(rep, name, x, freqs, y, shift=42):
    """x, y int64 [B, S, H, 2P]; freqs int64 [S, P, 2]"""
    B, S, H, D = x.shape
    a = _obj(x).reshape(B, S, H, D // 2, 2)
    b = _obj(freqs).reshape(1, S, 1, D // 2, 2)
    yy = _obj(y).reshape(B, S, H, D // 2, 2)
    two = 1 << shift
    q = lambda u, v: (u * v) // two                      # floor: 0 <= r < 2^shift, as the circuit asserts
    y0 = q(a[..., 0], b[..., 0]) - q(a[..., 1], b[..., 1])
    y1 = q(a[..., 0], b[..., 1]) + q(a[..., 1], b[..., 0])
    bad = (y0 != yy[..., 0]) | (y1 != yy[..., 1])
    if bad.any():
        rep.fail("%s: y0 != q00 - q11 or y1 != q01 + q10" % name, int(bad.sum()))
    rep.count("rope", x.size)


# ---- softmax (ts:2727-2749) --------------------------------------------------------------------------
def check_softmax(rep, name, x, y):
    """x, y int64 [..., T]: rows along the last axis.  The circuit works on x + 2^63 as UInt64; d = max - x
    is the same either way."""
    t = tables()
    x = np.asarray(x, np.int64)
    T = x.shape[-1]
    xr, yr = x.reshape(-1, T), np.asarray(y, np.int64).reshape(-1, T)
    d = _obj(xr.max(1, keepdims=True)) - _obj(xr)                       # >= 0, may exceed 63 bits
    yq = (d * t["log2e19"]) >> 19
    k = yq >> 19
    f = (yq - (k << 19)) >> (19 - 8)
    big = np.frompyfunc(lambda v: v >= 64, 1, 1)(k).astype(bool)
    kk = np.where(big, 0, k).astype(np.int64)
    ff = np.where(big, 0, f).astype(np.int64)
    w = np.where(big, 0, t["q19"][ff] >> kk).astype(np.int64)
    s = w.sum(1, keepdims=True)
    want = np.where(s == 0, 0, (w << 19) // np.where(s == 0, 1, s))
    bad = want != yr
    if bad.any():
        rep.fail("%s: out != (w << 19) / sum w" % name, int(bad.sum()))
    rep.count("softmax", x.size)


# ---- sigmoid / SiLU (ts:3504-3555, 3652) -------------------------------------------------------------
def _sigmoid_q(x):
    """the circuit's q = 2^46 / (2^23 + u) for int64 x (Python integers)"""
    t = tables()
    p = -_obj(x) * t["log2e23"]
    y = p >> 23
    k = y >> 23
    f = y & ((1 << 23) - 1)
    f2 = (f >> (23 - 8)).astype(np.int64)
    tt = _obj(t["q23"][f2])

    def shift(tv, kv):
        if kv < 0:
            return 0 if -kv >= 63 else tv >> (-kv)
        return tv << kv
    u = np.frompyfunc(shift, 2, 1)(tt, k)
    return (1 << 46) // ((1 << 23) + u)


def check_sigmoid(rep, name, x, y):
    """x, y int64 of one shape, inside the kernel's domain |x| < 64 * 2^23 (beyond it the host returns x or
    0 by its own rule, int64_gemm.cu:986-991, which the circuit does not model: counted as warnings)"""
    x, y = np.asarray(x, np.int64).ravel(), np.asarray(y, np.int64).ravel()
    lim = 64 << 23
    inside = (x < lim) & (x > -lim)
    q = _sigmoid_q(x[inside])
    bad = q != _obj(y[inside])
    if bad.any():
        rep.fail("%s: sigmoid != 2^46 / (2^23 + u)" % name, int(bad.sum()))
    if (~inside).any():
        rep.warn("%s: inputs beyond +-64 * 2^23 follow the kernel's saturation rule" % name, int((~inside).sum()))
    rep.count("sigmoid", x.size)


def check_silu(rep, name, x, y):
    x, y = np.asarray(x, np.int64).ravel(), np.asarray(y, np.int64).ravel()
    lim = 64 << 23
    inside = (x < lim) & (x > -lim)
    xi = _obj(x[inside])
    prod = xi * _sigmoid_q(x[inside])
    host = prod >> 23                                                   # int64_gemm.cu:946: arithmetic shift
    circuit = np.frompyfunc(lambda v: -((-v) >> 23) if v < 0 else v >> 23, 1, 1)(prod)   # ts:3652: Int64.div
    yo = _obj(y[inside])
    bad = host != yo
    if bad.any():
        rep.fail("%s: silu != (x * q) >> 23" % name, int(bad.sum()))
    differs = (host != circuit) & ~bad
    if differs.any():
        rep.warn("%s: negative products where the circuit's truncating division differs from the kernel's shift"
                 % name, int(differs.sum()))
    if (~inside).any():
        rep.warn("%s: inputs beyond +-64 * 2^23 follow the kernel's saturation rule" % name, int((~inside).sum()))
    rep.count("silu", x.size)


# ---- selector (ts:4041-4595) -------------------------------------------------------------------------
def check_selector(rep, name, original, bias, indices, gate_weights, n_groups, topk_groups):
    """original int64 [T, E] (sigma), bias int32 [E], indices int64 [T, k], gate_weights int64 [T, k]"""
    T, E = original.shape
    k = indices.shape[1]
    scores = original + bias.astype(np.int64)[None, :]                   # ts:4041
    bad = 0
    if not np.array_equal(np.take_along_axis(original, indices, 1), gate_weights):
        rep.fail("%s: gate_weights != original_scores[indices]" % name,
                 int((np.take_along_axis(original, indices, 1) != gate_weights).sum()))
    g = scores.reshape(T, n_groups, E // n_groups)
    top2 = np.sort(g, -1)[:, :, -2:].sum(-1)                             # ts:4374-4376: the two largest per group
    for t in range(T):
        idx = indices[t]
        chosen = scores[t, idx]
        if len(set(idx.tolist())) != k or (np.diff(chosen) > 0).any():   # ts:4570, 4586: sorted candidates
            bad += 1
            continue
        groups = set((idx // (E // n_groups)).tolist())
        kept_threshold = np.sort(top2[t])[-topk_groups]
        if any(top2[t, gi] < kept_threshold for gi in groups):          # only groups among the largest top-2 sums
            bad += 1
            continue
        kept = [gi for gi in range(n_groups) if top2[t, gi] >= kept_threshold]
        if len(kept) == topk_groups:                                     # no tie between groups: the set is forced
            pool = np.concatenate([g[t, gi] for gi in kept])
            if np.sort(pool)[-k] > chosen.min():
                bad += 1
    if bad:
        rep.fail("%s: the chosen experts are not a sorted top-k of the kept groups" % name, bad)
    rep.count("selector", T)


# ---- a dump directory of one layer and position ------------------------------------------------------
def _load(files, key, dtype):
    return np.frombuffer(files[key], dtype=dtype) if key in files else None


def check_layer(files, prefix, dims, shifts, rep=None):
    """files: {relative path: bytes} (model_cases.read_dumps); prefix 'pos_P/layer_L/'.
    dims: dim, q_lora, kv_lora, inter (dense or shared-expert width), n_experts, n_groups, topk_groups, topk,
    moe_inter.  shifts: wq_a, wkv_a1, gate (the GEMM shifts whose remainders are dumped)."""
    rep = rep or Report()
    g = lambda n, dt=np.int64: _load(files, prefix + n + ".bin", dt)
    x = g("attn_norm_x")
    if x is not None:
        D = dims["dim"]
        check_norm(rep, prefix + "attn_norm", x.reshape(-1, D), g("attn_norm_weight", np.int32),
                   g("attn_norm_y").reshape(-1, D), g("attn_norm_rms"))
    x = g("wq_a_x")
    if x is not None:
        D, Q = dims["dim"], dims["q_lora"]
        check_gemm(rep, prefix + "wq_a", x.reshape(-1, D), g("wq_a_w", np.int32).reshape(Q, D),
                   g("wq_a_y").reshape(-1, Q), g("q_norm_r").reshape(-1, Q), shifts["wq_a"])
        check_norm(rep, prefix + "q_norm", g("q_norm_x").reshape(-1, Q), g("q_norm_weight", np.int32),
                   g("q_norm_y").reshape(-1, Q), g("q_norm_rms"))
    x = g("wkv_a1_x")
    if x is not None:
        D, C = dims["dim"], dims["kv_lora"]
        check_gemm(rep, prefix + "wkv_a1", x.reshape(-1, D), g("wkv_a1_w", np.int32).reshape(C, D),
                   g("wkv_a1_y").reshape(-1, C), g("wkv_a1_r").reshape(-1, C), shifts["wkv_a1"])
    x = g("scores_softmax_x")
    if x is not None:
        rows = g("attn_norm_x").size // dims["dim"] if g("attn_norm_x") is not None else None
        y = g("scores_softmax_y")
        T = x.size // (rows * dims["heads"]) if rows else None
        if T:
            check_softmax(rep, prefix + "scores_softmax", x.reshape(-1, T), y.reshape(-1, T))
    x = g("mlp_silu_x")
    if x is not None:
        check_silu(rep, prefix + "mlp_silu", x, g("mlp_silu_y"))
    x = g("sigmoid_gate_x")
    if x is not None:
        check_sigmoid(rep, prefix + "sigmoid_gate", x, g("sigmoid_gate_y"))
        E = dims["n_experts"]
        orig = g("gate_original_scores").reshape(-1, E)
        if not np.array_equal(orig, g("sigmoid_gate_y").reshape(-1, E)):
            rep.fail(prefix + "gate_original_scores != sigmoid_gate_y")
        check_selector(rep, prefix + "gate", orig, g("gate_bias", np.int32), g("gate_indices").reshape(-1, dims["topk"]),
                       g("gate_weights").reshape(-1, dims["topk"]), dims["n_groups"], dims["topk_groups"])
        r = g("sigmoid_gate_r")
        if ((r < 0) | (r >= (1 << min(shifts["gate"], 32)))).any():
            rep.fail(prefix + "sigmoid_gate_r outside [0, 2^min(s, 32))")
    for key in sorted(files):
        if key.startswith(prefix + "expert_") and key.endswith("_silu_x.bin"):
            stem = key[:-len("_x.bin")]
            check_silu(rep, stem, np.frombuffer(files[key], np.int64), np.frombuffer(files[stem + "_y.bin"], np.int64))
    return rep
