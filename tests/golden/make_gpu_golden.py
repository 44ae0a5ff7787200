"""Known-answer vectors from the reference's own CUDA kernels, run on a B200.

The reference has no tests or golden vectors of its own for these kernels, so its
library (built from its unmodified source by oracle/Makefile into oracle/_ref) is
run here on seeded inputs, called through ctypes exactly as the reference's
kernel.py does, and the inputs + outputs are stored in ref_gpu_vectors.npz.

    on a GPU box:   python tests/golden/make_gpu_golden.py <output>.npz
    then copy the file to tests/golden/ref_gpu_vectors.npz

check_against() replays every case through the CPU oracle (no GPU needed).
"""
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))

GEMM_SHIFTS = (0, 16, 29, 30, 31, 32, 33, 37, 63)


def _inputs():
    """Seeded inputs of every case (shared by the generator and the checker)."""
    rng = np.random.default_rng(20251125)
    c = {}

    def ri(shape, bits):
        lim = 1 << bits
        return rng.integers(-lim, lim, size=shape, dtype=np.int64)

    c["gemm_A"] = ri((2, 5, 37), 40)
    c["gemm_B32"] = ri((7, 37), 31).astype(np.int32)
    c["gemm_B64"] = ri((7, 37), 45)
    c["gemm_Abig"] = ri((1, 3, 64), 62)          # sums far beyond 2^63
    c["gemm_Bbig"] = ri((4, 64), 62)
    c["rope_A"] = ri((2, 3, 4, 32, 2), 40)
    ang = rng.uniform(0, 2 * np.pi, (3, 32))
    c["rope_T"] = np.stack([np.rint(np.cos(ang) * 2**42), np.rint(np.sin(ang) * 2**42)],
                           -1).astype(np.int64)
    c["rms_A"] = ri((4, 64), 37)
    c["rms_W32"] = ri((64,), 21).astype(np.int32)
    c["rms_W64"] = ri((64,), 40)
    c["rms_rms"] = np.array([123456789, 1, 2**33 + 5, 77], np.int64)
    c["e_q"] = ri((2, 3, 2, 8), 40)
    c["e_W1"] = ri((2, 8, 16), 31).astype(np.int32)
    c["e_A"] = ri((2, 3, 2, 16), 40)
    c["e_KV"] = ri((2, 5, 16), 36)
    c["e_P"] = rng.integers(0, 2**19, (2, 3, 2, 5), dtype=np.int64)
    c["e_W2"] = ri((2, 8, 16), 31).astype(np.int32)
    sm = np.rint(rng.standard_normal((1, 2, 3, 40)) * 4 * 2**19).astype(np.int64)
    sm[0, 0, 0, 7:] += -(64 << 36)
    sm[0, 1, 1, :] = -5
    c["sm_X"] = sm
    c["sm21_X"] = np.rint(rng.standard_normal((1, 2, 3, 40)) * 2 * 2**21).astype(np.int64)
    for frac in (23, 25):
        LIM = 64 << frac
        c["act%d_X" % frac] = np.concatenate([
            np.array([0, 1, -1, 5, -5, LIM - 1, -LIM + 1, LIM, -LIM]),
            rng.integers(-LIM, LIM, 1500),
            rng.integers(-LIM, -20 * 2**frac, 1500),   # exponent shifts that overflow 64 bits
            np.rint(rng.standard_normal(1087) * 2**frac).astype(np.int64),
        ]).astype(np.int64).reshape(1, 1, -1)
    return c


def generate(out_path):
    import ctypes
    import torch
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    from conftest import RefLib
    ref = RefLib(os.path.join(ROOT, "oracle", "_ref", "libint64gemm_ref.so")).lib
    dev = torch.device("cuda:0")
    c = _inputs()
    out = {}

    def g(a):
        return torch.from_numpy(np.ascontiguousarray(a)).to(dev)

    def z(shape):
        return torch.zeros(shape, dtype=torch.int64, device=dev)

    def keep(name, t):
        torch.cuda.synchronize()
        out[name] = t.cpu().numpy()

    A, B32, B64 = g(c["gemm_A"]), g(c["gemm_B32"]), g(c["gemm_B64"])
    for s in GEMM_SHIFTS:
        C, R = z((2, 5, 7)), z((2, 5, 7))
        ref.int64_32_bmm_broadcast_launcher(A.data_ptr(), B32.data_ptr(), C.data_ptr(), R.data_ptr(),
                                            1, 1, s, 2, 5, 37, 7)
        keep("gemm32_C_s%d" % s, C)
        keep("gemm32_R_s%d" % s, R)
    C, R = z((2, 5, 7)), z((2, 5, 7))
    ref.int64_64_bmm_broadcast_launcher(A.data_ptr(), B64.data_ptr(), C.data_ptr(), R.data_ptr(),
                                        3, 256, 29, 2, 5, 37, 7)
    keep("gemm64_C", C)
    keep("gemm64_R", R)
    Ab, Bb = g(c["gemm_Abig"]), g(c["gemm_Bbig"])
    C, R = z((1, 3, 4)), z((1, 3, 4))
    ref.int64_64_bmm_broadcast_launcher(Ab.data_ptr(), Bb.data_ptr(), C.data_ptr(), R.data_ptr(),
                                        1, 1, 40, 1, 3, 64, 4)
    keep("gemmbig_C", C)
    keep("gemmbig_R", R)

    Ar, Tr = g(c["rope_A"]), g(c["rope_T"])
    C = z(c["rope_A"].shape)
    ref.complex_int64_mul(Ar.data_ptr(), Tr.data_ptr(), C.data_ptr(), 2, 3, 4, 32)
    keep("rope_C", C)

    Am, rms = g(c["rms_A"]), g(c["rms_rms"])
    W32, W64 = g(c["rms_W32"]), g(c["rms_W64"])
    C = z((4, 64))
    ref.rms_norm_32(Am.data_ptr(), W32.data_ptr(), rms.data_ptr(), C.data_ptr(), 4, 64)
    keep("rms32_C", C)
    C = z((4, 64))
    ref.rms_norm_64(Am.data_ptr(), W64.data_ptr(), rms.data_ptr(), C.data_ptr(), 4, 64)
    keep("rms64_C", C)

    q, W1, Ae, KV, P, W2 = (g(c[k]) for k in ("e_q", "e_W1", "e_A", "e_KV", "e_P", "e_W2"))
    C = z((2, 3, 2, 16))
    ref.einsum_bshd_hdc_bshc(q.data_ptr(), W1.data_ptr(), C.data_ptr(), 29, 2, 3, 2, 8, 16)
    keep("e1_C", C)
    C = z((2, 3, 2, 5))
    ref.einsum_bshc_btc_bsht(Ae.data_ptr(), KV.data_ptr(), C.data_ptr(), 23, 2, 3, 2, 5, 16)
    keep("e2_C", C)
    C = z((2, 3, 2, 16))
    ref.einsum_bsht_btc_bshc(P.data_ptr(), KV.data_ptr(), C.data_ptr(), 23, 2, 3, 2, 5, 16)
    keep("e3_C", C)
    C = z((2, 3, 2, 8))
    ref.einsum_bshc_hdc_bshd(Ae.data_ptr(), W2.data_ptr(), C.data_ptr(), 30, 2, 3, 2, 8, 16)
    keep("e4_C", C)

    def host_lut(fn):
        t = torch.zeros((256,), dtype=torch.int64)
        fn(t.data_ptr())
        return t.to(dev)

    for frac, fn, init in ((19, ref.softmax_q19, ref.softmax_init_q19),
                           (21, ref.softmax_q21, ref.softmax_init_q21)):
        lut = host_lut(init)
        X = g(c["sm_X"] if frac == 19 else c["sm21_X"]).clone()
        C = z(X.shape)
        fn(X.data_ptr(), C.data_ptr(), lut.data_ptr(), 1, 2, 3, 40)
        keep("sm%d_C" % frac, C)
        keep("sm%d_W" % frac, X)     # the input buffer now holds the weights
    for frac, silu, sig, init in ((23, ref.silu_q23, ref.sigmoid_q23, ref.silu_init_q23),
                                  (25, ref.silu_q25, ref.sigmoid_q25, ref.silu_init_q25)):
        lut = host_lut(init)
        X = g(c["act%d_X" % frac])
        n = X.shape[-1]
        C = z(X.shape)
        silu(X.data_ptr(), C.data_ptr(), lut.data_ptr(), 1, 1, n)
        keep("silu%d_C" % frac, C)
        C = z(X.shape)
        sig(X.data_ptr(), C.data_ptr(), lut.data_ptr(), 1, 1, n)
        keep("sigmoid%d_C" % frac, C)
    os.makedirs(os.path.dirname(os.path.abspath(out_path)), exist_ok=True)
    np.savez_compressed(out_path, **out)
    print("wrote", out_path, "with", len(out), "arrays")


def check_against(v, orc):
    """Replays every stored case through the CPU oracle; returns the list of mismatches."""
    c = _inputs()
    bad = []

    def cmp(name, got):
        if name not in v.files:
            bad.append(name + " (missing)")
        elif not np.array_equal(v[name], got):
            bad.append("%s (%d words differ)" % (name, int((v[name] != got).sum())))

    for s in GEMM_SHIFTS:
        C, R = orc.gemm(c["gemm_A"], c["gemm_B32"], 1, 1, s, orc.R_LEGACY)
        cmp("gemm32_C_s%d" % s, C)
        cmp("gemm32_R_s%d" % s, R)
    C, R = orc.gemm(c["gemm_A"], c["gemm_B64"], 3, 256, 29, orc.R_LEGACY)
    cmp("gemm64_C", C)
    cmp("gemm64_R", R)
    C, R = orc.gemm(c["gemm_Abig"], c["gemm_Bbig"], 1, 1, 40, orc.R_LEGACY)
    cmp("gemmbig_C", C)
    cmp("gemmbig_R", R)
    cmp("rope_C", orc.rope(c["rope_A"], c["rope_T"], 42))
    cmp("rms32_C", orc.rms_norm_given(c["rms_A"], c["rms_W32"], c["rms_rms"]))
    cmp("rms64_C", orc.rms_norm_given(c["rms_A"], c["rms_W64"], c["rms_rms"]))
    cmp("e1_C", orc.einsum_bshd_hdc_bshc(c["e_q"], c["e_W1"], 29))
    cmp("e2_C", orc.einsum_bshc_btc_bsht(c["e_A"], c["e_KV"], 23))
    cmp("e3_C", orc.einsum_bsht_btc_bshc(c["e_P"], c["e_KV"], 23))
    cmp("e4_C", orc.einsum_bshc_hdc_bshd(c["e_A"], c["e_W2"], 30))
    for frac, key in ((19, "sm_X"), (21, "sm21_X")):
        C, W = orc.softmax(c[key], frac, want_weights=True)
        cmp("sm%d_C" % frac, C)
        cmp("sm%d_W" % frac, W)
    for frac in (23, 25):
        cmp("silu%d_C" % frac, orc.act(c["act%d_X" % frac], "silu", frac))
        cmp("sigmoid%d_C" % frac, orc.act(c["act%d_X" % frac], "sigmoid", frac))
    return bad


if __name__ == "__main__":
    generate(sys.argv[1] if len(sys.argv) > 1 else os.path.join(HERE, "ref_gpu_vectors.npz"))
