"""Drop-in replacement for the reference's ``inference/kernel.py`` on B200.

Same function names, argument meaning and return values as the reference module
(``inference/kernel.py:341-687``), so ``inference/model.py`` and
``inference/generate.py`` import it unchanged::

    from kernel import int64_bmm_broadcast, softmax_q19, RMS_Norm_int64, ...

Every function calls hand-written sm_100a CUDA through the C ABI of
``libint64gemm.so`` (``include/zkds_int64.h``).  There is no CPU or PyTorch
fallback: a missing library or a failing launch raises.

Differences from the reference module, all on the host side:
  * the library is looked up through ``$ZKDS_LIB``, then beside this file, then
    ``./libint64gemm.so`` (the reference only tries the last, kernel.py:206);
  * nothing is allocated on the GPU at import time;
  * launches go to torch's current stream and their status is checked;
  * ``RMS_Norm_int64`` computes the per-row rms on the GPU (the reference loops
    over every element on the host, kernel.py:477-494) and returns the same
    ``(C, rms)`` pair, ``rms`` being a CPU int64 tensor of at least 500 entries
    whose first M entries are the rows' rms;
  * the float / Triton helpers of the fp8 path (``act_quant``, ``weight_dequant``,
    ``fp8_gemm``) are importable but raise: the integer forward pass never
    reaches them.
"""
import ctypes
import os

import torch

_HERE = os.path.dirname(os.path.abspath(__file__))

ALGO_AUTO, ALGO_EXACT, ALGO_LIMB = 0, 1, 2
REMAINDER_LEGACY = 4
LIMBS_DYNAMIC = 8
CAUSAL_SKIP = 16
GROUP_ROWS_32, GROUP_ROWS_64 = 32, 64

# Remainder flavour of int64_bmm_broadcast.  True reproduces the reference binary:
# exact for c_rescale <= 31, the low 32 bits of the sum above that
# (int64_gemm.cu:22 builds its mask from a 32-bit 1).  False gives sum mod 2^s.
LEGACY_REMAINDER = True
# Contraction algorithm used by the functions below (ALGO_AUTO picks the tensor-core
# limb kernel when the shape allows it).
ALGO = ALGO_AUTO


def _find_library():
    cands = []
    if os.environ.get("ZKDS_LIB"):
        cands.append(os.environ["ZKDS_LIB"])
    cands.append(os.path.join(_HERE, "libint64gemm.so"))
    cands.append("./libint64gemm.so")
    for c in cands:
        if os.path.exists(c):
            return c
    raise OSError("libint64gemm.so not found (looked in %s); build it with "
                  "`python zk-deepseek_b200/build.py`" % ", ".join(cands))


lib = ctypes.CDLL(_find_library())

_vp, _ll, _i = ctypes.c_void_p, ctypes.c_longlong, ctypes.c_int


def _sig(name, argtypes, restype=_i):
    fn = getattr(lib, name)
    fn.argtypes = argtypes
    fn.restype = restype
    return fn


_sig("zkds_last_status", [])
_sig("zkds_last_cuda_error", [])
_sig("zkds_status_string", [_i], ctypes.c_char_p)
_sig("zkds_version", [], ctypes.c_char_p)
_sig("zkds_shutdown", [], None)
_sig("zkds_gemm", [_vp, _vp, _i, _vp, _vp, _ll, _ll, _ll, _ll, _ll, _ll, _ll, _i, _i, _i, _vp])
for _n in ("zkds_einsum_bshd_hdc_bshc", "zkds_einsum_bshc_btc_bsht", "zkds_einsum_bsht_btc_bshc",
           "zkds_einsum_bshc_hdc_bshd"):
    _sig(_n, [_vp, _vp, _vp, _ll, _ll, _ll, _ll, _ll, _ll, _i, _i, _i, _vp])
_sig("zkds_rope", [_vp, _vp, _vp, _ll, _ll, _ll, _ll, _i, _vp])
_sig("zkds_rms_norm", [_vp, _vp, _i, _vp, _vp, _ll, _ll, _ll, _ll, _vp])
_sig("zkds_rms_norm_apply", [_vp, _vp, _i, _vp, _vp, _ll, _ll, _vp])
_sig("zkds_softmax", [_vp, _vp, _vp, _vp, _ll, _ll, _i, _vp])
_sig("zkds_act", [_vp, _vp, _vp, _ll, _i, _i, _vp])
_sig("zkds_lut", [_vp, _i])
_sig("zkds_device_status", [_i])
_sig("zkds_timing_record", [ctypes.c_longlong, ctypes.POINTER(ctypes.c_double)])
_sig("zkds_timing", [_i], None)
_sig("zkds_last_kernel_ms", [], ctypes.c_float)
_sig("zkds_timing_totals", [ctypes.POINTER(ctypes.c_double), ctypes.POINTER(ctypes.c_double),
                            ctypes.POINTER(ctypes.c_longlong)], None)
_sig("zkds_planes_create", [_vp, _i, _ll, _ll, _ll, _ll, _ll, _ll, _ll, _i, ctypes.POINTER(_vp), _vp])
_sig("zkds_planes_limbs", [_vp])
_sig("zkds_planes_destroy", [_vp])
_sig("zkds_einsum_bshc_btc_bsht_ex", [_vp, _vp, _vp, _ll, _ll, _ll, _ll, _ll, _ll, _vp, _ll, _ll, _i, _ll,
                                      _ll, _i, _i, _i, _vp])
_sig("zkds_mla_scores", [_vp, _vp, _vp, _vp, _vp, _ll, _ll, _ll, _ll, _ll, _ll, _ll, _ll, _ll, _ll, _i, _ll, _ll,
                         _i, _i, _i, _vp])
_sig("zkds_softmax_causal", [_vp, _vp, _vp, _ll, _ll, _ll, _ll, _ll, _vp])
_sig("zkds_softmax_pv", [_vp, _vp, _vp, _vp, _ll, _ll, _ll, _ll, _ll, _ll, _i, _ll, _i, _i, _i, _vp])
_sig("zkds_einsum_bsht_btc_bshc_causal", [_vp, _vp, _vp, _ll, _ll, _ll, _ll, _ll, _ll, _ll, _i, _i, _i, _vp])
_sig("zkds_grouped_prepared", [_vp, _vp, _vp, _ll, _vp, _ll, _ll, _ll, _vp, _ll, _i, _i, _vp])
_sig("zkds_glu_prepared", [_vp, _vp, _ll, _vp, _ll, _vp, _vp, _vp, _ll, _vp, _ll, _i, _i, _vp])
_sig("zkds_grouped_gather_prepared", [_vp, _vp, _vp, _vp, _ll, _vp, _ll, _ll, _ll, _vp, _ll, _i, _i, _vp])
_sig("zkds_glu_q23", [_vp, _vp, _ll, _vp, _vp, _vp, _ll, _ll, _vp])
_sig("zkds_gather_rows", [_vp, _vp, _vp, _ll, _ll, _vp])
_sig("zkds_moe_combine", [_vp, _vp, _vp, _vp, _vp, _ll, _i, _ll, _vp])
_sig("zkds_gate_select", [_vp, _vp, _ll, _i, _i, _i, _i, _vp, _vp, _vp, _vp])
_sig("zkds_cache_planes_append", [_vp, _vp, _vp, _vp, _ll, _ll, _ll, _ll, _ll, _ll, _i, _vp])
_sig("zkds_mla_scores_cached", [_vp, _vp, _vp, _ll, _vp, _ll, _ll, _ll, _ll, _ll, _ll, _ll, _ll, _ll, _ll, _i, _ll,
                                _ll, _i, _i, _i, _vp])
_sig("zkds_softmax_pv_cached", [_vp, _vp, _ll, _vp, _vp, _ll, _ll, _ll, _ll, _ll, _ll, _i, _ll, _i, _i, _i, _vp])
_sig("zkds_grouped_gather_parts_prepared", [_vp, _i, _ll, _vp, _vp, _vp, _ll, _vp, _ll, _vp, _ll, _i, _i, _vp])
_sig("zkds_moe_combine_peer", [_vp, _vp, _vp, _ll, _i, _ll, _ll, _vp, _i, _i, _vp])
_sig("zkds_moe_sum_slots", [_vp, _vp, _vp, _ll, _i, _ll, _i, _i, _vp, _vp])
_sig("zkds_peer_barrier", [_vp, _i, _i, ctypes.c_ulonglong, _vp, _vp])
_sig("zkds_contraction_prepared", [_vp, _ll, _ll, _vp, _i, _vp, _vp, _ll, _ll, _ll, _ll, _ll, _ll, _ll,
                                   _i, _i, _vp])


ERR_RANGE = 2           # ZKDS_ERR_RANGE: an operand did not fit the limb count promised for it


class ZkdsError(RuntimeError):
    """A library call or a finished kernel reported a non-zero status (`.status`)."""

    def __init__(self, message, status=0):
        super().__init__(message)
        self.status = status


def _check(status, what):
    if status != 0:
        msg = lib.zkds_status_string(status).decode()
        if status == 3:
            msg += " (cudaError %d)" % lib.zkds_last_cuda_error()
        raise ZkdsError("%s: %s" % (what, msg), status)


def _stream():
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


class _NoSwitch:
    def __enter__(self):
        return self

    def __exit__(self, *exc):
        return False


_NO_SWITCH = _NoSwitch()


def _on(device):
    """context that makes `device` current for a library call; nothing to do (and nothing to pay: the guard
    costs several microseconds per call) when it already is"""
    if device.index is None or device.index == torch.cuda.current_device():
        return _NO_SWITCH
    return torch.cuda.device(device)


def _dev_i64(t, name):
    if t.dtype != torch.int64:
        raise TypeError("%s must be int64, got %s" % (name, t.dtype))
    if not t.is_cuda:
        raise ValueError("%s must be a CUDA tensor" % name)
    if not t.is_contiguous():
        raise ValueError("%s must be contiguous" % name)
    return t


# ---- float helpers of the fp8 path: not part of the integer forward pass -------------

def act_quant(x, block_size=128):
    raise NotImplementedError("act_quant belongs to the fp8 path; the integer model never calls it")


def weight_dequant(x, s, block_size=128):
    raise NotImplementedError("weight_dequant belongs to the fp8 path (offline conversion only)")


def fp8_gemm(a, a_s, b, b_s):
    raise NotImplementedError("fp8_gemm belongs to the fp8 path; the integer model never calls it")


# ---- contractions --------------------------------------------------------------------

def int64_bmm_broadcast(A, B, a_rescale, b_rescale, c_rescale, a_limbs=0, b_limbs=0):
    """(Bdim, M, K) int64 x (N, K) int32|int64 -> (C, R), each (Bdim, M, N) int64.

    C = (sum_k (A/a_rescale)*(B/b_rescale)) >> c_rescale with the sum held in 128 bits;
    R is the remainder (kernel.py:341-371, int64_gemm.cu:6-90).  a_limbs/b_limbs are
    optional operand-range hints (signed 8-bit limb counts); 0 measures them.
    """
    _dev_i64(A, "A")
    if not B.is_cuda or not B.is_contiguous():
        raise ValueError("B must be a contiguous CUDA tensor")
    if B.dtype not in (torch.int64, torch.int32):
        raise TypeError("Unsupported B type: %s" % B.dtype)
    Bdim, M, K = A.shape
    N, K2 = B.shape
    assert K2 == K
    C = torch.empty((Bdim, M, N), dtype=torch.int64, device=A.device)
    R = torch.empty((Bdim, M, N), dtype=torch.int64, device=A.device)
    flags = ALGO | (REMAINDER_LEGACY if LEGACY_REMAINDER else 0)
    with _on(A.device):
        _check(lib.zkds_gemm(A.data_ptr(), B.data_ptr(), 32 if B.dtype == torch.int32 else 64,
                             C.data_ptr(), R.data_ptr(), int(a_rescale), int(b_rescale),
                             int(c_rescale), Bdim, M, K, N, a_limbs, b_limbs, flags, _stream()),
               "int64_bmm_broadcast")
    return (C, R)


def _einsum(fn_name, A, B, out_shape, rescale, dims, a_limbs, b_limbs):
    _dev_i64(A, "A")
    if not B.is_cuda or not B.is_contiguous():
        raise ValueError("B must be a contiguous CUDA tensor")
    C = torch.empty(out_shape, dtype=torch.int64, device=A.device)
    with _on(A.device):
        _check(getattr(lib, fn_name)(A.data_ptr(), B.data_ptr(), C.data_ptr(), int(rescale), *dims,
                                     a_limbs, b_limbs, ALGO, _stream()), fn_name)
    return C


def einsum_bshd_hdc_bshc(A, B, rescale, a_limbs=0, b_limbs=0):
    """out[b,s,h,c] = (rescale//2 + sum_d A[b,s,h,d] * B[h,d,c]) >> rescale; B int32."""
    assert A.shape[2] == B.shape[0] and A.shape[3] == B.shape[1]
    assert B.dtype == torch.int32
    Bn, S, H, D = A.shape
    Cp = B.shape[2]
    return _einsum("zkds_einsum_bshd_hdc_bshc", A, B, [Bn, S, H, Cp], rescale, (Bn, S, H, D, Cp),
                   a_limbs, b_limbs)


def einsum_bshc_btc_bsht(A, B, rescale, a_limbs=0, b_limbs=0):
    """out[b,s,h,t] = (rescale//2 + sum_c A[b,s,h,c] * B[b,t,c]) >> rescale; B int64."""
    Bn, S, H, Cd = A.shape
    T = B.shape[1]
    assert Bn == B.shape[0] and Cd == B.shape[2]
    _dev_i64(B, "B")
    return _einsum("zkds_einsum_bshc_btc_bsht", A, B, [Bn, S, H, T], rescale, (Bn, S, H, T, Cd),
                   a_limbs, b_limbs)


def einsum_bsht_btc_bshc(A, B, rescale, a_limbs=0, b_limbs=0):
    """out[b,s,h,c] = (rescale//2 + sum_t A[b,s,h,t] * B[b,t,c]) >> rescale; B int64."""
    Bn, S, H, T = A.shape
    Cd = B.shape[2]
    assert Bn == B.shape[0] and T == B.shape[1]
    _dev_i64(B, "B")
    return _einsum("zkds_einsum_bsht_btc_bshc", A, B, [Bn, S, H, Cd], rescale, (Bn, S, H, T, Cd),
                   a_limbs, b_limbs)


def einsum_bshc_hdc_bshd(A, B, rescale, a_limbs=0, b_limbs=0):
    """out[b,s,h,d] = (sum_c A[b,s,h,c] * B[h,d,c]) >> rescale (no rounding term); B int32."""
    Bn, S, H, Cd = A.shape
    D = B.shape[1]
    assert H == B.shape[0] and Cd == B.shape[2]
    assert B.dtype == torch.int32
    return _einsum("zkds_einsum_bshc_hdc_bshd", A, B, [Bn, S, H, D], rescale, (Bn, S, H, D, Cd),
                   a_limbs, b_limbs)


# ---- static weights prepared once ---------------------------------------------------------

def device_status(clear=True, sync=False):
    """Raises if a finished tensor-core kernel gave up a bounded wait, or if an operand did not
    fit the limb count a caller promised through a_limbs (that call's result is wrong).  The flags
    are written by kernels: `sync=True` first waits for torch's current stream."""
    if sync:
        torch.cuda.current_stream().synchronize()
    _check(lib.zkds_device_status(1 if clear else 0), "device status")


def kernel_timing(enable):
    """True/1: event pair around each tensor-core launch; 2: also accumulate totals (waits per launch)"""
    lib.zkds_timing(int(enable))


def kernel_timing_records():
    """per-launch records since kernel_timing(2): dicts with batches, M, N, K, la, lb, ms, grouped"""
    out, buf, i = [], (ctypes.c_double * 8)(), 0
    while lib.zkds_timing_record(ctypes.c_longlong(i), buf):
        out.append(dict(batches=int(buf[0]), M=int(buf[1]), N=int(buf[2]), K=int(buf[3]), la=int(buf[4]),
                        lb=int(buf[5]), ms=buf[6], grouped=bool(int(buf[7]) & 1), b_batched=bool(int(buf[7]) & 2)))
        i += 1
    return out


def kernel_timing_totals():
    """(total ms, total int8 ops = limb pairs x 2MNK, launches) since kernel_timing(2)"""
    ms, ops, n = ctypes.c_double(), ctypes.c_double(), ctypes.c_longlong()
    lib.zkds_timing_totals(ctypes.byref(ms), ctypes.byref(ops), ctypes.byref(n))
    return ms.value, ops.value, n.value


def last_kernel_ms():
    return float(lib.zkds_last_kernel_ms())


def limb_kernel_takes(K, a_limbs, b_limbs):
    """True when the tensor-core limb kernel handles a contraction of depth K with these limb
    counts (mirrors the launcher: int32 diagonal bound, tile and pipeline fit)."""
    if K <= 0 or not (1 <= a_limbs <= 9 and 1 <= b_limbs <= 9):
        return False
    if min(a_limbs, b_limbs) * K >= 131072:
        return False
    diagonals = a_limbs + b_limbs - 1
    smem_max = 227 * 1024 - 4096
    for nt in (128, 64, 32, 16):
        if b_limbs * nt > 256 or diagonals * nt > 512:
            continue
        if smem_max // (a_limbs * 16384 + b_limbs * nt * 128) >= 2:
            return True
    return False


class WeightPlanes:
    """Signed 8-bit limb planes of a static weight, split once and kept on the device.

    ``W`` is (N, K) for a plain linear layer or (H, N, K) / (H, K, N) for the per-head MLA
    weights; ``k_last`` says whether K is the last (contiguous) dimension.
    """

    def __init__(self, W, k_last=True, div=1, limbs=0):
        assert W.is_cuda and W.is_contiguous() and W.dtype in (torch.int32, torch.int64)
        if W.ndim == 2:
            nb, (rows, K) = 1, W.shape
            s_batch, s_row, s_k = 0, K, 1
            assert k_last
        else:
            nb = W.shape[0]
            if k_last:
                rows, K = W.shape[1], W.shape[2]
                s_row, s_k = K, 1
            else:
                K, rows = W.shape[1], W.shape[2]
                s_row, s_k = 1, rows
            s_batch = rows * K
        self.nb, self.N, self.K = nb, rows, K
        self.device = W.device
        h = _vp()
        with _on(W.device):
            _check(lib.zkds_planes_create(W.data_ptr(), 32 if W.dtype == torch.int32 else 64, nb, rows,
                                          K, s_batch, s_row, s_k, int(div), limbs, ctypes.byref(h),
                                          _stream()), "zkds_planes_create")
        self.handle = h
        self.limbs = lib.zkds_planes_limbs(h)

    def __del__(self):
        h, self.handle = getattr(self, "handle", None), None
        if h and lib is not None:        # `lib` is already gone at interpreter shutdown
            lib.zkds_planes_destroy(h)


def _a_flags(a_limbs, dynamic):
    return LIMBS_DYNAMIC if (dynamic and a_limbs > 0) else 0


def linear_prepared(A, planes, c_rescale, a_rescale=1, a_limbs=0, want_remainder=False, dynamic=False):
    """int64_bmm_broadcast against prepared weights: A (Bdim, M, K) -> C (Bdim, M, N) [, R].

    a_limbs: 0 measures the range of A (host synchronisation); > 0 promises that A fits that
    many signed 8-bit limbs; with dynamic=True it is only an upper bound and the count used is
    derived on the device."""
    _dev_i64(A, "A")
    Bdim, M, K = A.shape
    assert K == planes.K and planes.nb == 1
    C = torch.empty((Bdim, M, planes.N), dtype=torch.int64, device=A.device)
    R = torch.empty_like(C) if want_remainder else None
    flags = (REMAINDER_LEGACY if LEGACY_REMAINDER else 0) | _a_flags(a_limbs, dynamic)
    with _on(A.device):
        _check(lib.zkds_contraction_prepared(A.data_ptr(), M * K, K, planes.handle, 0, C.data_ptr(),
                                             R.data_ptr() if want_remainder else None, M * planes.N,
                                             planes.N, Bdim, M, int(a_rescale), 0, int(c_rescale),
                                             a_limbs, flags, _stream()), "linear_prepared")
    return (C, R) if want_remainder else C


def einsum_heads_prepared(A, planes, rescale, rounding, a_limbs=0, dynamic=False):
    """out[b,s,h,n] = (addend + sum_k A[b,s,h,k] * W[h,n,k]) >> rescale with per-head prepared
    weights; addend = rescale // 2 when ``rounding`` (einsum_bshd_hdc_bshc) else 0
    (einsum_bshc_hdc_bshd)."""
    _dev_i64(A, "A")
    Bn, S, H, K = A.shape
    assert H == planes.nb and K == planes.K
    N = planes.N
    C = torch.empty((Bn, S, H, N), dtype=torch.int64, device=A.device)
    with _on(A.device):
        _check(lib.zkds_contraction_prepared(A.data_ptr(), K, H * K, planes.handle, 1, C.data_ptr(), None,
                                             N, H * N, H, Bn * S, 1, int(rescale) // 2 if rounding else 0,
                                             int(rescale), a_limbs, _a_flags(a_limbs, dynamic), _stream()),
               "einsum_heads_prepared")
    return C


def _group_rows_flag(max_rows):
    """flag for a promised bound on the rows of every group (None or > 64: no promise)"""
    if max_rows is None or max_rows > 64:
        return 0
    return GROUP_ROWS_32 if max_rows <= 32 else GROUP_ROWS_64


def grouped_prepared(A, planes, tile_group, c_rescale, a_limbs=0, dynamic=False, group_shift=None,
                     n_split=0, row_index=None, max_group_rows=None):
    """Routed-expert linear layer: A flat (n_tiles*128, K), tile_group int32 (n_tiles,) on the
    device (expert of each 128-row tile, negative = unused) -> C (n_tiles*128, N).
    group_shift: optional int32 (experts, 2) device tensor of per-expert shifts for the output
    columns below / from n_split; otherwise the uniform c_rescale.
    row_index: optional int32 (n_tiles*128,) device tensor; row m of the grouped matrix is then
    A[row_index[m]] (zeros where negative) and A is the un-gathered (tokens, K) matrix: the
    index_select of model.py:1372-1378 happens inside the limb split (a_limbs must be given).
    max_group_rows: a bound on the rows of every group that the caller can prove (decode: a token names an
    expert at most once, so no expert has more rows than there are tokens); up to 64 the kernel then fetches
    only the first 32 / 64 rows of every tile."""
    gflag = _group_rows_flag(max_group_rows)
    if group_shift is not None:
        assert group_shift.dtype == torch.int32 and group_shift.is_cuda and group_shift.is_contiguous()
    _dev_i64(A, "A")
    assert tile_group.dtype == torch.int32 and tile_group.is_cuda and tile_group.is_contiguous()
    n_tiles = tile_group.numel()
    C = torch.empty((n_tiles * 128, planes.N), dtype=torch.int64, device=A.device)
    gs = group_shift.data_ptr() if group_shift is not None else None
    with _on(A.device):
        if row_index is None:
            assert A.shape == (n_tiles * 128, planes.K)
            _check(lib.zkds_grouped_prepared(A.data_ptr(), planes.handle, tile_group.data_ptr(), n_tiles,
                                             C.data_ptr(), 1, 0, int(c_rescale), gs, int(n_split), a_limbs,
                                             _a_flags(a_limbs, dynamic) | gflag, _stream()), "grouped_prepared")
        else:
            assert row_index.dtype == torch.int32 and row_index.is_cuda and row_index.is_contiguous()
            assert row_index.numel() == n_tiles * 128 and A.dim() == 2 and A.shape[1] == planes.K and a_limbs > 0
            if A.shape[0] == 0:      # nothing to gather from (every index is negative): one row of zeros
                A = torch.zeros((1, planes.K), dtype=torch.int64, device=A.device)
            _check(lib.zkds_grouped_gather_prepared(A.data_ptr(), row_index.data_ptr(), planes.handle,
                                                    tile_group.data_ptr(), n_tiles, C.data_ptr(), 1, 0,
                                                    int(c_rescale), gs, int(n_split), a_limbs,
                                                    _a_flags(a_limbs, dynamic) | gflag, _stream()), "grouped_prepared")
    return C


def glu_prepared(r1, r2, planes, c_rescale, ld=None, a_limbs=3, dynamic=True, tile_group=None,
                 group_shift=None, n_split=0, max_group_rows=None):
    """w2 of a gated MLP with the gate inside its limb split: C = (h @ W2^T) >> c_rescale with
    h = (silu_q23(r1) * r2) >> 23 (model.py:1034-1049, 1271-1281); h only ever exists as int8 limb
    planes.  r1, r2: (rows, K) views sharing the row stride ld (default K); planes: prepared W2, or
    the experts' stacked W2 together with tile_group (and group_shift) as in grouped_prepared.
    Returns None when the kernel does not take the shape (use glu_q23 and the linear layer then)."""
    for t_, name in ((r1, "r1"), (r2, "r2")):     # strided row views of one buffer are the normal case
        assert t_.dtype == torch.int64 and t_.is_cuda and t_.dim() == 2 and t_.stride(1) == 1, name
    rows, n = r1.shape
    ld = n if ld is None else ld
    assert r2.shape == r1.shape and n == planes.K and a_limbs > 0
    assert rows <= 1 or (r1.stride(0) == ld and r2.stride(0) == ld)
    lut = _lut_on(EXP2_FRAC_LUT_Q23, r1.device, "silu_init_q23")
    if tile_group is not None:
        assert tile_group.dtype == torch.int32 and tile_group.is_cuda and tile_group.is_contiguous()
        assert rows == tile_group.numel() * 128
    if group_shift is not None:
        assert group_shift.dtype == torch.int32 and group_shift.is_cuda and group_shift.is_contiguous()
    C = torch.empty((rows, planes.N), dtype=torch.int64, device=r1.device)
    with _on(r1.device):
        rc = lib.zkds_glu_prepared(r1.data_ptr(), r2.data_ptr(), ld, lut.data_ptr(), rows, planes.handle,
                                   tile_group.data_ptr() if tile_group is not None else None, C.data_ptr(),
                                   int(c_rescale), group_shift.data_ptr() if group_shift is not None else None,
                                   int(n_split), a_limbs,
                                   _a_flags(a_limbs, dynamic) | (_group_rows_flag(max_group_rows) if tile_group is not None else 0),
                                   _stream())
    if rc == 6:
        return None
    _check(rc, "glu_prepared")
    return C


def attention_scores_fused(A, KV, rescale, addin=None, mul=0, div=0, causal=False, start_pos=0,
                           mask_value=-(64 << 36), a_limbs=0, b_limbs=0, dynamic=False):
    """einsum_bshc_btc_bsht with the element-wise tail of the MLA scores in its epilogue:
    out = floor(((sum >> rescale, rounded as the einsum does) + addin) * mul / div) + causal mask
    (model.py:884-905).  mul = div = 0 skips the rescale, addin=None the addition."""
    _dev_i64(A, "A")
    _dev_i64(KV, "KV")
    Bn, S, H, Cd = A.shape
    T = KV.shape[1]
    assert Bn == KV.shape[0] and Cd == KV.shape[2]
    if addin is not None:
        _dev_i64(addin, "addin")
        assert tuple(addin.shape) == (Bn, S, H, T)
    C = torch.empty((Bn, S, H, T), dtype=torch.int64, device=A.device)
    with _on(A.device):
        _check(lib.zkds_einsum_bshc_btc_bsht_ex(A.data_ptr(), KV.data_ptr(), C.data_ptr(), int(rescale), Bn,
                                                S, H, T, Cd, addin.data_ptr() if addin is not None else None,
                                                int(mul), int(div), 1 if causal else 0, int(start_pos),
                                                int(mask_value), a_limbs, b_limbs,
                                                ALGO | _a_flags(a_limbs, dynamic), _stream()),
               "attention_scores_fused")
    return C


def mla_scores_fused(q_abs, kv, q_pe, pe, rescale1=23, rescale2=21, mul=94, div=695, causal=False,
                     start_pos=0, mask_value=-(64 << 36), a_limbs=0, b_limbs=0, dynamic=False,
                     skip_masked=False):
    """scores = ((score1 + score2) * mul // div) (+ causal mask) with score1 = einsum(q_abs, kv) at
    rescale1 and score2 = einsum(q_pe, pe) at rescale2, in one tensor-core pass (model.py:884-905).
    Returns None when the fused kernel does not take the shape (caller falls back)."""
    for t, n in ((q_abs, "q_abs"), (kv, "kv"), (q_pe, "q_pe"), (pe, "pe")):
        _dev_i64(t, n)
    Bn, S, H, C1 = q_abs.shape
    T, C2 = kv.shape[1], q_pe.shape[3]
    assert kv.shape == (Bn, T, C1) and q_pe.shape == (Bn, S, H, C2) and pe.shape == (Bn, T, C2)
    out = torch.empty((Bn, S, H, T), dtype=torch.int64, device=q_abs.device)
    with _on(q_abs.device):
        rc = lib.zkds_mla_scores(q_abs.data_ptr(), kv.data_ptr(), q_pe.data_ptr(), pe.data_ptr(), out.data_ptr(),
                                 Bn, S, H, T, C1, C2, int(rescale1), int(rescale2), int(mul), int(div),
                                 1 if causal else 0, int(start_pos), int(mask_value), a_limbs, b_limbs,
                                 _a_flags(a_limbs, dynamic) | (CAUSAL_SKIP if (skip_masked and causal) else 0),
                                 _stream())
    if rc == 6:          # ZKDS_ERR_UNSUPPORTED
        return None
    _check(rc, "mla_scores_fused")
    return out


class CachePlanes:
    """The MLA latent cache of one layer kept as int8 limb planes (decode): `score` [limbs, B, capacity,
    C1 + round16(C2)] is the cache side of the fused score kernel, `value` [limbs, B, C1, capacity] the KV
    operand of P . KV.  append() splits only the new positions; scores() / softmax_pv() read the planes in
    place, so a decode step neither copies nor re-splits the cache.  `limbs` is a promise (values beyond it
    raise device_status()).  `filled` = positions [0, filled) hold the cache's contents."""

    def __init__(self, batch, capacity, c1, c2, limbs, device):
        self.batch, self.c1, self.c2, self.limbs = int(batch), int(c1), int(c2), int(limbs)
        self.capacity = (int(capacity) + 15) // 16 * 16
        pitch = self.c1 + (self.c2 + 15) // 16 * 16
        self.score = torch.zeros((self.limbs, self.batch, self.capacity, pitch), dtype=torch.int8, device=device)
        self.value = torch.zeros((self.limbs, self.batch, self.c1, self.capacity), dtype=torch.int8, device=device)
        self.filled = 0

    def append(self, kv_new, pe_new, start_pos):
        """kv_new [B, S, C1], pe_new [B, S, C2] -> positions [start_pos, start_pos + S)"""
        _dev_i64(kv_new, "kv_new")
        _dev_i64(pe_new, "pe_new")
        Bn, S, _ = kv_new.shape
        assert Bn == self.batch and kv_new.shape[2] == self.c1 and pe_new.shape == (Bn, S, self.c2)
        assert start_pos + S <= self.capacity
        with _on(kv_new.device):
            _check(lib.zkds_cache_planes_append(kv_new.data_ptr(), pe_new.data_ptr(), self.score.data_ptr(),
                                                self.value.data_ptr(), Bn, S, self.c1, self.c2, int(start_pos),
                                                self.capacity, self.limbs, _stream()), "cache_planes_append")
        self.filled = max(self.filled, start_pos + S) if start_pos <= self.filled else self.filled

    def scores(self, q_abs, q_pe, T, rescale1=23, rescale2=21, mul=94, div=695, causal=False, start_pos=0,
               mask_value=-(64 << 36), a_limbs=3, dynamic=True):
        """mla_scores_fused against positions [0, T) of the planes; None when the kernel declines the shape"""
        _dev_i64(q_abs, "q_abs")
        _dev_i64(q_pe, "q_pe")
        Bn, S, H, C1 = q_abs.shape
        assert Bn == self.batch and C1 == self.c1 and q_pe.shape == (Bn, S, H, self.c2) and T <= self.capacity
        out = torch.empty((Bn, S, H, T), dtype=torch.int64, device=q_abs.device)
        with _on(q_abs.device):
            rc = lib.zkds_mla_scores_cached(q_abs.data_ptr(), q_pe.data_ptr(), self.score.data_ptr(), self.capacity,
                                            out.data_ptr(), Bn, S, H, int(T), C1, self.c2, int(rescale1),
                                            int(rescale2), int(mul), int(div), 1 if causal else 0, int(start_pos),
                                            int(mask_value), a_limbs, self.limbs, _a_flags(a_limbs, dynamic),
                                            _stream())
        if rc == 6:
            return None
        _check(rc, "mla_scores_cached")
        return out

    def softmax_pv(self, scores, rescale=23, a_limbs=3, valid_start=None):
        """softmax_pv_fused with KV = positions [0, T) of the planes; None when the kernel declines the shape.
        valid_start: row (b, s, h) owns columns t <= valid_start + s only, the others are neither read nor
        weighted (a decode step pads its score rows to a multiple of four columns this way)."""
        _dev_i64(scores, "scores")
        Bn, S, H, T = scores.shape
        assert Bn == self.batch and T <= self.capacity
        lut = _lut_on(EXP2_FRAC_LUT_Q19, scores.device, "softmax_init_q19")
        out = torch.empty((Bn, S, H, self.c1), dtype=torch.int64, device=scores.device)
        with _on(scores.device):
            rc = lib.zkds_softmax_pv_cached(scores.data_ptr(), self.value.data_ptr(), self.capacity, out.data_ptr(),
                                            lut.data_ptr(), int(rescale), Bn, S, H, T, self.c1,
                                            0 if valid_start is None else 1,
                                            0 if valid_start is None else int(valid_start), a_limbs,
                                            self.limbs, ALGO_LIMB, _stream())
        if rc == 6:
            return None
        _check(rc, "softmax_pv_cached")
        return out


def gate_select(sigma, bias, n_groups, topk_groups, topk):
    """The gate after its sigmoid (model.py:1140-1211) in one kernel: sigma int64 [T, E], bias int32 [E] or
    None -> (weights int64 [T, topk], indices int64 [T, topk], raw int64 [T, topk]) with
    raw = sigma[indices] and weights = ((raw * 2^23) // sum raw) * 5 // 2.  Experts in descending order of
    sigma + bias, lower index on ties.  Returns None for shapes the kernel does not take."""
    _dev_i64(sigma, "sigma")
    T, E = sigma.shape
    if bias is not None and (bias.dtype != torch.int32 or not bias.is_contiguous() or bias.numel() != E):
        return None
    idx = torch.empty((T, topk), dtype=torch.int64, device=sigma.device)
    raw = torch.empty_like(idx)
    w = torch.empty_like(idx)
    with _on(sigma.device):
        rc = lib.zkds_gate_select(sigma.data_ptr(), bias.data_ptr() if bias is not None else None, T, E,
                                  int(n_groups), int(topk_groups), int(topk), idx.data_ptr(), raw.data_ptr(),
                                  w.data_ptr(), _stream())
    if rc == 6:
        return None
    _check(rc, "gate_select")
    return w, idx, raw


def softmax_q19_causal(R, C, start_pos=0):
    """Q19 softmax of causal scores [B, S, H, T] that reads and writes only columns <= start_pos + s
    of each row (the masked part of R may be unwritten, the masked part of C stays untouched).
    Returns False when the kernel does not take the shape."""
    _dev_i64(R, "R")
    _dev_i64(C, "C")
    Bn, S, H, T = R.shape
    lut = _lut_on(EXP2_FRAC_LUT_Q19, R.device, "softmax_init_q19")
    with _on(R.device):
        rc = lib.zkds_softmax_causal(R.data_ptr(), C.data_ptr(), lut.data_ptr(), Bn, S, H, T, int(start_pos),
                                     _stream())
    if rc == 6:
        return False
    _check(rc, "softmax_q19_causal")
    return True


def softmax_pv_fused(scores, kv, rescale=23, causal_skip=False, start_pos=0, a_limbs=0, b_limbs=0,
                     dynamic=False):
    """einsum_bsht_btc_bshc(softmax_q19(scores), kv, rescale) in one call: scores [B, S, H, T], kv
    [B, T, C] -> [B, S, H, C] (model.py:911-926).  The probabilities go from the softmax kernel straight
    into the limb planes of the contraction and are never stored as int64; `scores` is not modified.
    causal_skip: only columns t <= start_pos + s of a row are read.  Returns None when the kernel does
    not take the shape (use softmax_q19 and the einsum then)."""
    _dev_i64(scores, "scores")
    _dev_i64(kv, "kv")
    Bn, S, H, T = scores.shape
    Cd = kv.shape[2]
    assert Bn == kv.shape[0] and T == kv.shape[1]
    lut = _lut_on(EXP2_FRAC_LUT_Q19, scores.device, "softmax_init_q19")
    out = torch.empty((Bn, S, H, Cd), dtype=torch.int64, device=scores.device)
    flags = ALGO_LIMB | (LIMBS_DYNAMIC if dynamic else 0)
    with _on(scores.device):
        rc = lib.zkds_softmax_pv(scores.data_ptr(), kv.data_ptr(), out.data_ptr(), lut.data_ptr(), int(rescale),
                                 Bn, S, H, T, Cd, 1 if causal_skip else 0, int(start_pos), a_limbs, b_limbs,
                                 flags, _stream())
    if rc == 6:
        return None
    _check(rc, "softmax_pv_fused")
    return out


def einsum_bsht_btc_bshc_causal(A, B, rescale, start_pos=0, a_limbs=3, b_limbs=0):
    """einsum_bsht_btc_bshc for causal probabilities: only columns t <= start_pos + s of A are read."""
    _dev_i64(A, "A")
    _dev_i64(B, "B")
    Bn, S, H, T = A.shape
    Cd = B.shape[2]
    assert Bn == B.shape[0] and T == B.shape[1]
    C = torch.empty((Bn, S, H, Cd), dtype=torch.int64, device=A.device)
    with _on(A.device):
        _check(lib.zkds_einsum_bsht_btc_bshc_causal(A.data_ptr(), B.data_ptr(), C.data_ptr(), int(rescale), Bn, S,
                                                    H, T, Cd, int(start_pos), a_limbs, b_limbs, 0, _stream()),
               "einsum_bsht_btc_bshc_causal")
    return C


def glu_q23(r1, r2, ld=None, want_silu=False):
    """h = (silu_q23(r1) * r2) >> 23 (model.py:1034-1048).  r1, r2: (..., n) views sharing the row
    stride ld (default n).  Returns h, or (h, silu(r1)) when want_silu."""
    n = r1.shape[-1]
    rows = r1.numel() // n if ld is None else r1.shape[0]
    ld = n if ld is None else ld
    lut = _lut_on(EXP2_FRAC_LUT_Q23, r1.device, "silu_init_q23")
    h = torch.empty((rows, n), dtype=torch.int64, device=r1.device)
    s1 = torch.empty_like(h) if want_silu else None
    with _on(r1.device):
        _check(lib.zkds_glu_q23(r1.data_ptr(), r2.data_ptr(), ld, h.data_ptr(),
                                s1.data_ptr() if want_silu else None, lut.data_ptr(), rows, n, _stream()),
               "glu_q23")
    return (h, s1) if want_silu else h


def gather_rows(src, index):
    """dst[r] = src[index[r]] (zeros where index[r] < 0); index int32 on the device."""
    _dev_i64(src, "src")
    assert index.dtype == torch.int32 and index.is_cuda
    rows, cols = index.numel(), src.shape[-1]
    if src.shape[0] == 0:       # nothing to gather from (a rank that received no rows): all padding
        return torch.zeros((rows, cols), dtype=torch.int64, device=src.device)
    dst = torch.empty((rows, cols), dtype=torch.int64, device=src.device)
    with _on(src.device):
        _check(lib.zkds_gather_rows(src.data_ptr(), index.data_ptr(), dst.data_ptr(), rows, cols, _stream()),
               "gather_rows")
    return dst


def moe_combine(out, pos, w, base=None):
    """y[t] = base[t] + sum_slot floor(out[pos[t, slot]] * w[t, slot] / 2^23) (model.py:1379-1383)."""
    _dev_i64(out, "out")
    _dev_i64(w, "w")
    assert pos.dtype == torch.int32 and pos.is_cuda and pos.is_contiguous()
    tokens, slots = pos.shape
    cols = out.shape[-1]
    y = torch.empty((tokens, cols), dtype=torch.int64, device=out.device)
    with _on(out.device):
        _check(lib.zkds_moe_combine(out.data_ptr(), pos.data_ptr(), w.data_ptr(),
                                    base.data_ptr() if base is not None else None, y.data_ptr(), tokens,
                                    slots, cols, _stream()), "moe_combine")
    return y


# ---- expert parallelism over peer memory ------------------------------------------------

def _ptr_array(ptrs):
    return (ctypes.c_void_p * len(ptrs))(*[int(p_) for p_ in ptrs])


def grouped_gather_parts_prepared(part_ptrs, rows_per_part, row_index, planes, tile_group, c_rescale, a_limbs,
                                  dynamic=True, group_shift=None, n_split=0, max_group_rows=None):
    """grouped_prepared(row_index=...) whose source rows lie in len(part_ptrs) buffers of rows_per_part rows
    each (device addresses; the token rows of every GPU, read in place): row_index[m] = g names row
    g % rows_per_part of buffer g // rows_per_part.  The caller keeps the buffers alive and synchronised."""
    assert row_index.dtype == torch.int32 and row_index.is_cuda and row_index.is_contiguous()
    assert tile_group.dtype == torch.int32 and tile_group.is_cuda and tile_group.is_contiguous()
    n_tiles = tile_group.numel()
    assert row_index.numel() == n_tiles * 128 and a_limbs > 0
    if group_shift is not None:
        assert group_shift.dtype == torch.int32 and group_shift.is_cuda and group_shift.is_contiguous()
    C = torch.empty((n_tiles * 128, planes.N), dtype=torch.int64, device=row_index.device)
    with _on(row_index.device):
        _check(lib.zkds_grouped_gather_parts_prepared(
            _ptr_array(part_ptrs), len(part_ptrs), int(rows_per_part), row_index.data_ptr(), planes.handle,
            tile_group.data_ptr(), n_tiles, C.data_ptr(), int(c_rescale),
            group_shift.data_ptr() if group_shift is not None else None, int(n_split), a_limbs,
            _a_flags(a_limbs, dynamic) | _group_rows_flag(max_group_rows), _stream()), "grouped_gather_parts_prepared")
    return C


def moe_combine_peer(out, pos, w, tokens_per_part, slot_ptrs, my_part):
    """the owner's half of the combine: for every gathered token with a local expert, the weighted sum of its
    local experts' rows goes to slot (token, my_part) of the token's home GPU (slot_ptrs: device addresses of
    the GPUs' [tokens_per_part, parts, cols] slot buffers)."""
    _dev_i64(out, "out")
    _dev_i64(w, "w")
    assert pos.dtype == torch.int32 and pos.is_cuda and pos.is_contiguous()
    tokens, slots = pos.shape
    with _on(out.device):
        _check(lib.zkds_moe_combine_peer(out.data_ptr(), pos.data_ptr(), w.data_ptr(), tokens, slots, out.shape[-1],
                                         int(tokens_per_part), _ptr_array(slot_ptrs), len(slot_ptrs), int(my_part),
                                         _stream()), "moe_combine_peer")


def moe_sum_slots(base, slot_rows, indices, experts_per_part):
    """the home GPU's half: y[t] = base[t] + the slots of the owners of token t's experts
    (slot_rows [tokens, parts, cols], indices [tokens, k] int64 global expert ids)."""
    _dev_i64(slot_rows, "slot_rows")
    _dev_i64(indices, "indices")
    tokens, parts, cols = slot_rows.shape
    assert indices.shape[0] == tokens
    if base is not None:
        _dev_i64(base, "base")
        assert base.shape == (tokens, cols)
    y = torch.empty((tokens, cols), dtype=torch.int64, device=slot_rows.device)
    with _on(slot_rows.device):
        _check(lib.zkds_moe_sum_slots(base.data_ptr() if base is not None else None, slot_rows.data_ptr(),
                                      indices.data_ptr(), tokens, indices.shape[1], cols, parts,
                                      int(experts_per_part), y.data_ptr(), _stream()), "moe_sum_slots")
    return y


def peer_barrier(flag_ptrs, my_part, epoch, status):
    """barrier between the GPUs on the current stream (flag_ptrs: device addresses of every GPU's flag array;
    status: int32 device tensor that becomes 1 if the bounded wait ran out)."""
    assert status.dtype == torch.int32 and status.is_cuda
    with _on(status.device):
        _check(lib.zkds_peer_barrier(_ptr_array(flag_ptrs), len(flag_ptrs), int(my_part), int(epoch),
                                     status.data_ptr(), _stream()), "peer_barrier")


# ---- RoPE ----------------------------------------------------------------------------

def complex_int64_mul_broadcast(A, B, shift=42):
    """A (batch, seq, heads, pairs, 2) times the table B (1, seq, 1, pairs, 2).

    Every product keeps bits [shift, shift+64) of the 128-bit product
    (kernel.py:373-395, int64_gemm.cu:223-272; the reference fixes shift = 42).
    """
    _dev_i64(A, "A")
    _dev_i64(B, "B")
    batch, seq, head, pairs = A.shape[0], A.shape[1], A.shape[2], A.shape[3]
    assert B.numel() == seq * pairs * 2, "table must hold one entry per (seq, pair)"
    C = torch.empty(A.shape, dtype=torch.int64, device=A.device)
    with _on(A.device):
        _check(lib.zkds_rope(A.data_ptr(), B.data_ptr(), C.data_ptr(), batch, seq, head, pairs,
                             int(shift), _stream()), "complex_int64_mul_broadcast")
    return C


# ---- RMSNorm -------------------------------------------------------------------------

_RMS_HOST_ENTRIES = 500  # length of the reference's global rms buffer (kernel.py:525)


def rms_norm_int64_device(A, W, eps, dim):
    """Fused RMSNorm, everything on the device: returns (C, rms) with rms int64 [M] on the GPU."""
    _dev_i64(A, "A")
    assert A.ndim == 2 and W.is_cuda and W.is_contiguous()
    assert W.dtype in (torch.int32, torch.int64)
    M, N = A.shape
    C = torch.empty((M, N), dtype=torch.int64, device=A.device)
    rms = torch.empty((M,), dtype=torch.int64, device=A.device)
    with _on(A.device):
        _check(lib.zkds_rms_norm(A.data_ptr(), W.data_ptr(), 32 if W.dtype == torch.int32 else 64,
                                 C.data_ptr(), rms.data_ptr(), M, N, int(eps), int(dim), _stream()),
               "RMS_Norm_int64")
    return C, rms


def RMS_Norm_int64(A, W, eps, dim):
    """Reference surface (kernel.py:528-550): returns (C, rms_cpu)."""
    C, rms_gpu = rms_norm_int64_device(A, W, eps, dim)
    M = A.shape[0]
    rms = torch.zeros((max(_RMS_HOST_ENTRIES, M),), dtype=torch.int64, device="cpu")
    rms[:M] = rms_gpu.cpu()
    return (C, rms)


def rms_norm_apply(A, W, rms):
    """C = floor(A*W / rms[row]) with a caller-provided device rms (int64_gemm.cu:365-385)."""
    _dev_i64(A, "A")
    _dev_i64(rms, "rms")
    M, N = A.shape
    C = torch.empty((M, N), dtype=torch.int64, device=A.device)
    with _on(A.device):
        _check(lib.zkds_rms_norm_apply(A.data_ptr(), W.data_ptr(),
                                       32 if W.dtype == torch.int32 else 64, rms.data_ptr(),
                                       C.data_ptr(), M, N, _stream()), "rms_norm_apply")
    return C


# zkdata dumps.  ASYNC_DUMPS = False writes every file before saveTensor returns, as the reference does (a
# device-to-host copy that stalls the host on the GPU at every dump site).  True: the copy into a pinned host
# buffer is queued on the CURRENT stream (so it reads the tensor exactly where the call stands, before any
# later kernel can overwrite it, e.g. softmax_q19 clobbering its input) and a writer thread stores the file
# once the copy's event has fired; flush_dumps() returns when every file is on disk.  Same bytes either way.
ASYNC_DUMPS = False
_DUMP_QUEUE = None
_DUMP_THREAD = None
_DUMP_ERRORS = []
_PINNED_FREE = {}            # bytes -> [pinned uint8 tensors]: cudaHostAlloc is slow, buffers are reused


def _dump_worker():
    while True:
        item = _DUMP_QUEUE.get()
        try:
            if item is None:
                return
            fileName, buf, nbytes, event = item
            event.synchronize()
            with open(fileName, "wb") as f:
                f.write(buf.numpy()[:nbytes].tobytes())
            _PINNED_FREE.setdefault(buf.numel(), []).append(buf)
        except Exception as err:  # noqa: BLE001 - reported by flush_dumps
            _DUMP_ERRORS.append(err)
        finally:
            _DUMP_QUEUE.task_done()


def flush_dumps():
    """waits until every dump queued by saveTensor is written; raises the first error a write met"""
    if _DUMP_QUEUE is not None:
        _DUMP_QUEUE.join()
    if _DUMP_ERRORS:
        err = _DUMP_ERRORS[0]
        del _DUMP_ERRORS[:]
        raise err


def saveTensor(fileName, t):
    """Raw little-endian C-order dump, no header (kernel.py:553-565)."""
    global _DUMP_QUEUE, _DUMP_THREAD
    t = t.detach()
    if not (ASYNC_DUMPS and t.device.type == "cuda"):
        if t.device.type != "cpu":
            t = t.cpu()
        with open(fileName, "wb") as f:
            f.write(t.contiguous().numpy().tobytes(order="C"))
        return
    import queue
    import threading
    if _DUMP_QUEUE is None:
        _DUMP_QUEUE = queue.Queue()
        _DUMP_THREAD = threading.Thread(target=_dump_worker, daemon=True)
        _DUMP_THREAD.start()
    src = t.contiguous().view(-1).view(torch.uint8)
    nbytes = src.numel()
    size = max(4096, 1 << (max(nbytes, 1) - 1).bit_length())          # size classes: powers of two
    free = _PINNED_FREE.get(size)
    buf = free.pop() if free else torch.empty(size, dtype=torch.uint8, pin_memory=True)
    buf[:nbytes].copy_(src, non_blocking=True)                        # stream-ordered read of the tensor
    event = torch.cuda.Event()
    event.record()
    _DUMP_QUEUE.put((fileName, buf, nbytes, event))


# ---- lookup tables --------------------------------------------------------------------

LOG_TABLE_SIZE = 8
EXP2_FRAC_LUT_Q21 = None
EXP2_FRAC_LUT_Q19 = None
EXP2_FRAC_LUT_Q25 = None
EXP2_FRAC_LUT_Q23 = None


def _host_lut(kind):
    t = torch.zeros((2 ** LOG_TABLE_SIZE,), dtype=torch.int64, device="cpu")
    _check(lib.zkds_lut(t.data_ptr(), kind), "zkds_lut")
    return t


def softmax_init_q19():
    global EXP2_FRAC_LUT_Q19
    EXP2_FRAC_LUT_Q19 = _host_lut(0).cuda()


def softmax_init_q21():
    global EXP2_FRAC_LUT_Q21
    EXP2_FRAC_LUT_Q21 = _host_lut(1).cuda()


def silu_init_q23():
    global EXP2_FRAC_LUT_Q23
    EXP2_FRAC_LUT_Q23 = _host_lut(2).cuda()


def silu_init_q25():
    global EXP2_FRAC_LUT_Q25
    EXP2_FRAC_LUT_Q25 = _host_lut(3).cuda()


def _lut_on(lut, dev, what):
    if lut is None:
        raise RuntimeError("call %s() first" % what)
    return lut if lut.device == dev else lut.to(dev)


# ---- softmax ----------------------------------------------------------------------------

# The reference leaves the unnormalised weights in its input buffer R
# (int64_gemm.cu:708,729).  Keep that side effect by default; model code that never
# looks at R again can switch it off and save a third of the memory traffic.
SOFTMAX_WRITES_WEIGHTS = True


def _softmax(R, C, lut, frac, what):
    _dev_i64(R, "R")
    _dev_i64(C, "C")
    T = R.shape[-1]
    rows = R.numel() // T if T else 0
    w = R.data_ptr() if SOFTMAX_WRITES_WEIGHTS else None
    with _on(R.device):
        _check(lib.zkds_softmax(R.data_ptr(), w, C.data_ptr(), lut.data_ptr(), rows, T, frac,
                                _stream()), what)


def softmax_q21(R, C):
    _softmax(R, C, _lut_on(EXP2_FRAC_LUT_Q21, R.device, "softmax_init_q21"), 21, "softmax_q21")


def softmax_q19(R, C):
    _softmax(R, C, _lut_on(EXP2_FRAC_LUT_Q19, R.device, "softmax_init_q19"), 19, "softmax_q19")


# ---- SiLU / sigmoid ---------------------------------------------------------------------

def _act(R, C, lut, frac, silu, what):
    _dev_i64(R, "R")
    _dev_i64(C, "C")
    with _on(R.device):
        _check(lib.zkds_act(R.data_ptr(), C.data_ptr(), lut.data_ptr(), R.numel(), frac, silu,
                            _stream()), what)


def silu_q25(R, C):
    _act(R, C, _lut_on(EXP2_FRAC_LUT_Q25, R.device, "silu_init_q25"), 25, 1, "silu_q25")


def sigmoid_q25(R, C):
    _act(R, C, _lut_on(EXP2_FRAC_LUT_Q25, R.device, "silu_init_q25"), 25, 0, "sigmoid_q25")


def silu_q23(R, C):
    _act(R, C, _lut_on(EXP2_FRAC_LUT_Q23, R.device, "silu_init_q23"), 23, 1, "silu_q23")


def sigmoid_q23(R, C):
    _act(R, C, _lut_on(EXP2_FRAC_LUT_Q23, R.device, "silu_init_q23"), 23, 0, "sigmoid_q23")
