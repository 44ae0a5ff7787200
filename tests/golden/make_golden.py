"""Regenerates the CPU-side golden fixtures from the reference checkout.

Run where the reference is mounted:  python tests/golden/make_golden.py [REF_ROOT]

  ts_tables.json  the two 256-entry exp2 tables and the LOG2E constants that the
                  reference's circuits hard-code (zk/src/index.ts), read as text
  ref_luts.json   the four tables produced by the reference's own host functions
                  (softmax_init_q19/q21, silu_init_q23/q25), called through
                  ctypes from the library oracle/Makefile builds out of the
                  reference's source
"""
import ctypes
import json
import os
import re
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))


def ts_tables(ref_root):
    src = open(os.path.join(ref_root, "zk/src/index.ts"), encoding="utf-8").read()
    out = {}
    for name in ("q19Table", "q23Table"):
        body = re.search(r"const %s = \[(.*?)\]" % name, src, re.S).group(1)
        vals = [int(v) for v in re.findall(r"UInt64\.from\((\d+)n\)", body)]
        assert len(vals) == 256, (name, len(vals))
        out[name] = vals
    out["LOG2E_Q19"] = int(re.search(r"const LOG2E_Q19 = UInt64\.from\((\d+)n\)", src).group(1))
    out["LOG2E_Q23"] = int(re.search(r"const LOG2E_Q23 = (\d+)n", src).group(1))
    return out


def ref_luts():
    so = os.path.join(ROOT, "oracle/_ref/libint64gemm_ref.so")
    lib = ctypes.CDLL(so)
    out = {}
    for name in ("softmax_init_q19", "softmax_init_q21", "silu_init_q23", "silu_init_q25"):
        buf = (ctypes.c_int64 * 256)()
        getattr(lib, name)(buf)
        out[name] = list(buf)
    return out


if __name__ == "__main__":
    ref_root = sys.argv[1] if len(sys.argv) > 1 else os.environ.get("ZKDS_REFERENCE", "")
    if not os.path.isdir(ref_root):
        sys.exit("usage: make_golden.py <reference checkout>   (or set ZKDS_REFERENCE)")
    json.dump(ts_tables(ref_root), open(os.path.join(HERE, "ts_tables.json"), "w"))
    json.dump(ref_luts(), open(os.path.join(HERE, "ref_luts.json"), "w"))
    print("wrote ts_tables.json, ref_luts.json")
