"""Generates tests/golden/ref_model_vectors.npz by running the reference's OWN, unmodified
inference/model.py + inference/kernel.py on a GPU, and executes the drop-in claim on the way.

    python tests/golden/make_model_golden.py --reference <checkout>/inference [--out FILE] [--keep DIR]

Needs a CUDA device, the reference checkout (not part of this repository; pass its location or set
ZKDS_REFERENCE_INFERENCE), its library built by oracle/Makefile (oracle/_ref/libint64gemm_ref.so) and this
repository's library.  Every arm runs the cases of model_cases.py in a process of its own:

    ref   reference model.py, reference kernel.py, ./libint64gemm.so -> the reference's library
    so    reference model.py, reference kernel.py, ./libint64gemm.so -> this repository's library
    py    reference model.py, this repository's kernel.py imported as `kernel`
    ours  this repository's model.py and kernel.py

`ref` is what the fixture records (outputs and every zkdata dump file: digests, and the data itself when
small).  `so` and `py` must reproduce it byte for byte — that is the drop-in check; `ours` is compared
too so that one run tells everything.  The reference stays inside its own limits here (batch 1, at most
500 rows per RMSNorm, T, C, D, H at most 1024; kernel.py:525, int64_gemm.cu:419-545).
"""
import argparse
import importlib
import importlib.util
import json
import os
import pickle
import subprocess
import sys
import tempfile

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
PKG = os.path.join(ROOT, "zk-deepseek_b200")
sys.path.insert(0, HERE)
import model_cases as mc  # noqa: E402

ARMS = ("ref", "so", "py", "ours")


def run_arm(arm, reference, work):
    """child process: import the modules of this arm and run every case"""
    import torch
    dev = torch.device("cuda:0")
    run = os.path.join(work, "run_" + arm)
    os.makedirs(run, exist_ok=True)
    os.chdir(run)
    if arm in ("ref", "so"):
        target = (os.path.join(ROOT, "oracle", "_ref", "libint64gemm_ref.so") if arm == "ref"
                  else os.path.join(PKG, "libint64gemm.so"))
        if os.path.lexists("libint64gemm.so"):
            os.remove("libint64gemm.so")
        os.symlink(target, "libint64gemm.so")          # kernel.py:206 loads ./libint64gemm.so
        sys.path.insert(0, reference)
        Kmod = importlib.import_module("kernel")
        M = importlib.import_module("model")
    elif arm == "py":
        spec = importlib.util.spec_from_file_location("kernel", os.path.join(PKG, "kernel.py"))
        Kmod = importlib.util.module_from_spec(spec)
        sys.modules["kernel"] = Kmod
        spec.loader.exec_module(Kmod)
        sys.path.insert(0, reference)
        M = importlib.import_module("model")           # the reference's model.py on this kernel.py
    else:
        sys.path.insert(0, ROOT)
        Kmod = importlib.import_module("zk-deepseek_b200.kernel")
        M = importlib.import_module("zk-deepseek_b200.model")
    assert os.path.dirname(os.path.abspath(M.__file__)) == (PKG if arm == "ours" else os.path.abspath(reference))
    res = {"modules": {"model": M.__file__, "kernel": Kmod.__file__}}
    real_stdout = sys.stdout
    sys.stdout = open(os.devnull, "w")                 # the reference prints every intermediate
    try:
        for name in mc.CASES:
            out, dumps = mc.run_case(M, Kmod, name, dev, run)
            res[name] = (out, mc.normalise_dumps(dumps))
    finally:
        sys.stdout = real_stdout
    if arm in ("py", "ours"):
        Kmod.device_status()
    with open(os.path.join(work, arm + ".pkl"), "wb") as f:
        pickle.dump(res, f, protocol=4)


def compare(base, other, label):
    """list of differences between two arms' results"""
    diffs = []
    for name in mc.CASES:
        bo, bd = base[name]
        oo, od = other[name]
        for k in bo:
            if k not in oo or bo[k].shape != oo[k].shape or not np.array_equal(bo[k], oo[k]):
                n = -1 if k not in oo or bo[k].shape != oo[k].shape else int((bo[k] != oo[k]).sum())
                diffs.append("%s: %s/%s differs (%d words)" % (label, name, k, n))
        for k in bd:
            if k not in od:
                diffs.append("%s: %s dump %s missing" % (label, name, k))
            elif bd[k] != od[k]:
                if k.endswith("gate_indices.bin"):
                    a = np.sort(np.frombuffer(bd[k], np.int64).reshape(-1, mc.CASES[name]["args"]["n_activated_experts"]), -1)
                    b = np.sort(np.frombuffer(od[k], np.int64).reshape(a.shape), -1)
                    if np.array_equal(a, b):
                        continue                       # same experts, tie order only
                diffs.append("%s: %s dump %s differs (%d vs %d bytes)" % (label, name, k, len(bd[k]), len(od[k])))
        for k in od:
            if k not in bd:
                diffs.append("%s: %s dump %s is extra" % (label, name, k))
    return diffs


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", default=os.environ.get("ZKDS_REFERENCE_INFERENCE"),
                    help="directory holding the reference's kernel.py and model.py")
    ap.add_argument("--out", default=os.path.join(HERE, "ref_model_vectors.npz"))
    ap.add_argument("--work", default=None)
    ap.add_argument("--arm", default=None, choices=ARMS)
    ap.add_argument("--arms", default=",".join(ARMS))
    ap.add_argument("--keep", default=None, help="also store every arm's raw results (pickle) in this directory")
    opt = ap.parse_args()
    if not opt.reference or not os.path.exists(os.path.join(opt.reference, "model.py")):
        sys.exit("pass --reference <checkout>/inference (the directory with model.py and kernel.py)")
    opt.reference = os.path.abspath(opt.reference)
    if opt.arm:
        run_arm(opt.arm, opt.reference, opt.work)
        return
    work = opt.keep or tempfile.mkdtemp(prefix="zkds_model_golden_")
    os.makedirs(work, exist_ok=True)
    arms = opt.arms.split(",")
    results, status = {}, {}
    for arm in arms:
        r = subprocess.run([sys.executable, os.path.abspath(__file__), "--reference", opt.reference, "--arm", arm,
                            "--work", work], capture_output=True, text=True)
        status[arm] = r.returncode
        if r.returncode != 0:
            print("arm %s failed (%d):\n%s" % (arm, r.returncode, (r.stdout + r.stderr)[-4000:]))
            continue
        with open(os.path.join(work, arm + ".pkl"), "rb") as f:
            results[arm] = pickle.load(f)
        print("arm %-4s ok   model=%s kernel=%s" % (arm, results[arm]["modules"]["model"],
                                                  results[arm]["modules"]["kernel"]))
    if "ref" not in results:
        sys.exit("the reference arm did not run: no fixture written")
    ref = results["ref"]
    meta = {"arms": status, "diffs": {}, "cases": {}}
    for arm in arms:
        if arm != "ref" and arm in results:
            d = compare(ref, results[arm], arm)
            meta["diffs"][arm] = d
            print("arm %-4s vs ref: %s" % (arm, "identical" if not d else "%d differences" % len(d)))
            for line in d[:40]:
                print("   " + line)
    arrays = {}
    for name in mc.CASES:
        out, dumps = ref[name]
        w, _ = mc.case_data(name)
        rec = {"weights_sha256": mc.weights_digest(w), "outputs": {}, "dumps": {}}
        for k, v in out.items():
            v = np.ascontiguousarray(v)
            rec["outputs"][k] = {"shape": list(v.shape), "dtype": str(v.dtype), "sha256": mc.digest(v.tobytes())}
            if v.nbytes <= mc.KEEP_BYTES or k in ("freqs", "tokens"):
                arrays["%s/out/%s" % (name, k)] = v
        for k, data in dumps.items():
            rec["dumps"][k] = {"bytes": len(data), "sha256": mc.digest(data)}
            if len(data) <= mc.KEEP_BYTES:
                arrays["%s/dump/%s" % (name, k)] = np.frombuffer(data, np.uint8)
        meta["cases"][name] = rec
    arrays["meta"] = np.frombuffer(json.dumps(meta).encode(), np.uint8)
    np.savez_compressed(opt.out, **arrays)
    print("wrote %s (%d arrays, %d bytes)" % (opt.out, len(arrays), os.path.getsize(opt.out)))
    bad = [a for a in arms if status.get(a) != 0 or meta["diffs"].get(a)]
    sys.exit(1 if bad else 0)


if __name__ == "__main__":
    main()
