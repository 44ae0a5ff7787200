"""Model-level parity pinned by the reference's own model.py.

tests/golden/ref_model_vectors.npz holds what the reference's unmodified inference/model.py +
inference/kernel.py + library produced on a B200 for the seeded cases of tests/golden/model_cases.py
(outputs of every step and every zkdata dump file; generator: tests/golden/make_model_golden.py).

  * CPU: oracle/model_oracle.py replays the cases -> the numpy restatement is pinned;
  * GPU: this repository's model.py replays them -> outputs and dump bytes identical;
  * GPU, only where a reference checkout is reachable ($ZKDS_REFERENCE_INFERENCE): the reference's model.py is
    run again on this repository's library and on this repository's kernel.py (the drop-in claim).
"""
import importlib
import json
import os
import subprocess
import sys

import numpy as np
import pytest

from conftest import PKG, ROOT

GOLDEN = os.path.join(ROOT, "tests", "golden")
sys.path.insert(0, GOLDEN)
import model_cases as mc  # noqa: E402

FIXTURE = os.path.join(GOLDEN, "ref_model_vectors.npz")


@pytest.fixture(scope="module")
def fx():
    z = np.load(FIXTURE)
    meta = json.loads(bytes(z["meta"]).decode())
    return z, meta


def check_against_fixture(fx, name, out, files, what):
    z, meta = fx
    rec = meta["cases"][name]
    problems = []
    for k, r in rec["outputs"].items():
        if k == "freqs" and k not in out:
            continue
        v = np.ascontiguousarray(out[k])
        if list(v.shape) != r["shape"] or str(v.dtype) != r["dtype"]:
            problems.append("%s: output %s is %s %s, fixture %s %s" % (name, k, v.dtype, v.shape, r["dtype"], r["shape"]))
        elif mc.digest(v.tobytes()) != r["sha256"]:
            key = "%s/out/%s" % (name, k)
            n = int((z[key] != v).sum()) if key in z else -1
            problems.append("%s: output %s differs from the reference (%d words)" % (name, k, n))
    for k, r in rec["dumps"].items():
        if k not in files:
            problems.append("%s: dump %s not written" % (name, k))
            continue
        data = files[k]
        if len(data) != r["bytes"] or mc.digest(data) != r["sha256"]:
            if k.endswith("gate_indices.bin") and len(data) == r["bytes"] and ("%s/dump/%s" % (name, k)) in z:
                topk = mc.CASES[name]["args"]["n_activated_experts"]
                a = np.sort(np.frombuffer(bytes(z["%s/dump/%s" % (name, k)]), np.int64).reshape(-1, topk), -1)
                b = np.sort(np.frombuffer(data, np.int64).reshape(-1, topk), -1)
                if np.array_equal(a, b):
                    continue        # the same experts in another order: a score tie left to torch.topk
            problems.append("%s: dump %s differs from the reference (%d vs %d bytes)" % (name, k, len(data), r["bytes"]))
    extra = sorted(set(files) - set(rec["dumps"]))
    if extra:
        problems.append("%s: dump files the reference does not write: %s" % (name, extra[:5]))
    assert not problems, "%s:\n  " % what + "\n  ".join(problems[:30])


def test_fixture_records_the_drop_in_run(fx):
    """the generation run compared three more arms with the reference arm: the reference's model.py on this
    library (`so`), on this kernel.py (`py`), and this repository's model.py (`ours`)"""
    _, meta = fx
    assert meta["arms"].get("ref") == 0
    for arm in ("so", "py", "ours"):
        assert meta["arms"].get(arm) == 0, "arm %s did not run in the generation run" % arm
        assert meta["diffs"].get(arm) == [], meta["diffs"].get(arm)


@pytest.mark.parametrize("name", list(mc.CASES))
def test_weights_are_the_generation_run_s(fx, name):
    w, _ = mc.case_data(name)
    assert mc.weights_digest(w) == fx[1]["cases"][name]["weights_sha256"], \
        "numpy's bounded-integer stream changed: regenerate the fixture"


@pytest.mark.parametrize("name", list(mc.CASES))
def test_model_oracle_replays_the_reference(fx, orc, name):
    from oracle import model_oracle as mo
    freqs = fx[0]["%s/out/freqs" % name] if ("%s/out/freqs" % name) in fx[0] else None
    out, files = mc.run_case_oracle(mo, name, freqs)
    files = mc.normalise_dumps(files)
    check_against_fixture(fx, name, out, files, "numpy model oracle vs reference model.py")


@pytest.mark.gpu
@pytest.mark.parametrize("name", list(mc.CASES))
def test_cuda_model_replays_the_reference(fx, kmod, dev, tmp_path, name):
    M = importlib.import_module(PKG + ".model")
    out, dumps = mc.run_case(M, kmod, name, dev, str(tmp_path))
    kmod.device_status()
    check_against_fixture(fx, name, out, mc.normalise_dumps(dumps), "CUDA model vs reference model.py")


@pytest.mark.gpu
def test_reference_model_runs_on_this_library(dev, tmp_path):
    """drop-in, executed: only where the reference checkout is reachable"""
    ref = os.environ.get("ZKDS_REFERENCE_INFERENCE")
    if not ref or not os.path.exists(os.path.join(ref, "model.py")):
        pytest.skip("no reference checkout here (set ZKDS_REFERENCE_INFERENCE); the generation run's result is "
                    "recorded in the fixture")
    if not os.path.exists(os.path.join(ROOT, "oracle", "_ref", "libint64gemm_ref.so")):
        pytest.skip("reference library not built (oracle/_ref)")
    r = subprocess.run([sys.executable, os.path.join(GOLDEN, "make_model_golden.py"), "--reference", ref,
                        "--arms", "ref,so,py", "--out", str(tmp_path / "again.npz"), "--keep", str(tmp_path)],
                       capture_output=True, text=True)
    assert r.returncode == 0, (r.stdout + r.stderr)[-3000:]
