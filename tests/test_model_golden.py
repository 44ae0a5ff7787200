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


def check_against_fixture(fx, name, out, files, what, outputs=True):
    z, meta = fx
    rec = meta["cases"][name]
    problems = []
    for k, r in rec["outputs"].items() if outputs else ():
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


def _write_converted_checkpoint(ck, a, w):
    """the converted layout generate.py reads: embed/norm/head_int.safetensors, layer-{i}.safetensors with
    Block's state-dict keys (convert2.py:13-32,591), experts-{layer}/{i}.safetensors"""
    import torch
    from safetensors.torch import save_file
    tt = lambda x: torch.from_numpy(np.ascontiguousarray(x))
    sc = lambda v: torch.tensor(v, dtype=torch.int32)
    for name in ("embed", "norm", "head"):
        save_file({"weight": tt(w[name])}, os.path.join(ck, name + "_int.safetensors"))

    def mlp(prefix, p, sd):
        for n in ("w1", "w2", "w3"):
            sd[prefix + n + ".weight"] = tt(p[n])
            sd[prefix + n + ".scale"] = sc(p[n + "_scale"])

    for i, p in enumerate(w["layers"]):
        sd = {"attn_norm.weight": tt(p["attn_norm"]), "ffn_norm.weight": tt(p["ffn_norm"]),
              "attn.q_norm.weight": tt(p["attn"]["q_norm"]), "attn.kv_norm.weight": tt(p["attn"]["kv_norm"])}
        for n in ("wq_a", "wq_b1", "wq_b2", "wkv_a1", "wkv_a2", "wkv_b_1", "wkv_b_2", "wo"):
            sd["attn.%s.weight" % n] = tt(p["attn"][n])
            if n + "_scale" in p["attn"]:
                sd["attn.%s.scale" % n] = sc(p["attn"][n + "_scale"])
        f = p["ffn"]
        if "experts" in f:
            sd["ffn.gate.weight"], sd["ffn.gate.scale"] = tt(f["gate"]["weight"]), sc(f["gate"]["scale"])
            sd["ffn.gate.bias"] = tt(f["gate"]["bias"])
            mlp("ffn.shared_experts.", f["shared"], sd)
            mc.write_experts(ck, i, f["experts"])
        else:
            mlp("ffn.", f, sd)
        save_file(sd, os.path.join(ck, "layer-%d.safetensors" % i))


@pytest.mark.gpu
def test_generate_from_a_converted_checkpoint_gives_the_reference_tokens(fx, kmod, dev, tmp_path):
    """load_resident + generate() (this repository's generate.py) on the `tf` case: the tokens and the
    pos_{p}/tokens.bin files are those of the reference's model.py driven by its own token loop"""
    M = importlib.import_module(PKG + ".model")
    G = importlib.import_module(PKG + ".generate")
    c = mc.CASES["tf"]
    w, x = mc.case_data("tf")
    ck = str(tmp_path / "ckpt")
    os.makedirs(ck)
    a = M.ModelArgs(**c["args"])
    _write_converted_checkpoint(ck, a, w)
    model = G.load_resident(ck, a, dev)
    want = fx[0]["tf/out/tokens"]
    prompt = [int(v) for v in x["prompt"]]
    zk = str(tmp_path / "zk")
    M.snark, M.zkDataDir = True, zk
    try:
        trace = []
        got = G.generate(model, [prompt], c["new_tokens"], eos_id=-5, temperature=0.0, trace=trace)
    finally:
        M.snark, M.zkDataDir = False, "../zkdata"
    assert got == [want[len(prompt):].tolist()]
    assert not any(s.get("rerun_measured") for s in trace)
    pos = 0
    for n in (len(prompt), 1, 1):
        toks = np.fromfile(os.path.join(zk, "pos_%d" % pos, "tokens.bin"), np.int64)
        assert np.array_equal(toks, want[pos:pos + n])
        pos += n
    # the layer dumps written on the way are the reference's too
    dumps = mc.normalise_dumps({k: v for k, v in mc.read_dumps(zk).items() if not k.endswith("tokens.bin")})
    check_against_fixture(fx, "tf", {}, dumps, "dumps written under generate()", outputs=False)
    kmod.device_status()


@pytest.mark.gpu
def test_asynchronous_dump_writer_gives_the_same_files(fx, kmod, dev, tmp_path):
    """kernel.ASYNC_DUMPS: dumps leave through pinned buffers and a writer thread; after flush_dumps() the
    files are byte for byte the reference's (the `tf` case: scores dumped before softmax overwrites them)"""
    M = importlib.import_module(PKG + ".model")
    kmod.ASYNC_DUMPS = True
    try:
        out, _ = mc.run_case(M, kmod, "tf", dev, str(tmp_path))
        kmod.flush_dumps()
    finally:
        kmod.ASYNC_DUMPS = False
    dumps = mc.read_dumps(os.path.join(str(tmp_path), "zkdata_tf"))
    check_against_fixture(fx, "tf", out, mc.normalise_dumps(dumps), "asynchronous dumps vs reference model.py")
