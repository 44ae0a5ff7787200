"""The circuit-acceptance checker (oracle/circuit_check.py: the constraints of zk/src/index.ts restated in
Python, node and o1js being unavailable) over the zkdata dumps of the seeded model cases.

  * CPU: the dumps the numpy model oracle writes are accepted; a dump with one corrupted word is refused,
    family by family (so the checker does check);
  * GPU: the dumps this repository's model.py writes on the device are accepted.
Known disagreements between the reference's host code and its circuits are warnings, not failures.
"""
import importlib
import os
import sys

import numpy as np
import pytest

from conftest import PKG, ROOT

sys.path.insert(0, os.path.join(ROOT, "tests", "golden"))
import model_cases as mc  # noqa: E402

FIXTURE = os.path.join(ROOT, "tests", "golden", "ref_model_vectors.npz")
SHIFTS = {"tf": {"wq_a": 30, "wkv_a1": 29, "gate": 31}, "mla_full": {"wq_a": 30, "wkv_a1": 29, "gate": 0},
          "gate_full": {"wq_a": 0, "wkv_a1": 0, "gate": 33}, "moe_wide": {"wq_a": 0, "wkv_a1": 0, "gate": 31}}


def _dims(name):
    a = mc.CASES[name]["args"]
    return dict(dim=a["dim"], q_lora=a["q_lora_rank"], kv_lora=a["kv_lora_rank"], heads=a["n_heads"],
                n_experts=a["n_routed_experts"], n_groups=a["n_expert_groups"], topk_groups=a["n_limited_groups"],
                topk=a["n_activated_experts"])


def _prefixes(files):
    return sorted({k.rsplit("/", 1)[0] + "/" for k in files if k.startswith("pos_")})


def _check_all(cc, name, files):
    rep = cc.Report()
    for prefix in _prefixes(files):
        cc.check_layer(files, prefix, _dims(name), SHIFTS[name], rep)
    return rep


@pytest.fixture(scope="module")
def oracle_dumps(orc):
    from oracle import model_oracle as mo
    z = np.load(FIXTURE)
    out = {}
    for name in mc.CASES:
        freqs = z["%s/out/freqs" % name] if ("%s/out/freqs" % name) in z else None
        out[name] = mc.run_case_oracle(mo, name, freqs)[1]
    return out


@pytest.mark.parametrize("name", list(mc.CASES))
def test_checker_accepts_the_oracle_s_dumps(oracle_dumps, name):
    from oracle import circuit_check as cc
    rep = _check_all(cc, name, oracle_dumps[name])
    assert rep.ok(), rep.failures[:10]
    assert sum(rep.checked.values()) > 0
    # the only warnings are the documented host / circuit disagreements
    for w in rep.warnings:
        assert ("truncating division" in w or "host formula" in w or "32-bit mask" in w
                or "saturation rule" in w), w


@pytest.mark.parametrize("family,key,word", [
    ("norm", "pos_0/layer_0/attn_norm_y.bin", 5), ("norm", "pos_0/layer_0/q_norm_rms.bin", 0),
    ("gemm", "pos_0/layer_0/wq_a_y.bin", 17), ("gemm", "pos_0/layer_0/wkv_a1_r.bin", 3),
    ("softmax", "pos_0/layer_0/scores_softmax_y.bin", 1), ("silu", "pos_0/layer_0/mlp_silu_y.bin", 9),
    ("sigmoid", "pos_0/layer_1/sigmoid_gate_y.bin", 2), ("selector", "pos_0/layer_1/gate_indices.bin", 4),
    ("selector", "pos_0/layer_1/gate_weights.bin", 0), ("silu", None, 1)])
def test_checker_refuses_a_corrupted_dump(oracle_dumps, family, key, word):
    from oracle import circuit_check as cc
    files = dict(oracle_dumps["tf"])
    if key is None:
        key = next(k for k in sorted(files) if "expert_" in k and k.endswith("_silu_y.bin"))
    a = np.frombuffer(files[key], np.int64).copy()
    a[word] += 1
    if key.endswith("gate_indices.bin"):
        a[word] = (a[word] + 7) % 32
    files[key] = a.tobytes()
    rep = _check_all(cc, "tf", files)
    assert not rep.ok(), "a corrupted %s went unnoticed" % key
    assert any(key.rsplit("/", 1)[1].split("_")[0] in f or family in f or key[:-6].rsplit("/", 1)[1][:8] in f
               for f in rep.failures), rep.failures


def test_checker_rope_relation():
    from oracle import circuit_check as cc
    from oracle import oracle as orc
    orc.build()
    rng = np.random.default_rng(3)
    x = rng.integers(-2**21, 2**21, (1, 5, 3, 16), dtype=np.int64)
    fr = rng.integers(-2**42, 2**42, (5, 8, 2), dtype=np.int64)
    y = orc.rope(x.reshape(1, 5, 3, 8, 2), fr, 42).reshape(1, 5, 3, 16)
    rep = cc.Report()
    cc.check_rope(rep, "rope", x, fr, y)
    assert rep.ok()
    y[0, 2, 1, 3] -= 1
    cc.check_rope(rep, "rope", x, fr, y)
    assert not rep.ok()


@pytest.mark.gpu
@pytest.mark.parametrize("name", ["tf", "gate_full", "moe_wide"])
def test_checker_accepts_the_cuda_model_s_dumps(kmod, dev, tmp_path, name):
    from oracle import circuit_check as cc
    M = importlib.import_module(PKG + ".model")
    _, dumps = mc.run_case(M, kmod, name, dev, str(tmp_path))
    rep = _check_all(cc, name, mc.normalise_dumps(dumps))
    assert rep.ok(), rep.failures[:10]
    assert sum(rep.checked.values()) > 0
