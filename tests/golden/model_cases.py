"""Seeded model-level cases shared by the fixture generator (make_model_golden.py) and the
tests that replay its fixture (ref_model_vectors.npz).

A case fixes the ModelArgs, the weights (drawn here from numpy's PCG64 bounded-integer
generator, so nothing but a seed has to be stored), the inputs and the sequence of forward
calls.  `run_case` drives any module with the class surface of the reference's
inference/model.py (the reference's own module or this repository's), `run_case_oracle` the
numpy restatement.  Both return {name: ndarray} of outputs plus the zkdata dump files.

Scales follow the reference's fixed-point flow (residual 2^31, attn-normed 2^21, q 2^19,
kv 2^23, ffn-normed / SiLU 2^23, logits 2^21): convert2.py:37-88,250-295, model.py:702-712.
"""
import hashlib
import math
import os

import numpy as np

MASK_VALUE = -(64 << 36)            # model.py:1555

_TF = dict(max_seq_len=64, vocab_size=512, dim=7168, inter_dim=256, moe_inter_dim=64, n_layers=2,
           n_dense_layers=1, n_heads=4, n_routed_experts=32, n_shared_experts=1, n_activated_experts=8,
           n_expert_groups=8, n_limited_groups=4, score_func="sigmoid", route_scale=2.5, q_lora_rank=128,
           kv_lora_rank=64, qk_nope_head_dim=32, qk_rope_head_dim=16, v_head_dim=32)
_FULL = dict(max_seq_len=16384, vocab_size=512, dim=7168, inter_dim=18432, moe_inter_dim=2048, n_layers=1,
             n_dense_layers=1, n_heads=128, n_routed_experts=256, n_shared_experts=1, n_activated_experts=8,
             n_expert_groups=8, n_limited_groups=4, score_func="sigmoid", route_scale=2.5, q_lora_rank=1536,
             kv_lora_rank=512, qk_nope_head_dim=128, qk_rope_head_dim=64, v_head_dim=128)
_WIDE = dict(_TF, n_routed_experts=16, n_activated_experts=4, n_expert_groups=4, n_limited_groups=2)

CASES = {
    # embed -> dense Block -> MoE Block -> norm -> head, greedy: a 12-token prefill and two decode steps
    "tf": dict(kind="transformer", args=_TF, seed=101, prompt_len=12, new_tokens=3),
    # one attention layer at the full DeepSeek-V3 width with the YaRN-corrected table
    "mla_full": dict(kind="mla", args=_FULL, seed=102, steps=(12, 1)),
    # the 256-expert gate with its bias: top-2-sum group scores, 4 of 8 groups, top 8
    "gate_full": dict(kind="gate", args=_FULL, seed=103, tokens=48),
    # experts that receive more than 128 rows each
    "moe_wide": dict(kind="moe", args=_WIDE, seed=104, tokens=640),
}


# ------------------------------------------------------------------------------------------
# weights
def _wmat(rng, out_f, in_f, bits, dtype=np.int32):
    a = min(int(round(1.7 * 2.0 ** bits / math.sqrt(in_f))), 2 ** 31 - 1 if dtype == np.int32 else 2 ** 62)
    return rng.integers(-a, a + 1, (out_f, in_f), dtype=np.int64).astype(dtype)


def _nvec(rng, n, bits, dtype=np.int32):
    return (2 ** bits + rng.integers(-2 ** (bits - 2), 2 ** (bits - 2), n, dtype=np.int64)).astype(dtype)


def mla_weights(rng, a):
    H = a["n_heads"]
    return {"wq_a": _wmat(rng, a["q_lora_rank"], a["dim"], 30), "q_norm": _nvec(rng, a["q_lora_rank"], 19),
            "wq_b1": _wmat(rng, H * a["qk_nope_head_dim"], a["q_lora_rank"], 30),
            "wq_b2": _wmat(rng, H * a["qk_rope_head_dim"], a["q_lora_rank"], 30),
            "wkv_a1": _wmat(rng, a["kv_lora_rank"], a["dim"], 29),
            "wkv_a2": _wmat(rng, a["qk_rope_head_dim"], a["dim"], 29),
            "kv_norm": _nvec(rng, a["kv_lora_rank"], 23),
            "wkv_b_1": _wmat(rng, H * a["qk_nope_head_dim"], a["kv_lora_rank"], 31), "wkv_b_1_scale": 31,
            "wkv_b_2": _wmat(rng, H * a["v_head_dim"], a["kv_lora_rank"], 30), "wkv_b_2_scale": 30,
            "wo": _wmat(rng, a["dim"], H * a["v_head_dim"], 31), "wo_scale": 31}


def mlp_weights(rng, dim, inter, s1=31, s3=31, s2=29):
    return {"w1": _wmat(rng, inter, dim, s1), "w1_scale": s1, "w3": _wmat(rng, inter, dim, s3), "w3_scale": s3,
            "w2": _wmat(rng, dim, inter, s2), "w2_scale": s2}


def gate_weights(rng, a, scale=31):
    return {"weight": _wmat(rng, a["n_routed_experts"], a["dim"], scale), "scale": scale,
            "bias": (2 ** 20 + rng.integers(-2 ** 19, 2 ** 19, a["n_routed_experts"], dtype=np.int64)
                     ).astype(np.int32)}


def moe_weights(rng, a):
    return {"gate": gate_weights(rng, a),
            "shared": mlp_weights(rng, a["dim"], a["n_shared_experts"] * a["moe_inter_dim"], 32, 32, 28),
            "experts": [mlp_weights(rng, a["dim"], a["moe_inter_dim"], 31 + (i % 3), 31 + (i % 2), 28 + (i % 3))
                        for i in range(a["n_routed_experts"])]}


def block_weights(rng, a, layer_id):
    p = {"attn": mla_weights(rng, a), "attn_norm": _nvec(rng, a["dim"], 21), "ffn_norm": _nvec(rng, a["dim"], 23)}
    if layer_id < a["n_dense_layers"]:
        p["ffn"] = mlp_weights(rng, a["dim"], a["inter_dim"])
    else:
        p["ffn"] = moe_weights(rng, a)
    return p


def case_data(name):
    """(weights, inputs) of a case, as numpy arrays"""
    c = CASES[name]
    a = c["args"]
    rng = np.random.Generator(np.random.PCG64(c["seed"]))
    kind = c["kind"]
    if kind == "transformer":
        w = {"embed": rng.integers(-2 ** 28, 2 ** 28, (a["vocab_size"], a["dim"]), dtype=np.int64),
             "norm": _nvec(rng, a["dim"], 15, np.int64),
             "head": _wmat(rng, a["vocab_size"], a["dim"], 43, np.int64),
             "layers": [block_weights(rng, a, i) for i in range(a["n_layers"])]}
        x = {"prompt": rng.integers(0, a["vocab_size"], c["prompt_len"], dtype=np.int64)}
    elif kind == "mla":
        w = mla_weights(rng, a)
        x = {"x%d" % i: rng.integers(-2 ** 22, 2 ** 22, (1, S, a["dim"]), dtype=np.int64)
             for i, S in enumerate(c["steps"])}
    elif kind == "gate":
        w = gate_weights(rng, a, 33)
        x = {"x": rng.integers(-2 ** 24, 2 ** 24, (c["tokens"], a["dim"]), dtype=np.int64)}
    elif kind == "moe":
        w = moe_weights(rng, a)
        x = {"x": rng.integers(-2 ** 24, 2 ** 24, (1, c["tokens"], a["dim"]), dtype=np.int64)}
    else:
        raise KeyError(kind)
    return w, x


def weights_digest(w):
    """sha256 over every array of a weight tree in a fixed order: detects a drifting generator"""
    h = hashlib.sha256()

    def walk(o):
        if isinstance(o, dict):
            for k in sorted(o):
                h.update(k.encode())
                walk(o[k])
        elif isinstance(o, (list, tuple)):
            for v in o:
                walk(v)
        elif isinstance(o, np.ndarray):
            h.update(np.ascontiguousarray(o).tobytes())
        else:
            h.update(repr(o).encode())
    walk(w)
    return h.hexdigest()


# ------------------------------------------------------------------------------------------
# driving a torch module tree with the reference's class surface
def _t(arr, dev):
    import torch
    return torch.from_numpy(np.ascontiguousarray(arr)).to(dev)


def _set_linear(mod, w, scale, dev):
    import torch
    mod.weight = _t(w, dev)
    if scale is not None:
        mod.scale = torch.tensor(scale, dtype=torch.int32, device=dev)


def load_mla(attn, p, dev):
    for n in ("wq_a", "wq_b1", "wq_b2", "wkv_a1", "wkv_a2"):
        _set_linear(getattr(attn, n), p[n], None, dev)
    for n in ("wkv_b_1", "wkv_b_2", "wo"):
        _set_linear(getattr(attn, n), p[n], p[n + "_scale"], dev)
    attn.q_norm.weight = _t(p["q_norm"], dev)
    attn.kv_norm.weight = _t(p["kv_norm"], dev)


def load_mlp(mlp, p, dev):
    for n in ("w1", "w2", "w3"):
        _set_linear(getattr(mlp, n), p[n], p[n + "_scale"], dev)


def write_experts(ckpt, layer_id, experts):
    """experts-{layer}/{i}.safetensors with the keys Expert_int's state dict has (model.py:1359-1363)"""
    import torch
    from safetensors.torch import save_file
    d = os.path.join(ckpt, "experts-%d" % layer_id)
    os.makedirs(d, exist_ok=True)
    for i, e in enumerate(experts):
        sd = {}
        for n in ("w1", "w2", "w3"):
            sd[n + ".weight"] = torch.from_numpy(e[n])
            sd[n + ".scale"] = torch.tensor(e[n + "_scale"], dtype=torch.int32)
        save_file(sd, os.path.join(d, "%d.safetensors" % i))


def build_moe(M, layer_id, a, p, dev, ckpt):
    import torch
    write_experts(ckpt, layer_id, p["experts"])
    with torch.device(dev):
        moe = M.MoE(layer_id, a, ckpt)
    _set_linear(moe.gate, p["gate"]["weight"], p["gate"]["scale"], dev)
    moe.gate.bias = _t(p["gate"]["bias"], dev)
    load_mlp(moe.shared_experts, p["shared"], dev)
    if hasattr(moe, "set_experts"):         # resident experts: read the same files once
        moe.set_experts()
    return moe


def build_block(M, layer_id, a, p, dev, ckpt):
    import torch
    if "experts" in p["ffn"]:
        write_experts(ckpt, layer_id, p["ffn"]["experts"])
    with torch.device(dev):
        blk = M.Block(layer_id, a, ckpt)
    load_mla(blk.attn, p["attn"], dev)
    blk.attn_norm.weight = _t(p["attn_norm"], dev)
    blk.ffn_norm.weight = _t(p["ffn_norm"], dev)
    if "experts" in p["ffn"]:
        f = p["ffn"]
        _set_linear(blk.ffn.gate, f["gate"]["weight"], f["gate"]["scale"], dev)
        blk.ffn.gate.bias = _t(f["gate"]["bias"], dev)
        load_mlp(blk.ffn.shared_experts, f["shared"], dev)
        if hasattr(blk.ffn, "set_experts"):
            blk.ffn.set_experts()
    else:
        load_mlp(blk.ffn, p["ffn"], dev)
    return blk


def _np(tensor):
    return tensor.detach().cpu().numpy().copy()


def read_dumps(zkdir):
    """{relative path: bytes} of every file under the dump directory"""
    out = {}
    for root, _, files in os.walk(zkdir):
        for f in files:
            p = os.path.join(root, f)
            with open(p, "rb") as fh:
                out[os.path.relpath(p, zkdir).replace(os.sep, "/")] = fh.read()
    return out


def run_case(M, Kmod, name, dev, workdir):
    """Run a case on module M (class surface of inference/model.py) with kernel module Kmod.
    Returns (outputs {name: ndarray}, dumps {relative path: bytes})."""
    import torch
    c = CASES[name]
    a = M.ModelArgs(**c["args"])
    w, x = case_data(name)
    zk = os.path.join(workdir, "zkdata_" + name)
    ckpt = os.path.join(workdir, "ckpt_" + name)
    os.makedirs(zk, exist_ok=True)
    os.makedirs(ckpt, exist_ok=True)
    old = (M.snark, M.zkDataDir)
    M.snark, M.zkDataDir = True, zk
    Kmod.softmax_init_q19()
    Kmod.silu_init_q23()
    out = {}
    try:
        with torch.inference_mode():
            kind = c["kind"]
            if kind == "transformer":
                with torch.device(dev):
                    model = M.Transformer(a)
                model.embed.weight = _t(w["embed"], dev)
                model.norm.weight = _t(w["norm"], dev)
                model.head.weight = _t(w["head"], dev)
                for i in range(a.n_layers):
                    model.layers[i] = build_block(M, i, a, w["layers"][i], dev, ckpt)
                seq = [int(v) for v in x["prompt"]]
                prev = 0
                for step in range(c["new_tokens"]):
                    toks = torch.tensor([seq[prev:]], dtype=torch.long, device=dev)
                    h, pos, S = model.prep_inference(toks, prev)
                    out["step%d_embed" % step] = _np(h)
                    for i in range(a.n_layers):
                        h = model.layer_inference(i, h, pos, S)
                        out["step%d_layer%d" % (step, i)] = _np(h)
                    logits = model.finish_inference(h)
                    out["step%d_logits" % step] = _np(logits)
                    prev = len(seq)
                    seq.append(int(logits.argmax(dim=-1).view(-1)[0]))
                out["tokens"] = np.array(seq, dtype=np.int64)
                out["freqs"] = _np(model.freqs_cis[:len(seq)])
            elif kind == "mla":
                with torch.device(dev):
                    attn = M.MLA(0, a)
                    freqs = M.precompute_freqs_cis(a)
                load_mla(attn, w, dev)
                pos = 0
                for i, S in enumerate(c["steps"]):
                    mask = None
                    if S > 1:
                        mask = torch.full((S, S), MASK_VALUE, dtype=torch.int64, device=dev).triu_(1)
                    y = attn(_t(x["x%d" % i], dev), pos, freqs[pos:pos + S].to(dev), mask)
                    out["step%d_out" % i] = _np(y)
                    pos += S
                out["freqs"] = _np(freqs[:pos])
                out["kv_cache"] = _np(attn.kv_cache[:, :pos])
                out["pe_cache"] = _np(attn.pe_cache[:, :pos])
            elif kind == "gate":
                with torch.device(dev):
                    gate = M.Gate(1, a)
                _set_linear(gate, w["weight"], w["scale"], dev)
                gate.bias = _t(w["bias"], dev)
                os.makedirs(os.path.join(zk, "pos_0", "layer_1"), exist_ok=True)
                wts, idx = gate(0, _t(x["x"], dev))
                out["weights"], out["indices"] = _np(wts), _np(idx)
            elif kind == "moe":
                moe = build_moe(M, 1, a, w, dev, ckpt)
                os.makedirs(os.path.join(zk, "pos_0", "layer_1"), exist_ok=True)
                out["out"] = _np(moe(0, _t(x["x"], dev)))
            torch.cuda.synchronize()
    finally:
        M.snark, M.zkDataDir = old
    return out, read_dumps(zk)


# ------------------------------------------------------------------------------------------
# the numpy restatement on the same cases
def _oracle_dump_files(dumps, pos, layer):
    files = {}
    for k, v in dumps.items():
        path = "freqs_cis.bin" if k == "freqs_cis" else "pos_%d/layer_%d/%s.bin" % (pos, layer, k)
        files[path] = np.ascontiguousarray(v).tobytes()
    return files


def run_case_oracle(mo, name, freqs, indices=None):
    """The same case through oracle/model_oracle.py.  `freqs` is the RoPE table of the fixture (the
    table is float32 work of the device it was computed on, so it is an input here).  `indices`
    optionally fixes the experts chosen per call (list in call order) to follow score ties."""
    c = CASES[name]
    a = c["args"]
    w, x = case_data(name)
    out, files = {}, {}
    kind = c["kind"]
    H = a["n_heads"]
    g = (a["n_expert_groups"], a["n_limited_groups"], a["n_activated_experts"])
    if kind == "transformer":
        from oracle import oracle as orc
        L = a["n_layers"]
        kv = [np.zeros((1, a["max_seq_len"], a["kv_lora_rank"]), np.int64) for _ in range(L)]
        pe = [np.zeros((1, a["max_seq_len"], a["qk_rope_head_dim"]), np.int64) for _ in range(L)]
        seq = [int(v) for v in x["prompt"]]
        prev = 0
        for step in range(c["new_tokens"]):
            toks = np.array(seq[prev:])
            S = len(toks)
            h = w["embed"][toks][None]                                # F.embedding, model.py:145
            out["step%d_embed" % step] = h
            fr = freqs[prev:prev + S]
            mask = mo.causal_mask(S)
            for i in range(L):
                p = w["layers"][i]
                d = {}
                if "experts" in p["ffn"]:
                    ffn = lambda y, p=p, d=d: mo.moe_forward(p["ffn"], y, *g, dumps=d)[0]
                else:
                    ffn = lambda y, p=p, d=d: mo.mlp_forward(p["ffn"], y, d)
                h = mo.block_forward(p, h, prev, fr, mask, kv[i], pe[i], H, ffn, d)
                out["step%d_layer%d" % (step, i)] = h
                files.update(_oracle_dump_files(d, prev, i))
            hn = mo.rms_norm(h, w["norm"])[0][:, -1]                  # model.py:1572
            logits = orc.gemm(hn[None], w["head"], 1, 256, 29, orc.R_LEGACY)[0]     # model.py:1517-1519
            out["step%d_logits" % step] = logits
            prev = len(seq)
            seq.append(int(np.argmax(logits.reshape(-1))))
        out["tokens"] = np.array(seq, dtype=np.int64)
    elif kind == "mla":
        kv = np.zeros((1, a["max_seq_len"], a["kv_lora_rank"]), np.int64)
        pe = np.zeros((1, a["max_seq_len"], a["qk_rope_head_dim"]), np.int64)
        pos = 0
        for i, S in enumerate(c["steps"]):
            d = {}
            out["step%d_out" % i] = mo.mla_forward(w, x["x%d" % i], pos, freqs[pos:pos + S], mo.causal_mask(S),
                                                   kv, pe, H, d)
            files.update(_oracle_dump_files(d, pos, 0))
            pos += S
        out["kv_cache"], out["pe_cache"] = kv[:, :pos].copy(), pe[:, :pos].copy()
    elif kind == "gate":
        d = {}
        original, biased = mo.gate_scores(w, x["x"], d)
        idx, _ = mo.gate_select(biased, *g, True)
        wts, raw = mo.gate_weights(original, idx)
        d.update(gate_indices=idx, gate_weights=raw)
        out["weights"], out["indices"] = wts, idx
        files.update(_oracle_dump_files(d, 0, 1))
    elif kind == "moe":
        d = {}
        out["out"] = mo.moe_forward(w, x["x"], *g, dumps=d)[0]
        files.update(_oracle_dump_files(d, 0, 1))
    return out, files


# ------------------------------------------------------------------------------------------
# fixture records: digest + shape, and the data itself when small
KEEP_BYTES = 16384
RMS_ENTRIES = 500       # kernel.py:525: the dumped rms buffer; only the first S entries are defined


def rms_rows(path, dumps):
    """number of meaningful entries of a *_rms.bin dump = rows of the tensor the norm ran on"""
    stem = path[:-len("_rms.bin")]
    return len(dumps[stem + "_x.bin"]) // len(dumps[stem + "_weight.bin"]) * 4 // 8


def normalise_dumps(dumps):
    """cut every *_rms.bin to its defined prefix (the reference writes its whole 500-entry global
    buffer, stale beyond the rows of the call: model.py:793,1458)"""
    out = {}
    for path, data in dumps.items():
        if path.endswith("_rms.bin"):
            data = data[:8 * rms_rows(path, dumps)]
        out[path] = data
    return out


def digest(data):
    return hashlib.sha256(data).hexdigest()
