"""Model-level parity on the GPU: the integer DeepSeek-V3 modules (Linear_int ... Block) built on
the sm_100a kernels against the numpy restatement of the reference's model graph, bit-exact,
including the zkdata dumps."""
import importlib
import os

import numpy as np
import pytest
import torch

from conftest import PKG

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def M(kmod):
    m = importlib.import_module(PKG + ".model")
    kmod.softmax_init_q19()
    kmod.silu_init_q23()
    return m


@pytest.fixture(scope="module")
def mo():
    from oracle import model_oracle
    return model_oracle


def small_args(M, **kw):
    a = M.ModelArgs(max_seq_len=64, vocab_size=512, dim=256, inter_dim=384, moe_inter_dim=64, n_layers=2,
                    n_dense_layers=1, n_heads=4, n_routed_experts=16, n_shared_experts=1,
                    n_activated_experts=4, n_expert_groups=4, n_limited_groups=2, score_func="sigmoid",
                    route_scale=2.5, q_lora_rank=96, kv_lora_rank=64, qk_nope_head_dim=32,
                    qk_rope_head_dim=16, v_head_dim=32)
    for k, v in kw.items():
        setattr(a, k, v)
    return a


def w32(rng, out_f, in_f, bits=30):
    w = np.rint(rng.standard_normal((out_f, in_f)) * 2.0**bits / np.sqrt(in_f))
    return np.clip(w, -2**31, 2**31 - 1).astype(np.int32)


def norm_w(rng, n, bits=19):
    return (2**bits + np.rint(rng.standard_normal(n) * 2.0**(bits - 3))).astype(np.int32)


def mla_weights(rng, a):
    H = a.n_heads
    return {"wq_a": w32(rng, a.q_lora_rank, a.dim), "q_norm": norm_w(rng, a.q_lora_rank),
            "wq_b1": w32(rng, H * a.qk_nope_head_dim, a.q_lora_rank),
            "wq_b2": w32(rng, H * a.qk_rope_head_dim, a.q_lora_rank),
            "wkv_a1": w32(rng, a.kv_lora_rank, a.dim, 29), "wkv_a2": w32(rng, a.qk_rope_head_dim, a.dim, 29),
            "kv_norm": norm_w(rng, a.kv_lora_rank, 23),
            "wkv_b_1": w32(rng, H * a.qk_nope_head_dim, a.kv_lora_rank, 31), "wkv_b_1_scale": 31,
            "wkv_b_2": w32(rng, H * a.v_head_dim, a.kv_lora_rank), "wkv_b_2_scale": 30,
            "wo": w32(rng, a.dim, H * a.v_head_dim), "wo_scale": 30}


def mlp_weights(rng, dim, inter, s1=31, s3=31, s2=29):
    return {"w1": w32(rng, inter, dim, s1), "w1_scale": s1, "w3": w32(rng, inter, dim, s3), "w3_scale": s3,
            "w2": w32(rng, dim, inter, s2), "w2_scale": s2}


def t(a, dev):
    return torch.from_numpy(np.ascontiguousarray(a)).to(dev)


def load_linear(mod, w, scale, dev):
    mod.weight = t(w, dev)
    if scale is not None:
        mod.scale = torch.tensor(scale, dtype=torch.int32, device=dev)


def load_mla(attn, p, dev):
    for n in ("wq_a", "wq_b1", "wq_b2", "wkv_a1", "wkv_a2"):
        load_linear(getattr(attn, n), p[n], None, dev)
    for n in ("wkv_b_1", "wkv_b_2", "wo"):
        load_linear(getattr(attn, n), p[n], p[n + "_scale"], dev)
    attn.q_norm.weight = t(p["q_norm"], dev)
    attn.kv_norm.weight = t(p["kv_norm"], dev)


def load_mlp(mlp, p, dev):
    for n in ("w1", "w2", "w3"):
        load_linear(getattr(mlp, n), p[n], p[n + "_scale"], dev)


def same(got, want, what):
    got = got.cpu().numpy()
    assert got.shape == want.shape, (what, got.shape, want.shape)
    bad = int((got != want).sum())
    assert bad == 0, "%s: %d of %d words differ" % (what, bad, want.size)


def freqs_table(M, a):
    return M.precompute_freqs_cis(a)


def read_dump(path, dtype):
    return np.fromfile(path, dtype=dtype)


@pytest.mark.parametrize("act_limbs", [4, 0])
def test_mla_prefill_then_decode_with_dumps(M, mo, kmod, dev, tmp_path, act_limbs):
    a = small_args(M)
    rng = np.random.default_rng(1)
    p = mla_weights(rng, a)
    attn = M.MLA(0, a).to(dev)
    load_mla(attn, p, dev)
    freqs = freqs_table(M, a)
    kv_cache = np.zeros((1, a.max_seq_len, a.kv_lora_rank), np.int64)
    pe_cache = np.zeros((1, a.max_seq_len, a.qk_rope_head_dim), np.int64)
    M.ACT_LIMBS, M.snark, M.zkDataDir = act_limbs, True, str(tmp_path)
    attn.score_limbs = (5, 5) if act_limbs else (0, 0)
    try:
        pos = 0
        for S in (24, 1, 3):
            x = np.rint(rng.standard_normal((1, S, a.dim)) * 2.0**21).astype(np.int64)
            fr = freqs[pos:pos + S]
            mask_np = mo.causal_mask(S) if pos == 0 else None
            mask = t(mask_np, dev) if mask_np is not None else None
            dumps = {}
            want = mo.mla_forward(p, x, pos, fr.numpy(), mask_np, kv_cache, pe_cache, a.n_heads, dumps)
            got = attn(t(x, dev), pos, fr.to(dev), mask)
            same(got, want, "MLA output at pos %d" % pos)
            d = os.path.join(str(tmp_path), "pos_%d" % pos, "layer_0")
            for name, arr in dumps.items():
                if name == "freqs_cis":
                    path = os.path.join(str(tmp_path), "freqs_cis.bin")
                else:
                    path = os.path.join(d, name + ".bin")
                arr = np.ascontiguousarray(arr)
                file = read_dump(path, arr.dtype)
                if name.endswith("_rms"):          # the reference dumps its whole 500-entry buffer
                    assert file.size >= 500
                    file = file[:arr.size]
                assert np.array_equal(file, arr.ravel()), name
            pos += S
        kmod.device_status()
    finally:
        M.ACT_LIMBS, M.snark, M.zkDataDir = 4, False, "../zkdata"


def test_mla_prefill_with_masked_half_skipped(M, mo, kmod, dev):
    """causal_skip leaves the masked scores / probabilities uncomputed; the layer output is unchanged"""
    a = small_args(M, kv_lora_rank=128, n_heads=8)
    rng = np.random.default_rng(11)
    p = mla_weights(rng, a)
    attn = M.MLA(0, a).to(dev)
    load_mla(attn, p, dev)
    attn.score_limbs = (5, 4)
    attn.causal_skip = True
    freqs = freqs_table(M, a)
    S = 40
    x = np.rint(rng.standard_normal((1, S, a.dim)) * 2.0**21).astype(np.int64)
    kv_cache = np.zeros((1, a.max_seq_len, a.kv_lora_rank), np.int64)
    pe_cache = np.zeros((1, a.max_seq_len, a.qk_rope_head_dim), np.int64)
    mask_np = mo.causal_mask(S)
    want = mo.mla_forward(p, x, 0, freqs[:S].numpy(), mask_np, kv_cache, pe_cache, a.n_heads)
    got = attn(t(x, dev), 0, freqs[:S].to(dev), t(mask_np, dev))
    same(got, want, "MLA output with the masked half skipped")
    kmod.device_status()


def test_mla_decode_reads_resident_cache_planes(M, mo, kmod, dev):
    """Decode steps read the latent cache from resident limb planes (one new position split per step, score
    rows padded to four columns, the padding never read).  Against the oracle: a prefill, then single-token steps
    through every residue of the position modulo 4, a two-token step (leaves the planes, marks its positions
    stale), more single-token steps (the stale positions are split again), a second prefill from position 0 and
    another decode step; and with batch 3, where every sequence has its own cache row."""
    a = small_args(M, kv_lora_rank=128, n_heads=8)
    rng = np.random.default_rng(21)
    p = mla_weights(rng, a)
    freqs = freqs_table(M, a)
    taken = []
    plain = kmod.CachePlanes.softmax_pv

    def counted(self, *args, **kw):
        out = plain(self, *args, **kw)
        taken.append(out is not None)
        return out
    kmod.CachePlanes.softmax_pv = counted
    try:
        _resident_cache_steps(M, mo, kmod, dev, a, rng, p, freqs)
    finally:
        kmod.CachePlanes.softmax_pv = plain
    assert len(taken) == 16 and all(taken), "the resident planes did not serve every decode step"
    kmod.device_status()


def _resident_cache_steps(M, mo, kmod, dev, a, rng, p, freqs):
    for batch in (1, 3):
        attn = M.MLA(0, a, batch).to(dev)
        load_mla(attn, p, dev)
        attn.score_limbs = (5, 4)
        assert attn.resident_cache
        kv_cache = [np.zeros((1, a.max_seq_len, a.kv_lora_rank), np.int64) for _ in range(batch)]
        pe_cache = [np.zeros((1, a.max_seq_len, a.qk_rope_head_dim), np.int64) for _ in range(batch)]
        pos, used_planes = 0, 0
        for S in (13, 1, 1, 1, 1, 1, 2, 1, 1, -9, 1):
            if S < 0:                       # a new prompt: prefill from position 0 again
                pos, S = 0, -S
            x = np.rint(rng.standard_normal((batch, S, a.dim)) * 2.0**21).astype(np.int64)
            fr = freqs[pos:pos + S]
            mask_np = mo.causal_mask(S) if pos == 0 else None
            mask = t(mask_np, dev) if mask_np is not None else None
            want = np.concatenate([mo.mla_forward(p, x[b:b + 1], pos, fr.numpy(), mask_np, kv_cache[b], pe_cache[b],
                                                  a.n_heads) for b in range(batch)])
            before = attn._planes.filled if attn._planes is not None else -1
            got = attn(t(x, dev), pos, fr.to(dev), mask)
            same(got, want, "MLA output at pos %d, batch %d" % (pos, batch))
            if S == 1 and mask is None:
                assert attn._planes is not None and attn._planes.filled == pos + 1
                used_planes += 1
            elif attn._planes is not None:
                assert attn._planes.filled <= min(before, pos)
            pos += S
        assert used_planes == 8
        # the same steps with the planes switched off give the same words (and the caches agree)
        attn.resident_cache = False
        x = np.rint(rng.standard_normal((batch, 1, a.dim)) * 2.0**21).astype(np.int64)
        want = np.concatenate([mo.mla_forward(p, x[b:b + 1], pos, freqs[pos:pos + 1].numpy(), None, kv_cache[b],
                                              pe_cache[b], a.n_heads) for b in range(batch)])
        same(attn(t(x, dev), pos, freqs[pos:pos + 1].to(dev), None), want, "planes off")


def test_mlp_expert_shapes_and_shifts(M, mo, kmod, dev):
    rng = np.random.default_rng(2)
    for (dim, inter, s1, s3) in ((256, 384, 31, 31), (256, 200, 31, 33)):   # equal shifts: stacked GEMM
        p = mlp_weights(rng, dim, inter, s1, s3)
        x = np.rint(rng.standard_normal((1, 37, dim)) * 2.0**23).astype(np.int64)
        want = mo.mlp_forward(p, x)
        mlp = M.MLP_int(0, dim, inter).to(dev)
        load_mlp(mlp, p, dev)
        same(mlp(0, t(x, dev)), want, "MLP_int")
        ex = M.Expert_int(0, 3, dim, inter).to(dev)
        load_mlp(ex, p, dev)
        same(ex(0, t(x, dev)), want, "Expert_int")
    kmod.device_status()


def moe_weights(rng, a, with_bias):
    g = {"weight": w32(rng, a.n_routed_experts, a.dim, 30), "scale": 30}
    g["bias"] = (np.rint(rng.standard_normal(a.n_routed_experts) * 2.0**18) + 2**20).astype(np.int32) \
        if with_bias else None
    return {"gate": g, "shared": mlp_weights(rng, a.dim, a.n_shared_experts * a.moe_inter_dim),
            "experts": [mlp_weights(rng, a.dim, a.moe_inter_dim, 31 + (i % 2), 31, 29 + (i % 3))
                        for i in range(a.n_routed_experts)]}


def build_moe(M, a, p, dev):
    moe = M.MoE(1, a).to(dev)
    load_linear(moe.gate, p["gate"]["weight"], p["gate"]["scale"], dev)
    if p["gate"]["bias"] is not None:
        moe.gate.bias = t(p["gate"]["bias"], dev)
    load_mlp(moe.shared_experts, p["shared"], dev)
    experts = []
    for i, e in enumerate(p["experts"]):
        ex = M.Expert_int(1, i, a.dim, a.moe_inter_dim).to(dev)
        load_mlp(ex, e, dev)
        experts.append(ex)
    moe.set_experts(experts)
    return moe


def check_selection(biased_masked, indices):
    """the GPU's expert choice is a valid top-k of the (group-masked) scores: equal sorted values"""
    want = -np.sort(-biased_masked, -1)[:, :indices.shape[1]]
    got = -np.sort(-np.take_along_axis(biased_masked, indices, 1), -1)
    assert np.array_equal(want, got)


def test_moe_layer_small(M, mo, kmod, dev):
    a = small_args(M)
    rng = np.random.default_rng(3)
    p = moe_weights(rng, a, with_bias=False)
    moe = build_moe(M, a, p, dev)
    for T in (1, 50, 300):
        x = np.rint(rng.standard_normal((1, T, a.dim)) * 2.0**23).astype(np.int64)
        xg = t(x, dev)
        w_gpu, idx_gpu = moe.gate(0, xg.view(-1, a.dim))
        idx = idx_gpu.cpu().numpy()
        original, biased = mo.gate_scores(p["gate"], x[0])
        _, masked = mo.gate_select(biased, a.n_expert_groups, a.n_limited_groups, a.n_activated_experts, False)
        check_selection(masked, idx)
        want, w_want, _ = mo.moe_forward(p, x, a.n_expert_groups, a.n_limited_groups, a.n_activated_experts,
                                         indices=idx)
        same(w_gpu, w_want, "gate weights")
        same(moe(0, xg), want, "MoE output, T=%d" % T)
    kmod.device_status()


def test_optimistic_group_rows_are_checked_on_the_device(M, mo, kmod, dev):
    """72 tokens, 16 experts, top-4: 18 rows per expert on average, so the grouped GEMMs are launched with the
    optimistic 64-row bound (a bound is only certain up to 64 tokens).  Here every token names expert 0: 72 rows
    in one group break the promise, the device flag says so
    (ERR_RANGE) instead of dropping rows silently, and the same call without the promise gives the oracle's
    words."""
    a = small_args(M)
    rng = np.random.default_rng(41)
    p = moe_weights(rng, a, with_bias=False)
    moe = build_moe(M, a, p, dev)
    T = 72
    x = np.rint(rng.standard_normal((1, T, a.dim)) * 2.0**23).astype(np.int64)
    idx = np.stack([np.array([0] + list(rng.choice(np.arange(1, 16), 3, replace=False))) for _ in range(T)])
    original, _ = mo.gate_scores(p["gate"], x[0])
    w, _ = mo.gate_weights(original, idx)
    xg, ig, wg = t(x[0], dev), t(idx.astype(np.int64), dev), t(w, dev)
    assert M.OPTIMISTIC_GROUP_ROWS
    torch.cuda.synchronize()
    kmod.device_status()
    moe.experts_forward(0, xg, wg, ig)
    torch.cuda.synchronize()
    with pytest.raises(kmod.ZkdsError) as err:
        kmod.device_status()
    assert err.value.status == kmod.ERR_RANGE
    M.OPTIMISTIC_GROUP_ROWS = False
    try:
        got = moe.experts_forward(0, xg, wg, ig)
    finally:
        M.OPTIMISTIC_GROUP_ROWS = True
    want = np.zeros((T, a.dim), np.int64)
    for e in range(16):
        rows, slot = np.where(idx == e)
        if len(rows):
            want[rows] += (mo.mlp_forward(p["experts"][e], x[:, rows])[0] * w[rows, slot][:, None]) >> 23
    same(got, want, "routed experts, promise off")
    kmod.device_status()


def test_expert_parallel_over_peer_memory_one_rank(M, mo, kmod, dev):
    """The peer-memory expert-parallel path (rows read in place by the owner's limb split, weighted sums written
    into the home GPU's slots, flag barriers) with a process group of one rank: this GPU is its own peer, so the
    symmetric buffers, the multi-buffer gather, the slot write, the slot sum and the barrier kernel all run.  The
    result is the MoE layer's and the oracle's.  More ranks: bench.py --workload moe --gpus N checks rows of the
    actual pass against the oracle."""
    import importlib
    import os
    import socket
    import torch.distributed as dist
    par = importlib.import_module(M.__name__.rsplit(".", 1)[0] + ".parallel")
    a = small_args(M)
    rng = np.random.default_rng(31)
    p = moe_weights(rng, a, with_bias=False)
    moe = build_moe(M, a, p, dev)
    started = False
    if not dist.is_initialized():
        with socket.socket() as so:
            so.bind(("127.0.0.1", 0))
            port = so.getsockname()[1]
        os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
        dist.init_process_group("nccl", rank=0, world_size=1, device_id=torch.device(dev))
        started = True
    try:
        for T in (300, 40, 300):          # the second call has fewer tokens than the buffers hold
            x = np.rint(rng.standard_normal((1, T, a.dim)) * 2.0**23).astype(np.int64)
            xg = t(x, dev).view(-1, a.dim)
            w_gpu, idx_gpu = moe.gate(0, xg)
            y, _ = par.expert_parallel_forward_peer(
                moe, kmod, 0, xg.contiguous(), w_gpu, idx_gpu,
                before_sync=lambda: moe.shared_experts(0, xg[None]).view(-1, a.dim).contiguous())
            want, _, _ = mo.moe_forward(p, x, a.n_expert_groups, a.n_limited_groups, a.n_activated_experts,
                                        indices=idx_gpu.cpu().numpy())
            same(y[None], want, "peer path, T=%d" % T)
            same(moe(0, xg[None]), want, "single-GPU path, T=%d" % T)
        par.peer_exchange(None, 1, a.dim, xg.device).raise_if_timed_out()
        kmod.device_status()
    finally:
        if started:
            par._exchanges.clear()
            dist.destroy_process_group()


def test_gate_with_bias_dim_7168(M, mo, kmod, dev):
    """the gate bias exists only for dim == 7168 (model.py:1093): grouped top-2-sum selection"""
    a = small_args(M, dim=7168, n_routed_experts=256, n_expert_groups=8, n_limited_groups=4,
                   n_activated_experts=8)
    rng = np.random.default_rng(4)
    g = {"weight": w32(rng, 256, 7168, 33), "scale": 33,
         "bias": (np.rint(rng.standard_normal(256) * 2.0**19) + 2**21).astype(np.int32)}
    gate = M.Gate(3, a).to(dev)
    load_linear(gate, g["weight"], g["scale"], dev)
    gate.bias = t(g["bias"], dev)
    x = np.rint(rng.standard_normal((64, 7168)) * 2.0**23).astype(np.int64)
    w_gpu, idx_gpu = gate(0, t(x, dev))
    original, biased = mo.gate_scores(g, x)
    idx_o, masked = mo.gate_select(biased, 8, 4, 8, True)
    check_selection(masked, idx_gpu.cpu().numpy())
    w_want, _ = mo.gate_weights(original, idx_gpu.cpu().numpy())
    same(w_gpu, w_want, "gate weights")
    # without score ties the oracle's own selection is the same set of experts
    assert np.array_equal(np.sort(idx_o, -1), np.sort(idx_gpu.cpu().numpy(), -1))
    kmod.device_status()


def test_block_dense_and_moe(M, mo, kmod, dev):
    a = small_args(M)
    rng = np.random.default_rng(5)
    freqs = freqs_table(M, a)
    for layer_id in (0, 1):
        pa = mla_weights(rng, a)
        p = {"attn": pa, "attn_norm": norm_w(rng, a.dim, 21), "ffn_norm": norm_w(rng, a.dim, 23)}
        blk = M.Block(layer_id, a).to(dev)
        load_mla(blk.attn, pa, dev)
        blk.attn_norm.weight = t(p["attn_norm"], dev)
        blk.ffn_norm.weight = t(p["ffn_norm"], dev)
        S = 20
        x = np.rint(rng.standard_normal((1, S, a.dim)) * 2.0**31).astype(np.int64)
        if layer_id < a.n_dense_layers:
            pf = mlp_weights(rng, a.dim, a.inter_dim)
            load_mlp(blk.ffn, pf, dev)
            ffn = lambda h: mo.mlp_forward(pf, h)
        else:
            pf = moe_weights(rng, a, False)
            blk.ffn = build_moe(M, a, pf, dev)
            holder = {}

            def ffn(h, pf=pf, holder=holder):
                idx = blk.ffn.gate(0, t(h, dev).view(-1, a.dim))[1].cpu().numpy()
                return mo.moe_forward(pf, h, a.n_expert_groups, a.n_limited_groups, a.n_activated_experts,
                                      indices=idx)[0]
        kv = np.zeros((1, a.max_seq_len, a.kv_lora_rank), np.int64)
        pe = np.zeros((1, a.max_seq_len, a.qk_rope_head_dim), np.int64)
        mask_np = mo.causal_mask(S)
        want = mo.block_forward(p, x, 0, freqs[:S].numpy(), mask_np, kv, pe, a.n_heads, ffn)
        got = blk(t(x, dev), 0, freqs[:S].to(dev), t(mask_np, dev))
        same(got, want, "Block %d" % layer_id)
    kmod.device_status()


def test_transformer_steps(M, kmod, dev):
    """prep_inference / layer_inference / finish_inference wiring on a two-layer model"""
    a = small_args(M)
    rng = np.random.default_rng(6)
    with torch.device(dev):
        model = M.Transformer(a)
    model.embed.weight = t(np.rint(rng.standard_normal((a.vocab_size, a.dim)) * 2.0**31).astype(np.int64), dev)
    model.norm.weight = t(norm_w(rng, a.dim, 15).astype(np.int64), dev)
    model.head.weight = t(np.rint(rng.standard_normal((a.vocab_size, a.dim)) * 2.0**43 / 16).astype(np.int64), dev)
    for i in range(a.n_layers):
        blk = M.Block(i, a).to(dev)
        load_mla(blk.attn, mla_weights(rng, a), dev)
        blk.attn_norm.weight = t(norm_w(rng, a.dim, 21), dev)
        blk.ffn_norm.weight = t(norm_w(rng, a.dim, 23), dev)
        if i < a.n_dense_layers:
            load_mlp(blk.ffn, mlp_weights(rng, a.dim, a.inter_dim), dev)
        else:
            blk.ffn = build_moe(M, a, moe_weights(rng, a, False), dev)
        model.layers[i] = blk
    tokens = torch.randint(0, a.vocab_size, (1, 9), device=dev)
    h, pos, S = model.prep_inference(tokens, 0)
    for i in range(a.n_layers):
        h = model.layer_inference(i, h, pos, S)
    logits = model.finish_inference(h)
    assert logits.shape == (1, 1, a.vocab_size) and logits.dtype == torch.int64
    # the head divides its int64 weight by 2^8 before the product (model.py:1519)
    from oracle import oracle as orc
    hn, _ = orc.rms_norm(h[0].cpu().numpy(), model.norm.weight.cpu().numpy(), 1, a.dim)
    want, _ = orc.gemm(hn[None, -1:], model.head.weight.cpu().numpy(), 1, 256, 29)
    same(logits, want, "logits")
    kmod.device_status()


def _small_transformer(M, a, rng, dev, batch, gate_bias=True):
    with torch.device(dev):
        model = M.Transformer(a)
    model.embed.weight = t(np.rint(rng.standard_normal((a.vocab_size, a.dim)) * 2.0**31).astype(np.int64), dev)
    model.norm.weight = t(norm_w(rng, a.dim, 15).astype(np.int64), dev)
    model.head.weight = t(np.rint(rng.standard_normal((a.vocab_size, a.dim)) * 2.0**43 / 16).astype(np.int64), dev)
    for i in range(a.n_layers):
        blk = M.Block(i, a, cache_batch=batch).to(dev)
        load_mla(blk.attn, mla_weights(rng, a), dev)
        blk.attn_norm.weight = t(norm_w(rng, a.dim, 21), dev)
        blk.ffn_norm.weight = t(norm_w(rng, a.dim, 23), dev)
        if i < a.n_dense_layers:
            load_mlp(blk.ffn, mlp_weights(rng, a.dim, a.inter_dim), dev)
        else:
            blk.ffn = build_moe(M, a, moe_weights(rng, a, gate_bias), dev)    # dumps write the gate bias
        model.layers[i] = blk
    return model


def test_generate_loop(M, kmod, dev, tmp_path):
    """generate() (generate.py:164-286) on a two-layer model, two prompts of different length: the
    cached decode must give the very tokens a from-scratch prefill of every prefix gives (integer
    arithmetic: no tolerance), prompt tokens are never overwritten, eos ends a sequence, and with
    snark the token files appear under pos_{p}/"""
    import importlib
    G = importlib.import_module(M.__name__.rsplit(".", 1)[0] + ".generate")
    a = small_args(M)
    model = _small_transformer(M, a, np.random.default_rng(8), dev, batch=2)
    prompts = [[5, 17, 300, 2, 41], [9, 100, 7]]
    trace = []
    out = G.generate(model, prompts, 4, eos_id=-5, temperature=0.0, trace=trace)
    assert [len(o) for o in out] == [4, 4]
    assert [s["pos"] for s in trace] == list(range(3, 9))
    # the longer prompt's own tokens at positions 3 and 4 survive
    assert trace[0]["next_token"][0] == prompts[0][3]
    assert trace[1]["next_token"][0] == prompts[0][4]

    # from-scratch check: every generated token equals the argmax after a fresh prefill of its prefix
    ref = _small_transformer(M, a, np.random.default_rng(8), dev, batch=1)
    for b, prompt in enumerate(prompts):
        seq = list(prompt)
        for step in range(4):
            toks = torch.tensor([seq], dtype=torch.long, device=dev)
            h, pos, S = ref.prep_inference(toks, 0)
            for i in range(a.n_layers):
                h = ref.layer_inference(i, h, pos, S)
            nxt = int(ref.finish_inference(h).argmax(dim=-1).view(-1)[0])
            assert nxt == out[b][step], "sequence %d, new token %d" % (b, step)
            seq.append(nxt)

    # eos: the first sequence stops at its second new token
    model2 = _small_transformer(M, a, np.random.default_rng(8), dev, batch=2)
    eos = out[0][1]
    cut = G.generate(model2, prompts, 4, eos_id=eos, temperature=0.0)
    assert cut[0] == out[0][:out[0].index(eos)]
    assert cut[1] == (out[1][:out[1].index(eos)] if eos in out[1] else out[1])

    # dumps: tokens.bin of the prefill and of the first decode step
    model3 = _small_transformer(M, a, np.random.default_rng(8), dev, batch=1)
    M.snark, M.zkDataDir = True, str(tmp_path)
    try:
        probe_trace = []
        G.generate(model3, [prompts[1]], 2, eos_id=-5, temperature=0.0, layer_probe=True, trace=probe_trace)
    finally:
        M.snark, M.zkDataDir = False, "../zkdata"
    assert np.array_equal(read_dump(os.path.join(str(tmp_path), "pos_0", "tokens.bin"), np.int64), prompts[1])
    assert read_dump(os.path.join(str(tmp_path), "pos_3", "tokens.bin"), np.int64).tolist() == [out[1][0]]
    # the probe of the last layer is the token the step produces
    assert probe_trace[0]["layer_tokens"][-1] == probe_trace[0]["next_token"]
    kmod.device_status()


def test_resident_checkpoint_loader(M, kmod, dev, tmp_path):
    """a checkpoint directory in the converted layout (embed/norm/head_int, layer-{i}, experts-{l}/{i}
    safetensors) loaded with every layer resident generates the tokens of the model it was written from"""
    import importlib
    from safetensors.torch import save_file, save_model
    G = importlib.import_module(M.__name__.rsplit(".", 1)[0] + ".generate")
    a = small_args(M)
    # no gate bias: like the reference, Gate only registers (and so only saves) one at dim 7168
    model = _small_transformer(M, a, np.random.default_rng(9), dev, batch=1, gate_bias=False)
    ck = str(tmp_path)
    save_model(model.embed, os.path.join(ck, "embed_int.safetensors"))
    save_model(model.norm, os.path.join(ck, "norm_int.safetensors"))
    save_model(model.head, os.path.join(ck, "head_int.safetensors"))
    for i, blk in enumerate(model.layers):
        sd = {k: v.contiguous() for k, v in blk.state_dict().items()}
        save_file(sd, os.path.join(ck, "layer-%d.safetensors" % i))
        if isinstance(blk.ffn, M.MoE):
            os.makedirs(os.path.join(ck, "experts-%d" % i), exist_ok=True)
            moe, I = blk.ffn, a.moe_inter_dim
            for j in range(a.n_routed_experts):
                e = M.Expert_int(i, j, a.dim, I).to(dev)
                e.w1.weight, e.w3.weight = moe.experts_w13[j, :I].clone(), moe.experts_w13[j, I:].clone()
                e.w2.weight = moe.experts_w2[j].clone()
                e.w1.scale, e.w3.scale, e.w2.scale = (moe.experts_shift[j, c].clone() for c in range(3))
                save_model(e, os.path.join(ck, "experts-%d/%d.safetensors" % (i, j)))
    loaded = G.load_resident(ck, a, dev)
    prompts = [[11, 250, 3, 77]]
    want = G.generate(model, prompts, 3, eos_id=-5, temperature=0.0)
    got = G.generate(loaded, prompts, 3, eos_id=-5, temperature=0.0)
    assert got == want
    kmod.device_status()


def test_activation_beyond_the_limb_bound_is_caught(M, mo, kmod, dev):
    """ACT_LIMBS promises |x| < 2^31 for every activation entering a GEMM.  An attn_norm weight near 2^30
    breaks the promise (normed values reach 2^30 * x / rms): the direct inference calls raise instead of
    returning wrong logits, generate() re-runs the step with measured limb counts and produces the tokens of
    a model that measured from the start."""
    import importlib
    G = importlib.import_module(M.__name__.rsplit(".", 1)[0] + ".generate")
    a = small_args(M)

    def build():
        model = _small_transformer(M, a, np.random.default_rng(12), dev, batch=1, gate_bias=False)
        w = model.layers[0].attn_norm.weight
        model.layers[0].attn_norm.weight = (w.to(torch.int64) << 9).to(torch.int32)       # 2^21 -> 2^30
        return model

    model = build()
    toks = torch.tensor([[5, 17, 300, 2, 41, 7]], dtype=torch.long, device=dev)
    h, pos, S = model.prep_inference(toks, 0)
    for i in range(a.n_layers):
        h = model.layer_inference(i, h, pos, S)
    with pytest.raises(kmod.ZkdsError) as info:
        model.finish_inference(h)
    assert info.value.status == kmod.ERR_RANGE
    kmod.device_status()                                   # the flag was cleared by the raise

    trace = []
    got = G.generate(build(), [toks[0].tolist()], 3, eos_id=-5, temperature=0.0, trace=trace)
    assert trace[0].get("rerun_measured") is True
    ref = build()
    with M.measured_limbs(ref):
        want = G.generate(ref, [toks[0].tolist()], 3, eos_id=-5, temperature=0.0)
    assert got == want
    assert M.ACT_LIMBS == 4
    kmod.device_status()


@pytest.mark.parametrize("E,groups,keep,topk,with_bias", [(256, 8, 4, 8, True), (256, 8, 4, 8, False),
                                                          (16, 4, 2, 4, False), (64, 1, 1, 6, True), (32, 8, 4, 8, True)])
def test_fused_gate_selection(M, mo, kmod, dev, E, groups, keep, topk, with_bias):
    """K.gate_select against the reference's torch ops (run here on the same tensors) and the numpy oracle:
    the same weights always; the same experts, in the same order when no two scores of a row are equal; with
    deliberately tied scores still a valid top-k of the masked scores and the lower index first."""
    rng = np.random.default_rng(E + topk)
    T = 300
    bias = (2**20 + rng.integers(-2**19, 2**19, E, dtype=np.int64)).astype(np.int32) if with_bias else None
    # scores (sigma + bias) that are distinct within a row, so that torch.topk's order is defined
    distinct = np.stack([rng.permutation(E) for _ in range(T)]).astype(np.int64) * 2**14 + \
        rng.integers(0, 2**14, (T, E), dtype=np.int64) + 2**21
    sig = distinct - (bias.astype(np.int64) if with_bias else 0)
    sg, bg = t(sig, dev), (t(bias, dev) if with_bias else None)
    w, idx, raw = kmod.gate_select(sg, bg, groups, keep, topk)
    # the reference's ops (model.py:1140-1211)
    scores = sg + bg if with_bias else sg
    if groups > 1:
        s3 = scores.view(T, groups, -1)
        gsc = s3.topk(2, dim=-1)[0].sum(-1) if with_bias else s3.amax(-1)
        gi = gsc.topk(keep, dim=-1)[1]
        gm = s3.new_ones(T, groups, dtype=torch.bool).scatter_(1, gi, False)
        scores = s3.masked_fill(gm.unsqueeze(-1), -(1 << 42)).flatten(1)
    ti = torch.topk(scores, topk, dim=-1)[1]
    tw = sg.gather(1, ti)
    same(raw, tw.cpu().numpy(), "raw weights")
    same(idx, ti.cpu().numpy(), "indices")
    same(w, ((tw * (2 ** 23)) // tw.sum(-1, keepdim=True) * 5 // 2).cpu().numpy(), "weights")
    # oracle
    original, biased = sig, (sig + bias.astype(np.int64) if with_bias else sig)
    oi, masked = mo.gate_select(biased, groups, keep, topk, with_bias)
    same(idx, oi, "indices vs oracle")
    same(w, mo.gate_weights(original, oi)[0], "weights vs oracle")
    # ties: quantise the scores so that many are equal
    sig2 = (sig >> 19) << 19
    w2, idx2, raw2 = kmod.gate_select(t(sig2, dev), None, groups, keep, topk)
    oi2, masked2 = mo.gate_select(sig2, groups, keep, topk, False)
    same(idx2, oi2, "tied scores: the lower index first, as the oracle's stable sort")
    check_selection(masked2, idx2.cpu().numpy())
    kmod.device_status()
