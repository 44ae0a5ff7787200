"""numpy restatement of the reference's integer model graph (inference/model.py) on top of
the CPU oracle's kernels.  TEST INFRASTRUCTURE ONLY — the checker for the model-level
parity tests; nothing on the product path imports it.

Weights are plain dicts of numpy arrays.  The torch glue of the reference is restated with
numpy's wrapping int64 arithmetic and floor division (`//`), which match torch's on int64.
Every function cites the reference lines it follows.
"""
import numpy as np

from . import oracle as orc

MASK_VALUE = -(64 << 36)        # model.py:1555


def linear(x, W, shift, x_r=1, w_r=1, legacy=True):
    """linear_int (model.py:193-207): x [B, M, K] -> (q, r)"""
    return orc.gemm(x, W, x_r, w_r, shift, orc.R_LEGACY if legacy else orc.R_MATH)


def rms_norm(x, w):
    """RMSNorm_int.forward (model.py:486-493): x [1, M, dim] -> (y [1, M, dim], rms [M])"""
    c, rms = orc.rms_norm(x[0], w, 1, x.shape[-1])
    return c[None], rms


def rotary(x, freqs):
    """apply_rotary_emb (model.py:611-637): x [B, S, H, 2P], freqs [S, P, 2]"""
    B, S, H, D = x.shape
    return orc.rope(np.ascontiguousarray(x).reshape(B, S, H, D // 2, 2), freqs, 42).reshape(B, S, H, D)


def causal_mask(seqlen):
    """Transformer.layer_inference (model.py:1553-1555)"""
    return np.triu(np.full((seqlen, seqlen), MASK_VALUE, np.int64), 1) if seqlen > 1 else None


def mla_forward(p, x, start_pos, freqs, mask, kv_cache, pe_cache, n_heads, dumps=None, s_q=30, s_kv=29):
    """MLA.forward, absorbed path (model.py:747-957).  p: wq_a, q_norm, wq_b1, wq_b2, wkv_a1,
    wkv_a2, kv_norm, wkv_b_1, wkv_b_2, wo (int32 arrays) and the shifts wkv_b_1_scale,
    wkv_b_2_scale, wo_scale.  kv_cache / pe_cache [1, max_seq, .] are updated in place.
    s_q / s_kv: the shifts of wq_a, wq_b and of wkv_a (30 and 29 in the reference, model.py:702-712)."""
    B, S, _ = x.shape
    end = start_pos + S
    H = n_heads
    d = dumps if dumps is not None else {}
    q_down, q_rem = linear(x, p["wq_a"], s_q)
    d.update(wq_a_x=x, wq_a_w=p["wq_a"].view(np.uint32), wq_a_y=q_down, q_norm_r=q_rem)
    q_normed, rms = rms_norm(q_down, p["q_norm"])
    d.update(q_norm_x=q_down, q_norm_weight=p["q_norm"].view(np.uint32), q_norm_rms=rms, q_norm_y=q_normed)
    q_nope = linear(q_normed, p["wq_b1"], s_q)[0].reshape(B, S, H, -1)
    q_pe = linear(q_normed, p["wq_b2"], s_q)[0].reshape(B, S, H, -1)
    d.update(q_pe_x=q_pe, freqs_cis=freqs)
    q_pe = rotary(q_pe, freqs)
    d.update(q_pe_y=p["q_norm"].view(np.uint32))            # model.py:819 writes the norm weight
    kv, kv_rem = linear(x, p["wkv_a1"], s_kv)
    d.update(wkv_a1_x=x, wkv_a1_w=p["wkv_a1"].view(np.uint32), wkv_a1_y=kv, wkv_a1_r=kv_rem)
    k_pe = linear(x, p["wkv_a2"], s_kv)[0]
    k_pe = rotary(k_pe[:, :, None, :], freqs)
    C = p["wkv_b_1"].shape[1]
    w1 = p["wkv_b_1"].reshape(H, -1, C)
    q_abs = orc.einsum_bshd_hdc_bshc(q_nope, w1, p["wkv_b_1_scale"])
    kv_normed, _ = rms_norm(kv, p["kv_norm"])
    kv_cache[:B, start_pos:end] = kv_normed
    pe_cache[:B, start_pos:end] = k_pe[:, :, 0]
    kv_all = np.ascontiguousarray(kv_cache[:B, :end])
    pe_all = np.ascontiguousarray(pe_cache[:B, :end])
    score1 = orc.einsum_bshc_btc_bsht(q_abs, kv_all, 23)
    score2 = orc.einsum_bshc_btc_bsht(q_pe, pe_all, 21)
    scores = (score1 + score2) * 94 // 695                   # model.py:897
    if mask is not None:
        scores = scores + mask[:, None, :]                   # model.py:905
    d.update(scores_softmax_x=scores)
    probs = orc.softmax(scores, 19)
    d.update(scores_softmax_y=probs)
    ctx = orc.einsum_bsht_btc_bshc(probs, kv_all, 23)
    w2 = p["wkv_b_2"].reshape(H, -1, C)
    out = orc.einsum_bshc_hdc_bshd(ctx, w2, p["wkv_b_2_scale"])
    return linear(out.reshape(B, S, -1), p["wo"], p["wo_scale"])[0]


def mlp_forward(p, x, dumps=None, prefix="mlp"):
    """MLP_int.forward (model.py:1018-1049) / Expert_int.forward (model.py:1247-1281)"""
    r1 = linear(x, p["w1"], p["w1_scale"])[0]
    s1 = orc.act(r1, "silu", 23)
    if dumps is not None:
        dumps[prefix + "_silu_x"] = r1
        dumps[prefix + "_silu_y"] = s1
    r2 = linear(x, p["w3"], p["w3_scale"])[0]
    return linear((s1 * r2) >> 23, p["w2"], p["w2_scale"])[0]


def gate_scores(p, x, dumps=None):
    """Gate.forward up to the biased scores (model.py:1099-1147): x [T, dim]"""
    scores, rem = linear(x[None], p["weight"], p["scale"])
    sig = orc.act(scores, "sigmoid", 23)
    if dumps is not None:
        dumps.update(sigmoid_gate_x=scores, sigmoid_gate_r=rem, sigmoid_gate_y=sig,
                     gate_original_scores=sig[0])
        if p.get("bias") is not None:
            dumps["gate_bias"] = p["bias"].view(np.uint32)
    original = sig[0]
    biased = original + p["bias"].astype(np.int64) if p.get("bias") is not None else original
    return original, biased


def gate_select(biased, n_groups, topk_groups, topk, has_bias=True):
    """grouped top-k (model.py:1154-1188).  Ties are broken towards the lower index; the
    reference leaves them to torch.topk."""
    T = biased.shape[0]
    scores = biased
    if n_groups > 1:
        g = scores.reshape(T, n_groups, -1)
        if has_bias:
            group_scores = np.sort(g, -1)[:, :, -2:].sum(-1)
        else:
            group_scores = g.max(-1)
        keep = np.argsort(-group_scores, -1, kind="stable")[:, :topk_groups]
        gmask = np.ones((T, n_groups), bool)
        np.put_along_axis(gmask, keep, False, 1)
        scores = np.where(gmask[:, :, None], -(1 << 42), g).reshape(T, -1)
    return np.argsort(-scores, -1, kind="stable")[:, :topk], scores


def gate_weights(original, indices):
    """model.py:1190-1211: gather, normalise to 2^23, scale by 5 // 2"""
    w = np.take_along_axis(original, indices, 1)
    raw = w
    w = (w * (2 ** 23)) // w.sum(-1, keepdims=True)
    return w * 5 // 2, raw


def moe_forward(p, x, n_groups, topk_groups, topk, indices=None, dumps=None):
    """MoE.forward (model.py:1325-1383).  p: gate{weight,scale,bias}, shared{w1,w2,w3,+scales},
    experts: list of {w1,w2,w3,+scales}.  `indices` overrides the expert selection (to follow a
    GPU run through a score tie)."""
    shape = x.shape
    z = mlp_forward(p["shared"], x, dumps)
    x2 = x.reshape(-1, shape[-1])
    original, biased = gate_scores(p["gate"], x2, dumps)
    if indices is None:
        indices, _ = gate_select(biased, n_groups, topk_groups, topk, p["gate"].get("bias") is not None)
    weights, raw = gate_weights(original, indices)
    if dumps is not None:
        dumps.update(gate_indices=indices, gate_weights=raw)
    y = np.zeros_like(x2)
    for i, e in enumerate(p["experts"]):
        idx, top = np.where(indices == i)
        if idx.size == 0:
            continue
        y2 = mlp_forward(e, x2[idx][None], dumps, "expert_%d" % i)[0]
        y[idx] += y2 * weights[idx, top, None] // (1 << 23)
    return (y + z.reshape(-1, shape[-1])).reshape(shape), weights, indices


def block_forward(p, x, start_pos, freqs, mask, kv_cache, pe_cache, n_heads, ffn, dumps=None):
    """Block.forward (model.py:1430-1475); ffn(x) is the MLP or MoE closure"""
    normed, rms = rms_norm(x, p["attn_norm"])
    if dumps is not None:
        dumps.update(attn_norm_x=x, attn_norm_weight=p["attn_norm"].view(np.uint32), attn_norm_y=normed,
                     attn_norm_rms=rms)
    attned = mla_forward(p["attn"], normed, start_pos, freqs, mask, kv_cache, pe_cache, n_heads, dumps)
    x = x + attned * (2 ** 12)
    ffn_normed, _ = rms_norm(x, p["ffn_norm"])
    return x + ffn(ffn_normed) * (2 ** 8)
