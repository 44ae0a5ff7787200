"""Integer DeepSeek-V3 modules on the B200 kernels: the call surface of the reference's
``inference/model.py`` for its int64 forward pass.

Class and function names, constructor arguments, buffer names (``weight``, ``scale``,
``bias``) and ``forward`` signatures follow the reference so that ``inference/generate.py``
and converted checkpoints work unchanged:

    linear_int                    model.py:193-207     Linear_int / Linear_rescale_int   :209-274
    Column/RowParallelLinear_*    model.py:357-448     RMSNorm_int                       :477-493
    precompute_freqs_cis          model.py:496-608     apply_rotary_emb                  :611-637
    MLA                           model.py:652-957     MLP_int                           :994-1049
    Gate                          model.py:1052-1212   Expert_int                        :1214-1281
    MoE                           model.py:1283-1383   Block                             :1401-1475
    Transformer                   model.py:1477-1583   ParallelEmbedding                 :104-150

What differs is how the work is done, never the integers produced:
  * static weights are split into signed 8-bit limb planes once and the GEMMs run on the
    tensor-core limb kernel; activation limb counts are upper bounds checked on the device;
  * `(score1 + score2) * 94 // 695 + mask` is the epilogue of the second score contraction;
  * w1 and w3 of an MLP are one stacked GEMM followed by one fused SiLU-multiply-shift kernel;
  * routed experts stay resident and run as one grouped GEMM over token rows sorted by
    expert (the reference loads every expert from disk inside the loop, model.py:1359-1363);
  * per-layer ``scale`` buffers are read once (``.item()`` synchronises) and cached;
  * with ``world_size > 1`` heads / experts / output columns are split so that every output
    column sees its full K: the reference's row-parallel all_reduce of already-shifted partial
    sums (model.py:441-445) is not bit-exact against one GPU and is not reproduced.

``snark`` gates the zkdata dumps exactly as in the reference (file names, dtypes, raw
little-endian C order), including ``q_pe_y.bin`` holding ``q_norm.weight`` (model.py:819).
"""
import math
import os
from dataclasses import dataclass
from typing import Literal, Optional, Tuple

import torch
import torch.distributed as dist
import torch.nn.functional as F
from torch import nn

try:  # drop-in use: this directory first on sys.path, as `from kernel import ...`
    from . import kernel as K
except ImportError:  # pragma: no cover
    import kernel as K

world_size = 1
rank = 0
block_size = 128
gemm_impl: Literal["bf16", "fp8"] = "bf16"
attn_impl: Literal["naive", "absorb"] = "absorb"

snark = False
zkDataDir = "../zkdata"

# Upper bound (signed 8-bit limbs) promised for activations entering a GEMM; the limb count
# actually used is derived on the device, data beyond the bound raises K.device_status().
# 0 measures every activation on the device with a host synchronisation.
ACT_LIMBS = 4
# A result computed from an activation beyond the promised bound is wrong, and only a device flag says
# so.  With CHECK_STATUS the flag is read wherever a result leaves the model: at the end of
# Transformer.finish_inference (one stream synchronisation per step, where the caller reads the logits
# anyway) and after every Block whose dumps are written.  generate() re-runs a flagged step with measured
# limb counts instead of raising.
CHECK_STATUS = True
# Gate: bias, grouped top-k selection and weights in one kernel (K.gate_select) instead of the reference's
# torch ops.  Same experts and weights; under score ties the kernel takes the lower index, which is the set
# torch.topk takes, while the ORDER torch gives equal scores is unspecified (False keeps the torch ops).
FUSED_GATE = True
# Routed experts with few rows each (decode): up to 64 tokens no expert can have more rows than tokens, and the
# grouped GEMMs fetch only 32 / 64 rows per tile.  With OPTIMISTIC_GROUP_ROWS the smaller box is also promised
# where it is merely expected (mean rows per expert <= 8: box 32, <= 20: box 64); a group that breaks the promise
# raises the device flag (ZkdsError with ERR_RANGE where results leave the model) and generate() repeats the step
# under measured_limbs, which switches the optimistic promise off.
OPTIMISTIC_GROUP_ROWS = True
# token-parallel MoE on GPUs of one node: rows and results move over peer memory inside the expert kernels
# (parallel.expert_parallel_forward_peer); False = NCCL all-to-all of packed rows
PEER_EXPERTS = True


@dataclass
class ModelArgs:
    """Model hyper-parameters; same fields and defaults as the reference (model.py:27-92)."""
    max_batch_size: int = 8
    max_seq_len: int = 4096 * 4
    dtype: Literal["bf16", "fp8"] = "bf16"
    vocab_size: int = 102400
    dim: int = 2048
    inter_dim: int = 10944
    moe_inter_dim: int = 1408
    n_layers: int = 27
    n_dense_layers: int = 1
    n_heads: int = 16
    n_routed_experts: int = 64
    n_shared_experts: int = 2
    n_activated_experts: int = 6
    n_expert_groups: int = 1
    n_limited_groups: int = 1
    score_func: Literal["softmax", "sigmoid"] = "softmax"
    route_scale: float = 1.
    q_lora_rank: int = 0
    kv_lora_rank: int = 512
    qk_nope_head_dim: int = 128
    qk_rope_head_dim: int = 64
    v_head_dim: int = 128
    original_seq_len: int = 4096
    rope_theta: float = 10000.0
    rope_factor: float = 40
    beta_fast: int = 32
    beta_slow: int = 1
    mscale: float = 1.


def _ver(t):
    """version counter of a weight tensor for the cache keys of its limb planes.  Tensors created under
    torch.inference_mode() have none: they cannot be modified in place outside it either, so 0 is enough."""
    return 0 if t.is_inference() else t._version


def saveTensor(fileName, t):
    K.saveTensor(fileName, t)


def _dump_dir(start_pos, layer_id):
    d = f"{zkDataDir}/pos_{start_pos}/layer_{layer_id}"
    os.makedirs(d, exist_ok=True)
    return d


class ParallelEmbedding(nn.Module):
    """int64 embedding table split over ranks by vocabulary rows (model.py:104-150)."""

    def __init__(self, vocab_size: int, dim: int):
        super().__init__()
        self.vocab_size, self.dim = vocab_size, dim
        assert vocab_size % world_size == 0
        self.part_vocab_size = vocab_size // world_size
        self.vocab_start_idx = rank * self.part_vocab_size
        self.vocab_end_idx = self.vocab_start_idx + self.part_vocab_size
        self.register_buffer("weight", torch.empty(self.part_vocab_size, dim, dtype=torch.int64))

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        if world_size > 1:
            mask = (x < self.vocab_start_idx) | (x >= self.vocab_end_idx)
            x = x - self.vocab_start_idx
            x[mask] = 0
        y = F.embedding(x, self.weight)
        if world_size > 1:
            y[mask] = 0
            dist.all_reduce(y)
        return y


def linear_int(x, weight, x_rescale, weight_rescale, res_rescale, bias=None):
    """(q, r) = int64_bmm_broadcast(x, weight, ...) (model.py:193-207); ranges measured."""
    if weight.element_size() <= 1:
        raise NotImplementedError("fp8 weights belong to the float path, not to the integer model")
    return K.int64_bmm_broadcast(x, weight, x_rescale, weight_rescale, res_rescale)


class Linear_int(nn.Module):
    """Linear layer on an int32 / int64 weight [out, in]; forward returns (quotient, remainder)."""
    dtype = torch.int64

    def __init__(self, layer_id, in_features, out_features, x_rescale, weight_rescale, res_rescale, dtype,
                 bias: bool = False):
        super().__init__()
        self.layer_id = layer_id
        self.in_features, self.out_features = in_features, out_features
        self.x_rescale, self.weight_rescale, self.res_rescale = x_rescale, weight_rescale, res_rescale
        self.register_buffer("weight", torch.empty(out_features, in_features, dtype=dtype))
        if bias:
            self.bias = nn.Parameter(torch.empty(out_features))
        else:
            self.register_parameter("bias", None)
        self._planes = None
        self._planes_key = None
        self._scale_cache = None
        self.act_limbs = None       # None: module default ACT_LIMBS

    # -- prepared weights -------------------------------------------------------------------
    def planes(self):
        key = (self.weight.data_ptr(), _ver(self.weight), self.weight.device)
        if self._planes is None or self._planes_key != key:
            self._planes = K.WeightPlanes(self.weight, div=self.weight_rescale)
            self._planes_key = key
        return self._planes

    def shift(self):
        """the per-layer `scale` buffer as a Python int, read once (it is static)"""
        key = (self.scale.data_ptr(), _ver(self.scale))
        if self._scale_cache is None or self._scale_cache[0] != key:
            self._scale_cache = (key, int(self.scale.item()))
        return self._scale_cache[1]

    def _run(self, x, shift, want_remainder):
        lim = ACT_LIMBS if (self.act_limbs is None or ACT_LIMBS == 0) else self.act_limbs
        pl = self.planes()
        lead = x.shape[:-1]
        x3 = x.reshape(1, -1, x.shape[-1])          # every leading dimension is just more rows
        if lim > 0 and K.limb_kernel_takes(x.shape[-1], lim, pl.limbs):
            res = K.linear_prepared(x3, pl, shift, a_rescale=self.x_rescale, a_limbs=lim,
                                    want_remainder=want_remainder, dynamic=True)
        else:
            q, r = K.int64_bmm_broadcast(x3.contiguous(), self.weight, self.x_rescale, self.weight_rescale, shift)
            res = (q, r) if want_remainder else q
        if want_remainder:
            return res[0].view(*lead, -1), res[1].view(*lead, -1)
        return res.view(*lead, -1)

    def forward(self, x):
        return self._run(x, self.res_rescale, True)


class Linear_rescale_int(Linear_int):
    """Linear_int whose shift is the int32 `scale` buffer of the checkpoint; returns the quotient."""

    def __init__(self, layer_id, in_features, out_features, x_rescale, weight_rescale, dtype, bias=False):
        super().__init__(layer_id, in_features, out_features, x_rescale, weight_rescale, 1, dtype, bias)
        self.register_buffer("scale", torch.tensor(0, dtype=torch.int32))

    def forward(self, x):
        return self._run(x, self.shift(), False)


class ColumnParallelLinear_int(Linear_int):
    """Output features split over ranks (each column sees the full K: exact)."""

    def __init__(self, layer_id, in_features, out_features, x_rescale, weight_rescale, res_rescale, dtype,
                 bias=False, parallel=True):
        parts = world_size if parallel else 1
        assert out_features % parts == 0
        self.part_out_features = out_features // parts
        super().__init__(layer_id, in_features, self.part_out_features, x_rescale, weight_rescale,
                         res_rescale, dtype, bias)

    def forward(self, x):
        return self._run(x, self.res_rescale, False)


class ColumnParallelLinear_rescale_int(Linear_int):
    def __init__(self, layer_id, in_features, out_features, x_rescale, weight_rescale, dtype, bias=False,
                 parallel=True):
        parts = world_size if parallel else 1
        assert out_features % parts == 0
        self.part_out_features = out_features // parts
        super().__init__(layer_id, in_features, self.part_out_features, x_rescale, weight_rescale, 1, dtype,
                         bias)
        self.register_buffer("scale", torch.tensor(0, dtype=torch.int32))

    def forward(self, x):
        return self._run(x, self.shift(), False)


class RowParallelLinear_rescale_int(Linear_int):
    """The reference splits K over ranks and all-reduces shifted partial sums (model.py:413-448),
    which is not bit-exact against one GPU.  Here the layer keeps its full K and splits its OUTPUT
    columns over ranks; the caller all-gathers (see MLA / MLP_int)."""

    def __init__(self, layer_id, in_features, out_features, x_rescale, weight_rescale, res_rescale, dtype,
                 bias=False, parallel=True):
        self.parts = world_size if parallel else 1
        assert out_features % self.parts == 0
        self.part_out_features = out_features // self.parts
        super().__init__(layer_id, in_features, self.part_out_features, x_rescale, weight_rescale,
                         res_rescale, dtype, bias)
        self.register_buffer("scale", torch.tensor(0, dtype=torch.int32))

    def forward(self, x):
        y = self._run(x, self.shift(), False)
        if self.parts > 1:
            y = _all_gather_last(y)
        return y


def _all_gather_last(y):
    """concatenate the ranks' column blocks along the last dimension"""
    parts = [torch.empty_like(y) for _ in range(world_size)]
    dist.all_gather(parts, y.contiguous())
    return torch.cat(parts, dim=-1)


class RMSNorm_int(nn.Module):
    """floor(x * w / isqrt((1 + sum x^2) // dim)) (model.py:477-493); returns (y[None], rms_cpu)."""

    def __init__(self, dim: int, dtype, eps: float = 1e-6):
        super().__init__()
        self.dim, self.eps = dim, eps
        self.register_buffer("weight", torch.ones(dim, dtype=dtype))

    def forward(self, x):
        rows = x.reshape(-1, x.shape[-1])            # the reference handles x[0] of a [1, S, dim] input
        if snark:
            c, rms = K.RMS_Norm_int64(rows, self.weight, 1, self.dim)
        else:  # the rms stays on the device: no host copy unless a dump needs it
            c, rms = K.rms_norm_int64_device(rows, self.weight, 1, self.dim)
        return (c.view(x.shape), rms)


def precompute_freqs_cis(args: ModelArgs) -> torch.Tensor:
    """round(cis(t * f) * 2^42) as int64 [max_seq_len, rope/2, 2] with the YaRN frequency
    correction, float32 arithmetic as in the reference (model.py:496-608)."""
    dim, seqlen = args.qk_rope_head_dim, args.max_seq_len
    base, factor = args.rope_theta, args.rope_factor

    def correction_dim(num_rotations):
        return dim * math.log(args.original_seq_len / (num_rotations * 2 * math.pi)) / (2 * math.log(base))

    freqs = 1.0 / (base ** (torch.arange(0, dim, 2, dtype=torch.float32) / dim))
    if seqlen > args.original_seq_len:
        low = max(math.floor(correction_dim(args.beta_fast)), 0)
        high = min(math.ceil(correction_dim(args.beta_slow)), dim - 1)
        hi = high + 0.001 if low == high else high
        ramp = torch.clamp((torch.arange(dim // 2, dtype=torch.float32) - low) / (hi - low), 0, 1)
        smooth = 1 - ramp
        freqs = freqs / factor * (1 - smooth) + freqs * smooth
    ang = torch.outer(torch.arange(seqlen), freqs)
    cis = torch.view_as_real(torch.polar(torch.ones_like(ang), ang))
    return (cis * (2 ** 42)).round().to(torch.int64)


def apply_rotary_emb(x: torch.Tensor, freqs_cis: torch.Tensor) -> torch.Tensor:
    x = x.contiguous().view(*x.shape[:-1], -1, 2)
    freqs_cis = freqs_cis.contiguous().view(1, x.size(1), 1, x.size(-2), 2)
    return K.complex_int64_mul_broadcast(x, freqs_cis).flatten(3)


class MLA(nn.Module):
    """Absorbed multi-head latent attention in int64 (model.py:652-957)."""

    def __init__(self, layer_id, args: ModelArgs, cache_batch: int = 1, seq_parallel: bool = False):
        super().__init__()
        self.layer_id = layer_id
        # With world_size > 1: False keeps the reference's layout (every rank sees all tokens, heads and
        # output columns are split, two all-gathers).  True is the prefill layout for one sequence: every
        # rank holds S / world_size consecutive tokens, the down projections, their norms and wo run on the
        # local tokens with whole weights, the attention core runs on all tokens for the local heads, and
        # the two layouts are exchanged with one small all-gather (normed latents) and one all-to-all
        # (attention output).  Exact either way: no sum is ever split.
        self.seq_parallel = seq_parallel
        self.dim, self.n_heads = args.dim, args.n_heads
        self.n_local_heads = args.n_heads // world_size
        self.q_lora_rank, self.kv_lora_rank = args.q_lora_rank, args.kv_lora_rank
        self.qk_nope_head_dim, self.qk_rope_head_dim = args.qk_nope_head_dim, args.qk_rope_head_dim
        self.qk_head_dim = args.qk_nope_head_dim + args.qk_rope_head_dim
        self.v_head_dim = args.v_head_dim
        if self.q_lora_rank == 0:
            raise NotImplementedError("the integer model requires q_lora_rank > 0 (model.py:695-697)")
        i32 = torch.int32
        self.wq_a = Linear_int(layer_id, self.dim, self.q_lora_rank, 1, 1, 30, i32)
        self.q_norm = RMSNorm_int(self.q_lora_rank, i32)
        self.wq_b1 = ColumnParallelLinear_int(layer_id, self.q_lora_rank, self.n_heads * args.qk_nope_head_dim,
                                              1, 1, 30, i32)
        self.wq_b2 = ColumnParallelLinear_int(layer_id, self.q_lora_rank, self.n_heads * args.qk_rope_head_dim,
                                              1, 1, 30, i32)
        self.wkv_a1 = Linear_int(layer_id, self.dim, self.kv_lora_rank, 1, 1, 29, i32)
        self.wkv_a2 = Linear_int(layer_id, self.dim, self.qk_rope_head_dim, 1, 1, 29, i32)
        self.kv_norm = RMSNorm_int(self.kv_lora_rank, i32)
        self.wkv_b_1 = ColumnParallelLinear_rescale_int(layer_id, self.kv_lora_rank,
                                                        self.n_heads * self.qk_nope_head_dim, 1, 1, i32)
        self.wkv_b_2 = ColumnParallelLinear_rescale_int(layer_id, self.kv_lora_rank,
                                                        self.n_heads * self.v_head_dim, 1, 1, i32)
        self.wo = RowParallelLinear_rescale_int(layer_id, self.n_heads * self.v_head_dim, self.dim, 1, 1, 1, i32,
                                                parallel=not seq_parallel)
        self.softmax_scale1, self.softmax_scale2 = 94, 695
        # the reference keeps one sequence (model.py:740-744); cache_batch > 1 serves batched decode
        self.register_buffer("kv_cache", torch.zeros(cache_batch, args.max_seq_len, self.kv_lora_rank,
                                                     dtype=torch.int64), persistent=False)
        self.register_buffer("pe_cache", torch.zeros(cache_batch, args.max_seq_len, self.qk_rope_head_dim,
                                                     dtype=torch.int64), persistent=False)
        self._head_planes = {}
        self.score_limbs = (0, 0)   # (a, b) limb bounds of the score contractions; 0 = measure
        # Prefill with the causal mask: do not compute, write or read the masked half of the score
        # and probability tensors.  The layer's output is unchanged (a masked score always gets
        # weight 0, int64_gemm.cu:706-710); only the masked entries of the two tensors are left
        # undefined, so it is switched off whenever they are dumped (snark).
        self.causal_skip = False
        # Decode (no mask) reads the latent cache from resident limb planes (K.CachePlanes): a step splits only
        # its new position instead of copying and re-splitting the whole cache twice.  Needs promised limb
        # bounds (score_limbs); the int64 caches stay the reference copy (dumps, prefill, measured reruns) and
        # positions written by any other path are re-split lazily before the next decode step.
        self.resident_cache = True
        self._planes = None

    def _cache_planes(self, bsz, limbs):
        pl = self._planes
        if pl is None or pl.batch != bsz or pl.limbs != limbs or pl.score.device != self.kv_cache.device:
            pl = self._planes = K.CachePlanes(bsz, self.kv_cache.shape[1], self.kv_lora_rank, self.qk_rope_head_dim,
                                              limbs, self.kv_cache.device)
        return pl

    def _per_head_planes(self, lin, k_last):
        """limb planes of wkv_b_1 / wkv_b_2 viewed per head: [H, 128, 512]"""
        key = (lin.weight.data_ptr(), _ver(lin.weight), k_last)
        ent = self._head_planes.get(id(lin))
        if ent is None or ent[0] != key:
            w = lin.weight.view(self.n_local_heads, -1, self.kv_lora_rank)
            ent = (key, K.WeightPlanes(w, k_last=k_last))
            self._head_planes[id(lin)] = ent
        return ent[1]

    def forward(self, x, start_pos, freqs_cis, mask):
        if self.seq_parallel and world_size > 1:
            return self._forward_seq_parallel(x, start_pos, freqs_cis, mask)
        bsz, seqlen, _ = x.size()
        end_pos = start_pos + seqlen
        lim = ACT_LIMBS
        d = None
        q_down, q_down_rem = self.wq_a(x)
        if snark:
            d = _dump_dir(start_pos, self.layer_id)
            saveTensor(f"{d}/wq_a_x.bin", x)
            saveTensor(f"{d}/wq_a_w.bin", self.wq_a.weight.view(torch.uint32))
            saveTensor(f"{d}/wq_a_y.bin", q_down)
            saveTensor(f"{d}/q_norm_r.bin", q_down_rem)
        q_normed, rms = self.q_norm(q_down)
        if snark:
            saveTensor(f"{d}/q_norm_x.bin", q_down)
            saveTensor(f"{d}/q_norm_weight.bin", self.q_norm.weight.view(torch.uint32))
            saveTensor(f"{d}/q_norm_rms.bin", rms)
            saveTensor(f"{d}/q_norm_y.bin", q_normed)
        q_nope = self.wq_b1(q_normed).view(bsz, seqlen, self.n_local_heads, self.qk_nope_head_dim)
        q_pe = self.wq_b2(q_normed).view(bsz, seqlen, self.n_local_heads, self.qk_rope_head_dim)
        if snark:
            saveTensor(f"{d}/q_pe_x.bin", q_pe)
            saveTensor(f"{zkDataDir}/freqs_cis.bin", freqs_cis)
        q_pe = apply_rotary_emb(q_pe, freqs_cis)
        if snark:  # the reference writes q_norm.weight under this name (model.py:819)
            saveTensor(f"{d}/q_pe_y.bin", self.q_norm.weight.view(torch.uint32))
        kv, kv_rem = self.wkv_a1(x)
        if snark:
            saveTensor(f"{d}/wkv_a1_x.bin", x)
            saveTensor(f"{d}/wkv_a1_w.bin", self.wkv_a1.weight.view(torch.uint32))
            saveTensor(f"{d}/wkv_a1_y.bin", kv)
            saveTensor(f"{d}/wkv_a1_r.bin", kv_rem)
        k_pe, _ = self.wkv_a2(x)
        k_pe = apply_rotary_emb(k_pe.unsqueeze(2), freqs_cis)
        kv_normed, rms = self.kv_norm(kv)
        ctx = self._core(q_nope, q_pe, kv_normed, k_pe.squeeze(2), bsz, seqlen, start_pos, mask, d)
        return self._finish(ctx, lim)

    def _forward_seq_parallel(self, x, start_pos, freqs_cis, mask):
        """x [1, S / world_size, dim]: this rank's consecutive tokens of one sequence; freqs_cis and mask
        cover all S tokens.  Returns the layer output for the same local tokens."""
        if snark:
            raise NotImplementedError("the zkdata dumps are written from the one-GPU layout")
        bsz, s_loc, _ = x.size()
        assert bsz == 1
        S = s_loc * world_size
        fr_loc = freqs_cis[rank * s_loc:(rank + 1) * s_loc]
        q_normed, _ = self.q_norm(self.wq_a(x)[0])
        kv_normed, _ = self.kv_norm(self.wkv_a1(x)[0])
        k_pe = apply_rotary_emb(self.wkv_a2(x)[0].unsqueeze(2), fr_loc).squeeze(2)
        qr, C = self.q_lora_rank, self.kv_lora_rank
        local = torch.cat([q_normed, kv_normed, k_pe], dim=-1)[0].contiguous()         # [s_loc, q + C + rope]
        full = torch.empty((S, local.shape[1]), dtype=torch.int64, device=x.device)
        dist.all_gather_into_tensor(full, local)         # token blocks in rank order: the whole [S, .] matrix
        q_all = full[:, :qr].contiguous()[None]
        q_nope = self.wq_b1(q_all).view(1, S, self.n_local_heads, self.qk_nope_head_dim)
        q_pe = self.wq_b2(q_all).view(1, S, self.n_local_heads, self.qk_rope_head_dim)
        q_pe = apply_rotary_emb(q_pe, freqs_cis)
        ctx = self._core(q_nope, q_pe, full[:, qr:qr + C][None], full[:, qr + C:][None], 1, S, start_pos, mask, None)
        out = self._project_heads(ctx, ACT_LIMBS)                                       # [1, S, local heads * v]
        # head-split -> token-split: rank j receives its token block from every rank's heads
        cols = out.shape[-1]
        recv = torch.empty((world_size, s_loc, cols), dtype=torch.int64, device=x.device)
        dist.all_to_all_single(recv, out.view(world_size, s_loc, cols))
        del out
        rows = recv.permute(1, 0, 2).reshape(1, s_loc, world_size * cols)               # heads in rank order
        return self.wo(rows)

    def _core(self, q_nope, q_pe, kv_normed, k_pe, bsz, seqlen, start_pos, mask, d):
        """caches, scores, softmax, P . KV for the local heads: returns ctx [b, s, h, c]"""
        end_pos = start_pos + seqlen
        lim = ACT_LIMBS
        # q_nope . W_uk per head  (einsum_bshd_hdc_bshc, weight [H, D, C]: K is the middle axis)
        shift1 = self.wkv_b_1.shift()
        if lim > 0 and K.limb_kernel_takes(self.qk_nope_head_dim, lim, 5):
            q_abs = K.einsum_heads_prepared(q_nope.contiguous(), self._per_head_planes(self.wkv_b_1, False),
                                            shift1, True, a_limbs=lim, dynamic=True)
        else:
            w1 = self.wkv_b_1.weight.view(self.n_local_heads, -1, self.kv_lora_rank)
            q_abs = K.einsum_bshd_hdc_bshc(q_nope.contiguous(), w1.contiguous(), shift1)
        self.kv_cache[:bsz, start_pos:end_pos] = kv_normed
        self.pe_cache[:bsz, start_pos:end_pos] = k_pe
        al, bl = self.score_limbs
        dyn = al > 0
        if (self.resident_cache and mask is None and seqlen == 1 and not snark and K.ALGO != K.ALGO_EXACT
                and al > 0 and bl > 0):
            pl = self._cache_planes(bsz, bl)
            if pl.filled < start_pos:      # positions another path wrote (prefill, a filled cache): split them once
                pl.append(self.kv_cache[:bsz, pl.filled:start_pos].contiguous(),
                          self.pe_cache[:bsz, pl.filled:start_pos].contiguous(), pl.filled)
            pl.append(kv_normed.contiguous(), k_pe.contiguous(), start_pos)
            # score rows padded to a multiple of four columns (what the softmax-to-planes kernel reads); the
            # padding columns come from cache positions that are not in use and are never read: the softmax
            # and P . KV stop at column start_pos
            t4 = (end_pos + 3) // 4 * 4
            scores = pl.scores(q_abs, q_pe.contiguous(), t4, 23, 21, self.softmax_scale1, self.softmax_scale2,
                               a_limbs=al, dynamic=True)
            if scores is not None:
                ctx = pl.softmax_pv(scores, 23, a_limbs=3, valid_start=start_pos)
                if ctx is not None:
                    return ctx
        elif self._planes is not None:
            self._planes.filled = min(self._planes.filled, start_pos)     # these positions changed under the planes
        kv_all = self.kv_cache[:bsz, :end_pos].contiguous()
        pe_all = self.pe_cache[:bsz, :end_pos].contiguous()

        # scores = (score1 + score2) * 94 // 695 (+ mask): the tail runs in the second epilogue
        causal = mask is not None and start_pos == 0 and _is_causal_mask(mask, seqlen)
        scores = None
        if K.ALGO != K.ALGO_EXACT:
            skip = causal and self.causal_skip and not snark and dyn and bl > 0
            scores = K.mla_scores_fused(q_abs, kv_all, q_pe.contiguous(), pe_all, 23, 21, self.softmax_scale1,
                                        self.softmax_scale2, causal=causal, a_limbs=al, b_limbs=bl, dynamic=dyn,
                                        skip_masked=skip)
            if scores is not None and skip:
                ctx = K.softmax_pv_fused(scores, kv_all, 23, causal_skip=True, start_pos=0, a_limbs=3, b_limbs=bl)
                if ctx is not None:
                    del scores
                    return ctx
                probs = torch.empty_like(scores)
                if K.softmax_q19_causal(scores, probs, 0):
                    del scores
                    ctx = K.einsum_bsht_btc_bshc_causal(probs, kv_all, 23, 0, a_limbs=3, b_limbs=bl)
                    del probs
                    return ctx
                # softmax shape not taken by the causal kernel: recompute the scores in full
                scores = K.mla_scores_fused(q_abs, kv_all, q_pe.contiguous(), pe_all, 23, 21, self.softmax_scale1,
                                            self.softmax_scale2, causal=causal, a_limbs=al, b_limbs=bl,
                                            dynamic=dyn)
        if scores is None:      # shape outside the fused kernel: two contractions, tail in the second
            score1 = K.attention_scores_fused(q_abs, kv_all, 23, a_limbs=al, b_limbs=bl, dynamic=dyn)
            scores = K.attention_scores_fused(q_pe.contiguous(), pe_all, 21, addin=score1,
                                              mul=self.softmax_scale1, div=self.softmax_scale2, causal=causal,
                                              start_pos=0, a_limbs=al, b_limbs=bl, dynamic=dyn)
            del score1
        if mask is not None and not causal:
            scores += mask.unsqueeze(1)
        if snark:
            saveTensor(f"{d}/scores_softmax_x.bin", scores)
        elif K.ALGO != K.ALGO_EXACT:
            # softmax and P . KV in one call: the probabilities only ever exist as int8 limb planes
            ctx = K.softmax_pv_fused(scores, kv_all, 23, a_limbs=3, b_limbs=bl)
            if ctx is not None:
                del scores
                return ctx
        probs = torch.empty_like(scores)
        K.softmax_q19(scores, probs)
        del scores
        if snark:
            saveTensor(f"{d}/scores_softmax_y.bin", probs)
        # probabilities are in [0, 2^19]: three limbs
        ctx = K.einsum_bsht_btc_bshc(probs, kv_all, 23, a_limbs=3 if dyn else 0, b_limbs=bl)
        del probs
        return ctx

    def _finish(self, ctx, lim):
        """ctx [b, s, h, c] -> per-head W_uv, concatenate heads, output projection"""
        out = self._project_heads(ctx, lim)
        if world_size > 1:
            out = _all_gather_last(out)      # heads of every rank, then a column-split wo
        return self.wo(out)

    def _project_heads(self, ctx, lim):
        """ctx [b, s, h, c] -> per-head W_uv -> [b, s, h * v]"""
        shift2 = self.wkv_b_2.shift()
        if lim > 0 and K.limb_kernel_takes(self.kv_lora_rank, lim, 5):
            out = K.einsum_heads_prepared(ctx, self._per_head_planes(self.wkv_b_2, True), shift2, False,
                                          a_limbs=lim, dynamic=True)
        else:
            w2 = self.wkv_b_2.weight.view(self.n_local_heads, -1, self.kv_lora_rank)
            out = K.einsum_bshc_hdc_bshd(ctx, w2.contiguous(), shift2)
        return out.flatten(2)


def _is_causal_mask(mask, seqlen):
    """True for the mask the reference builds (model.py:1555): -(64<<36) strictly above the
    diagonal of a [seqlen, seqlen] matrix, zeros elsewhere.  Identity-cached per tensor."""
    cached = getattr(mask, "_zkds_causal", None)
    if cached is not None:
        return cached
    ok = (mask.shape == (seqlen, seqlen) and mask.dtype == torch.int64 and bool(
        torch.equal(mask, torch.full_like(mask, -(64 << 36)).triu_(1))))
    try:
        mask._zkds_causal = ok
    except AttributeError:
        pass
    return ok


class MLP_int(nn.Module):
    """w2((silu_q23(w1 x) * w3 x) >> 23) (model.py:994-1049); w1 and w3 run as one stacked GEMM
    when their shifts agree."""

    def __init__(self, layer_id, dim: int, inter_dim: int, parallel: bool = True):
        super().__init__()
        self.layer_id = layer_id
        self.inter_dim = inter_dim
        self.parts = world_size if parallel else 1
        i32 = torch.int32
        self.w1 = ColumnParallelLinear_rescale_int(layer_id, dim, inter_dim, 1, 1, i32, parallel=parallel)
        self.w2 = RowParallelLinear_rescale_int(layer_id, inter_dim, dim, 1, 1, 1, i32, parallel=parallel)
        self.w3 = ColumnParallelLinear_rescale_int(layer_id, dim, inter_dim, 1, 1, i32, parallel=parallel)
        self._w13 = None

    def _stacked(self):
        key = (self.w1.weight.data_ptr(), _ver(self.w1.weight), self.w3.weight.data_ptr(),
               _ver(self.w3.weight))
        if self._w13 is None or self._w13[0] != key:
            w13 = torch.cat([self.w1.weight, self.w3.weight], dim=0).contiguous()
            self._w13 = (key, K.WeightPlanes(w13))
        return self._w13[1]

    def forward(self, start_pos: int, x: torch.Tensor) -> torch.Tensor:
        s1, s3 = self.w1.shift(), self.w3.shift()
        lim = ACT_LIMBS
        n = self.w1.weight.shape[0]
        if lim > 0 and s1 == s3 and K.limb_kernel_takes(x.shape[-1], lim, 5):
            r13 = K.linear_prepared(x.reshape(1, -1, x.shape[-1]), self._stacked(), s1, a_limbs=lim, dynamic=True)
            r13 = r13.view(-1, 2 * n)
            r1, r2, ld = r13[:, :n], r13[:, n:], 2 * n
        else:
            r1 = self.w1(x).view(-1, n)
            r2 = self.w3(x).view(-1, n)
            ld = n
        if snark:
            h, sl = K.glu_q23(r1, r2, ld=ld, want_silu=True)
            d = _dump_dir(start_pos, self.layer_id)
            saveTensor(f"{d}/mlp_silu_x.bin", r1.contiguous().view(x.shape[0], -1, n))
            saveTensor(f"{d}/mlp_silu_y.bin", sl.view(x.shape[0], -1, n))
        else:
            if self.parts == 1 and lim > 0 and self.w2.x_rescale == 1 and \
                    K.limb_kernel_takes(n, lim, self.w2.planes().limbs):
                # gate and down projection in one call: h only exists as limb planes
                out = K.glu_prepared(r1, r2, self.w2.planes(), self.w2.shift(), ld=ld, a_limbs=lim, dynamic=True)
                if out is not None:
                    return out.view(*x.shape[:-1], -1)
            h = K.glu_q23(r1, r2, ld=ld)
        h = h.view(*x.shape[:-1], n)
        if self.parts > 1:
            h = _all_gather_last(h)
        return self.w2(h)


class Gate(nn.Module):
    """Sigmoid gate with grouped top-k routing in integers (model.py:1052-1212)."""

    def __init__(self, layer_id: int, args: ModelArgs):
        super().__init__()
        self.layer_id = layer_id
        self.dim = args.dim
        self.topk = args.n_activated_experts
        self.n_groups, self.topk_groups = args.n_expert_groups, args.n_limited_groups
        self.score_func, self.route_scale = args.score_func, args.route_scale
        self.register_buffer("weight", torch.empty(args.n_routed_experts, args.dim, dtype=torch.int32))
        self.register_buffer("scale", torch.tensor(0, dtype=torch.int32))
        if self.dim == 7168:
            self.register_buffer("bias", torch.empty(args.n_routed_experts, dtype=torch.int32))
        else:
            self.bias = None
        self._lin = None

    def _linear(self):
        key = (self.weight.data_ptr(), _ver(self.weight), self.scale.data_ptr(), _ver(self.scale))
        if self._lin is None or self._lin[0] != key:
            self._lin = (key, K.WeightPlanes(self.weight), int(self.scale.item()))
        return self._lin[1], self._lin[2]

    def forward(self, start_pos: int, x: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
        if self.score_func != "sigmoid":
            raise NotImplementedError("the integer model routes with the sigmoid score function")
        x3 = x.view(1, -1, self.dim)
        planes, rescale = self._linear()
        lim = ACT_LIMBS
        if lim > 0 and K.limb_kernel_takes(self.dim, lim, planes.limbs):
            scores, scores_rem = K.linear_prepared(x3, planes, rescale, a_limbs=lim, want_remainder=True,
                                                   dynamic=True)
        else:
            scores, scores_rem = linear_int(x3, self.weight, 1, 1, rescale)
        sig = torch.empty_like(scores)
        if snark:
            d = _dump_dir(start_pos, self.layer_id)
            saveTensor(f"{d}/sigmoid_gate_x.bin", scores)
            saveTensor(f"{d}/sigmoid_gate_r.bin", scores_rem)
        K.sigmoid_q23(scores, sig)
        if snark:
            saveTensor(f"{d}/sigmoid_gate_y.bin", sig)
        scores = sig.squeeze(0)
        original_scores = scores
        if self.bias is not None:
            scores = scores + self.bias
        if snark:
            saveTensor(f"{d}/gate_original_scores.bin", original_scores.contiguous())
            saveTensor(f"{d}/gate_bias.bin", self.bias.view(torch.uint32))
        T = scores.size(0)
        fused = K.gate_select(original_scores.contiguous(), self.bias, self.n_groups, self.topk_groups, self.topk) \
            if FUSED_GATE else None
        if fused is not None:
            weights, indices, raw = fused
            if snark:
                saveTensor(f"{d}/gate_indices.bin", indices)
                saveTensor(f"{d}/gate_weights.bin", raw)
            return weights, indices
        if self.n_groups > 1:
            scores = scores.view(T, self.n_groups, -1)
            if self.bias is None:
                group_scores = scores.amax(dim=-1)
            else:
                group_scores = scores.topk(2, dim=-1)[0].sum(dim=-1)
            indices = group_scores.topk(self.topk_groups, dim=-1)[1]
            gmask = scores.new_ones(T, self.n_groups, dtype=torch.bool).scatter_(1, indices, False)
            scores = scores.masked_fill(gmask.unsqueeze(-1), -(1 << 42)).flatten(1)
        indices = torch.topk(scores, self.topk, dim=-1)[1]
        weights = original_scores.gather(1, indices)
        if snark:
            saveTensor(f"{d}/gate_indices.bin", indices.contiguous())
            saveTensor(f"{d}/gate_weights.bin", weights.contiguous())
        weights = (weights * (2 ** 23)) // weights.sum(dim=-1, keepdim=True)
        weights = weights * 5 // 2
        return weights, indices


class Expert_int(nn.Module):
    """One routed expert (model.py:1214-1281): w2((silu_q23(w1 x) * w3 x) >> 23)."""

    def __init__(self, layer_id, idx, dim: int, inter_dim: int):
        super().__init__()
        self.layer_id, self.idx = layer_id, idx
        i32 = torch.int32
        self.w1 = Linear_rescale_int(layer_id, dim, inter_dim, 1, 1, i32)
        self.w2 = Linear_rescale_int(layer_id, inter_dim, dim, 1, 1, i32)
        self.w3 = Linear_rescale_int(layer_id, dim, inter_dim, 1, 1, i32)

    def forward(self, start_pos: int, x: torch.Tensor) -> torch.Tensor:
        n = self.w1.weight.shape[0]
        r1 = self.w1(x).view(-1, n)
        r2 = self.w3(x).view(-1, n)
        if snark:
            h, sl = K.glu_q23(r1, r2, want_silu=True)
            d = _dump_dir(start_pos, self.layer_id)
            saveTensor(f"{d}/expert_{self.idx}_silu_x.bin", r1.view(x.shape[0], -1, n))
            saveTensor(f"{d}/expert_{self.idx}_silu_y.bin", sl.view(x.shape[0], -1, n))
        else:
            h = K.glu_q23(r1, r2)
        return self.w2(h.view(*x.shape[:-1], n))


class MoE(nn.Module):
    """Shared expert + sigmoid-gated top-k routed experts (model.py:1283-1383).

    Experts of this rank are kept resident as two stacked weights (`experts_w13` [E, 2I, dim],
    `experts_w2` [E, dim, I]) with per-expert shifts `experts_shift` [E, 3] (w1, w3, w2) and run as
    grouped GEMMs over token rows sorted by expert.  `set_experts()` fills them from Expert_int
    modules or from the checkpoint's `experts-{layer}/{i}.safetensors` files."""

    def __init__(self, layer_id, args: ModelArgs, ckpt_path=None, token_parallel: bool = False):
        super().__init__()
        self.layer_id, self.ckpt_path = layer_id, ckpt_path
        # False: every rank sees all tokens (the reference's layout under tensor parallelism),
        # runs its own experts on them and the partial sums are all-reduced (exact: integer adds).
        # True: every rank holds its own tokens; rows travel to the experts' owners and back with
        # all-to-all, gate and shared expert run on the local tokens with whole weights.
        self.token_parallel = token_parallel
        self.last_counts = None
        self.dim, self.moe_inter_dim = args.dim, args.moe_inter_dim
        assert args.n_routed_experts % world_size == 0
        self.n_routed_experts = args.n_routed_experts
        self.n_local_experts = args.n_routed_experts // world_size
        self.n_activated_experts = args.n_activated_experts
        self.experts_start_idx = rank * self.n_local_experts
        self.experts_end_idx = self.experts_start_idx + self.n_local_experts
        self.gate = Gate(layer_id, args)
        self.shared_experts = MLP_int(layer_id, args.dim, args.n_shared_experts * args.moe_inter_dim,
                                      parallel=not token_parallel)
        E, I, D = self.n_local_experts, args.moe_inter_dim, args.dim
        self.register_buffer("experts_w13", torch.empty(E, 2 * I, D, dtype=torch.int32), persistent=False)
        self.register_buffer("experts_w2", torch.empty(E, D, I, dtype=torch.int32), persistent=False)
        self.register_buffer("experts_shift", torch.zeros(E, 3, dtype=torch.int32), persistent=False)
        self._planes = None

    def set_experts(self, experts=None):
        """copy the local experts' weights into the stacked buffers (from modules, or from disk)"""
        for j in range(self.n_local_experts):
            i = self.experts_start_idx + j
            if experts is not None:
                e = experts[j]
            else:
                from safetensors.torch import load_model
                e = Expert_int(self.layer_id, i, self.dim, self.moe_inter_dim)
                load_model(e, os.path.join(self.ckpt_path, f"experts-{self.layer_id}/{i}.safetensors"))
            I = self.moe_inter_dim
            self.experts_w13[j, :I].copy_(e.w1.weight)
            self.experts_w13[j, I:].copy_(e.w3.weight)
            self.experts_w2[j].copy_(e.w2.weight)
            self.experts_shift[j] = torch.stack([e.w1.scale, e.w3.scale, e.w2.scale]).to(torch.int32)
        self._planes = None

    def _prepared(self):
        key = (_ver(self.experts_w13), _ver(self.experts_w2), _ver(self.experts_shift),
               self.experts_w13.data_ptr())
        if self._planes is None or self._planes[0] != key:
            sh = self.experts_shift
            s13 = torch.stack([sh[:, 0], sh[:, 1]], dim=1).contiguous()
            s2 = torch.stack([sh[:, 2], sh[:, 2]], dim=1).contiguous()
            self._planes = (key, K.WeightPlanes(self.experts_w13), K.WeightPlanes(self.experts_w2), s13, s2)
        return self._planes[1:]

    def route(self, indices, max_pairs=None):
        """rows sorted by local expert and padded to 128 per expert.  Returns
        row_src int32 [R] (token of each row, -1 = padding), pos int32 [T, k] (row of each
        (token, slot), -1 = not a local expert), tile_group int32 [R / 128].
        max_pairs: a bound on the (token, slot) pairs that name a local expert when the caller knows one
        smaller than T * k (expert parallelism: most slots of a received row belong to other ranks)."""
        T, k = indices.shape
        E = self.n_local_experts
        dev = indices.device
        flat = indices.flatten() - self.experts_start_idx
        local = (flat >= 0) & (flat < E)
        key = torch.where(local, flat, torch.full_like(flat, E))
        order = torch.argsort(key, stable=True)
        skey = key[order]
        # every tensor below has a static shape and nothing is read back: no host synchronisation
        counts = torch.zeros(E + 1, dtype=torch.int64, device=dev).index_add_(0, key, torch.ones_like(key))[:E]
        padded = (counts + 127) // 128 * 128
        pad_end = torch.cumsum(padded, 0)
        pad_start = pad_end - padded
        start = torch.cumsum(counts, 0) - counts
        n_tiles = ((T * k if max_pairs is None else min(T * k, max_pairs)) + E * 127) // 128
        R = n_tiles * 128
        ar = torch.arange(T * k, device=dev)
        valid = skey < E
        e_safe = torch.clamp(skey, max=E - 1)
        rows = torch.where(valid, pad_start[e_safe] + (ar - start[e_safe]), torch.full_like(ar, R))
        row_src = torch.full((R + 1,), -1, dtype=torch.int32, device=dev)      # slot R swallows the rest
        row_src.scatter_(0, rows, (order // k).to(torch.int32))
        row_src = row_src[:R].contiguous()
        pos = torch.empty((T * k,), dtype=torch.int32, device=dev)
        pos[order] = torch.where(valid, rows, torch.full_like(rows, -1)).to(torch.int32)
        tile_start = torch.arange(n_tiles, device=dev) * 128
        g = torch.searchsorted(pad_end, tile_start, right=True)
        tile_group = torch.where(tile_start < pad_end[-1], g, torch.full_like(g, -1)).to(torch.int32)
        return row_src, pos.view(T, k), tile_group, counts

    def experts_forward(self, start_pos, x, weights, indices, base=None, max_pairs=None, parts=None, combine=None):
        """sum over the local experts of expert(x) * w // 2^23, added to `base`.
        parts = (device addresses, rows per buffer): the token rows lie in several buffers (every rank's rows,
        read in place; `indices` then covers all of them) instead of x.  combine(out, pos): what to do with the
        experts' output rows instead of the local weighted sum."""
        w13, w2, s13, s2 = self._prepared()
        lim = ACT_LIMBS if ACT_LIMBS > 0 else 5
        row_src, pos, tile_group, counts = self.route(indices, max_pairs)
        self.last_counts = counts          # rows per local expert of the latest call (device tensor, not read here)
        I = self.moe_inter_dim
        # a token names an expert at most once: no expert receives more rows than there are token rows
        n_rows = indices.shape[0]
        few = n_rows if n_rows <= 64 else None
        if OPTIMISTIC_GROUP_ROWS and n_rows > 32:
            mean_rows = n_rows * indices.shape[1] / float(self.n_routed_experts)
            if mean_rows <= 8:
                few = 32
            elif mean_rows <= 20 and few is None:
                few = 64
        finish = combine if combine is not None else (
            lambda out, pos: K.moe_combine(out, pos, weights.contiguous(), base))
        # the dispatch gather (model.py:1372-1378) runs inside the limb split of the first GEMM
        if parts is not None:
            r13 = K.grouped_gather_parts_prepared(parts[0], parts[1], row_src, w13, tile_group, 0, a_limbs=lim,
                                                  dynamic=True, group_shift=s13, n_split=I, max_group_rows=few)
        else:
            r13 = K.grouped_prepared(x.contiguous(), w13, tile_group, 0, a_limbs=lim, dynamic=True, group_shift=s13,
                                     n_split=I, row_index=row_src, max_group_rows=few)
        if snark:
            h, sl = K.glu_q23(r13[:, :I], r13[:, I:], ld=2 * I, want_silu=True)
            self._dump_experts(start_pos, r13[:, :I], sl, counts)
        else:
            out = K.glu_prepared(r13[:, :I], r13[:, I:], w2, 0, ld=2 * I, a_limbs=lim, dynamic=True,
                                 tile_group=tile_group, group_shift=s2, n_split=0, max_group_rows=few)
            if out is not None:
                return finish(out, pos)
            h = K.glu_q23(r13[:, :I], r13[:, I:], ld=2 * I)
        out = K.grouped_prepared(h, w2, tile_group, 0, a_limbs=lim, dynamic=True, group_shift=s2, n_split=0,
                                 max_group_rows=few)
        return finish(out, pos)

    def _dump_experts(self, start_pos, r1, sl, counts):
        d = _dump_dir(start_pos, self.layer_id)
        cnt = counts.tolist()
        row = 0
        for j, c in enumerate(cnt):
            if c:
                i = self.experts_start_idx + j
                saveTensor(f"{d}/expert_{i}_silu_x.bin", r1[row:row + c].contiguous()[None])
                saveTensor(f"{d}/expert_{i}_silu_y.bin", sl[row:row + c].contiguous()[None])
            row += (c + 127) // 128 * 128

    def forward(self, start_pos: int, x: torch.Tensor) -> torch.Tensor:
        shape = x.size()
        if world_size > 1 and self.token_parallel:
            from . import parallel
            x2 = x.view(-1, self.dim)
            weights, indices = self.gate(start_pos, x2)
            if PEER_EXPERTS and x2.is_cuda and not snark and parallel.peer_available():
                # rows read and results written over peer memory by the expert kernels themselves; the shared
                # expert runs while the pair count travels to the host and is added by the slot sum
                y, _ = parallel.expert_parallel_forward_peer(
                    self, K, start_pos, x2.contiguous(), weights, indices,
                    before_sync=lambda: self.shared_experts(start_pos, x).view(-1, self.dim).contiguous())
                return y.view(shape)
            # the shared expert runs while the dispatch counts travel to the host
            y, z = parallel.expert_parallel_forward(self, start_pos, x2, weights, indices,
                                                    before_sync=lambda: self.shared_experts(start_pos, x))
            return (y + z.view(-1, self.dim)).view(shape)
        z = self.shared_experts(start_pos, x)
        x = x.view(-1, self.dim)
        weights, indices = self.gate(start_pos, x)
        if world_size > 1:
            y = self.experts_forward(start_pos, x, weights, indices)
            dist.all_reduce(y)                        # model.py:1381-1382
            return (y + z.view(-1, self.dim)).view(shape)
        y = self.experts_forward(start_pos, x, weights, indices, base=z.view(-1, self.dim).contiguous())
        return y.view(shape)


class Block(nn.Module):
    """attn_norm -> MLA -> residual (x 2^12) -> ffn_norm -> MLP | MoE -> residual (x 2^8)
    (model.py:1401-1475)."""

    def __init__(self, layer_id: int, args: ModelArgs, ckpt_path=None, cache_batch: int = 1):
        super().__init__()
        self.layer_id, self.ckpt_path = layer_id, ckpt_path
        self.attn = MLA(layer_id, args, cache_batch)
        self.ffn = (MLP_int(layer_id, args.dim, args.inter_dim) if layer_id < args.n_dense_layers
                    else MoE(layer_id, args, ckpt_path))
        self.attn_norm = RMSNorm_int(args.dim, torch.int32)
        self.ffn_norm = RMSNorm_int(args.dim, torch.int32)

    def forward(self, x, start_pos, freqs_cis, mask):
        atten_normed, rms = self.attn_norm(x)
        if snark:
            d = _dump_dir(start_pos, self.layer_id)
            saveTensor(f"{d}/attn_norm_x.bin", x)
            saveTensor(f"{d}/attn_norm_weight.bin", self.attn_norm.weight.view(torch.uint32))
            saveTensor(f"{d}/attn_norm_y.bin", atten_normed)
            saveTensor(f"{d}/attn_norm_rms.bin", rms)
        attned = self.attn(atten_normed, start_pos, freqs_cis, mask)
        x = x + attned * (2 ** 12)
        ffn_normed, rms = self.ffn_norm(x)
        ffned = self.ffn(start_pos, ffn_normed)
        x = x + ffned * (2 ** 8)
        if snark and CHECK_STATUS:      # dumps of a step whose limb bound did not hold must not be trusted
            K.device_status(sync=True)
        return x


class Transformer(nn.Module):
    """Embedding, per-layer inference steps, final norm and head (model.py:1477-1583)."""

    def __init__(self, args: ModelArgs):
        global world_size, rank
        world_size = dist.get_world_size() if dist.is_initialized() else 1
        rank = dist.get_rank() if dist.is_initialized() else 0
        super().__init__()
        self.args = args
        self.max_seq_len = args.max_seq_len
        self.embed = ParallelEmbedding(args.vocab_size, args.dim)
        self.layers = torch.nn.ModuleList()
        for _ in range(args.n_layers):
            self.layers.append(nn.Module())
        self.norm = RMSNorm_int(args.dim, torch.int64)
        self.head = ColumnParallelLinear_int(-1, args.dim, args.vocab_size, 1, (1 << 8), 29, torch.int64)
        self.register_buffer("freqs_cis", precompute_freqs_cis(args), persistent=False)
        self._luts_ready = False

    @torch.inference_mode()
    def prep_inference(self, tokens: torch.Tensor, start_pos: int = 0):
        if not self._luts_ready:   # the tables are constants: built once, not every step
            K.softmax_init_q19()
            K.softmax_init_q21()
            K.silu_init_q23()
            self._luts_ready = True
        seqlen = tokens.size(1)
        return (self.embed(tokens), start_pos, seqlen)

    @torch.inference_mode()
    def layer_inference(self, layer_id, h, start_pos, seqlen):
        freqs_cis = self.freqs_cis[start_pos:start_pos + seqlen]
        mask = None
        if seqlen > 1:
            mask = torch.full((seqlen, seqlen), -(64 << 36), dtype=torch.int64, device=h.device).triu_(1)
            mask._zkds_causal = True
        return self.layers[layer_id](h, start_pos, freqs_cis, mask)

    @torch.inference_mode()
    def finish_inference(self, h):
        h = self.norm(h)[0][:, -1].contiguous()          # last position of every sequence: [B, dim]
        logits = self.head(h[None, :])      # [1, B, vocab] (B = 1 in the reference)
        if world_size > 1:
            logits = _all_gather_last(logits)
        if CHECK_STATUS:
            K.device_status(sync=True)      # raises ZkdsError (status ERR_RANGE) if a limb bound did not hold
        return logits


class measured_limbs:
    """Context manager: every activation's limb count is measured on the device (ACT_LIMBS = 0, score
    contractions included) instead of promised.  Slower (one host synchronisation per GEMM), never wrong;
    generate() uses it to re-run a step whose promised bound did not hold."""

    def __init__(self, model):
        self.model = model

    def __enter__(self):
        global ACT_LIMBS, OPTIMISTIC_GROUP_ROWS
        self.saved = (ACT_LIMBS, [(m, m.score_limbs, m.causal_skip) for m in self.model.modules()
                                  if isinstance(m, MLA)], OPTIMISTIC_GROUP_ROWS)
        ACT_LIMBS = 0
        OPTIMISTIC_GROUP_ROWS = False
        for m, _, _ in self.saved[1]:
            m.score_limbs, m.causal_skip = (0, 0), False
        return self

    def __exit__(self, *exc):
        global ACT_LIMBS, OPTIMISTIC_GROUP_ROWS
        ACT_LIMBS = self.saved[0]
        OPTIMISTIC_GROUP_ROWS = self.saved[2]
        for m, sl, cs in self.saved[1]:
            m.score_limbs, m.causal_skip = sl, cs
        return False
