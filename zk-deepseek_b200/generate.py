"""Token generation over the integer model with every layer resident on the GPU.

Follows the loop of the reference's `generate()` (inference/generate.py:164-286): the prompt
is run as one prefill, then one position per step; `prompt_mask` keeps prompt tokens from being
overwritten when the prompts of a batch have different lengths; a sequence finishes at `eos_id`;
with `snark` set in the model module every step writes `pos_{p}/tokens.bin` next to the layer
dumps (generate.py:218-220).

Differences, all on the host side of the hot path:
  * the reference rebuilds `Block(i)` from its state dict and moves the latent caches to the GPU
    for every layer of every step (generate.py:231-244) because the 671B model does not fit one
    GPU; here the layers, their limb planes, the caches and the lookup tables stay resident;
  * the per-layer debug projection through `norm` and `head` (generate.py:246-259) is off unless
    `layer_probe=True`; it then returns the same per-layer candidate token ids instead of printing;
  * `sample()` in the reference has its stochastic branch switched off (`sample_open = False`,
    generate.py:80) and returns the argmax for every temperature; the same is done here.
"""
import os
from typing import List, Optional

import torch

try:
    from . import model as M
except ImportError:  # pragma: no cover - drop-in use with this directory first on sys.path
    import model as M


def load_resident(ckpt_path: str, args, device="cuda", cache_batch: int = 1, prepare: bool = True):
    """Builds a `Transformer` with every layer on `device` from a converted checkpoint directory:
    `embed_int.safetensors`, `norm_int.safetensors`, `head_int.safetensors` (generate.py:53-60),
    `layer-{i}.safetensors` (generate.py:344-345, loaded with strict=False as generate.py:238 does) and
    `experts-{layer}/{i}.safetensors` (model.py:1361-1363).  The reference keeps the layer state dicts on the
    host and rebuilds one `Block` at a time; here all of them stay resident, and with `prepare` the limb
    planes of every static weight are built once at load instead of at first use."""
    from safetensors.torch import load_file, load_model
    with torch.device(device):
        model = M.Transformer(args)
    load_model(model.embed, os.path.join(ckpt_path, "embed_int.safetensors"))
    load_model(model.norm, os.path.join(ckpt_path, "norm_int.safetensors"))
    load_model(model.head, os.path.join(ckpt_path, "head_int.safetensors"))
    for i in range(args.n_layers):
        with torch.device(device):
            blk = M.Block(i, args, ckpt_path, cache_batch=cache_batch)
        blk.load_state_dict(load_file(os.path.join(ckpt_path, f"layer-{i}.safetensors"), device=str(device)),
                            strict=False)
        if isinstance(blk.ffn, M.MoE):
            blk.ffn.set_experts()
        model.layers[i] = blk
    if prepare:
        for mod in model.modules():
            if isinstance(mod, M.Linear_int):
                mod.planes()
            elif isinstance(mod, M.MoE):
                mod._prepared()
    return model


def sample(logits: torch.Tensor, temperature: float = 1.0) -> torch.Tensor:
    """generate.py:62-143 with `sample_open = False`: the argmax over the vocabulary."""
    return logits.argmax(dim=-1)


def _forward_step(model, toks, prev_pos, layer_probe):
    """one pass over all layers; finish_inference raises ZkdsError if a kernel flagged its operands"""
    h, start_pos, seqlen = model.prep_inference(toks, prev_pos)
    layer_tokens = []
    for i in range(model.args.n_layers):
        h = model.layer_inference(i, h, start_pos, seqlen)
        if layer_probe:
            probe = model.head(model.norm(h)[0][:, -1].contiguous()[None, :])
            layer_tokens.append(probe.argmax(dim=-1).view(-1).tolist())
    return model.finish_inference(h), layer_tokens


@torch.inference_mode()
def generate(model, prompt_tokens: List[List[int]], max_new_tokens: int, eos_id: int,
             temperature: float = 1.0, layer_probe: bool = False,
             trace: Optional[list] = None) -> List[List[int]]:
    """Returns the completion tokens of every prompt (generate.py:164-286).

    model: a `Transformer` whose `layers[i]` are loaded `Block`s (caches sized for the batch).
    trace: optional list; receives one dict per step (`pos`, `next_token`, and `layer_tokens` when
    `layer_probe` is set) in place of the reference's progress prints.
    """
    args = model.args
    device = model.freqs_cis.device
    prompt_lens = [len(t) for t in prompt_tokens]
    assert max(prompt_lens) <= args.max_seq_len, \
        f"Prompt length exceeds model maximum sequence length (max_seq_len={args.max_seq_len})"
    total_len = min(args.max_seq_len, max_new_tokens + max(prompt_lens))
    tokens = torch.full((len(prompt_tokens), total_len), -1, dtype=torch.long, device=device)
    for i, t in enumerate(prompt_tokens):
        tokens[i, :len(t)] = torch.tensor(t, dtype=torch.long, device=device)
    prev_pos = 0
    finished = torch.zeros(len(prompt_tokens), dtype=torch.bool, device=device)
    prompt_mask = tokens != -1
    for cur_pos in range(min(prompt_lens), total_len):
        if M.snark:
            os.makedirs(f"{M.zkDataDir}/pos_{prev_pos}", exist_ok=True)
            M.saveTensor(f"{M.zkDataDir}/pos_{prev_pos}/tokens.bin", tokens[0][prev_pos:cur_pos].cpu())
        rerun = False
        try:
            logits, layer_tokens = _forward_step(model, tokens[:, prev_pos:cur_pos], prev_pos, layer_probe)
        except M.K.ZkdsError as err:
            if err.status != M.K.ERR_RANGE:
                raise
            # an activation exceeded the limb bound promised for it (M.ACT_LIMBS, MLA.score_limbs): that
            # pass's numbers are wrong.  The step only wrote cache rows it owns, so it is simply run again
            # with every limb count measured on the device.
            with M.measured_limbs(model):
                logits, layer_tokens = _forward_step(model, tokens[:, prev_pos:cur_pos], prev_pos, layer_probe)
            rerun = True
        next_token = (sample(logits, temperature) if temperature > 0 else logits.argmax(dim=-1)).view(-1)
        next_token = torch.where(prompt_mask[:, cur_pos], tokens[:, cur_pos], next_token)
        tokens[:, cur_pos] = next_token
        finished |= torch.logical_and(~prompt_mask[:, cur_pos], next_token == eos_id)
        prev_pos = cur_pos
        if trace is not None:
            step = {"pos": cur_pos, "next_token": next_token.tolist()}
            if rerun:
                step["rerun_measured"] = True
            if layer_probe:
                step["layer_tokens"] = layer_tokens
            trace.append(step)
        if finished.all():
            break
    completion_tokens = []
    for i, toks in enumerate(tokens.tolist()):
        toks = toks[prompt_lens[i]:prompt_lens[i] + max_new_tokens]
        if eos_id in toks:
            toks = toks[:toks.index(eos_id)]
        completion_tokens.append(toks)
    return completion_tokens
