"""The reference's HuggingFace multi-LoRA path, restated for a machine without peft.

TEST INFRASTRUCTURE ONLY (see ``oracle/__init__.py``).  Also the timed CPU
baseline of the benchmark.

Follows ``huggingface/generation/gen_lora.py:21-57,114-116``: a transformers
``LlamaForCausalLM`` whose target ``nn.Linear`` modules are replaced by a LoRA
layer, driven by ``model.generate(..., adapter_names=[...], do_sample=False)``.
The third-party ``peft`` package (v0.15.1 in the reference's README) is not
installed here, so its two jobs are restated: (1) module replacement
(``get_peft_model`` / ``inject_adapter_in_model``, gen_lora.py:41-44) and
(2) handing the per-row ``adapter_names`` list to every LoRA layer (peft does
this with forward hooks; here a shared context object is used).  The layer
arithmetic is ``oracle.ops.gather_bmm_linear`` (lora_gatherbmm_linear_layer.py:
14-20).
"""
from __future__ import annotations

import torch
from torch import nn

from . import ops


class _Ctx:
    adapter_ids = None  # list[int] per batch row, or None = adapters disabled


class GatherBMMLinearCPU(nn.Module):
    """Stand-in for ``GatherBMMLinear`` with the attributes the reference
    forward reads: ``base_layer``, ``lora_A[name].weight`` [r,in],
    ``lora_B[name].weight`` [out,r], ``scaling[name]``."""

    def __init__(self, base_layer: nn.Linear, ctx: _Ctx):
        super().__init__()
        self.base_layer = base_layer
        self.lora_A = nn.ModuleDict()
        self.lora_B = nn.ModuleDict()
        self.scaling = {}
        self._ctx = ctx

    def add_adapter(self, name, A, B, scaling):
        la = nn.Linear(A.shape[1], A.shape[0], bias=False)
        lb = nn.Linear(B.shape[1], B.shape[0], bias=False)
        la.weight.data = A.to(self.base_layer.weight.dtype)
        lb.weight.data = B.to(self.base_layer.weight.dtype)
        self.lora_A[name] = la
        self.lora_B[name] = lb
        self.scaling[name] = scaling

    def forward(self, x):
        ids = self._ctx.adapter_ids
        if ids is None:
            return self.base_layer(x)
        names = [f"adapter{i}" for i in ids]
        A = {n: self.lora_A[n].weight for n in set(names)}
        B = {n: self.lora_B[n].weight for n in set(names)}
        uniq = sorted(set(names))
        idx = [uniq.index(n) for n in names]
        return ops.gather_bmm_linear(
            x, self.base_layer.weight, [A[n] for n in uniq], [B[n] for n in uniq],
            [self.scaling[n] for n in uniq], idx, self.base_layer.bias)


def build_hf_model(cfg, weights, adapters=(), scales=(), dtype=torch.float32):
    """cfg: dict with the LlamaConfig field names of
    ``tvm/llama_auto_batcher/llama_for_causal_lm.py:10-21``."""
    from transformers import LlamaConfig, LlamaForCausalLM

    hf_cfg = LlamaConfig(
        hidden_size=cfg["hidden_size"], intermediate_size=cfg["intermediate_size"],
        num_attention_heads=cfg["num_attention_heads"], num_hidden_layers=cfg["num_hidden_layers"],
        num_key_value_heads=cfg["num_key_value_heads"], rms_norm_eps=cfg["rms_norm_eps"],
        vocab_size=cfg["vocab_size"], rope_theta=cfg["rope_theta"], head_dim=cfg["head_dim"],
        max_position_embeddings=4096, tie_word_embeddings=False, attention_bias=False,
        mlp_bias=False, attn_implementation="eager", bos_token_id=None, eos_token_id=None,
        pad_token_id=None,
    )
    hf_cfg.rope_parameters = {"rope_type": "default", "rope_theta": float(cfg["rope_theta"])}
    with torch.device("meta"):
        model = LlamaForCausalLM(hf_cfg)
    model = model.to_empty(device="cpu").to(dtype)
    sd = {k: v.to(dtype) for k, v in weights.items()}
    missing, unexpected = model.load_state_dict(sd, strict=False)
    assert not [m for m in missing if "rotary" not in m and "inv_freq" not in m], missing
    assert not unexpected, unexpected
    # meta-device construction skips buffer init: rebuild the rotary table
    rot = model.model.rotary_emb
    d = cfg["head_dim"]
    inv = 1.0 / (cfg["rope_theta"] ** (torch.arange(0, d, 2, dtype=torch.float32) / d))
    rot.inv_freq = inv
    if hasattr(rot, "original_inv_freq"):
        rot.original_inv_freq = inv.clone()
    rot.attention_scaling = 1.0
    ctx = _Ctx()
    if adapters:
        for L, layer in enumerate(model.model.layers):
            for blk_name in ("self_attn", "mlp"):
                blk = getattr(layer, blk_name)
                for pname, child in list(blk.named_children()):
                    ka = f"layers.{L}.{blk_name}.{pname}.lora_A.weight"
                    if not isinstance(child, nn.Linear) or ka not in adapters[0]:
                        continue
                    wrapped = GatherBMMLinearCPU(child, ctx)
                    for i, ad in enumerate(adapters):
                        wrapped.add_adapter(f"adapter{i}", ad[ka], ad[ka.replace("lora_A", "lora_B")], scales[i])
                    setattr(blk, pname, wrapped)
    model.eval()
    model._mlora_ctx = ctx
    return model


@torch.no_grad()
def generate(model, prompts, adapter_ids, gen_len):
    """``model.generate(**tokens, adapter_names=adapters, max_new_tokens=gen_len,
    do_sample=False)`` (gen_lora.py:116).  prompts: LongTensor [B,S] of equal
    length (the reference replicates one prompt).  Returns new tokens [B,gen_len]."""
    model._mlora_ctx.adapter_ids = None if adapter_ids is None else [int(i) for i in adapter_ids]
    out = model.generate(
        input_ids=prompts, attention_mask=torch.ones_like(prompts), max_new_tokens=gen_len,
        min_new_tokens=gen_len, do_sample=False, use_cache=True, pad_token_id=0,
    )
    return out[:, prompts.shape[1]:]


@torch.no_grad()
def forward_logits(model, tokens, adapter_ids):
    """Full-sequence logits [B,S,V] (teacher-forced comparison)."""
    model._mlora_ctx.adapter_ids = None if adapter_ids is None else [int(i) for i in adapter_ids]
    return model(input_ids=tokens, use_cache=False).logits.float()


@torch.no_grad()
def time_decode_sample(cfg, weights_fn, adapters_fn, scales, adapter_ids, ctx_len, layer_counts=(1, 3),
                       steps=2, warmup=1, dtype=torch.float32):
    """Times batched single-token decode steps of the HF path on this machine's CPU cores.

    A full 7B fp32 model does not fit a per-commit benchmark, so the step is timed on
    truncated models of ``layer_counts`` layers (same per-layer shapes, KV cache pre-filled
    with ``ctx_len`` random tokens through ``DynamicCache.update``) and extrapolated linearly
    in the layer count: t(L) = t_head + L * t_layer.  ``weights_fn(n_layers)`` /
    ``adapters_fn(n_layers)`` build the truncated state dict / adapter dicts.
    Returns dict(per_layer_s, head_s, full_step_s, samples=[(L, seconds)]).
    """
    import time

    from torch import nn as _nn
    from transformers import DynamicCache

    B = len(adapter_ids)
    l_max = max(layer_counts)
    c = dict(cfg, num_hidden_layers=l_max)
    model = build_hf_model(c, weights_fn(l_max), adapters_fn(l_max), scales, dtype=dtype)
    model._mlora_ctx.adapter_ids = [int(i) for i in adapter_ids]
    all_layers = list(model.model.layers)
    g = torch.Generator().manual_seed(0)
    kv_fill = torch.randn(B, c["num_key_value_heads"], ctx_len, c["head_dim"], generator=g).to(dtype)
    samples = []
    for L in layer_counts:  # the same model truncated to its first L layers
        model.model.layers = _nn.ModuleList(all_layers[:L])
        model.config.num_hidden_layers = L
        best = None
        for it in range(warmup + steps):
            cache = DynamicCache()
            for l in range(L):  # the step's own torch.cat makes fresh per-layer buffers; the fill is shared
                cache.update(kv_fill, kv_fill, l)
            tok = torch.randint(0, c["vocab_size"], (B, 1), generator=g)
            pos = torch.full((B, 1), ctx_len, dtype=torch.long)
            t0 = time.perf_counter()
            out = model(input_ids=tok, past_key_values=cache, position_ids=pos, use_cache=True)
            out.logits[:, -1].argmax(-1)
            dt = time.perf_counter() - t0
            if it >= warmup:
                best = dt if best is None else min(best, dt)
        samples.append((L, best))
    (l0, t0), (l1, t1) = samples[0], samples[-1]
    per_layer = max((t1 - t0) / (l1 - l0), 0.0) if l1 != l0 else t0 / l0
    head = max(t0 - l0 * per_layer, 0.0)
    full = head + cfg["num_hidden_layers"] * per_layer
    return dict(per_layer_s=per_layer, head_s=head, full_step_s=full, samples=samples)
