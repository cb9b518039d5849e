"""Seeded synthetic models, adapters and request batches.

The reference runs pretrained Llama weights, adapter files written by
``init_peft_weights/lora_weights.py`` and one English prompt replicated over
the batch (``huggingface/generation/gen_lora.py:96-98``); none of those are
available offline, so every workload here is random data with the same
shapes, drawn from fixed seeds: tokens 0, base weights 1, adapters 2,
adapter ids 3, prompt lengths 4.
"""
from __future__ import annotations

import math

import numpy as np
import torch

SEED_TOKENS, SEED_WEIGHTS, SEED_ADAPTERS, SEED_IDS, SEED_LENS = 0, 1, 2, 3, 4

ATTN_PROJ = ("q_proj", "k_proj", "v_proj", "o_proj")
MLP_PROJ = ("gate_proj", "up_proj", "down_proj")


def llama_config(name: str) -> dict:
    """Field names of ``tvm/llama_auto_batcher/llama_for_causal_lm.py:10-21``."""
    base = dict(rms_norm_eps=1e-5, vocab_size=32000, rope_theta=10000.0)
    if name == "tiny":  # the CPU-runnable plumbing case
        return dict(base, name=name, hidden_size=256, intermediate_size=688, num_attention_heads=4,
                    num_hidden_layers=2, num_key_value_heads=4, head_dim=64)
    if name == "llama2-7b":
        return dict(base, name=name, hidden_size=4096, intermediate_size=11008, num_attention_heads=32,
                    num_hidden_layers=32, num_key_value_heads=32, head_dim=128)
    if name == "llama2-13b":
        return dict(base, name=name, hidden_size=5120, intermediate_size=13824, num_attention_heads=40,
                    num_hidden_layers=40, num_key_value_heads=40, head_dim=128)
    raise KeyError(name)


def proj_shape(cfg: dict, proj: str):
    """(out_features, in_features) of a projection."""
    H, I = cfg["hidden_size"], cfg["intermediate_size"]
    D, Hq, Hkv = cfg["head_dim"], cfg["num_attention_heads"], cfg["num_key_value_heads"]
    return {
        "q_proj": (Hq * D, H), "k_proj": (Hkv * D, H), "v_proj": (Hkv * D, H), "o_proj": (H, Hq * D),
        "gate_proj": (I, H), "up_proj": (I, H), "down_proj": (H, I),
    }[proj]


def _gen(seed, device):
    g = torch.Generator(device=device)
    g.manual_seed(seed)
    return g


def base_weights(cfg: dict, dtype=torch.float32, device="cpu", n_layers=None) -> dict:
    """HF-named state dict, every matrix ~ N(0, 0.02), norm weights 1 + N(0, 0.02)."""
    g = _gen(SEED_WEIGHTS, device)
    H, V = cfg["hidden_size"], cfg["vocab_size"]
    L = cfg["num_hidden_layers"] if n_layers is None else n_layers

    def mat(o, i):
        return (torch.randn(o, i, generator=g, device=device, dtype=torch.float32) * 0.02).to(dtype)

    def vec(n):
        return (1.0 + 0.02 * torch.randn(n, generator=g, device=device, dtype=torch.float32)).to(dtype)

    w = {"model.embed_tokens.weight": mat(V, H)}
    for l in range(L):
        p = f"model.layers.{l}."
        for proj in ATTN_PROJ:
            w[p + f"self_attn.{proj}.weight"] = mat(*proj_shape(cfg, proj))
        for proj in MLP_PROJ:
            w[p + f"mlp.{proj}.weight"] = mat(*proj_shape(cfg, proj))
        w[p + "input_layernorm.weight"] = vec(H)
        w[p + "post_attention_layernorm.weight"] = vec(H)
    w["model.norm.weight"] = vec(H)
    w["lm_head.weight"] = mat(V, H)
    return w


def lora_adapters(cfg: dict, n_adapters: int, ranks, targets=ATTN_PROJ, dtype=torch.float32,
                  device="cpu", n_layers=None):
    """Adapter dicts keyed like the reference's adapter files
    (``init_peft_weights/lora_weights.py:18-23``): ``lora_A`` [r,in] ~ kaiming
    uniform(a=sqrt 5) = U(+-1/sqrt(in)), ``lora_B`` [out,r] ~ N(0, 0.02).
    ``ranks`` is an int or a sequence cycled over the adapters."""
    g = _gen(SEED_ADAPTERS, device)
    L = cfg["num_hidden_layers"] if n_layers is None else n_layers
    ranks = [ranks] if isinstance(ranks, int) else list(ranks)
    out = []
    for a in range(n_adapters):
        r = ranks[a % len(ranks)]
        d = {}
        for l in range(L):
            for proj in targets:
                blk = "self_attn" if proj in ATTN_PROJ else "mlp"
                o, i = proj_shape(cfg, proj)
                bound = 1.0 / math.sqrt(i)
                A = (torch.rand(r, i, generator=g, device=device, dtype=torch.float32) * 2 - 1) * bound
                B = torch.randn(o, r, generator=g, device=device, dtype=torch.float32) * 0.02
                d[f"layers.{l}.{blk}.{proj}.lora_A.weight"] = A.to(dtype)
                d[f"layers.{l}.{blk}.{proj}.lora_B.weight"] = B.to(dtype)
        out.append(d)
    return out


def adapter_ids_uniform(n_requests: int, n_adapters: int) -> np.ndarray:
    return np.random.default_rng(SEED_IDS).integers(0, n_adapters, n_requests).astype(np.int32)


def adapter_ids_zipf(n_requests: int, n_adapters: int, s: float = 1.1) -> np.ndarray:
    p = np.arange(1, n_adapters + 1, dtype=np.float64) ** (-s)
    p /= p.sum()
    return np.random.default_rng(SEED_IDS).choice(n_adapters, size=n_requests, p=p).astype(np.int32)


def request_mix(request_type: str, batch_size: int, seed: int = SEED_IDS) -> np.ndarray:
    """The reference's three request mixes (``huggingface/generation/gen_lora.py:77-85``): ``uniform`` = sorted
    draws from ``[0, ceil(sqrt(B)))`` (same-adapter rows contiguous), ``distinct`` = every request its own adapter,
    ``identical`` = one adapter for all.  Seeded (the reference draws from numpy's global generator)."""
    if request_type == "uniform":
        hi = int(np.ceil(np.sqrt(batch_size)))
        return np.sort(np.random.default_rng(seed).integers(0, hi, batch_size)).astype(np.int32)
    if request_type == "distinct":
        return np.arange(batch_size, dtype=np.int32)
    if request_type == "identical":
        return np.zeros(batch_size, dtype=np.int32)
    raise ValueError(f"unknown request_type {request_type}")


def request_mix_by_rank(request_type: str, batch_size: int, num_seqs_per_adapter, lora_ranks, seed: int = SEED_IDS):
    """The auto-batcher driver's batch (``tvm/llama_auto_batcher/main.py:24-35``): one group of requests per adapter
    rank, weight ids inside a group drawn per ``request_type``, and ``batch_size - sum(groups)`` requests WITHOUT
    adapter padded in front.  Returns ``(ranks, wids)``, each ``[batch_size]`` with -1 for the padding rows."""
    if sum(num_seqs_per_adapter) > batch_size:
        raise ValueError("more adapter requests than the batch holds")
    ranks = [r for n, r in zip(num_seqs_per_adapter, lora_ranks) for _ in range(n)]
    if request_type == "identical":
        wids = [0] * sum(num_seqs_per_adapter)
    else:
        wids = [int(w) for g, n in enumerate(num_seqs_per_adapter) for w in request_mix(request_type, n, seed + g)]
    pad = [-1] * (batch_size - sum(num_seqs_per_adapter))
    return np.asarray(pad + ranks, dtype=np.int32), np.asarray(pad + wids, dtype=np.int32)


def prompts(n_requests: int, length: int, vocab: int) -> np.ndarray:
    return np.random.default_rng(SEED_TOKENS).integers(0, vocab, (n_requests, length)).astype(np.int32)


def prompt_lengths(n_requests: int, lo: int, hi: int) -> np.ndarray:
    return np.random.default_rng(SEED_LENS).integers(lo, hi + 1, n_requests).astype(np.int32)


def operator_case(T: int, in_features=4096, out_features=4096, n_adapters=16, rank=16,
                  dtype=torch.bfloat16, device="cpu"):
    """The operator micro-benchmark: x ~ N(0,1), W ~ N(0,0.02), A ~ U(+-1/64),
    B ~ N(0,0.02), per-token ids uniform in [0, n_adapters), scale 2.0
    (shapes of ``tvm/lora_only/single_rank.py:66-103,142-155``).
    A is stored [N, r, in] and B [N, out, r] (peft's per-adapter layout)."""
    g = _gen(SEED_WEIGHTS, device)
    x = torch.randn(T, in_features, generator=g, device=device, dtype=torch.float32).to(dtype)
    W = (torch.randn(out_features, in_features, generator=g, device=device, dtype=torch.float32) * 0.02).to(dtype)
    A = ((torch.rand(n_adapters, rank, in_features, generator=g, device=device, dtype=torch.float32) * 2 - 1)
         / 64.0).to(dtype)
    B = (torch.randn(n_adapters, out_features, rank, generator=g, device=device, dtype=torch.float32) * 0.02).to(dtype)
    ids = torch.from_numpy(adapter_ids_uniform(T, n_adapters)).to(device)
    return dict(x=x, W=W, A=A, B=B, ids=ids, scale=2.0)
