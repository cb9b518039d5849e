"""LoRA adapter files in the reference's on-disk format.

One safetensors file per adapter, named ``r{rank}_a{id}.safetensors``
(``init_peft_weights/lora_weights.py:24``; read at ``huggingface/generation/gen_lora.py:48`` and
``tvm/llama_auto_batcher/compile_tvm.py:302``), holding for every layer ``L`` and target projection
``P`` the fp32 tensors

    layers.{L}.self_attn.{P}.lora_A.weight   [rank, in_features]
    layers.{L}.self_attn.{P}.lora_B.weight   [out_features, rank]

(the reference writes q_proj and v_proj only, ``lora_weights.py:16-23``; k/o and
``layers.{L}.mlp.{gate,up,down}_proj`` use the same key pattern here).  ``PackedLlama`` consumes the
dict ``load_adapter`` returns.
"""
from __future__ import annotations

import os

import torch

from . import synth


def adapter_path(directory: str, rank: int, adapter_id: int) -> str:
    return os.path.join(directory, f"r{rank}_a{adapter_id}.safetensors")


def load_adapter(path: str) -> dict:
    from safetensors.torch import load_file
    return load_file(path)


def save_adapter(path: str, tensors: dict) -> None:
    from safetensors.torch import save_file
    os.makedirs(os.path.dirname(path) or ".", exist_ok=True)
    save_file({k: v.detach().to(torch.float32).contiguous().cpu() for k, v in tensors.items()}, path)


def write_adapter_files(directory: str, cfg: dict, ranks, n_adapters: int, targets=("q_proj", "v_proj"),
                        scaling_factor: float = 0.01, seed: int = synth.SEED_ADAPTERS) -> list:
    """Seeded equivalent of ``init_peft_weights/lora_weights.py:11-25``: ``n_adapters`` files for every
    rank in ``ranks``, entries ``scaling_factor * randn``.  Returns the paths written."""
    g = torch.Generator().manual_seed(seed)
    paths = []
    for rank in ranks:
        for a in range(n_adapters):
            t = {}
            for l in range(cfg["num_hidden_layers"]):
                for proj in targets:
                    blk = "self_attn" if proj in synth.ATTN_PROJ else "mlp"
                    out_f, in_f = synth.proj_shape(cfg, proj)
                    t[f"layers.{l}.{blk}.{proj}.lora_A.weight"] = scaling_factor * torch.randn(rank, in_f, generator=g)
                    t[f"layers.{l}.{blk}.{proj}.lora_B.weight"] = scaling_factor * torch.randn(out_f, rank, generator=g)
            path = adapter_path(directory, rank, a)
            save_adapter(path, t)
            paths.append(path)
    return paths
