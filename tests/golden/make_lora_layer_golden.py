"""Generates lora_layer_golden.npz by running the reference's own LoRA layer.

    python tests/golden/make_lora_layer_golden.py <path-to-reference-checkout>

``huggingface/custom_peft/lora_gatherbmm_linear_layer.py`` derives from
``peft.tuners.lora.Linear`` (third party, not installed here).  A minimal
stand-in base class that only *holds state* (base_layer, lora_A, lora_B,
scaling, lora_dropout, flags) is registered under that module name, then the
reference file is imported unmodified and its ``forward`` is executed: every
arithmetic step recorded below is the reference's own code.
"""
import os
import sys
import types

import numpy as np
import torch
from torch import nn

if len(sys.argv) != 2:
    sys.exit(f"usage: python {sys.argv[0]} <path-to-reference-checkout>")
ref = sys.argv[1]


class _StandInLinear(nn.Module):
    def __init__(self, base_layer):
        super().__init__()
        self.base_layer = base_layer
        self.lora_A = nn.ModuleDict()
        self.lora_B = nn.ModuleDict()
        self.lora_dropout = nn.ModuleDict()
        self.scaling = {}
        self.use_dora = {}
        self.disable_adapters = False
        self.merged = False
        self.active_adapters = []

    def _check_forward_args(self, x, *args, **kwargs):
        names = kwargs.get("adapter_names")
        if names is not None and len(names) != len(x):
            raise ValueError("adapter_names length must match batch")


for name in ("peft", "peft.tuners", "peft.tuners.lora"):
    sys.modules[name] = types.ModuleType(name)
sys.modules["peft.tuners.lora"].Linear = _StandInLinear
sys.path.insert(0, os.path.join(ref, "huggingface"))
from custom_peft.lora_gatherbmm_linear_layer import GatherBMMLinear  # noqa: E402


def case(seed, B, S, fin, fout, n_ad, r, alpha):
    g = torch.Generator().manual_seed(seed)
    base = nn.Linear(fin, fout, bias=False)
    base.weight.data = torch.randn(fout, fin, generator=g) * 0.05
    layer = GatherBMMLinear(base)
    for i in range(n_ad):
        n = f"adapter{i}"
        la, lb = nn.Linear(fin, r, bias=False), nn.Linear(r, fout, bias=False)
        la.weight.data = (torch.rand(r, fin, generator=g) * 2 - 1) / fin ** 0.5
        lb.weight.data = torch.randn(fout, r, generator=g) * 0.05
        layer.lora_A[n], layer.lora_B[n] = la, lb
        layer.lora_dropout[n] = nn.Identity()
        layer.scaling[n] = alpha / r
        layer.use_dora[n] = False
    layer.eval()
    x = torch.randn(B, S, fin, generator=g)
    ids = torch.randint(0, n_ad, (B,), generator=g)
    with torch.no_grad():
        y = layer(x, adapter_names=[f"adapter{int(i)}" for i in ids])
        layer.disable_adapters = True
        y_base = layer(x)
    return dict(
        x=x.numpy(), W=base.weight.data.numpy(), ids=ids.numpy().astype(np.int32),
        A=np.stack([layer.lora_A[f"adapter{i}"].weight.data.numpy() for i in range(n_ad)]),
        B=np.stack([layer.lora_B[f"adapter{i}"].weight.data.numpy() for i in range(n_ad)]),
        scale=np.float32(alpha / r), y=y.numpy(), y_base=y_base.numpy())


def main():
    out = {}
    specs = [(0, 4, 1, 64, 48, 4, 8, 16), (1, 5, 3, 32, 80, 3, 4, 8), (2, 1, 1, 256, 256, 1, 16, 32),
             (3, 9, 2, 128, 64, 16, 16, 32), (4, 32, 1, 256, 256, 16, 16, 32)]
    for i, s in enumerate(specs):
        for k, v in case(*s).items():
            out[f"c{i}_{k}"] = v
    out["n_cases"] = np.int32(len(specs))
    dst = os.path.join(os.path.dirname(os.path.abspath(__file__)), "lora_layer_golden.npz")
    np.savez_compressed(dst, **out)
    print("wrote", dst, os.path.getsize(dst), "bytes")


if __name__ == "__main__":
    main()
