"""``MultiLoraLinear``: the B200 stand-in for the reference's ``GatherBMMLinear``.

Same ``forward(x, *args, adapter_names=[...], **kwargs)`` signature and the
same state a peft ``LoraLayer`` exposes to that forward
(``huggingface/custom_peft/lora_gatherbmm_linear_layer.py:5-54``): ``base_layer``,
``lora_A[name].weight`` [r,in], ``lora_B[name].weight`` [out,r], ``scaling[name]``,
``lora_dropout[name]``, ``disable_adapters``, ``merged``, ``active_adapters``,
``_check_forward_args``.  It can be registered with peft exactly like the
reference class (``lora_config._register_custom_module({nn.Linear: MultiLoraLinear})``,
``huggingface/generation/gen_lora.py:37-39``) when peft is installed, and works
stand-alone when it is not.

Where the reference re-gathers every row's A and B with two ``torch.stack``
calls and runs two ``torch.bmm`` per call, this layer keeps packed device
stacks and makes two library calls: the LoRA shrink and the base projection
with the expand fused into its output write.  Arithmetic is bf16 with fp32
accumulation; inputs of another dtype are converted and the result cast back.
"""
from __future__ import annotations

from typing import Any

import torch
from torch import nn

from . import ops


class MultiLoraLinear(nn.Module):
    def __init__(self, base_layer: nn.Linear, adapter_name: str = None, r: int = 0, lora_alpha: float = 1.0,
                 **kwargs):
        super().__init__()
        self.base_layer = base_layer
        self.in_features, self.out_features = base_layer.in_features, base_layer.out_features
        self.lora_A = nn.ModuleDict()
        self.lora_B = nn.ModuleDict()
        self.lora_dropout = nn.ModuleDict()
        self.scaling = {}
        self.r = {}
        self.use_dora = {}
        self.disable_adapters = False
        self.merged = False
        self.active_adapters = []
        self._packed = None  # (key, LoraStack, name -> slot, packed base weight)
        if adapter_name is not None and r > 0:
            self.update_layer(adapter_name, r, lora_alpha)

    # -- peft-compatible state management ---------------------------------------------------------------
    def update_layer(self, adapter_name, r, lora_alpha, lora_dropout=0.0, **kwargs):
        """Adds an (initialised-to-zero-B) adapter, like ``LoraLayer.update_layer``."""
        dev, dt = self.base_layer.weight.device, self.base_layer.weight.dtype
        self.lora_A[adapter_name] = nn.Linear(self.in_features, r, bias=False, device=dev, dtype=dt)
        self.lora_B[adapter_name] = nn.Linear(r, self.out_features, bias=False, device=dev, dtype=dt)
        nn.init.zeros_(self.lora_B[adapter_name].weight)
        self.lora_dropout[adapter_name] = nn.Dropout(lora_dropout) if lora_dropout > 0 else nn.Identity()
        self.scaling[adapter_name] = lora_alpha / r
        self.r[adapter_name] = r
        self.use_dora[adapter_name] = False
        if adapter_name not in self.active_adapters:
            self.active_adapters.append(adapter_name)
        self._packed = None

    def set_adapter_weights(self, adapter_name, A, B):
        """A [r,in], B [out,r] (the on-disk layout of ``init_peft_weights/lora_weights.py:16-23``)."""
        self.lora_A[adapter_name].weight.data = A.to(self.lora_A[adapter_name].weight)
        self.lora_B[adapter_name].weight.data = B.to(self.lora_B[adapter_name].weight)
        self._packed = None

    def invalidate(self):
        """Call after changing adapter or base weights in place."""
        self._packed = None

    def _check_forward_args(self, x, *args, **kwargs):
        names = kwargs.get("adapter_names")
        if names is None:
            return
        if len(x) != len(names):
            raise ValueError(f"Length of `adapter_names` should be the same as the number of inputs, but got "
                             f"{len(names)} and {len(x)} respectively.")
        if self.merged:
            raise ValueError("Cannot pass `adapter_names` when there are merged adapters, please call "
                             "`unmerge_adapter` first.")

    def unmerge(self):
        self.merged = False

    # -- packing ------------------------------------------------------------------------------------------
    def _pack(self):
        names = sorted(self.lora_A.keys())
        key = tuple((n, self.lora_A[n].weight.data_ptr(), self.lora_B[n].weight.data_ptr(), self.scaling[n])
                    for n in names) + (self.base_layer.weight.data_ptr(),)
        if self._packed is not None and self._packed[0] == key:
            return self._packed
        dev = self.base_layer.weight.device
        W = self.base_layer.weight.detach().to(torch.bfloat16).contiguous()
        Wp = ops.PackedWeight(W)
        stack, slot_of = None, {}
        if names:
            r_hi = max(self.r[n] for n in names)
            r_max = 16 if r_hi <= 16 else 32 if r_hi <= 32 else -(-r_hi // 64) * 64
            A_all = torch.zeros(len(names), r_max, self.in_features, dtype=torch.bfloat16, device=dev)
            B_all = torch.zeros(len(names), self.out_features, r_max, dtype=torch.bfloat16, device=dev)
            for s, n in enumerate(names):
                r = self.r[n]
                A_all[s, :r] = self.lora_A[n].weight.detach().to(torch.bfloat16)
                B_all[s, :, :r] = self.lora_B[n].weight.detach().to(torch.bfloat16)
                slot_of[n] = s
            stack = ops.LoraStack(A_all, B_all, torch.tensor([self.r[n] for n in names], dtype=torch.int32, device=dev),
                                  torch.tensor([self.scaling[n] for n in names], dtype=torch.float32, device=dev),
                                  r_max, 1, (0, self.out_features))
            if r_max <= 128:
                stack.pack_b()
        self._packed = (key, stack, slot_of, Wp)
        return self._packed

    # -- forward ---------------------------------------------------------------------------------------------
    def _run(self, x, slots_per_batch_row):
        """x [B,S,in] (or [T,in]); one slot per leading row, shared by that row's S tokens."""
        _, stack, _, Wp = self._pack()
        lead = x.shape[:-1]
        x2 = x.reshape(-1, self.in_features).to(torch.bfloat16).contiguous()
        slots = None
        if slots_per_batch_row is not None and stack is not None:
            per_row = x2.shape[0] // len(slots_per_batch_row)
            slots = torch.tensor(slots_per_batch_row, dtype=torch.int32).repeat_interleave(per_row).to(x2.device)
        y = ops.linear(x2, Wp, stack if slots is not None else None, slots)
        if self.base_layer.bias is not None:
            y = y + self.base_layer.bias.to(y.dtype)
        return y.reshape(*lead, self.out_features).to(x.dtype)

    def forward(self, x: torch.Tensor, *args: Any, **kwargs: Any) -> torch.Tensor:
        self._check_forward_args(x, *args, **kwargs)
        adapter_names = kwargs.pop("adapter_names", None)
        if not x.is_cuda:
            raise RuntimeError("MultiLoraLinear runs on a CUDA device only (there is no CPU path)")
        if self.disable_adapters:
            if self.merged:
                self.unmerge()
            return self._run(x, None)
        if adapter_names is not None:
            _, _, slot_of, _ = self._pack()
            # "__base__" is peft's name for "no adapter on this row"
            return self._run(x, [slot_of.get(n, -1) for n in adapter_names])
        if self.merged:
            return self._run(x, None)
        active = [n for n in self.active_adapters if n in self.lora_A]
        if any(self.use_dora.get(n) for n in active):
            raise NotImplementedError("DoRA adapters are not supported")
        if not active:
            return self._run(x, None)
        if len(active) == 1:
            _, _, slot_of, _ = self._pack()
            n_rows = x.shape[0] if x.dim() > 1 else 1
            return self._run(x, [slot_of[active[0]]] * n_rows)
        # several active adapters apply to every row: their deltas add, one pass per adapter
        _, stack, slot_of, Wp = self._pack()
        x2 = x.reshape(-1, self.in_features).to(torch.bfloat16).contiguous()
        y = None
        for i, n in enumerate(active):
            slots = torch.full((x2.shape[0],), slot_of[n], dtype=torch.int32, device=x2.device)
            yi = ops.linear(x2, Wp, stack, slots).float()
            y = yi if y is None else y + (yi - base)
            if i == 0:
                base = ops.linear(x2, Wp).float()
        y = y.to(torch.bfloat16)
        if self.base_layer.bias is not None:
            y = y + self.base_layer.bias.to(y.dtype)
        return y.reshape(*x.shape[:-1], self.out_features).to(x.dtype)


def wrap_model(model: nn.Module, target_modules=("q_proj", "v_proj")):
    """Replaces every ``nn.Linear`` whose attribute name is in ``target_modules`` by a
    :class:`MultiLoraLinear` (what ``get_peft_model`` + ``inject_adapter_in_model`` do in
    ``huggingface/generation/gen_lora.py:41-44``).  Returns the list of wrapped layers."""
    wrapped = []
    for parent in list(model.modules()):
        for name, child in list(parent.named_children()):
            if name in target_modules and isinstance(child, nn.Linear):
                layer = MultiLoraLinear(child)
                setattr(parent, name, layer)
                wrapped.append(layer)
    return wrapped
