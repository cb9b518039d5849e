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
        self._ctx = None     # shared AdapterContext (set by MultiLoraModel): per-call adapter names + slot-tensor cache
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
    def _slot_tensor(self, slots_per_batch_row, per_row, device):
        """int32 [rows] on the device: built once per (adapter list, tokens per row) and shared by every layer of
        the model through the context -- one small host-to-device copy per generate step, not one per layer."""
        key = (tuple(slots_per_batch_row), per_row, str(device))
        cache = self._ctx.slot_cache if self._ctx is not None else None
        if cache is not None and key in cache:
            return cache[key]
        t = torch.tensor(slots_per_batch_row, dtype=torch.int32).repeat_interleave(per_row).pin_memory() \
            .to(device, non_blocking=True)
        if cache is not None:
            if len(cache) > 64:
                cache.clear()
            cache[key] = t
        return t

    def _run(self, x, slots_per_batch_row):
        """x [B,S,in] (or [T,in]); one slot per leading row, shared by that row's S tokens."""
        _, stack, _, Wp = self._pack()
        lead = x.shape[:-1]
        x2 = x.reshape(-1, self.in_features)
        if x2.dtype != torch.bfloat16 or not x2.is_contiguous():
            x2 = x2.to(torch.bfloat16).contiguous()
        slots = None
        if slots_per_batch_row is not None and stack is not None:
            slots = self._slot_tensor(slots_per_batch_row, x2.shape[0] // len(slots_per_batch_row), x2.device)
        y = ops.linear(x2, Wp, stack if slots is not None else None, slots)
        if self.base_layer.bias is not None:
            y = y + self.base_layer.bias.to(y.dtype)
        y = y.reshape(*lead, self.out_features)
        return y if y.dtype == x.dtype else y.to(x.dtype)

    def forward(self, x: torch.Tensor, *args: Any, **kwargs: Any) -> torch.Tensor:
        self._check_forward_args(x, *args, **kwargs)
        adapter_names = kwargs.pop("adapter_names", None)
        if adapter_names is None and self._ctx is not None:
            adapter_names = self._ctx.adapter_names  # handed over by MultiLoraModel (peft does this with forward hooks)
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


class AdapterContext:
    """What peft passes to every LoRA layer of a model during one ``generate`` / ``forward`` call: the per-row
    adapter names (``adapter_names=`` of ``model.generate``, ``gen_lora.py:116``).  Also holds the device slot
    tensors built from them, shared by all layers."""

    def __init__(self):
        self.adapter_names = None
        self.slot_cache = {}


class MultiLoraModel:
    """A HuggingFace causal LM whose target ``nn.Linear`` modules are :class:`MultiLoraLinear` layers, with the
    adapters of ``get_hf_model`` (``huggingface/generation/gen_lora.py:21-57``) injected and loaded, driven like
    the reference drives its peft model: ``model.generate(**tokens, adapter_names=[...], max_new_tokens=n,
    do_sample=False)`` (``gen_lora.py:116``)."""

    def __init__(self, model, layers):
        self.model, self.layers, self.ctx = model, layers, AdapterContext()
        for layer in layers:
            layer._ctx = self.ctx

    def _call(self, fn, adapter_names, *args, **kwargs):
        if adapter_names is not None:
            adapter_names = list(adapter_names)
        self.ctx.adapter_names = adapter_names
        try:
            with torch.no_grad():
                return fn(*args, **kwargs)
        finally:
            self.ctx.adapter_names = None

    def generate(self, *args, adapter_names=None, **kwargs):
        return self._call(self.model.generate, adapter_names, *args, **kwargs)

    def __call__(self, *args, adapter_names=None, **kwargs):
        return self._call(self.model, adapter_names, *args, **kwargs)

    def disable_adapter(self):
        """Context manager: the base model alone (peft's ``with model.disable_adapter():``)."""
        import contextlib

        @contextlib.contextmanager
        def ctx():
            old = [layer.disable_adapters for layer in self.layers]
            for layer in self.layers:
                layer.disable_adapters = True
            try:
                yield self
            finally:
                for layer, o in zip(self.layers, old):
                    layer.disable_adapters = o
        return ctx()

    # hot add / remove of one adapter (files in the format of adapters.py)
    def add_adapter(self, name, tensors, r, lora_alpha):
        for layer in self.layers:
            layer.update_layer(name, r, lora_alpha)
        _load_into(self.model, name, tensors)
        self.ctx.slot_cache.clear()

    def remove_adapter(self, name):
        for layer in self.layers:
            if name in layer.lora_A:
                del layer.lora_A[name], layer.lora_B[name], layer.lora_dropout[name]
                layer.scaling.pop(name), layer.r.pop(name), layer.use_dora.pop(name)
                if name in layer.active_adapters:
                    layer.active_adapters.remove(name)
                layer.invalidate()
        self.ctx.slot_cache.clear()


def _load_into(model, adapter, tensors):
    """The reference's key map (``gen_lora.py:50``): file key ``layers.{L}.self_attn.q_proj.lora_A.weight`` is peft's
    parameter ``base_model.model.model.layers.{L}.self_attn.q_proj.lora_A.{adapter}.weight``; here the same path
    under the unwrapped HF model: ``model.layers.{L}.self_attn.q_proj`` -> ``lora_A[adapter].weight``."""
    root = model.get_submodule("model") if hasattr(model, "model") else model
    loaded = 0
    for k, v in tensors.items():
        if not k.endswith(".weight"):
            continue
        path, which = k[: -len(".weight")].rsplit(".", 1)  # "layers.3.self_attn.q_proj", "lora_A"
        try:
            mod = root.get_submodule(path)
        except AttributeError:
            continue
        if not isinstance(mod, MultiLoraLinear) or adapter not in getattr(mod, which):
            continue
        p = getattr(mod, which)[adapter].weight
        if tuple(p.shape) != tuple(v.shape):
            raise ValueError(f"{k}: file holds {tuple(v.shape)}, the layer expects {tuple(p.shape)}")
        p.data = v.to(dtype=p.dtype, device=p.device)
        mod.invalidate()
        loaded += 1
    if loaded == 0:
        raise ValueError(f"no tensor of adapter '{adapter}' matched a wrapped layer")
    return loaded


def get_hf_model(base_model, adapter_dir, unique_adapters, r=64, lora_alpha=32, target_modules=("q_proj", "v_proj")):
    """``get_hf_model`` of ``huggingface/generation/gen_lora.py:21-57`` on a model the caller has built: wraps the
    target projections (``:30-44``), injects every adapter of ``unique_adapters`` (names ``adapter{i}``), loads
    ``{adapter_dir}/r{r}_a{i}.safetensors`` into them (``:46-53``) and returns a :class:`MultiLoraModel`."""
    from . import adapters as adapter_io

    layers = wrap_model(base_model, target_modules)
    names = sorted(unique_adapters)
    for name in names:
        for layer in layers:
            layer.update_layer(name, r, lora_alpha)
    for name in names:
        path = adapter_io.adapter_path(adapter_dir, r, int(name.replace("adapter", "")))
        _load_into(base_model, name, adapter_io.load_adapter(path))
    base_model.eval()
    return MultiLoraModel(base_model, layers)
