"""``B200VM``: the function table the reference's executor drives, backed by libmlora.

The reference compiles its model to a TVM Relax VM and calls it by name
(``tvm/llama_auto_batcher/llama_exec_graph.py:41,67,81-84,112,126``); the module
spec is written at ``tvm/llama_auto_batcher/compile_tvm.py:211-285``:

    embed(input_ids int32 [B,S], params) -> hidden [B,S,H]
    create_paged_kv_cache(ShapeTuple[max_batch], ShapeTuple[max_total_seq_len],
                          ShapeTuple[prefill_chunk], ShapeTuple[page_size]) -> cache
    prefill_no_adapter(hidden [1,S,H], cache, params)
    prefill_a{t}(hidden, cache, wids int32 [1], params)
    decode_no_adapter(hidden [B,1,H], cache, params)
    decode_a{t}(hidden, cache, wids int32 [B], params)
    mixed_decode_a{t0}_a{t1}...(hidden, cache, a{t0}_sids, a{t0}_wids, a{t1}_sids, a{t1}_wids, ..., params)

all returning ``(logits fp32 [B,1,V], cache)``, plus the runtime's global functions
``vm.builtin.kv_state_add_sequence / kv_state_begin_forward / kv_state_end_forward``.
This class offers exactly those names and argument orders.  TVM is not needed:
arrays are accepted as numpy arrays, torch tensors or :class:`NDArray`, and
results come back as :class:`NDArray` (``.numpy()`` like ``tvm.nd.NDArray``).

Underneath there is ONE decode entry (per-row adapter slots); the named
variants only translate their (type, sids, wids) arguments into that slot
vector, so no function per subset of adapter types has to exist
(the reference synthesises 2^types - 1 of them, ``compile_tvm.py:196-208``).
"""
from __future__ import annotations

import re

import numpy as np
import torch

from . import kv_cache as kvc
from . import ops
from .model import Engine, PackedLlama


class ShapeTuple(tuple):
    """Stand-in for ``tvm.runtime.ShapeTuple``."""

    def __new__(cls, values):
        return super().__new__(cls, [int(v) for v in values])


class NDArray:
    """Device array with the two members the reference's executor uses: ``.numpy()`` and ``.shape``."""

    def __init__(self, tensor: torch.Tensor):
        self.tensor = tensor

    @property
    def shape(self):
        return tuple(self.tensor.shape)

    def numpy(self):
        t = self.tensor
        return (t.float() if t.dtype == torch.bfloat16 else t).cpu().numpy()


def array(values, device="cuda", dtype=None):
    """Stand-in for ``tvm.nd.array(np_array, device)``."""
    t = torch.as_tensor(np.asarray(values))
    if dtype is not None:
        t = t.to(dtype)
    return NDArray(t.to(device))


def _tensor(x, device, dtype=None):
    if isinstance(x, NDArray):
        t = x.tensor
    elif isinstance(x, torch.Tensor):
        t = x
    else:
        t = torch.as_tensor(np.asarray(x))
    t = t.to(device)
    return t if dtype is None else t.to(dtype)


class B200VM:
    def __init__(self, model: PackedLlama, type_slot_base=(0,)):
        """``type_slot_base[t]`` = first slot of adapter type ``t`` in the model's packed stacks; the slot of
        (type t, weight id w) is ``type_slot_base[t] + w`` (the reference uses the raw weight id as the index
        into that type's stack, ``compile_tvm.py:298-313``)."""
        self.model = model
        self.type_slot_base = list(type_slot_base)
        self.params = object()  # opaque token handed back as the trailing "params" argument
        self._engines = {}

    # ---- table lookup ---------------------------------------------------------------------------------------
    def __getitem__(self, name):
        if name == "embed":
            return self._embed
        if name == "create_paged_kv_cache":
            return self._create_paged_kv_cache
        if name == "prefill_no_adapter":
            return lambda h, kv, params=None: self._run(h, kv, None, prefill=True)
        if name == "decode_no_adapter":
            return lambda h, kv, params=None: self._run(h, kv, None, prefill=False)
        m = re.fullmatch(r"(prefill|decode)_a(\d+)", name)
        if m:
            t, pre = int(m.group(2)), m.group(1) == "prefill"
            self._check_type(t)
            return lambda h, kv, wids, params=None: self._run(h, kv, [(t, None, wids)], prefill=pre)
        m = re.fullmatch(r"mixed_decode((?:_a\d+)+)", name)
        if m:
            types = [int(v) for v in re.findall(r"_a(\d+)", m.group(1))]
            for t in types:
                self._check_type(t)

            def mixed(h, kv, *args):
                ids = args[: 2 * len(types)]
                if len(ids) != 2 * len(types):
                    raise TypeError(f"{name} expects {2 * len(types)} index arrays")
                return self._run(h, kv, [(t, ids[2 * i], ids[2 * i + 1]) for i, t in enumerate(types)], prefill=False)
            return mixed
        raise KeyError(name)

    # ---- what the device-resident decode loop needs from the table ---------------------------------------
    def engine_for(self, kv):
        """The engine created with this cache by ``create_paged_kv_cache``."""
        return self._engines[id(kv)]

    def slot_of(self, adapter_info):
        """Packed-stack slot of ``{"tid", "wid"}`` (None -> -1, no adapter)."""
        if adapter_info is None:
            return -1
        self._check_type(adapter_info["tid"])
        return self.type_slot_base[adapter_info["tid"]] + int(adapter_info["wid"])

    def _check_type(self, t):
        if t >= len(self.type_slot_base):
            raise KeyError(f"adapter type {t} is not loaded")

    # ---- functions -------------------------------------------------------------------------------------------
    def _embed(self, input_ids, params=None):
        ids = _tensor(input_ids, self.model.device, torch.int32)
        B, S = ids.shape
        out = torch.empty(B * S, self.model.H, dtype=torch.bfloat16, device=self.model.device)
        ops.embed(ids.reshape(-1).contiguous(), self.model.embed, out_bf16=out)
        return NDArray(out.view(B, S, self.model.H))

    def _create_paged_kv_cache(self, max_batch, max_total_seq_len, prefill_chunk, page_size):
        m = self.model
        kv = kvc.PagedKVCache(m.L, m.Hkv, m.D, int(max_batch[0]), int(max_total_seq_len[0]), int(prefill_chunk[0]),
                              int(page_size[0]), m.device)
        self._engines[id(kv)] = Engine(m, kv, max(int(prefill_chunk[0]), int(max_batch[0])))
        return kv

    def _run(self, hidden, kv, type_args, prefill):
        eng = self._engines[id(kv)]
        m = self.model
        h = _tensor(hidden, m.device, torch.bfloat16)
        B, S, _ = h.shape
        T = B * S
        if getattr(kv, "_rows", None) is None:
            raise RuntimeError("kv_state_begin_forward must be called before the model function")
        row_slot, row_pos = kv._rows
        if row_slot.numel() != T:
            raise ValueError(f"begin_forward announced {row_slot.numel()} rows, hidden has {T}")
        eng.row_slot[:T].copy_(row_slot)
        eng.row_pos[:T].copy_(row_pos)
        # (type, sids, wids) -> one adapter slot per batch row; rows not listed have no adapter.  This is
        # what take(hidden, sids) + write_tensor_part(delta, sids) amount to (compile_tvm.py:135-155).
        use_lora = type_args is not None and m.n_adapters > 0
        if use_lora:
            slots = torch.full((B,), -1, dtype=torch.int32, device=m.device)
            for t, sids, wids in type_args:
                w = _tensor(wids, m.device, torch.int32).reshape(-1) + self.type_slot_base[t]
                if sids is None:
                    if w.numel() != B:
                        raise ValueError(f"wids has {w.numel()} entries for a batch of {B}")
                    slots = w
                else:
                    slots[_tensor(sids, m.device, torch.int64).reshape(-1)] = w
            eng.slots[:T].copy_(slots.repeat_interleave(S) if S > 1 else slots)
            eng.n_distinct = int(torch.unique(slots[slots >= 0]).numel())
        h2 = h.reshape(T, m.H).contiguous()
        if prefill:
            # the reference keeps only the last token before lm_head (llama_for_causal_lm.py:130-137)
            last = (torch.arange(B, device=m.device, dtype=torch.int32) + 1) * S - 1
            eng.last_rows[:B].copy_(last)
            logits, _ = eng.forward(T, False, use_lora, eng.last_rows, B, hidden=h2)
        else:
            logits, _ = eng.forward(T, True, use_lora, hidden=h2)
        return NDArray(logits.clone().view(B, 1, m.V)), kv


_GLOBAL_FUNCS = {
    "vm.builtin.kv_state_add_sequence": kvc.kv_state_add_sequence,
    "vm.builtin.kv_state_begin_forward": kvc.kv_state_begin_forward,
    "vm.builtin.kv_state_end_forward": kvc.kv_state_end_forward,
}


def get_global_func(name):
    """Stand-in for ``tvm.get_global_func`` for the three KV-state functions."""
    return _GLOBAL_FUNCS[name]
