"""Llama decoder with per-request LoRA on the libmlora kernels.

The graph is the one of ``tvm/llama_auto_batcher/llama_for_causal_lm.py``
(``LlamaFFN`` :28-36, ``LlamaAttention`` :38-67, ``LlamaDecoderLayer`` :71-84,
``LlamaModel`` :86-100, ``get_logits`` :124-128, last-token slice of prefill
:130-137) with the LoRA application of ``compile_tvm.py:115-161``, lowered by
hand to this kernel sequence per layer:

    residual_rmsnorm -> lora_shrink(q,k,v) -> linear(W_qkv, +expand)
    -> paged_attention (RoPE + append fused for decode)
    -> lora_shrink(o) -> linear(W_o, +expand)
    -> residual_rmsnorm -> linear(W_gate|W_up, +expand, SiLU*up) -> linear(W_down, +expand)

Weights are packed once at load: q,k,v rows concatenated; gate/up rows
interleaved in blocks of 8 so SiLU*up happens in the projection epilogue;
adapters stacked per projection as A_all [N, n_mod*r_max, in] / B_all
[N, out, r_max] (the stacking ``prepare_model_weights`` does at
``compile_tvm.py:296-314``, kept K-contiguous instead of transposed).
"""
from __future__ import annotations

import os

from dataclasses import dataclass, field

import numpy as np
import torch

from . import ops
from .kv_cache import PagedKVCache
from .ops import LoraStack, LORA_PER_ROW, OUT_F32, SHARE_LORA_KERNEL, SILU_MUL

ATTN_PROJ = ("q_proj", "k_proj", "v_proj", "o_proj")
MLP_PROJ = ("gate_proj", "up_proj", "down_proj")


def interleave_gate_up(g, u):
    """[I,K],[I,K] -> [2I,K] with rows 16j..16j+7 = gate 8j.., rows 16j+8..16j+15 = up 8j..
    (works for any trailing shape; used for weights and for LoRA B matrices)."""
    I = g.shape[0]
    return torch.stack([g.reshape(I // 8, 8, *g.shape[1:]), u.reshape(I // 8, 8, *u.shape[1:])], 1) \
        .reshape(2 * I, *g.shape[1:]).contiguous()


@dataclass
class LayerWeights:
    ln1: torch.Tensor
    ln2: torch.Tensor
    w_qkv: torch.Tensor
    w_o: torch.Tensor
    w_gu: torch.Tensor
    w_down: torch.Tensor
    lora: dict = field(default_factory=dict)  # "qkv" | "o" | "gu" | "down" -> LoraStack


class PackedLlama:
    """Device-resident packed weights.  ``weights`` is an HF-named state dict, ``adapters`` a list
    of dicts keyed like the reference's adapter files
    (``layers.{L}.self_attn.q_proj.lora_A.weight`` [r,in] / ``lora_B.weight`` [out,r],
    ``init_peft_weights/lora_weights.py:18-23``), ``scales[i]`` = alpha/r of adapter i.
    Adapter ``i`` occupies slot ``i`` of every stack."""

    def __init__(self, cfg, weights, adapters=(), scales=(), device="cuda", n_layers=None, pack=True,
                 tp_rank=0, tp_size=1, adapter_capacity=None, max_rank=None, adapter_targets=None):
        """pack=True stores every projection matrix and adapter B stack in the pre-tiled layouts of
        mlora_pack_weight / mlora_pack_lora_b (one bulk copy per pipeline stage).

        tp_size > 1: Megatron-style tensor parallelism.  q/k/v and gate/up are column-parallel (this
        rank keeps the rows of its heads / its slice of the intermediate features), o and down are
        row-parallel (this rank keeps the matching input columns; the partial outputs are summed by an
        all-reduce), lm_head is vocabulary-parallel.  Adapters follow their projection: on a
        column-parallel projection A is replicated and B sliced by rows; on a row-parallel one A is
        sliced by columns and B replicated, so each rank's LoRA partial rides in its GEMM partial and
        the one all-reduce sums both.

        ``adapter_capacity`` / ``max_rank`` / ``adapter_targets``: room for adapters added later with
        :meth:`add_adapter` (slots, widest rank, projection names when no adapter is given at construction)."""
        self.cfg = dict(cfg)
        self.pack = pack
        self.tp_rank, self.tp_size = int(tp_rank), int(tp_size)
        self.device = torch.device(device)
        c = self.cfg
        self.H, self.I, self.V = c["hidden_size"], c["intermediate_size"], c["vocab_size"]
        self.Hq, self.Hkv, self.D = c["num_attention_heads"], c["num_key_value_heads"], c["head_dim"]
        G, R = self.tp_size, self.tp_rank
        if self.Hq % G or self.Hkv % G or self.I % (8 * G) or self.V % G:
            raise ValueError(f"tp_size {G} must divide heads ({self.Hq}/{self.Hkv}), intermediate/8 and vocab")
        self.Hq_full, self.Hkv_full, self.I_full, self.V_full = self.Hq, self.Hkv, self.I, self.V
        self.Hq, self.Hkv, self.I, self.V = self.Hq // G, self.Hkv // G, self.I // G, self.V // G
        self.vocab_offset = R * self.V
        self._q_rows = slice(R * self.Hq * self.D, (R + 1) * self.Hq * self.D)
        self._kv_rows = slice(R * self.Hkv * self.D, (R + 1) * self.Hkv * self.D)
        self._i_rows = slice(R * self.I, (R + 1) * self.I)
        self.L = c["num_hidden_layers"] if n_layers is None else n_layers
        self.eps, self.theta = float(c["rms_norm_eps"]), float(c["rope_theta"])
        if self.I % 8:
            raise ValueError("intermediate_size must be a multiple of 8")
        bf = lambda t: t.to(device=self.device, dtype=torch.bfloat16).contiguous()
        self.embed = bf(weights["model.embed_tokens.weight"])
        self.norm = bf(weights["model.norm.weight"])
        lm = weights["lm_head.weight"][self.vocab_offset:self.vocab_offset + self.V]
        self.lm_head = ops.PackedWeight(bf(lm)) if pack else bf(lm)
        # adapter slots: the adapters given now fill slots 0..n-1; ``adapter_capacity`` reserves further (empty) slots
        # that add_adapter() fills later without moving any buffer (captured graphs stay valid)
        n_slots = max(len(adapters), int(adapter_capacity or 0))
        self.n_adapters = n_slots
        self._free_slots = list(range(n_slots - 1, len(adapters) - 1, -1))
        self.adapter_targets = tuple(adapter_targets) if adapter_targets else None
        ranks = []
        for ad in adapters:  # an adapter's rank = the largest over its projections
            ranks.append(max(v.shape[0] for k, v in ad.items() if k.endswith("lora_A.weight")))
        top = max(ranks + [int(max_rank or 0)]) if (ranks or max_rank) else 0
        self.ranks_host = ranks + [0] * (n_slots - len(ranks))
        self.r_max = (16 if top <= 16 else 32 if top <= 32 else -(-top // 64) * 64) if n_slots else 0
        if self.r_max > 64:
            raise ValueError(f"adapter rank {top} exceeds 64, the widest rank pitch the projection kernels take")
        if n_slots:
            self.ranks = torch.tensor(self.ranks_host, dtype=torch.int32, device=self.device)
            self.scales = torch.tensor(list(scales) + [0.0] * (n_slots - len(ranks)), dtype=torch.float32, device=self.device)
        self.layers = []
        for l in range(self.L):
            p = f"model.layers.{l}."
            w = lambda n: weights[p + n + ".weight"]
            pk = lambda t: ops.PackedWeight(bf(t)) if pack else bf(t)
            lw = LayerWeights(
                ln1=bf(w("input_layernorm")), ln2=bf(w("post_attention_layernorm")),
                w_qkv=pk(torch.cat([w("self_attn.q_proj")[self._q_rows], w("self_attn.k_proj")[self._kv_rows],
                                    w("self_attn.v_proj")[self._kv_rows]], 0)),
                w_o=pk(w("self_attn.o_proj")[:, self._q_rows]),
                w_gu=pk(interleave_gate_up(w("mlp.gate_proj")[self._i_rows], w("mlp.up_proj")[self._i_rows])),
                w_down=pk(w("mlp.down_proj")[:, self._i_rows]))
            if n_slots:
                self._pack_lora(l, lw, adapters)
            self.layers.append(lw)

    # -- adapter stacks ---------------------------------------------------------------------------------------
    def _stack_specs(self):
        qd, kvd = self.Hq * self.D, self.Hkv * self.D
        return {"qkv": ("self_attn", ("q_proj", "k_proj", "v_proj"), (qd, kvd, kvd), self.H, False),
                "o": ("self_attn", ("o_proj",), (self.H,), qd, False),
                "gu": ("mlp", ("gate_proj", "up_proj"), (self.I, self.I), self.H, True),
                "down": ("mlp", ("down_proj",), (self.H,), self.I, False)}

    def _adapter_slices(self, l, ad, blk, proj):
        """(A [r,in], B [out,r]) of one projection of one adapter, cut to this rank's tensor-parallel share."""
        ka = f"layers.{l}.{blk}.{proj}.lora_A.weight"
        if ka not in ad:
            return None
        A, B = ad[ka], ad[ka.replace("lora_A", "lora_B")]
        rows_of = {"q_proj": self._q_rows, "k_proj": self._kv_rows, "v_proj": self._kv_rows,
                   "gate_proj": self._i_rows, "up_proj": self._i_rows}
        cols_of = {"o_proj": self._q_rows, "down_proj": self._i_rows}
        if proj in rows_of:      # column-parallel: B follows the output rows of this rank
            B = B[rows_of[proj]]
        else:                    # row-parallel: A follows the input columns of this rank
            A = A[:, cols_of[proj]]
        return A, B

    def _one_adapter(self, l, key, ad):
        """A_one [n_mod*r_max, in] and B_one [out_total, pitch] (zero padded, bf16, on the device) of adapter ``ad``
        for stack ``key`` of layer ``l``."""
        blk, projs, outs, in_f, interleave = self._stack_specs()[key]
        r_max, dev = self.r_max, self.device
        A_one = torch.zeros(len(projs) * r_max, in_f, dtype=torch.bfloat16, device=dev)
        parts = [torch.zeros(o, r_max, dtype=torch.bfloat16, device=dev) for o in outs]
        for m, proj in enumerate(projs):
            ab = self._adapter_slices(l, ad, blk, proj)
            if ab is None:
                continue
            A, B = ab
            r = A.shape[0]
            if r > r_max:
                raise ValueError(f"adapter rank {r} exceeds the stack's rank pitch {r_max}")
            A_one[m * r_max:m * r_max + r] = A.to(device=dev, dtype=torch.bfloat16)
            parts[m][:, :r] = B.to(device=dev, dtype=torch.bfloat16)
        if interleave:
            # gate rows carry [B_gate | 0], up rows [0 | B_up]: one dot product against [u_gate | u_up]
            z = torch.zeros_like(parts[0])
            B_one = interleave_gate_up(torch.cat([parts[0], z], 1), torch.cat([z, parts[1]], 1))
        else:
            B_one = torch.cat(parts, 0)
        return A_one, B_one.contiguous()

    def _pack_lora(self, l, lw, adapters):
        N, r_max, dev = self.n_adapters, self.r_max, self.device
        for key, (blk, projs, outs, in_f, interleave) in self._stack_specs().items():
            named = any(f"layers.{l}.{blk}.{p}.lora_A.weight" in ad for ad in adapters for p in projs)
            wanted = self.adapter_targets is not None and any(p in self.adapter_targets for p in projs)
            if not (named or wanted):
                continue
            pitch = 2 * r_max if interleave else r_max
            A_all = torch.zeros(N, len(projs) * r_max, in_f, dtype=torch.bfloat16, device=dev)
            B_all = torch.zeros(N, sum(outs), pitch, dtype=torch.bfloat16, device=dev)
            for s, ad in enumerate(adapters):
                A_all[s], B_all[s] = self._one_adapter(l, key, ad)
            offs = tuple(int(x) for x in np.cumsum([0] + list(outs)))
            st = LoraStack(A_all, B_all, self.ranks, self.scales, r_max, len(projs), offs)
            st.bytes_per_adapter = 2 * (A_all[0].numel() + sum(outs) * r_max)
            # mixed ranks: a second, rank-compact copy of B for the per-row expand (batches where every row brings
            # its own adapter); not for stacks with spare slots, whose rows must stay writable in place
            mixed = any(r != r_max for r in self.ranks_host)
            if mixed and not interleave and not self._free_slots and N == len(adapters):
                st.split_b(self.ranks_host)
            if self.pack and all(o % 128 == 0 for o in offs[1:-1]):
                st.pack_b()
            lw.lora[key] = st

    def add_adapter(self, adapter: dict, scale: float) -> int:
        """Loads one more adapter into a free slot (reserved with ``adapter_capacity``) while the model is serving:
        only that slot's rows of the stacks, its rank and its scale are written, so buffers -- and CUDA graphs
        captured over them -- stay as they are.  Returns the slot.  (The loader half of the reference's adapter
        files, ``init_peft_weights/lora_weights.py`` / ``compile_tvm.py:296-314``, made incremental.)"""
        if not self._free_slots:
            raise RuntimeError("no free adapter slot: construct PackedLlama with a larger adapter_capacity")
        rank = max(v.shape[0] for k, v in adapter.items() if k.endswith("lora_A.weight"))
        if rank > self.r_max:
            raise ValueError(f"adapter rank {rank} exceeds the rank pitch {self.r_max} the stacks were built with")
        slot = self._free_slots.pop()
        for l, lw in enumerate(self.layers):
            for key, st in lw.lora.items():
                A_one, B_one = self._one_adapter(l, key, adapter)
                st.A_all[slot].copy_(A_one)
                st.write_b_slot(slot, B_one)
                st._all_full_rank = None
                st.B_split = st.rank_tbl = None
        self.ranks[slot] = rank
        self.scales[slot] = float(scale)
        self.ranks_host[slot] = rank
        return slot

    def remove_adapter(self, slot: int) -> None:
        """Empties a slot (zero rank, zero scale, zero rows: the kernels multiply padding rather than look ranks up).
        Requests must have stopped naming the slot."""
        if slot in self._free_slots or not 0 <= slot < self.n_adapters:
            raise ValueError(f"adapter slot {slot} is not in use")
        for lw in self.layers:
            for st in lw.lora.values():
                st.A_all[slot].zero_()
                st.write_b_slot(slot, None)
                st._all_full_rank = None
        self.ranks[slot] = 0
        self.scales[slot] = 0.0
        self.ranks_host[slot] = 0
        self._free_slots.append(slot)

    def weight_bytes(self):
        """Bytes of base weights one decode step streams (all layers + final norm + lm_head)."""
        n = self.norm.numel() + self.lm_head.numel()
        for lw in self.layers:
            n += lw.ln1.numel() + lw.ln2.numel() + lw.w_qkv.numel() + lw.w_o.numel() + lw.w_gu.numel() + lw.w_down.numel()
        return 2 * n

    def lora_bytes_per_adapter(self):
        n = 0
        for lw in self.layers:
            for st in lw.lora.values():
                n += st.bytes_per_adapter
        return n


class Engine:
    """Runs prefill / decode forwards of a :class:`PackedLlama` over a :class:`PagedKVCache`.

    All activations live in buffers sized for ``max_rows`` rows, allocated once, so a forward does
    no allocation and can be captured in a CUDA graph."""

    def __init__(self, model: PackedLlama, kv: PagedKVCache, max_rows: int, collective=None):
        """``collective`` (tensor parallelism only): object with ``all_reduce_sum(t)`` (in place) and
        ``all_gather(t) -> [G, *t.shape]``; see ``sharding.DistCollective``."""
        self.m, self.kv, self.max_rows = model, kv, int(max_rows)
        self.coll = collective
        if model.tp_size > 1 and collective is None:
            raise ValueError("a tensor-parallel model needs a collective")
        m, dev, T = model, model.device, int(max_rows)
        bf = dict(dtype=torch.bfloat16, device=dev)
        f32 = dict(dtype=torch.float32, device=dev)
        qkv_out = (m.Hq + 2 * m.Hkv) * m.D
        self.res = torch.zeros(T, m.H, **f32)
        self.res2 = torch.zeros(T, m.H, **f32)  # the fused norm + shrink moves the residual between two buffers
        self.xn = torch.zeros(T, m.H, **bf)
        self.qkv = torch.zeros(T, qkv_out, **bf)
        self.attn = torch.zeros(T, m.Hq * m.D, **bf)
        self.y = torch.zeros(T, m.H, **bf)
        self.act = torch.zeros(T, m.I, **bf)
        self.u = torch.zeros(T, max(3 * m.r_max, 8), **f32)
        self.logits = torch.zeros(T, m.V, **f32)
        self.next_tok = torch.zeros(T, dtype=torch.int32, device=dev)
        self.tokens = torch.zeros(T, dtype=torch.int32, device=dev)
        self.slots = torch.full((T,), -1, dtype=torch.int32, device=dev)
        self.row_slot = torch.zeros(T, dtype=torch.int32, device=dev)
        self.row_pos = torch.zeros(T, dtype=torch.int32, device=dev)
        self.last_rows = torch.zeros(T, dtype=torch.int32, device=dev)
        self.iota = torch.arange(T, dtype=torch.int32, device=dev)
        self.xn_last = torch.zeros(T, m.H, **bf)
        # scratch sized for the largest projection of this model at max_rows
        lib = ops._lib.lib()
        need = max(lib.mlora_linear_workspace(T, k, n) for k, n in
                   ((m.H, qkv_out), (m.Hq * m.D, m.H), (m.H, 2 * m.I), (m.I, m.H), (m.H, m.V)))
        # (+ the pre-activations of a gate|up call that takes the per-row expand: decode passes of up to 128 rows)
        need = max(need, lib.mlora_linear_workspace_flags(min(T, 128), m.H, 2 * m.I, SILU_MUL | LORA_PER_ROW))
        # The engine owns its scratch: captured graphs hold these addresses, so the buffers live as long as the
        # engine and are never shared with (or outgrown by) other callers on the device.
        self.ws_linear = ops.new_workspace(need, dev)
        self.ws_attn = ops.new_workspace(lib.mlora_paged_attention_workspace(T, m.Hq, m.D, 16), dev)
        # the o-projection's shrink computed in the attention launch (decode passes): its own zero-initialised scratch.
        # Measured on the benchmark's step: 32 launches fewer but 0.035 ms slower (the tail sits on the attention
        # kernel's critical path, the separate shrink launch overlaps the projection's weight prefetch), so off unless asked for
        self.fuse_o_shrink = os.environ.get("MLORA_FUSE_O_SHRINK", "0") == "1"
        self.ws_oshrink = ops.new_workspace(lib.mlora_paged_attention_shrink_workspace(min(T, 1024), m.Hq, max(m.r_max, 8)), dev)
        # prompt passes: tiles of <= 128 consecutive rows of one sequence for the tensor-core attention
        self.tc_prefill = os.environ.get("MLORA_TC_PREFILL", "1") != "0" and m.D == 128 and kv.page_size == 16
        self.pf_tiles = torch.zeros((T + 127) // 128 + kv.max_batch + 1, 4, dtype=torch.int32, device=dev)
        self.pf_status = torch.zeros(1, dtype=torch.int32, device=dev)
        self._n_pf_tiles = 0
        self._graphs = {}
        self.n_distinct = 0  # distinct adapters among the rows staged for the next pass (set with self.slots)
        self.fuse_norm_shrink = os.environ.get("MLORA_FUSE_NORM_SHRINK", "1") != "0"
        # decode passes of <= 32 rows: the residual add + RMSNorm between the o projection and gate|up folded into the two
        # projections' epilogues (mlora_linear_norm) -- one launch fewer per layer.  Measured on the benchmark's step: the
        # two folding projections run a kernel variant of their own (69 registers more per thread), and a step that
        # alternates between two variants loses more than the 32 launches save: 5.03 ms against 4.99, so off unless asked for
        self.fold_norm = os.environ.get("MLORA_FOLD_NORM", "0") == "1"
        self.sumsq = torch.zeros(-(-m.H // 128) * 32, dtype=torch.float32, device=dev)
        # decode-size passes can run everything between two attention calls as one persistent launch
        # (mlora_decode_chain); measured slower than the separate launches on the benchmark's step, so off unless asked for
        self.use_chain = os.environ.get("MLORA_CHAIN", "0") == "1"
        # "2": only gate|up -> down (two projections with nothing between them) as one launch
        self.chain_mlp = os.environ.get("MLORA_CHAIN", "0") == "2"

    # ------------------------------------------------------------------------------------------
    def status_word(self) -> int:
        """Status word of the projection kernels' scratch (synchronises): non-zero after a bounded wait expired
        somewhere since the buffer was last cleared; the outputs since then are undefined."""
        return ops.status_word(self.ws_linear)

    def check_status(self):
        """Raises if a projection kernel gave up a bounded wait, after re-zeroing the scratch (arrival counters of
        split tiles may be stale after such a failure) so that the engine stays usable."""
        st = self.status_word()
        if st:
            self.ws_linear.zero_()
            raise RuntimeError(f"mlora: a projection kernel gave up a bounded wait (status bits {st:#x}); "
                               "the results of this pass are undefined")

    @staticmethod
    def _full_rank(stack):
        """Do all adapters of the stack fill its rank pitch?  (Looked up once per stack.)"""
        v = getattr(stack, "_all_full_rank", None)
        if v is None:
            v = bool((stack.ranks == stack.r_max).all().item())
            stack._all_full_rank = v
        return v

    def _lora_flags(self, T, stack, flags):
        """The tensor-core expand holds the operands of a token tile's distinct adapters in a shared-memory cache
        (16 KB, 64 KB at 128-token tiles); a decode batch that brings more distinct adapters than fit (e.g. every
        request its own) takes the expand laid out by (row, output feature) instead."""
        if T > 128:
            return flags
        bn = 16 if T <= 16 else 32 if T <= 32 else 64 if T <= 64 else 128
        pitch = stack.r_max * (2 if flags & SILU_MUL else 1)  # interleaved gate/up: one operand of both modules' ranks
        cap = ((64 if bn == 128 else 16) * 1024) // (bn * pitch * 2)
        return flags | LORA_PER_ROW if self.n_distinct > max(cap, 1) else flags

    def _reduce_norm(self, delta, res, w, out, reduce=True):
        """res += delta (summed over the tensor-parallel ranks when ``delta`` is a row-parallel partial), out =
        RMSNorm(res) * w: one fused exchange kernel when the collective has one, else all-reduce + norm kernel."""
        m = self.m
        if m.tp_size > 1 and reduce and delta is not None:
            fused = getattr(self.coll, "allreduce_rmsnorm", None)
            if fused is not None and fused(delta, res, w, m.eps, out):
                return
            self.coll.all_reduce_sum(delta)
        ops.residual_rmsnorm(delta, res, w, m.eps, out=out)

    def _mlp_chained(self, T, lw, slots, xn, act, y):
        """gate|up (SiLU) -> down as ONE persistent launch (mlora_decode_chain with two phases); False when the shapes
        do not fit it or the switch is off."""
        m = self.m
        if not (self.chain_mlp and m.pack and 0 < T <= 32):
            return False
        steps = []
        for x, W, out, key, fl in ((xn, lw.w_gu, act, "gu", SILU_MUL), (act, lw.w_down, y, "down", 0)):
            st = ops.ChainStep(x=x, W=W, y=out, flags=fl)
            stack = lw.lora.get(key)
            if stack is not None and slots is not None:
                if self._lora_flags(T, stack, fl) & LORA_PER_ROW:
                    return False
                r_tot = stack.r_max * stack.n_mod
                st.stack, st.u = stack, self.u.view(-1)[: T * r_tot].view(T, r_tot)
            steps.append(st)
        if steps[0].stack is not None and steps[1].stack is not None:
            return False  # (the two shrink outputs would share one buffer inside one launch)
        if not ops.chain_supported(T, steps):
            return False
        ops.decode_chain(steps, slots, m.ranks if m.n_adapters else None, m.scales if m.n_adapters else None, m.n_adapters,
                         self.ws_linear)
        return True

    def _proj(self, x, W, stack, slots, out, flags=0):
        T = x.shape[0]
        if stack is not None and slots is not None:
            r_tot = stack.r_max * stack.n_mod
            u = self.u.view(-1)[: T * r_tot].view(T, r_tot)
            ops.lora_shrink(x, stack, slots, out=u)
            return ops.linear(x, W, stack, slots, u=u, flags=self._lora_flags(T, stack, flags), out=out,
                              work=self.ws_linear)
        # a projection without adapters inside a pass that has some: same kernel variant as its neighbours
        return ops.linear(x, W, flags=flags | (SHARE_LORA_KERNEL if slots is not None else 0), out=out,
                          work=self.ws_linear)

    # ------------------------------------------------------------------------------------------
    def _chain_plan(self, T, slots):
        """The decode pass as chained launches: [norm + q/k/v of layer 0], then per layer one chain
        [o, norm + gate|up, down, norm + q/k/v of the next layer (or the final norm + lm_head)] after its
        attention call.  None when some phase does not fit ``mlora_decode_chain``."""
        m = self.m
        if not (self.use_chain and m.pack and m.tp_size == 1 and 0 < T <= 32):
            return None
        res, xn, qkv, attn, y, act = self.res[:T], self.xn[:T], self.qkv[:T], self.attn[:T], self.y[:T], self.act[:T]

        def step(x, W, out, stack, flags=0, norm_w=None, delta=None):
            st = ops.ChainStep(x=x, W=W, y=out, flags=flags)
            if norm_w is not None:
                st.res, st.delta, st.norm_w, st.eps = res, delta, norm_w, m.eps
            if stack is not None and slots is not None:
                if self._lora_flags(T, stack, flags) & LORA_PER_ROW:
                    return None
                r_tot = stack.r_max * stack.n_mod
                st.stack, st.u = stack, self.u.view(-1)[: T * r_tot].view(T, r_tot)
            return st

        chains = []
        lw0 = m.layers[0]
        chains.append([step(xn, lw0.w_qkv, qkv, lw0.lora.get("qkv"), norm_w=lw0.ln1, delta=None)])
        for l, lw in enumerate(m.layers):
            ch = [step(attn, lw.w_o, y, lw.lora.get("o")),
                  step(xn, lw.w_gu, act, lw.lora.get("gu"), flags=SILU_MUL, norm_w=lw.ln2, delta=y),
                  step(act, lw.w_down, y, lw.lora.get("down"))]
            if l + 1 < len(m.layers):
                nx = m.layers[l + 1]
                ch.append(step(xn, nx.w_qkv, qkv, nx.lora.get("qkv"), norm_w=nx.ln1, delta=y))
            else:
                ch.append(step(xn, m.lm_head, self.logits[:T], None, flags=OUT_F32, norm_w=m.norm, delta=y))
            chains.append(ch)
        for ch in chains:
            if any(s is None for s in ch) or not ops.chain_supported(T, ch):
                return None
        # every u view shares one buffer: the q/k/v, o, gate|up and down shrinks of a chain run one after the other
        return chains

    def _forward_chained(self, T, chains, slots, hidden):
        m, kv = self.m, self.kv
        res, qkv, attn = self.res[:T], self.qkv[:T], self.attn[:T]
        row_slot, row_pos = self.row_slot[:T], self.row_pos[:T]
        if hidden is None:
            ops.embed(self.tokens[:T], m.embed, res=res)
        else:
            ops.embed(self.iota[:T], hidden, res=res)
        ranks = m.ranks if m.n_adapters else None
        scales = m.scales if m.n_adapters else None
        run = lambda ch: ops.decode_chain(ch, slots, ranks, scales, m.n_adapters, self.ws_linear)
        run(chains[0])
        for l in range(len(m.layers)):
            ops.paged_attention(qkv, kv.k_pages(l), kv.v_pages(l), kv.block_table, row_slot, row_pos, m.Hq, m.Hkv, m.D,
                                kv.page_size, m.theta, True, out=attn, work=self.ws_attn)
            run(chains[l + 1])
        ops.argmax(self.logits[:T], out=self.next_tok[:T])
        return self.logits[:T], self.next_tok[:T]

    def forward(self, T: int, fused_append: bool, use_lora: bool = True, lm_rows=None, n_lm=None, hidden=None):
        """One pass over the T rows staged in self.tokens / self.slots / self.row_slot /
        self.row_pos.  Logits (fp32) land in self.logits[:n_lm], greedy tokens in self.next_tok.
        ``lm_rows`` (device int32 [n_lm]) selects the rows that get logits (prefill: last token of
        each sequence); None = every row.  ``hidden`` (bf16 [T,H]) replaces the embedding lookup."""
        m, kv = self.m, self.kv
        tok, slots = self.tokens[:T], (self.slots[:T] if (use_lora and m.n_adapters) else None)
        if fused_append and lm_rows is None:
            chains = self._chain_plan(T, slots)
            if chains is not None:
                return self._forward_chained(T, chains, slots, hidden)
        row_slot, row_pos = self.row_slot[:T], self.row_pos[:T]
        res, xn, qkv, attn, y, act = self.res[:T], self.xn[:T], self.qkv[:T], self.attn[:T], self.y[:T], self.act[:T]
        if hidden is None:
            ops.embed(tok, m.embed, res=res)
        else:  # hidden states handed in by the caller (the VM's separate "embed" function): bf16 [T,H] -> fp32 residual
            ops.embed(self.iota[:T], hidden, res=res)
        delta = None
        res_other = self.res2[:T]
        for l, lw in enumerate(m.layers):
            st = lw.lora.get("qkv")
            if (st is not None and slots is not None and T < 256 and m.H <= 8192 and self.fuse_norm_shrink
                    and m.tp_size == 1 and self._full_rank(st)):  # (the fused kernel reads every rank row of the pitch)
                # one launch: residual add + RMSNorm + the shrink that reads the normalised rows
                r_tot = st.r_max * st.n_mod
                u = self.u.view(-1)[: T * r_tot].view(T, r_tot)
                ops.residual_rmsnorm_shrink(delta, res, res_other, lw.ln1, m.eps, xn, st, slots, u)
                res, res_other = res_other, res
                ops.linear(xn, lw.w_qkv, st, slots, u=u, flags=self._lora_flags(T, st, 0), out=qkv, work=self.ws_linear)
            else:
                self._reduce_norm(delta, res, lw.ln1, xn, reduce=l > 0)
                self._proj(xn, lw.w_qkv, st, slots, qkv)
            kp, vp = kv.k_pages(l), kv.v_pages(l)
            if not fused_append:
                ops.kv_append_rope(qkv, kp, vp, kv.block_table, row_slot, row_pos, m.Hq, m.Hkv, m.D, kv.page_size,
                                   m.theta)
            st_o = lw.lora.get("o")
            lora_o = st_o is not None and slots is not None
            u_o = self.u.view(-1)[: T * st_o.r_max].view(T, st_o.r_max) if lora_o else None
            if (lora_o and self.fuse_o_shrink and fused_append and T <= 1024
                    and ops.attention_shrink_fits(T, m.Hq, kv.block_table.shape[1], st_o)):
                # attention and the o-projection's shrink in one launch; the projection then only expands
                ops.paged_attention_shrink(qkv, kp, vp, kv.block_table, row_slot, row_pos, m.Hq, m.Hkv, m.D, kv.page_size,
                                           m.theta, fused_append, attn, st_o, slots, u_o, self.ws_oshrink)
            else:
                if not fused_append and self.tc_prefill and self._n_pf_tiles > 0:
                    ops.prefill_attention(qkv, kp, vp, kv.block_table, self.pf_tiles, self._n_pf_tiles, m.Hq, m.Hkv, m.D,
                                          kv.page_size, attn, self.pf_status)
                else:
                    ops.paged_attention(qkv, kp, vp, kv.block_table, row_slot, row_pos, m.Hq, m.Hkv, m.D, kv.page_size,
                                        m.theta, fused_append, out=attn, work=self.ws_attn)
                if lora_o:
                    ops.lora_shrink(attn, st_o, slots, out=u_o)
            fl_o = self._lora_flags(T, st_o, 0) if lora_o else (SHARE_LORA_KERNEL if slots is not None else 0)
            if (self.fold_norm and fused_append and T <= 32 and m.tp_size == 1 and not self.chain_mlp
                    and not fl_o & LORA_PER_ROW and (lw.lora.get("gu") is None or slots is None)):
                # residual add + RMSNorm folded into the two projections around it: o writes the residual, the rows
                # times the norm weight and per-tile sums of squares; gate|up scales its output rows by their 1/rms
                ops.linear_norm(attn, lw.w_o, st_o if lora_o else None, slots, u=u_o, flags=fl_o, out=xn, work=self.ws_linear,
                                res=res, norm_w=lw.ln2, sumsq_out=self.sumsq)
                ops.linear_norm(xn, lw.w_gu, flags=SILU_MUL | (SHARE_LORA_KERNEL if slots is not None else 0), out=act,
                                work=self.ws_linear, sumsq_in=self.sumsq, n_sumsq_in=-(-m.H // 128), eps=m.eps, norm_dim=m.H)
                self._proj(act, lw.w_down, lw.lora.get("down"), slots, y)
            else:
                if lora_o:
                    ops.linear(attn, lw.w_o, st_o, slots, u=u_o, flags=fl_o, out=y, work=self.ws_linear)
                else:
                    ops.linear(attn, lw.w_o, flags=fl_o, out=y, work=self.ws_linear)
                # row-parallel partials (base + LoRA) -> full o_proj output, added to the residual, normalised
                self._reduce_norm(y, res, lw.ln2, xn)
                if not self._mlp_chained(T, lw, slots, xn, act, y):
                    self._proj(xn, lw.w_gu, lw.lora.get("gu"), slots, act, flags=SILU_MUL)
                    self._proj(act, lw.w_down, lw.lora.get("down"), slots, y)
            delta = y  # (under tensor parallelism still a partial sum: reduced together with the next norm)
        self._reduce_norm(delta, res, m.norm, xn)
        if lm_rows is not None:
            xl = ops.embed(lm_rows[:n_lm], xn, out_bf16=self.xn_last[:n_lm])  # row gather
        else:
            n_lm, xl = T, xn
        ops.linear(xl, m.lm_head, flags=OUT_F32 | (SHARE_LORA_KERNEL if slots is not None else 0), out=self.logits[:n_lm],
                   work=self.ws_linear)
        ops.argmax(self.logits[:n_lm], out=self.next_tok[:n_lm])
        if m.tp_size > 1:
            # vocabulary-parallel greedy token: every rank offers (its best logit, its global index); the
            # winner is the highest logit, lowest rank on ties (= lowest index, as np.argmax)
            lg, tk = self.logits[:n_lm], self.next_tok[:n_lm]
            best = lg.gather(1, tk.long().unsqueeze(1)).squeeze(1)
            pair = torch.stack([best, (tk + m.vocab_offset).float()], 1)
            allp = self.coll.all_gather(pair)                       # [G, n_lm, 2]
            win = allp[:, :, 0].argmax(0)                           # first maximum along ranks
            tk.copy_(allp[win, torch.arange(n_lm, device=lg.device), 1].int())
        return self.logits[:n_lm], self.next_tok[:n_lm]

    # ------------------------------------------------------------------------------------------
    def _stage(self, dst, values, dtype):
        t = torch.as_tensor(np.asarray(values), dtype=dtype)
        dst[: t.numel()].copy_(t.pin_memory(), non_blocking=True)

    def prefill(self, seq_ids, prompts, adapter_slots, use_lora=True):
        """Prefill whole prompts (lists of token ids) of already-added sequences, chunked to
        max_rows rows per pass.  Returns (logits [n_seq,V] fp32, next tokens [n_seq] int32)."""
        kv = self.kv
        out_logits = torch.empty(len(seq_ids), self.m.V, dtype=torch.float32, device=self.m.device)
        out_tok = torch.empty(len(seq_ids), dtype=torch.int32, device=self.m.device)
        # rows: (seq index, position) in sequence order, cut into chunks
        pending = [(i, 0) for i in range(len(seq_ids))]
        while pending:
            rows_left = self.max_rows
            chunk = []  # (seq index, start, n)
            nxt = []
            for i, start in pending:
                n_total = len(prompts[i])
                if rows_left == 0:
                    nxt.append((i, start))
                    continue
                n = min(rows_left, n_total - start)
                chunk.append((i, start, n))
                rows_left -= n
                if start + n < n_total:
                    nxt.append((i, start + n))
            pending = nxt
            T = sum(n for _, _, n in chunk)
            toks = np.concatenate([np.asarray(prompts[i][s:s + n], dtype=np.int32) for i, s, n in chunk])
            slots = np.concatenate([np.full(n, adapter_slots[i], dtype=np.int32) for i, _, n in chunk])
            row_slot, row_pos = kv.begin_forward([seq_ids[i] for i, _, _ in chunk], [n for _, _, n in chunk])
            self._stage(self.tokens, toks, torch.int32)
            self._stage(self.slots, slots, torch.int32)
            self.n_distinct = len({int(s) for s in slots if s >= 0})
            self.row_slot[:T].copy_(row_slot)
            self.row_pos[:T].copy_(row_pos)
            # tiles of the tensor-core prompt attention: <= 128 consecutive rows of one sequence each
            tiles, a0 = [], 0
            for i, s0, n in chunk:
                for off in range(0, n, 128):
                    tiles.append((kv.slot(seq_ids[i]), a0 + off, min(128, n - off), s0 + off))
                a0 += n
            self._n_pf_tiles = 0
            if self.tc_prefill and len(tiles) <= self.pf_tiles.shape[0]:
                self._stage(self.pf_tiles.view(-1), np.asarray(tiles, dtype=np.int32).reshape(-1), torch.int32)
                self._n_pf_tiles = len(tiles)
            ends, fin, a = [], [], 0
            for i, s, n in chunk:
                a += n
                if s + n == len(prompts[i]):
                    ends.append(a - 1)
                    fin.append(i)
            if ends:
                self._stage(self.last_rows, ends, torch.int32)
                lg, tk = self.forward(T, False, use_lora, self.last_rows, len(ends))
                idx = torch.tensor(fin, device=self.m.device)
                out_logits[idx] = lg
                out_tok[idx] = tk
            else:
                self._stage(self.last_rows, [T - 1], torch.int32)
                self.forward(T, False, use_lora, self.last_rows, 1)
            kv.end_forward()
            self._n_pf_tiles = 0
        self.check_status()  # (synchronises; prefill is not the latency-critical call)
        if int(self.pf_status.item()):
            self.pf_status.zero_()
            raise RuntimeError("mlora: the prompt attention kernel gave up a bounded wait; this pass's results are undefined")
        return out_logits, out_tok

    def decode(self, seq_ids, tokens, adapter_slots, use_lora=True):
        """One eager decode step (host builds the row tables, as the reference's executor does)."""
        B = len(seq_ids)
        row_slot, row_pos = self.kv.begin_forward(seq_ids, [1] * B)
        self._stage(self.tokens, tokens, torch.int32)
        self._stage(self.slots, adapter_slots, torch.int32)
        self.n_distinct = len({int(s) for s in adapter_slots if s >= 0})
        self.row_slot[:B].copy_(row_slot)
        self.row_pos[:B].copy_(row_pos)
        out = self.forward(B, True, use_lora)
        self.kv.end_forward()
        return out

    # -- CUDA-graph decode: the whole step, including position bookkeeping, is one graph ---------------
    def capture_decode(self, seq_ids, adapter_slots, use_lora=True, reserve_tokens=0, feed_back=True):
        """Capture a decode step for this batch.  Rows follow ``seq_ids``; each replay consumes
        self.tokens[:B] (device) and leaves greedy tokens in self.next_tok[:B]."""
        B, kv = len(seq_ids), self.kv
        for sid in seq_ids:
            kv.reserve(sid, kv.length(sid) + reserve_tokens + 1)
        self._stage(self.row_slot, [kv.slot(s) for s in seq_ids], torch.int32)
        self._stage(self.slots, adapter_slots, torch.int32)
        self.n_distinct = len({int(s) for s in adapter_slots if s >= 0})
        torch.cuda.synchronize()
        saved = kv.seq_lens.clone()

        def step():
            ops.kv_begin_decode(self.row_slot[:B], kv.seq_lens, self.row_pos[:B])
            self.forward(B, True, use_lora)
            if feed_back:  # the greedy tokens become the next step's input without leaving the device
                self.tokens[:B].copy_(self.next_tok[:B])

        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            step()  # warm-up outside capture (lazy module loading, attribute setting)
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            step()
        kv.seq_lens.copy_(saved)  # warm-up advanced the device lengths; capture itself runs nothing
        torch.cuda.synchronize()
        return DecodeGraph(self, g, list(seq_ids), B)


class DecodeGraph:
    def __init__(self, engine, graph, seq_ids, B):
        self.engine, self.graph, self.seq_ids, self.B = engine, graph, seq_ids, B
        self._headroom = 0  # replays known to be covered by reserved pages (re-counted when it runs out)

    def replay(self):
        """One token for every row: consumes engine.tokens[:B], leaves greedy tokens in
        engine.next_tok[:B] (and, when captured with feed_back, back in engine.tokens).
        The step appends one token per sequence through block-table entries that must exist already:
        pages are reserved here when the host allocator still has some, else the replay is refused."""
        kv = self.engine.kv
        if self._headroom <= 0:
            for sid in self.seq_ids:
                kv.reserve(sid, kv.length(sid) + 1)  # raises when the pool or the row's table is exhausted
            self._headroom = min(kv.tokens_reserved(sid) - kv.length(sid) for sid in self.seq_ids)
        self._headroom -= 1
        self.graph.replay()
        self.engine.kv.note_device_decode(self.seq_ids)


class DecodeSession:
    """The batched greedy loop of one fused decode node (``tvm/llama_auto_batcher/llama_exec_graph.py:102-141``)
    with the batch state on the device: sequences finish on their end-of-sequence token or their own
    ``max_gen_len`` and leave the batch without the host rebuilding anything.  Every step is a CUDA-graph replay
    of ``decode_step_begin -> forward -> decode_step_end`` captured for a bucket of rows (powers of two up to the
    node's size); the host only learns the live count (4 bytes, every ``sync_every`` steps) to pick the bucket and
    to stop, and reads all generated tokens once at the end.

    ``seq_ids`` must already be in bucketing order (``LlamaSeqInfo.order_seqs``): rows of one adapter adjacent."""

    def __init__(self, engine: Engine, seq_ids, adapter_slots, first_tokens, max_gen, eos_id=None, use_lora=True):
        self.eng, self.seq_ids, self.use_lora = engine, list(seq_ids), use_lora
        kv, dev, n = engine.kv, engine.m.device, len(seq_ids)
        self.n = n
        self.max_len = int(max(max_gen)) + 1  # (a sequence always takes part in the node's first step)
        i32 = lambda v: torch.as_tensor(np.asarray(v, dtype=np.int32)).pin_memory().to(dev, non_blocking=True)
        self.live = torch.ones(n, dtype=torch.int32, device=dev)
        self.seq_slot = i32([kv.slot(s) for s in seq_ids])
        self.adapter_slot = i32(adapter_slots)
        self.last_tok = i32(first_tokens)
        self.max_gen = i32(max_gen)
        self.gen_count = torch.ones(n, dtype=torch.int32, device=dev)  # the prefill's token is the first one
        self.out_tokens = torch.zeros(n, self.max_len, dtype=torch.int32, device=dev)
        self.out_tokens[:, 0] = self.last_tok
        self.row_src = torch.full((max(n, 1),), -1, dtype=torch.int32, device=dev)
        self.n_live = torch.zeros(1, dtype=torch.int32, device=dev)
        self._n_live_host = torch.zeros(1, dtype=torch.int32).pin_memory()
        self.eos_id = -1 if eos_id is None else int(eos_id)
        self.n_distinct = len({int(a) for a in adapter_slots if a >= 0})
        for sid, g in zip(seq_ids, max_gen):
            kv.reserve(sid, kv.length(sid) + int(g) + 1)
        self._graphs = {}
        self.steps = 0
        self.d2h_bytes = 0

    def _step(self, rows):
        e = self.eng
        ops.decode_step_begin(self.live, self.seq_slot, self.adapter_slot, self.last_tok, rows, e.kv.seq_lens,
                              self.row_src, e.row_slot, e.row_pos, e.slots, e.tokens, self.n_live)
        e.n_distinct = self.n_distinct
        e.forward(rows, True, self.use_lora)
        ops.decode_step_end(self.row_src, e.next_tok, rows, self.live, self.last_tok, self.gen_count, self.max_gen,
                            self.out_tokens, self.eos_id, self.n_live)

    def _graph(self, rows):
        g = self._graphs.get(rows)
        if g is not None:
            return g
        e = self.eng
        state = (self.live, self.last_tok, self.gen_count, self.out_tokens, e.kv.seq_lens, self.n_live)
        saved = [t.clone() for t in state]
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            self._step(rows)  # warm-up outside capture; its effects are undone below
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            self._step(rows)
        for t, s in zip(state, saved):
            t.copy_(s)
        torch.cuda.synchronize()
        self._graphs[rows] = g
        return g

    @staticmethod
    def bucket(n_live, n):
        """Rows of the step that serves ``n_live`` live sequences: the next power of two, capped at the node's size."""
        b = 1
        while b < n_live:
            b *= 2
        return min(b, n)

    def run(self, sync_every=1):
        """Runs until every sequence has finished.  Returns the token lists (first token included) in the order of
        ``seq_ids``."""
        bound = self.n  # upper bound of the live count (sequences only ever leave)
        while bound > 0:
            g = self._graph(self.bucket(bound, self.n))
            for _ in range(max(1, sync_every)):
                g.replay()
                self.steps += 1
            self._n_live_host.copy_(self.n_live, non_blocking=True)
            torch.cuda.current_stream().synchronize()
            self.d2h_bytes += 4
            bound = int(self._n_live_host[0])
        counts = self.gen_count.cpu().tolist()
        toks = self.out_tokens.cpu().tolist()
        self.d2h_bytes += 4 * (self.n + self.out_tokens.numel())
        for sid, c in zip(self.seq_ids, counts):
            self.eng.kv.note_device_decode([sid], c - 1)
        return [t[:c] for t, c in zip(toks, counts)]
