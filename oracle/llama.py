"""CPU fp32 restatement of the reference's decoder with per-request LoRA.

TEST INFRASTRUCTURE ONLY (see ``oracle/__init__.py``).

Body follows ``tvm/llama_auto_batcher/llama_for_causal_lm.py``: FFN ``:28-36``,
attention split ``:38-67``, pre-norm layer ``:71-84``, model ``:86-100``,
``get_logits`` -> fp32 ``:124-128``, prefill keeps the last token ``:130-137``.
LoRA application follows ``compile_tvm.py:115-161`` (delta added to the
projection output), generalised from q/v to any subset of the seven
projections.  The KV cache here is dense per sequence; the paged cache of the
reference holds the same tokens in the same order, so results are equal.
"""
from __future__ import annotations

import math

import torch

from . import ops

PROJ = {
    "q_proj": "self_attn", "k_proj": "self_attn", "v_proj": "self_attn", "o_proj": "self_attn",
    "gate_proj": "mlp", "up_proj": "mlp", "down_proj": "mlp",
}


class OracleLlama:
    """weights: HF-named state dict; adapters: list of dicts keyed like the
    reference's adapter files (``init_peft_weights/lora_weights.py:18-23``):
    ``layers.{L}.self_attn.q_proj.lora_A.weight`` [r,in], ``...lora_B.weight``
    [out,r]; scales[i] = alpha/r of adapter i."""

    def __init__(self, cfg, weights, adapters=(), scales=(), act_dtype=None):
        """``act_dtype`` (e.g. ``torch.bfloat16``): round every activation the CUDA path stores between two
        kernels to that type (normalised rows, q/k/v, rotated keys, attention output, o/down outputs, the
        SiLU product) while all arithmetic stays fp32.  This separates "what bf16 activation storage costs"
        (fp32 oracle vs this) from "does the CUDA path compute the right thing" (CUDA vs this); the
        reference itself runs fp16/bf16 activations throughout (``gen_lora.py:28``, ``compile_tvm.py:289``)."""
        self.cfg = cfg
        self._r = (lambda t: t.to(act_dtype).float()) if act_dtype is not None else (lambda t: t)
        self.w = {k: v.float() for k, v in weights.items()}
        self.adapters = [{k: v.float() for k, v in a.items()} for a in adapters]
        self.scales = list(scales)
        self.k_cache = {}  # (sid, layer) -> [n, Hkv, D]
        self.v_cache = {}

    # -- projections --------------------------------------------------------
    def _proj(self, layer, name, x, slots):
        """x [T, in]; slots [T] adapter index per row (-1 none)."""
        w = self.w[f"model.layers.{layer}.{PROJ[name]}.{name}.weight"]
        y = x @ w.t()
        for t in range(x.shape[0]):
            s = int(slots[t])
            if s < 0:
                continue
            ka = f"layers.{layer}.{PROJ[name]}.{name}.lora_A.weight"
            if ka not in self.adapters[s]:
                continue
            A = self.adapters[s][ka]
            B = self.adapters[s][ka.replace("lora_A", "lora_B")]
            y[t] += self.scales[s] * (B @ (A @ x[t]))
        return y

    def _layer(self, layer, h, sids, positions, slots, seg):
        """h [T,H]; rows belong to sequences sids[t] at positions[t]; ``seg``
        lists (start,end) row ranges that form one sequence's contiguous
        chunk (prefill: one range of S rows; decode: T ranges of 1 row)."""
        c = self.cfg
        D, Hq, Hkv = c["head_dim"], c["num_attention_heads"], c["num_key_value_heads"]
        r = self._r
        xn = r(ops.rmsnorm(h, self.w[f"model.layers.{layer}.input_layernorm.weight"], c["rms_norm_eps"]))
        q = r(self._proj(layer, "q_proj", xn, slots)).view(-1, Hq, D)
        k = r(self._proj(layer, "k_proj", xn, slots)).view(-1, Hkv, D)
        v = r(self._proj(layer, "v_proj", xn, slots)).view(-1, Hkv, D)
        q = ops.rope_rotate_half(q, positions, c["rope_theta"])
        k = r(ops.rope_rotate_half(k, positions, c["rope_theta"]))
        attn = torch.zeros(h.shape[0], Hq, D)
        for (a, b) in seg:
            sid = int(sids[a])
            key = (sid, layer)
            if key in self.k_cache:
                self.k_cache[key] = torch.cat([self.k_cache[key], k[a:b]], 0)
                self.v_cache[key] = torch.cat([self.v_cache[key], v[a:b]], 0)
            else:
                self.k_cache[key] = k[a:b].clone()
                self.v_cache[key] = v[a:b].clone()
            K, V = self.k_cache[key], self.v_cache[key]
            n_new, n_all = b - a, K.shape[0]
            rep = Hq // Hkv
            Kr, Vr = K.repeat_interleave(rep, 1), V.repeat_interleave(rep, 1)
            s = torch.einsum("shd,nhd->hsn", q[a:b], Kr) / math.sqrt(D)
            qpos = torch.arange(n_all - n_new, n_all)[:, None]
            mask = torch.arange(n_all)[None, :] <= qpos
            s = s.masked_fill(~mask[None], float("-inf"))
            attn[a:b] = torch.einsum("hsn,nhd->shd", torch.softmax(s, -1), Vr)
        h = h + r(self._proj(layer, "o_proj", r(attn).reshape(h.shape[0], Hq * D), slots))
        xn = r(ops.rmsnorm(h, self.w[f"model.layers.{layer}.post_attention_layernorm.weight"], c["rms_norm_eps"]))
        g = self._proj(layer, "gate_proj", xn, slots)
        u = self._proj(layer, "up_proj", xn, slots)
        h = h + r(self._proj(layer, "down_proj", r(ops.silu_mul(g, u)), slots))
        return h

    def _body(self, tokens, sids, positions, slots, seg):
        h = self.w["model.embed_tokens.weight"][torch.as_tensor(tokens, dtype=torch.long)]
        for layer in range(self.cfg["num_hidden_layers"]):
            h = self._layer(layer, h, sids, positions, slots, seg)
        return self._r(ops.rmsnorm(h, self.w["model.norm.weight"], self.cfg["rms_norm_eps"]))

    # -- the two entry points of the executor (llama_exec_graph.py:58-141) ---
    def prefill(self, sid, tokens, slot):
        """One sequence, whole prompt; returns fp32 logits of the last token."""
        S = len(tokens)
        hn = self._body(tokens, [sid] * S, torch.arange(S), [slot] * S, [(0, S)])
        return hn[-1:] @ self.w["lm_head.weight"].t()

    def decode(self, sids, tokens, slots):
        """One token for each live sequence; returns fp32 logits [B,V]."""
        pos = torch.tensor([self.k_cache[(int(s), 0)].shape[0] for s in sids])
        B = len(sids)
        hn = self._body(tokens, sids, pos, slots, [(i, i + 1) for i in range(B)])
        return hn @ self.w["lm_head.weight"].t()

    def greedy(self, prompts, slots, gen_len):
        """Prefill each sequence then batched greedy decode (no EOS stop).
        Returns (tokens [B,gen_len], logits list per step)."""
        B = len(prompts)
        out = [[] for _ in range(B)]
        all_logits = []
        first = []
        for b in range(B):
            lg = self.prefill(b, prompts[b], slots[b])
            first.append(lg)
            out[b].append(int(lg.argmax()))
        all_logits.append(torch.cat(first, 0))
        for _ in range(gen_len - 1):
            lg = self.decode(list(range(B)), [o[-1] for o in out], slots)
            all_logits.append(lg)
            for b in range(B):
                out[b].append(int(lg[b].argmax()))
        return torch.tensor(out), all_logits
