"""CPU restatement (torch, fp32 unless said otherwise) of the hot-path operators.

TEST INFRASTRUCTURE ONLY (see ``oracle/__init__.py``).
"""
from __future__ import annotations

import math

import torch


# --------------------------------------------------------------------------
# LoRA on top of a base projection
# --------------------------------------------------------------------------
def gather_bmm_linear(x, weight, lora_A, lora_B, scaling, ids, bias=None):
    """``GatherBMMLinear.forward``, gather branch.

    Follows ``huggingface/custom_peft/lora_gatherbmm_linear_layer.py:14-20``:
    ``result = base_layer(x)``; per row ``i`` the adapter's ``A`` ([r,in]) and
    ``B * scaling`` ([out,r], scale folded into B *before* the matmul) are
    stacked and transposed, dropout is the identity in eval mode, and
    ``result += bmm(bmm(x, A_g), B_g)``.

    x [B,S,in]; weight [out,in]; lora_A[n] [r,in]; lora_B[n] [out,r];
    scaling[n] float; ids[B] ints (index into the lists).
    """
    result = torch.nn.functional.linear(x, weight, bias)
    a_g = torch.stack([lora_A[int(i)] for i in ids], dim=0).transpose(1, 2)
    b_g = torch.stack([lora_B[int(i)] * scaling[int(i)] for i in ids], dim=0).transpose(1, 2)
    x_d = torch.stack([x[i].to(a_g.dtype) for i in range(len(ids))])
    out = torch.bmm(torch.bmm(x_d, a_g), b_g)
    return result + out.to(result.dtype)


def take_matmul_lora(x, p0, p1, wids, scaling):
    """The auto-batcher's synthesised adapter forward.

    Follows ``tvm/llama_auto_batcher/compile_tvm.py:106-112`` (stacked params,
    ``take`` by ``wids`` on axis 0), ``lora.py:20-24`` (``(x.A).B`` then
    ``* alpha/r`` *after* the matmuls) and ``tvm/custom/fuse_take_matmul.py:
    85-105`` (``out[b,s,n] = sum_k x[b,s,k] * W[idx[b],k,n]``).

    x [B,S,in]; p0 [N,in,r]; p1 [N,r,out]; wids [B].
    """
    wids = torch.as_tensor(wids, dtype=torch.long)
    u = torch.einsum("bsk,bkr->bsr", x, p0[wids])
    y = torch.einsum("bsr,brn->bsn", u, p1[wids])
    return y * scaling


def write_tensor_part(x, y, ids):
    """``Z = X; Z[ids[a]] = Y[a]`` -- ``tvm/custom/write_tensor_part.py:11-20``."""
    z = x.clone()
    for a, b in enumerate(ids):
        z[int(b)] = y[a]
    return z


def mixed_type_lora_delta(h, out_features, type_args):
    """LoRA delta of a batch that mixes adapter types.

    Follows ``tvm/llama_auto_batcher/compile_tvm.py:135-155``: start from
    zeros; for each type gather its rows ``take(h, sids)``, run that type's
    adapter with ``wids`` and scatter the rows back with ``write_tensor_part``.
    ``type_args`` is a list of ``(sids, wids, p0, p1, scaling)``.
    """
    delta = torch.zeros(h.shape[0], h.shape[1], out_features, dtype=h.dtype)
    for sids, wids, p0, p1, scaling in type_args:
        sids_t = torch.as_tensor(sids, dtype=torch.long)
        h_l = h[sids_t]
        d_l = take_matmul_lora(h_l, p0, p1, wids, scaling)
        delta = write_tensor_part(delta, d_l, sids)
    return delta


def multi_lora_linear(x, weight, A_all, B_all, ranks, scales, slots):
    """Row-wise ``y = x W^T + scale[s] * (x A[s]^T) B[s]^T`` for a flat batch.

    The flat-token form of the two functions above (they are equal in exact
    arithmetic; the scale is applied after the matmuls as in ``lora.py:23-24``).
    x [T,in]; weight [out,in]; A_all [N,r_max,in]; B_all [N,out,r_max];
    ranks[N]; scales[N]; slots[T] (``-1`` = no adapter).
    """
    y = x @ weight.t()
    for t in range(x.shape[0]):
        s = int(slots[t])
        if s < 0:
            continue
        r = int(ranks[s])
        u = A_all[s, :r] @ x[t]
        y[t] += scales[s] * (B_all[s, :, :r] @ u)
    return y


# --------------------------------------------------------------------------
# decoder body pieces (tvm/llama_auto_batcher/llama_for_causal_lm.py)
# --------------------------------------------------------------------------
def rmsnorm(x, w, eps):
    """``nn.RMSNorm(hidden, -1, eps, bias=False)`` -- llama_for_causal_lm.py:76-77,93."""
    xf = x.float()
    var = xf.pow(2).mean(-1, keepdim=True)
    return xf * torch.rsqrt(var + eps) * w.float()


def silu_mul(g, u):
    """``silu(gate) * up`` -- llama_for_causal_lm.py:36."""
    return torch.nn.functional.silu(g.float()) * u.float()


def rope_rotate_half(x, positions, theta):
    """Rotary embedding over the whole head (rotary_dim = head_dim, scale 1).

    The cache is created with ``rope_mode=INLINE, rope_scale=1,
    rope_theta=theta, rotary_dim=head_dim`` (llama_for_causal_lm.py:155-174);
    pairing is the Llama "rotate half" convention (dimension ``i`` pairs with
    ``i + d/2``), the same one transformers' Llama uses.
    x [T,H,D]; positions [T].
    """
    d = x.shape[-1]
    inv = theta ** (-torch.arange(0, d, 2, dtype=torch.float32) / d)
    ang = positions.float()[:, None] * inv[None, :]
    cos = torch.cos(ang)[:, None, :]
    sin = torch.sin(ang)[:, None, :]
    x1, x2 = x.float()[..., : d // 2], x.float()[..., d // 2:]
    return torch.cat([x1 * cos - x2 * sin, x2 * cos + x1 * sin], dim=-1)


def paged_gather(pages, block_table_row, n_tokens):
    """Gather ``n_tokens`` of one sequence out of paged storage.

    pages [n_pages, H, page_size, D]; block_table_row: page ids of the
    sequence in order.  Returns [n_tokens, H, D].
    """
    page_size = pages.shape[2]
    n_pg = (n_tokens + page_size - 1) // page_size
    idx = torch.as_tensor(block_table_row[:n_pg], dtype=torch.long)
    g = pages[idx]  # [n_pg, H, ps, D]
    g = g.permute(0, 2, 1, 3).reshape(n_pg * page_size, pages.shape[1], pages.shape[3])
    return g[:n_tokens]


def paged_attention_decode(q, k_pages, v_pages, block_table, seq_lens):
    """Single-query attention over a paged KV cache (keys already rotated).

    What ``paged_kv_cache.attention_with_fused_qkv`` computes for append
    length 1 (llama_for_causal_lm.py:55-64): softmax(q k^T / sqrt(d)) v over
    the pages listed in the block table.
    q [B,Hq,D]; pages [n_pages,Hkv,ps,D]; block_table [B,max_pages];
    seq_lens[B] = number of valid tokens (including the one just appended).
    """
    B, Hq, D = q.shape
    Hkv = k_pages.shape[1]
    rep = Hq // Hkv
    out = torch.zeros(B, Hq, D, dtype=torch.float32)
    for b in range(B):
        n = int(seq_lens[b])
        k = paged_gather(k_pages, block_table[b], n).float()
        v = paged_gather(v_pages, block_table[b], n).float()
        k = k.repeat_interleave(rep, dim=1)
        v = v.repeat_interleave(rep, dim=1)
        s = torch.einsum("hd,nhd->hn", q[b].float(), k) / math.sqrt(D)
        p = torch.softmax(s, dim=-1)
        out[b] = torch.einsum("hn,nhd->hd", p, v)
    return out


def causal_attention(q, k, v):
    """Dense causal attention for one sequence (prefill): q,k,v [S,H,D]."""
    S, Hq, D = q.shape
    rep = Hq // k.shape[1]
    k = k.float().repeat_interleave(rep, dim=1)
    v = v.float().repeat_interleave(rep, dim=1)
    s = torch.einsum("shd,nhd->hsn", q.float(), k) / math.sqrt(D)
    mask = torch.ones(S, S, dtype=torch.bool).tril()
    s = s.masked_fill(~mask[None], float("-inf"))
    p = torch.softmax(s, dim=-1)
    return torch.einsum("hsn,nhd->shd", p, v)
