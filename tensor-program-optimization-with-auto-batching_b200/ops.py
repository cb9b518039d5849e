"""Operator wrappers: torch CUDA tensors in, C-ABI calls on the current stream.

torch is used for device memory and streams only; every computation below
happens inside ``libmlora.so``.
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass

import torch

from . import _lib
from ._lib import check

OUT_F32, SILU_MUL, FORCE_SIMT, W_PACKED, B_PACKED, SHARE_LORA_KERNEL, LORA_PER_ROW, B_SPLIT = 1, 2, 4, 8, 16, 32, 64, 128


def _ptr(t):
    return None if t is None else C.c_void_p(t.data_ptr())


def _stream():
    return C.c_void_p(torch.cuda.current_stream().cuda_stream)


def _need_cuda(*ts):
    for t in ts:
        if t is not None and not t.is_cuda:
            raise ValueError("mlora operators need CUDA tensors (there is no CPU path)")


_workspaces = {}
_retired = []  # outgrown buffers stay alive: a captured CUDA graph may still hold their address


def workspace(nbytes: int, device, tag="default"):
    """The fallback scratch buffer of calls that bring none: one per (device, current stream, tag), grown
    on demand, never freed.  Zero-filled when created: the split-K arrival counters of ``mlora_linear``
    must start at zero (they reset themselves).  Long-lived users (``model.Engine``) own their scratch
    and pass it with ``work=`` instead."""
    dev = torch.device(device)
    idx = dev.index if dev.index is not None else torch.cuda.current_device()
    key = (idx, torch.cuda.current_stream(idx).cuda_stream, tag)
    buf = _workspaces.get(key)
    if buf is None or buf.numel() < nbytes:
        if buf is not None:
            _retired.append(buf)
        buf = torch.zeros(max(int(nbytes), 256), dtype=torch.uint8, device=device)
        _workspaces[key] = buf
    return buf


def new_workspace(nbytes: int, device):
    """A zero-filled scratch buffer owned by the caller (see ``mlora_linear`` for the zero-fill rule)."""
    return torch.zeros(max(int(nbytes), 256), dtype=torch.uint8, device=device)


def status_word(work) -> int:
    """The status word at the start of a projection scratch buffer (0 = no bounded wait ever expired)."""
    return int(work[:4].view(torch.int32).item())


# ---------------------------------------------------------------- bucketing
@dataclass
class Buckets:
    perm: torch.Tensor          # [n] int32
    sorted_tid: torch.Tensor    # [n] int32
    sorted_wid: torch.Tensor    # [n] int32
    seg_offsets: torch.Tensor   # [n_keys+1] int32 (first n_seg+1 valid)
    seg_tid: torch.Tensor       # [n_keys]
    seg_wid: torch.Tensor       # [n_keys]
    counts: torch.Tensor        # [n_types+2]: n_seg, rows without adapter, rows per type


def bucket_sort(tids, wids, n_types: int, n_wids: int, by_type_only: bool = False) -> Buckets:
    _need_cuda(tids, wids)
    n = wids.numel()
    dev = wids.device
    nt = max(n_types, 1) if tids is None else n_types
    n_keys = nt + 1 if by_type_only else 1 + nt * n_wids
    i32 = dict(dtype=torch.int32, device=dev)
    out = Buckets(torch.empty(n, **i32), torch.empty(n, **i32), torch.empty(n, **i32),
                  torch.zeros(n_keys + 1, **i32), torch.full((n_keys,), -2, **i32),
                  torch.full((n_keys,), -2, **i32), torch.zeros(nt + 2, **i32))
    wb = _lib.lib().mlora_bucket_sort_workspace(n, nt, n_wids)
    ws = workspace(wb, dev, "bucket") if wb else None
    check(_lib.lib().mlora_bucket_sort(
        _ptr(tids), _ptr(wids), n, n_types, n_wids, int(by_type_only), _ptr(out.perm), _ptr(out.sorted_tid),
        _ptr(out.sorted_wid), _ptr(out.seg_offsets), _ptr(out.seg_tid), _ptr(out.seg_wid), _ptr(out.counts),
        _ptr(ws), wb, _stream()), "mlora_bucket_sort")
    return out


# ---------------------------------------------------------------- LoRA + projection
@dataclass
class LoraStack:
    """Packed adapters of one (fused) projection.

    A_all [N, n_mod*r_max, in] bf16, B_all [N, out, r_max] bf16 (module m of
    adapter s uses rows m*r_max.. of A and its own rows of B; for an interleaved
    gate/up stack B_all is [N, out, 2*r_max] with the other module's half zero),
    r_max a multiple of 8 (16, 32 or 64 for the tensor-core expand), padding
    beyond an adapter's rank zero, ranks [N] int32,
    scales [N] float32 (alpha/r), mod_offsets: host list of n_mod+1 output-row
    offsets.
    """
    A_all: torch.Tensor
    B_all: torch.Tensor
    ranks: torch.Tensor
    scales: torch.Tensor
    r_max: int
    n_mod: int = 1
    mod_offsets: tuple = None
    b_packed: bool = False   # B_all holds the tiled layout of mlora_pack_lora_b (uint8 buffer)
    n_out: int = 0           # output features (needed once B_all is packed)
    B_split: torch.Tensor = None   # rank-compact copy for the per-row expand: [slices, out, 8] bf16 (see split_b)
    rank_tbl: torch.Tensor = None  # int32 [2N]: ranks (rounded up to 8), then each adapter's first slice

    def split_b(self, ranks_host):
        """Builds the rank-compact "split" layout from the row-major B_all (call BEFORE pack_b): adapter s becomes
        ceil(rank[s] / 8) slices [out, 8], stored one after the other; a table gives each adapter's first slice.
        The per-row expand (``LORA_PER_ROW``) then reads rank * out * 2 bytes per row and nothing else."""
        if self.b_packed:
            raise ValueError("split_b needs the row-major B_all (call it before pack_b)")
        N, out, pitch = self.B_all.shape
        n_sl = [-(-int(r) // 8) for r in ranks_host]
        first = [0]
        for n in n_sl:
            first.append(first[-1] + n)
        dev = self.B_all.device
        if first[-1] == 0:
            return self
        idx_slot = torch.tensor([s for s, n in enumerate(n_sl) for _ in range(n)], device=dev)
        idx_sl = torch.tensor([j for n in n_sl for j in range(n)], device=dev)
        B5 = self.B_all.view(N, out, pitch // 8, 8)
        self.B_split = B5[idx_slot, :, idx_sl, :].contiguous()            # [slices, out, 8]
        self.rank_tbl = torch.tensor([8 * n for n in n_sl] + first[:-1], dtype=torch.int32, device=dev)
        return self

    def pack_b(self, interleaved: bool = False):
        """Replace B_all by its pre-tiled form (tensor-core expand only; modules must be tile aligned)."""
        if self.b_packed:
            return self
        N, out, pitch = self.B_all.shape
        n = _lib.lib().mlora_packed_lora_b_bytes(N, out, pitch)
        buf = torch.empty(n, dtype=torch.uint8, device=self.B_all.device)
        check(_lib.lib().mlora_pack_lora_b(_ptr(self.B_all), N, out, pitch, _ptr(buf), _stream()), "mlora_pack_lora_b")
        self.B_all, self.b_packed, self.n_out = buf, True, out
        return self


def _write_b_slot(self, slot: int, B_one):
    """Replace one adapter's rows of B_all (``B_one`` [out, pitch] bf16, or None = zeros), packed or not."""
    if not self.b_packed:
        if B_one is None:
            self.B_all[slot].zero_()
        else:
            self.B_all[slot].copy_(B_one)
        return
    N = self.A_all.shape[0]
    per = self.B_all.numel() // N  # bytes of one slot: tiles are laid out slot-major
    region = self.B_all[slot * per:(slot + 1) * per]
    if B_one is None:
        region.zero_()
        return
    out, pitch = B_one.shape
    assert _lib.lib().mlora_packed_lora_b_bytes(1, out, pitch) == per
    check(_lib.lib().mlora_pack_lora_b(_ptr(B_one.contiguous()), 1, out, pitch, _ptr(region), _stream()), "mlora_pack_lora_b")


LoraStack.write_b_slot = _write_b_slot


def lora_shrink(x, stack: LoraStack, slots, out=None):
    _need_cuda(x, slots)
    T, K = x.shape
    r_tot = stack.r_max * stack.n_mod
    u = out if out is not None else torch.empty(T, r_tot, dtype=torch.float32, device=x.device)
    check(_lib.lib().mlora_lora_shrink(_ptr(x), x.stride(0), _ptr(stack.A_all), _ptr(stack.ranks), _ptr(slots),
                                       stack.A_all.shape[0], T, K, stack.r_max, stack.n_mod, _ptr(u), _stream()), "mlora_lora_shrink")
    return u


class PackedWeight:
    """W [out,in] in the tiled layout of ``mlora_pack_weight`` (see include/mlora.h)."""

    def __init__(self, W):
        _need_cuda(W)
        if W.dtype != torch.bfloat16 or not W.is_contiguous():
            raise ValueError("PackedWeight needs a contiguous bf16 matrix")
        self.shape = tuple(W.shape)
        self.dtype = W.dtype
        n = _lib.lib().mlora_packed_weight_bytes(W.shape[0], W.shape[1])
        self.data = torch.empty(n, dtype=torch.uint8, device=W.device)
        check(_lib.lib().mlora_pack_weight(_ptr(W), W.shape[0], W.shape[1], _ptr(self.data), _stream()),
              "mlora_pack_weight")

    def data_ptr(self):
        return self.data.data_ptr()

    def numel(self):
        return self.shape[0] * self.shape[1]

    @property
    def is_cuda(self):
        return True


def linear(x, W, stack: LoraStack = None, slots=None, u=None, flags: int = 0, out=None, use_workspace=True,
           with_shrink=False, work=None):
    """y = x W^T (+ LoRA expand of ``u``) ; see ``mlora_linear`` in include/mlora.h.
    ``W`` is a bf16 [out,in] tensor or a :class:`PackedWeight`.  ``with_shrink``: ``u`` is scratch and
    the shrink is part of the call (``mlora_lora_linear``).  ``work``: the caller's own zero-initialised
    scratch buffer (default: the per-stream fallback buffer)."""
    _need_cuda(x, W)
    if x.dtype != torch.bfloat16 or W.dtype != torch.bfloat16:
        raise ValueError("mlora.linear needs bf16 x and W")
    if isinstance(W, PackedWeight):
        flags |= W_PACKED
    split = stack is not None and bool(flags & LORA_PER_ROW) and stack.B_split is not None and not flags & SILU_MUL
    if stack is not None and stack.b_packed and not split:
        flags |= B_PACKED
    if split:
        flags |= B_SPLIT
    T, K = x.shape
    N = W.shape[0]
    cols = N // 2 if flags & SILU_MUL else N
    if out is None:
        out = torch.empty(T, cols, dtype=torch.float32 if flags & OUT_F32 else torch.bfloat16, device=x.device)
    mod = None
    if stack is not None and u is None:
        if with_shrink:
            u = torch.empty(T, stack.r_max * stack.n_mod, dtype=torch.float32, device=x.device)
        else:
            u = lora_shrink(x, stack, slots)
    if stack is not None and stack.n_mod > 1 and not flags & SILU_MUL:
        mod = (C.c_int32 * (stack.n_mod + 1))(*stack.mod_offsets)
    wb = _lib.lib().mlora_linear_workspace_flags(T, K, N, flags if stack is not None else 0) if use_workspace else 0
    if work is not None and wb:
        if work.numel() < wb:
            raise ValueError(f"mlora.linear: scratch of {wb} bytes needed, {work.numel()} given")
        ws, wb = work, work.numel()
    else:
        ws = workspace(wb, x.device, "linear") if wb else None
    if stack is not None and with_shrink:
        check(_lib.lib().mlora_lora_linear(
            _ptr(x), x.stride(0), _ptr(W), _ptr(out), out.stride(0), T, K, N, _ptr(stack.A_all), _ptr(u),
            _ptr(stack.B_all), _ptr(stack.ranks), _ptr(stack.scales), _ptr(slots), stack.A_all.shape[0],
            stack.r_max, stack.n_mod, mod, flags, _ptr(ws), wb, _stream()), "mlora_lora_linear")
        return out
    check(_lib.lib().mlora_linear(
        _ptr(x), x.stride(0), _ptr(W), _ptr(out), out.stride(0), T, K, N,
        _ptr(u) if stack is not None else None,
        (_ptr(stack.B_split) if split else _ptr(stack.B_all)) if stack is not None else None,
        (_ptr(stack.rank_tbl) if split else _ptr(stack.ranks)) if stack is not None else None,
        _ptr(stack.scales) if stack is not None else None,
        _ptr(slots) if stack is not None else None, stack.A_all.shape[0] if stack is not None else 0,
        stack.r_max if stack is not None else 0,
        stack.n_mod if stack is not None else 1, mod, flags, _ptr(ws), wb, _stream()), "mlora_linear")
    return out


def linear_norm(x, W, stack: LoraStack = None, slots=None, u=None, flags: int = 0, out=None, work=None, res=None,
                norm_w=None, sumsq_out=None, sumsq_in=None, n_sumsq_in=0, eps=0.0, norm_dim=0):
    """``mlora_linear_norm``: a decode-size projection (T <= 32) that takes part in a folded residual add + RMSNorm.
    Producer (``res``, ``norm_w``, ``sumsq_out``): res += y; out = bf16(res * norm_w) and per-128-output sums of
    squares; consumer (``sumsq_in``, ``n_sumsq_in``, ``eps``, ``norm_dim``): output rows scaled by their input
    rows' 1/rms before the activation.  ``u`` must already hold the shrink outputs when ``stack`` is given."""
    _need_cuda(x, W)
    if isinstance(W, PackedWeight):
        flags |= W_PACKED
    if stack is not None and stack.b_packed:
        flags |= B_PACKED
    T, K = x.shape
    N = W.shape[0]
    cols = N // 2 if flags & SILU_MUL else N
    if out is None:
        out = torch.empty(T, cols, dtype=torch.float32 if flags & OUT_F32 else torch.bfloat16, device=x.device)
    if stack is not None and u is None:
        raise ValueError("mlora.linear_norm: pass the shrink outputs u")
    mod = None
    if stack is not None and stack.n_mod > 1 and not flags & SILU_MUL:
        mod = (C.c_int32 * (stack.n_mod + 1))(*stack.mod_offsets)
    wb = _lib.lib().mlora_linear_workspace(T, K, N)
    if work is not None:
        if work.numel() < wb:
            raise ValueError(f"mlora.linear_norm: scratch of {wb} bytes needed, {work.numel()} given")
        ws, wb = work, work.numel()
    else:
        ws = workspace(wb, x.device, "linear")
    if res is not None and (res.dtype != torch.float32 or sumsq_out is None or sumsq_out.numel() < -(-N // 128) * 32):
        raise ValueError("mlora.linear_norm: res must be fp32 and sumsq_out hold ceil(out/128)*32 floats")
    check(_lib.lib().mlora_linear_norm(
        _ptr(x), x.stride(0), _ptr(W), _ptr(out), out.stride(0), T, K, N,
        _ptr(u) if stack is not None else None, _ptr(stack.B_all) if stack is not None else None,
        _ptr(stack.ranks) if stack is not None else None, _ptr(stack.scales) if stack is not None else None,
        _ptr(slots) if stack is not None else None, stack.A_all.shape[0] if stack is not None else 0,
        stack.r_max if stack is not None else 0, stack.n_mod if stack is not None else 1, mod, flags, _ptr(ws), wb,
        _ptr(res), res.stride(0) if res is not None else 0, _ptr(norm_w), _ptr(sumsq_out), _ptr(sumsq_in),
        int(n_sumsq_in), float(eps), int(norm_dim), _stream()), "mlora_linear_norm")
    return out


# ---------------------------------------------------------------- chained decode projections
@dataclass
class ChainStep:
    """One phase of :func:`decode_chain`: optional residual add + RMSNorm writing ``x``, optional LoRA shrink
    of ``x`` into ``u``, then ``y = x W^T`` (+ expand).  ``W`` must be a :class:`PackedWeight`, ``stack`` a
    :class:`LoraStack` with a packed B."""
    x: torch.Tensor
    W: "PackedWeight"
    y: torch.Tensor
    flags: int = 0
    res: torch.Tensor = None      # fp32 [T,in]: res += delta; x = RMSNorm(res) * norm_w
    delta: torch.Tensor = None
    norm_w: torch.Tensor = None
    eps: float = 0.0
    stack: "LoraStack" = None
    u: torch.Tensor = None


def chain_supported(T: int, steps) -> bool:
    """Can these phases run as one ``mlora_decode_chain`` launch?  (decode-size batch, packed operands, tensor-core
    expand, norm inputs up to 8192 wide)"""
    if not (0 < T <= 32 and 1 <= len(steps) <= _lib.CHAIN_MAX_PHASES):
        return False
    for st in steps:
        if not isinstance(st.W, PackedWeight) or st.x.stride(0) % 8 or st.W.shape[1] % 8:
            return False
        if st.res is not None and (st.W.shape[1] > 8192 or st.x.stride(0) != st.W.shape[1]):
            return False
        if st.stack is not None:
            k = st.stack
            pitch = 2 * k.r_max if st.flags & SILU_MUL else k.r_max
            if not k.b_packed or pitch not in (16, 32, 64, 128) or k.n_mod > 4:
                return False
            if not st.flags & SILU_MUL and k.n_mod > 1 and any(o % 128 for o in k.mod_offsets[1:-1]):
                return False
    return True


def decode_chain(steps, slots, ranks, scales, n_adapters: int, work):
    """Up to six dependent projections (with the row operations between them) in one persistent launch;
    see ``mlora_decode_chain`` in include/mlora.h.  ``work``: zero-initialised scratch as for :func:`linear`."""
    n = len(steps)
    arr = (_lib.ChainPhase * n)()
    T = steps[0].x.shape[0]
    for i, st in enumerate(steps):
        _need_cuda(st.x, st.y)
        ph = arr[i]
        ph.d_x, ph.ldx, ph.d_Wp = st.x.data_ptr(), st.x.stride(0), st.W.data_ptr()
        ph.d_y, ph.ldy = st.y.data_ptr(), st.y.stride(0)
        ph.in_, ph.out, ph.flags, ph.eps = st.W.shape[1], st.W.shape[0], st.flags, st.eps
        ph.d_res = st.res.data_ptr() if st.res is not None else None
        ph.d_delta = st.delta.data_ptr() if st.delta is not None else None
        ph.d_norm_w = st.norm_w.data_ptr() if st.norm_w is not None else None
        if st.stack is not None:
            k = st.stack
            ph.d_A_all, ph.d_u, ph.d_Bp = k.A_all.data_ptr(), st.u.data_ptr(), k.B_all.data_ptr()
            ph.r_max, ph.n_mod = k.r_max, k.n_mod
            if k.n_mod > 1 and k.mod_offsets is not None:
                for m, o in enumerate(k.mod_offsets):
                    ph.mod_offsets[m] = o
        else:
            ph.d_A_all = ph.d_u = ph.d_Bp = None
            ph.r_max, ph.n_mod = 0, 1
    check(_lib.lib().mlora_decode_chain(arr, n, T, _ptr(slots), _ptr(ranks), _ptr(scales), n_adapters, _ptr(work),
                                        work.numel(), _stream()), "mlora_decode_chain")


# ---------------------------------------------------------------- row ops
def residual_rmsnorm(delta, res, w, eps: float, out=None):
    _need_cuda(res, w)
    T, H = res.shape
    if out is None:
        out = torch.empty(T, H, dtype=torch.bfloat16, device=res.device)
    check(_lib.lib().mlora_residual_rmsnorm(_ptr(delta), _ptr(res), _ptr(w), eps, _ptr(out), T, H, _stream()),
          "mlora_residual_rmsnorm")
    return out


def residual_rmsnorm_shrink(delta, res_in, res_out, w, eps: float, out, stack: LoraStack, slots, u):
    """Fused residual add + RMSNorm + LoRA shrink of the projection that reads ``out`` (see include/mlora.h)."""
    _need_cuda(res_in, w)
    T, H = res_in.shape
    check(_lib.lib().mlora_residual_rmsnorm_shrink(
        _ptr(delta), _ptr(res_in), _ptr(res_out), _ptr(w), eps, _ptr(out), T, H, _ptr(stack.A_all), _ptr(slots),
        stack.A_all.shape[0], stack.r_max * stack.n_mod, _ptr(u), _stream()), "mlora_residual_rmsnorm_shrink")
    return out


def embed(ids, E, res=None, out_bf16=None):
    _need_cuda(ids, E)
    T = ids.numel()
    V, H = E.shape
    if res is None and out_bf16 is None:
        res = torch.empty(T, H, dtype=torch.float32, device=E.device)
    check(_lib.lib().mlora_embed(_ptr(ids), _ptr(E), T, H, V, _ptr(res), _ptr(out_bf16), _stream()), "mlora_embed")
    return res if res is not None else out_bf16


def argmax(logits, out=None):
    _need_cuda(logits)
    T, V = logits.shape
    if out is None:
        out = torch.empty(T, dtype=torch.int32, device=logits.device)
    check(_lib.lib().mlora_argmax(_ptr(logits), logits.stride(0), T, V, _ptr(out), _stream()), "mlora_argmax")
    return out


# ---------------------------------------------------------------- paged KV
def kv_append_rope(qkv, k_pages, v_pages, block_table, row_slot, row_pos, Hq, Hkv, D, page_size, theta):
    _need_cuda(qkv, k_pages)
    T = qkv.shape[0]
    check(_lib.lib().mlora_kv_append_rope(
        _ptr(qkv), qkv.stride(0), _ptr(k_pages), _ptr(v_pages), _ptr(block_table), block_table.shape[1],
        _ptr(row_slot), _ptr(row_pos), T, Hq, Hkv, D, page_size, theta, _stream()), "mlora_kv_append_rope")


def paged_attention(qkv, k_pages, v_pages, block_table, row_slot, row_pos, Hq, Hkv, D, page_size, theta,
                    fused_append: bool, out=None, n_splits: int = 0, work=None):
    _need_cuda(qkv, k_pages)
    T = qkv.shape[0]
    if out is None:
        out = torch.empty(T, Hq * D, dtype=torch.bfloat16, device=qkv.device)
    if work is not None:
        ws, wb = work, work.numel()
    else:
        wb = _lib.lib().mlora_paged_attention_workspace(T, Hq, D, n_splits)
        ws = workspace(wb, qkv.device, "attn") if wb else None
    check(_lib.lib().mlora_paged_attention(
        _ptr(qkv), qkv.stride(0), _ptr(k_pages), _ptr(v_pages), _ptr(block_table), block_table.shape[1],
        _ptr(row_slot), _ptr(row_pos), T, Hq, Hkv, D, page_size, theta, int(fused_append), _ptr(out),
        out.stride(0), n_splits, _ptr(ws), wb, _stream()), "mlora_paged_attention")
    return out


def prefill_attention(qkv, k_pages, v_pages, block_table, tiles, n_tiles, Hq, Hkv, D, page_size, out, status=None):
    """Causal attention of prompt rows on the tensor cores (``mlora_prefill_attention``); ``tiles`` int32 [n,4] on the
    device: (cache slot, first row, rows <= 128, position of the first row)."""
    _need_cuda(qkv, k_pages)
    check(_lib.lib().mlora_prefill_attention(
        _ptr(qkv), qkv.stride(0), _ptr(k_pages), _ptr(v_pages), k_pages.shape[0], _ptr(block_table), block_table.shape[1],
        _ptr(tiles), n_tiles, Hq, Hkv, D, page_size, qkv.shape[0], _ptr(out), out.stride(0), _ptr(status), _stream()),
        "mlora_prefill_attention")
    return out


def attention_shrink_fits(T, Hq, max_pages, stack) -> bool:
    """Can the o-projection's shrink ride in the attention launch?  (one CTA per (row, head), one module)"""
    return stack.n_mod == 1 and _lib.lib().mlora_paged_attention_splits(T, Hq, max_pages) == 1


def paged_attention_shrink(qkv, k_pages, v_pages, block_table, row_slot, row_pos, Hq, Hkv, D, page_size, theta,
                           fused_append: bool, out, stack: LoraStack, slots, u, work):
    """Attention plus, in the same launch, ``u = A[slot] . out`` for the projection that reads ``out``
    (see ``mlora_paged_attention_shrink``).  ``work``: zero-initialised scratch of
    ``mlora_paged_attention_shrink_workspace`` bytes owned by the caller."""
    _need_cuda(qkv, k_pages)
    T = qkv.shape[0]
    check(_lib.lib().mlora_paged_attention_shrink(
        _ptr(qkv), qkv.stride(0), _ptr(k_pages), _ptr(v_pages), _ptr(block_table), block_table.shape[1],
        _ptr(row_slot), _ptr(row_pos), T, Hq, Hkv, D, page_size, theta, int(fused_append), _ptr(out), out.stride(0),
        _ptr(stack.A_all), _ptr(stack.ranks), _ptr(slots), stack.A_all.shape[0], stack.r_max, _ptr(u), _ptr(work),
        work.numel(), _stream()), "mlora_paged_attention_shrink")
    return out


def kv_begin_decode(row_slot, seq_lens, row_pos):
    check(_lib.lib().mlora_kv_begin_decode(_ptr(row_slot), _ptr(seq_lens), _ptr(row_pos), row_slot.numel(),
                                           _stream()), "mlora_kv_begin_decode")


def decode_step_begin(live, seq_slot, adapter_slot, last_tok, n_rows, seq_lens, row_src, row_slot, row_pos, row_adapter,
                      row_tok, n_live):
    check(_lib.lib().mlora_decode_step_begin(_ptr(live), _ptr(seq_slot), _ptr(adapter_slot), _ptr(last_tok), live.numel(),
                                             n_rows, _ptr(seq_lens), _ptr(row_src), _ptr(row_slot), _ptr(row_pos),
                                             _ptr(row_adapter), _ptr(row_tok), _ptr(n_live), _stream()),
          "mlora_decode_step_begin")


def decode_step_end(row_src, next_tok, n_rows, live, last_tok, gen_count, max_gen, out_tokens, eos_id, n_live):
    check(_lib.lib().mlora_decode_step_end(_ptr(row_src), _ptr(next_tok), n_rows, _ptr(live), _ptr(last_tok), _ptr(gen_count),
                                           _ptr(max_gen), _ptr(out_tokens), out_tokens.stride(0), eos_id, _ptr(n_live),
                                           _stream()), "mlora_decode_step_end")


def launch_count() -> int:
    return int(_lib.lib().mlora_launch_count())
