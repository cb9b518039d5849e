"""Paged KV cache: device pages + block tables, host-side page allocator.

Stands in for the object ``vm["create_paged_kv_cache"]`` returns and for the
``vm.builtin.kv_state_*`` functions the reference executor calls
(``tvm/llama_auto_batcher/llama_exec_graph.py:38-46,66,75-79,85,121-127``;
cache parameters ``tvm/llama_auto_batcher/llama_for_causal_lm.py:148-174``).

Layout in HBM: one tensor ``[n_layers, 2, n_pages, Hkv, page_size, D]`` bf16
(K pages then V pages of a layer), a block table ``[max_batch, max_pages]``
int32 and ``seq_lens [max_batch]`` int32.  Page ids are handed out by a host
free list; the device tables are refreshed with small async copies when they
change.  A decode step captured in a CUDA graph advances ``seq_lens`` on the
device itself (``mlora_kv_begin_decode``), so pages for the tokens a graph
will append must be reserved ahead with :meth:`reserve`.
"""
from __future__ import annotations

import numpy as np
import torch

from . import ops


class PagedKVCache:
    def __init__(self, n_layers, n_kv_heads, head_dim, max_batch, max_total_seq_len, prefill_chunk_size,
                 page_size, device, max_seq_len=None):
        if page_size not in (16, 32):
            raise ValueError("page_size must be 16 or 32")
        self.n_layers, self.Hkv, self.D = n_layers, n_kv_heads, head_dim
        self.max_batch, self.page_size = int(max_batch), int(page_size)
        self.prefill_chunk_size = int(prefill_chunk_size)
        self.device = torch.device(device)
        ps = self.page_size
        # every sequence may leave one page partly filled
        self.n_pages = (int(max_total_seq_len) + ps - 1) // ps + self.max_batch
        per_seq = int(max_seq_len) if max_seq_len else int(max_total_seq_len)
        self.max_pages = min((per_seq + ps - 1) // ps + 1, self.n_pages)
        self.pages = torch.zeros(n_layers, 2, self.n_pages, n_kv_heads, ps, head_dim, dtype=torch.bfloat16,
                                 device=self.device)
        self.block_table = torch.zeros(self.max_batch, self.max_pages, dtype=torch.int32, device=self.device)
        self.seq_lens = torch.zeros(self.max_batch, dtype=torch.int32, device=self.device)
        # host mirrors; device refreshes go through a fresh pinned staging tensor per copy, so a
        # later host-side update can never race with an asynchronous copy still in the stream
        self._bt_host = np.zeros((self.max_batch, self.max_pages), dtype=np.int32)
        self._len_host = np.zeros(self.max_batch, dtype=np.int32)
        self._free = list(range(self.n_pages - 1, -1, -1))
        self._slot_of = {}           # sid -> slot
        self._free_slots = list(range(self.max_batch - 1, -1, -1))
        self._n_pages_of = {}        # sid -> pages held
        self._pending = None

    # -- layer views -----------------------------------------------------------------------------
    def k_pages(self, layer):
        return self.pages[layer, 0]

    def v_pages(self, layer):
        return self.pages[layer, 1]

    # -- sequences -----------------------------------------------------------------------------
    def add_sequence(self, sid):
        if sid in self._slot_of:
            raise ValueError(f"sequence {sid} is already in the cache")
        if not self._free_slots:
            raise RuntimeError("no free sequence slot (max_batch reached)")
        slot = self._free_slots.pop()
        self._slot_of[sid] = slot
        self._n_pages_of[sid] = 0
        self._len_host[slot] = 0
        self._push(self.seq_lens[slot:slot + 1], self._len_host[slot:slot + 1])
        return slot

    def _push(self, dst, src_np):
        dst.copy_(torch.from_numpy(np.ascontiguousarray(src_np)).pin_memory(), non_blocking=True)

    def remove_sequence(self, sid):
        slot = self._slot_of.pop(sid)
        n = self._n_pages_of.pop(sid)
        self._free.extend(int(p) for p in self._bt_host[slot, :n].tolist()[::-1])
        self._free_slots.append(slot)

    def slot(self, sid):
        return self._slot_of[sid]

    def length(self, sid):
        return int(self._len_host[self._slot_of[sid]])

    def tokens_reserved(self, sid):
        """Tokens the pages held by ``sid`` have room for."""
        return self._n_pages_of[sid] * self.page_size

    def reserve(self, sid, n_tokens):
        """Make sure pages exist for ``n_tokens`` total tokens of sequence ``sid``."""
        slot = self._slot_of[sid]
        need = (int(n_tokens) + self.page_size - 1) // self.page_size
        have = self._n_pages_of[sid]
        if need <= have:
            return
        if need > self.max_pages:
            raise RuntimeError(f"sequence {sid} needs {need} pages, block table holds {self.max_pages}")
        if need - have > len(self._free):
            raise RuntimeError("paged KV cache is out of pages")
        for p in range(have, need):
            self._bt_host[slot, p] = self._free.pop()
        self._n_pages_of[sid] = need
        self._push(self.block_table[slot, have:need], self._bt_host[slot, have:need])

    # -- the reference's forward protocol -------------------------------------------------------------
    def begin_forward(self, seq_ids, append_lens):
        """Reserve pages for the rows of this forward and return (row_slot, row_pos) device tensors:
        one row per appended token, sequences in the order given."""
        seq_ids = [int(s) for s in seq_ids]
        append_lens = [int(a) for a in append_lens]
        slots, pos = [], []
        for sid, a in zip(seq_ids, append_lens):
            slot = self._slot_of[sid]
            n0 = int(self._len_host[slot])
            self.reserve(sid, n0 + a)
            slots.extend([slot] * a)
            pos.extend(range(n0, n0 + a))
        self._pending = (seq_ids, append_lens)
        row_slot = torch.tensor(slots, dtype=torch.int32).pin_memory().to(self.device, non_blocking=True)
        row_pos = torch.tensor(pos, dtype=torch.int32).pin_memory().to(self.device, non_blocking=True)
        return row_slot, row_pos

    def end_forward(self):
        seq_ids, append_lens = self._pending
        self._pending = None
        for sid, a in zip(seq_ids, append_lens):
            slot = self._slot_of[sid]
            self._len_host[slot] += a
        slots = sorted(self._slot_of[s] for s in seq_ids)
        lo, hi = slots[0], slots[-1] + 1
        self._push(self.seq_lens[lo:hi], self._len_host[lo:hi])

    def note_device_decode(self, seq_ids, n_steps=1):
        """Tell the host mirror that a captured decode step advanced these sequences on the device."""
        for sid in seq_ids:
            self._len_host[self._slot_of[int(sid)]] += n_steps

    # -- checks used by tests ---------------------------------------------------------------------
    def gather(self, sid, layer):
        """(K, V) of a sequence as dense [n, Hkv, D] tensors (block-table gather)."""
        slot = self._slot_of[sid]
        n = int(self._len_host[slot])
        ps = self.page_size
        n_pg = (n + ps - 1) // ps
        idx = torch.from_numpy(self._bt_host[slot, :n_pg].astype(np.int64)).to(self.device)
        out = []
        for kv in (0, 1):
            g = self.pages[layer, kv][idx].permute(0, 2, 1, 3).reshape(n_pg * ps, self.Hkv, self.D)
            out.append(g[:n])
        return out


# The three global functions of the reference's runtime, same names and argument order.
def kv_state_add_sequence(kv: PagedKVCache, sid):
    kv.add_sequence(int(sid))


def kv_state_begin_forward(kv: PagedKVCache, seq_ids, append_lens):
    kv._rows = kv.begin_forward(list(seq_ids), list(append_lens))


def kv_state_end_forward(kv: PagedKVCache):
    kv.end_forward()
    kv._rows = None
