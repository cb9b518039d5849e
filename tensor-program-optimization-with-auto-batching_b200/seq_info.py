"""``LlamaSeqInfo`` with the bucketing done on the device.

Same methods and return values as the reference's host class
(``tvm/llama_auto_batcher/llama_seq_info.py``): per-sequence adapter / type /
generation-length table, ``order_seqs`` (stable sort of a batch: no-adapter
rows first, then adapter type id, then weight id, ``:61-75``) and
``get_decode_method`` (per-type position / weight-id lists and the name of the
decode function to call, ``:77-104``).  The integer work runs in
``mlora_bucket_sort`` on the GPU.  The reference-named methods copy the results
back and return the reference's Python lists (a synchronising call: the
executor's device-resident decode loop makes it once per fused decode node, to
put the batch in adapter order; after that the per-step regrouping the
reference does on the host is the stable compaction inside
``mlora_decode_step_begin``).  The ``*_device`` variants leave the results on
the device for callers that gather by ``perm`` there.
"""
from __future__ import annotations

import numpy as np
import torch

from . import ops


class LlamaSeqInfo:
    def __init__(self, max_gen_len, device="cuda"):
        self.sid_2_info = {}  # sid -> {"adapter": {"tid", "wid"} | None, "max_gen_len"}
        self.adapter_types = []
        self.max_gen_len = max_gen_len
        self.device = torch.device(device)

    # ---- bookkeeping: identical to the reference ---------------------------------------------------------
    def add_sequence(self, sid):
        assert sid not in self.sid_2_info, f"sequence with id {sid} has already been added"
        self.sid_2_info[sid] = {"adapter": None, "max_gen_len": self.max_gen_len}

    def set_max_gen_len(self, sid, max_gen_len):
        if max_gen_len is None:
            max_gen_len = self.max_gen_len
        if max_gen_len > self.max_gen_len:
            print(f"[WARN] you are trying to set a max_gen_len of {max_gen_len} for sequence {sid} which is bigger "
                  f"than the maximum {self.max_gen_len}. Setting max_gen_len to {self.max_gen_len}.")
            max_gen_len = self.max_gen_len
        self.sid_2_info[sid]["max_gen_len"] = max_gen_len

    def set_adapter(self, sid, config, wid):
        try:
            tid = self.adapter_types.index(config)
        except ValueError:
            tid = len(self.adapter_types)
            self.adapter_types.append(config)
        adapter = {"tid": tid, "wid": wid}
        if self.sid_2_info[sid]["adapter"] is not None:
            print(f"[WARN] you are setting adapter {adapter} for sequence {sid} but it has already been set to "
                  f"{self.sid_2_info[sid]['adapter']}")
        self.sid_2_info[sid]["adapter"] = adapter

    def get_adapter_configs(self):
        return self.adapter_types

    def get_wids_per_type(self):
        out = [set() for _ in self.adapter_types]
        for e in self.sid_2_info.values():
            if e["adapter"] is not None:
                out[e["adapter"]["tid"]].add(e["adapter"]["wid"])
        return out

    def get_num_adapters_per_type(self):
        return [len(s) for s in self.get_wids_per_type()]

    def get_num_sequences(self):
        return len(self.sid_2_info)

    def update_max_gen_len(self, max_gen_len):
        self.max_gen_len = max_gen_len

    def get_max_gen_len(self, sid):
        return self.sid_2_info[sid]["max_gen_len"]

    def get_adapter_info(self, sid):
        return self.sid_2_info[sid]["adapter"]

    # ---- bucketing on the device ---------------------------------------------------------------------------
    def _ids(self, sids):
        tids = np.array([-1 if self.sid_2_info[s]["adapter"] is None else self.sid_2_info[s]["adapter"]["tid"]
                         for s in sids], dtype=np.int32)
        wids = np.array([-1 if self.sid_2_info[s]["adapter"] is None else self.sid_2_info[s]["adapter"]["wid"]
                         for s in sids], dtype=np.int32)
        return tids, wids

    def _n_wids(self):
        hi = 0
        for e in self.sid_2_info.values():
            if e["adapter"] is not None:
                hi = max(hi, e["adapter"]["wid"])
        return hi + 1

    def order_seqs_device(self, sids):
        """Device-resident result: ``Buckets`` (perm, sorted tid/wid, segment table, counts)."""
        tids, wids = self._ids(sids)
        return ops.bucket_sort(torch.from_numpy(tids).to(self.device), torch.from_numpy(wids).to(self.device),
                               len(self.adapter_types), self._n_wids(), by_type_only=False)

    def order_seqs(self, sids):
        sids = list(sids)
        if len(self.adapter_types) == 0:
            return sids, [i for i in range(len(sids))]
        perm = self.order_seqs_device(sids).perm.cpu().tolist()
        return [sids[p] for p in perm], perm

    def decode_method_device(self, sids):
        tids, wids = self._ids(sids)
        return ops.bucket_sort(torch.from_numpy(tids).to(self.device), torch.from_numpy(wids).to(self.device),
                               len(self.adapter_types), self._n_wids(), by_type_only=True)

    def get_decode_method(self, sids):
        n_types = len(self.adapter_types)
        if n_types == 0:
            return "decode_no_adapter", []
        b = self.decode_method_device(sids)
        counts = b.counts.cpu().tolist()
        perm, swid = b.perm.cpu().tolist(), b.sorted_wid.cpu().tolist()
        non_empty = [t for t in range(n_types) if counts[2 + t] > 0]
        no_adapter = counts[1] > 0
        if no_adapter and not non_empty:
            return "decode_no_adapter", []
        if not no_adapter and len(non_empty) == 1:
            return f"decode_a{non_empty[0]}", [swid]
        name = "mixed_decode_" + "_".join(f"a{t}" for t in non_empty)
        params, off = [], counts[1]
        for t in range(n_types):
            c = counts[2 + t]
            if c:
                params += [perm[off:off + c], swid[off:off + c]]
            off += c
        return name, params
