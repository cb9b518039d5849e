"""CPU restatement of the auto-batcher's request->adapter bucketing.

TEST INFRASTRUCTURE ONLY (see ``oracle/__init__.py``).  Integer work: every
result here must be reproduced bit-exactly by the CUDA path.

A sequence's adapter is described by two integers: ``tid`` (adapter *type*,
i.e. index of its (rank, alpha) config) and ``wid`` (weight id inside that
type).  ``tid == -1`` means "no adapter".
"""
from __future__ import annotations

import numpy as np


def order_seqs(sids, tids, wids, n_types):
    """Stable sort of a batch by (has_adapter, tid, wid); no-adapter rows first.

    Follows ``tvm/llama_auto_batcher/llama_seq_info.py:61-75``: the reference
    sorts ``(i, sid, adapter, tid|inf, wid|inf)`` tuples with Python's stable
    ``sorted`` on key ``(adapter is not None, tid, wid)`` and returns
    ``(ordered_sids, original_positions)``.  With no adapter type registered
    at all the batch is returned unchanged (``:62-63``).
    """
    sids = list(sids)
    n = len(sids)
    if n_types == 0:
        return sids, list(range(n))
    keys = []
    for i in range(n):
        has = tids[i] >= 0
        keys.append((has, tids[i] if has else 0, wids[i] if has else 0, i))
    order = [k[3] for k in sorted(keys)]  # index as last key component == stable
    return [sids[i] for i in order], order


def get_decode_method(tids, wids, n_types):
    """Per-type position / weight-id lists and the compiled function name.

    Follows ``tvm/llama_auto_batcher/llama_seq_info.py:77-104``.  ``tids`` /
    ``wids`` describe the batch *in the order it will be decoded*; positions
    are indices into that batch.  Returns ``(name, params)`` where params is
    ``[]`` (no adapter anywhere), ``[wids]`` (one type covers every row) or
    ``[sids_t0, wids_t0, sids_t1, wids_t1, ...]`` over the non-empty types.
    """
    no_adapter = False
    a_sids = [[] for _ in range(n_types)]
    a_wids = [[] for _ in range(n_types)]
    for i in range(len(tids)):
        if tids[i] < 0:
            no_adapter = True
            continue
        a_sids[tids[i]].append(i)
        a_wids[tids[i]].append(int(wids[i]))
    non_empty = [t for t in range(n_types) if a_sids[t]]
    if no_adapter and not non_empty:
        return "decode_no_adapter", []
    if not no_adapter and len(non_empty) == 1:
        return f"decode_a{non_empty[0]}", [a_wids[non_empty[0]]]
    name = "mixed_decode_" + "_".join(f"a{t}" for t in non_empty)
    params = []
    for t in non_empty:
        params.append(a_sids[t])
        params.append(a_wids[t])
    return name, params


def segment_sort(slots):
    """Tokens-per-adapter segment sort used by the LoRA gather-matmul.

    ``slots[t]`` is the adapter slot of row ``t`` (``-1`` = none).  Returns
    ``(perm, seg_offsets, seg_slot)``: ``perm`` is the stable permutation that
    groups rows by slot with no-adapter rows first (the single-type case of
    ``llama_seq_info.py:61-75``; it is what ``gen_lora.py:78`` gets from
    ``np.sort`` for its "uniform" request mix), segment ``s`` covers
    ``perm[seg_offsets[s]:seg_offsets[s+1]]`` and all of its rows use
    ``seg_slot[s]``.
    """
    slots = np.asarray(slots, dtype=np.int64)
    perm = np.argsort(slots, kind="stable").astype(np.int32)
    sorted_slots = slots[perm]
    if len(slots) == 0:
        return perm, np.zeros(1, np.int32), np.zeros(0, np.int32)
    starts = np.flatnonzero(np.r_[True, sorted_slots[1:] != sorted_slots[:-1]])
    seg_offsets = np.r_[starts, len(slots)].astype(np.int32)
    seg_slot = sorted_slots[starts].astype(np.int32)
    return perm, seg_offsets, seg_slot


def bfs_fuse_decode_seqids(per_seq_ops, batchable=("decode",)):
    """Which sequence ids end up in each fused batchable op.

    Follows ``tvm/llama_auto_batcher/exec_graph.py:55-69,85-107``: a
    level-synchronous BFS from the source variables; all ops of a batchable
    type that sit on the same BFS level are merged.  ``per_seq_ops[s]`` is the
    chain of op types of sequence ``s`` (each op consumes the previous op's
    output).  Returns ``{(level, op_type): sorted(seqids)}`` -- the reference
    merges in Python-set iteration order, so only the *set* of fused ids is
    defined; ``order_seqs`` normalises the order afterwards.
    """
    fused = {}
    depth = max((len(c) for c in per_seq_ops), default=0)
    for lvl in range(depth):
        for sid, chain in enumerate(per_seq_ops):
            if lvl < len(chain) and chain[lvl] in batchable:
                fused.setdefault((lvl, chain[lvl]), []).append(sid)
    return {k: sorted(v) for k, v in fused.items()}
