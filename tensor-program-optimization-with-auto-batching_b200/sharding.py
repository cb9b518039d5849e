"""Adapter-sharded data parallelism: one process per GPU, no collective on the data path.

Requests are independent, so a batch is split across ranks by the adapter each
request uses: every rank holds the full base weights, only its own adapters'
A/B stacks and only its own requests' KV pages.  The only exchange is the
gather of generated token ids at the end (host side, ``all_gather_object``).
The reference is single-device (``tvm/llama_auto_batcher/llama_auto_batcher.py:17``);
this is the multi-GPU form of its request->adapter bucketing.
"""
from __future__ import annotations

import threading

import numpy as np


def adapter_owner(adapter_ids, world_size: int, n_adapters: int, policy: str = "block"):
    """Rank that owns each adapter id.  ``block``: contiguous ranges of
    ceil(n_adapters / world_size) adapters; ``balanced``: greedy bin packing by request
    count (for skewed, e.g. Zipf, popularity).  Requests without adapter (id < 0) are
    dealt round-robin by the caller."""
    adapter_ids = np.asarray(adapter_ids)
    if policy == "block":
        per = -(-n_adapters // world_size)
        return np.minimum(np.arange(n_adapters) // per, world_size - 1).astype(np.int32)
    counts = np.bincount(adapter_ids[adapter_ids >= 0], minlength=n_adapters)
    owner = np.zeros(n_adapters, dtype=np.int32)
    load = np.zeros(world_size, dtype=np.int64)
    for a in np.argsort(-counts, kind="stable"):
        r = int(np.argmin(load))
        owner[a] = r
        load[r] += counts[a]
    return owner


def shard_requests(adapter_ids, world_size: int, n_adapters: int, policy: str = "block"):
    """Returns ``(owner, per_rank)``: ``per_rank[r]`` = indices (ascending) of the requests
    rank ``r`` serves."""
    adapter_ids = np.asarray(adapter_ids)
    owner = adapter_owner(adapter_ids, world_size, n_adapters, policy)
    per_rank = [[] for _ in range(world_size)]
    rr = 0
    for i, a in enumerate(adapter_ids.tolist()):
        if a < 0:
            per_rank[rr % world_size].append(i)
            rr += 1
        else:
            per_rank[int(owner[a])].append(i)
    return owner, per_rank


def local_adapter_slots(adapter_ids, owner, rank: int):
    """Adapters a rank holds (ascending global ids) and the map global id -> local slot."""
    mine = [int(a) for a in np.flatnonzero(np.asarray(owner) == rank)]
    return mine, {a: s for s, a in enumerate(mine)}


def gather_results(local_indices, local_tokens, n_requests: int, group=None):
    """Collect per-rank token lists back into request order (host-side, after generation).
    ``local_tokens[j]`` belongs to request ``local_indices[j]``."""
    import torch.distributed as dist

    payload = (list(local_indices), [list(map(int, t)) for t in local_tokens])
    if dist.is_available() and dist.is_initialized() and dist.get_world_size(group) > 1:
        gathered = [None] * dist.get_world_size(group)
        dist.all_gather_object(gathered, payload, group=group)
    else:
        gathered = [payload]
    out = [None] * n_requests
    for idx, toks in gathered:
        for i, t in zip(idx, toks):
            out[i] = t
    return out


# ---- tensor parallelism: the exchange step -------------------------------------------------------------
class DistCollective:
    """NCCL (or gloo) collectives of a ``torch.distributed`` process group, one process per GPU."""

    def __init__(self, group=None):
        import torch.distributed as dist
        self.dist, self.group = dist, group
        self.size = dist.get_world_size(group)

    def all_reduce_sum(self, t):
        self.dist.all_reduce(t, op=self.dist.ReduceOp.SUM, group=self.group)

    def all_gather(self, t):
        import torch
        out = torch.empty((self.size,) + tuple(t.shape), dtype=t.dtype, device=t.device)
        self.dist.all_gather_into_tensor(out, t.contiguous(), group=self.group)
        return out


class ThreadCollective:
    """The same interface for G ranks that run as threads of ONE process on ONE GPU (tests on a single
    device: kernels that wait on one another must not run as separate processes there).  Host-side
    rendezvous; every rank synchronises the device before and after, so it is slow and only for checks."""

    class Shared:
        def __init__(self, size):
            self.size = size
            self.barrier = threading.Barrier(size)
            self.slots = [None] * size
            self.result = None

    def __init__(self, shared, rank):
        self.sh, self.rank, self.size = shared, rank, shared.size

    def _exchange(self, t, fn):
        import torch
        torch.cuda.synchronize()
        self.sh.slots[self.rank] = t
        self.sh.barrier.wait()
        if self.rank == 0:
            self.sh.result = fn(self.sh.slots)
            torch.cuda.synchronize()
        self.sh.barrier.wait()
        res = self.sh.result
        self.sh.barrier.wait()
        return res

    def all_reduce_sum(self, t):
        import torch
        # summed in rank order in fp32, rounded once: what a tree/ring all-reduce of bf16 partials approximates
        res = self._exchange(t, lambda ts: torch.stack([x.float() for x in ts]).sum(0))
        t.copy_(res.to(t.dtype))
        torch.cuda.synchronize()

    def all_gather(self, t):
        import torch
        return self._exchange(t, lambda ts: torch.stack(list(ts))).clone()
