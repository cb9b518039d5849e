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


class PeerCollective:
    """The exchange step in the library's own kernel (``mlora_tp_allreduce_rmsnorm``): every rank stores its partial
    rows into the peers' memory over NVLink and reduces what lands in its own, fused with the residual add + RMSNorm
    that follows -- one launch where the NCCL form takes an all-reduce and a norm kernel.  One process per GPU; the
    arenas are exchanged as CUDA IPC handles through the process group at construction.  Row counts beyond the
    kernel's limit (prefill passes) and the small token all-gather go through ``DistCollective``."""

    MAX_ROWS = 512

    def __init__(self, max_rows, hidden, group=None):
        import ctypes as C

        import torch
        import torch.distributed as dist

        from . import _lib
        self._lib, self._check, self._C, self._torch = _lib.lib(), _lib.check, C, torch
        self.dist, self.group = dist, group
        self.size, self.rank = dist.get_world_size(group), dist.get_rank(group)
        self.max_rows, self.hidden = min(int(max_rows), self.MAX_ROWS), int(hidden)
        self.fallback = DistCollective(group)
        ctx = C.c_void_p()
        self._check(self._lib.mlora_tp_create(self.rank, self.size, self.max_rows, self.hidden, C.byref(ctx)), "mlora_tp_create")
        self.ctx = ctx
        mine = (C.c_ubyte * 64)()
        self._check(self._lib.mlora_tp_export(ctx, mine), "mlora_tp_export")
        handles = [None] * self.size
        dist.all_gather_object(handles, bytes(mine), group=group)
        for g, h in enumerate(handles):
            if g != self.rank:
                self._check(self._lib.mlora_tp_connect(ctx, g, (C.c_ubyte * 64).from_buffer_copy(h)), "mlora_tp_connect")
        dist.barrier(group=group)

    def _fits(self, t):
        return t.dim() == 2 and t.shape[0] <= self.max_rows and t.shape[1] == self.hidden and t.dtype == self._torch.bfloat16 \
            and t.is_contiguous()

    def _stream(self):
        return self._C.c_void_p(self._torch.cuda.current_stream().cuda_stream)

    def all_reduce_sum(self, t):
        if not self._fits(t):
            return self.fallback.all_reduce_sum(t)
        p = self._C.c_void_p(t.data_ptr())
        self._check(self._lib.mlora_tp_allreduce_rmsnorm(self.ctx, p, None, None, 0.0, p, t.shape[0], t.shape[1], self._stream()),
                    "mlora_tp_allreduce_rmsnorm")

    def allreduce_rmsnorm(self, partial, res, w, eps, out):
        """res += sum over ranks of ``partial``; out = RMSNorm(res) * w.  False when the shape does not fit the kernel
        (the caller then takes all_reduce_sum + the norm kernel)."""
        if not self._fits(partial):
            return False
        vp = lambda t: self._C.c_void_p(t.data_ptr())
        self._check(self._lib.mlora_tp_allreduce_rmsnorm(self.ctx, vp(partial), vp(res), vp(w), float(eps), vp(out), partial.shape[0],
                                                         partial.shape[1], self._stream()), "mlora_tp_allreduce_rmsnorm")
        return True

    def all_gather(self, t):
        return self.fallback.all_gather(t)

    def status(self):
        v = self._C.c_int32(0)
        self._check(self._lib.mlora_tp_status(self.ctx, self._C.byref(v)), "mlora_tp_status")
        return int(v.value)

    def set_spin_limit(self, polls):
        self._check(self._lib.mlora_tp_set_spin_limit(self.ctx, int(polls)), "mlora_tp_set_spin_limit")

    def reset(self):
        """After a failed exchange: every rank, between two barriers."""
        self.dist.barrier(group=self.group)
        self._check(self._lib.mlora_tp_reset(self.ctx), "mlora_tp_reset")
        self.dist.barrier(group=self.group)


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
