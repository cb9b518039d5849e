"""Adapter-sharded data parallelism: partition logic and the 2-rank gather, on CPU with gloo."""
import os
import socket

import numpy as np
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from conftest import PKG, ROOT, load


def test_block_and_balanced_partitions_cover_every_request_once():
    sh, synth = load("sharding"), load("synth")
    for world in (1, 2, 4, 8):
        for ids in (synth.adapter_ids_uniform(32 * world, 16 * world), synth.adapter_ids_zipf(64, 64),
                    np.array([-1, 3, -1, 0, 3, 3], dtype=np.int32)):
            n_ad = int(max(ids.max() + 1, 1))
            for policy in ("block", "balanced"):
                owner, per_rank = sh.shard_requests(ids, world, n_ad, policy)
                flat = sorted(i for r in per_rank for i in r)
                assert flat == list(range(len(ids)))
                for r, reqs in enumerate(per_rank):
                    assert reqs == sorted(reqs)
                    for i in reqs:
                        assert ids[i] < 0 or owner[ids[i]] == r  # a request lives where its adapter lives
                held = [sh.local_adapter_slots(ids, owner, r)[0] for r in range(world)]
                assert sorted(a for h in held for a in h) == list(range(n_ad))
    # balanced policy evens out a Zipf-skewed load better than contiguous blocks
    ids = load("synth").adapter_ids_zipf(512, 64)
    loads = {}
    for policy in ("block", "balanced"):
        _, per_rank = sh.shard_requests(ids, 8, 64, policy)
        loads[policy] = max(len(r) for r in per_rank)
    assert loads["balanced"] <= loads["block"]


def _worker(rank, world, port, ret):
    import importlib
    import sys
    sys.path.insert(0, ROOT)
    sh = importlib.import_module(f"{PKG}.sharding")
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    ids = np.array([0, 5, 2, 7, 1, 6, 3, 4, 0, 7], dtype=np.int32)
    owner, per_rank = sh.shard_requests(ids, world, 8, "block")
    mine = per_rank[rank]
    # each rank "generates" tokens for its own requests only: token = 100*request + adapter
    toks = [[100 * i + int(ids[i]), rank] for i in mine]
    out = sh.gather_results(mine, toks, len(ids))
    # the MAX-over-ranks timing reduction the benchmark uses
    t = torch.tensor([1.0 + rank], dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    if rank == 0:
        ret["out"], ret["tmax"], ret["owner"] = out, float(t), owner.tolist()
    dist.barrier()
    dist.destroy_process_group()


def test_two_rank_gather_restores_request_order():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    ret = mp.Manager().dict()
    mp.spawn(_worker, args=(2, port, ret), nprocs=2, join=True)
    out = ret["out"]
    ids = [0, 5, 2, 7, 1, 6, 3, 4, 0, 7]
    assert ret["owner"] == [0, 0, 0, 0, 1, 1, 1, 1]
    assert ret["tmax"] == 2.0
    for i, (tok, rank) in enumerate(out):
        assert tok == 100 * i + ids[i]
        assert rank == (0 if ids[i] < 4 else 1)
