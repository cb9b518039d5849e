"""Tensor parallelism (column/row-parallel projections, LoRA partials folded into the row-parallel sum,
vocabulary-parallel lm_head) against the single-device oracle."""
import os
import socket
import threading

import numpy as np
import pytest
import torch

from conftest import PKG, ROOT, load
from oracle import llama as ollama

pytestmark = pytest.mark.gpu
ATOL, RTOL = 2e-2, 1e-2


def _case(synth):
    cfg = synth.llama_config("tiny")
    w = {k: v.bfloat16() for k, v in synth.base_weights(cfg).items()}
    ads = synth.lora_adapters(cfg, 3, [8, 16, 16], targets=synth.ATTN_PROJ + synth.MLP_PROJ)
    ads = [{k: v.bfloat16() for k, v in a.items()} for a in ads]
    scales = [2.0, 1.0, 0.5]
    P = synth.prompts(4, 21, cfg["vocab_size"])
    ids = [2, -1, 0, 1]
    return cfg, w, ads, scales, P, ids


def _run_rank(rank, G, cfg, w, ads, scales, P, ids, dev, coll, steps, feed, out):
    model_mod, kv_mod = load("model"), load("kv_cache")
    pm = model_mod.PackedLlama(cfg, w, ads, scales, device=dev, tp_rank=rank, tp_size=G)
    kv = kv_mod.PagedKVCache(pm.L, pm.Hkv, pm.D, 4, 4 * 40, 40, 16, dev, max_seq_len=40)
    eng = model_mod.Engine(pm, kv, 64, collective=coll)
    for s in range(4):
        kv.add_sequence(s)
    lg, tok = eng.prefill([0, 1, 2, 3], [list(p) for p in P], ids)
    res = [(lg.clone(), tok.clone())]
    for st in range(steps):
        lg, tok = eng.decode([0, 1, 2, 3], feed[st], ids)
        res.append((lg.clone(), tok.clone()))
    torch.cuda.synchronize()
    out[rank] = res


def test_two_way_tensor_parallel_matches_oracle_on_one_gpu(synth, cuda):
    """Both ranks run as threads on one GPU; the all-reduce is a host-side rendezvous (ThreadCollective)."""
    sharding = load("sharding")
    cfg, w, ads, scales, P, ids = _case(synth)
    oracle = ollama.OracleLlama(cfg, w, ads, scales)
    want_tok, want_logits = oracle.greedy([list(p) for p in P], ids, 4)
    feed = [want_tok[:, s].tolist() for s in range(3)]
    G = 2
    shared = sharding.ThreadCollective.Shared(G)
    out = [None] * G
    errs = []

    def body(r):
        try:
            _run_rank(r, G, cfg, w, ads, scales, P, ids, cuda, sharding.ThreadCollective(shared, r), 3, feed, out)
        except Exception as e:  # noqa: BLE001
            errs.append(e)
            shared.barrier.abort()

    ts = [threading.Thread(target=body, args=(r,)) for r in range(G)]
    [t.start() for t in ts]
    [t.join() for t in ts]
    assert not errs, errs
    for step in range(4):
        full = torch.cat([out[r][step][0] for r in range(G)], 1).float().cpu()  # vocabulary slices side by side
        torch.testing.assert_close(full, want_logits[step], atol=ATOL, rtol=RTOL)
        assert torch.equal(out[0][step][1], out[1][step][1])  # every rank ends with the same global token
        assert out[0][step][1].cpu().tolist() == full.argmax(-1).tolist()


def _nccl_worker(rank, G, port, q):
    import importlib
    import sys
    sys.path.insert(0, ROOT)
    import torch.distributed as dist
    synth = importlib.import_module(f"{PKG}.synth")
    sharding = importlib.import_module(f"{PKG}.sharding")
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=G, device_id=dev)
    cfg, w, ads, scales, P, ids = _case(synth)
    oracle = ollama.OracleLlama(cfg, w, ads, scales)
    want_tok, _ = oracle.greedy([list(p) for p in P], ids, 3)
    feed = [want_tok[:, s].tolist() for s in range(2)]
    out = [None] * G
    _run_rank(rank, G, cfg, w, ads, scales, P, ids, dev, sharding.DistCollective(), 2, feed, out)
    q.put((rank, [(lg.float().cpu(), tk.cpu()) for lg, tk in out[rank]]))
    dist.barrier()
    dist.destroy_process_group()


def test_two_way_tensor_parallel_over_nccl(synth, cuda):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_nccl_worker, args=(r, 2, port, q)) for r in range(2)]
    [p.start() for p in procs]
    got = dict(q.get(timeout=300) for _ in range(2))
    [p.join(60) for p in procs]
    cfg, w, ads, scales, P, ids = _case(synth)
    oracle = ollama.OracleLlama(cfg, w, ads, scales)
    _, want_logits = oracle.greedy([list(p) for p in P], ids, 3)
    for step in range(3):
        full = torch.cat([got[r][step][0] for r in range(2)], 1)
        torch.testing.assert_close(full, want_logits[step], atol=ATOL, rtol=RTOL)
        assert torch.equal(got[0][step][1], got[1][step][1])


def _peer_worker(rank, G, port, q, two_step):
    """The library's own exchange kernel (stores into the peers' memory, per-row flags, local reduction) on real
    peers: op-level bit-exactness, the bounded wait running out, recovery, and the tensor-parallel decoder.
    ``two_step``: the form the library takes by itself beyond four ranks (rows reduced at their owner, sums gathered)."""
    import importlib
    import sys
    sys.path.insert(0, ROOT)
    os.environ["MLORA_TP_TWO_STEP"] = "1" if two_step else "0"
    import torch.distributed as dist
    synth = importlib.import_module(f"{PKG}.synth")
    sharding = importlib.import_module(f"{PKG}.sharding")
    ops = importlib.import_module(f"{PKG}.ops")
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=G, device_id=dev)
    report = {}
    try:
        # ---- 1. the exchange alone, many in a row (two alternating buffers, exchange numbers) -----------------
        worst = 0
        for T, H in ((128, 5120), (5, 256), (32, 4096), (7, 8192)):
            coll = sharding.PeerCollective(T, H)
            for it in range(12):
                g = torch.Generator().manual_seed(1000 * it + T)
                parts = [torch.randn(T, H, generator=g).bfloat16() for _ in range(G)]
                res0 = torch.randn(T, H, generator=g)
                w = (1 + 0.1 * torch.randn(H, generator=g)).bfloat16().to(dev)
                total = torch.stack([p.float() for p in parts]).sum(0).bfloat16()  # rank order, fp32, rounded once
                mine = parts[rank].to(dev)
                if it % 3 == 2:  # plain all-reduce, in place
                    coll.all_reduce_sum(mine)
                    ok = torch.equal(mine.cpu(), total)
                else:
                    res, out = res0.to(dev), torch.empty(T, H, dtype=torch.bfloat16, device=dev)
                    assert coll.allreduce_rmsnorm(mine, res, w, 1e-5, out)
                    res_want = res0.to(dev)
                    out_want = ops.residual_rmsnorm(total.to(dev), res_want, w, 1e-5)
                    ok = torch.equal(res, res_want) and torch.equal(out, out_want)
                worst += 0 if ok else 1
            assert coll.status() == 0
        report["op_mismatches"] = worst
        # ---- 2. a peer that never shows up: the wait runs out, the status says who, the context recovers -----------
        coll = sharding.PeerCollective(16, 256)
        x = torch.ones(16, 256, dtype=torch.bfloat16, device=dev)
        if rank == 0:
            coll.set_spin_limit(2000)   # ~0.2 ms
            coll.all_reduce_sum(x)      # rank 1 makes no matching call
            torch.cuda.synchronize()
            report["status_after_timeout"] = coll.status()
            coll.set_spin_limit(1 << 22)
        coll.reset()
        x = torch.full((16, 256), float(rank + 1), dtype=torch.bfloat16, device=dev)
        coll.all_reduce_sum(x)
        torch.cuda.synchronize()
        report["after_reset_ok"] = bool((x == sum(range(1, G + 1))).all()) and coll.status() == 0
        # ---- 3. the tensor-parallel decoder over the fused exchange ------------------------------------------------
        cfg, w_, ads, scales, P, ids = _case(synth)
        oracle = ollama.OracleLlama(cfg, w_, ads, scales)
        want_tok, _ = oracle.greedy([list(p) for p in P], ids, 3)
        feed = [want_tok[:, s].tolist() for s in range(2)]
        out = [None] * G
        _run_rank(rank, G, cfg, w_, ads, scales, P, ids, dev, sharding.PeerCollective(64, cfg["hidden_size"]), 2, feed, out)
        # (numpy: pickled by value -- tensors would travel as shared-memory handles that need this process alive)
        report["model"] = [(lg.float().cpu().numpy(), tk.cpu().numpy()) for lg, tk in out[rank]]
        q.put((rank, report))
    except Exception as e:  # noqa: BLE001
        q.put((rank, {"error": repr(e)}))
    q.close()
    q.join_thread()  # the report is in the pipe before the process leaves
    torch.cuda.synchronize()
    dist.barrier()  # nobody leaves while a peer may still store into its memory
    os._exit(0)


@pytest.mark.parametrize("two_step", [False, True])
def test_two_way_tensor_parallel_over_peer_memory_exchange(synth, cuda, two_step):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_peer_worker, args=(r, 2, port, q, two_step)) for r in range(2)]
    [p.start() for p in procs]
    got = dict(q.get(timeout=300) for _ in range(2))
    [p.join(60) for p in procs]
    for r in range(2):
        assert "error" not in got[r], got[r]
        assert got[r]["op_mismatches"] == 0
        assert got[r]["after_reset_ok"]
    assert got[0]["status_after_timeout"] == 0b10   # rank 1's rows never came
    cfg, w, ads, scales, P, ids = _case(synth)
    oracle = ollama.OracleLlama(cfg, w, ads, scales)
    _, want_logits = oracle.greedy([list(p) for p in P], ids, 3)
    for step in range(3):
        full = torch.cat([torch.from_numpy(got[r]["model"][step][0]) for r in range(2)], 1)
        torch.testing.assert_close(full, want_logits[step], atol=ATOL, rtol=RTOL)
        assert np.array_equal(got[0]["model"][step][1], got[1]["model"][step][1])
