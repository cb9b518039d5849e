#!/usr/bin/env python
"""Benchmark: multi-LoRA decode tokens/s, Llama-2-7B shape, 32 requests / 16 rank-16 adapters per GPU.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

One "step" = one decode step (one token for each of the 32 requests of a GPU) at context
512+ tokens, paged KV (block 16), LoRA on q/k/v/o.  Prints ONE JSON line (rank 0).
N > 1 is launched with torch.distributed.run, one rank per GPU: requests are sharded by
adapter id, every rank serves 32 requests of its own 16 adapters (weak scaling), no
collective on the data path; timing is bracketed by a barrier and reduced with MAX.

All inputs are seeded synthetic data of the named shapes (random-init weights, random
token ids); nothing is read from outside this repository.
"""
from __future__ import annotations

import argparse
import importlib
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)
PKG = "tensor-program-optimization-with-auto-batching_b200"

METRIC = "multi-LoRA decode tokens/s (Llama-7B shape, 32 req/16 adapters)"
N_REQ, N_ADAPTERS, RANK, ALPHA, PROMPT_LEN, PAGE = 32, 16, 16, 32, 512, 16
FALLBACK_HBM_GBS = 6650.0


def load(sub):
    return importlib.import_module(f"{PKG}.{sub}")


def measured_peak():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        with open(p) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    return FALLBACK_HBM_GBS, "fallback"


class ClockSampler:
    """Samples SM clock and throttle reasons with nvidia-smi while the timed region runs."""

    Q = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index, self.rows, self.proc = index, [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", str(self.index), f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                 "-lms", "100"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in self.rows:
            try:
                sm.append(float(r[0]))
                mx.append(float(r[1]))
            except (ValueError, IndexError):
                continue
            for n, v in zip(names, r[3:7]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "samples": len(sm), "reasons": sorted(reasons)}


# ----------------------------------------------------------------------------------------------
def cpu_reference_step(cfg, synth, steps, warmup):
    """The reference's HF CPU path on this box's cores: seconds per full-model decode step,
    from a bounded sample (1- and 3-layer truncations at the same shapes, extrapolated)."""
    import torch
    from oracle import hf_path

    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    ids = synth.adapter_ids_uniform(N_REQ, N_ADAPTERS)
    r = hf_path.time_decode_sample(
        cfg, lambda L: synth.base_weights(cfg, n_layers=L),
        lambda L: synth.lora_adapters(cfg, N_ADAPTERS, RANK, n_layers=L), [ALPHA / RANK] * N_ADAPTERS, ids,
        PROMPT_LEN, layer_counts=(1, 3), steps=max(1, min(steps, 3)), warmup=max(1, min(warmup, 1)))
    sample = (f"HF LlamaForCausalLM fp32 + restated GatherBMMLinear, batch {N_REQ}, ctx {PROMPT_LEN}, timed on "
              f"1- and 3-layer truncations ({r['samples'][0][1]:.3f}s, {r['samples'][-1][1]:.3f}s per step), "
              f"extrapolated to {cfg['num_hidden_layers']} layers")
    return N_REQ / r["full_step_s"], cores, sample, r


def run_13b_shape(args):
    """Side measurement, not the benchmark line: one GPU holding the whole Llama-2-13B shape (tensor parallel size 1)
    with the adapter mix of the 13B configuration -- 128 requests, 128 adapters whose ranks cycle 8/16/32/64 on
    q/k/v/o, every request its own adapter -- at a short context (128-token prompts: 128 x 1 K tokens of KV would
    not leave room beside 26 GB of weights and 27 GB of adapters).  Decode steps in a CUDA graph, CUDA-event timed."""
    import numpy as np
    import torch

    ops, synth, model_mod, kv_mod = load("ops"), load("synth"), load("model"), load("kv_cache")
    load("build").build()
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    cfg = synth.llama_config("llama2-13b")
    L = args.layers or cfg["num_hidden_layers"]
    cfg = dict(cfg, num_hidden_layers=L)
    n_req = n_ad = 128
    prompt_len, steps, warm = 128, max(8, min(args.steps, 32)), 3
    w = synth.base_weights(cfg, dtype=torch.bfloat16, device=dev)
    ads = synth.lora_adapters(cfg, n_ad, [8, 16, 32, 64], dtype=torch.bfloat16, device=dev)
    pm = model_mod.PackedLlama(cfg, w, ads, [2.0] * n_ad, device=dev)
    del w, ads
    torch.cuda.empty_cache()
    max_len = prompt_len + 2 * (steps + warm) + 8
    kv = kv_mod.PagedKVCache(pm.L, pm.Hkv, pm.D, n_req, n_req * max_len, prompt_len, PAGE, dev, max_seq_len=max_len)
    eng = model_mod.Engine(pm, kv, max_rows=8192)
    sids = list(range(n_req))
    for sid in sids:
        kv.add_sequence(sid)
    prompts = [p.tolist() for p in synth.prompts(n_req, prompt_len, cfg["vocab_size"])]
    slots = [int(i) for i in np.random.default_rng(synth.SEED_IDS).permutation(n_ad)]
    _, first_tok = eng.prefill(sids, prompts, slots)
    res = {}
    for name, use_lora in (("lora", True), ("base", False)):
        graph = eng.capture_decode(sids, slots, use_lora=use_lora, reserve_tokens=steps + warm + 2)
        eng.tokens[:n_req].copy_(first_tok)
        len0, len0_host = kv.seq_lens.clone(), kv._len_host.copy()
        for _ in range(warm):
            graph.replay()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            graph.replay()
        e1.record()
        torch.cuda.synchronize()
        res[name] = e0.elapsed_time(e1) / steps
        kv.seq_lens.copy_(len0)
        kv._len_host[:] = len0_host
    peak, src = measured_peak()
    wbytes = L * 2 * (4 * 5120 * 5120 + 3 * 5120 * 13824) + 2 * 32000 * 5120
    kvbytes = n_req * (prompt_len + warm + steps // 2) * 2 * 5120 * 2 * L
    abytes = sum(L * 2 * r * (3 * 5120 + 3 * 5120 + 5120 + 5120) for r in ([8, 16, 32, 64] * 32))
    emit({"side_measurement": "llama2-13b shape on ONE GPU (tensor parallel size 1), 128 requests x 128 adapters (ranks 8/16/32/64), "
                              "128-token prompts", "layers": L, "ms_per_step_with_lora": res["lora"],
          "ms_per_step_base_only": res["base"], "tokens_per_s": n_req / res["lora"] * 1e3,
          "lora_overhead_frac": res["lora"] / res["base"] - 1.0,
          "algorithmic_gb_per_step": (wbytes + kvbytes + abytes) / 1e9,
          "hbm_frac_of_measured": (wbytes + kvbytes + abytes) / (res["lora"] * 1e6) / peak, "peak_source": src,
          "status": eng.status_word()})


def run_prefill_heavy(args):
    """Side measurement (its own JSON line): the prefill-heavy configuration on one GPU -- Llama-2-7B shape, 64
    requests x 512-token prompts, 64 rank-64 adapters on all seven projections, adapter ids Zipf(1.1) (skewed segment
    sizes for the grouped shrink), then 16 greedy decode tokens.  Prefill is timed with CUDA events over the engine's
    own passes (4 passes of 8192 rows); flops are the algorithmic ones of the workload."""
    import numpy as np
    import torch

    ops, synth, model_mod, kv_mod = load("ops"), load("synth"), load("model"), load("kv_cache")
    load("build").build()
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    cfg = synth.llama_config("llama2-7b")
    L = args.layers or cfg["num_hidden_layers"]
    cfg = dict(cfg, num_hidden_layers=L)
    n_req = n_ad = 64
    rank, prompt_len, gen = 64, 512, 16
    w = synth.base_weights(cfg, dtype=torch.bfloat16, device=dev)
    ads = synth.lora_adapters(cfg, n_ad, rank, targets=synth.ATTN_PROJ + synth.MLP_PROJ, dtype=torch.bfloat16, device=dev)
    pm = model_mod.PackedLlama(cfg, w, ads, [0.5] * n_ad, device=dev)
    del w, ads
    torch.cuda.empty_cache()
    ids = [int(i) for i in synth.adapter_ids_zipf(n_req, n_ad)]
    prompts = [p.tolist() for p in synth.prompts(n_req, prompt_len, cfg["vocab_size"])]
    max_len = prompt_len + gen + 4
    sids = list(range(n_req))
    times = []
    for rep in range(2):  # first pass warms up (lazy kernel loading); the second is the measured one
        kv = kv_mod.PagedKVCache(pm.L, pm.Hkv, pm.D, n_req, n_req * max_len, prompt_len, PAGE, dev, max_seq_len=max_len)
        eng = model_mod.Engine(pm, kv, max_rows=8192)
        for sid in sids:
            kv.add_sequence(sid)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        e0.record()
        _, first_tok = eng.prefill(sids, prompts, ids)
        e1.record()
        torch.cuda.synchronize()
        times.append(e0.elapsed_time(e1))
        if rep == 0:
            del eng, kv
            torch.cuda.empty_cache()
    ms_prefill = times[-1]
    graph = eng.capture_decode(sids, ids, reserve_tokens=gen + 2)
    eng.tokens[:n_req].copy_(first_tok)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    graph.replay()
    e0.record()
    for _ in range(gen - 1):
        graph.replay()
    e1.record()
    torch.cuda.synchronize()
    ms_decode = e0.elapsed_time(e1) / (gen - 1)
    H, I, V = cfg["hidden_size"], cfg["intermediate_size"], cfg["vocab_size"]
    tokens = n_req * prompt_len
    base = 2.0 * (4 * H * H + 3 * H * I) * tokens * L
    lora = 2.0 * rank * (4 * (H + H) + 2 * (H + I) + (I + H)) * tokens * L
    attn = 4.0 * H * L * n_req * prompt_len * (prompt_len + 1) / 2
    head = 2.0 * V * H * n_req
    peaks = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json"))) if os.path.exists(os.path.join(ROOT, "MEASURED_PEAKS.json")) else {}
    tpk = float(peaks.get("bf16_tflops_sustained", 1400.0))
    fl = base + lora + attn + head
    emit({"workload": "llama2-7b shape, prefill-heavy", "layers": L, "requests": n_req, "prompt_len": prompt_len,
          "adapters": n_ad, "adapter_rank": rank, "adapter_targets": "q/k/v/o/gate/up/down", "adapter_ids": "Zipf(1.1) seed 3",
          "distinct_adapters_in_batch": len(set(ids)), "prefill_ms": ms_prefill, "prefill_tokens_per_s": tokens / ms_prefill * 1e3,
          "prefill_tflops": fl / ms_prefill / 1e9, "flops": {"base": base, "lora": lora, "attention": attn, "lm_head": head},
          "peak_tflops_sustained": tpk, "frac_of_tensor_peak": fl / ms_prefill / 1e9 / tpk,
          "decode_ms_per_step": ms_decode, "decode_tokens_per_s": n_req / ms_decode * 1e3, "decode_tokens": gen,
          "tc_status_word": eng.status_word(), "dtype": "bf16", "data": "synthetic"})


def run_13b_tp(args, rank, world, local_rank):
    """The tensor-parallel configuration: Llama-2-13B shape, 128 requests, prompt lengths U[128,1024], 128 adapters
    with ranks cycling 8/16/32/64 on q/k/v/o, paged KV (block 16), tensor parallel size = number of ranks
    (column-parallel q/k/v/gate/up, row-parallel o/down + one NCCL all-reduce each, vocabulary-parallel lm_head).
    One JSON line (its own, not the benchmark's): tokens/s over K CUDA-graph decode steps, per-rank algorithmic
    bytes and HBM fraction, and the CUDA-event time of the step's all-reduces replayed alone."""
    import numpy as np
    import torch
    import torch.distributed as dist

    synth, model_mod, kv_mod, ops, sharding = (load(m) for m in ("synth", "model", "kv_cache", "ops", "sharding"))
    load("build").build()
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    cfg = synth.llama_config("llama2-13b")
    coll = None
    if world > 1:  # the exchange step: NCCL, or the library's own kernel over peer memory
        coll = sharding.PeerCollective(128, cfg["hidden_size"]) if args.tp_collective == "peer" else sharding.DistCollective()
    L = args.layers or cfg["num_hidden_layers"]
    cfg = dict(cfg, num_hidden_layers=L)
    n_req = n_ad = 128
    K, W = max(4, min(args.steps, 64)), max(3, args.warmup)
    ranks = [8, 16, 32, 64]
    w = synth.base_weights(cfg, dtype=torch.bfloat16, device=dev)
    ads = synth.lora_adapters(cfg, n_ad, ranks, dtype=torch.bfloat16, device=dev)
    pm = model_mod.PackedLlama(cfg, w, ads, [2.0] * n_ad, device=dev, tp_rank=rank, tp_size=world)
    del w, ads
    torch.cuda.empty_cache()
    lens = [int(x) for x in synth.prompt_lengths(n_req, 128, 1024)]
    total_steps = 2 * (K + W) + 8
    max_len = max(lens) + total_steps + 1
    kv = kv_mod.PagedKVCache(pm.L, pm.Hkv, pm.D, n_req, sum(lens) + n_req * (total_steps + 1), 1024, PAGE, dev,
                             max_seq_len=max_len)
    eng = model_mod.Engine(pm, kv, max_rows=4096, collective=coll)
    sids = list(range(n_req))
    for sid in sids:
        kv.add_sequence(sid)
    rng = np.random.default_rng(synth.SEED_TOKENS)
    prompts = [rng.integers(0, cfg["vocab_size"], n).tolist() for n in lens]
    slots = [int(i) for i in np.random.default_rng(synth.SEED_IDS).permutation(n_ad)]  # every request its own adapter
    t0 = time.perf_counter()
    _, first_tok = eng.prefill(sids, prompts, slots)
    torch.cuda.synchronize()
    prefill_s = time.perf_counter() - t0

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()

    def max_over_ranks(x):
        if world == 1:
            return x
        t = torch.tensor([x], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    graph = eng.capture_decode(sids, slots, reserve_tokens=total_steps)
    eng.tokens[:n_req].copy_(first_tok)
    for _ in range(W):
        graph.replay()
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    e0.record()
    for _ in range(K):
        graph.replay()
    e1.record()
    barrier()
    ms_step = max_over_ranks(e0.elapsed_time(e1)) / K
    clocks = sampler.stop() if rank == 0 else None
    status = eng.status_word()

    # the exchange steps of one decode step alone, each with the residual add + RMSNorm it feeds (2 per layer), in both
    # forms: NCCL all-reduce + norm kernel, and the fused peer-memory kernel
    ms_coll = {}
    if world > 1:
        y, xn, lnw = eng.y[:n_req], eng.xn[:n_req], pm.layers[0].ln2
        res_tmp = torch.zeros(n_req, pm.H, device=dev)
        forms = {"nccl": sharding.DistCollective()}
        if args.tp_collective == "peer":
            forms["peer"] = coll

        def exchanges(c):
            fused = getattr(c, "allreduce_rmsnorm", None)
            for _ in range(2 * pm.L):
                if fused is None or not fused(y, res_tmp, lnw, pm.eps, xn):
                    c.all_reduce_sum(y)
                    ops.residual_rmsnorm(y, res_tmp, lnw, pm.eps, out=xn)
        for name, c in forms.items():
            side = torch.cuda.Stream()
            side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(side):
                exchanges(c)
            torch.cuda.current_stream().wait_stream(side)
            torch.cuda.synchronize()
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g):
                exchanges(c)
            for _ in range(3):
                g.replay()
            barrier()
            e0.record()
            for _ in range(10):
                g.replay()
            e1.record()
            barrier()
            ms_coll[name] = max_over_ranks(e0.elapsed_time(e1)) / 10
            del g

    peak, src = measured_peak()
    H, I, V = 5120, 13824, 32000
    ctx_mean = float(np.mean(lens)) + W + (K - 1) / 2.0
    wbytes = (L * 2 * (4 * H * H + 3 * H * I) + 2 * V * H) / world + (2 * L + 1) * 2 * H
    # adapter bytes a step reads, by rank of the adapter (A and B of q/k/v/o; the sharded halves split by `world`)
    r_each = [ranks[i % 4] for i in range(n_ad)]
    abytes = sum(L * 2 * r * ((3 * H + 3 * H / world) + (H / world + H)) for r in r_each)
    kvbytes = n_req * (ctx_mean + 1) * 2 * (H / world) * 2 * L
    per_rank = wbytes + abytes + kvbytes
    if rank == 0:
        emit({"workload": "llama2-13b shape, tensor parallel", "metric": "multi-LoRA decode tokens/s (Llama-13B shape, "
              "128 req/128 adapters, tensor parallel)", "value": n_req / ms_step * 1e3, "unit": "tokens/s",
              "n_gpus": world, "tp_size": world, "layers": L, "steps": K, "warmup": W, "ms_per_step": ms_step,
              "scaling": "strong", "dtype": "bf16", "data": "synthetic",
              "config": {"requests": n_req, "adapters": n_ad, "adapter_ranks": ranks, "prompt_lens": "U[128,1024] seed 4",
                         "mean_ctx": ctx_mean, "parallelism": f"tp{world} (Megatron column/row + " + ("fused peer-memory exchange" if args.tp_collective == "peer" else "NCCL all-reduce") + ")"},
              "per_rank": {"algorithmic_bytes": per_rank, "achieved_gbs": per_rank / (ms_step * 1e6),
                           "hbm_frac": per_rank / (ms_step * 1e6) / peak, "peak_gbs": peak, "peak_source": src},
              "collectives": {"exchanges_per_step": 2 * L, "bytes_each": n_req * H * 2,
                              "impl_in_step": "fused peer-memory kernel (mlora_tp_allreduce_rmsnorm)" if args.tp_collective == "peer"
                              else "NCCL all-reduce via torch.distributed + norm kernel",
                              "ms_alone_per_step_with_their_norms": ms_coll,
                              "share_of_step": (ms_coll.get(args.tp_collective, 0.0) / ms_step) if ms_step else None,
                              "peer_status": coll.status() if args.tp_collective == "peer" and world > 1 else None},
              "clocks": clocks, "prefill_seconds_untimed": prefill_s, "tc_status_word": status})
    if world > 1:
        # The step's CUDA graph holds NCCL kernels: tearing the process group down while such graphs exist was seen
        # to block forever, so the ranks meet once more and then leave without the orderly teardown.
        torch.cuda.synchronize()
        dist.barrier()
        sys.stdout.flush()
        sys.stderr.flush()
        os._exit(0)


def run_reference(args, rank, world):
    if rank != 0:
        return
    synth = load("synth")
    cfg = synth.llama_config("llama2-7b")
    tps, cores, sample, r = cpu_reference_step(cfg, synth, args.steps, args.warmup)
    line = {
        "impl": "reference", "metric": METRIC, "value": tps, "unit": "tokens/s", "n_gpus": args.gpus,
        # a full-model CPU step takes seconds: at most 3 steps of each truncation are timed, whatever was asked for
        "steps": max(1, min(args.steps, 3)), "warmup": max(1, min(args.warmup, 1)), "steps_requested": args.steps,
        "ms_per_step": 1e3 * r["full_step_s"], "extrapolated": True,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": workload_config(args.gpus),
        "cpu_baseline": {"value": tps, "unit": "tokens/s", "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": tps, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    emit(line)


def workload_config(n_gpus, strong=False):
    if strong:
        return {
            "workload": "llama2-7b-shape multi-LoRA decode, strong-scaling side line: the SAME 32 requests x 16 rank-16 "
                        "adapters (alpha 32) on q/k/v/o spread over the GPUs by adapter, 512-token prompts, paged KV block 16",
            "requests_per_gpu": N_REQ / n_gpus, "adapters_per_gpu": N_ADAPTERS / n_gpus, "global_batch": N_REQ,
            "prompt_len": PROMPT_LEN, "parallelism": f"adapter-sharded replicas x{n_gpus} (no collective), fixed total batch",
            "l2": "inputs exceed L2 (13.2 GB of weights streamed per step on every GPU)",
        }
    return {
        "workload": "llama2-7b-shape multi-LoRA decode: 32 layers, hidden 4096, 32x128 heads, inter 11008, "
                    "vocab 32000; per GPU 32 requests x 16 rank-16 adapters (alpha 32) on q/k/v/o, 512-token "
                    "prompts, paged KV block 16, greedy decode",
        "requests_per_gpu": N_REQ, "adapters_per_gpu": N_ADAPTERS, "global_batch": N_REQ * n_gpus,
        "prompt_len": PROMPT_LEN, "parallelism": f"adapter-sharded replicas x{n_gpus} (no collective)",
        "l2": "inputs exceed L2 (13.2 GB of weights + ~9 GB of KV streamed per step)",
    }


# ----------------------------------------------------------------------------------------------
def run_ours(args, rank, world, local_rank):
    import numpy as np
    import torch

    synth, model_mod, kv_mod, ops, sharding = (load(m) for m in ("synth", "model", "kv_cache", "ops", "sharding"))
    load("build").build()
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    dist = None
    if world > 1:
        import torch.distributed as dist
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=dev)

    def barrier():
        torch.cuda.synchronize()
        if dist is not None:
            dist.barrier()

    def max_over_ranks(x):
        if dist is None:
            return x
        t = torch.tensor([x], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    K, W = args.steps, args.warmup
    cfg = synth.llama_config("llama2-7b")
    L = args.layers or cfg["num_hidden_layers"]
    cfg = dict(cfg, num_hidden_layers=L)

    # ---- the global batch and its shard ---------------------------------------------------------------
    # rank r owns adapters [16r, 16r+16); its 32 requests draw their adapter uniformly from those
    strong = args.scaling == "strong"
    if strong:  # the SAME 32 requests over 16 adapters, spread over the ranks by adapter (side line, not the benchmark's)
        ids_global = np.random.default_rng(synth.SEED_IDS).integers(0, N_ADAPTERS, N_REQ).astype(np.int32)
        owner, per_rank = sharding.shard_requests(ids_global, world, N_ADAPTERS, "balanced")
    else:
        ids_global = np.concatenate([
            N_ADAPTERS * r + np.random.default_rng(synth.SEED_IDS + r).integers(0, N_ADAPTERS, N_REQ) for r in range(world)
        ]).astype(np.int32)
        owner, per_rank = sharding.shard_requests(ids_global, world, N_ADAPTERS * world, "block")
    mine = per_rank[rank]
    held, slot_of = sharding.local_adapter_slots(ids_global, owner, rank)
    slots = [slot_of[int(ids_global[i])] for i in mine]
    B = len(mine)
    prompts_all = synth.prompts(N_REQ * (1 if strong else world), PROMPT_LEN, cfg["vocab_size"])
    prompts = [prompts_all[i].tolist() for i in mine]

    # ---- model ------------------------------------------------------------------------------------------
    w = synth.base_weights(cfg, dtype=torch.bfloat16, device=dev)
    ads = synth.lora_adapters(cfg, len(held), RANK, dtype=torch.bfloat16, device=dev)
    pm = model_mod.PackedLlama(cfg, w, ads, [ALPHA / RANK] * len(held), device=dev)
    del w, ads
    torch.cuda.empty_cache()
    total_steps = 2 * (K + W) + 8
    max_len = PROMPT_LEN + total_steps + 1
    kv = kv_mod.PagedKVCache(pm.L, pm.Hkv, pm.D, B, B * max_len, PROMPT_LEN, PAGE, dev, max_seq_len=max_len)
    eng = model_mod.Engine(pm, kv, max_rows=max(4096, B))  # prefill in passes of 4096 rows; decode uses B rows
    sids = list(range(B))
    for s in sids:
        kv.add_sequence(s)

    # ---- prefill through the product path (untimed set-up) ---------------------------------------------
    t0 = time.perf_counter()
    if args.skip_prefill:
        g = torch.Generator(device=dev).manual_seed(synth.SEED_TOKENS)
        for s in sids:
            kv.reserve(s, PROMPT_LEN)
        kv.pages.copy_(torch.randn(kv.pages.shape, generator=g, device=dev, dtype=torch.float32).to(torch.bfloat16)
                       if kv.pages.numel() < (1 << 28) else
                       torch.randn(kv.pages.shape, generator=g, device=dev, dtype=torch.bfloat16))
        kv._len_host[:B] = PROMPT_LEN
        kv.seq_lens[:B] = PROMPT_LEN
        first_tok = torch.from_numpy(np.asarray([p[-1] for p in prompts], dtype=np.int32)).to(dev)
    else:
        _, first_tok = eng.prefill(sids, prompts, slots)
    torch.cuda.synchronize()
    prefill_s = time.perf_counter() - t0

    launches0 = ops.launch_count()
    graph = eng.capture_decode(sids, slots, reserve_tokens=total_steps)
    launches_per_step = (ops.launch_count() - launches0) // 2  # one warm-up run + one capture
    eng.tokens[:B].copy_(first_tok)
    len0 = kv.seq_lens.clone()
    len0_host = kv._len_host.copy()

    def rewind():
        kv.seq_lens.copy_(len0)
        kv._len_host[:] = len0_host
        eng.tokens[:B].copy_(first_tok)

    # ---- timed region 1: inputs resident in HBM ------------------------------------------------------
    for _ in range(W):
        graph.replay()
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    ev0.record()
    for _ in range(K):
        graph.replay()
    ev1.record()
    barrier()
    ms_total = max_over_ranks(ev0.elapsed_time(ev1))
    clocks = sampler.stop() if rank == 0 else None
    ctx_end = PROMPT_LEN + W + K
    status = eng.status_word()

    # ---- timed region 2: end to end through the public step call, host buffers ---------------------------
    rewind()
    tok_host = torch.empty(B, dtype=torch.int32).pin_memory()
    tok_host.copy_(first_tok.cpu())
    out_host = torch.empty(B, dtype=torch.int32).pin_memory()

    def step_host():
        eng.tokens[:B].copy_(tok_host, non_blocking=True)   # H2D of this step's inputs
        graph.replay()
        out_host.copy_(eng.next_tok[:B], non_blocking=True)  # D2H of this step's result
        torch.cuda.current_stream().synchronize()
        tok_host.copy_(out_host)

    for _ in range(W):
        step_host()
    barrier()
    ev0.record()
    for _ in range(K):
        step_host()
    ev1.record()
    barrier()
    ms_e2e = max_over_ranks(ev0.elapsed_time(ev1))

    # ---- base-only decode (same batch, adapters off): the denominator of the LoRA overhead ------------------
    rewind()
    graph_base = eng.capture_decode(sids, slots, use_lora=False, reserve_tokens=total_steps)
    rewind()
    for _ in range(W):
        graph_base.replay()
    barrier()
    ev0.record()
    for _ in range(K):
        graph_base.replay()
    ev1.record()
    barrier()
    ms_base = max_over_ranks(ev0.elapsed_time(ev1)) / K

    # ---- kernel-only passes for the roofline: the projection launches, then the attention launches -------
    peak, peak_src = measured_peak()
    n_uniq = len(set(slots))
    rewind()
    roof = kernel_rooflines(eng, pm, kv, B, slots, ops, torch, ctx=PROMPT_LEN + W + K // 2, n_uniq=n_uniq, peak=peak)

    # ---- algorithmic bytes of one whole step (mean context over the timed region) ------------------------
    ctx_mean = PROMPT_LEN + W + (K - 1) / 2.0
    kv_tok_bytes = 2 * pm.Hkv * pm.D * 2 * pm.L
    step_bytes = (pm.weight_bytes() + n_uniq * pm.lora_bytes_per_adapter() + B * ctx_mean * kv_tok_bytes
                  + B * kv_tok_bytes + B * pm.H * 2)
    ms_step = ms_total / K
    tokens_total = B * K
    if dist is not None:
        t = torch.tensor([tokens_total], dtype=torch.float64, device=dev)
        dist.all_reduce(t)
        tokens_total = float(t.item())
    value = tokens_total / (ms_total / 1e3)
    e2e_value = tokens_total / (ms_e2e / 1e3)

    # ---- the operator micro-benchmark (T = 1, 8, 32, 128), outside every timed region ---------------------------
    op_rows = None
    if rank == 0 and world == 1 and not args.no_operator:
        torch.cuda.synchronize()
        op_rows = operator_rows(ops, synth, dev, torch)

    line = None
    if rank == 0:
        line = {
            "metric": METRIC, "value": value, "unit": "tokens/s", "n_gpus": world, "steps": K, "warmup": W,
            "ms_per_step": ms_step, "higher_is_better": True, "scaling": args.scaling, "vs_baseline": None,
            "dtype": "bf16", "data": "synthetic", "config": dict(workload_config(world, strong), layers=L,
                                                                  ctx_start=PROMPT_LEN + W, ctx_end=ctx_end),
            "e2e": {"value": e2e_value, "unit": "tokens/s", "h2d_bytes_per_step": 4 * B, "d2h_bytes_per_step": 4 * B,
                    "ms_per_step": ms_e2e / K,
                    "call": "Engine decode step: pinned int32 token ids -> device, CUDA-graph step (device-side position "
                            "bookkeeping, 32 layers, lm_head, on-device argmax), int32 next tokens -> pinned host"},
            "gpu_launches": launches_per_step * K, "launches_per_step": launches_per_step,
            "roofline": roof["linear"], "roofline_attention": roof["attention"],
            "step_hbm": {"algorithmic_bytes": step_bytes, "achieved_gbs": step_bytes / (ms_step * 1e6),
                         "peak_gbs": peak, "peak_source": peak_src,
                         "frac": step_bytes / (ms_step * 1e6) / peak,
                         "frac_of_8tbs": step_bytes / (ms_step * 1e6) / 8000.0},
            "lora_overhead": {"base_only_ms_per_step": ms_base, "with_lora_ms_per_step": ms_step,
                              "overhead_frac": ms_step / ms_base - 1.0},
            "clocks": clocks, "prefill_seconds_untimed": prefill_s, "tc_status_word": status,
            "operator_microbench": op_rows,
        }
        if world == 1 and not args.no_cpu:
            # CPU leg (outside every timed region): the oracle as the timed baseline, and as the checker of the
            # CUDA path at the benchmark's own widths (2-layer truncation, graph replays)
            tps, cores, sample, _ = cpu_reference_step(synth.llama_config("llama2-7b"), synth, 2, 1)
            line["cpu_baseline"] = {"value": tps, "unit": "tokens/s", "cores": cores, "kind": "port", "sample": sample}
            del graph, graph_base, eng, kv, pm
            torch.cuda.empty_cache()
            from oracle import parity as oparity
            line["parity"] = oparity.decode_parity_at_benchmark_shape(load, dev)
        else:
            line["cpu_baseline"] = None
            line["parity"] = None
    if dist is not None:
        dist.barrier()
        dist.destroy_process_group()
    if line is not None:
        emit(line)


def ncu_traffic():
    """DRAM read + write bytes of one ncu-captured launch of each hot kernel next to that launch's algorithmic
    bytes, from profiles/ncu_traffic.txt (lines: kernel  dram_read_MB  dram_write_MB  algorithmic_MB  summary)."""
    out = {}
    path = os.path.join(ROOT, "profiles", "ncu_traffic.txt")
    if os.path.exists(path):
        with open(path) as f:
            for ln in f:
                parts = ln.split()
                if len(parts) >= 5 and not ln.startswith("#"):
                    rd, wr, alg = (float(x) for x in parts[1:4])
                    out[parts[0]] = ((rd + wr) / alg, f"profiles/{parts[4]} ({rd + wr:.1f} MB of DRAM traffic for {alg:.1f} MB algorithmic)")
    return out


def kernel_rooflines(eng, pm, kv, B, slots, ops, torch, ctx, n_uniq, peak, reps=5):
    """CUDA-event timing of (a) every tensor-core projection launch of one decode step and (b) every
    paged-attention launch of one step, each captured alone in a graph and replayed back to back.
    The operands cycle through all layers' weights / KV pages (13 GB / ~9 GB), far beyond L2."""
    T = B
    sl = eng.slots[:T]
    x, act, qkv, attn, y = eng.xn[:T], eng.act[:T], eng.qkv[:T], eng.attn[:T], eng.y[:T]
    peak_src = "measured" if os.path.exists(os.path.join(ROOT, "MEASURED_PEAKS.json")) else "fallback"

    def u_for(st):
        r_tot = st.r_max * st.n_mod
        return eng.u.view(-1)[: T * r_tot].view(T, r_tot)

    def lin_bytes(W, st, out_f32=False, silu=False):
        out_f, in_f = W.shape
        b = 2 * out_f * in_f + 2 * T * in_f + (4 if out_f32 else 2) * T * (out_f // 2 if silu else out_f)
        if st is not None:
            b += n_uniq * 2 * out_f * st.r_max + 4 * T + 4 * T * st.r_max * st.n_mod
        return b

    def linears():
        n, total = 0, 0
        for lw in pm.layers:
            for W, key, src, dst, fl in ((lw.w_qkv, "qkv", x, qkv, 0), (lw.w_o, "o", attn, y, 0),
                                         (lw.w_gu, "gu", x, act, ops.SILU_MUL), (lw.w_down, "down", act, y, 0)):
                st = lw.lora.get(key)
                if st is not None:
                    ops.linear(src, W, st, sl, u=u_for(st), flags=fl, out=dst, work=eng.ws_linear)
                else:  # as the engine issues it: same kernel variant as the LoRA projections around it
                    ops.linear(src, W, flags=fl | ops.SHARE_LORA_KERNEL, out=dst, work=eng.ws_linear)
                n += 1
                total += lin_bytes(W, st, silu=bool(fl & ops.SILU_MUL))
        ops.linear(x, pm.lm_head, flags=ops.OUT_F32 | ops.SHARE_LORA_KERNEL, out=eng.logits[:T], work=eng.ws_linear)
        return n + 1, total + lin_bytes(pm.lm_head, None, out_f32=True)

    def attentions():
        for l in range(pm.L):
            ops.paged_attention(qkv, kv.k_pages(l), kv.v_pages(l), kv.block_table, eng.row_slot[:T], eng.row_pos[:T],
                                pm.Hq, pm.Hkv, pm.D, kv.page_size, pm.theta, True, out=attn, work=eng.ws_attn)
        return pm.L, pm.L * (T * (ctx + 1) * 2 * pm.Hkv * pm.D * 2 + T * (pm.Hq + 2 * pm.Hkv) * pm.D * 2
                             + T * pm.Hq * pm.D * 2)

    eng.row_pos[:T].fill_(ctx)
    out = {}
    traffic = ncu_traffic()
    for name, fn, kernel in (("linear", linears, "linear_tc_kernel"), ("attention", attentions, "paged_attn_kernel")):
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            n, total = fn()
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            fn()
        for _ in range(3):
            g.replay()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        e0.record()
        for _ in range(reps):
            g.replay()
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1) / reps
        achieved = total / (ms * 1e6)
        out[name] = {"bound": "hbm", "kernel": kernel, "achieved": achieved, "peak": peak, "unit": "GB/s",
                     "frac": achieved / peak, "peak_source": peak_src + " copy bandwidth",
                     "launches": n, "avg_launch_us": 1e3 * ms / n, "algorithmic_bytes_per_launch": total / n,
                     # DRAM read+write bytes per launch: ncu capture of one launch of this kernel at the benchmark's
                     # shapes (profiles/), as a ratio to that launch's algorithmic bytes, applied to the step's
                     # average launch (traffic grows in proportion: the weights / KV pages dominate both)
                     "traffic": traffic[name][0] * total / n if name in traffic else None,
                     "traffic_source": traffic[name][1] if name in traffic else None}
    return out


def operator_rows(ops, synth, dev, torch):
    """The operator micro-benchmark: y = x W^T + 2 (x A[id]) B[id], W [4096,4096], 16 rank-16 adapters,
    T in {1, 8, 32, 128} (shapes of tvm/lora_only/single_rank.py).  CUDA-event time of the shrink +
    projection pair (one mlora_lora_linear call) in a graph over 20 weight copies (671 MB, beyond L2); one JSON line."""
    peak, src = measured_peak()
    rows = []
    for T in (1, 8, 32, 128):
        c = synth.operator_case(T, device=dev)
        Ws = [ops.PackedWeight((torch.randn(4096, 4096, device=dev) * 0.02).to(torch.bfloat16)) for _ in range(20)]
        st = ops.LoraStack(c["A"], c["B"], torch.full((N_ADAPTERS,), RANK, dtype=torch.int32, device=dev),
                           torch.full((N_ADAPTERS,), c["scale"], device=dev), RANK, 1, (0, 4096)).pack_b()
        slots = c["ids"].to(torch.int32)
        out = torch.empty(T, 4096, dtype=torch.bfloat16, device=dev)
        res = {}
        u = torch.empty(T, RANK, dtype=torch.float32, device=dev)
        for name in ("lora", "base"):
            def body():
                for W in Ws:
                    if name == "lora":  # mlora_lora_linear: shrink kernel, then projection with the expand fused in
                        ops.linear(c["x"], W, st, slots, u=u, out=out, with_shrink=True)
                    else:
                        ops.linear(c["x"], W, out=out)
            body()
            torch.cuda.synchronize()
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g):
                body()
            for _ in range(3):
                g.replay()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            torch.cuda.synchronize()
            e0.record()
            for _ in range(5):
                g.replay()
            e1.record()
            torch.cuda.synchronize()
            res[name] = 1e3 * e0.elapsed_time(e1) / (5 * len(Ws))
        n_uniq = len(set(slots.tolist()))
        by = 2 * 4096 * 4096 + n_uniq * 2 * RANK * (4096 + 4096) + 2 * T * 4096 * 2 + 4 * T
        rows.append({"T": T, "us_with_lora": res["lora"], "us_base_only": res["base"],
                     "lora_overhead_frac": res["lora"] / res["base"] - 1.0, "algorithmic_bytes": by,
                     "achieved_gbs": by / (res["lora"] * 1e3), "frac_of_peak": by / (res["lora"] * 1e3) / peak})
    return {"case": "y = x W^T + 2 (x A[id]) B[id], W [4096,4096] bf16, 16 rank-16 adapters, ids uniform; shrink + "
                    "projection as one mlora_lora_linear call, CUDA-event timed in a graph over 20 weight copies",
            "peak_gbs": peak, "peak_source": src, "rows": rows}


def run_operator_case(ops, synth, dev, torch):
    emit(dict(operator_rows(ops, synth, dev, torch), kernel_case="operator"))


def run_kernel_case(which):
    """A few launches of one hot kernel on a case sized for an ncu capture: operands larger than L2
    (126 MB) but well under 1 GB, decode shapes of the benchmark."""
    import torch

    ops, synth = load("ops"), load("synth")
    load("build").build()
    dev = torch.device("cuda", 0)
    T = N_REQ
    if which == "operator":
        return run_operator_case(ops, synth, dev, torch)
    if which == "linear":
        # the q/k/v projection of one layer with its LoRA stack: 4 weight copies = 403 MB
        c = synth.operator_case(T, 4096, 12288, N_ADAPTERS, RANK, device=dev)
        Ws = [ops.PackedWeight((torch.randn(12288, 4096, device=dev) * 0.02).to(torch.bfloat16)) for _ in range(4)]
        A = torch.cat([c["A"]] * 3, 1).contiguous()
        st = ops.LoraStack(A, c["B"], torch.full((N_ADAPTERS,), RANK, dtype=torch.int32, device=dev),
                           torch.full((N_ADAPTERS,), ALPHA / RANK, device=dev), RANK, 3, (0, 4096, 8192, 12288)).pack_b()
        slots = c["ids"].to(torch.int32)
        u = ops.lora_shrink(c["x"], st, slots)
        out = torch.empty(T, 12288, dtype=torch.bfloat16, device=dev)
        for i in range(6):
            ops.linear(c["x"], Ws[i % 4], st, slots, u=u, out=out)
        # CUDA-event time of the same launch, warm, inside a graph (4 weight copies per replay)
        torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            for W in Ws:
                ops.linear(c["x"], W, st, slots, u=u, out=out)
        for _ in range(3):
            g.replay()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(10):
            g.replay()
        e1.record()
        torch.cuda.synchronize()
        us = 1e3 * e0.elapsed_time(e1) / 40
        by = 2 * 12288 * 4096 + len(set(slots.tolist())) * 2 * 12288 * RANK + 2 * T * 4096 + 2 * T * 12288 + 4 * T + 4 * T * 3 * RANK
        peak, src = measured_peak()
        emit({"kernel_case": which, "us_per_launch": us, "algorithmic_bytes": by, "achieved_gbs": by / us / 1e3,
                          "frac_of_peak": by / us / 1e3 / peak, "peak_source": src, "launches": ops.launch_count()})
        return
    elif which == "chain":
        # one layer segment of the benchmark's model as ONE persistent launch (mlora_decode_chain): o -> norm -> gate|up
        # -> down -> norm + q/k/v shrink -> q/k/v, 32 rows, 16 rank-16 adapters on q/k/v/o; two weight sets = 810 MB
        model_mod = load("model")
        H, I, r = 4096, 11008, RANK
        g = torch.Generator(device=dev).manual_seed(0)
        mat = lambda o, i: (torch.randn(o, i, device=dev, generator=g) * 0.02).to(torch.bfloat16)

        def stack(in_f, outs):
            n_mod = len(outs)
            A = ((torch.rand(N_ADAPTERS, n_mod * r, in_f, device=dev, generator=g) * 2 - 1) / in_f ** 0.5).to(torch.bfloat16)
            B = (torch.randn(N_ADAPTERS, sum(outs), r, device=dev, generator=g) * 0.02).to(torch.bfloat16)
            offs = [0]
            for o in outs:
                offs.append(offs[-1] + o)
            return ops.LoraStack(A, B, torch.full((N_ADAPTERS,), r, dtype=torch.int32, device=dev),
                                 torch.full((N_ADAPTERS,), ALPHA / RANK, device=dev), r, n_mod, tuple(offs)).pack_b()
        sets = []
        for _ in range(2):
            sets.append(dict(w_o=ops.PackedWeight(mat(H, H)), w_gu=ops.PackedWeight(model_mod.interleave_gate_up(mat(I, H), mat(I, H))),
                             w_down=ops.PackedWeight(mat(H, I)), w_qkv=ops.PackedWeight(mat(3 * H, H)),
                             st_o=stack(H, [H]), st_qkv=stack(H, [H, H, H])))
        ln = (1 + 0.1 * torch.randn(H, device=dev, generator=g)).to(torch.bfloat16)
        attn = torch.randn(T, H, device=dev, generator=g).to(torch.bfloat16)
        res = torch.randn(T, H, device=dev, generator=g)
        y, xn, act, qkv = (torch.zeros(T, n, dtype=torch.bfloat16, device=dev) for n in (H, H, I, 3 * H))
        u = torch.zeros(T, 3 * r, dtype=torch.float32, device=dev)
        slots = torch.from_numpy(synth.adapter_ids_uniform(T, N_ADAPTERS)).to(dev)
        lib = load("_lib").lib()
        work = ops.new_workspace(max(lib.mlora_linear_workspace(T, k, n) for k, n in ((H, H), (H, 2 * I), (I, H), (H, 3 * H))), dev)

        def segment(c):
            S = ops.ChainStep
            ops.decode_chain([S(x=attn, W=c["w_o"], y=y, stack=c["st_o"], u=u.view(-1)[: T * r].view(T, r)),
                              S(x=xn, W=c["w_gu"], y=act, flags=ops.SILU_MUL, res=res, delta=y, norm_w=ln, eps=1e-5),
                              S(x=act, W=c["w_down"], y=y),
                              S(x=xn, W=c["w_qkv"], y=qkv, res=res, delta=y, norm_w=ln, eps=1e-5, stack=c["st_qkv"], u=u)],
                             slots, c["st_o"].ranks, c["st_o"].scales, N_ADAPTERS, work)
        for i in range(4):
            segment(sets[i % 2])
        torch.cuda.synchronize()
        gr = torch.cuda.CUDAGraph()
        with torch.cuda.graph(gr):
            for c in sets:
                segment(c)
        for _ in range(3):
            gr.replay()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(10):
            gr.replay()
        e1.record()
        torch.cuda.synchronize()
        us = 1e3 * e0.elapsed_time(e1) / 20
        n_uniq = len(set(slots.tolist()))
        by = 2 * (4 * H * H + 3 * H * I) + n_uniq * 2 * r * (H + H + H + 3 * H) + 2 * T * (H + H + I + H) + 2 * T * (H + I + H + 3 * H) + 2 * 8 * T * H
        peak, src = measured_peak()
        emit({"kernel_case": which, "us_per_launch": us, "algorithmic_bytes": by, "achieved_gbs": by / us / 1e3,
              "frac_of_peak": by / us / 1e3 / peak, "peak_source": src, "status": ops.status_word(work), "launches": ops.launch_count()})
        return
    elif which == "expand":
        # a 13B-shaped projection (5120 x 5120) over 128 rows that each bring their own adapter (128 adapters, ranks
        # cycling 8/16/32/64 in a pitch-64 stack): base projection + per-row expand, CUDA-event timed in a graph
        T, H, n_ad, rp = 128, 5120, 128, 64
        g = torch.Generator(device=dev).manual_seed(0)
        x = torch.randn(T, H, device=dev, generator=g).to(torch.bfloat16)
        Ws = [ops.PackedWeight((torch.randn(H, H, device=dev, generator=g) * 0.02).to(torch.bfloat16)) for _ in range(6)]
        ranks = [(8, 16, 32, 64)[i % 4] for i in range(n_ad)]
        A = (torch.randn(n_ad, rp, H, device=dev, generator=g) * 0.02).to(torch.bfloat16)
        B = (torch.randn(n_ad, H, rp, device=dev, generator=g) * 0.02).to(torch.bfloat16)
        for i, r in enumerate(ranks):
            A[i, r:] = 0
            B[i, :, r:] = 0
        mk = lambda: ops.LoraStack(A, B.clone(), torch.tensor(ranks, dtype=torch.int32, device=dev),
                                   torch.full((n_ad,), 0.5, device=dev), rp, 1, (0, H))
        st = mk().pack_b()                       # padded to the rank pitch (pre-tiled)
        st_split = mk().split_b(ranks).pack_b()  # + the rank-compact copy the per-row expand prefers
        slots = torch.randperm(n_ad, device=dev, generator=g)[:T].to(torch.int32)
        out = torch.empty(T, H, dtype=torch.bfloat16, device=dev)
        u = torch.empty(T, rp, dtype=torch.float32, device=dev)
        res = {}
        for name in ("base", "shrink", "per_row_padded", "tensor_core_stages", "per_row_split"):
            def body():
                for W in Ws:
                    if name == "base":
                        ops.linear(x, W, out=out)
                    elif name == "shrink":
                        ops.lora_shrink(x, st, slots, out=u)
                    elif name == "per_row_split":
                        ops.linear(x, W, st_split, slots, u=u, out=out, flags=ops.LORA_PER_ROW)
                    else:
                        ops.linear(x, W, st, slots, u=u, out=out, flags=ops.LORA_PER_ROW if name == "per_row_padded" else 0)
            body()
            torch.cuda.synchronize()
            gr = torch.cuda.CUDAGraph()
            with torch.cuda.graph(gr):
                body()
            gr.replay()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(3):
                gr.replay()
            e1.record()
            torch.cuda.synchronize()
            res[name] = 1e3 * e0.elapsed_time(e1) / (3 * len(Ws))
        emit({"kernel_case": which, "us": res, "bytes_W": 2 * H * H, "bytes_B_by_rank": sum(2 * H * r for r in ranks),
              "bytes_B_padded": n_ad * 2 * H * rp, "status": ops.status_word(ops.workspace(4, dev, "linear")),
              "launches": ops.launch_count()})
        return
    elif which == "prefill":
        # prefill-size q/k/v projection: 8192 prompt rows (16 requests x 512, one adapter per request), shrink as
        # a grouped GEMM + projection with the expand as extra MMA stages; CUDA-event TFLOP/s of the pair
        T = 8192
        c = synth.operator_case(T, 4096, 12288, N_ADAPTERS, RANK, device=dev)
        W = ops.PackedWeight((torch.randn(12288, 4096, device=dev) * 0.02).to(torch.bfloat16))
        A = torch.cat([c["A"]] * 3, 1).contiguous()
        st = ops.LoraStack(A, c["B"], torch.full((N_ADAPTERS,), RANK, dtype=torch.int32, device=dev),
                           torch.full((N_ADAPTERS,), ALPHA / RANK, device=dev), RANK, 3, (0, 4096, 8192, 12288)).pack_b()
        slots = torch.arange(T, device=dev, dtype=torch.int32) // 512 % N_ADAPTERS
        out = torch.empty(T, 12288, dtype=torch.bfloat16, device=dev)
        u = torch.empty(T, 3 * RANK, dtype=torch.float32, device=dev)
        res = {}
        for name in ("base", "lora"):
            ev = [torch.cuda.Event(enable_timing=True) for _ in range(2)]
            for i in range(5):
                if i == 2:
                    ev[0].record()
                if name == "lora":
                    ops.lora_shrink(c["x"], st, slots, out=u)
                    ops.linear(c["x"], W, st, slots, u=u, out=out)
                else:
                    ops.linear(c["x"], W, out=out)
            ev[1].record()
            torch.cuda.synchronize()
            res[name] = ev[0].elapsed_time(ev[1]) / 3
        fl = 2.0 * T * 4096 * 12288
        peaks = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json"))) if os.path.exists(os.path.join(ROOT, "MEASURED_PEAKS.json")) else {}
        tpk = float(peaks.get("bf16_tflops", 1590.0))  # burst figure: the kernel is timed alone
        emit({"kernel_case": which, "T": T, "ms_base": res["base"], "ms_with_lora": res["lora"],
                          "tflops_base": fl / res["base"] / 1e9, "tflops_with_lora": (fl + 2.0 * T * 48 * (4096 + 4096)) / res["lora"] / 1e9,
                          "peak_tflops": tpk, "frac_base": fl / res["base"] / 1e9 / tpk,
                          "status": ops.status_word(ops.workspace(4, dev, "linear")), "launches": ops.launch_count()})
        return
    elif which == "prefill-lora":
        # what the LoRA expand adds to a prompt-size projection, by shape of the batch: the q/k/v projection of 8192 rows
        # with no adapter, one adapter per 256-token tile, four per tile; rank-16 and rank-64 stacks; CUDA events
        T, NA = 8192, 16
        x = (torch.randn(T, 4096, device=dev) * 0.5).to(torch.bfloat16)
        W = ops.PackedWeight((torch.randn(12288, 4096, device=dev) * 0.02).to(torch.bfloat16))
        out = torch.empty(T, 12288, dtype=torch.bfloat16, device=dev)

        def timed(fn):
            ev = [torch.cuda.Event(enable_timing=True) for _ in range(2)]
            for i in range(6):
                if i == 2:
                    ev[0].record()
                fn()
            ev[1].record()
            torch.cuda.synchronize()
            return ev[0].elapsed_time(ev[1]) / 4 * 1e3

        rows = {"base_us": timed(lambda: ops.linear(x, W, out=out))}
        for R in (16, 64):
            A = (torch.randn(NA, 3 * R, 4096, device=dev) * 0.02).to(torch.bfloat16)
            B = (torch.randn(NA, 12288, R, device=dev) * 0.02).to(torch.bfloat16)
            st = ops.LoraStack(A, B, torch.full((NA,), R, dtype=torch.int32, device=dev), torch.full((NA,), 2.0, device=dev),
                               R, 3, (0, 4096, 8192, 12288)).pack_b()
            u = torch.zeros(T, 3 * R, dtype=torch.float32, device=dev)
            ar = torch.arange(T, device=dev, dtype=torch.int32)
            cases = {"no_adapter": torch.full((T,), -1, dtype=torch.int32, device=dev), "one_per_tile": ar // 512 % NA,
                     "four_per_tile": ar // 64 % NA}
            for name, slots in cases.items():
                rows[f"rank{R}_expand_{name}_us"] = timed(lambda: ops.linear(x, W, st, slots, u=u, out=out))
            slots = cases["one_per_tile"]
            rows[f"rank{R}_shrink_us"] = timed(lambda: ops.lora_shrink(x, st, slots, out=u))
            rows[f"rank{R}_shrink_plus_expand_us"] = timed(lambda: (ops.lora_shrink(x, st, slots, out=u),
                                                                     ops.linear(x, W, st, slots, u=u, out=out)))
        emit(dict(rows, kernel_case=which, T=T, status=ops.status_word(ops.workspace(4, dev, "linear")), launches=ops.launch_count()))
        return
    elif which == "prefill-attn":
        # one layer's prompt attention: 16 requests x 512 rows, 32 x 128 heads, keys / values appended first
        Hq = Hkv = 32
        D, S, n_seq = 128, 512, 16
        T = S * n_seq
        n_pg = S // PAGE
        kp = torch.zeros(n_seq * n_pg, Hkv, PAGE, D, device=dev, dtype=torch.bfloat16)
        vp = torch.zeros_like(kp)
        bt = torch.randperm(n_seq * n_pg, device=dev).to(torch.int32).view(n_seq, n_pg)
        qkv = torch.randn(T, 3 * Hq * D, device=dev, dtype=torch.bfloat16)
        slot = torch.arange(T, device=dev, dtype=torch.int32) // S
        pos = torch.arange(T, device=dev, dtype=torch.int32) % S
        tiles = torch.tensor([(q, q * S + o, 128, o) for q in range(n_seq) for o in range(0, S, 128)], dtype=torch.int32, device=dev)
        out = torch.empty(T, Hq * D, dtype=torch.bfloat16, device=dev)
        status = torch.zeros(1, dtype=torch.int32, device=dev)
        ev = [torch.cuda.Event(enable_timing=True) for _ in range(4)]
        for i in range(5):
            if i == 2:
                ev[0].record()
            ops.kv_append_rope(qkv, kp, vp, bt, slot, pos, Hq, Hkv, D, PAGE, 10000.0)
        ev[1].record()
        for i in range(5):
            if i == 2:
                ev[2].record()
            ops.prefill_attention(qkv, kp, vp, bt, tiles, tiles.shape[0], Hq, Hkv, D, PAGE, out, status)
        ev[3].record()
        torch.cuda.synchronize()
        us_app, us_att = ev[0].elapsed_time(ev[1]) / 3 * 1e3, ev[2].elapsed_time(ev[3]) / 3 * 1e3
        fl = 4.0 * Hq * D * n_seq * S * (S + 1) / 2
        by_app = T * 3 * Hq * D * 2 + T * Hq * D * 2 + 2 * T * Hkv * D * 2  # read q|k|v, write q, k and v pages
        emit({"kernel_case": which, "rows": T, "us_append_rope": us_app, "append_rope_gbs": by_app / us_app / 1e3,
              "us_attention": us_att, "attention_tflops_causal": fl / us_att / 1e6, "status": int(status.item()),
              "launches": ops.launch_count()})
        return
    else:
        # one layer's attention at context 576: 32 rows x 32 heads, 302 MB of KV
        Hq = Hkv = 32
        D, ctx = 128, 576
        n_pg = ctx // PAGE + 1
        kp = torch.randn(T * n_pg, Hkv, PAGE, D, device=dev, dtype=torch.bfloat16)
        vp = torch.randn(T * n_pg, Hkv, PAGE, D, device=dev, dtype=torch.bfloat16)
        bt = torch.arange(T * n_pg, device=dev, dtype=torch.int32).view(T, n_pg)
        qkv = torch.randn(T, 3 * Hq * D, device=dev, dtype=torch.bfloat16)
        slot = torch.arange(T, device=dev, dtype=torch.int32)
        pos = torch.full((T,), ctx, device=dev, dtype=torch.int32)
        for _ in range(4):
            ops.paged_attention(qkv, kp, vp, bt, slot, pos, Hq, Hkv, D, PAGE, 10000.0, True)
    torch.cuda.synchronize()
    emit({"kernel_case": which, "launches": ops.launch_count()})


_RESULT_FD = None


def emit(line: dict):
    """The result line, on the process's original stdout."""
    data = (json.dumps(line) + "\n").encode()
    if _RESULT_FD is None:
        sys.stdout.write(data.decode())
        sys.stdout.flush()
    else:
        os.write(_RESULT_FD, data)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=128)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--layers", type=int, default=0, help="debug: truncate the model (the number is then not a bench value)")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--no-operator", action="store_true", help="skip the operator micro-benchmark rows")
    ap.add_argument("--scaling", default="weak", choices=["weak", "strong"],
                    help="weak (the benchmark): 32 requests and 16 adapters PER GPU; strong (side line): the same 32 requests "
                         "spread over the GPUs by adapter")
    ap.add_argument("--tp-collective", default="nccl", choices=["nccl", "peer"],
                    help="13b-tp workload: the exchange after row-parallel projections -- NCCL all-reduce + norm kernel, or "
                         "the library's fused peer-memory kernel")
    ap.add_argument("--skip-prefill", action="store_true",
                    help="profiling aid: fill the KV cache with seeded random values instead of running prefill "
                         "(the number is then not a bench value)")
    ap.add_argument("--kernel-case", default="", choices=["", "linear", "attention", "operator", "prefill", "prefill-lora", "prefill-attn", "expand", "chain"],
                    help="profiling aid: launch one kernel a few times on a small case (> L2, < 1 GB) and exit")
    ap.add_argument("--workload", default="", choices=["", "13b-shape", "13b-tp", "prefill-heavy"],
                    help="side measurements (own JSON line, not the benchmark's): 13b-shape = the 13B shape and adapter "
                         "mix on one GPU; 13b-tp = the tensor-parallel configuration, tp size = number of ranks "
                         "(launch with torch.distributed.run); prefill-heavy = 64 x 512-token prompts, 64 rank-64 adapters on "
                         "seven projections, Zipf ids, 16 decode tokens")
    args = ap.parse_args()
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    # stdout carries exactly one line, the JSON: whatever libraries write to file descriptor 1 meanwhile (NCCL prints its
    # version banner there) goes to stderr
    global _RESULT_FD
    sys.stdout.flush()
    _RESULT_FD = os.dup(1)
    os.dup2(2, 1)
    if args.workload == "13b-shape":
        run_13b_shape(args)
    elif args.workload == "13b-tp":
        run_13b_tp(args, rank, world, local_rank)
    elif args.workload == "prefill-heavy":
        run_prefill_heavy(args)
    elif args.kernel_case:
        run_kernel_case(args.kernel_case)
    elif args.impl == "reference":
        run_reference(args, rank, world)
    else:
        run_ours(args, rank, world, local_rank)


if __name__ == "__main__":
    main()
