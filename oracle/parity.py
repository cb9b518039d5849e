"""Parity check of the CUDA decode path at the benchmark's own shapes.  TEST INFRASTRUCTURE ONLY.

Runs a layer-truncated model of the benchmark's shape (Llama-2-7B widths: hidden 4096, 32 x 128 heads,
intermediate 11008, vocabulary 32000; 32 requests over 16 rank-16 adapters on q/k/v/o) through the
product's engine on the GPU -- prefill, then teacher-forced decode steps as CUDA-graph replays, i.e. the
exact kernels, tile splits and fusions the timed benchmark runs -- and compares with
``oracle.llama.OracleLlama`` (fp32, CPU) on the same bf16-rounded weights.  Used by
``tests/test_model_gpu.py`` (which asserts the bars) and by the CPU-baseline leg of ``bench.py`` (which
prints the figures beside the timing).  The product package never imports this module.
"""
from __future__ import annotations

import torch

from . import bucketing
from . import llama as ollama

ATOL, RTOL = 2e-2, 1e-2  # bf16 logits against the fp32 oracle


def _rel_excess(got, want):
    """max over elements of |got-want| / (ATOL + RTOL*|want|): <= 1 means inside the stated tolerance."""
    return float(((got - want).abs() / (ATOL + RTOL * want.abs())).max())


def decode_parity_at_benchmark_shape(load, device, layers=2, n_req=32, n_adapters=16, rank=16, alpha=32,
                                     prompt_len=64, steps=4, config="llama2-7b", use_graph=True):
    """``load(sub)`` imports a module of the product package.  Returns a dict of figures:
    logits_max_abs, logits_rel (worst |diff| / (atol + rtol |want|)), greedy_agree (teacher-forced
    fraction of equal argmax), ids_bit_exact (device bucketing of the batch's adapter ids == oracle),
    tc_status_word, positions compared."""
    synth, model_mod, kv_mod, ops = load("synth"), load("model"), load("kv_cache"), load("ops")
    cfg = dict(synth.llama_config(config), num_hidden_layers=layers)
    w = {k: v.bfloat16() for k, v in synth.base_weights(cfg).items()}
    ads = [{k: v.bfloat16() for k, v in a.items()} for a in synth.lora_adapters(cfg, n_adapters, rank)]
    scales = [alpha / rank] * n_adapters
    ids = [int(i) for i in synth.adapter_ids_uniform(n_req, n_adapters)]
    P = synth.prompts(n_req, prompt_len, cfg["vocab_size"])
    oracle = ollama.OracleLlama(cfg, w, ads, scales)
    want_tok, want_logits = oracle.greedy([list(p) for p in P], ids, steps + 1)

    pm = model_mod.PackedLlama(cfg, w, ads, scales, device=device)
    max_len = prompt_len + steps + 2
    kv = kv_mod.PagedKVCache(pm.L, pm.Hkv, pm.D, n_req, n_req * max_len, prompt_len, 16, device, max_seq_len=max_len)
    eng = model_mod.Engine(pm, kv, max_rows=max(n_req * prompt_len // 2, n_req))  # two prefill passes
    sids = list(range(n_req))
    for s in sids:
        kv.add_sequence(s)
    lg, tok = eng.prefill(sids, [list(p) for p in P], ids)
    got = [lg.float().cpu()]
    agree = int((tok.cpu() == want_tok[:, 0]).sum())
    graph = eng.capture_decode(sids, ids, reserve_tokens=steps + 1, feed_back=False) if use_graph else None
    for step in range(1, steps + 1):
        feed = want_tok[:, step - 1].to(torch.int32)
        if graph is not None:
            eng.tokens[:n_req].copy_(feed.to(device))
            graph.replay()
            lg, tok = eng.logits[:n_req], eng.next_tok[:n_req]
        else:
            lg, tok = eng.decode(sids, feed.tolist(), ids)
        got.append(lg.float().cpu().clone())
        agree += int((tok.cpu() == want_tok[:, step]).sum())
    torch.cuda.synchronize()
    max_abs = max(float((g - w_).abs().max()) for g, w_ in zip(got, want_logits))
    rel = max(_rel_excess(g, w_) for g, w_ in zip(got, want_logits))

    # request -> adapter bucketing of this batch on the device against the oracle's stable sort
    wids = torch.tensor(ids, dtype=torch.int32, device=device)
    b = ops.bucket_sort(None, wids, 1, n_adapters)
    perm, off, seg = bucketing.segment_sort(ids)
    n_seg = int(b.counts[0])
    ids_ok = (n_seg == len(seg) and b.perm.cpu().tolist() == perm.tolist()
              and b.seg_offsets[: n_seg + 1].cpu().tolist() == off.tolist()
              and b.seg_wid[:n_seg].cpu().tolist() == seg.tolist())
    status = int(eng.status_word())
    return {"logits_max_abs": max_abs, "logits_rel": rel, "greedy_agree": agree / (n_req * (steps + 1)),
            "ids_bit_exact": bool(ids_ok), "tc_status_word": status, "positions": n_req * (steps + 1),
            "case": f"{config} widths, {layers} layers, {n_req} requests x {n_adapters} rank-{rank} adapters, "
                    f"{prompt_len}-token prompts, prefill + {steps} teacher-forced decode steps"
                    f"{' as CUDA-graph replays' if use_graph else ''} vs fp32 CPU oracle",
            "tolerance": {"atol": ATOL, "rtol": RTOL, "greedy_agree_min": 0.95}}
