"""Parity check of the CUDA decode path at the benchmark's own shapes.  TEST INFRASTRUCTURE ONLY.

Runs a layer-truncated model of the benchmark's shape (Llama-2-7B widths: hidden 4096, 32 x 128 heads,
intermediate 11008, vocabulary 32000; 32 requests over 16 rank-16 adapters on q/k/v/o) through the
product's engine on the GPU -- prefill, then teacher-forced decode steps as CUDA-graph replays, i.e. the
exact kernels, tile splits and fusions the timed benchmark runs -- and compares with
``oracle.llama.OracleLlama`` on the same bf16-rounded weights, twice: against the all-fp32 form, and against
the form that rounds the stored activations to bf16 where the CUDA path stores them (arithmetic still fp32).
With N(0, 0.02) random-init weights the logits of this shape have a standard deviation of about 1.28 (0.32 for
the 256-wide plumbing model), and bf16 storage of activations alone -- the second form against the first, no
GPU involved -- moves them by up to 0.086 (rms 0.016).  Two bf16 pipelines with different summation orders
differ from each other by about as much, so the max-abs 2e-2 bar (6 % of a logit standard deviation on the
plumbing model, where the other tests assert it) cannot be met by ANY pipeline that stores bf16 activations at
this logit scale.  What is checked here instead: the CUDA path's error against the fp32 form is no larger than
the error bf16 storage alone causes (max-abs and rms, 30 % slack for the extreme-value statistic), the bar in
units of the logit scale, and greedy agreement.  Used by
``tests/test_model_gpu.py`` (which asserts the bars) and by the CPU-baseline leg of ``bench.py`` (which
prints the figures beside the timing).  The product package never imports this module.
"""
from __future__ import annotations

import torch

from . import bucketing
from . import llama as ollama

ATOL, RTOL = 2e-2, 1e-2  # bf16 logits against the fp32 oracle


PLUMBING_LOGIT_STD = 0.32  # logit standard deviation of the 256-wide plumbing model the 2e-2 bar is quoted on


def _rel_excess(got, want, atol_scale=1.0):
    """max over elements of |got-want| / (atol_scale*ATOL + RTOL*|want|): <= 1 means inside the tolerance."""
    return float(((got - want).abs() / (atol_scale * ATOL + RTOL * want.abs())).max())


def decode_parity_at_benchmark_shape(load, device, layers=2, n_req=32, n_adapters=16, rank=16, alpha=32,
                                     prompt_len=64, steps=4, config="llama2-7b", use_graph=True):
    """``load(sub)`` imports a module of the product package.  Returns a dict of figures:
    logits_max_abs / logits_rms_err / logits_rel against the fp32 form (logits_rel = worst |diff| / (s*atol + rtol
    |want|) with s = logit_std / 0.32, see the module text), bf16_storage_alone_max_abs / _rms_err (the two CPU
    forms against each other: what bf16 activation storage costs by itself), greedy_agree (teacher-forced
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
    # the same tokens through the bf16-activation-storage form (teacher-forced with the fp32 form's tokens)
    emu = ollama.OracleLlama(cfg, w, ads, scales, act_dtype=torch.bfloat16)
    emu_logits = [torch.cat([emu.prefill(b, list(P[b]), ids[b]) for b in range(n_req)])]
    for step in range(1, steps + 1):
        emu_logits.append(emu.decode(list(range(n_req)), want_tok[:, step - 1].tolist(), ids))

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
    sigma = float(torch.cat(want_logits).std())
    scale = max(1.0, sigma / PLUMBING_LOGIT_STD)
    rel = max(_rel_excess(g, w_, scale) for g, w_ in zip(got, want_logits))
    rms = lambda a, b: float((torch.cat(a) - torch.cat(b)).pow(2).mean().sqrt())
    err_rms, storage_rms = rms(got, want_logits), rms(emu_logits, want_logits)
    emu_abs = max(float((g - w_).abs().max()) for g, w_ in zip(got, emu_logits))
    storage_abs = max(float((a - b).abs().max()) for a, b in zip(emu_logits, want_logits))

    # request -> adapter bucketing of this batch on the device against the oracle's stable sort
    wids = torch.tensor(ids, dtype=torch.int32, device=device)
    b = ops.bucket_sort(None, wids, 1, n_adapters)
    perm, off, seg = bucketing.segment_sort(ids)
    n_seg = int(b.counts[0])
    ids_ok = (n_seg == len(seg) and b.perm.cpu().tolist() == perm.tolist()
              and b.seg_offsets[: n_seg + 1].cpu().tolist() == off.tolist()
              and b.seg_wid[:n_seg].cpu().tolist() == seg.tolist())
    status = int(eng.status_word())
    return {"logits_max_abs": max_abs, "logits_rel": rel, "logit_std": sigma, "atol_scale_vs_fp32": scale,
            "logits_rms_err": err_rms, "bf16_storage_alone_max_abs": storage_abs,
            "bf16_storage_alone_rms_err": storage_rms, "logits_max_abs_vs_bf16_storage_oracle": emu_abs,
            "greedy_agree": agree / (n_req * (steps + 1)),
            "ids_bit_exact": bool(ids_ok), "tc_status_word": status, "positions": n_req * (steps + 1),
            "case": f"{config} widths, {layers} layers, {n_req} requests x {n_adapters} rank-{rank} adapters, "
                    f"{prompt_len}-token prompts, prefill + {steps} teacher-forced decode steps"
                    f"{' as CUDA-graph replays' if use_graph else ''} vs fp32 CPU oracle",
            "tolerance": {"atol": ATOL, "rtol": RTOL, "greedy_agree_min": 0.95}}
