"""Pins the decoder-body oracle against the transformers ``LlamaForCausalLM`` installed on this machine.

The reference delegates the decoder arithmetic (RMSNorm, rotate-half RoPE, causal attention, SiLU MLP)
to third-party code -- transformers on its HuggingFace path (``huggingface/generation/gen_lora.py:28,116``)
and TVM's paged KV cache on its auto-batcher path -- and ships no golden vectors for it.  What can be
checked here is that the two CPU restatements the tests use as the checker agree with that third-party
implementation on the plumbing configuration at its full size: ``oracle.llama.OracleLlama`` (the form the
GPU parity tests compare with) and ``oracle.hf_path`` (transformers model + restated LoRA layer, the
form the CPU baseline times).  CPU only.
"""
import pytest
import torch

from conftest import load
from oracle import hf_path
from oracle import llama as ollama

# two fp32 implementations of the same arithmetic with different summation orders
LOGIT_ATOL = 1e-5


@pytest.fixture(scope="module")
def plumbing_case():
    """4 requests x 512 tokens, tiny 2-layer model, 4 rank-8 adapters (alpha 16) on q/k/v/o, ids [0,1,2,3]."""
    synth = load("synth")
    torch.set_num_threads(min(8, torch.get_num_threads()))
    cfg = synth.llama_config("tiny")
    w = synth.base_weights(cfg)
    ads = synth.lora_adapters(cfg, 4, 8)
    scales = [16 / 8] * 4
    P = synth.prompts(4, 512, cfg["vocab_size"])
    return synth, cfg, w, ads, scales, P


def test_greedy_generation_equals_transformers_on_the_plumbing_config(plumbing_case):
    """32 greedy tokens: identical token ids; teacher-forced logits within 1e-5 at every generated position."""
    synth, cfg, w, ads, scales, P = plumbing_case
    ids, gen = [0, 1, 2, 3], 32
    hf = hf_path.build_hf_model(cfg, w, ads, scales)
    prompts = torch.from_numpy(P).long()
    hf_tok = hf_path.generate(hf, prompts, ids, gen)
    oracle = ollama.OracleLlama(cfg, w, ads, scales)
    tok, logits = oracle.greedy([list(p) for p in P], ids, gen)
    assert torch.equal(tok, hf_tok)
    full = torch.cat([prompts, tok[:, :-1]], 1)
    hf_logits = hf_path.forward_logits(hf, full, ids)  # [B, S+gen-1, V]
    S = prompts.shape[1]
    worst = max(float((hf_logits[:, S - 1 + i] - logits[i]).abs().max()) for i in range(gen))
    assert worst <= LOGIT_ATOL, worst
    # the adapters matter: the base-only model generates something else
    base_tok = hf_path.generate(hf, prompts, None, gen)
    assert not torch.equal(base_tok, hf_tok)


def test_adapters_on_all_seven_projections_and_none(plumbing_case):
    """Prefill logits with adapters on q/k/v/o/gate/up/down (one rank: the gather form stacks the adapters of a
    batch, ``lora_gatherbmm_linear_layer.py:16-17``, so they share a rank), and with adapters switched off."""
    synth, cfg, w, _, _, P = plumbing_case
    ads = synth.lora_adapters(cfg, 3, 16, targets=synth.ATTN_PROJ + synth.MLP_PROJ)
    scales = [2.0, 1.0, 0.25]
    prompts = torch.from_numpy(P[:, :96]).long()
    hf = hf_path.build_hf_model(cfg, w, ads, scales)
    ids = [2, 0, 1, 0]
    want = hf_path.forward_logits(hf, prompts, ids)[:, -1]
    oracle = ollama.OracleLlama(cfg, w, ads, scales)
    got = torch.cat([oracle.prefill(b, prompts[b].tolist(), ids[b]) for b in range(4)])
    assert float((got - want).abs().max()) <= LOGIT_ATOL
    want0 = hf_path.forward_logits(hf, prompts, None)[:, -1]
    base = ollama.OracleLlama(cfg, w)
    got0 = torch.cat([base.prefill(b, prompts[b].tolist(), -1) for b in range(4)])
    assert float((got0 - want0).abs().max()) <= LOGIT_ATOL
    assert float((got0 - got).abs().max()) > 1e-3


def test_decode_step_with_cache_equals_full_forward(plumbing_case):
    """The oracle's incremental decode (dense per-sequence KV) equals a full forward over the longer sequence:
    what the paged cache must reproduce."""
    synth, cfg, w, ads, scales, P = plumbing_case
    ids = [1, 3, 3, 0]
    oracle = ollama.OracleLlama(cfg, w, ads, scales)
    for b in range(4):
        oracle.prefill(b, P[b, :40].tolist(), ids[b])
    nxt = P[:, 40].tolist()
    step = oracle.decode([0, 1, 2, 3], nxt, ids)
    fresh = ollama.OracleLlama(cfg, w, ads, scales)
    full = torch.cat([fresh.prefill(b, P[b, :41].tolist(), ids[b]) for b in range(4)])
    assert float((step - full).abs().max()) <= LOGIT_ATOL


def test_cpu_baseline_timer_runs_real_decode_steps(plumbing_case):
    """``time_decode_sample`` (the benchmark's CPU baseline): positive, increasing times for two truncations,
    a per-layer time consistent with them, and a KV cache that really holds ``ctx_len`` tokens per layer."""
    synth, cfg, _, _, _, _ = plumbing_case
    from transformers import DynamicCache

    seen = []
    orig = DynamicCache.update

    def spy(self, k, v, layer_idx, *a, **kw):
        out = orig(self, k, v, layer_idx, *a, **kw)
        seen.append((layer_idx, out[0].shape[-2]))
        return out

    DynamicCache.update = spy
    try:
        r = hf_path.time_decode_sample(
            cfg, lambda L: synth.base_weights(cfg, n_layers=L), lambda L: synth.lora_adapters(cfg, 4, 8, n_layers=L),
            [2.0] * 4, [0, 1, 2, 3], ctx_len=64, layer_counts=(1, 2), steps=1, warmup=1)
    finally:
        DynamicCache.update = orig
    (l0, t0), (l1, t1) = r["samples"]
    assert (l0, l1) == (1, 2) and t0 > 0 and t1 > 0
    assert r["per_layer_s"] >= 0 and r["full_step_s"] > 0
    assert abs(r["head_s"] + 2 * r["per_layer_s"] - r["full_step_s"]) < 1e-9  # tiny config has 2 layers
    # inside a timed step the model appended one token to a cache that already held ctx_len tokens
    assert (0, 65) in seen and (1, 65) in seen
