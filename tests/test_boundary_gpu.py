"""The two reference-facing boundaries on the GPU: the HF LoRA layer and the auto-batcher's VM function table."""
import json
import os

import numpy as np
import pytest
import torch
from torch import nn

from conftest import load
from oracle import llama as ollama, ops as oops

pytestmark = pytest.mark.gpu
G = os.path.join(os.path.dirname(__file__), "golden")
ATOL, RTOL = 2e-2, 1e-2


def test_multi_lora_linear_matches_reference_layer_golden(cuda):
    """Same forward(x, adapter_names=...) call as the reference GatherBMMLinear, same numbers (to bf16)."""
    ll = load("lora_linear")
    z = np.load(os.path.join(G, "lora_layer_golden.npz"))
    for i in range(int(z["n_cases"])):
        x = torch.from_numpy(z[f"c{i}_x"]).bfloat16()
        W = torch.from_numpy(z[f"c{i}_W"]).bfloat16()
        A = torch.from_numpy(z[f"c{i}_A"]).bfloat16()
        B = torch.from_numpy(z[f"c{i}_B"]).bfloat16()
        ids, scale = z[f"c{i}_ids"], float(z[f"c{i}_scale"])
        n, r = A.shape[0], A.shape[1]
        base = nn.Linear(W.shape[1], W.shape[0], bias=False)
        base.weight.data = W.clone()
        layer = ll.MultiLoraLinear(base.to(cuda).to(torch.bfloat16))
        for a in range(n):
            layer.update_layer(f"adapter{a}", r, scale * r)
            layer.set_adapter_weights(f"adapter{a}", A[a], B[a])
        names = [f"adapter{int(k)}" for k in ids]
        y = layer(x.to(cuda), adapter_names=names).float().cpu()
        want = oops.gather_bmm_linear(x.float(), W.float(), list(A.float()), list(B.float()), [scale] * n, ids)
        torch.testing.assert_close(y, want, atol=ATOL, rtol=RTOL)
        torch.testing.assert_close(y, torch.from_numpy(z[f"c{i}_y"]), atol=5e-2, rtol=5e-2)
        # adapters disabled == base layer; wrong adapter_names length is rejected like peft does
        layer.disable_adapters = True
        yb = layer(x.to(cuda)).float().cpu()
        torch.testing.assert_close(yb, torch.from_numpy(z[f"c{i}_y_base"]), atol=5e-2, rtol=5e-2)
        layer.disable_adapters = False
        with pytest.raises(ValueError):
            layer(x.to(cuda), adapter_names=names + ["adapter0"])
        # single active adapter applies to every row (the reference's last branch)
        layer.active_adapters = ["adapter0"]
        y1 = layer(x.to(cuda)).float().cpu()
        w1 = oops.gather_bmm_linear(x.float(), W.float(), list(A.float()), list(B.float()), [scale] * n,
                                    [0] * x.shape[0])
        torch.testing.assert_close(y1, w1, atol=ATOL, rtol=RTOL)


def test_seq_info_device_bucketing_matches_reference_golden(cuda):
    si = load("seq_info")
    with open(os.path.join(G, "bucketing_golden.json")) as f:
        cases = json.load(f)["order_cases"]
    for c in cases:
        info = si.LlamaSeqInfo(32, cuda)
        for sid in range(len(c["tids"])):
            info.add_sequence(sid)
        # register types in index order so that tid == index, then attach adapters
        types = sorted({t for t in c["tids"] if t >= 0})
        dummy = 10 ** 6
        info.add_sequence(dummy)
        for t in types:
            info.set_adapter(dummy, ("cfg", t), 0)
            info.sid_2_info[dummy]["adapter"] = None
        del info.sid_2_info[dummy]
        for sid, (t, w) in enumerate(zip(c["tids"], c["wids"])):
            if t >= 0:
                info.set_adapter(sid, ("cfg", t), w)
        assert info.get_num_adapters_per_type() == c["num_adapters_per_type"]
        ordered, pos = info.order_seqs(c["batch"])
        assert ordered == c["ordered"] and pos == c["positions"]
        for st in c["steps"]:
            name, params = info.get_decode_method(st["live"])
            assert name == st["name"] and params == st["params"]


def test_vm_function_table_runs_the_reference_executor_protocol(synth, cuda):
    """Drives B200VM the way llama_exec_graph.py does: embed, kv_state_*, prefill_a{t}, mixed_decode_..."""
    vm_mod, model_mod, si = load("vm"), load("model"), load("seq_info")
    cfg = synth.llama_config("tiny")
    w = {k: v.bfloat16() for k, v in synth.base_weights(cfg).items()}
    # two adapter types: type 0 = rank 8 (2 adapters), type 1 = rank 16 (1 adapter); slots 0,1 | 2
    ads8 = synth.lora_adapters(cfg, 2, 8, targets=("q_proj", "v_proj"))
    ads16 = synth.lora_adapters(cfg, 3, 16, targets=("q_proj", "v_proj"))[2:]
    ads = [{k: v.bfloat16() for k, v in a.items()} for a in ads8 + ads16]
    scales = [0.5, 0.5, 0.5]
    pm = model_mod.PackedLlama(cfg, w, ads, scales, device=cuda)
    vm = vm_mod.B200VM(pm, type_slot_base=[0, 2])
    gf = vm_mod.get_global_func
    S = 24
    P = synth.prompts(4, S, cfg["vocab_size"])
    # sequences: 0 -> no adapter, 1 -> (type 0, wid 1), 2 -> (type 1, wid 0), 3 -> (type 0, wid 0)
    adapters = {0: None, 1: (0, 1), 2: (1, 0), 3: (0, 0)}
    slot = {0: -1, 1: 1, 2: 2, 3: 0}
    info = si.LlamaSeqInfo(8, cuda)
    for sid, ad in adapters.items():
        info.add_sequence(sid)
    info.set_adapter(3, ("r", 8), 0)      # registers type 0 first
    info.set_adapter(1, ("r", 8), 1)
    info.set_adapter(2, ("r", 16), 0)
    oracle = ollama.OracleLlama(cfg, w, ads, scales)

    kv = vm["create_paged_kv_cache"](vm_mod.ShapeTuple([4]), vm_mod.ShapeTuple([4 * (S + 8)]),
                                     vm_mod.ShapeTuple([S]), vm_mod.ShapeTuple([16]))
    outputs = {}
    for sid in range(4):  # execute_prefill, llama_exec_graph.py:58-92
        tokens = np.asarray(P[sid:sid + 1], dtype="int32")
        gf("vm.builtin.kv_state_add_sequence")(kv, sid)
        hidden = vm["embed"](vm_mod.array(tokens, cuda), vm.params)
        gf("vm.builtin.kv_state_begin_forward")(kv, vm_mod.ShapeTuple([sid]), vm_mod.ShapeTuple([S]))
        ad = info.get_adapter_info(sid)
        if ad is None:
            logits, kv = vm["prefill_no_adapter"](hidden, kv, vm.params)
        else:
            wid = vm_mod.array(np.asarray([ad["wid"]], dtype="int32"), cuda)
            logits, kv = vm[f"prefill_a{ad['tid']}"](hidden, kv, wid, vm.params)
        gf("vm.builtin.kv_state_end_forward")(kv)
        want = oracle.prefill(sid, list(P[sid]), slot[sid])
        assert logits.numpy().shape == (1, 1, cfg["vocab_size"])
        torch.testing.assert_close(torch.from_numpy(logits.numpy())[0], want, atol=ATOL, rtol=RTOL)
        outputs[sid] = [int(np.argmax(logits.numpy()))]

    # execute_decode, llama_exec_graph.py:102-141: order, pick the method, run it
    seqs, positions = info.order_seqs([0, 1, 2, 3])
    assert seqs == [0, 3, 1, 2]
    for step in range(3):
        tok = np.array([[outputs[s][-1]] for s in seqs]).astype("int32")
        hidden = vm["embed"](vm_mod.array(tok, cuda), vm.params)
        name, plist = info.get_decode_method(seqs)
        assert name == "mixed_decode_a0_a1"
        plist = [vm_mod.array(np.asarray(ids, dtype="int32"), cuda) for ids in plist]
        gf("vm.builtin.kv_state_begin_forward")(kv, vm_mod.ShapeTuple(seqs), vm_mod.ShapeTuple([1] * len(seqs)))
        logits, kv = vm[name](hidden, kv, *plist, vm.params)
        gf("vm.builtin.kv_state_end_forward")(kv)
        lg = torch.from_numpy(logits.numpy())[:, 0]
        want = oracle.decode(seqs, [outputs[s][-1] for s in seqs], [slot[s] for s in seqs])
        torch.testing.assert_close(lg, want, atol=ATOL, rtol=RTOL)
        for i, s in enumerate(seqs):
            outputs[s].append(int(want[i].argmax()))  # teacher-forced on the oracle's token

    # a batch of one type only uses decode_a{t}(hidden, kv, wids)
    name, plist = info.get_decode_method([3, 1])
    assert name == "decode_a0" and plist == [[0, 1]]


def test_hf_model_with_injected_adapter_files_generates_like_the_cpu_hf_path(synth, cuda, tmp_path):
    """``get_hf_model`` + ``generate(adapter_names=...)`` of huggingface/generation/gen_lora.py:21-57,114-116 on a
    transformers ``LlamaForCausalLM`` (bf16, on the GPU) whose q/k/v/o projections are ``MultiLoraLinear`` layers
    loaded from adapter files in the reference's format, against the CPU HF path (fp32 model + the restated
    GatherBMMLinear) on the same files."""
    from oracle import hf_path

    ll, adapter_io = load("lora_linear"), load("adapters")
    cfg = synth.llama_config("tiny")
    w = {k: v.bfloat16() for k, v in synth.base_weights(cfg).items()}
    r, alpha, n_ad = 8, 16, 4
    adapter_io.write_adapter_files(str(tmp_path), cfg, [r], n_ad, targets=synth.ATTN_PROJ, scaling_factor=0.05)
    ads = [{k: v.bfloat16() for k, v in adapter_io.load_adapter(adapter_io.adapter_path(str(tmp_path), r, a)).items()}
           for a in range(n_ad)]
    ids = [2, 0, 3, 0]
    names = [f"adapter{i}" for i in ids]
    prompts = torch.from_numpy(synth.prompts(4, 48, cfg["vocab_size"])).long()
    gen = 8

    cpu = hf_path.build_hf_model(cfg, w, ads, [alpha / r] * n_ad)
    want_tok = hf_path.generate(cpu, prompts, ids, gen)
    want_logits = hf_path.forward_logits(cpu, torch.cat([prompts, want_tok[:, :-1]], 1), ids)

    base = hf_path.build_hf_model(cfg, w, dtype=torch.bfloat16).to(cuda)
    model = ll.get_hf_model(base, str(tmp_path), {f"adapter{i}" for i in range(n_ad)}, r=r, lora_alpha=alpha,
                            target_modules=synth.ATTN_PROJ)
    assert len(model.layers) == 4 * cfg["num_hidden_layers"]
    launches0 = load("ops").launch_count()
    out = model.generate(input_ids=prompts.to(cuda), attention_mask=torch.ones_like(prompts).to(cuda),
                         adapter_names=names, max_new_tokens=gen, min_new_tokens=gen, do_sample=False, pad_token_id=0)
    got_tok = out[:, prompts.shape[1]:].cpu()
    assert load("ops").launch_count() > launches0          # the projections ran in the library
    assert len(model.ctx.slot_cache) == 2                   # one slot tensor for the prompt pass, one for all decode steps
    # teacher-forced logits (transformers' own bf16 ops sit between the projections: a wider bar than the engine's)
    got_logits = model(input_ids=torch.cat([prompts, want_tok[:, :-1]], 1).to(cuda), adapter_names=names).logits.float().cpu()
    S = prompts.shape[1]
    torch.testing.assert_close(got_logits[:, S - 1:], want_logits[:, S - 1:], atol=6e-2, rtol=5e-2)
    agree = (got_logits[:, S - 1:].argmax(-1) == want_tok).float().mean()
    assert agree >= 0.95, agree
    # free-running tokens: wherever a row first departs, the CPU model's margin between the two tokens is a near-tie
    for b in range(4):
        d = (got_tok[b] != want_tok[b]).nonzero()
        if len(d):
            st = int(d[0])
            lg = want_logits[b, S - 1 + st]
            assert float(lg[want_tok[b, st]] - lg[got_tok[b, st]]) <= 0.12
    # adapters matter, and switching them off reproduces the base model
    with model.disable_adapter():
        base_logits = model(input_ids=prompts.to(cuda)).logits.float().cpu()
    want_base = hf_path.forward_logits(cpu, prompts, None)
    torch.testing.assert_close(base_logits[:, -1], want_base[:, -1], atol=6e-2, rtol=5e-2)
    assert float((base_logits[:, -1] - got_logits[:, S - 1]).abs().max()) > 0.05

    # hot add / remove of one adapter: the other rows' results do not move, the new adapter takes effect
    ref_rows = model(input_ids=prompts.to(cuda), adapter_names=names).logits[:, -1].float().cpu()
    extra = {k: 3.0 * v for k, v in adapter_io.load_adapter(adapter_io.adapter_path(str(tmp_path), r, 1)).items()}
    model.add_adapter("adapter9", extra, r, alpha)
    with_new = model(input_ids=prompts.to(cuda), adapter_names=["adapter9"] + names[1:]).logits[:, -1].float().cpu()
    assert torch.equal(with_new[1:], ref_rows[1:]) and not torch.equal(with_new[0], ref_rows[0])
    model.remove_adapter("adapter9")
    again = model(input_ids=prompts.to(cuda), adapter_names=names).logits[:, -1].float().cpu()
    assert torch.equal(again, ref_rows)
