"""Generates bucketing_golden.json by running the reference's own modules.

Run where the reference checkout is available:
    python tests/golden/make_bucketing_golden.py <path-to-reference-checkout>
It imports ``tvm/llama_auto_batcher/llama_seq_info.py`` and ``exec_graph.py``
unmodified (both are pure Python) and records their outputs for seeded
batches.  The JSON travels with the repository; the reference does not.
"""
import json
import os
import sys

import numpy as np

if len(sys.argv) != 2:
    sys.exit(f"usage: python {sys.argv[0]} <path-to-reference-checkout>")
ref = sys.argv[1]
sys.path.insert(0, os.path.join(ref, "tvm", "llama_auto_batcher"))
from llama_seq_info import LlamaSeqInfo  # noqa: E402
from exec_graph import ExecGraph  # noqa: E402


def make_case(rng, n, n_types, n_wids, p_none, drop):
    """n sequences; each gets no adapter with prob p_none, else (tid, wid)."""
    info = LlamaSeqInfo(32)
    configs = [("cfg", 8 << t) for t in range(n_types)]  # stands in for LoraConfig(r, alpha)
    tids, wids = [], []
    # register types in order so that tid == index
    reg = LlamaSeqInfo(32)
    for sid in range(n):
        info.add_sequence(sid)
    assigned = []
    for sid in range(n):
        if n_types == 0 or rng.random() < p_none:
            assigned.append(None)
        else:
            assigned.append((int(rng.integers(0, n_types)), int(rng.integers(0, n_wids))))
    # make tid == first-appearance index, as set_adapter does (llama_seq_info.py:17-23)
    for sid, a in enumerate(assigned):
        if a is not None:
            info.set_adapter(sid, configs[a[0]], a[1])
    for sid in range(n):
        ad = info.get_adapter_info(sid)
        tids.append(-1 if ad is None else ad["tid"])
        wids.append(-1 if ad is None else ad["wid"])
    batch = [int(s) for s in rng.permutation(n)]
    ordered, positions = info.order_seqs(batch)
    steps = []
    live = list(ordered)
    while True:
        name, params = info.get_decode_method(live)
        steps.append({"live": list(live), "name": name, "params": [[int(v) for v in p] for p in params]})
        if len(live) <= 1 or not drop:
            break
        keep = rng.random(len(live)) > 0.35
        live = [s for s, k in zip(live, keep) if k]
        if not live:
            break
    return {
        "n_types": len(info.get_adapter_configs()), "tids": tids, "wids": wids, "batch": batch,
        "ordered": [int(s) for s in ordered], "positions": [int(p) for p in positions], "steps": steps,
        "num_adapters_per_type": info.get_num_adapters_per_type(),
    }


def fuse_case(n_seq):
    """Graph of llama_auto_batcher.py:58-84 for n_seq sequences, fused."""
    g = ExecGraph(["decode"])
    for sid in range(n_seq):
        v = g.variable(None, True)
        for op in ("encode_prompt", "prefill", "decode", "decode_answer"):
            out = g.variable(None, False)
            g.operation(v, op, seqid=sid, output_var=out)
            v = out
        g.operation(v, "print", seqid=sid)
    g.fuse_batchable_ops()
    levels = []

    def rec(node_set):
        ops = [n for n in node_set if hasattr(n, "op_type")]
        if ops:
            levels.append(sorted((o.op_type, sorted(o.seqids)) for o in ops))
        return node_set
    g.ms_bfs(rec)
    return {"n_seq": n_seq, "levels": levels, "max_batch": g.get_max_batch_sizes()}


def main():
    rng = np.random.default_rng(1234)
    cases = []
    for n, nt, nw, pn, drop in [
        (1, 0, 1, 1.0, False), (1, 1, 1, 0.0, False), (4, 1, 4, 0.0, True), (8, 0, 1, 1.0, True),
        (8, 2, 3, 0.25, True), (32, 1, 16, 0.0, True), (32, 1, 16, 0.2, True), (33, 3, 5, 0.1, True),
        (128, 4, 32, 0.0, True), (128, 4, 32, 0.05, True), (257, 5, 7, 0.3, True), (64, 2, 1, 0.5, True),
        (1000, 4, 64, 0.1, False),
    ]:
        cases.append(make_case(rng, n, nt, nw, pn, drop))
    out = {"order_cases": cases, "fuse_cases": [fuse_case(n) for n in (1, 2, 7, 32)]}
    dst = os.path.join(os.path.dirname(os.path.abspath(__file__)), "bucketing_golden.json")
    with open(dst, "w") as f:
        json.dump(out, f)
    print("wrote", dst, os.path.getsize(dst), "bytes")


if __name__ == "__main__":
    main()
