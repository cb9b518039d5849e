"""The CPU oracle against outputs of the reference's own code (golden files)."""
import json
import os

import numpy as np
import torch

from oracle import bucketing, ops as oops

G = os.path.join(os.path.dirname(__file__), "golden")


def _cases():
    with open(os.path.join(G, "bucketing_golden.json")) as f:
        return json.load(f)


def test_order_seqs_matches_reference():
    for c in _cases()["order_cases"]:
        tids = [c["tids"][s] for s in c["batch"]]
        wids = [c["wids"][s] for s in c["batch"]]
        ordered, pos = bucketing.order_seqs(c["batch"], tids, wids, c["n_types"])
        assert ordered == c["ordered"]
        assert pos == c["positions"]


def test_get_decode_method_matches_reference():
    for c in _cases()["order_cases"]:
        for st in c["steps"]:
            tids = [c["tids"][s] for s in st["live"]]
            wids = [c["wids"][s] for s in st["live"]]
            name, params = bucketing.get_decode_method(tids, wids, c["n_types"])
            assert name == st["name"]
            assert params == st["params"]


def test_fused_decode_levels_match_reference():
    for c in _cases()["fuse_cases"]:
        chains = [["encode_prompt", "prefill", "decode", "decode_answer", "print"]] * c["n_seq"]
        fused = bucketing.bfs_fuse_decode_seqids(chains)
        ref_decode = [op for lvl in c["levels"] for op in lvl if op[0] == "decode"]
        assert len(ref_decode) == 1 and len(fused) == 1
        assert list(fused.values())[0] == ref_decode[0][1]
        assert c["max_batch"]["decode"] == c["n_seq"]


def test_segment_sort_is_stable_and_complete():
    rng = np.random.default_rng(0)
    for n in (0, 1, 5, 64, 1000):
        slots = rng.integers(-1, 7, n)
        perm, off, seg = bucketing.segment_sort(slots)
        assert sorted(perm.tolist()) == list(range(n))
        for s in range(len(seg)):
            rows = perm[off[s]:off[s + 1]]
            assert (slots[rows] == seg[s]).all()
            assert (np.diff(rows) > 0).all()  # stable
        assert (np.diff(seg) > 0).all()


def test_gather_bmm_linear_matches_reference_layer():
    z = np.load(os.path.join(G, "lora_layer_golden.npz"))
    for i in range(int(z["n_cases"])):
        x, W = torch.from_numpy(z[f"c{i}_x"]), torch.from_numpy(z[f"c{i}_W"])
        A, B = torch.from_numpy(z[f"c{i}_A"]), torch.from_numpy(z[f"c{i}_B"])
        ids, scale = z[f"c{i}_ids"], float(z[f"c{i}_scale"])
        n = A.shape[0]
        y = oops.gather_bmm_linear(x, W, list(A), list(B), [scale] * n, ids)
        assert torch.equal(y, torch.from_numpy(z[f"c{i}_y"]))  # same ops, same order: bit-exact
        # the flat-token form and the TVM-side form agree with it to fp32 rounding
        Bsz, S, _ = x.shape
        flat = oops.multi_lora_linear(x.reshape(Bsz * S, -1), W, A, B, [A.shape[1]] * n, [scale] * n,
                                      np.repeat(ids, S)).reshape(Bsz, S, -1)
        torch.testing.assert_close(flat, y, atol=2e-5, rtol=1e-5)
        tvm_form = torch.nn.functional.linear(x, W) + oops.take_matmul_lora(
            x, A.transpose(1, 2).contiguous(), B.transpose(1, 2).contiguous(), ids, scale)
        torch.testing.assert_close(tvm_form, y, atol=2e-5, rtol=1e-5)
        torch.testing.assert_close(torch.nn.functional.linear(x, W), torch.from_numpy(z[f"c{i}_y_base"]))


def test_mixed_type_delta_equals_flat_form():
    g = torch.Generator().manual_seed(5)
    Bsz, fin, fout = 7, 32, 24
    h = torch.randn(Bsz, 1, fin, generator=g)
    types = []
    flat_delta = torch.zeros(Bsz, 1, fout)
    rows = {0: ([1, 4, 6], [0, 1, 0], 4, 2.0), 1: ([0, 3], [2, 0], 8, 0.5)}  # row 2 and 5 have no adapter
    for t, (sids, wids, r, sc) in rows.items():
        p0 = torch.randn(3, fin, r, generator=g) * 0.1
        p1 = torch.randn(3, r, fout, generator=g) * 0.1
        types.append((sids, wids, p0, p1, sc))
        for s, w in zip(sids, wids):
            flat_delta[s] = (h[s] @ p0[w]) @ p1[w] * sc
    d = oops.mixed_type_lora_delta(h, fout, types)
    torch.testing.assert_close(d, flat_delta)
