"""Parity of each CUDA operator (called through the C ABI) against the CPU oracle."""
import json
import math
import os

import numpy as np
import pytest
import torch

from conftest import load
from oracle import bucketing, ops as oops

pytestmark = pytest.mark.gpu
G = os.path.join(os.path.dirname(__file__), "golden")

# bf16 outputs vs an fp32 oracle fed the same bf16-rounded inputs
ATOL, RTOL = 2e-2, 1e-2


def _i32(a, dev):
    return torch.as_tensor(np.asarray(a, dtype=np.int32), device=dev)


# ----------------------------------------------------------------------------- bucketing
def _run_bucket(ops, dev, tids, wids, n_types, n_wids, by_type):
    b = ops.bucket_sort(_i32(tids, dev) if tids is not None else None, _i32(wids, dev), n_types, n_wids, by_type)
    torch.cuda.synchronize()
    return b


def test_bucket_sort_matches_reference_golden(ops, cuda):
    with open(os.path.join(G, "bucketing_golden.json")) as f:
        cases = json.load(f)["order_cases"]
    for c in cases:
        nt = c["n_types"]
        tids = [c["tids"][s] for s in c["batch"]]
        wids = [c["wids"][s] for s in c["batch"]]
        n_wids = max(max(wids) + 1, 1)
        b = _run_bucket(ops, cuda, tids, wids, nt, n_wids, False)
        perm = b.perm.cpu().tolist()
        if nt > 0:  # with no adapter type the reference returns the batch unchanged; a stable sort agrees
            assert perm == c["positions"]
        assert [c["batch"][p] for p in perm] == c["ordered"]
        # per-step method selection on the (already ordered, shrinking) live batch
        for st in c["steps"]:
            lt = [c["tids"][s] for s in st["live"]]
            lw = [c["wids"][s] for s in st["live"]]
            bt = _run_bucket(ops, cuda, lt, lw, nt, n_wids, True)
            counts = bt.counts.cpu().tolist()
            p = bt.perm.cpu().tolist()
            sw = bt.sorted_wid.cpu().tolist()
            non_empty = [t for t in range(nt) if counts[2 + t] > 0]
            no_adapter = counts[1] > 0
            if no_adapter and not non_empty:
                name, params = "decode_no_adapter", []
            elif not no_adapter and len(non_empty) == 1:
                name, params = f"decode_a{non_empty[0]}", [sw]
            else:
                name = "mixed_decode_" + "_".join(f"a{t}" for t in non_empty)
                params, off = [], counts[1]
                for t in range(nt):
                    if counts[2 + t]:
                        params += [p[off:off + counts[2 + t]], sw[off:off + counts[2 + t]]]
                    off += counts[2 + t]
            assert name == st["name"]
            assert params == st["params"]


@pytest.mark.parametrize("n", [0, 1, 31, 32, 1024, 1025, 5000, 40000])
def test_bucket_sort_segments(ops, cuda, n):
    rng = np.random.default_rng(n)
    n_ad = 16 if n < 5000 else 64
    slots = rng.integers(-1, n_ad, n).astype(np.int32)
    if n == 32:
        slots[:] = 3  # one giant segment
    b = _run_bucket(ops, cuda, None, slots, 1, n_ad, False)
    perm, off, seg = bucketing.segment_sort(slots)
    n_seg = int(b.counts[0])
    assert n_seg == len(seg)
    assert b.perm.cpu().numpy().tolist() == perm.tolist()
    assert b.seg_offsets[: n_seg + 1].cpu().numpy().tolist() == off.tolist()
    assert b.seg_wid[:n_seg].cpu().numpy().tolist() == seg.tolist()
    assert b.sorted_wid.cpu().numpy().tolist() == slots[perm].tolist()
    assert int(b.counts[1]) == int((slots < 0).sum())


# ----------------------------------------------------------------------------- LoRA + projection
def _stack(ops, A, B, ranks, scales, dev, n_mod=1, mod_offsets=None):
    """Packs A [N, n_mod*r, K] / B [N, out, r] into stacks whose rank pitch is 16, 32 or 64 (zero padded)."""
    r = B.shape[2]
    rp = 16 if r <= 16 else 32 if r <= 32 else 64
    Ap = torch.zeros(A.shape[0], n_mod * rp, A.shape[2], dtype=A.dtype)
    for m in range(n_mod):
        Ap[:, m * rp:m * rp + r] = A[:, m * r:(m + 1) * r]
    Bp = torch.zeros(B.shape[0], B.shape[1], rp, dtype=B.dtype)
    Bp[..., :r] = B
    return ops.LoraStack(Ap.to(dev), Bp.to(dev), _i32(ranks, dev), torch.tensor(scales, dtype=torch.float32, device=dev),
                         rp, n_mod, mod_offsets)


@pytest.mark.parametrize("T", [1, 8, 32, 128])
def test_operator_case_against_oracle(ops, synth, cuda, T):
    """The operator micro-benchmark shapes: y = x W^T + 2 (x A[id]) B[id]."""
    c = synth.operator_case(T)
    st = _stack(ops, c["A"], c["B"], [16] * 16, [c["scale"]] * 16, cuda)
    ids = c["ids"].to(cuda)
    x, W = c["x"].to(cuda), c["W"].to(cuda)
    want = oops.multi_lora_linear(c["x"].float(), c["W"].float(), c["A"].float(), c["B"].float(), [16] * 16,
                                  [c["scale"]] * 16, c["ids"])
    for flags in (ops.FORCE_SIMT, 0):
        y = ops.linear(x, W, st, ids, flags=flags)
        torch.testing.assert_close(y.float().cpu(), want, atol=ATOL, rtol=RTOL)
    base = ops.linear(x, W)
    torch.testing.assert_close(base.float().cpu(), c["x"].float() @ c["W"].float().t(), atol=ATOL, rtol=RTOL)


def test_lora_layer_golden_through_cuda(ops, cuda):
    """Reference GatherBMMLinear outputs (fp32) vs the CUDA path on bf16-rounded copies."""
    z = np.load(os.path.join(G, "lora_layer_golden.npz"))
    for i in range(int(z["n_cases"])):
        x = torch.from_numpy(z[f"c{i}_x"]).bfloat16()
        W = torch.from_numpy(z[f"c{i}_W"]).bfloat16()
        A = torch.from_numpy(z[f"c{i}_A"]).bfloat16()
        B = torch.from_numpy(z[f"c{i}_B"]).bfloat16()
        ids, scale = z[f"c{i}_ids"], float(z[f"c{i}_scale"])
        Bsz, S, fin = x.shape
        n, r = A.shape[0], A.shape[1]
        st = _stack(ops, A, B, [r] * n, [scale] * n, cuda)
        slots = _i32(np.repeat(ids, S), cuda)
        y = ops.linear(x.reshape(Bsz * S, fin).to(cuda), W.to(cuda), st, slots).float().cpu().reshape(Bsz, S, -1)
        # bf16 rounding of inputs and output: compare with the fp32 reference output loosely ...
        torch.testing.assert_close(y, torch.from_numpy(z[f"c{i}_y"]), atol=5e-2, rtol=5e-2)
        # ... and tightly with the oracle on the same rounded inputs
        want = oops.gather_bmm_linear(x.float(), W.float(), list(A.float()), list(B.float()), [scale] * n, ids)
        torch.testing.assert_close(y, want, atol=ATOL, rtol=RTOL)


def test_mixed_ranks_no_adapter_rows_and_modules(ops, cuda):
    g = torch.Generator().manual_seed(11)
    T, K, outs = 13, 320, (64, 32, 32)
    N_out = sum(outs)
    ranks = [8, 16, 32, 64, 16]
    r_max, n_mod, n_ad = 64, 3, len(ranks)
    x = torch.randn(T, K, generator=g).bfloat16()
    W = (torch.randn(N_out, K, generator=g) * 0.05).bfloat16()
    A = (torch.randn(n_ad, n_mod * r_max, K, generator=g) * 0.05).bfloat16()
    B = (torch.randn(n_ad, N_out, r_max, generator=g) * 0.05).bfloat16()
    scales = [2.0, 1.0, 0.5, 0.25, 4.0]
    slots = np.array([0, 1, -1, 2, 3, 4, 4, -1, 0, 3, 1, 2, 0], dtype=np.int32)
    offs = (0, 64, 96, 128)
    st = _stack(ops, A, B, ranks, scales, cuda, n_mod, offs)
    y = ops.linear(x.to(cuda), W.to(cuda), st, _i32(slots, cuda)).float().cpu()
    want = x.float() @ W.float().t()
    for t in range(T):
        s = int(slots[t])
        if s < 0:
            continue
        r = ranks[s]
        for m in range(n_mod):
            u = A[s, m * r_max:m * r_max + r].float() @ x[t].float()
            want[t, offs[m]:offs[m + 1]] += scales[s] * (B[s, offs[m]:offs[m + 1], :r].float() @ u)
    torch.testing.assert_close(y, want, atol=ATOL, rtol=RTOL)


@pytest.mark.parametrize("T,r", [(5, 16), (32, 16), (40, 32), (130, 64)])
def test_fused_qkv_modules_on_tensor_cores(ops, cuda, T, r):
    """Three modules of 256/128/128 rows (tile-aligned): the expand runs as extra MMA stages."""
    g = torch.Generator().manual_seed(T + r)
    K, outs, n_ad = 512, (256, 128, 128), 6
    offs = (0, 256, 384, 512)
    x = torch.randn(T, K, generator=g).bfloat16()
    W = (torch.randn(512, K, generator=g) * 0.05).bfloat16()
    A = (torch.randn(n_ad, 3 * r, K, generator=g) * 0.05).bfloat16()
    B = (torch.randn(n_ad, 512, r, generator=g) * 0.05).bfloat16()
    ranks = [r, r // 2, r, 8, r, r][:n_ad]
    for s in range(n_ad):  # zero the padding beyond each adapter's rank
        for m in range(3):
            A[s, m * r + ranks[s]:(m + 1) * r] = 0
        B[s, :, ranks[s]:] = 0
    scales = [2.0, 1.0, 0.5, 1.5, 3.0, 0.25]
    slots = torch.randint(-1, n_ad, (T,), generator=g).int()
    st = _stack(ops, A, B, ranks, scales, cuda, 3, offs)
    want = x.float() @ W.float().t()
    for t in range(T):
        s = int(slots[t])
        if s < 0:
            continue
        for m in range(3):
            u = A[s, m * r:(m + 1) * r].float() @ x[t].float()
            want[t, offs[m]:offs[m + 1]] += scales[s] * (B[s, offs[m]:offs[m + 1]].float() @ u)
    y = ops.linear(x.to(cuda), W.to(cuda), st, slots.to(cuda)).float().cpu()
    y2 = ops.linear(x.to(cuda), W.to(cuda), st, slots.to(cuda), flags=ops.FORCE_SIMT).float().cpu()
    torch.cuda.synchronize()
    assert int(ops.workspace(4, cuda, "linear")[:4].view(torch.int32)) == 0, "a bounded wait expired"
    torch.testing.assert_close(y, want, atol=ATOL, rtol=RTOL)
    torch.testing.assert_close(y2, want, atol=ATOL, rtol=RTOL)


@pytest.mark.parametrize("T,r", [(4, 16), (32, 16), (70, 64)])
def test_gate_up_silu_with_lora(ops, cuda, T, r):
    """Interleaved gate/up with LoRA on both: B rows carry [gate half | up half] with the other half zero."""
    model = load("model")
    g = torch.Generator().manual_seed(T)
    K, I, n_ad = 256, 384, 3
    x = torch.randn(T, K, generator=g).bfloat16()
    Wg = (torch.randn(I, K, generator=g) * 0.05).bfloat16()
    Wu = (torch.randn(I, K, generator=g) * 0.05).bfloat16()
    Ag = (torch.randn(n_ad, r, K, generator=g) * 0.05).bfloat16()
    Au = (torch.randn(n_ad, r, K, generator=g) * 0.05).bfloat16()
    Bg = (torch.randn(n_ad, I, r, generator=g) * 0.05).bfloat16()
    Bu = (torch.randn(n_ad, I, r, generator=g) * 0.05).bfloat16()
    slots = torch.randint(-1, n_ad, (T,), generator=g).int()
    z = torch.zeros_like(Bg)
    B_all = torch.stack([model.interleave_gate_up(torch.cat([Bg, z], 2)[s], torch.cat([z, Bu], 2)[s])
                         for s in range(n_ad)])
    st = ops.LoraStack(torch.cat([Ag, Au], 1).to(cuda), B_all.to(cuda), _i32([r] * n_ad, cuda),
                       torch.full((n_ad,), 2.0, device=cuda), r, 2, None)
    Wi = model.interleave_gate_up(Wg, Wu)
    gate, up = x.float() @ Wg.float().t(), x.float() @ Wu.float().t()
    for t in range(T):
        s = int(slots[t])
        if s >= 0:
            gate[t] += 2.0 * (Bg[s].float() @ (Ag[s].float() @ x[t].float()))
            up[t] += 2.0 * (Bu[s].float() @ (Au[s].float() @ x[t].float()))
    want = oops.silu_mul(gate, up)
    # ... and the same with the expand laid out by (row, output feature) in front of the activation: what a batch with
    # many distinct adapters takes (fp32 pre-activations in the scratch buffer's tail, activation in the expand kernel)
    for flags in (ops.SILU_MUL, ops.SILU_MUL | ops.FORCE_SIMT, ops.SILU_MUL | ops.LORA_PER_ROW,
                  ops.SILU_MUL | ops.LORA_PER_ROW | ops.FORCE_SIMT):
        y = ops.linear(x.to(cuda), Wi.to(cuda), st, slots.to(cuda), flags=flags).float().cpu()
        torch.testing.assert_close(y, want, atol=ATOL, rtol=RTOL)
    launches = ops.launch_count()
    stp = ops.LoraStack(torch.cat([Ag, Au], 1).to(cuda), B_all.to(cuda).clone(), _i32([r] * n_ad, cuda),
                        torch.full((n_ad,), 2.0, device=cuda), r, 2, None).pack_b()
    y = ops.linear(x.to(cuda), ops.PackedWeight(Wi.to(cuda)), stp, slots.to(cuda),
                   flags=ops.SILU_MUL | ops.LORA_PER_ROW).float().cpu()
    torch.testing.assert_close(y, want, atol=ATOL, rtol=RTOL)
    assert ops.launch_count() - launches >= 3  # shrink, projection, expand: the per-row form really ran
    torch.cuda.synchronize()
    assert int(ops.workspace(4, cuda, "linear")[:4].view(torch.int32)) == 0


@pytest.mark.parametrize("T,K,I", [(3, 256, 688), (32, 512, 1024)])
def test_gate_up_silu_interleaved(ops, cuda, T, K, I):
    g = torch.Generator().manual_seed(3)
    x = torch.randn(T, K, generator=g).bfloat16()
    Wg = (torch.randn(I, K, generator=g) * 0.05).bfloat16()
    Wu = (torch.randn(I, K, generator=g) * 0.05).bfloat16()
    Wi = torch.stack([Wg.view(I // 8, 8, K), Wu.view(I // 8, 8, K)], 1).reshape(2 * I, K).contiguous()
    want = oops.silu_mul(x.float() @ Wg.float().t(), x.float() @ Wu.float().t())
    for flags in (ops.SILU_MUL | ops.FORCE_SIMT, ops.SILU_MUL):
        y = ops.linear(x.to(cuda), Wi.to(cuda), flags=flags).float().cpu()
        torch.testing.assert_close(y, want, atol=ATOL, rtol=RTOL)


def test_f32_logits_and_argmax(ops, cuda):
    g = torch.Generator().manual_seed(4)
    T, K, V = 5, 256, 32000
    x = torch.randn(T, K, generator=g).bfloat16()
    W = (torch.randn(V, K, generator=g) * 0.05).bfloat16()
    lg = ops.linear(x.to(cuda), W.to(cuda), flags=ops.OUT_F32)
    assert lg.dtype == torch.float32
    want = x.float() @ W.float().t()
    torch.testing.assert_close(lg.cpu(), want, atol=1e-3, rtol=1e-3)
    tok = ops.argmax(lg).cpu()
    assert tok.tolist() == lg.cpu().argmax(-1).tolist()
    # ties resolve to the first index, like numpy
    tie = torch.zeros(3, 1000, device=cuda)
    tie[0, [7, 500]] = 1.0
    tie[1, 999] = 2.0
    assert ops.argmax(tie).cpu().tolist() == [7, 999, 0]


# ----------------------------------------------------------------------------- row ops
@pytest.mark.parametrize("H", [256, 4096, 5120, 11008])
def test_residual_rmsnorm(ops, cuda, H):
    g = torch.Generator().manual_seed(H)
    T = 7
    res = torch.randn(T, H, generator=g)
    delta = torch.randn(T, H, generator=g).bfloat16()
    w = (1 + 0.1 * torch.randn(H, generator=g)).bfloat16()
    r = res.clone().to(cuda)
    out = ops.residual_rmsnorm(delta.to(cuda), r, w.to(cuda), 1e-5)
    new_res = res + delta.float()
    assert torch.equal(r.cpu(), new_res)  # one fp32 add per element: bit-exact
    torch.testing.assert_close(out.float().cpu(), oops.rmsnorm(new_res, w, 1e-5), atol=ATOL, rtol=RTOL)
    out2 = ops.residual_rmsnorm(None, r, w.to(cuda), 1e-5)
    assert torch.equal(out2, out)


def test_embed(ops, cuda):
    g = torch.Generator().manual_seed(8)
    E = torch.randn(1000, 256, generator=g).bfloat16()
    ids = torch.tensor([0, 999, 5, 5, 17], dtype=torch.int32)
    res = ops.embed(ids.to(cuda), E.to(cuda))
    assert torch.equal(res.cpu(), E[ids.long()].float())


# ----------------------------------------------------------------------------- paged KV
def _paged_case(seed, B, Hq, Hkv, D, ps, lens, dev, max_pages=None):
    """Random cache with shuffled page ids; returns tensors on CPU (bf16) + tables."""
    g = torch.Generator().manual_seed(seed)
    need = [(n + 1 + ps - 1) // ps for n in lens]
    max_pages = max_pages or max(need) + 1
    n_pages = sum(need) + 3
    page_ids = torch.randperm(n_pages, generator=g)[: sum(need)].tolist()
    bt = np.full((B, max_pages), -1, dtype=np.int32)
    it = iter(page_ids)
    for b in range(B):
        for p in range(need[b]):
            bt[b, p] = next(it)
    kp = torch.randn(n_pages, Hkv, ps, D, generator=g).bfloat16()
    vp = torch.randn(n_pages, Hkv, ps, D, generator=g).bfloat16()
    qkv = torch.randn(B, (Hq + 2 * Hkv) * D, generator=g).bfloat16()
    return kp, vp, qkv, bt


@pytest.mark.parametrize("Hq,Hkv,D,ps", [(4, 4, 64, 16), (32, 32, 128, 16), (8, 2, 128, 16), (4, 2, 64, 32),
                                         (4, 4, 128, 32)])
@pytest.mark.parametrize("n_splits", [1, 3, 0])
def test_paged_attention_decode_fused_append(ops, cuda, Hq, Hkv, D, ps, n_splits):
    lens = [0, 1, 15, 16, 17, 100, 511]
    B = len(lens)
    theta = 10000.0
    kp, vp, qkv, bt = _paged_case(1, B, Hq, Hkv, D, ps, lens, cuda)
    kp_d, vp_d = kp.to(cuda), vp.to(cuda)
    slot = np.arange(B, dtype=np.int32)[::-1].copy()  # rows use slots in reverse order
    bt_by_slot = np.zeros_like(bt)
    for b in range(B):
        bt_by_slot[slot[b]] = bt[b]
    pos = np.array(lens, dtype=np.int32)
    out = ops.paged_attention(qkv.to(cuda), kp_d, vp_d, _i32(bt_by_slot, cuda), _i32(slot, cuda), _i32(pos, cuda),
                              Hq, Hkv, D, ps, theta, True, n_splits=n_splits).float().cpu()
    # oracle: rotate q and new k, append, attend
    q = qkv[:, : Hq * D].view(B, Hq, D)
    k = qkv[:, Hq * D:(Hq + Hkv) * D].view(B, Hkv, D)
    v = qkv[:, (Hq + Hkv) * D:].view(B, Hkv, D)
    qr = oops.rope_rotate_half(q, torch.from_numpy(pos), theta)
    kr = oops.rope_rotate_half(k, torch.from_numpy(pos), theta).bfloat16()
    kp2, vp2 = kp.clone(), vp.clone()
    for b in range(B):
        page = bt[b, lens[b] // ps]
        kp2[page, :, lens[b] % ps] = kr[b]
        vp2[page, :, lens[b] % ps] = v[b]
    want = oops.paged_attention_decode(qr, kp2, vp2, bt, pos + 1).reshape(B, Hq * D)
    torch.testing.assert_close(out, want, atol=ATOL, rtol=RTOL)
    # block-table gather / append: the pages now hold exactly the oracle's bytes
    torch.testing.assert_close(kp_d.cpu().float(), kp2.float(), atol=1e-2, rtol=1e-2)
    assert torch.equal(vp_d.cpu(), vp2)
    untouched = torch.ones(kp.shape[0], dtype=torch.bool)
    untouched[[bt[b, lens[b] // ps] for b in range(B)]] = False
    assert torch.equal(kp_d.cpu()[untouched], kp[untouched])


def test_append_then_attention_prefill_rows(ops, cuda):
    """Prefill form: a chunk of rows of two sequences appended, then attended causally."""
    Hq, Hkv, D, ps, theta = 4, 4, 64, 16, 10000.0
    g = torch.Generator().manual_seed(2)
    S = [37, 20]
    T = sum(S)
    qkv = torch.randn(T, (Hq + 2 * Hkv) * D, generator=g).bfloat16()
    slot = np.array([1] * S[0] + [0] * S[1], dtype=np.int32)
    pos = np.array(list(range(S[0])) + list(range(S[1])), dtype=np.int32)
    bt = np.array([[5, 2, 7, -1], [0, 6, 1, 3]], dtype=np.int32)  # by slot
    kp = torch.zeros(8, Hkv, ps, D, dtype=torch.bfloat16, device=cuda)
    vp = torch.zeros_like(kp)
    qkv_d = qkv.to(cuda)
    ops.kv_append_rope(qkv_d, kp, vp, _i32(bt, cuda), _i32(slot, cuda), _i32(pos, cuda), Hq, Hkv, D, ps, theta)
    out = ops.paged_attention(qkv_d, kp, vp, _i32(bt, cuda), _i32(slot, cuda), _i32(pos, cuda), Hq, Hkv, D, ps,
                              theta, False).float().cpu()
    q = qkv[:, : Hq * D].view(T, Hq, D)
    k = qkv[:, Hq * D:(Hq + Hkv) * D].view(T, Hkv, D)
    v = qkv[:, (Hq + Hkv) * D:].view(T, Hkv, D)
    qr = oops.rope_rotate_half(q, torch.from_numpy(pos), theta).bfloat16()
    kr = oops.rope_rotate_half(k, torch.from_numpy(pos), theta).bfloat16()
    torch.testing.assert_close(qkv_d[:, : Hq * D].float().cpu(), qr.float().view(T, -1), atol=1e-2, rtol=1e-2)
    a, want = 0, []
    for n in S:
        want.append(oops.causal_attention(qr[a:a + n], kr[a:a + n], v[a:a + n]).reshape(n, Hq * D))
        a += n
    torch.testing.assert_close(out, torch.cat(want), atol=ATOL, rtol=RTOL)
    # gather through the block table returns the appended keys in order
    got = oops.paged_gather(kp.cpu(), bt[1], S[0])
    torch.testing.assert_close(got.float(), kr[: S[0]].float(), atol=1e-2, rtol=1e-2)


@pytest.mark.parametrize("Hq,Hkv", [(4, 4), (8, 2)])
def test_prompt_attention_on_tensor_cores(ops, cuda, Hq, Hkv):
    """Tiles of <= 128 prompt rows: ragged lengths, a 300-row prompt cut into three tiles, one row, and a chunk that
    continues a sequence whose first 70 tokens are already in the pages.  Against the single-query kernel on the same
    pages and against the oracle's causal attention."""
    D, ps, theta = 128, 16, 10000.0
    g = torch.Generator().manual_seed(11)
    # (slot, tokens already cached, new rows)
    seqs = [(2, 0, 300), (0, 0, 1), (3, 70, 45), (1, 0, 128), (4, 0, 17)]
    max_pages = 24
    n_pages = 64
    perm = torch.randperm(n_pages, generator=g).tolist()
    bt = np.full((5, max_pages), -1, dtype=np.int32)
    it = iter(perm)
    for slot, old, n in seqs:
        for p in range((old + n + ps - 1) // ps):
            bt[slot, p] = next(it)
    # pages start out as NaN: what lies behind a sequence's last token must not reach any output
    kp = torch.full((n_pages, Hkv, ps, D), float("nan"), dtype=torch.bfloat16, device=cuda)
    vp = torch.full_like(kp, float("nan"))
    W = (Hq + 2 * Hkv) * D
    hist = {}
    # the earlier chunk of slot 3 goes in first, through the same append kernel
    for slot, old, n in seqs:
        if old:
            h = torch.randn(old, W, generator=g).bfloat16()
            hist[slot] = h
            ops.kv_append_rope(h.to(cuda), kp, vp, _i32(bt, cuda), _i32(np.full(old, slot, np.int32), cuda),
                               _i32(np.arange(old, dtype=np.int32), cuda), Hq, Hkv, D, ps, theta)
    T = sum(n for _, _, n in seqs)
    qkv = torch.randn(T, W, generator=g).bfloat16()
    slot_rows = np.concatenate([np.full(n, s, np.int32) for s, _, n in seqs])
    pos_rows = np.concatenate([np.arange(o, o + n, dtype=np.int32) for _, o, n in seqs])
    qkv_d = qkv.to(cuda)
    ops.kv_append_rope(qkv_d, kp, vp, _i32(bt, cuda), _i32(slot_rows, cuda), _i32(pos_rows, cuda), Hq, Hkv, D, ps, theta)
    tiles, a = [], 0
    for s, o, n in seqs:
        for off in range(0, n, 128):
            tiles.append((s, a + off, min(128, n - off), o + off))
        a += n
    status = torch.zeros(1, dtype=torch.int32, device=cuda)
    out = torch.full((T, Hq * D), float("nan"), dtype=torch.bfloat16, device=cuda)
    ops.prefill_attention(qkv_d, kp, vp, _i32(bt, cuda), _i32(np.asarray(tiles, np.int32), cuda), len(tiles), Hq, Hkv, D, ps,
                          out, status)
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    ref = ops.paged_attention(qkv_d, kp, vp, _i32(bt, cuda), _i32(slot_rows, cuda), _i32(pos_rows, cuda), Hq, Hkv, D, ps,
                              theta, False)
    torch.testing.assert_close(out.float().cpu(), ref.float().cpu(), atol=ATOL, rtol=RTOL)
    # oracle: rotate, then causal attention over history + chunk
    a, want = 0, []
    for s, o, n in seqs:
        rows = qkv[a:a + n]
        full = torch.cat([hist[s], rows]) if o else rows
        pos = torch.arange(o + n)
        q = oops.rope_rotate_half(full[:, : Hq * D].view(-1, Hq, D), pos, theta).bfloat16()
        k = oops.rope_rotate_half(full[:, Hq * D:(Hq + Hkv) * D].view(-1, Hkv, D), pos, theta).bfloat16()
        v = full[:, (Hq + Hkv) * D:].view(-1, Hkv, D)
        want.append(oops.causal_attention(q, k, v)[o:].reshape(n, Hq * D))
        a += n
    torch.testing.assert_close(out.float().cpu(), torch.cat(want).float(), atol=ATOL, rtol=RTOL)
    # sizes outside the kernel's range are refused, not mis-computed
    with pytest.raises(Exception):
        ops.prefill_attention(qkv_d, kp, vp, _i32(bt, cuda), _i32(np.asarray(tiles, np.int32), cuda), len(tiles), Hq, Hkv, 64,
                              ps, out, status)


@pytest.mark.parametrize("T,H,I,lora", [(32, 4096, 11008, True), (1, 4096, 11008, False), (7, 1024, 2816, True), (5, 320, 256, True)])
def test_residual_and_norm_folded_into_the_projections(ops, cuda, T, H, I, lora):
    """o projection -> residual add -> RMSNorm -> gate|up (SiLU) with the add and the norm folded into the two
    projections' epilogues (``mlora_linear_norm``), against the three separate calls and against fp32 arithmetic."""
    g = torch.Generator().manual_seed(T + H)
    attn = torch.randn(T, H, generator=g).bfloat16().to(cuda)
    res0 = torch.randn(T, H, generator=g).to(cuda)
    Wo = (torch.randn(H, H, generator=g) * 0.03).bfloat16().to(cuda)
    Wgu = (torch.randn(2 * I, H, generator=g) * 0.03).bfloat16().to(cuda)  # rows interleaved gate/up in blocks of 8
    w = (1.0 + 0.1 * torch.randn(H, generator=g)).bfloat16().to(cuda)
    eps = 1e-5
    st = slots = u = None
    if lora:
        n_ad, r = 3, 16
        A = (torch.randn(n_ad, r, H, generator=g) * 0.05).bfloat16().to(cuda)
        B = (torch.randn(n_ad, H, r, generator=g) * 0.05).bfloat16().to(cuda)
        st = ops.LoraStack(A, B, _i32([r] * n_ad, cuda), torch.full((n_ad,), 2.0, device=cuda), r, 1, (0, H))
        if H % 128 == 0:
            st = st.pack_b()
        slots = (torch.arange(T) % (n_ad + 1) - 1).int().to(cuda)
        u = ops.lora_shrink(attn, st, slots)
    Wo_p, Wgu_p = ops.PackedWeight(Wo), ops.PackedWeight(Wgu)
    # separate calls
    y = ops.linear(attn, Wo_p, st, slots, u=u)
    res_a = res0.clone()
    h_a = ops.residual_rmsnorm(y, res_a, w, eps)
    act_a = ops.linear(h_a, Wgu_p, flags=ops.SILU_MUL)
    # folded
    res_b = res0.clone()
    n_part = -(-H // 128)
    sumsq = torch.full((n_part * 32,), float("nan"), device=cuda)
    h_b = ops.linear_norm(attn, Wo_p, st, slots, u=u, res=res_b, norm_w=w, sumsq_out=sumsq)
    act_b = ops.linear_norm(h_b, Wgu_p, flags=ops.SILU_MUL, sumsq_in=sumsq, n_sumsq_in=n_part, eps=eps, norm_dim=H)
    torch.cuda.synchronize()
    assert int(ops.workspace(4, cuda, "linear")[:4].view(torch.int32)) == 0, "a bounded wait expired"
    # the residual: fp32 accumulator added directly (the separate path rounds y to bf16 first)
    torch.testing.assert_close(res_b, res_a, atol=4e-2, rtol=1e-2)
    want_res = res0 + (attn.float() @ Wo.float().t() + (0 if not lora else sum(
        2.0 * ((slots == s).float()[:, None] * (attn.float() @ A[s].float().t()) @ B[s].float().t()) for s in range(n_ad))))
    torch.testing.assert_close(res_b, want_res, atol=2e-2, rtol=1e-2)
    assert (res_b - want_res).abs().max() <= (res_a - want_res).abs().max() + 1e-3
    # sums of squares of the new residual rows, per block of 128 features
    ss = sumsq.view(n_part, 32)[:, :T].sum(0)
    torch.testing.assert_close(ss, (res_b * res_b).sum(1), rtol=1e-4, atol=1e-3)
    # the activation.  The two paths round the normalised rows at different points (bf16(x*w/rms) against bf16(x*w)
    # with 1/rms applied in fp32 afterwards), so they differ from each other by what each differs from exact
    # arithmetic: silu(g)*u of gate/up values of a few units, each carrying ~5e-3 of accumulated input rounding
    # (the same two roundings emulated in fp32 on the CPU differ by up to 0.1 + 2 % at these sizes).
    torch.testing.assert_close(act_b.float(), act_a.float(), atol=1e-1, rtol=2e-2)
    rstd = torch.rsqrt((want_res * want_res).mean(1, keepdim=True) + eps)
    hh = (want_res * rstd * w.float()) @ Wgu.float().t()
    # de-interleave: blocks of 8 gate rows then 8 up rows
    hh = hh.view(T, -1, 2, 8)
    want_act = (torch.nn.functional.silu(hh[:, :, 0]) * hh[:, :, 1]).reshape(T, -1)
    torch.testing.assert_close(act_b.float(), want_act, atol=1e-1, rtol=2e-2)
    err_b = (act_b.float() - want_act).pow(2).mean().sqrt().item()
    err_a = (act_a.float() - want_act).pow(2).mean().sqrt().item()
    assert err_b <= 1.1 * err_a + 1e-4, (err_b, err_a)  # the folded form is no further from exact arithmetic
    # refused where the kernel cannot do it
    with pytest.raises(Exception):
        ops.linear_norm(attn.repeat(40, 1)[:40], Wo_p, res=res0.repeat(40, 1)[:40].contiguous(), norm_w=w, sumsq_out=sumsq)


def test_kv_begin_decode(ops, cuda):
    seq = _i32([5, 0, 9, 3], cuda)
    rows = _i32([2, 0], cuda)
    pos = torch.empty(2, dtype=torch.int32, device=cuda)
    ops.kv_begin_decode(rows, seq, pos)
    assert pos.cpu().tolist() == [9, 5] and seq.cpu().tolist() == [6, 0, 10, 3]


@pytest.mark.parametrize("T,K,N", [(1, 64, 128), (16, 256, 256), (32, 4096, 4096), (33, 688, 256), (128, 4096, 512),
                                   (200, 512, 384), (7, 1024, 200), (32, 11008, 4096), (300, 256, 12288)])
def test_tensor_core_projection_shapes(ops, cuda, T, K, N):
    """Ragged K / out / T, several token tiles, split-K and no split: tcgen05 path == CUDA-core path == oracle."""
    g = torch.Generator().manual_seed(T * 7 + K)
    x = torch.randn(T, K, generator=g).bfloat16()
    W = (torch.randn(N, K, generator=g) * 0.05).bfloat16()
    n_ad, r = 5, 16
    A = (torch.randn(n_ad, r, K, generator=g) * 0.05).bfloat16()
    B = (torch.randn(n_ad, N, r, generator=g) * 0.05).bfloat16()
    slots = torch.randint(-1, n_ad, (T,), generator=g).int()
    st = _stack(ops, A, B, [r] * n_ad, [1.5] * n_ad, cuda)
    want = oops.multi_lora_linear(x.float(), W.float(), A.float(), B.float(), [r] * n_ad, [1.5] * n_ad, slots)
    xd, Wd, sd = x.to(cuda), W.to(cuda), slots.to(cuda)
    y_tc = ops.linear(xd, Wd, st, sd)
    y_tc2 = ops.linear(xd, Wd, st, sd)
    y_simt = ops.linear(xd, Wd, st, sd, flags=ops.FORCE_SIMT)
    torch.cuda.synchronize()
    assert int(ops.workspace(4, cuda, "linear")[:4].view(torch.int32)) == 0, "a bounded wait expired"
    torch.testing.assert_close(y_tc.float().cpu(), want, atol=ATOL, rtol=RTOL)
    assert torch.equal(y_tc, y_tc2)  # split-K partials are summed in a fixed order
    torch.testing.assert_close(y_tc.float(), y_simt.float(), atol=ATOL, rtol=RTOL)


@pytest.mark.parametrize("T,K,N", [(32, 4096, 4096), (33, 688, 256), (7, 1024, 200), (130, 512, 384)])
def test_packed_weight_equals_row_major(ops, cuda, T, K, N):
    """The pre-tiled weight layout is a pure re-arrangement: results are bit-identical."""
    g = torch.Generator().manual_seed(K + N)
    x = torch.randn(T, K, generator=g).bfloat16().to(cuda)
    W = (torch.randn(N, K, generator=g) * 0.05).bfloat16().to(cuda)
    y0 = ops.linear(x, W)
    y1 = ops.linear(x, ops.PackedWeight(W))
    assert torch.equal(y0, y1)
    torch.testing.assert_close(y1.float().cpu(), x.float().cpu() @ W.float().cpu().t(), atol=ATOL, rtol=RTOL)


@pytest.mark.parametrize("T,r", [(32, 16), (9, 32), (70, 64)])
def test_packed_lora_stack_equals_row_major(ops, cuda, T, r):
    """Pre-tiled B stacks are a pure re-arrangement of B_all: bit-identical results."""
    g = torch.Generator().manual_seed(r)
    K, N, n_ad = 256, 384, 5
    x = torch.randn(T, K, generator=g).bfloat16().to(cuda)
    W = (torch.randn(N, K, generator=g) * 0.05).bfloat16().to(cuda)
    A = (torch.randn(n_ad, 3 * r, K, generator=g) * 0.05).bfloat16()
    B = (torch.randn(n_ad, N, r, generator=g) * 0.05).bfloat16()
    slots = torch.randint(-1, n_ad, (T,), generator=g).int().to(cuda)
    st = _stack(ops, A, B, [r] * n_ad, [1.5] * n_ad, cuda, 3, (0, 128, 256, 384))
    y0 = ops.linear(x, W, st, slots)
    st2 = _stack(ops, A, B, [r] * n_ad, [1.5] * n_ad, cuda, 3, (0, 128, 256, 384)).pack_b()
    y1 = ops.linear(x, ops.PackedWeight(W), st2, slots)
    assert torch.equal(y0, y1)


@pytest.mark.parametrize("T,r,K,N", [(1, 16, 4096, 3072), (32, 16, 4096, 1536), (9, 32, 1024, 384), (70, 64, 688, 384),
                                     (200, 16, 512, 3072)])
def test_lora_linear_one_call(ops, cuda, T, r, K, N):
    """mlora_lora_linear (shrink + projection in one C call, u as caller scratch) against the two calls;
    repeated calls on one scratch buffer and no expired wait."""
    g = torch.Generator().manual_seed(T * 7 + r)
    n_ad, third = 5, N // 3
    offs = (0, third, 2 * third, N)
    x = torch.randn(T, K, generator=g).bfloat16().to(cuda)
    W = (torch.randn(N, K, generator=g) * 0.05).bfloat16().to(cuda)
    A = (torch.randn(n_ad, 3 * r, K, generator=g) * 0.05).bfloat16()
    B = (torch.randn(n_ad, N, r, generator=g) * 0.05).bfloat16()
    ranks = [r, r // 2, r, 8, r]
    for s in range(n_ad):
        for m in range(3):
            A[s, m * r + ranks[s]:(m + 1) * r] = 0
        B[s, :, ranks[s]:] = 0
    slots = torch.randint(-1, n_ad, (T,), generator=g).int().to(cuda)
    st = _stack(ops, A, B, ranks, [1.5, 2.0, 0.5, 1.0, 3.0], cuda, 3, offs).pack_b()
    Wp = ops.PackedWeight(W)
    want = ops.linear(x, Wp, st, slots)
    u_want = ops.lora_shrink(x, st, slots)
    for _ in range(3):
        u = torch.full((T, 3 * st.r_max), float("nan"), device=cuda)
        got = ops.linear(x, Wp, st, slots, u=u, with_shrink=True)
        torch.cuda.synchronize()
        assert int(ops.workspace(4, cuda, "linear")[:4].view(torch.int32)) == 0, "a bounded wait expired"
        rows = (slots >= 0).nonzero().flatten()
        torch.testing.assert_close(u[rows], u_want[rows], atol=1e-3, rtol=1e-4)
        torch.testing.assert_close(got.float(), want.float(), atol=ATOL, rtol=RTOL)


def test_lora_linear_one_call_gate_up(ops, cuda):
    """The same through the interleaved gate/up projection with SiLU*up in the output write."""
    g = torch.Generator().manual_seed(5)
    T, K, I, r, n_ad = 24, 512, 1024, 16, 4
    x = torch.randn(T, K, generator=g).bfloat16().to(cuda)
    Wg = (torch.randn(I, K, generator=g) * 0.05).bfloat16()
    Wu = (torch.randn(I, K, generator=g) * 0.05).bfloat16()
    A = (torch.randn(n_ad, 2 * r, K, generator=g) * 0.05).bfloat16()
    Bg = (torch.randn(n_ad, I, r, generator=g) * 0.05).bfloat16()
    Bu = (torch.randn(n_ad, I, r, generator=g) * 0.05).bfloat16()
    model = load("model")
    z = torch.zeros_like(Bg)
    B = torch.stack([model.interleave_gate_up(torch.cat([Bg, z], 2)[s], torch.cat([z, Bu], 2)[s]) for s in range(n_ad)])
    W = model.interleave_gate_up(Wg, Wu).to(cuda)
    slots = torch.randint(-1, n_ad, (T,), generator=g).int().to(cuda)
    st = ops.LoraStack(A.to(cuda), B.to(cuda), _i32([r] * n_ad, cuda), torch.full((n_ad,), 2.0, device=cuda), r, 2, None)
    want = ops.linear(x, W, st, slots, flags=ops.SILU_MUL)
    got = ops.linear(x, W, st, slots, flags=ops.SILU_MUL, with_shrink=True)
    torch.cuda.synchronize()
    assert int(ops.workspace(4, cuda, "linear")[:4].view(torch.int32)) == 0, "a bounded wait expired"
    torch.testing.assert_close(got.float(), want.float(), atol=ATOL, rtol=RTOL)


@pytest.mark.parametrize("T,K,r,n_mod,mixing", [(256, 4096, 16, 3, "runs"), (300, 688, 8, 3, "runs"), (1000, 1024, 64, 3, "runs"),
                                                (384, 512, 16, 1, "random"), (257, 4096, 64, 2, "random"),
                                                (512, 256, 128, 2, "random")])
def test_prefill_shrink_on_tensor_cores(ops, cuda, T, K, r, n_mod, mixing):
    """T >= 256 rows take the grouped-GEMM shrink: contiguous runs of one adapter (prompt rows) and fully mixed
    rows (many distinct adapters per 128-row tile -> several passes), rows without adapter, ragged T and K."""
    g = torch.Generator().manual_seed(T + r)
    n_ad = 24
    x = torch.randn(T, K, generator=g).bfloat16()
    A = (torch.randn(n_ad, n_mod * r, K, generator=g) * 0.05).bfloat16()
    ranks = [(r, r // 2, r)[s % 3] for s in range(n_ad)]
    for s in range(n_ad):
        for m in range(n_mod):
            A[s, m * r + ranks[s]:(m + 1) * r] = 0
    if mixing == "runs":
        ids = torch.randint(-1, n_ad, (T // 50 + 1,), generator=g)
        slots = ids.repeat_interleave(50)[:T].int()
    else:
        slots = torch.randint(-1, n_ad, (T,), generator=g).int()
    slots[-1] = n_ad + 3  # out of range = no adapter
    B = torch.zeros(n_ad, 128, r, dtype=torch.bfloat16)
    st = ops.LoraStack(A.to(cuda), B.to(cuda), _i32(ranks, cuda), torch.ones(n_ad, device=cuda), r, n_mod,
                       tuple(range(0, 128 * n_mod + 1, 128)) if n_mod > 1 else None)
    u = torch.full((T, n_mod * r), float("nan"), device=cuda)
    ops.lora_shrink(x.to(cuda), st, slots.to(cuda), out=u)
    want = torch.zeros(T, n_mod * r)
    for t in range(T):
        s = int(slots[t])
        if 0 <= s < n_ad:
            want[t] = A[s].float() @ x[t].float()
    torch.testing.assert_close(u.cpu(), want, atol=2e-3, rtol=1e-4)


@pytest.mark.parametrize("T,K,N,lora,run", [(2048, 256, 12288, False, 300), (2000, 320, 12288, True, 300),
                                             (5000, 128, 6144, True, 300), (2304, 192, 12288, True, 20),
                                             (1500, 256, 12288, True, 300), (1100, 128, 24576, True, 7)])
def test_prefill_size_projection_in_waves(ops, cuda, T, K, N, lora, run):
    """Enough tiles that the projection kernel deals whole tiles in L2-friendly waves instead of stream-K ranges
    (ragged last token tile, narrower last token-tile group), with the LoRA expand and the grouped-GEMM shrink.
    From about 600 whole 256-token tiles on the kernel takes 256-token tiles (the first four cases and the last),
    else 128-token ones; adapters changing every ``run`` rows put more adapters into a tile than its operand cache
    holds (the stages then go through the token ring)."""
    g = torch.Generator().manual_seed(T)
    x = torch.randn(T, K, generator=g).bfloat16().to(cuda)
    W = (torch.randn(N, K, generator=g) * 0.05).bfloat16().to(cuda)
    want = x.float() @ W.float().t()
    st = slots = None
    if lora:
        n_ad, r, third = (6 if run >= 100 else 24), 16, N // 3
        A = (torch.randn(n_ad, 3 * r, K, generator=g) * 0.05).bfloat16().to(cuda)
        B = (torch.randn(n_ad, N, r, generator=g) * 0.05).bfloat16().to(cuda)
        slots = (torch.arange(T) // run % (n_ad + 1) - 1).int().to(cuda)  # runs of rows, some without adapter
        st = ops.LoraStack(A, B, _i32([r] * n_ad, cuda), torch.full((n_ad,), 2.0, device=cuda), r, 3,
                           (0, third, 2 * third, N)).pack_b()
        for s in range(n_ad):
            rows = (slots == s).nonzero().flatten()
            for m in range(3):
                u = x[rows].float() @ A[s, m * r:(m + 1) * r].float().t()
                want[rows, m * third:(m + 1) * third] += 2.0 * (u @ B[s, m * third:(m + 1) * third].float().t())
    y = ops.linear(x, ops.PackedWeight(W), st, slots)
    torch.cuda.synchronize()
    assert int(ops.workspace(4, cuda, "linear")[:4].view(torch.int32)) == 0, "a bounded wait expired"
    torch.testing.assert_close(y.float(), want, atol=ATOL, rtol=RTOL)


@pytest.mark.parametrize("T,H,r,n_mod", [(1, 4096, 16, 3), (32, 4096, 16, 3), (7, 5120, 64, 1), (40, 256, 8, 3), (3, 8192, 32, 2)])
def test_fused_rmsnorm_and_shrink(ops, cuda, T, H, r, n_mod):
    """mlora_residual_rmsnorm_shrink against the two kernels it replaces: new residual, normalised rows and shrink
    outputs (the shrink reads the bf16-rounded normalised row in both forms, so the results differ only by fp32
    summation order); the input residual buffer is left untouched."""
    g = torch.Generator().manual_seed(T + H)
    n_ad = 5
    res = torch.randn(T, H, generator=g).to(cuda)
    delta = torch.randn(T, H, generator=g).bfloat16().to(cuda)
    w = (1.0 + 0.1 * torch.randn(H, generator=g)).bfloat16().to(cuda)
    A = (torch.randn(n_ad, n_mod * r, H, generator=g) * 0.05).bfloat16().to(cuda)
    B = torch.zeros(n_ad, 128 * n_mod, r, dtype=torch.bfloat16, device=cuda)
    st = ops.LoraStack(A, B, _i32([r] * n_ad, cuda), torch.ones(n_ad, device=cuda), r, n_mod,
                       tuple(range(0, 128 * n_mod + 1, 128)) if n_mod > 1 else None)
    slots = torch.randint(-1, n_ad, (T,), generator=g).int().to(cuda)
    # reference: the two separate kernels
    res_ref = res.clone()
    xn_ref = ops.residual_rmsnorm(delta, res_ref, w, 1e-5)
    u_ref = ops.lora_shrink(xn_ref, st, slots)
    # fused
    res_in, res_out = res.clone(), torch.full_like(res, float("nan"))
    xn = torch.empty(T, H, dtype=torch.bfloat16, device=cuda)
    u = torch.full((T, n_mod * r), float("nan"), device=cuda)
    ops.residual_rmsnorm_shrink(delta, res_in, res_out, w, 1e-5, xn, st, slots, u)
    torch.cuda.synchronize()
    assert torch.equal(res_in, res)
    assert torch.equal(res_out, res_ref)
    assert torch.equal(xn, xn_ref)
    rows = (slots >= 0).nonzero().flatten()
    torch.testing.assert_close(u[rows], u_ref[rows], atol=1e-3, rtol=1e-4)
    assert float(u[(slots < 0).nonzero().flatten()].abs().sum()) == 0.0


@pytest.mark.parametrize("tp", [1, 2, 8])
def test_projection_on_13b_tensor_parallel_shapes(ops, cuda, tp):
    """Llama-2-13B projections (hidden 5120, intermediate 13824) as a rank sees them under tensor parallelism 1/2/8
    -- row and k-block counts that are not powers of two, e.g. in = 640 or 1728 -- at decode and prefill sizes."""
    H, I = 5120, 13824
    shapes = {"qkv": (3 * H // tp, H), "o": (H, H // tp), "gu": (2 * I // tp, H), "down": (H, I // tp)}
    for name, (out_f, in_f) in shapes.items():
        g = torch.Generator(device=cuda).manual_seed(out_f + in_f)
        W = (torch.randn(out_f, in_f, device=cuda, generator=g) * 0.02).bfloat16()
        Wp = ops.PackedWeight(W)
        for T in (1, 32, 600):
            x = torch.randn(T, in_f, device=cuda, generator=g).bfloat16()
            y = ops.linear(x, Wp, flags=ops.SILU_MUL if name == "gu" else 0).float()
            ref = x.float() @ W.float().t()
            if name == "gu":
                r = ref.view(T, out_f // 16, 2, 8)
                ref = (torch.nn.functional.silu(r[:, :, 0]) * r[:, :, 1]).reshape(T, out_f // 2)
            torch.cuda.synchronize()
            assert int(ops.workspace(4, cuda, "linear")[:4].view(torch.int32)) == 0, "a bounded wait expired"
            torch.testing.assert_close(y, ref, atol=2e-2 + 1e-2 * float(ref.abs().max()), rtol=0)


@pytest.mark.parametrize("T,n_ad,r,K,N", [(128, 128, 64, 512, 640), (32, 32, 64, 1024, 256), (100, 60, 32, 256, 384), (16, 16, 64, 256, 128)])
def test_every_row_its_own_adapter(ops, cuda, T, n_ad, r, K, N):
    """More distinct adapters in a token tile than the shared-memory operand cache holds (every request with its own
    adapter, ranks cycling 8/16/32/64 padded to the pitch): the expand is served in rounds of the cache."""
    g = torch.Generator().manual_seed(T + n_ad)
    x = torch.randn(T, K, generator=g).bfloat16()
    W = (torch.randn(N, K, generator=g) * 0.05).bfloat16()
    ranks = [min(r, (8, 16, 32, 64)[i % 4]) for i in range(n_ad)]
    A = (torch.randn(n_ad, r, K, generator=g) * 0.05).bfloat16()
    B = (torch.randn(n_ad, N, r, generator=g) * 0.05).bfloat16()
    for i, rk in enumerate(ranks):
        A[i, rk:] = 0
        B[i, :, rk:] = 0
    slots = torch.randperm(n_ad, generator=g)[:T].int() if n_ad >= T else torch.randint(0, n_ad, (T,), generator=g).int()
    slots[T // 2] = -1
    st = ops.LoraStack(A.to(cuda), B.to(cuda), _i32(ranks, cuda), torch.full((n_ad,), 0.5, device=cuda), r, 1, (0, N)).pack_b()
    want = x.float() @ W.float().t()
    for t in range(T):
        s = int(slots[t])
        if s >= 0:
            want[t] += 0.5 * (B[s].float() @ (A[s].float() @ x[t].float()))
    for _ in range(2):  # twice: the cache hand-shake counters carry over nothing between launches
        y = ops.linear(x.to(cuda), ops.PackedWeight(W.to(cuda)), st, slots.to(cuda)).float().cpu()
        torch.cuda.synchronize()
        assert int(ops.workspace(4, cuda, "linear")[:4].view(torch.int32)) == 0, "a bounded wait expired"
        torch.testing.assert_close(y, want, atol=ATOL, rtol=RTOL)
    # the same through the per-row expand (base projection, then a kernel laid out by (row, output feature)), with
    # the pre-tiled and the row-major B stack, bf16 and fp32 outputs
    st_rm = ops.LoraStack(A.to(cuda), B.to(cuda), _i32(ranks, cuda), torch.full((n_ad,), 0.5, device=cuda), r, 1, (0, N))
    for stack in (st, st_rm):
        y = ops.linear(x.to(cuda), ops.PackedWeight(W.to(cuda)), stack, slots.to(cuda), flags=ops.LORA_PER_ROW).float().cpu()
        torch.testing.assert_close(y, want, atol=ATOL, rtol=RTOL)
    y32 = ops.linear(x.to(cuda), W.to(cuda), st_rm, slots.to(cuda), flags=ops.LORA_PER_ROW | ops.OUT_F32).cpu()
    torch.testing.assert_close(y32, want, atol=ATOL, rtol=RTOL)
    # the rank-compact split layout (every adapter stored as rank/8 slices [out, 8]): same sums in the same order
    st_sp = ops.LoraStack(A.to(cuda), B.to(cuda), _i32(ranks, cuda), torch.full((n_ad,), 0.5, device=cuda), r, 1, (0, N))
    st_sp.split_b(ranks)
    assert st_sp.B_split.shape == (sum(rk // 8 for rk in ranks), N, 8)          # rank-proportional storage
    assert st_sp.rank_tbl.cpu().tolist()[:n_ad] == ranks
    y32s = ops.linear(x.to(cuda), W.to(cuda), st_sp, slots.to(cuda), flags=ops.LORA_PER_ROW | ops.OUT_F32).cpu()
    assert torch.equal(y32s, y32)
    ys = ops.linear(x.to(cuda), ops.PackedWeight(W.to(cuda)), st_sp.pack_b(), slots.to(cuda), flags=ops.LORA_PER_ROW).float().cpu()
    torch.testing.assert_close(ys, want, atol=ATOL, rtol=RTOL)


def test_per_row_expand_with_fused_modules(ops, cuda):
    """Per-row expand over a fused q/k/v stack (three modules, each reading its own slice of u), rank pitches 16 and 32."""
    for r in (16, 32):
        g = torch.Generator().manual_seed(r)
        T, K, n_ad, offs = 50, 256, 40, (0, 256, 384, 512)
        x = torch.randn(T, K, generator=g).bfloat16()
        W = (torch.randn(512, K, generator=g) * 0.05).bfloat16()
        A = (torch.randn(n_ad, 3 * r, K, generator=g) * 0.05).bfloat16()
        B = (torch.randn(n_ad, 512, r, generator=g) * 0.05).bfloat16()
        slots = torch.randint(-1, n_ad, (T,), generator=g).int()
        st = _stack(ops, A, B, [r] * n_ad, [1.5] * n_ad, cuda, 3, offs)
        want = x.float() @ W.float().t()
        for t in range(T):
            s = int(slots[t])
            if s >= 0:
                for m in range(3):
                    u = A[s, m * r:(m + 1) * r].float() @ x[t].float()
                    want[t, offs[m]:offs[m + 1]] += 1.5 * (B[s, offs[m]:offs[m + 1]].float() @ u)
        y = ops.linear(x.to(cuda), W.to(cuda), st, slots.to(cuda), flags=ops.LORA_PER_ROW).float().cpu()
        y2 = ops.linear(x.to(cuda), ops.PackedWeight(W.to(cuda)), st.pack_b(), slots.to(cuda), flags=ops.LORA_PER_ROW).float().cpu()
        torch.testing.assert_close(y, want, atol=ATOL, rtol=RTOL)
        torch.testing.assert_close(y2, want, atol=ATOL, rtol=RTOL)
        # split layout with mixed ranks over the three modules (rank below the pitch for every third adapter)
        rk = [r if i % 3 else 8 for i in range(n_ad)]
        A2, B2 = A.clone(), B.clone()
        for i, q in enumerate(rk):
            for m in range(3):
                A2[i, m * r + q:(m + 1) * r] = 0
            B2[i, :, q:] = 0
        st2 = _stack(ops, A2, B2, rk, [1.5] * n_ad, cuda, 3, offs)
        ya = ops.linear(x.to(cuda), W.to(cuda), st2, slots.to(cuda), flags=ops.LORA_PER_ROW | ops.OUT_F32).cpu()
        st2.split_b(rk)
        yb = ops.linear(x.to(cuda), W.to(cuda), st2, slots.to(cuda), flags=ops.LORA_PER_ROW | ops.OUT_F32).cpu()
        assert torch.equal(ya, yb)


def test_attention_with_the_output_projection_shrink_in_its_tail(ops, cuda):
    """``mlora_paged_attention_shrink``: the same attention output, bit for bit, plus u = A[slot] . out computed by the
    (row, head) CTAs themselves (per-head partial sums added in head order by the last head to finish); compared
    with the separate shrink kernel on the attention output, twice in a row (the arrival counters reset themselves)."""
    Hq, Hkv, D, ps, theta = 32, 32, 128, 16, 10000.0
    lens = [int(n) for n in np.random.default_rng(3).integers(40, 300, 24)]
    B = len(lens)
    kp, vp, qkv, bt = _paged_case(7, B, Hq, Hkv, D, ps, lens, cuda)
    slot_rows, pos = _i32(np.arange(B), cuda), _i32(lens, cuda)
    g = torch.Generator().manual_seed(11)
    for r, ranks in ((16, [16] * 6), (64, [8, 16, 32, 64, 64, 16])):
        n_ad = len(ranks)
        A = (torch.randn(n_ad, r, Hq * D, generator=g) * 0.05).bfloat16()
        for i, rk in enumerate(ranks):
            A[i, rk:] = 0
        st = ops.LoraStack(A.to(cuda), torch.zeros(n_ad, 8, r, dtype=torch.bfloat16, device=cuda), _i32(ranks, cuda),
                           torch.ones(n_ad, device=cuda), r, 1, (0, 8))
        slots = torch.randint(-1, n_ad, (B,), generator=g).int().to(cuda)
        assert ops.attention_shrink_fits(B, Hq, bt.shape[1], st)
        work = ops.new_workspace(load("_lib").lib().mlora_paged_attention_shrink_workspace(B, Hq, r), cuda)
        for rep in range(2):
            kp1, vp1, kp2, vp2 = kp.to(cuda), vp.to(cuda), kp.to(cuda), vp.to(cuda)
            want = ops.paged_attention(qkv.to(cuda), kp1, vp1, _i32(bt, cuda), slot_rows, pos, Hq, Hkv, D, ps, theta, True)
            u_want = ops.lora_shrink(want, st, slots)
            out = torch.empty_like(want)
            u = torch.full((B, r), float("nan"), device=cuda)
            ops.paged_attention_shrink(qkv.to(cuda), kp2, vp2, _i32(bt, cuda), slot_rows, pos, Hq, Hkv, D, ps, theta, True,
                                       out, st, slots, u, work)
            torch.cuda.synchronize()
            assert torch.equal(out, want) and torch.equal(kp1, kp2) and torch.equal(vp1, vp2)
            torch.testing.assert_close(u, u_want, atol=2e-3, rtol=2e-3)
            assert float(u[slots < 0].abs().sum()) == 0.0
        assert int(work[: 4 * B].view(torch.int32).abs().sum()) == 0
    # few rows: the library would split the context; the fused form is refused with the way out in the message
    with pytest.raises(Exception, match="split-context"):
        ops.paged_attention_shrink(qkv[:2].to(cuda), kp.to(cuda), vp.to(cuda), _i32(bt[:2], cuda), slot_rows[:2], pos[:2], 4, 4, D,
                                   ps, theta, True, torch.empty(2, 4 * D, dtype=torch.bfloat16, device=cuda), st, slots[:2],
                                   torch.empty(2, 64, device=cuda), work)
