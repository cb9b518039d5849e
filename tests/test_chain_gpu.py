"""``mlora_decode_chain``: several dependent projections (with the residual + RMSNorm and LoRA shrink between
them) in one persistent launch must give the same bits as the same sequence of separate calls, whose results the
other tests hold against the CPU oracle; plus an oracle check of its own and the failure path of its waits."""
import pytest
import torch

from conftest import load
from oracle import ops as oops

pytestmark = pytest.mark.gpu


def _stack(ops, n_ad, r, in_f, outs, dev, g, interleave=False, ranks=None):
    """A packed LoRA stack over modules with ``outs`` output rows each (all reading the same input)."""
    n_mod = len(outs)
    A = ((torch.rand(n_ad, n_mod * r, in_f, generator=g) * 2 - 1) / in_f ** 0.5).bfloat16()
    Bs = [(torch.randn(n_ad, o, r, generator=g) * 0.02).bfloat16() for o in outs]
    rk = torch.full((n_ad,), r, dtype=torch.int32) if ranks is None else torch.tensor(ranks, dtype=torch.int32)
    for s in range(n_ad):
        for m in range(n_mod):
            A[s, m * r + int(rk[s]):(m + 1) * r] = 0
            Bs[m][s, :, int(rk[s]):] = 0
    if interleave:
        model = load("model")
        z = torch.zeros_like(Bs[0])
        g2, u2 = torch.cat([Bs[0], z], 2), torch.cat([z, Bs[1]], 2)
        B = torch.stack([model.interleave_gate_up(g2[s], u2[s]) for s in range(n_ad)])
    else:
        B = torch.cat(Bs, 1)
    offs = [0]
    for o in outs:
        offs.append(offs[-1] + o)
    st = ops.LoraStack(A.to(dev), B.contiguous().to(dev), rk.to(dev), torch.linspace(0.5, 2.0, n_ad).to(dev), r, n_mod,
                       tuple(offs))
    st.host = (A, Bs)
    return st.pack_b()


def _layer_case(ops, dev, T, H, I, n_ad, r, seed, lora_mlp=False, ranks=None):
    g = torch.Generator().manual_seed(seed)
    model = load("model")
    mat = lambda o, i: (torch.randn(o, i, generator=g) * 0.02).bfloat16()
    host = dict(w_o=mat(H, H), w_g=mat(I, H), w_u=mat(I, H), w_down=mat(H, I), w_qkv=mat(3 * H, H),
                ln2=(1 + 0.1 * torch.randn(H, generator=g)).bfloat16(), ln1=(1 + 0.1 * torch.randn(H, generator=g)).bfloat16())
    c = dict(host=host)
    c["w_o"], c["w_down"], c["w_qkv"] = (ops.PackedWeight(host[k].to(dev)) for k in ("w_o", "w_down", "w_qkv"))
    c["w_gu"] = ops.PackedWeight(model.interleave_gate_up(host["w_g"], host["w_u"]).to(dev))
    c["ln1"], c["ln2"] = host["ln1"].to(dev), host["ln2"].to(dev)
    c["st_o"] = _stack(ops, n_ad, r, H, [H], dev, g, ranks=ranks)
    c["st_qkv"] = _stack(ops, n_ad, r, H, [H, H, H], dev, g, ranks=ranks)
    c["st_gu"] = _stack(ops, n_ad, r, H, [I, I], dev, g, interleave=True) if lora_mlp else None
    c["st_down"] = _stack(ops, n_ad, r, I, [H], dev, g) if lora_mlp and I <= 8192 else None
    c["attn"] = torch.randn(T, H, generator=g).bfloat16().to(dev)
    c["res0"] = torch.randn(T, H, generator=g).to(dev)
    slots = torch.randint(-1, n_ad, (T,), generator=g).to(torch.int32)
    c["slots_host"] = slots
    c["slots"] = slots.to(dev)
    return c


def _run(ops, c, T, H, I, chained, dev, work):
    bf = dict(dtype=torch.bfloat16, device=dev)
    res = c["res0"].clone()
    y, xn, act, qkv = (torch.zeros(T, n, **bf) for n in (H, H, I, 3 * H))
    us = {k: torch.zeros(T, (c[k].r_max * c[k].n_mod) if c[k] is not None else 8, dtype=torch.float32, device=dev)
          for k in ("st_o", "st_gu", "st_down", "st_qkv")}
    sl = c["slots"]
    if chained:
        S = ops.ChainStep
        steps = [S(x=c["attn"], W=c["w_o"], y=y, stack=c["st_o"], u=us["st_o"]),
                 S(x=xn, W=c["w_gu"], y=act, flags=ops.SILU_MUL, res=res, delta=y, norm_w=c["ln2"], eps=1e-5,
                   stack=c["st_gu"], u=us["st_gu"] if c["st_gu"] is not None else None),
                 S(x=act, W=c["w_down"], y=y, stack=c["st_down"], u=us["st_down"] if c["st_down"] is not None else None),
                 S(x=xn, W=c["w_qkv"], y=qkv, res=res, delta=y, norm_w=c["ln1"], eps=1e-5, stack=c["st_qkv"], u=us["st_qkv"])]
        assert ops.chain_supported(T, steps)
        st = c["st_o"]
        ops.decode_chain(steps, sl, st.ranks, st.scales, st.A_all.shape[0], work)
    else:
        def proj(x, W, st, u, out, flags=0):
            if st is None:
                return ops.linear(x, W, flags=flags, out=out, work=work)
            ops.lora_shrink(x, st, sl, out=u)
            return ops.linear(x, W, st, sl, u=u, flags=flags, out=out, work=work)
        proj(c["attn"], c["w_o"], c["st_o"], us["st_o"], y)
        ops.residual_rmsnorm(y, res, c["ln2"], 1e-5, out=xn)
        proj(xn, c["w_gu"], c["st_gu"], us["st_gu"], act, ops.SILU_MUL)
        proj(act, c["w_down"], c["st_down"], us["st_down"], y)
        ops.residual_rmsnorm(y, res, c["ln1"], 1e-5, out=xn)
        proj(xn, c["w_qkv"], c["st_qkv"], us["st_qkv"], qkv)
    torch.cuda.synchronize()
    return dict(res=res, y=y, xn=xn, act=act, qkv=qkv, u_qkv=us["st_qkv"])


@pytest.mark.parametrize("T,H,I,n_ad,r,lora_mlp", [
    (32, 4096, 11008, 16, 16, False),   # the benchmark's layer
    (7, 4096, 11008, 16, 16, False),    # 16-token tile, ragged batch
    (32, 1024, 2048, 6, 32, True),      # adapters on all seven projections, rank 32 (gate|up pitch 64)
    (12, 512, 1376, 3, 64, True),       # rank 64, ragged tiles (1376 = 10.75 row tiles per module)
    (1, 256, 688, 2, 16, True),         # a single row; K of the down projection not a multiple of 64
])
def test_chain_equals_separate_calls_bit_for_bit(ops, cuda, T, H, I, n_ad, r, lora_mlp):
    c = _layer_case(ops, cuda, T, H, I, n_ad, r, seed=T + H)
    lib = load("_lib").lib()
    need = max(lib.mlora_linear_workspace(T, k, n) for k, n in ((H, H), (H, 2 * I), (I, H), (H, 3 * H)))
    work = ops.new_workspace(need, cuda)
    want = _run(ops, c, T, H, I, False, cuda, work)
    for rep in range(3):  # back to back: the barrier counters reset themselves
        got = _run(ops, c, T, H, I, True, cuda, work)
        assert ops.status_word(work) == 0
        for k in want:
            assert torch.equal(got[k], want[k]), (k, rep, float((got[k].float() - want[k].float()).abs().max()))
    assert int(work[8:12].view(torch.int32)) == 0 and int(work[64:136].view(torch.int32).abs().sum()) == 0


def test_chain_against_the_cpu_oracle(ops, cuda):
    """The same layer segment on the CPU in fp32 (weights as rounded to bf16, stored activations rounded where the
    kernel stores them)."""
    T, H, I, n_ad, r = 9, 512, 1376, 4, 16
    c = _layer_case(ops, cuda, T, H, I, n_ad, r, seed=5)
    lib = load("_lib").lib()
    work = ops.new_workspace(max(lib.mlora_linear_workspace(T, k, n) for k, n in ((H, 2 * I), (I, H), (H, 3 * H))), cuda)
    got = _run(ops, c, T, H, I, True, cuda, work)
    h = c["host"]
    R = lambda t: t.bfloat16().float()
    slots = c["slots_host"].tolist()

    def lora(x, st, m, out_lo, out_hi):
        A, Bs = st.host
        d = torch.zeros(T, out_hi - out_lo)
        for t, s in enumerate(slots):
            if s >= 0:
                u = A[s, m * st.r_max:(m + 1) * st.r_max].float() @ x[t]
                d[t] = float(st.scales[s]) * (Bs[m][s].float() @ u)
        return d

    attn = c["attn"].float().cpu()
    y = R(attn @ h["w_o"].float().t() + lora(attn, c["st_o"], 0, 0, H))
    res = c["res0"].cpu() + y
    xn = R(oops.rmsnorm(res, h["ln2"], 1e-5))
    act = R(oops.silu_mul(xn @ h["w_g"].float().t(), xn @ h["w_u"].float().t()))
    y2 = R(act @ h["w_down"].float().t())
    res = res + y2
    xn2 = R(oops.rmsnorm(res, h["ln1"], 1e-5))
    qkv = xn2 @ h["w_qkv"].float().t() + torch.cat([lora(xn2, c["st_qkv"], m, m * H, (m + 1) * H) for m in range(3)], 1)
    torch.testing.assert_close(got["res"].cpu(), res, atol=2e-2, rtol=1e-2)
    torch.testing.assert_close(got["act"].float().cpu(), act, atol=2e-2, rtol=1e-2)
    torch.testing.assert_close(got["qkv"].float().cpu(), qkv, atol=2e-2, rtol=1e-2)


def test_chain_gives_up_cleanly_when_the_status_word_is_set(ops, cuda):
    """Every wait of the kernel also watches the status word, which is how one CTA's failure reaches the others.
    With the word set beforehand each grid-barrier wait returns at once: the launch ends without hanging, leaves
    the word set (the results are undefined) and its barrier counters at zero; after clearing the word the same
    buffers give the right answer again."""
    T, H, I = 8, 256, 688
    c = _layer_case(ops, cuda, T, H, I, 2, 16, seed=1)
    lib = load("_lib").lib()
    work = ops.new_workspace(max(lib.mlora_linear_workspace(T, k, n) for k, n in ((H, 2 * I), (I, H), (H, 3 * H))), cuda)
    want = _run(ops, c, T, H, I, False, cuda, work)
    work[:4].view(torch.int32).fill_(256)
    _run(ops, c, T, H, I, True, cuda, work)
    assert ops.status_word(work) != 0
    assert int(work[8:12].view(torch.int32)) == 0 and int(work[64:136].view(torch.int32).abs().sum()) == 0
    work.zero_()
    got = _run(ops, c, T, H, I, True, cuda, work)
    assert ops.status_word(work) == 0
    for k in want:
        assert torch.equal(got[k], want[k]), k
