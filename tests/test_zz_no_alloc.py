"""The allocation-free paged-attention entry point (scratch inside the library image).

Collected last on purpose (file name): a run that stops at the first failure has then already run
every other test.  Calls the C ABI directly, twice in a row, and compares with the ordinary entry
point that takes a caller-provided scratch buffer.
"""
import ctypes as C

import numpy as np
import pytest
import torch

from conftest import load
from oracle import ops as oops

pytestmark = pytest.mark.gpu


def _case(seed, B, Hq, Hkv, D, ps, lens, dev):
    g = torch.Generator().manual_seed(seed)
    need = [(n + 1 + ps - 1) // ps for n in lens]
    max_pages = max(need) + 1
    n_pages = sum(need) + 2
    ids = torch.randperm(n_pages, generator=g)[: sum(need)].tolist()
    bt = np.zeros((B, max_pages), dtype=np.int32)
    it = iter(ids)
    for b in range(B):
        for p in range(need[b]):
            bt[b, p] = next(it)
    kp = torch.randn(n_pages, Hkv, ps, D, generator=g).bfloat16().to(dev)
    vp = torch.randn(n_pages, Hkv, ps, D, generator=g).bfloat16().to(dev)
    qkv = torch.randn(B, (Hq + 2 * Hkv) * D, generator=g).bfloat16().to(dev)
    i32 = lambda a: torch.as_tensor(np.asarray(a, dtype=np.int32), device=dev)
    return kp, vp, qkv, i32(bt), i32(np.arange(B)), i32(lens), max_pages


def _oracle_decode(kp, vp, qkv, bt, lens, Hq, Hkv, D, ps, theta):
    """What the call must produce, on the CPU: rotate q and the new k, append k/v at position len, attend."""
    B = len(lens)
    kp, vp, qkv, bt = kp.cpu().clone(), vp.cpu().clone(), qkv.cpu(), bt.cpu().numpy()
    pos = torch.tensor(lens)
    q = qkv[:, : Hq * D].view(B, Hq, D)
    k = qkv[:, Hq * D:(Hq + Hkv) * D].view(B, Hkv, D)
    v = qkv[:, (Hq + Hkv) * D:].view(B, Hkv, D)
    qr = oops.rope_rotate_half(q, pos, theta)
    kr = oops.rope_rotate_half(k, pos, theta).bfloat16()
    for b in range(B):
        page = bt[b, lens[b] // ps]
        kp[page, :, lens[b] % ps] = kr[b]
        vp[page, :, lens[b] % ps] = v[b]
    return oops.paged_attention_decode(qr, kp, vp, bt, np.asarray(lens) + 1).reshape(B, Hq * D)


def test_static_scratch_entry_matches_caller_scratch_entry(cuda):
    """Runs where a caller may not allocate: the library's own 16 MiB array stands in for the scratch
    buffer.  Two back-to-back calls share that array; each must equal the result of the ordinary call."""
    lib = load("_lib").lib()
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    ptr = lambda t: C.c_void_p(t.data_ptr())
    assert lib.mlora_paged_attention_static_max_bytes() == 16 << 20
    Hq, Hkv, D, ps, theta = 8, 4, 128, 16, 10000.0
    for call, (lens, n_splits) in enumerate([([5, 200, 77, 16, 331], 4), ([640, 3, 129], 7)]):
        B = len(lens)
        kp, vp, qkv, bt, slot, pos, max_pages = _case(10 + call, B, Hq, Hkv, D, ps, lens, cuda)
        kp2, vp2 = kp.clone(), vp.clone()
        out_a = torch.zeros(B, Hq * D, dtype=torch.bfloat16, device=cuda)
        out_b = torch.zeros_like(out_a)
        nbytes = lib.mlora_paged_attention_workspace(B, Hq, D, n_splits)
        work = torch.empty(nbytes, dtype=torch.uint8, device=cuda)
        rc = lib.mlora_paged_attention(ptr(qkv), qkv.stride(0), ptr(kp), ptr(vp), ptr(bt), max_pages, ptr(slot),
                                       ptr(pos), B, Hq, Hkv, D, ps, theta, 1, ptr(out_a), out_a.stride(0), n_splits,
                                       ptr(work), nbytes, stream)
        assert rc == 0, lib.mlora_last_error()
        rc = lib.mlora_paged_attention_static(ptr(qkv), qkv.stride(0), ptr(kp2), ptr(vp2), ptr(bt), max_pages,
                                              ptr(slot), ptr(pos), B, Hq, Hkv, D, ps, theta, 1, ptr(out_b),
                                              out_b.stride(0), n_splits, stream)
        assert rc == 0, lib.mlora_last_error()
        torch.cuda.synchronize()
        torch.testing.assert_close(out_b.float(), out_a.float(), atol=2e-2, rtol=1e-2)
        assert torch.equal(out_b, out_a)  # same kernels, same order of operations
        assert torch.equal(kp2, kp) and torch.equal(vp2, vp)  # the fused append wrote the same pages
        assert out_a.float().abs().sum() > 0
        # and both equal the CPU oracle (bf16 result against fp32: the tolerance of the other attention tests)
        kp0, vp0, _, _, _, _, _ = _case(10 + call, B, Hq, Hkv, D, ps, lens, cuda)
        want = _oracle_decode(kp0, vp0, qkv, bt, lens, Hq, Hkv, D, ps, theta)
        torch.testing.assert_close(out_b.float().cpu(), want, atol=2e-2, rtol=1e-2)

    # n_splits = 0, the form an embedder uses: the library picks the split count itself (here 2: 48 rows x 8
    # heads leave SMs idle unless every row's context is cut in two); its own choices always fit the array
    # (at most 592 (row, head) pairs x 16 splits x (D+2) floats = 4.9 MB), so nothing is ever refused in this form
    lens = [int(n) for n in np.random.default_rng(5).integers(200, 700, 48)]
    B, Hq2 = len(lens), 8
    kp, vp, qkv, bt, slot, pos, max_pages = _case(77, B, Hq2, Hkv, D, ps, lens, cuda)
    kp0, vp0 = kp.clone(), vp.clone()
    out = torch.zeros(B, Hq2 * D, dtype=torch.bfloat16, device=cuda)
    rc = lib.mlora_paged_attention_static(ptr(qkv), qkv.stride(0), ptr(kp), ptr(vp), ptr(bt), max_pages, ptr(slot),
                                          ptr(pos), B, Hq2, Hkv, D, ps, theta, 1, ptr(out), out.stride(0), 0, stream)
    assert rc == 0, lib.mlora_last_error()
    torch.cuda.synchronize()
    want = _oracle_decode(kp0, vp0, qkv, bt, lens, Hq2, Hkv, D, ps, theta)
    torch.testing.assert_close(out.float().cpu(), want, atol=2e-2, rtol=1e-2)

    # invalid arguments are reported as such before any size is computed from them
    for bad_T, bad_splits in ((-1, 4), (B, 65)):
        rc = lib.mlora_paged_attention_static(ptr(qkv), qkv.stride(0), ptr(kp), ptr(vp), ptr(bt), max_pages,
                                              ptr(slot), ptr(pos), bad_T, Hq2, Hkv, D, ps, theta, 1, ptr(out),
                                              out.stride(0), bad_splits, stream)
        assert rc == -1, (rc, lib.mlora_last_error())

    # a request whose partial results do not fit the built-in array is refused, with the sizes in the message
    rc = lib.mlora_paged_attention_static(ptr(qkv), qkv.stride(0), ptr(kp), ptr(vp), ptr(bt), max_pages, ptr(slot),
                                          ptr(pos), 4096, 64, 64, 128, ps, theta, 1, ptr(out_b), out_b.stride(0), 16,
                                          stream)
    assert rc == -3 and b"16777216" in lib.mlora_last_error()
