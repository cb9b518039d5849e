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

    # a request whose partial results do not fit the built-in array is refused, with the sizes in the message
    rc = lib.mlora_paged_attention_static(ptr(qkv), qkv.stride(0), ptr(kp), ptr(vp), ptr(bt), max_pages, ptr(slot),
                                          ptr(pos), 4096, 64, 64, 128, ps, theta, 1, ptr(out_b), out_b.stride(0), 16,
                                          stream)
    assert rc == -3 and b"16777216" in lib.mlora_last_error()
