"""Seeded request mixes with the shapes of the reference's drivers."""
import numpy as np
import pytest

from conftest import load


def test_reference_request_mixes():
    synth = load("synth")
    u = synth.request_mix("uniform", 32)
    assert u.tolist() == sorted(u.tolist()) and u.min() >= 0 and u.max() < 6   # ceil(sqrt(32)) = 6, sorted
    assert synth.request_mix("uniform", 32).tolist() == u.tolist()              # seeded
    assert synth.request_mix("distinct", 5).tolist() == [0, 1, 2, 3, 4]
    assert synth.request_mix("identical", 4).tolist() == [0, 0, 0, 0]
    with pytest.raises(ValueError):
        synth.request_mix("zipf", 4)
    ranks, wids = synth.request_mix_by_rank("distinct", 10, [3, 4], [8, 64])
    assert ranks.tolist() == [-1, -1, -1, 8, 8, 8, 64, 64, 64, 64]               # rows without adapter in front
    assert wids.tolist() == [-1, -1, -1, 0, 1, 2, 0, 1, 2, 3]
    ranks, wids = synth.request_mix_by_rank("uniform", 8, [4, 4], [16, 32])
    assert (wids >= 0).all() and wids[:4].tolist() == sorted(wids[:4].tolist()) and wids.max() < 2
    with pytest.raises(ValueError):
        synth.request_mix_by_rank("identical", 2, [3], [8])


def test_zipf_ids_are_skewed_and_uniform_ids_cover_the_range():
    synth = load("synth")
    z = synth.adapter_ids_zipf(4096, 64)
    counts = np.bincount(z, minlength=64)
    assert counts[0] > 4 * counts[32:].mean() and z.min() >= 0 and z.max() < 64
    u = synth.adapter_ids_uniform(4096, 16)
    assert set(u.tolist()) == set(range(16))
