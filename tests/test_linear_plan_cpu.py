"""Host-side planning of the tensor-core projection (``mlora_linear_plan``): whatever the shape, every tile -- or, at decode
sizes, every k-block of every tile -- is dealt to exactly one CTA.  No GPU: the plan is arithmetic on the shape (the SM
count falls back to a B200's 148 without a device)."""
import ctypes as C

import pytest

from conftest import load

SHAPES = [
    # T, in, out
    (1, 4096, 4096), (8, 4096, 12288), (32, 4096, 22016), (32, 11008, 4096), (32, 4096, 32000), (64, 4096, 22016),
    (128, 5120, 5120), (200, 256, 384), (512, 4096, 12288), (1000, 320, 12288), (1100, 128, 24576), (2048, 256, 12288),
    (4096, 4096, 4096), (4096, 11008, 4096), (5000, 128, 6144), (8192, 4096, 12288), (8192, 4096, 22016),
    (8192, 11008, 4096), (8192, 4096, 4096), (8200, 4096, 12288 + 64), (16384, 4096, 12288), (40000, 4096, 12288),
]


def _plan(T, K, N):
    lib = load("_lib").lib()
    v = (C.c_int32 * 12)()
    assert lib.mlora_linear_plan(T, K, N, v) == 0
    keys = ("bn", "grid", "row_tiles", "tok_tiles", "k_blocks", "per_cta", "gt", "lanes", "steps", "groups", "ch_last")
    return dict(zip(keys, list(v)))


def _walk(p, cta):
    """Tiles CTA ``cta`` visits, in order (the kernel's wave_tile, restated)."""
    out = []
    if p["lanes"] > 0:  # lane form
        j, lane = cta % p["gt"], cta // p["gt"]
        for g in range(p["groups"]):
            for s in range(p["steps"]):
                row, tok = lane + s * p["lanes"], g * p["gt"] + j
                if lane < p["lanes"] and row < p["row_tiles"] and tok < p["tok_tiles"]:
                    out.append(tok * p["row_tiles"] + row)
        return out
    full = p["groups"]  # chunk form: full groups of gt token tiles, then one narrower group
    for g in range(full + 1):
        gt = p["gt"] if g < full else p["tok_tiles"] - full * p["gt"]
        ch = p["steps"] if g < full else p["ch_last"]
        for qi in range(ch):
            q = cta * ch + qi
            if q < p["row_tiles"] * gt:
                j = q // p["row_tiles"]
                out.append((g * p["gt"] + j) * p["row_tiles"] + q % p["row_tiles"])
    return out


@pytest.mark.parametrize("T,K,N", SHAPES)
def test_every_tile_is_dealt_exactly_once(T, K, N):
    p = _plan(T, K, N)
    assert p["bn"] in (16, 32, 64, 128, 256) and 1 <= p["grid"] <= 148
    assert p["row_tiles"] == -(-N // 128) and p["tok_tiles"] == -(-T // p["bn"]) and p["k_blocks"] == -(-K // 64)
    n_tiles = p["row_tiles"] * p["tok_tiles"]
    if p["gt"] == 0:
        # contiguous ranges of k-block steps: CTA c owns [c * per_cta, (c + 1) * per_cta) of tiles * k_blocks
        total = n_tiles * p["k_blocks"]
        assert (p["grid"] - 1) * p["per_cta"] < total <= p["grid"] * p["per_cta"]
        assert p["bn"] <= 128
        return
    seen = []
    for c in range(p["grid"]):
        seen += _walk(p, c)
    assert sorted(seen) == list(range(n_tiles)), "a tile is missing or dealt twice"
    if p["lanes"] > 0:
        assert p["lanes"] == p["grid"] // p["gt"]
        assert p["gt"] == 1 or p["gt"] * p["bn"] * K * 2 <= 48e6  # the group's token rows stay L2-resident
        # at every step the CTAs of one lane -- one per token tile of the group -- read the same row tile (from HBM once)
        for lane in range(p["lanes"]):
            ctas = [c for c in range(p["grid"]) if c // p["gt"] == lane]
            assert len(ctas) == p["gt"]
            for s_ in range(p["steps"]):
                row = lane + s_ * p["lanes"]
                if row < p["row_tiles"]:
                    toks = sorted(t // p["row_tiles"] for c in ctas for t in _walk(p, c) if t % p["row_tiles"] == row)
                    assert toks == list(range(p["tok_tiles"]))  # every token tile, through this lane only
    slots = p["grid"] * (p["groups"] * p["steps"] + p["ch_last"])
    assert n_tiles / slots > 0.6, "more than 40 % of the slots idle"


def test_prompt_passes_take_256_token_tiles_and_decode_sizes_do_not():
    assert _plan(8192, 4096, 12288)["bn"] == 256
    assert _plan(8192, 4096, 4096)["bn"] == 256
    assert _plan(4096, 4096, 4096)["bn"] == 256      # 512 tiles >= 3 rounds of the grid
    assert _plan(1024, 4096, 4096)["bn"] == 128      # too few whole tiles for 256-token ones
    assert _plan(32, 4096, 4096)["bn"] == 32 and _plan(32, 4096, 4096)["gt"] == 0
    assert _plan(16, 4096, 4096)["bn"] == 16
    p = _plan(8192, 4096, 12288)
    assert (p["gt"], p["lanes"], p["steps"], p["groups"]) == (16, 9, 11, 2)
