"""CPU tests of the tensor-parallel FFN's host logic: shard bounds, Q8_0 block slicing, and that the
rank-ordered sum of the shard results (computed with the CPU restatement) is the unsharded FFN."""
import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
import __graft_entry__ as entry  # noqa: E402


def test_shard_bounds_tile_the_ffn_dimension():
    pkg = entry.load_package()
    for F in (1024, 17408):
        for world in (1, 2, 4, 8):
            spans = [pkg.tp.shard_bounds(F, world, r) for r in range(world)]
            assert spans[0][0] == 0 and spans[-1][1] == F
            assert all(a[1] == b[0] for a, b in zip(spans, spans[1:]))
            assert all((hi - lo) % 128 == 0 for lo, hi in spans)
    with pytest.raises(ValueError):
        pkg.tp.shard_bounds(1024, 3, 0)
    with pytest.raises(ValueError):
        pkg.tp.shard_bounds(17408, 16, 0)        # 1088 rows: not whole 128-row tiles


def test_sharded_sum_is_the_unsharded_ffn(orc):
    pkg = entry.load_package()
    H, F, N_OUT, M = 128, 512, 96, 3
    rng = np.random.default_rng(3)
    wg, wu = rng.normal(0, 0.05, (F, H)).astype(np.float32), rng.normal(0, 0.05, (F, H)).astype(np.float32)
    wd = rng.normal(0, 0.05, (N_OUT, F)).astype(np.float32)
    gate, up, down = orc.quantize_q8_0(wg), orc.quantize_q8_0(wu), orc.quantize_q8_0(wd)
    x = rng.normal(0, 1, (M, H)).astype(np.float32)
    q, d = orc.quantize_act(x)

    def ffn(world):
        f = F // world
        total = None
        for r in range(world):
            gu, dn = pkg.tp.shard_blocks(gate, up, down, F, H, N_OUT, world, r)
            assert gu.shape == (2 * f, H // 32, 34) and dn.shape == (N_OUT, f // 32, 34)
            y = orc.gemm_engine(gu, 2 * f, H, q, d)
            g, u = y[:, :f], y[:, f:]
            h = (g / (np.float32(1) + np.exp(-g, dtype=np.float32)) * u).astype(np.float32)
            hq, hd = orc.quantize_act(h)
            part = orc.gemm_engine(dn, N_OUT, f, hq, hd)
            total = part if total is None else (total + part).astype(np.float32)
        return total

    full = ffn(1)
    for world in (2, 4):
        assert np.abs(ffn(world) - full).max() / np.abs(full).max() < 1e-5
    # and the slices really are the weights' rows / K columns
    gu, dn = pkg.tp.shard_blocks(gate, up, down, F, H, N_OUT, 4, 1)
    assert np.array_equal(orc.dequant_q8_0(gu, 256, H)[:128], orc.dequant_q8_0(gate, F, H)[128:256])
    assert np.array_equal(orc.dequant_q8_0(dn, N_OUT, 128), orc.dequant_q8_0(down, N_OUT, F)[:, 128:256])
