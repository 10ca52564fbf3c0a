"""The Blackwell device model and policy: every emitted rTile is buildable and sane."""
import ctypes

import pytest
from hypothesis import given, settings, strategies as st

from mlir_roller_b200 import analyze, arch
from mlir_roller_b200.analyze import (MODE_1XTF32, MODE_3XTF32, MODE_BF16, MODE_F16, MatmulConfig,
                                      get_roller_hints)

TILES = {(t[0], t[1], t[2]) for t in arch.B200_KERNEL_TILES}
SKINNY = {(t[0], t[1]) for t in arch.B200_KERNEL_TILES if t[5] == 2}
TILES_16 = {(t[0], t[1], t[2]) for t in arch.B200_KERNEL_TILES if t[6] > 0}


def check_hint(h, M, N, K, mode):
    dev = arch.B200()
    sixteen = mode in (MODE_BF16, MODE_F16)
    assert (h.block_tile[0], h.block_tile[1], h.cta_group) in (TILES_16 if sixteen else TILES)
    assert h.rstep == (64 if sixteen else 32) and h.mode == mode
    assert h.matmul_config.el_bits == (16 if sixteen else 32)
    if h.layout == 3:
        # the CUDA-core kernel for a C of few rows: fp32-accurate class only, no tensor memory
        assert mode == MODE_3XTF32 and (h.block_tile, h.cta_group, h.tmem_cols) == ([16, 256], 1, 0)
        assert h.grid_size == -(-M // 16) * -(-N // 256) and h.est_us > 0 and h.valid
        return
    skinny = h.layout == 2
    assert skinny == ((h.block_tile[0], h.block_tile[1]) in SKINNY)
    assert h.tmem_cols == 2 * h.block_tile[0 if skinny else 1] <= dev.tmem_columns
    assert h.smem_cost * h.stages + 2048 <= dev.smem_cap == 227 * 1024
    assert h.block_tile[1 if skinny else 0] == 128 * h.cta_group
    assert h.grid_size == -(-M // h.block_tile[0]) * -(-N // h.block_tile[1])
    assert h.num_wave == -(-h.grid_size // (dev.compute_max_core // h.cta_group))
    assert h.est_us > 0 and h.valid


@pytest.mark.parametrize("mode", [MODE_1XTF32, MODE_3XTF32])
def test_readme_and_config_shapes(mode):
    shapes = [(2048, 2048, 2048), (8192, 4096, 4096), (4097, 2049, 8193), (16, 8192, 8192),
              (16384, 16384, 16384), (1024, 4096, 4096), (4096, 8192, 16384), (1, 1, 1)]
    for M, N, K in shapes:
        hints = get_roller_hints(MatmulConfig(M, N, K, 32), arch.B200(), topk=20, mode=mode)
        assert 1 <= len(hints) <= len(TILES)
        assert len({(h.block_tile[0], h.block_tile[1], h.cta_group) for h in hints}) == len(hints)
        est = [h.est_us for h in hints]
        assert est == sorted(est)
        for h in hints:
            check_hint(h, M, N, K, mode)


def test_large_square_prefers_the_cta_pair_tile():
    for mode in (MODE_1XTF32, MODE_3XTF32):
        top = get_roller_hints(MatmulConfig(8192, 8192, 8192, 32), arch.B200(), topk=1, mode=mode)[0]
        assert (top.block_tile, top.cta_group) == ([256, 256], 2)


def test_topk_and_dispatch():
    cfg = MatmulConfig(4096, 4096, 4096, 32)
    assert len(get_roller_hints(cfg, arch.B200(), topk=2)) == 2
    # the generic policy is still what a non-B200 device model gets
    assert get_roller_hints(cfg, arch.CUDA(), topk=1)[0].block_tile == [128, 128]
    with pytest.raises(ValueError):
        get_roller_hints(MatmulConfig(64, 64, 64, 8), arch.B200())
    with pytest.raises(ValueError):
        analyze.BlackwellPolicy(cfg, arch.B200(), mode=2)
    with pytest.raises(ValueError):
        analyze.BlackwellPolicy(cfg, arch.B200(), mode=MODE_BF16)   # fp32 elements, 16-bit mode


@pytest.mark.parametrize("mode", [None, MODE_BF16, MODE_F16])
def test_sixteen_bit_configs(mode):
    """A 16-bit MatmulConfig (el_bits = 16, src/analyze.py:31) ranks the 16-bit kernels: reduce
    step 64, same tiles, bf16 unless fp16 is asked for."""
    shapes = [(2048, 2048, 2048), (8192, 4096, 4096), (4097, 2049, 8193), (16, 8192, 8192), (1, 1, 1)]
    for M, N, K in shapes:
        hints = get_roller_hints(MatmulConfig(M, N, K, 16), arch.B200(), topk=20, mode=mode)
        assert 1 <= len(hints) <= len(TILES_16)
        assert [h.est_us for h in hints] == sorted(h.est_us for h in hints)
        for h in hints:
            check_hint(h, M, N, K, MODE_BF16 if mode is None else mode)
            assert h.smem_cost == (h.block_tile[0] + h.block_tile[1]) // h.cta_group * 128
    top = get_roller_hints(MatmulConfig(8192, 8192, 8192, 16), arch.B200(), topk=1)[0]
    assert (top.block_tile, top.cta_group) == ([256, 256], 2)
    assert "bf16" in top.kernel
    skinny = get_roller_hints(MatmulConfig(16, 8192, 8192, 16), arch.B200(), topk=1)[0]
    assert skinny.layout == 2
    # a TF32 mode on a 16-bit config falls back to bf16 rather than mixing types
    assert get_roller_hints(MatmulConfig(512, 512, 512, 16), arch.B200(), topk=1,
                            mode=MODE_3XTF32)[0].mode == MODE_BF16


@settings(max_examples=150, deadline=None)
@given(st.integers(1, 20000), st.integers(1, 20000), st.integers(1, 20000),
       st.sampled_from([MODE_1XTF32, MODE_3XTF32]))
def test_any_ragged_shape_gets_valid_hints(M, N, K, mode):
    hints = get_roller_hints(MatmulConfig(M, N, K, 32), arch.B200(), topk=3, mode=mode)
    assert hints
    for h in hints:
        check_hint(h, M, N, K, mode)


def test_tile_table_matches_the_library():
    """The table the search ranks is exactly what libroller_b200 was compiled with."""
    from mlir_roller_b200 import _lib
    lib_tiles = [(k.block_m, k.block_n, k.cta_group, k.stages_1x, k.stages_3x, k.layout, k.stages_16)
                 for k in _lib.kernel_tiles()]
    assert sorted(lib_tiles) == sorted(arch.B200_KERNEL_TILES)
    for k in _lib.kernel_tiles():
        want_tmem = 0 if k.layout == 3 else 2 * (k.block_m if k.layout == 2 else k.block_n)
        assert k.rstep == 32 and k.tmem_cols == want_tmem
        assert max(k.smem_1x, k.smem_3x, k.smem_16) <= 227 * 1024
        assert k.rstep_16 in (0, 64) and (k.rstep_16 == 0) == (k.stages_16 == 0)
        assert isinstance(k, ctypes.Structure)


def test_tune_cache_roundtrip(tmp_path):
    from mlir_roller_b200 import roller
    cfg = MatmulConfig(2048, 4096, 1024, 32)
    hint = get_roller_hints(cfg, arch.B200(), topk=1)[0]
    cache = roller.TuneCache(tmp_path / "tune.json")
    assert cache.get(cfg, 3) is None
    cache.put(cfg, 3, hint, 0.123)
    again = roller.TuneCache(tmp_path / "tune.json")
    assert again.get(cfg, 3) == (hint.block_tile[0], hint.block_tile[1], hint.cta_group, 0.123)
    assert again.get(cfg, 1) is None and again.get(MatmulConfig(1, 2, 3, 32), 3) is None
    (tmp_path / "broken.json").write_text("{not json")
    assert roller.TuneCache(tmp_path / "broken.json").table == {}


def test_estimate_counts_the_cut_along_k_of_leftover_tiles():
    """The library deals leftover tiles out along K when that pays (in units of 8 k-blocks for
    the modes that do not drain often); the estimate follows the same rule, so an under-filled
    grid with a long reduction is not charged a whole wave."""
    dev = arch.B200()
    def top(M, N, K, bits, mode):
        return get_roller_hints(MatmulConfig(M, N, K, bits), dev, topk=1, mode=mode)[0]
    h = top(4096, 64, 8192, 32, MODE_1XTF32)       # 16 or 32 tiles for 74 / 148 workers
    kb_us = dev.kblock_us[(h.block_tile[0], h.block_tile[1], h.cta_group)][0]
    assert h.est_us < 0.75 * (8192 // 32) * kb_us
    h = top(2048, 2048, 2048, 32, MODE_1XTF32)     # short reduction: whole tiles
    kb_us = dev.kblock_us[(h.block_tile[0], h.block_tile[1], h.cta_group)][0]
    assert h.est_us >= (2048 // 32) * kb_us
    # a ragged last wave of a long reduction: 256 tiles on 74 CTA pairs
    h = top(4096, 4096, 8192, 32, MODE_1XTF32)
    assert (h.block_tile, h.cta_group) == ([256, 256], 2)
    assert h.est_us < 3.8 * (8192 // 32) * dev.kblock_us[(256, 256, 2)][0]
