"""Host-side tile choices of the GEMM wrappers (pure arithmetic, no GPU)."""
from dlslime_b200.ops import gemm


def test_wide_tiles_are_picked_where_512_wide_columns_fill_the_grid():
    assert gemm._wide_tiles_pay(8192, 8192)          # 32 x 16 = 512 tiles: 6.9 waves of 74 pairs
    assert gemm._wide_tiles_pay(4096, 4096)          # 2 waves either way: the wide tiles move fewer bytes
    assert not gemm._wide_tiles_pay(8192, 3584)      # 7 columns of 512 leave a quarter of the last wave empty; 16 x 224 fits
    assert not gemm._wide_tiles_pay(1000, 4096)      # 4 x 8 tiles do not fill 74 pairs; 256-wide tiles use twice as many


def test_grouped_tile_width_minimises_waves_and_prefers_the_wide_tile_on_ties():
    # many row tiles: the wave count hardly depends on the width, the widest tile wins
    assert gemm.pick_grouped_tile_n(288, 2048, swiglu=True) == 256
    assert gemm.pick_grouped_tile_n(288, 7168) == 256
    # 32 row tiles: 28 columns of 256 are 6.05 waves of 148 CTAs, 32 columns of 224 are 6.9
    assert gemm.pick_grouped_tile_n(32, 7168) == 224
    assert gemm.pick_grouped_tile_n(32, 2048, swiglu=True) == 128
    assert gemm.pick_grouped_tile_n(0, 256) in (256, 224, 192, 128)
