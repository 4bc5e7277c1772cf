"""The synthetic workload generator against the oracle's independent pair builder, and the
pair counts of the benchmark configurations."""
import numpy as np
import pytest

from cumm_b200 import workloads as W


def test_subm_tables_match_oracle(oracle):
    grid = (9, 30, 28)
    coords = W.sample_coords(4000, 21, grid)
    tb = W.build_tables(coords, grid=grid)
    idx, mask = oracle.build_pairs(coords, coords, grid, (3, 3, 3), (1, 1, 1), (1, 1, 1), (1, 1, 1))
    assert (idx == tb.indices).all()
    smask, order = oracle.sort_masks(mask)
    assert (smask == tb.mask).all() and (order == tb.mask_argsort).all()
    assert (oracle.backward_indices(idx, len(coords)) == tb.indices_bwd).all()
    # submanifold symmetry: backward table = forward table with the filter order reversed
    assert (tb.indices_bwd == tb.indices[::-1]).all()
    assert (tb.indices[13] == np.arange(len(coords))).all()
    # stable sort: ties keep the original order
    same = tb.mask[1:] == tb.mask[:-1]
    assert (np.diff(tb.mask_argsort)[same] > 0).all()


def test_regular_stride2_tables_match_oracle(oracle):
    grid = (9, 30, 28)
    coords = W.sample_coords(3000, 22, grid)
    tb = W.build_tables(coords, grid=grid, stride=(2, 2, 2), subm=False)
    oc, og = oracle.regular_out_coords(coords, grid, (3, 3, 3), (2, 2, 2), (1, 1, 1), (1, 1, 1))
    assert og == [5, 15, 14]
    assert (oc == tb.out_coords).all()
    idx, mask = oracle.build_pairs(coords, oc, grid, (3, 3, 3), (2, 2, 2), (1, 1, 1), (1, 1, 1))
    assert (idx == tb.indices).all()
    assert (np.sort(mask, kind="stable") == tb.mask).all()
    # every input voxel appears exactly once per filter offset it can reach, and every pair inverts
    for f in range(27):
        o = np.nonzero(idx[f] >= 0)[0]
        assert (tb.indices_bwd[f, idx[f, o]] == o).all()
    assert tb.num_pairs == int((idx >= 0).sum()) == int((tb.indices_bwd >= 0).sum())


def test_benchmark_configuration_counts():
    """Pair counts of the benchmark voxel sets (seeded, so these are fixed numbers)."""
    coords = W.sample_coords(150000, 1)
    tb = W.build_tables(coords)
    assert tb.n_out == 150000 and tb.num_pairs == 156250
    tiles = (tb.n_out + 127) // 128
    steps = sum(bin(int(np.bitwise_or.reduce(tb.mask[t * 128:(t + 1) * 128]))).count("1") for t in range(tiles))
    assert tiles == 1172 and steps == 1350
    tb3 = W.build_tables(coords, stride=(2, 2, 2), subm=False)
    assert tb3.n_out == 491092 and tb3.num_pairs == 501289


def test_concat_scenes_renumbers_rows():
    grid = (6, 12, 12)
    scenes = [W.build_tables(W.sample_coords(300, [4, b], grid, batch=b), grid=grid) for b in range(3)]
    cat = W.concat_scenes(scenes)
    assert cat.n_out == 900 and cat.num_pairs == sum(s.num_pairs for s in scenes)
    for b, s in enumerate(scenes):
        blk = cat.indices[:, b * 300:(b + 1) * 300]
        assert ((blk >= 0) == (s.indices >= 0)).all()
        assert (blk[blk >= 0] == s.indices[s.indices >= 0] + b * 300).all()
    assert (cat.mask[1:] >= cat.mask[:-1]).all()


def test_dense_block_has_full_neighbourhoods():
    coords = W.dense_block_coords(6)
    tb = W.build_tables(coords, grid=(6, 6, 6))
    inner = ((coords[:, 1:] > 0) & (coords[:, 1:] < 5)).all(1)
    assert ((tb.indices[:, inner] >= 0).all())
