"""Neighbour tables built on the GPU against the host generator, bit for bit."""
import numpy as np
import pytest

import helpers as H
from cumm_b200 import workloads as W

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def torch(cuda_lib):
    import torch
    return torch


def gpu_tables(torch, coords, batch_size, grid, **kw):
    from cumm_b200.pairgen import build_tables_gpu
    t, oc = build_tables_gpu(torch.from_numpy(coords).cuda(), batch_size, grid, return_out_coords=True, **kw)
    torch.cuda.synchronize()
    H.check_status()
    return t, oc


def compare(torch, t, oc, ref, subm):
    def h(x):
        return x.cpu().numpy()
    assert t.n_out == ref.n_out and t.n_in == ref.n_in and t.kv == ref.kv
    if not subm:
        assert (h(oc) == ref.out_coords).all(), "active outputs / their order differ"
    assert (h(t.indices) == ref.indices).all(), "indices differ"
    assert (h(t.mask).view(np.uint32) == ref.mask).all(), "sorted masks differ"
    assert (h(t.mask_argsort) == ref.mask_argsort).all(), "mask_argsort differs (the sort must be stable)"
    assert (h(t.indices_bwd) == ref.indices_bwd).all(), "backward indices differ"
    assert (h(t.mask_bwd).view(np.uint32) == ref.mask_bwd).all(), "backward masks differ"
    assert (h(t.mask_argsort_bwd) == ref.mask_argsort_bwd).all(), "backward mask_argsort differs"
    tiles = (ref.n_out + 127) // 128
    want_mo = np.array([np.bitwise_or.reduce(ref.mask[i * 128:(i + 1) * 128]) for i in range(tiles)], np.uint32)
    assert (h(t.mask_output).view(np.uint32) == want_mo).all(), "per-tile masks differ"


@pytest.mark.parametrize("n", [1, 37, 3000])
def test_submanifold(torch, n):
    grid = (8, 24, 24)
    coords = W.sample_coords(n, 40 + n, grid)
    t, oc = gpu_tables(torch, coords, 1, grid)
    compare(torch, t, oc, W.build_tables(coords, grid=grid), True)


def test_submanifold_several_scenes(torch):
    grid = (8, 24, 24)
    coords = np.concatenate([W.sample_coords(1500 + 100 * b, [7, b], grid, batch=b) for b in range(3)])
    t, oc = gpu_tables(torch, coords, 3, grid)
    ref = W.build_tables(coords, grid=grid)
    compare(torch, t, oc, ref, True)
    # neighbours never cross scenes
    idx = t.indices.cpu().numpy()
    b_of = coords[:, 0]
    for f in range(27):
        o = np.nonzero(idx[f] >= 0)[0]
        assert (b_of[idx[f, o]] == b_of[o]).all()


@pytest.mark.parametrize("stride,pad,dil,ksize", [((2, 2, 2), None, (1, 1, 1), (3, 3, 3)),
                                                  ((2, 2, 2), (0, 0, 0), (1, 1, 1), (3, 3, 3)),
                                                  ((1, 1, 1), (2, 2, 2), (2, 2, 2), (3, 3, 3)),
                                                  ((2, 1, 2), (0, 1, 1), (1, 1, 1), (1, 3, 3)),
                                                  ((3, 3, 3), (1, 1, 1), (1, 1, 1), (2, 2, 2))])
def test_regular_convolution(torch, stride, pad, dil, ksize):
    grid = (9, 25, 23)
    coords = W.sample_coords(2500, 77, grid)
    kw = dict(ksize=ksize, stride=stride, dil=dil, subm=False)
    if pad is not None:
        kw["pad"] = pad
    t, oc = gpu_tables(torch, coords, 1, grid, **kw)
    compare(torch, t, oc, W.build_tables(coords, grid=grid, **kw), False)


@pytest.mark.parametrize("ksize,subm,stride", [((3, 3, 5), True, (1, 1, 1)), ((5, 5, 5), True, (1, 1, 1)),
                                               ((4, 4, 4), False, (2, 2, 2)), ((2, 4, 5), False, (1, 2, 1))])
def test_kernel_volumes_above_32(torch, ksize, subm, stride):
    """Several mask words per row (45, 125, 64 and 40 offsets): masks [n, words], sorted as one
    integer whose last word is the most significant, stable; per-tile masks per word."""
    grid = (10, 26, 22)
    coords = W.sample_coords(4000, 91, grid)
    kw = dict(ksize=ksize, stride=stride, subm=subm)
    t, oc = gpu_tables(torch, coords, 1, grid, **kw)
    ref = W.build_tables(coords, grid=grid, **kw)
    assert ref.mask.ndim == 2 and ref.mask.shape[1] == (t.kv + 31) // 32
    compare(torch, t, oc, ref, subm)


def test_benchmark_scene_full_size(torch):
    """The 150 000-voxel scene of the benchmark configurations, submanifold and stride 2."""
    coords = W.sample_coords(150000, 1)
    t, oc = gpu_tables(torch, coords, 1, W.GRID)
    compare(torch, t, oc, W.build_tables(coords), True)
    t2, oc2 = gpu_tables(torch, coords, 1, W.GRID, stride=(2, 2, 2), subm=False)
    ref2 = W.build_tables(coords, stride=(2, 2, 2), subm=False)
    assert ref2.n_out == 491092
    compare(torch, t2, oc2, ref2, False)


def test_coordinate_outside_the_grid_is_reported(torch):
    from cumm_b200 import _lib
    from cumm_b200.pairgen import build_tables_gpu
    grid = (8, 24, 24)
    coords = W.sample_coords(500, 3, grid)
    coords[17, 2] = 24  # y outside
    build_tables_gpu(torch.from_numpy(coords).cuda(), 1, grid)
    assert _lib.device_status() == 4
    assert _lib.device_status() == 0


def test_tables_feed_the_convolution(torch, oracle):
    """End to end: tables from the GPU builder drive the forward kernel."""
    from cumm_b200.conv.main import ConvMainUnitTest
    from cumm_b200.tensorview.gemm import ConvOpType, ConvParams
    grid = (8, 24, 24)
    coords = W.sample_coords(3000, 91, grid)
    t, _ = gpu_tables(torch, coords, 1, grid)
    ref = W.build_tables(coords, grid=grid)
    rng = np.random.default_rng(92)
    x = rng.standard_normal((ref.n_in, 64)).astype(np.float16)
    w = (rng.standard_normal((64, 27, 64)) / np.sqrt(27 * 64) * 4).astype(np.float16)
    p = ConvParams(3, ConvOpType.Forward)
    p.conv_algo_desp = H.conv_desp(ConvOpType.Forward, 64, 64)
    p.input, p.weight = H.dev(x, torch), H.dev(w, torch)
    out = torch.zeros((t.n_out, 64), dtype=torch.float16, device="cuda")
    p.output = out
    p.indices, p.mask, p.mask_argsort = t.indices, t.mask, t.mask_argsort
    ConvMainUnitTest.implicit_gemm2(p)
    torch.cuda.synchronize()
    H.check_status()
    want = oracle.mask_igemm(x, w, np.zeros((ref.n_out, 64), np.float16), ref.indices, ref.mask, ref.mask_argsort)
    H.assert_close_f16(out.cpu().numpy(), want, "forward on GPU-built tables")


def test_wide_tables_feed_the_convolution(torch, oracle):
    """Tables of a 3x3x5 kernel (45 offsets, two mask words per row) from the GPU builder drive the
    forward kernel and, through the backward tables, the input gradient."""
    from cumm_b200.conv.main import ConvMainUnitTest
    from cumm_b200.tensorview.gemm import ConvOpType, ConvParams
    grid, ksize, C, K = (8, 24, 24), (3, 3, 5), 64, 64
    kv = 45
    coords = W.sample_coords(3000, 93, grid)
    t, _ = gpu_tables(torch, coords, 1, grid, ksize=ksize)
    ref = W.build_tables(coords, grid=grid, ksize=ksize)
    rng = np.random.default_rng(94)
    x = rng.standard_normal((ref.n_in, C)).astype(np.float16)
    dout = rng.standard_normal((ref.n_out, K)).astype(np.float16)
    w = (rng.standard_normal((K, kv, C)) / np.sqrt(kv * C) * 4).astype(np.float16)
    for op, src, tabs, rtabs in ((ConvOpType.Forward, x, (t.indices, t.mask, t.mask_argsort),
                                  (ref.indices, ref.mask, ref.mask_argsort)),
                                 (ConvOpType.BackwardInput, dout, (t.indices_bwd, t.mask_bwd, t.mask_argsort_bwd),
                                  (ref.indices_bwd, ref.mask_bwd, ref.mask_argsort_bwd))):
        p = ConvParams(3, op)
        p.conv_algo_desp = H.conv_desp(op, C, K)
        p.conv_algo_desp.dynamic_mask = True
        out = torch.zeros((ref.n_out, K) if op == ConvOpType.Forward else (ref.n_in, C), dtype=torch.float16, device="cuda")
        if op == ConvOpType.Forward:
            p.input, p.output = H.dev(src, torch), out
        else:
            p.input, p.output = out, H.dev(src, torch)
        p.weight = H.dev(w, torch)
        p.indices, p.mask, p.mask_argsort = tabs
        ConvMainUnitTest.implicit_gemm2(p)
        torch.cuda.synchronize()
        H.check_status()
        if op == ConvOpType.Forward:
            want = oracle.mask_igemm(src, w, np.zeros((ref.n_out, K), np.float16), *rtabs)
        else:
            want = oracle.mask_igemm(src, w, np.zeros((ref.n_in, C), np.float16), *rtabs, is_dgrad=True)
        H.assert_close_f16(out.cpu().numpy(), want, f"{op.name} on GPU-built two-word tables")
