"""GPU parity: gather-GEMM-scatter GEMM (GemmParams with a_inds / c_inds, and the a_inds /
b_inds weight-gradient form) through the operator surface / C ABI, against the CPU oracle."""
import numpy as np
import pytest

import helpers as H
from cumm_b200 import workloads as W
from cumm_b200.gemm.main import GemmMainUnitTest
from cumm_b200.tensorview.gemm import Activation, GemmParams, ShuffleStrideType

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def torch(cuda_lib):
    import torch
    return torch


def test_dense_gemm_simulator_sized(torch, oracle):
    """A [128x64] @ B [64x128], both row-major, seed 0, uniform[-1,1): the case the
    reference runs through its CPU simulator."""
    rng = np.random.default_rng(0)
    a = rng.uniform(-1, 1, (128, 64)).astype(np.float32).astype(np.float16)
    b = rng.uniform(-1, 1, (64, 128)).astype(np.float32).astype(np.float16)
    p = GemmParams()
    p.algo_desp = H.gemm_desp(ShuffleStrideType.NoShuffle, trans_b=False, n=128, k=64)
    p.a, p.b = H.dev(a, torch), H.dev(b, torch)
    c = torch.zeros((128, 128), dtype=torch.float16, device="cuda")
    p.c = c
    GemmMainUnitTest.matmul2(p)
    torch.cuda.synchronize()
    H.check_status()
    H.assert_close_f16(c.cpu().numpy(), oracle.np_dense_gemm_tiled(a, b), "dense GEMM")


@pytest.mark.parametrize("m,k,n,trans_b", [(1, 64, 64, True), (128, 64, 64, True), (129, 64, 64, False),
                                            (5000, 64, 64, True), (5000, 128, 128, False), (3000, 32, 96, True),
                                            (3000, 256, 64, True), (2000, 24, 40, False), (64000, 128, 128, True)])
def test_shuffle_ac(torch, oracle, m, k, n, trans_b):
    rng = np.random.default_rng(m + k)
    rows_a, rows_c = m + 500, m + 300
    a = rng.uniform(-1, 1, (rows_a, k)).astype(np.float16)
    b = rng.uniform(-1, 1, (n, k) if trans_b else (k, n)).astype(np.float16)
    ai = rng.permutation(rows_a)[:m].astype(np.int32)
    ci = rng.permutation(rows_c)[:m].astype(np.int32)
    c0 = rng.uniform(-1, 1, (rows_c, n)).astype(np.float16)
    p = GemmParams()
    p.algo_desp = H.gemm_desp(ShuffleStrideType.ShuffleAC, trans_b=trans_b, n=n, k=k)
    p.a, p.b = H.dev(a, torch), H.dev(b, torch)
    c = H.dev(c0, torch)
    p.c = c
    p.a_inds, p.c_inds = H.dev(ai, torch), H.dev(ci, torch)
    GemmMainUnitTest.matmul2(p)
    torch.cuda.synchronize()
    H.check_status()
    got = c.cpu().numpy()
    want = oracle.gemm_shuffle_ac(a, b, c0.copy(), ai, ci, trans_b=trans_b)
    H.assert_close_f16(got, want, "ShuffleAC")
    untouched = np.setdiff1d(np.arange(rows_c), ci)
    assert (got[untouched] == c0[untouched]).all(), "rows outside c_inds must not be written"


def test_shuffle_ac_beta_bias_act(torch, oracle):
    rng = np.random.default_rng(17)
    m, k, n = 2000, 64, 128
    a = rng.uniform(-1, 1, (2500, k)).astype(np.float16)
    b = rng.uniform(-1, 1, (n, k)).astype(np.float16)
    ai = rng.permutation(2500)[:m].astype(np.int32)
    ci = rng.permutation(2200)[:m].astype(np.int32)
    c0 = rng.uniform(-1, 1, (2200, n)).astype(np.float16)
    for d, beta, act in ((None, 1.0, Activation.None_), ("bias", 1.0, Activation.ReLU), ("rows", 0.5, Activation.LeakyReLU)):
        p = GemmParams()
        p.algo_desp = H.gemm_desp(ShuffleStrideType.ShuffleAC, n=n, k=k)
        p.a, p.b = H.dev(a, torch), H.dev(b, torch)
        c = H.dev(c0, torch)
        p.c = c
        p.a_inds, p.c_inds = H.dev(ai, torch), H.dev(ci, torch)
        p.beta, p.alpha, p.act_type, p.act_alpha = beta, 0.75, act, 0.2
        dn = None
        if d == "bias":
            dn = rng.uniform(-1, 1, n).astype(np.float16)
        elif d == "rows":
            dn = rng.uniform(-1, 1, (2200, n)).astype(np.float16)
        if dn is not None:
            p.d = H.dev(dn, torch)
        GemmMainUnitTest.matmul2(p)
        torch.cuda.synchronize()
        H.check_status()
        want = oracle.gemm_shuffle_ac(a, b, c0.copy(), ai, ci, d=dn, alpha=0.75, beta=beta, act_type=int(act),
                                      act_alpha=0.2)
        H.assert_close_f16(c.cpu().numpy(), want, f"ShuffleAC d={d}")


def test_native_sparse_conv_as_27_gemm_calls(torch, oracle):
    """Gather-GEMM-scatter submanifold conv: one GemmParams call per filter offset on a
    strided slice of the [K, kv, C] weight, accumulating with beta = 1."""
    grid = (8, 24, 24)
    coords = W.sample_coords(3000, 77, grid)
    tb = W.build_tables(coords, grid=grid)
    rng = np.random.default_rng(78)
    C = K = 64
    x = rng.standard_normal((tb.n_in, C)).astype(np.float16)
    w = (rng.standard_normal((K, 27, C)) / np.sqrt(27 * C) * 4).astype(np.float16)
    xd, wd = H.dev(x, torch), H.dev(w, torch)
    out = torch.zeros((tb.n_out, K), dtype=torch.float16, device="cuda")
    want = np.zeros((tb.n_out, K), np.float16)  # same call sequence on the oracle: fp16 round trip per offset
    for f, (i_idx, o_idx) in enumerate(oracle.np_pairs(tb.indices)):
        if len(o_idx) == 0:
            continue
        oracle.gemm_shuffle_ac(x, np.ascontiguousarray(w[:, f, :]), want, i_idx.astype(np.int32),
                               o_idx.astype(np.int32), beta=1.0)
        p = GemmParams()
        p.algo_desp = H.gemm_desp(ShuffleStrideType.ShuffleAC, trans_b=True, n=K, k=C)
        p.a = xd
        p.b = wd[:, f, :]  # [K, C] view with row stride kv*C
        p.c = out
        p.a_inds, p.c_inds = H.dev(i_idx.astype(np.int32), torch), H.dev(o_idx.astype(np.int32), torch)
        p.beta = 1.0
        GemmMainUnitTest.matmul2(p)
    torch.cuda.synchronize()
    H.check_status()
    H.assert_close_f16(out.cpu().numpy(), want, "27-call native conv")
    # and close to the single-rounding result (looser: up to 27 fp16 roundings per element)
    np.testing.assert_allclose(out.cpu().numpy().astype(np.float32), oracle.np_forward(x, w, tb.indices),
                               rtol=3e-2, atol=3e-2)


@pytest.mark.parametrize("kk,m,n", [(1, 64, 64), (200, 64, 64), (5000, 64, 64), (5000, 128, 128), (3000, 128, 64),
                                     (3000, 24, 40), (64000, 128, 128)])
def test_shuffle_ab(torch, oracle, kk, m, n):
    rng = np.random.default_rng(kk + m)
    rows = kk + 700
    a = rng.uniform(-1, 1, (rows, m)).astype(np.float16)
    b = rng.uniform(-1, 1, (rows, n)).astype(np.float16)
    ai = rng.permutation(rows)[:kk].astype(np.int32)
    bi = rng.permutation(rows)[:kk].astype(np.int32)
    p = GemmParams()
    p.algo_desp = H.gemm_desp(ShuffleStrideType.ShuffleAB, trans_a=True, trans_b=False, n=n)
    p.a, p.b = H.dev(a, torch), H.dev(b, torch)
    c = torch.zeros((m, n), dtype=torch.float16, device="cuda")
    p.c = c
    p.a_inds, p.b_inds = H.dev(ai, torch), H.dev(bi, torch)
    p.split_k_slices = 8
    GemmMainUnitTest.matmul2(p)
    torch.cuda.synchronize()
    H.check_status()
    want = oracle.gemm_shuffle_ab(a, b, np.zeros((m, n), np.float16), ai, bi)
    s = max(1.0, float(np.sqrt(kk)) / 4)
    H.assert_close_f16(c.cpu().numpy() / s, want.astype(np.float32) / s, "ShuffleAB")


def test_out_of_range_row_index_sets_status_not_fault(torch):
    """An index beyond the operand's rows is never dereferenced; the status word reports it."""
    from cumm_b200 import _lib
    rng = np.random.default_rng(1)
    a = rng.uniform(-1, 1, (100, 64)).astype(np.float16)
    b = rng.uniform(-1, 1, (64, 64)).astype(np.float16)
    ai = np.arange(50, dtype=np.int32)
    ai[7] = 100000
    p = GemmParams()
    p.algo_desp = H.gemm_desp(ShuffleStrideType.ShuffleAC, n=64, k=64)
    p.a, p.b = H.dev(a, torch), H.dev(b, torch)
    p.c = torch.zeros((50, 64), dtype=torch.float16, device="cuda")
    p.a_inds, p.c_inds = H.dev(ai, torch), H.dev(np.arange(50, dtype=np.int32), torch)
    GemmMainUnitTest.matmul2(p)
    assert _lib.device_status() == 2
    assert _lib.device_status() == 0
    assert (p.c[7] == 0).all()


@pytest.mark.parametrize("tile_n,tile_k", [(64, 64), (64, 128), (128, 64), (128, 128)])
def test_shuffle_ac_every_tile_shape(torch, oracle, tile_n, tile_k):
    """The descriptor's tile shape selects the kernel variant; all of them compute the same thing."""
    rng = np.random.default_rng(5)
    m, k, n = 3000, 128, 128
    a = rng.uniform(-1, 1, (m + 100, k)).astype(np.float16)
    b = rng.uniform(-1, 1, (n, k)).astype(np.float16)
    ai = rng.permutation(m + 100)[:m].astype(np.int32)
    ci = rng.permutation(m)[:m].astype(np.int32)
    p = GemmParams()
    p.algo_desp = H.gemm_desp(ShuffleStrideType.ShuffleAC)
    p.algo_desp.tile_shape = [128, tile_n, tile_k]
    p.algo_desp.warp_tile_shape = [128, tile_n, tile_k]
    p.a, p.b = H.dev(a, torch), H.dev(b, torch)
    c = torch.zeros((m, n), dtype=torch.float16, device="cuda")
    p.c = c
    p.a_inds, p.c_inds = H.dev(ai, torch), H.dev(ci, torch)
    GemmMainUnitTest.matmul2(p)
    torch.cuda.synchronize()
    H.check_status()
    want = oracle.gemm_shuffle_ac(a, b, np.zeros((m, n), np.float16), ai, ci)
    H.assert_close_f16(c.cpu().numpy(), want, f"ShuffleAC tile {tile_n}x{tile_k}")


def test_unknown_tile_shape_is_refused(torch):
    p = GemmParams()
    p.algo_desp = H.gemm_desp(ShuffleStrideType.ShuffleAC)
    p.algo_desp.tile_shape = [128, 96, 64]
    p.algo_desp.warp_tile_shape = [128, 96, 64]
    p.a = torch.zeros((10, 64), dtype=torch.float16, device="cuda")
    p.b = torch.zeros((64, 64), dtype=torch.float16, device="cuda")
    p.c = torch.zeros((10, 64), dtype=torch.float16, device="cuda")
    p.a_inds = p.c_inds = torch.arange(10, dtype=torch.int32, device="cuda")
    with pytest.raises(RuntimeError, match="can't find any suitable algo"):
        GemmMainUnitTest.matmul2(p)


def _layer_as_calls(torch, tb, x, w, out):
    """The GemmParams of a native sparse convolution: one ShuffleAC call per filter offset with pairs."""
    xd, wd = H.dev(x, torch), H.dev(w, torch)
    K, C = w.shape[0], w.shape[2]
    calls = []
    for f in range(tb.kv):
        o_idx = np.nonzero(tb.indices[f] >= 0)[0].astype(np.int32)
        if len(o_idx) == 0:
            continue
        p = GemmParams()
        p.algo_desp = H.gemm_desp(ShuffleStrideType.ShuffleAC, trans_b=True, n=K, k=C)
        p.a, p.b, p.c = xd, wd[:, f, :], out
        p.a_inds, p.c_inds = H.dev(tb.indices[f][o_idx], torch), H.dev(o_idx, torch)
        p.beta = 1.0
        calls.append(p)
    return calls


@pytest.mark.parametrize("n,C,K", [(3000, 64, 64), (2000, 128, 128), (600, 32, 64)])
def test_layer_sequence_in_one_launch(torch, oracle, n, C, K):
    """cb2_gemm_sequence_run: the calls of one layer as one launch, accumulating onto what the
    output held; fp32 sums over all offsets rounded once (the call-by-call run rounds 27 times)."""
    from cumm_b200.sequence import prepare_gemm_sequence
    grid = (8, 24, 24)
    tb = W.build_tables(W.sample_coords(n, 80 + n, grid), grid=grid)
    rng = np.random.default_rng(81 + n)
    x = rng.standard_normal((tb.n_in, C)).astype(np.float16)
    w = (rng.standard_normal((K, 27, C)) / np.sqrt(27 * C) * 4).astype(np.float16)
    init = rng.standard_normal((tb.n_out, K)).astype(np.float16)
    out = H.dev(init, torch)
    seq = prepare_gemm_sequence(_layer_as_calls(torch, tb, x, w, out))
    seq.launch()
    torch.cuda.synchronize()
    H.check_status()
    want = oracle.np_forward(x, w, tb.indices) + init.astype(np.float32)
    H.assert_close_f16(out.cpu().numpy(), want, "sequence, first launch")
    # a second launch reuses the tables and accumulates once more
    seq.launch()
    torch.cuda.synchronize()
    H.check_status()
    want2 = oracle.np_forward(x, w, tb.indices) + want.astype(np.float16).astype(np.float32)
    H.assert_close_f16(out.cpu().numpy(), want2, "sequence, second launch (tables reused)")
    # and the call-by-call run agrees to a few fp16 ulps
    out_c = H.dev(init, torch)
    for p in _layer_as_calls(torch, tb, x, w, out_c):
        GemmMainUnitTest.matmul2(p)
    torch.cuda.synchronize()
    out1 = H.dev(init, torch)
    prepare_gemm_sequence(_layer_as_calls(torch, tb, x, w, out1)).launch()
    torch.cuda.synchronize()
    np.testing.assert_allclose(out1.cpu().numpy().astype(np.float32), out_c.cpu().numpy().astype(np.float32),
                               rtol=2e-2, atol=2e-2)


def test_layer_sequence_refuses_calls_that_are_not_one_layer(torch):
    from cumm_b200.sequence import prepare_gemm_sequence
    grid = (8, 24, 24)
    tb = W.build_tables(W.sample_coords(500, 90, grid), grid=grid)
    x = np.zeros((tb.n_in, 64), np.float16)
    w = np.zeros((64, 27, 64), np.float16)
    out = torch.zeros((tb.n_out, 64), dtype=torch.float16, device="cuda")
    calls = _layer_as_calls(torch, tb, x, w, out)
    calls[3].beta = 0.0  # would overwrite instead of accumulate
    with pytest.raises(RuntimeError, match="does not fit the layer form"):
        prepare_gemm_sequence(calls).launch()
    calls = _layer_as_calls(torch, tb, x, w, out)
    calls[2].a = torch.zeros((tb.n_in, 64), dtype=torch.float16, device="cuda")  # another A
    with pytest.raises(RuntimeError, match="does not fit the layer form"):
        prepare_gemm_sequence(calls).launch()
    assert (out == 0).all()
