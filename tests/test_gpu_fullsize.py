"""GPU parity at the benchmark sizes (150 000 voxels): against the numpy statement of the
operators (the reference's own check loop, BLAS-backed so it finishes in seconds), and
through size-independent properties (linearity in the input, row-permutation invariance)."""
import numpy as np
import pytest

import helpers as H
from cumm_b200 import workloads as W

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def torch(cuda_lib):
    import torch
    return torch


@pytest.fixture(scope="module")
def scene():
    coords = W.sample_coords(150000, 1)
    return coords, W.build_tables(coords)


def test_mask_igemm_fp16_all_three_ops(torch, oracle, scene):
    _, tb = scene
    rng = np.random.default_rng(2)
    C = K = 128
    x = rng.standard_normal((tb.n_in, C)).astype(np.float16)
    dout = rng.standard_normal((tb.n_out, K)).astype(np.float16)
    w = (rng.standard_normal((27, C, K)) / np.sqrt(27 * C)).astype(np.float16).transpose(2, 0, 1).copy()
    out, mo = H.run_conv_fwd(torch, x, w, tb)
    H.assert_close_f16(out, oracle.np_forward(x, w, tb.indices), "forward")
    din = H.run_conv_dgrad(torch, dout, w, tb, use_reverse=True)
    H.assert_close_f16(din, oracle.np_dgrad(dout, w, tb.indices, tb.n_in), "dgrad")
    dw = H.run_conv_wgrad(torch, dout, x, tb, mo, fp32_out=True)
    want = oracle.np_wgrad(dout, x, tb.indices)
    H.assert_close_wgrad(dw, want, tb.indices, "wgrad (fp32 out)", kv_axis=1)
    H.check_status()
    # linearity: conv(2x) == 2 conv(x) exactly in fp16 (power-of-two scaling)
    out2, _ = H.run_conv_fwd(torch, (x * np.float16(2)).astype(np.float16), w, tb)
    normal = np.abs(out.astype(np.float32)) >= 2.0 ** -13  # fp16 subnormals do not scale exactly
    assert (out2.astype(np.float32)[normal] == 2 * out.astype(np.float32)[normal]).all()


def test_int8_stride2_bit_exact(torch, oracle, scene):
    coords, _ = scene
    tb = W.build_tables(coords, stride=(2, 2, 2), subm=False)
    assert tb.n_out == 491092
    rng = np.random.default_rng(3)
    C = K = 128
    x = rng.integers(-127, 128, (tb.n_in, C)).astype(np.int8)
    w = rng.integers(-127, 128, (K, 27, C)).astype(np.int8)
    scale = rng.uniform(1e-3, 1e-2, K).astype(np.float32)
    bias = rng.standard_normal(K).astype(np.float32)
    got = H.run_conv_s8(torch, x, w, scale, bias, tb)
    H.check_status()
    acc = oracle.np_forward_s8_acc(x, w, tb.indices)
    want = oracle.requant_s8(acc, scale, bias)
    assert (got == want).all(), f"{int((got != want).sum())} of {got.size} differ"


def test_eight_scene_batch_all_three_ops(torch, oracle):
    """The benchmark's own batch on one GPU: 8 scenes x 120 000 voxels with batch indices 0..7,
    tables built on the GPU, forward / input gradient / weight gradient over all 960 000 rows in
    one launch each -- compared scene by scene with the numpy statement on host-built tables."""
    from cumm_b200.layer import SparseConvLayer
    from cumm_b200.pairgen import build_tables_gpu
    n_scenes, per = 8, 120000
    coords = [W.sample_coords(per, [4, b], batch=b) for b in range(n_scenes)]
    tg = build_tables_gpu(torch.from_numpy(np.concatenate(coords)).cuda(), n_scenes, W.GRID)
    rng = np.random.default_rng([4, 100])
    C = K = 128
    x = rng.standard_normal((tg.n_in, C), dtype=np.float32).astype(np.float16)
    dout = rng.standard_normal((tg.n_out, K), dtype=np.float32).astype(np.float16)
    w = (rng.standard_normal((27, C, K), dtype=np.float32) / np.sqrt(27 * C)).astype(np.float16).transpose(2, 0, 1).copy()
    xd, dd, wd = H.dev(x, torch), H.dev(dout, torch), H.dev(w, torch)
    out = torch.zeros((tg.n_out, K), dtype=torch.float16, device="cuda")
    din = torch.zeros((tg.n_in, C), dtype=torch.float16, device="cuda")
    dw = torch.zeros((K, 27, C), dtype=torch.float32, device="cuda")
    layer = SparseConvLayer(tg, wd, xd, out, dd, din, dw)
    layer.fwd.launch()
    layer.dgrad.launch()
    layer.wgrad.launch()
    torch.cuda.synchronize()
    H.check_status()
    out, din, dw = out.cpu().numpy(), din.cpu().numpy(), dw.cpu().numpy()
    idx_g = tg.indices.cpu().numpy()
    want_dw = np.zeros((K, 27, C), np.float32)
    for b in range(n_scenes):
        tb = W.build_tables(coords[b])
        rows = slice(b * per, (b + 1) * per)
        blk = idx_g[:, rows]
        assert (np.where(blk >= 0, blk - b * per, -1) == tb.indices).all(), f"scene {b}: GPU-built table differs"
        H.assert_close_f16(out[rows], oracle.np_forward(x[rows], w, tb.indices), f"scene {b} forward")
        H.assert_close_f16(din[rows], oracle.np_dgrad(dout[rows], w, tb.indices, per), f"scene {b} dgrad")
        want_dw += oracle.np_wgrad(dout[rows], x[rows], tb.indices)
    H.assert_close_wgrad(dw, want_dw, idx_g, "eight-scene wgrad (fp32 out)")


def test_native_conv_as_27_gemm_calls_150k(torch, oracle, scene):
    """The gather-GEMM-scatter form of the same layer at C = K = 64 and full size: one ShuffleAC
    call per filter offset accumulating with beta = 1 into a zeroed output, as
    cumm/gemm/main_real.py:196-232 / cumm/conv/main_real_spconv.py:309-403 do."""
    from cumm_b200.gemm.main import GemmMainUnitTest
    from cumm_b200.tensorview.gemm import GemmParams, ShuffleStrideType
    _, tb = scene
    C = K = 64
    rng = np.random.default_rng(1)
    x = rng.standard_normal((tb.n_in, C), dtype=np.float32).astype(np.float16)
    w = (rng.standard_normal((K, 27, C), dtype=np.float32) / np.sqrt(27 * C)).astype(np.float16)
    xd, wd = H.dev(x, torch), H.dev(w, torch)
    out = torch.zeros((tb.n_out, K), dtype=torch.float16, device="cuda")
    for f in range(27):
        o_idx = np.nonzero(tb.indices[f] >= 0)[0].astype(np.int32)
        if len(o_idx) == 0:
            continue
        p = GemmParams()
        p.algo_desp = H.gemm_desp(ShuffleStrideType.ShuffleAC, n=K, k=C)
        p.a, p.b, p.c = xd, wd[:, f, :], out
        p.a_inds, p.c_inds = H.dev(tb.indices[f][o_idx], torch), H.dev(o_idx, torch)
        p.beta = 1.0
        GemmMainUnitTest.matmul2(p)
    torch.cuda.synchronize()
    H.check_status()
    want = oracle.np_forward(x, w, tb.indices)
    # up to 27 fp16 roundings of the running sum instead of one: a few ulps of |want| <= 4
    err = np.abs(out.cpu().numpy().astype(np.float32) - want)
    tol = 2e-2 + 1e-2 * np.abs(want)
    assert (err <= tol).all(), f"{int((err > tol).sum())} entries outside tolerance, max abs err {err.max():.4g}"


def test_layer_sequence_one_launch_150k(torch, oracle, scene):
    """The same layer through cb2_gemm_sequence_run: all 27 calls as one launch."""
    from cumm_b200.sequence import prepare_gemm_sequence
    from cumm_b200.tensorview.gemm import GemmParams, ShuffleStrideType
    _, tb = scene
    C = K = 64
    rng = np.random.default_rng(1)
    x = rng.standard_normal((tb.n_in, C), dtype=np.float32).astype(np.float16)
    w = (rng.standard_normal((K, 27, C), dtype=np.float32) / np.sqrt(27 * C)).astype(np.float16)
    xd, wd = H.dev(x, torch), H.dev(w, torch)
    out = torch.zeros((tb.n_out, K), dtype=torch.float16, device="cuda")
    calls = []
    for f in range(27):
        o_idx = np.nonzero(tb.indices[f] >= 0)[0].astype(np.int32)
        if len(o_idx) == 0:
            continue
        p = GemmParams()
        p.algo_desp = H.gemm_desp(ShuffleStrideType.ShuffleAC, n=K, k=C)
        p.a, p.b, p.c = xd, wd[:, f, :], out
        p.a_inds, p.c_inds = H.dev(tb.indices[f][o_idx], torch), H.dev(o_idx, torch)
        p.beta = 1.0
        calls.append(p)
    assert len(calls) == 27
    prepare_gemm_sequence(calls).launch()
    torch.cuda.synchronize()
    H.check_status()
    H.assert_close_f16(out.cpu().numpy(), oracle.np_forward(x, w, tb.indices), "27 calls in one launch")
