"""GPU parity: mask-based implicit-GEMM sparse convolution (forward, input gradient, weight
gradient, int8 inference) through the operator surface / C ABI, against the CPU oracle.
fp16 results within rtol 1e-2 / atol 1e-2 of the fp32-accumulated oracle; masks and int8
outputs bit-exact."""
import numpy as np
import pytest

import helpers as H
from cumm_b200 import workloads as W
from cumm_b200.tensorview.gemm import Activation, ConvOpType, ConvParams
from cumm_b200.conv.main import ConvMainUnitTest

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def torch(cuda_lib):
    import torch
    return torch


def make(n, seed, C, K, grid=(8, 24, 24), **kw):
    tb, coords = H.random_tables(n, seed, grid, **kw)
    rng = np.random.default_rng(seed + 1000)
    x = rng.standard_normal((tb.n_in, C)).astype(np.float16)
    w = (rng.standard_normal((K, tb.kv, C)) / np.sqrt(tb.kv * C) * 4).astype(np.float16)
    dout = rng.standard_normal((tb.n_out, K)).astype(np.float16)
    return tb, x, w, dout


@pytest.mark.parametrize("n,C,K", [(1, 64, 64), (127, 64, 64), (128, 128, 128), (129, 128, 128), (3000, 128, 128),
                                    (3000, 64, 64), (2500, 32, 64), (2500, 64, 128), (2500, 128, 64),
                                    (2000, 24, 40), (2000, 16, 16), (1500, 256, 256), (1500, 192, 136)])
def test_forward(torch, oracle, n, C, K):
    tb, x, w, _ = make(n, 100 + n + C, C, K)
    got, mo = H.run_conv_fwd(torch, x, w, tb)
    H.check_status()
    mo_ref = np.zeros_like(mo)
    want = oracle.mask_igemm(x, w, np.zeros((tb.n_out, K), np.float16), tb.indices, tb.mask, tb.mask_argsort,
                             mask_out=mo_ref)
    assert (mo == mo_ref).all(), "tile masks must be bit-exact"
    H.assert_close_f16(got, want, f"forward n={n} C={C} K={K}")


def test_forward_dense_neighbourhoods(torch, oracle):
    """Solid block: every tile carries all 27 offsets (the contraction-heavy regime)."""
    coords = W.dense_block_coords(12)
    tb = W.build_tables(coords, grid=(12, 12, 12))
    rng = np.random.default_rng(3)
    x = rng.standard_normal((tb.n_in, 64)).astype(np.float16)
    w = (rng.standard_normal((128, 27, 64)) / 16).astype(np.float16)
    got, _ = H.run_conv_fwd(torch, x, w, tb)
    H.check_status()
    want = oracle.mask_igemm(x, w, np.zeros((tb.n_out, 128), np.float16), tb.indices, tb.mask, tb.mask_argsort)
    H.assert_close_f16(got, want, "dense block forward")


def test_forward_regular_stride2(torch, oracle):
    tb, x, w, _ = make(2500, 31, 64, 64, stride=(2, 2, 2), subm=False)
    got, _ = H.run_conv_fwd(torch, x, w, tb)
    H.check_status()
    want = oracle.mask_igemm(x, w, np.zeros((tb.n_out, 64), np.float16), tb.indices, tb.mask, tb.mask_argsort)
    H.assert_close_f16(got, want, "stride-2 forward")


@pytest.mark.parametrize("act,act_alpha", [(Activation.ReLU, 0.0), (Activation.LeakyReLU, 0.1),
                                            (Activation.Sigmoid, 0.0)])
def test_forward_bias_activation(torch, oracle, act, act_alpha):
    tb, x, w, _ = make(1200, 41, 64, 128)
    bias = np.random.default_rng(1).standard_normal(128).astype(np.float16)
    got, _ = H.run_conv_fwd(torch, x, w, tb, bias=bias, beta=1.0, alpha=0.5, act=act, act_alpha=act_alpha)
    H.check_status()
    want = oracle.mask_igemm(x, w, np.zeros((tb.n_out, 128), np.float16), tb.indices, tb.mask, tb.mask_argsort,
                             d=bias, alpha=0.5, beta=1.0, act_type=int(act), act_alpha=act_alpha)
    H.assert_close_f16(got, want, f"bias+{act.name}")


def test_forward_mask_split_two_passes(torch, oracle):
    """The reference harness runs two launches, each with half of the filter offsets, the
    second accumulating with beta = 1 (cumm/conv/main_real_spconv.py:273-294)."""
    tb, x, w, _ = make(2000, 51, 128, 128)
    f1, f2 = 0b11111111111111, 0b1111111111111 << 14
    out1, mo1 = H.run_conv_fwd(torch, x, w, tb, mask_filter=f1)
    out2, mo2 = H.run_conv_fwd(torch, x, w, tb, mask_filter=f2, out_init=out1, beta=1.0)
    H.check_status()
    ref = np.zeros((tb.n_out, 128), np.float16)
    r1, r2 = np.zeros_like(mo1), np.zeros_like(mo2)
    oracle.mask_igemm(x, w, ref, tb.indices, tb.mask, tb.mask_argsort, mask_filter=f1, mask_out=r1)
    oracle.mask_igemm(x, w, ref, tb.indices, tb.mask, tb.mask_argsort, mask_filter=f2, beta=1.0, mask_out=r2)
    assert (mo1 == r1).all() and (mo2 == r2).all()
    H.assert_close_f16(out2, ref, "two-pass mask split")


def test_forward_no_neighbours_still_runs_epilogue(torch, oracle):
    """A tile whose mask is empty still writes act(beta * source) (cumm/conv/kernel.py:906-920)."""
    tb, x, w, _ = make(300, 61, 64, 64)
    init = np.random.default_rng(2).standard_normal((tb.n_out, 64)).astype(np.float16)
    got, mo = H.run_conv_fwd(torch, x, w, tb, mask_filter=0, out_init=init, beta=1.0)
    H.check_status()
    assert (mo == 0).all()
    H.assert_close_f16(got, init, "beta * source only")
    got, _ = H.run_conv_fwd(torch, x, w, tb, mask_filter=0, out_init=init, beta=0.0)
    assert (got == 0).all()


def test_forward_missing_pairs_everywhere(torch, oracle):
    """Mask bits set but every table entry -1: rows are zero-filled, nothing is read."""
    tb, x, w, _ = make(500, 71, 64, 64)
    tb.indices[:] = -1
    got, _ = H.run_conv_fwd(torch, x, w, tb)
    H.check_status()
    assert (got == 0).all()


@pytest.mark.parametrize("n,C,K", [(130, 64, 64), (3000, 128, 128), (2500, 64, 128), (2500, 128, 64), (2000, 24, 40),
                                    (1500, 256, 256)])
def test_backward_input(torch, oracle, n, C, K):
    tb, _, w, dout = make(n, 200 + n + C, C, K)
    got = H.run_conv_dgrad(torch, dout, w, tb)
    H.check_status()
    want = oracle.mask_igemm(dout, w, np.zeros((tb.n_in, C), np.float16), tb.indices_bwd, tb.mask_bwd,
                             tb.mask_argsort_bwd, is_dgrad=True)
    H.assert_close_f16(got, want, f"dgrad n={n} C={C} K={K}")
    got2 = H.run_conv_dgrad(torch, dout, w, tb, use_reverse=True)
    H.check_status()
    H.assert_close_f16(got2, want, "dgrad via reversed forward masks")


def test_backward_input_regular_conv(torch, oracle):
    tb, _, w, dout = make(2500, 231, 64, 64, stride=(2, 2, 2), subm=False)
    got = H.run_conv_dgrad(torch, dout, w, tb)
    H.check_status()
    want = oracle.np_dgrad(dout, w, tb.indices, tb.n_in)
    H.assert_close_f16(got, want, "stride-2 dgrad")


def test_backward_input_skips_empty_tiles(torch, oracle):
    """A tile with an empty mask is left untouched (cumm/conv/kernel.py:875-882)."""
    tb, _, w, dout = make(700, 241, 64, 64)
    init = np.random.default_rng(4).standard_normal((tb.n_in, 64)).astype(np.float16)
    got = H.run_conv_dgrad(torch, dout, w, tb, din_init=init, mask_filter=0)
    H.check_status()
    assert (got == init).all()


@pytest.mark.parametrize("n,C,K", [(100, 64, 64), (3000, 128, 128), (3000, 64, 64), (2500, 64, 128), (2500, 128, 64),
                                    (2000, 24, 40), (1500, 256, 192)])
def test_backward_weight(torch, oracle, n, C, K):
    tb, x, w, dout = make(n, 300 + n + C, C, K)
    _, mo = H.run_conv_fwd(torch, x, w, tb)
    got = H.run_conv_wgrad(torch, dout, x, tb, mo)
    H.check_status()
    want = oracle.mask_igemm_wgrad(dout, x, np.zeros((K, 27, C), np.float16), tb.indices, mo, tb.mask_argsort)
    H.assert_close_wgrad(got, want, tb.indices, f"wgrad n={n} C={C} K={K}")


def test_backward_weight_exact_on_small_integers(torch, oracle):
    """Inputs in {-2..2}: every product and partial sum is an integer that fp32 and fp16 hold
    exactly, so the result must equal the oracle's bit for bit whatever the summation order --
    a dropped or doubled row contribution cannot hide behind a tolerance."""
    tb, _, w, _ = make(3000, 333, 128, 128)
    rng = np.random.default_rng(334)
    x = rng.integers(-2, 3, (tb.n_in, 128)).astype(np.float16)
    dout = rng.integers(-2, 3, (tb.n_out, 128)).astype(np.float16)
    _, mo = H.run_conv_fwd(torch, x, w, tb)
    got = H.run_conv_wgrad(torch, dout, x, tb, mo)
    H.check_status()
    want = oracle.mask_igemm_wgrad(dout, x, np.zeros((128, 27, 128), np.float16), tb.indices, mo, tb.mask_argsort)
    assert np.abs(want.astype(np.float32)).max() < 2048 and (want != 0).mean() > 0.3, "degenerate test data"
    assert (got.view(np.uint16) == want.view(np.uint16)).all(), f"{int((got != want).sum())} entries differ"


def test_backward_weight_dense_block(torch, oracle):
    coords = W.dense_block_coords(12)
    tb = W.build_tables(coords, grid=(12, 12, 12))
    rng = np.random.default_rng(5)
    x = (rng.standard_normal((tb.n_in, 64)) / 4).astype(np.float16)
    dout = (rng.standard_normal((tb.n_out, 128)) / 4).astype(np.float16)
    w = np.zeros((128, 27, 64), np.float16)
    _, mo = H.run_conv_fwd(torch, x, w, tb)
    got = H.run_conv_wgrad(torch, dout, x, tb, mo)
    H.check_status()
    want = oracle.np_wgrad(dout, x, tb.indices)
    H.assert_close_f16(got, want, "dense block wgrad")


def test_backward_weight_split_filter_beta_and_fp32(torch, oracle):
    tb, x, w, dout = make(2000, 351, 64, 64)
    f1, f2 = 0b11111111111111, 0b1111111111111 << 14
    _, mo1 = H.run_conv_fwd(torch, x, w, tb, mask_filter=f1)
    _, mo2 = H.run_conv_fwd(torch, x, w, tb, mask_filter=f2)
    init = np.random.default_rng(6).standard_normal((64, 27, 64)).astype(np.float16)
    # pass 1 touches only the first 14 offsets; the others keep their previous content
    got1 = H.run_conv_wgrad(torch, dout, x, tb, mo1, dw_init=init, mask_filter=f1)
    ref = init.copy()
    oracle.mask_igemm_wgrad(dout, x, ref, tb.indices, mo1, tb.mask_argsort, mask_filter=f1)
    H.assert_close_wgrad(got1[:, :14], ref[:, :14], tb.indices[:14], "wgrad pass 1")
    assert (got1[:, 14:, :] == init[:, 14:, :]).all()
    got2 = H.run_conv_wgrad(torch, dout, x, tb, mo2, dw_init=got1, mask_filter=f2, beta=1.0, alpha=0.5)
    oracle.mask_igemm_wgrad(dout, x, ref, tb.indices, mo2, tb.mask_argsort, mask_filter=f2, beta=1.0, alpha=0.5)
    H.check_status()
    H.assert_close_wgrad(got2, ref, tb.indices, "wgrad pass 2")
    # fp32 output (the form the multi-GPU partial sums use)
    mo = mo1 | mo2
    got32 = H.run_conv_wgrad(torch, dout, x, tb, mo, fp32_out=True)
    want32 = oracle.mask_igemm_wgrad(dout, x, None, tb.indices, mo, tb.mask_argsort,
                                     out_f32=np.zeros((64, 27, 64), np.float32))
    np.testing.assert_allclose(got32, want32, rtol=1e-3, atol=1e-3)


@pytest.mark.parametrize("mask_width", [32, 64, 256])
def test_backward_weight_other_mask_widths(torch, oracle, mask_width):
    tb, x, w, dout = make(1500, 371, 64, 64)
    words = (tb.n_out + mask_width - 1) // mask_width
    rm = np.array([np.bitwise_or.reduce(tb.mask[i * mask_width:(i + 1) * mask_width]) for i in range(words)],
                  np.uint32)
    got = H.run_conv_wgrad(torch, dout, x, tb, rm, mask_width=mask_width)
    H.check_status()
    want = oracle.mask_igemm_wgrad(dout, x, np.zeros((64, 27, 64), np.float16), tb.indices, rm, tb.mask_argsort,
                                   mask_width=mask_width)
    H.assert_close_wgrad(got, want, tb.indices, f"wgrad mask_width={mask_width}")


@pytest.mark.parametrize("n,C,K", [(100, 128, 128), (3000, 128, 128), (2500, 64, 64), (2500, 128, 64), (2000, 32, 48),
                                    (1500, 256, 128)])
def test_int8_inference_bit_exact(torch, oracle, n, C, K):
    tb, _, _, _ = make(n, 400 + n + C, 16, 16, stride=(2, 2, 2), subm=False)
    rng = np.random.default_rng(n + C)
    x = rng.integers(-127, 128, (tb.n_in, C)).astype(np.int8)
    w = rng.integers(-127, 128, (K, 27, C)).astype(np.int8)
    scale = (rng.uniform(1e-3, 1e-2, K) / 16).astype(np.float32)
    bias = rng.standard_normal(K).astype(np.float32)
    got = H.run_conv_s8(torch, x, w, scale, bias, tb)
    H.check_status()
    want = oracle.mask_igemm_s8(x, w, np.zeros((tb.n_out, K), np.int8), scale, bias, tb.indices, tb.mask,
                                tb.mask_argsort)
    assert (want != 0).mean() > 0.5 and (np.abs(want.astype(int)) < 127).mean() > 0.5, "degenerate test data"
    assert (got == want).all(), f"{int((got != want).sum())} of {got.size} int8 outputs differ"


def test_int8_large_accumulators_bit_exact(torch, oracle):
    """Extreme int8 inputs on a dense block: |accumulator| reaches 127 * 127 * 128 * 27 > 2^24, far
    outside the range in which int32 -> float is a mantissa add, and part of the outputs saturate."""
    coords = W.dense_block_coords(10)
    tb = W.build_tables(coords)
    C = K = 128
    rng = np.random.default_rng(77)
    x = np.where(rng.random((tb.n_in, C)) < 0.9, 127, -127).astype(np.int8)
    w = np.where(rng.random((K, 27, C)) < 0.9, 127, -127).astype(np.int8)
    scale = (rng.uniform(1.5e-6, 4.5e-6, K)).astype(np.float32)
    bias = rng.standard_normal(K).astype(np.float32)
    got = H.run_conv_s8(torch, x, w, scale, bias, tb)
    H.check_status()
    want = oracle.mask_igemm_s8(x, w, np.zeros((tb.n_out, K), np.int8), scale, bias, tb.indices, tb.mask,
                                tb.mask_argsort)
    assert (np.abs(want.astype(int)) < 127).mean() > 0.2 and (want == 127).any(), "degenerate test data"
    assert (got == want).all(), f"{int((got != want).sum())} of {got.size} int8 outputs differ"


def test_int8_output_add_and_relu(torch, oracle):
    tb, _, _, _ = make(2000, 451, 16, 16)
    rng = np.random.default_rng(8)
    C = K = 128
    x = rng.integers(-127, 128, (tb.n_in, C)).astype(np.int8)
    w = rng.integers(-127, 128, (K, 27, C)).astype(np.int8)
    scale = (rng.uniform(1e-3, 1e-2, K) / 8).astype(np.float32)
    bias = rng.standard_normal(K).astype(np.float32)
    add = rng.integers(-127, 128, (tb.n_out, K)).astype(np.int8)
    got = H.run_conv_s8(torch, x, w, scale, bias, tb, output_add=add, beta=0.75, act=Activation.ReLU)
    H.check_status()
    want = oracle.mask_igemm_s8(x, w, np.zeros((tb.n_out, K), np.int8), scale, bias, tb.indices, tb.mask,
                                tb.mask_argsort, output_add=add, beta=0.75, act_type=1)
    assert (got == want).all()
    assert (got >= 0).all()


def test_errors_surface_as_exceptions(torch):
    tb, x, w, _ = make(300, 501, 64, 64)
    p = ConvParams(3, ConvOpType.Forward)
    p.conv_algo_desp = H.conv_desp(ConvOpType.Forward, 64, 64)
    p.input = torch.zeros((tb.n_in, 64), dtype=torch.float32, device="cuda")  # no fp32 kernel
    p.weight = torch.zeros((64, 27, 64), dtype=torch.float32, device="cuda")
    p.output = torch.zeros((tb.n_out, 64), dtype=torch.float32, device="cuda")
    p.indices = H.dev(tb.indices, torch)
    p.mask = H.mask_to_torch(tb.mask, torch)
    p.mask_argsort = H.dev(tb.mask_argsort, torch)
    with pytest.raises(RuntimeError, match="can't find any suitable algo"):
        ConvMainUnitTest.implicit_gemm2(p)
    q = ConvParams(3, ConvOpType.Forward)
    q.conv_algo_desp = H.conv_desp(ConvOpType.Forward, 64, 64)
    q.input = torch.zeros((tb.n_in, 64), dtype=torch.float16)  # host tensor: no CPU path
    q.weight = H.dev(w, torch)
    q.output = torch.zeros((tb.n_out, 64), dtype=torch.float16, device="cuda")
    with pytest.raises(RuntimeError, match="CUDA device"):
        ConvMainUnitTest.implicit_gemm2(q)
    H.check_status()


def _tiles_for(op, int8=False):
    return [tuple(d.tile_shape) for d in ConvMainUnitTest.get_all_conv_algo_desp()
            if d.op_type == op and bool(d.is_int8_inference) == int8 and not d.dynamic_mask]


def test_every_listed_tile_shape_computes_the_same(torch, oracle):
    """The descriptor's tile shape selects the kernel variant (what the tuner varies): every entry of
    get_all_conv_algo_desp gives the oracle's result."""
    tb, x, w, dout = make(2500, 611, 128, 128)
    want_f = oracle.mask_igemm(x, w, np.zeros((tb.n_out, 128), np.float16), tb.indices, tb.mask, tb.mask_argsort)
    want_d = oracle.mask_igemm(dout, w, np.zeros((tb.n_in, 128), np.float16), tb.indices_bwd, tb.mask_bwd,
                               tb.mask_argsort_bwd, is_dgrad=True)
    tiles_f, tiles_d, tiles_w = (_tiles_for(ConvOpType.Forward), _tiles_for(ConvOpType.BackwardInput),
                                 _tiles_for(ConvOpType.BackwardWeight))
    assert len(tiles_f) == 4 and len(tiles_d) == 4 and len(tiles_w) == 2
    mo = None
    for t in tiles_f:
        got, mo = H.run_conv_fwd(torch, x, w, tb, tile=t)
        H.check_status()
        H.assert_close_f16(got, want_f, f"forward tile {t}")
    for t in tiles_d:
        got = H.run_conv_dgrad(torch, dout, w, tb, tile=t)
        H.check_status()
        H.assert_close_f16(got, want_d, f"dgrad tile {t}")
    want_w = oracle.mask_igemm_wgrad(dout, x, np.zeros((128, 27, 128), np.float16), tb.indices, mo, tb.mask_argsort)
    for t in tiles_w:
        got = H.run_conv_wgrad(torch, dout, x, tb, mo, tile=t)
        H.check_status()
        H.assert_close_wgrad(got, want_w, tb.indices, f"wgrad tile {t}")


def test_timer_verbose_and_nvrtc_entry_point(torch, oracle, capsys, monkeypatch):
    """params.timer brackets the launch with one event pair filed under the algorithm name
    (cumm/conv/main.py:708); verbose prints registers and time (:723-729); run_nvrtc_conv_kernel
    throws without a run-time-compiled module (cumm/tensorview_bind.py:147-149) unless the caller
    opts into the prebuilt kernels."""
    import cumm_b200.tensorview.gemm as G
    from cumm_b200.tensorview import CUDAKernelTimer
    tb, x, w, _ = make(1500, 801, 64, 64)
    timer = CUDAKernelTimer(True)
    p = ConvParams(3, ConvOpType.Forward, timer)
    p.conv_algo_desp = H.conv_desp(ConvOpType.Forward, 64, 64)
    p.input, p.weight = H.dev(x, torch), H.dev(w, torch)
    p.output = torch.zeros((tb.n_out, 64), dtype=torch.float16, device="cuda")
    p.indices, p.mask, p.mask_argsort = H.dev(tb.indices, torch), H.mask_to_torch(tb.mask, torch), H.dev(tb.mask_argsort, torch)
    p.verbose = True
    ConvMainUnitTest.implicit_gemm2(p)
    name = p.conv_algo_desp.__repr__()
    times = timer.get_all_pair_time()
    assert list(times) == [name] and 0.0 < times[name] < 100.0  # milliseconds
    printed = capsys.readouterr().out
    assert name in printed and "kernel num regs:" in printed and "time:" in printed
    want = oracle.mask_igemm(x, w, np.zeros((tb.n_out, 64), np.float16), tb.indices, tb.mask, tb.mask_argsort)
    H.assert_close_f16(p.output.cpu().numpy(), want, "forward with timer")
    p.verbose, p.timer = False, None
    monkeypatch.delenv("CUMM_B200_NVRTC_USES_PREBUILT", raising=False)
    with pytest.raises(RuntimeError, match="you must use nvrtc kernel"):
        G.run_nvrtc_conv_kernel(p)
    monkeypatch.setattr(G, "NVRTC_ENTRY_POINTS_USE_PREBUILT", True)
    p.output.zero_()
    G.run_nvrtc_conv_kernel(p)
    torch.cuda.synchronize()
    H.assert_close_f16(p.output.cpu().numpy(), want, "forward through run_nvrtc_conv_kernel, opted in")
    H.check_status()
