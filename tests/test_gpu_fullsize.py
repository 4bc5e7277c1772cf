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
    np.testing.assert_allclose(dw, want, rtol=1e-2, atol=0.5)  # centre entries are sums of 150k products
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
