"""Dense (non-mask) convolution behind ConvParams (conv_algo_desp.mask_sparse = False), channels
last, against torch.nn.functional.conv{1,2,3}d and its autograd in fp32 on the CPU -- the check
the reference's own dense harness makes (cumm/conv/main_real.py:41-231)."""
import numpy as np
import pytest

import helpers as H
from cumm_b200.conv.main import ConvMainUnitTest
from cumm_b200.tensorview.gemm import ConvOpType, ConvParams

pytestmark = pytest.mark.gpu


def dense_params(op, ndim, C, K, padding, stride, dilation):
    p = ConvParams(ndim, op)
    d = H.conv_desp(op, C, K)
    d.ndim = ndim
    d.mask_sparse = False
    p.conv_algo_desp = d
    p.padding, p.stride, p.dilation = list(padding), list(stride), list(dilation)
    return p


def torch_reference(torch, x, w, dout, padding, stride, dilation):
    """x [N, *S, C], w [K, *k, C], dout [N, *So, K] (numpy fp16) -> out, din, dw in the same layouts (fp32)."""
    import torch.nn.functional as F
    ndim = x.ndim - 2
    to_cf = lambda a: torch.from_numpy(a.astype(np.float32)).movedim(-1, 1).contiguous()
    xt, wt = to_cf(x).requires_grad_(True), to_cf(w).requires_grad_(True)
    conv = {1: F.conv1d, 2: F.conv2d, 3: F.conv3d}[ndim]
    out = conv(xt, wt, None, stride=tuple(stride), padding=tuple(padding), dilation=tuple(dilation))
    din, dw = torch.autograd.grad(out, (xt, wt), to_cf(dout))
    back = lambda t: t.detach().movedim(1, -1).contiguous().numpy()
    return back(out), back(din), back(dw)


@pytest.mark.parametrize("shape,ksize,C,K,padding,stride,dilation", [
    ((2, 6, 10, 12), (3, 3, 3), 32, 48, (1, 1, 1), (1, 1, 1), (1, 1, 1)),
    ((1, 9, 11, 13), (3, 3, 3), 64, 64, (1, 1, 1), (2, 2, 2), (1, 1, 1)),
    ((2, 20, 24), (3, 3), 64, 128, (2, 2), (1, 1), (2, 2)),
    ((3, 200), (5,), 16, 24, (2,), (2,), (1,)),
    ((1, 5, 8, 8), (3, 5, 5), 16, 16, (1, 2, 2), (1, 1, 1), (1, 1, 1)),  # 75 filter offsets: three mask words
])
def test_dense_convolution_against_torch(cuda_lib, shape, ksize, C, K, padding, stride, dilation):
    import torch
    ndim = len(ksize)
    rng = np.random.default_rng(sum(shape) + C)
    x = rng.standard_normal(shape + (C,)).astype(np.float16)
    w = (rng.standard_normal((K,) + ksize + (C,)) / np.sqrt(np.prod(ksize) * C) * 4).astype(np.float16)
    out_sp = tuple((shape[1 + a] + 2 * padding[a] - dilation[a] * (ksize[a] - 1) - 1) // stride[a] + 1 for a in range(ndim))
    dout = rng.standard_normal((shape[0],) + out_sp + (K,)).astype(np.float16)
    want_out, want_din, want_dw = torch_reference(torch, x, w, dout, padding, stride, dilation)
    xd, wd, dd = H.dev(x, torch), H.dev(w, torch), H.dev(dout, torch)
    # forward
    p = dense_params(ConvOpType.Forward, ndim, C, K, padding, stride, dilation)
    out = torch.zeros(dout.shape, dtype=torch.float16, device="cuda")
    p.input, p.weight, p.output = xd, wd, out
    ConvMainUnitTest.implicit_gemm2(p)
    torch.cuda.synchronize()
    H.check_status()
    H.assert_close_f16(out.cpu().numpy(), want_out, "dense forward")
    # backward input
    q = dense_params(ConvOpType.BackwardInput, ndim, C, K, padding, stride, dilation)
    din = torch.zeros(x.shape, dtype=torch.float16, device="cuda")
    q.input, q.weight, q.output = din, wd, dd
    ConvMainUnitTest.implicit_gemm2(q)
    torch.cuda.synchronize()
    H.check_status()
    H.assert_close_f16(din.cpu().numpy(), want_din, "dense backward input")
    # backward weight: sums over all output positions; tolerance grows with their number
    r = dense_params(ConvOpType.BackwardWeight, ndim, C, K, padding, stride, dilation)
    dw = torch.zeros(w.shape, dtype=torch.float16, device="cuda")
    r.input, r.weight, r.output = xd, dw, dd
    r.mask_width = 128
    ConvMainUnitTest.implicit_gemm2(r)
    torch.cuda.synchronize()
    H.check_status()
    got = dw.cpu().numpy().astype(np.float32)
    n_pos = int(np.prod(dout.shape[:-1]))
    tol = H.ATOL * max(1.0, np.sqrt(n_pos) / 64.0) + H.RTOL * np.abs(want_dw)
    assert (np.abs(got - want_dw) <= tol).all(), f"dense backward weight: max abs err {np.abs(got - want_dw).max():.4g}"


def test_dense_convolution_checks_shapes(cuda_lib):
    import torch
    p = dense_params(ConvOpType.Forward, 3, 16, 16, (1, 1, 1), (1, 1, 1), (1, 1, 1))
    p.input = torch.zeros((1, 4, 4, 4, 16), dtype=torch.float16, device="cuda")
    p.weight = torch.zeros((16, 3, 3, 3, 16), dtype=torch.float16, device="cuda")
    p.output = torch.zeros((1, 4, 4, 5, 16), dtype=torch.float16, device="cuda")
    with pytest.raises(RuntimeError, match="output extent"):
        ConvMainUnitTest.implicit_gemm2(p)
    p.output = torch.zeros((64, 16), dtype=torch.float16, device="cuda")
    with pytest.raises(RuntimeError, match="channels-last"):
        ConvMainUnitTest.implicit_gemm2(p)
