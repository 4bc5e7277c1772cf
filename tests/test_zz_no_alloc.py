"""The allocation-free weight-gradient entry point (cb2_conv_backward_weight_static).

Some callers cannot allocate device memory at the point where they need the weight
gradient: they are inside a CUDA stream capture, or on a serving thread that must not
touch the allocator, or they are a plugin that is handed tensors but no allocator.  For
them the library keeps 16 MiB of scratch inside its own image, and this entry point uses
that instead of a workspace argument.  The test calls it through the C ABI twice in a row,
on different inputs (the second call finds the first call's leftovers in the scratch), and
checks each result against the regular entry point given an ordinary workspace.

This file is meant to be collected last, so that a run which stops at the first failure
has already executed every other test.
"""
import ctypes

import numpy as np
import pytest

import helpers as H
from cumm_b200 import _lib
from cumm_b200.tensorview.gemm import ConvOpType, ConvParams, _conv_args

pytestmark = pytest.mark.gpu


def _wgrad_args(torch, dout, x, tb, reduced_mask, dw, kv=27):
    p = ConvParams(3, ConvOpType.BackwardWeight)
    p.conv_algo_desp = H.conv_desp(ConvOpType.BackwardWeight, x.shape[1], dout.shape[1])
    p.input = H.dev(x, torch)
    p.weight = dw
    p.output = H.dev(dout, torch)
    p.indices = H.dev(tb.indices, torch)
    p.mask = H.mask_to_torch(reduced_mask, torch)
    p.mask_argsort = H.dev(tb.mask_argsort, torch)
    p.mask_width = 128
    p.split_k_slices = 32
    return p, _conv_args(p)


def test_static_scratch_weight_gradient_matches_regular_entry_point(cuda_lib):
    import torch
    L = cuda_lib
    assert L.cb2_static_scratch_bytes() == 16 << 20
    for n, C, K, seed in ((3000, 128, 128, 11), (1700, 64, 128, 12)):
        tb, coords = H.random_tables(n, seed, grid=(8, 24, 24))
        rng = np.random.default_rng(seed)
        x = rng.standard_normal((tb.n_in, C)).astype(np.float16)
        dout = rng.standard_normal((tb.n_out, K)).astype(np.float16)
        w = np.zeros((K, 27, C), np.float16)
        _, mo = H.run_conv_fwd(torch, x, w, tb)
        # regular entry point with a caller-provided workspace
        want = H.run_conv_wgrad(torch, dout, x, tb, mo)
        # allocation-free entry point, straight through the C ABI
        dw = torch.zeros((K, 27, C), dtype=torch.float16, device="cuda")
        params, args = _wgrad_args(torch, dout, x, tb, mo, dw)
        args.workspace, args.workspace_bytes = None, 0
        rc = L.cb2_conv_backward_weight_static(ctypes.byref(args), ctypes.c_void_p(0))
        assert rc == 0, _lib.last_error()
        st = ctypes.c_int(-1)
        assert L.cb2_static_status(ctypes.byref(st)) == 0 and st.value == 0
        got = dw.cpu().numpy()
        H.assert_close_wgrad(got, want, tb.indices, f"static-scratch wgrad n={n} C={C} K={K}")
        # allocates nothing: a repeat of the call (the first one on a device resolves the scratch
        # address) leaves the device's free memory and torch's allocator where they were
        torch.cuda.synchronize()
        free0, alloc0 = torch.cuda.mem_get_info()[0], torch.cuda.memory_allocated()
        rc = L.cb2_conv_backward_weight_static(ctypes.byref(args), ctypes.c_void_p(0))
        assert rc == 0, _lib.last_error()
        torch.cuda.synchronize()
        assert torch.cuda.mem_get_info()[0] == free0 and torch.cuda.memory_allocated() == alloc0
        assert L.cb2_static_status(ctypes.byref(st)) == 0 and st.value == 0
        H.assert_close_wgrad(dw.cpu().numpy(), want, tb.indices, "static-scratch wgrad, repeated call")
    H.check_status()


def test_static_scratch_refuses_what_does_not_fit(cuda_lib):
    import torch
    L = cuda_lib
    tb, _ = H.random_tables(600, 13, grid=(8, 24, 24))
    rng = np.random.default_rng(13)
    C = K = 256  # 4 (m, n) tile pairs: more partial sums than 16 MiB hold
    x = rng.standard_normal((tb.n_in, C)).astype(np.float16)
    dout = rng.standard_normal((tb.n_out, K)).astype(np.float16)
    mo = np.full((tb.n_out + 127) // 128, 0x7FFFFFF, np.uint32)
    dw = torch.zeros((K, 27, C), dtype=torch.float16, device="cuda")
    params, args = _wgrad_args(torch, dout, x, tb, mo, dw)
    rc = L.cb2_conv_backward_weight_static(ctypes.byref(args), ctypes.c_void_p(0))
    assert rc == _lib.CB2_ERR_RUNTIME
    assert "static scratch holds" in _lib.last_error()
    assert (dw == 0).all()
    # and the wrong op type is refused too
    args.op_type = 0
    assert L.cb2_conv_backward_weight_static(ctypes.byref(args), ctypes.c_void_p(0)) == _lib.CB2_ERR_RUNTIME
