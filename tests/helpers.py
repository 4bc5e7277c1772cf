"""Shared builders for the parity tests: seeded inputs, calls through the operator
surface (which goes through the C ABI), comparisons with the CPU oracle."""
from __future__ import annotations

import numpy as np

from cumm_b200 import workloads as W
from cumm_b200.conv.main import ConvMainUnitTest
from cumm_b200.gemm.main import GemmMainUnitTest
from cumm_b200.tensorview import float16, float32, int8, int32
from cumm_b200.tensorview.gemm import (Activation, ConvAlgoDesp, ConvOpType, ConvParams, GemmAlgoDesp,
                                       GemmParams, ShuffleStrideType)

RTOL = 1e-2  # fp16 output, fp32 accumulation (tolerance stated by the task for the fp16 path)
ATOL = 1e-2


def conv_desp(op, C, K, int8_inference=False):
    d = ConvAlgoDesp(3, op)
    if int8_inference:
        d.dtype_a = d.dtype_b = d.dtype_c = int8
        d.dacc, d.dcomp = int32, float32
        epa = 16
    else:
        d.dtype_a = d.dtype_b = d.dtype_c = float16
        d.dacc = d.dcomp = float32
        epa = 8
    ta, tb, tc = {ConvOpType.Forward: (False, True, False), ConvOpType.BackwardInput: (False, False, False),
                  ConvOpType.BackwardWeight: (True, False, False)}[ConvOpType(int(op))]
    d.trans_a, d.trans_b, d.trans_c = ta, tb, tc
    from cumm_b200.layer import default_tile
    d.tile_shape = default_tile(op, C, K, int8_inference)
    d.warp_tile_shape = list(d.tile_shape)
    d.tensorop = [128, d.tile_shape[1], 32 if int8_inference else 16]
    d.num_stage = 3
    d.algo = "Blackwell"
    d.split_k_serial = int(op) == ConvOpType.BackwardWeight
    d.element_per_access_a = d.element_per_access_b = d.element_per_access_c = epa
    d.mask_sparse = True
    d.increment_k_first = True
    d.is_int8_inference = int8_inference
    return d


def gemm_desp(shuffle, trans_a=False, trans_b=True, n=128, k=128):
    """n, k: output and reduction widths of the problem; the tile is the narrowest that covers them."""
    d = GemmAlgoDesp()
    d.dtype_a = d.dtype_b = d.dtype_c = float16
    d.dacc = d.dcomp = float32
    d.trans_a, d.trans_b, d.trans_c = trans_a, trans_b, False
    d.tile_shape = [128, 64 if n <= 64 else 128, 64 if k <= 64 else 128]
    d.warp_tile_shape = list(d.tile_shape)
    d.tensorop = [128, d.tile_shape[1], 16]
    d.num_stage = 3
    d.algo = "Blackwell"
    d.shuffle_type = shuffle
    d.split_k_serial = shuffle == ShuffleStrideType.ShuffleAB
    d.element_per_access_a = d.element_per_access_b = d.element_per_access_c = 8
    return d


def random_tables(n, seed, grid=(8, 24, 24), **kw):
    coords = W.sample_coords(n, seed, grid)
    return W.build_tables(coords, grid=grid, **kw), coords


def dev(x, torch):
    return torch.from_numpy(np.ascontiguousarray(x)).cuda()


def mask_to_torch(mask, torch):
    """uint32 masks travel as int32 bit patterns (torch has no general uint32 kernels)."""
    return torch.from_numpy(np.ascontiguousarray(mask).view(np.int32)).cuda()


def run_conv_fwd(torch, x, w, tb, *, out_init=None, beta=0.0, alpha=1.0, bias=None, act=Activation.None_,
                 act_alpha=0.0, mask_filter=0xFFFFFFFF, want_mask_out=True, tile=None):
    K, kv, C = w.shape
    p = ConvParams(3, ConvOpType.Forward)
    p.conv_algo_desp = conv_desp(ConvOpType.Forward, C, K)
    _apply_tile(p, tile)
    p.input = dev(x, torch)
    p.weight = dev(w, torch)
    out = torch.zeros((tb.n_out, K), dtype=torch.float16, device="cuda") if out_init is None else dev(out_init, torch)
    p.output = out
    p.indices = dev(tb.indices, torch)
    p.mask = mask_to_torch(tb.mask, torch)
    p.mask_argsort = dev(tb.mask_argsort, torch)
    mo = torch.zeros(((tb.n_out + 127) // 128,), dtype=torch.int32, device="cuda")
    if want_mask_out:
        p.mask_output = mo
    p.alpha, p.beta = alpha, beta
    p.act_type, p.act_alpha = act, act_alpha
    p.mask_filter = mask_filter
    if bias is not None:
        p.bias = dev(bias, torch)
    ConvMainUnitTest.implicit_gemm2(p)
    torch.cuda.synchronize()
    return out.cpu().numpy(), mo.cpu().numpy().view(np.uint32)


def run_conv_dgrad(torch, dout, w, tb, *, din_init=None, beta=0.0, use_reverse=False, mask_filter=0xFFFFFFFF,
                   tile=None):
    K, kv, C = w.shape
    p = ConvParams(3, ConvOpType.BackwardInput)
    p.conv_algo_desp = conv_desp(ConvOpType.BackwardInput, C, K)
    _apply_tile(p, tile)
    din = torch.zeros((tb.n_in, C), dtype=torch.float16, device="cuda") if din_init is None else dev(din_init, torch)
    p.input = din
    p.weight = dev(w, torch)
    p.output = dev(dout, torch)
    if use_reverse:
        # submanifold: the forward masks and sort serve, with the tile mask bit-reversed
        p.indices = dev(tb.indices_bwd, torch)
        p.mask = mask_to_torch(tb.mask, torch)
        p.mask_argsort = dev(tb.mask_argsort, torch)
        p.reverse_mask = True
    else:
        p.indices = dev(tb.indices_bwd, torch)
        p.mask = mask_to_torch(tb.mask_bwd, torch)
        p.mask_argsort = dev(tb.mask_argsort_bwd, torch)
    p.beta = beta
    p.mask_filter = mask_filter
    ConvMainUnitTest.implicit_gemm2(p)
    torch.cuda.synchronize()
    return din.cpu().numpy()


def run_conv_wgrad(torch, dout, x, tb, reduced_mask, *, kv=27, dw_init=None, beta=0.0, alpha=1.0,
                   mask_filter=0xFFFFFFFF, mask_width=128, fp32_out=False, tile=None):
    K, C = dout.shape[1], x.shape[1]
    p = ConvParams(3, ConvOpType.BackwardWeight)
    p.conv_algo_desp = conv_desp(ConvOpType.BackwardWeight, C, K)
    _apply_tile(p, tile)
    p.input = dev(x, torch)
    dt = torch.float32 if fp32_out else torch.float16
    dw = torch.zeros((K, kv, C), dtype=dt, device="cuda") if dw_init is None else dev(dw_init, torch)
    p.weight = dw
    p.output = dev(dout, torch)
    p.indices = dev(tb.indices, torch)
    p.mask = mask_to_torch(reduced_mask, torch)
    p.mask_argsort = dev(tb.mask_argsort, torch)
    p.mask_width = mask_width
    if mask_width < 128:
        p.conv_algo_desp.tile_shape[2] = mask_width  # the reference requires mask_width % tile_k == 0
    p.mask_filter = mask_filter
    p.alpha, p.beta = alpha, beta
    p.split_k_slices = 32
    ConvMainUnitTest.implicit_gemm2(p)
    torch.cuda.synchronize()
    return dw.cpu().numpy()


def run_conv_s8(torch, x, w, scale, bias, tb, *, output_add=None, beta=0.0, act=Activation.None_, act_alpha=0.0,
                tile=None):
    K, kv, C = w.shape
    p = ConvParams(3, ConvOpType.Forward)
    p.conv_algo_desp = conv_desp(ConvOpType.Forward, C, K, int8_inference=True)
    _apply_tile(p, tile)
    p.input = dev(x, torch)
    p.weight = dev(w, torch)
    out = torch.zeros((tb.n_out, K), dtype=torch.int8, device="cuda")
    p.output = out
    p.scale = dev(scale, torch)
    p.bias = dev(bias, torch)
    if output_add is not None:
        p.output_add = dev(output_add, torch)
    p.indices = dev(tb.indices, torch)
    p.mask = mask_to_torch(tb.mask, torch)
    p.mask_argsort = dev(tb.mask_argsort, torch)
    p.beta = beta
    p.act_type, p.act_alpha = act, act_alpha
    ConvMainUnitTest.implicit_gemm2(p)
    torch.cuda.synchronize()
    return out.cpu().numpy()


def _apply_tile(p, tile):
    if tile is not None:
        p.conv_algo_desp.tile_shape = list(tile)
        p.conv_algo_desp.warp_tile_shape = list(tile)


def check_status():
    from cumm_b200 import _lib
    st = _lib.device_status()
    assert st == 0, f"device status word = {st} (1: a bounded wait ran out, 2: row index out of range)"


def assert_close_f16(got, want, what=""):
    got = got.astype(np.float32)
    want = want.astype(np.float32)
    err = np.abs(got - want)
    tol = ATOL + RTOL * np.abs(want)
    bad = err > tol
    assert not bad.any(), (f"{what}: {int(bad.sum())} of {bad.size} elements outside rtol={RTOL} atol={ATOL}; "
                           f"max abs err {float(err.max()):.4g} at {np.unravel_index(err.argmax(), err.shape)}")


def assert_close_wgrad(got, want, indices, what="", kv_axis=1):
    """Weight gradient [K, kv, C] against the oracle, one filter offset at a time.  Both sides
    accumulate in fp32 and round once, so every offset is held to the plain rtol / atol; the
    absolute part grows with the square root of the offset's pair count only beyond 4096 pairs
    (the centre offset of a large scene sums 10^5 products and its entries are of order 10^2)."""
    got = np.moveaxis(got.astype(np.float32), kv_axis, 0)
    want = np.moveaxis(want.astype(np.float32), kv_axis, 0)
    pairs = (np.asarray(indices) >= 0).sum(axis=1)
    assert got.shape == want.shape and got.shape[0] == len(pairs)
    for f in range(got.shape[0]):
        atol = ATOL * max(1.0, float(np.sqrt(pairs[f])) / 64.0)
        err = np.abs(got[f] - want[f])
        bad = err > atol + RTOL * np.abs(want[f])
        assert not bad.any(), (f"{what}: filter offset {f} ({int(pairs[f])} pairs): {int(bad.sum())} of {bad.size} "
                               f"entries outside rtol={RTOL} atol={atol:.3g}; max abs err {float(err.max()):.4g}")
