"""Kernel volumes above 32 (several mask words per row; the reference's dynamic-mask kernels,
cumm/gemm/blockmma/mma.py:78-270).  On CPU: the C oracle's multi-word control flow against
the numpy statement of the operators, which never looks at masks.  On the GPU: the kernels
against the oracle, for 5x5x5 (125 offsets, four words) and 3x3x5 (45 offsets, two words)."""
import numpy as np
import pytest

import helpers as H
from cumm_b200 import workloads as W

GRID = (10, 20, 20)


def make(n, seed, ksize, C, K, **kw):
    coords = W.sample_coords(n, seed, GRID)
    tb = W.build_tables(coords, grid=GRID, ksize=ksize, **kw)
    rng = np.random.default_rng(seed + 1)
    x = rng.standard_normal((tb.n_in, C)).astype(np.float16)
    w = (rng.standard_normal((K, tb.kv, C)) / np.sqrt(tb.kv * C) * 6).astype(np.float16)
    dout = rng.standard_normal((tb.n_out, K)).astype(np.float16)
    return tb, x, w, dout


def tile_masks(mask, tile=128):
    n, words = mask.shape
    tiles = (n + tile - 1) // tile
    return np.stack([np.bitwise_or.reduce(mask[t * tile:(t + 1) * tile], axis=0) for t in range(tiles)])


@pytest.mark.parametrize("ksize", [(5, 5, 5), (3, 3, 5)])
def test_oracle_multi_word_masks_against_numpy_statement(oracle, ksize):
    tb, x, w, dout = make(1500, 900, ksize, 16, 24)
    words = (tb.kv + 31) // 32
    assert tb.mask.shape == (tb.n_out, words) and tb.kv > 32
    # the generator's masks are the table's, and sorted as one integer (last word most significant)
    m = tb.mask.astype(object)
    big = sum(m[:, i] << (32 * i) for i in range(words))
    assert all(big[i] <= big[i + 1] for i in range(len(big) - 1))
    assert (W.masks_from_indices(tb.indices)[tb.mask_argsort] == tb.mask).all()
    idx_c, mask_c = oracle.build_pairs(W.sample_coords(1500, 900, GRID), W.sample_coords(1500, 900, GRID), GRID, ksize,
                                       (1, 1, 1), tuple(k // 2 for k in ksize), (1, 1, 1))
    assert (idx_c == tb.indices).all() and (mask_c[tb.mask_argsort] == tb.mask).all()
    K, C = w.shape[0], w.shape[2]
    mo = np.zeros(((tb.n_out + 127) // 128, words), np.uint32)
    out = oracle.mask_igemm(x, w, np.zeros((tb.n_out, K), np.float16), tb.indices, tb.mask, tb.mask_argsort, mask_out=mo)
    assert (mo == tile_masks(tb.mask)).all()
    H.assert_close_f16(out, oracle.np_forward(x, w, tb.indices), "oracle forward")
    want_d = oracle.np_dgrad(dout, w, tb.indices, tb.n_in)
    din = oracle.mask_igemm(dout, w, np.zeros((tb.n_in, C), np.float16), tb.indices_bwd, tb.mask_bwd,
                            tb.mask_argsort_bwd, is_dgrad=True)
    H.assert_close_f16(din, want_d, "oracle dgrad")
    # submanifold: the forward masks serve the input gradient with reverse_mask
    din_r = oracle.mask_igemm(dout, w, np.zeros((tb.n_in, C), np.float16), tb.indices_bwd, tb.mask, tb.mask_argsort,
                              is_dgrad=True, reverse_mask=True)
    H.assert_close_f16(din_r, want_d, "oracle dgrad, reversed forward masks")
    dw = oracle.mask_igemm_wgrad(dout, x, np.zeros((K, tb.kv, C), np.float16), tb.indices, mo, tb.mask_argsort)
    H.assert_close_wgrad(dw, oracle.np_wgrad(dout, x, tb.indices), tb.indices, "oracle wgrad")
    # a filter applies to every word alike
    flt = 0x0F0F0F0F
    out_f = oracle.mask_igemm(x, w, np.zeros((tb.n_out, K), np.float16), tb.indices, tb.mask, tb.mask_argsort,
                              mask_filter=flt)
    keep = np.array([(flt >> (f & 31)) & 1 for f in range(tb.kv)], bool)
    idx_f = np.where(keep[:, None], tb.indices, -1)
    H.assert_close_f16(out_f, oracle.np_forward(x, w, idx_f), "oracle forward, filtered")


def run_params(torch, op, tb, **tensors):
    from cumm_b200.conv.main import ConvMainUnitTest
    from cumm_b200.tensorview.gemm import ConvParams
    p = ConvParams(3, op)
    C, K = tensors["weight"].shape[2], tensors["weight"].shape[0]
    p.conv_algo_desp = H.conv_desp(op, C, K, int8_inference=tensors.get("scale") is not None)
    p.conv_algo_desp.dynamic_mask = True
    for k, v in tensors.items():
        setattr(p, k, v)
    ConvMainUnitTest.implicit_gemm2(p)
    torch.cuda.synchronize()
    return p


@pytest.mark.gpu
@pytest.mark.parametrize("ksize,n,C,K", [((5, 5, 5), 3000, 64, 64), ((3, 3, 5), 2500, 128, 128), ((5, 5, 5), 700, 32, 48)])
def test_gpu_large_kernel_volume_all_ops(cuda_lib, oracle, ksize, n, C, K):
    import torch
    from cumm_b200.tensorview.gemm import ConvOpType
    tb, x, w, dout = make(n, 910 + n, ksize, C, K)
    words = (tb.kv + 31) // 32
    tiles = (tb.n_out + 127) // 128
    d = lambda a: H.dev(a, torch)
    dm = lambda a: torch.from_numpy(np.ascontiguousarray(a).view(np.int32)).cuda()
    # forward, with the per-tile masks
    out = torch.zeros((tb.n_out, K), dtype=torch.float16, device="cuda")
    mo = torch.zeros((tiles, words), dtype=torch.int32, device="cuda")
    run_params(torch, ConvOpType.Forward, tb, input=d(x), weight=d(w), output=out, indices=d(tb.indices),
               mask=dm(tb.mask), mask_argsort=d(tb.mask_argsort), mask_output=mo)
    H.check_status()
    mo_ref = np.zeros((tiles, words), np.uint32)
    want = oracle.mask_igemm(x, w, np.zeros((tb.n_out, K), np.float16), tb.indices, tb.mask, tb.mask_argsort,
                             mask_out=mo_ref)
    assert (mo.cpu().numpy().view(np.uint32) == mo_ref).all(), "tile masks must be bit-exact"
    H.assert_close_f16(out.cpu().numpy(), want, "forward")
    # input gradient: own backward masks, then the forward masks reversed
    want_d = oracle.mask_igemm(dout, w, np.zeros((tb.n_in, C), np.float16), tb.indices_bwd, tb.mask_bwd,
                               tb.mask_argsort_bwd, is_dgrad=True)
    for kw in (dict(mask=dm(tb.mask_bwd), mask_argsort=d(tb.mask_argsort_bwd)),
               dict(mask=dm(tb.mask), mask_argsort=d(tb.mask_argsort), reverse_mask=True)):
        din = torch.zeros((tb.n_in, C), dtype=torch.float16, device="cuda")
        run_params(torch, ConvOpType.BackwardInput, tb, input=din, weight=d(w), output=d(dout),
                   indices=d(tb.indices_bwd), **kw)
        H.check_status()
        H.assert_close_f16(din.cpu().numpy(), want_d, f"dgrad {sorted(kw)}")
    # weight gradient from the forward pass's tile masks
    dw = torch.zeros((K, tb.kv, C), dtype=torch.float16, device="cuda")
    run_params(torch, ConvOpType.BackwardWeight, tb, input=d(x), weight=dw, output=d(dout), indices=d(tb.indices),
               mask=mo, mask_argsort=d(tb.mask_argsort), mask_width=128, split_k_slices=32)
    H.check_status()
    want_w = oracle.mask_igemm_wgrad(dout, x, np.zeros((K, tb.kv, C), np.float16), tb.indices, mo_ref, tb.mask_argsort)
    H.assert_close_wgrad(dw.cpu().numpy(), want_w, tb.indices, "wgrad")


@pytest.mark.gpu
def test_gpu_large_kernel_volume_int8_and_filter(cuda_lib, oracle):
    import torch
    from cumm_b200.tensorview.gemm import ConvOpType
    tb, x, w, _ = make(2000, 930, (5, 5, 5), 64, 64)
    words = (tb.kv + 31) // 32
    rng = np.random.default_rng(931)
    d = lambda a: H.dev(a, torch)
    dm = lambda a: torch.from_numpy(np.ascontiguousarray(a).view(np.int32)).cuda()
    C = K = 128
    x8 = rng.integers(-127, 128, (tb.n_in, C)).astype(np.int8)
    w8 = rng.integers(-127, 128, (K, tb.kv, C)).astype(np.int8)
    scale = (rng.uniform(1e-3, 1e-2, K) / 16).astype(np.float32)
    bias = rng.standard_normal(K).astype(np.float32)
    o8 = torch.zeros((tb.n_out, K), dtype=torch.int8, device="cuda")
    run_params(torch, ConvOpType.Forward, tb, input=d(x8), weight=d(w8), output=o8, scale=d(scale), bias=d(bias),
               indices=d(tb.indices), mask=dm(tb.mask), mask_argsort=d(tb.mask_argsort))
    H.check_status()
    want8 = oracle.mask_igemm_s8(x8, w8, np.zeros((tb.n_out, K), np.int8), scale, bias, tb.indices, tb.mask, tb.mask_argsort)
    assert (o8.cpu().numpy() == want8).all()
    # fp16 forward under a filter that keeps every other group of four offsets in every word
    flt = 0x0F0F0F0F
    out = torch.zeros((tb.n_out, 64), dtype=torch.float16, device="cuda")
    run_params(torch, ConvOpType.Forward, tb, input=d(x), weight=d(w), output=out, indices=d(tb.indices),
               mask=dm(tb.mask), mask_argsort=d(tb.mask_argsort), mask_filter=flt)
    H.check_status()
    want = oracle.mask_igemm(x, w, np.zeros((tb.n_out, 64), np.float16), tb.indices, tb.mask, tb.mask_argsort,
                             mask_filter=flt)
    H.assert_close_f16(out.cpu().numpy(), want, "filtered forward")


def test_large_volume_needs_a_dynamic_mask_descriptor():
    """The static-mask descriptors stop at 32 offsets, as the reference's static kernels do."""
    from cumm_b200.tensorview import Tensor, float16, int32
    from cumm_b200.tensorview.gemm import ConvOpType, ConvParams, _conv_args
    p = ConvParams(3, ConvOpType.Forward)
    p.conv_algo_desp = H.conv_desp(ConvOpType.Forward, 64, 64)
    n = 256
    fake = lambda shape, dt: Tensor(256, list(shape), dt, 0)
    p.input, p.weight, p.output = fake((n, 64), float16), fake((64, 125, 64), float16), fake((n, 64), float16)
    p.indices, p.mask, p.mask_argsort = fake((125, n), int32), fake((n, 4), int32), fake((n,), int32)
    with pytest.raises(RuntimeError, match="dynamic-mask descriptor"):
        _conv_args(p)
    p.conv_algo_desp.dynamic_mask = True
    assert _conv_args(p).kernel_volume == 125
    p.mask = fake((n, 3), int32)
    with pytest.raises(RuntimeError, match="4 per row"):
        _conv_args(p)
