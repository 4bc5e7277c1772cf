"""Pins the CPU oracle to the reference's own host code: golden vectors generated from the
reference headers (tests/golden/make_golden.py) and, where it was built in this checkout,
the compiled reference shim itself (oracle/_ref)."""
import ctypes
import json
from pathlib import Path

import numpy as np
import pytest

GOLD = Path(__file__).resolve().parent / "golden"


@pytest.fixture(scope="module")
def gold():
    return np.load(GOLD / "numerics.npz")


def test_float_to_half_matches_reference_vectors(oracle, gold):
    f, want = gold["f32_to_f16_in"], gold["f32_to_f16_out"]
    got = np.array([oracle.float_to_half(v) for v in f], np.uint16)
    bad = np.nonzero(got != want)[0]
    assert len(bad) == 0, [(float(f[i]), hex(got[i]), hex(want[i])) for i in bad[:5]]


def test_float_to_half_matches_numpy(oracle):
    rng = np.random.default_rng(3)
    f = (rng.standard_normal(20000) * np.exp(rng.uniform(-18, 11, 20000))).astype(np.float32)
    got = np.array([oracle.float_to_half(v) for v in f], np.uint16)
    with np.errstate(over="ignore"):
        want = f.astype(np.float16).view(np.uint16)
    assert (got == want).all()


def test_half_to_float_all_values(oracle, gold):
    bits, want = gold["f16_bits"], gold["f16_to_f32"]
    got = np.array([oracle.half_to_float(int(b)) for b in bits], np.float32)
    assert (got.view(np.uint32) == want.view(np.uint32)).all()
    assert (bits.view(np.float16).astype(np.float32).view(np.uint32) == want.view(np.uint32)).all()


def test_float_to_s8_matches_reference_vectors(oracle, gold):
    s, want = gold["f32_to_s8_in"], gold["f32_to_s8_out"]
    got = np.array([oracle.float_to_s8(v) for v in s], np.int8)
    assert (got == want).all()
    # hand-checked values: ties go to even, saturation at both ends
    for v, q in ((0.5, 0), (1.5, 2), (2.5, 2), (127.5, 127), (200.0, 127), (-128.5, -128), (-300.0, -128)):
        assert oracle.float_to_s8(v) == q
    assert oracle.float_to_s8(float("nan")) == 0
    # beyond int32 the device converter saturates (the host twin of the reference is undefined there)
    assert oracle.float_to_s8(3e9) == 127 and oracle.float_to_s8(-3e9) == -128


def test_live_reference_shim_if_built(oracle):
    R = oracle.ref_lib()
    if R is None:
        pytest.skip("oracle/_ref not built in this checkout")
    rng = np.random.default_rng(11)
    for v in (rng.standard_normal(3000) * np.exp(rng.uniform(-20, 12, 3000))).astype(np.float32):
        assert oracle.float_to_half(float(v)) == R.ref_float_to_half(float(v))
    for v in (rng.standard_normal(3000) * 70).astype(np.float32):
        assert oracle.float_to_s8(float(v)) == R.ref_float_to_s8(float(v))


def test_requant_epilogue_is_fused_multiply_add(oracle):
    """t = fma(scale, float(acc), bias): a case where the unfused product rounds differently."""
    acc = np.array([[16777217, -33554433, 123456789, 7]], np.int32)
    scale = np.array([0.00390625, 1e-7, 3.3e-7, 0.5], np.float32)
    bias = np.array([0.5, 0.25, -0.5, 0.0], np.float32)
    got = oracle.requant_s8(acc, scale, bias)
    want = []
    for a, s, b in zip(acc[0], scale, bias):
        t = np.float32(np.float64(np.float32(a)) * np.float64(s) + np.float64(b))  # exact product, one rounding
        want.append(oracle.float_to_s8(float(t)))
    assert got[0].tolist() == want


def test_c_restatement_agrees_with_numpy_statement(oracle):
    """Device-control-flow C oracle vs the per-offset numpy gather-matmul-scatter
    (the reference's own check loop, cumm/conv/main_real_spconv.py:309-403)."""
    from cumm_b200 import workloads as W
    rng = np.random.default_rng(5)
    coords = W.sample_coords(900, 7, (6, 14, 14))
    tb = W.build_tables(coords, grid=(6, 14, 14))
    C, K, kv = 24, 40, 27
    x = rng.standard_normal((tb.n_in, C)).astype(np.float16)
    w = (rng.standard_normal((K, kv, C)) / 8).astype(np.float16)
    dout = rng.standard_normal((tb.n_out, K)).astype(np.float16)
    mo = np.zeros((tb.n_out + 127) // 128, np.uint32)
    out = oracle.mask_igemm(x, w, np.zeros((tb.n_out, K), np.float16), tb.indices, tb.mask, tb.mask_argsort,
                            mask_out=mo)
    ref = oracle.np_forward(x, w, tb.indices)
    np.testing.assert_allclose(out.astype(np.float32), ref, rtol=2e-3, atol=2e-3)
    din = oracle.mask_igemm(dout, w, np.zeros((tb.n_in, C), np.float16), tb.indices_bwd, tb.mask_bwd,
                            tb.mask_argsort_bwd, is_dgrad=True)
    np.testing.assert_allclose(din.astype(np.float32), oracle.np_dgrad(dout, w, tb.indices, tb.n_in),
                               rtol=2e-3, atol=2e-3)
    # submanifold: the forward masks and their sort serve the input gradient when the tile mask
    # is bit-reversed (the harness does this, cumm/conv/main_real_spconv.py:284-285)
    din2 = oracle.mask_igemm(dout, w, np.zeros((tb.n_in, C), np.float16), tb.indices_bwd, tb.mask,
                             tb.mask_argsort, is_dgrad=True, reverse_mask=True)
    np.testing.assert_allclose(din2.astype(np.float32), din.astype(np.float32), rtol=2e-3, atol=2e-3)
    dw = oracle.mask_igemm_wgrad(dout, x, np.zeros((K, kv, C), np.float16), tb.indices, mo, tb.mask_argsort)
    np.testing.assert_allclose(dw.astype(np.float32), oracle.np_wgrad(dout, x, tb.indices), rtol=5e-3, atol=5e-3)
    # int8: exact accumulators through float64 BLAS, then the separate epilogue
    x8 = rng.integers(-127, 128, (tb.n_in, 32)).astype(np.int8)
    w8 = rng.integers(-127, 128, (16, kv, 32)).astype(np.int8)
    scale = rng.uniform(1e-3, 1e-2, 16).astype(np.float32)
    bias = rng.standard_normal(16).astype(np.float32)
    o8 = oracle.mask_igemm_s8(x8, w8, np.zeros((tb.n_out, 16), np.int8), scale, bias, tb.indices, tb.mask,
                              tb.mask_argsort)
    acc = oracle.np_forward_s8_acc(x8, w8, tb.indices)
    assert (o8 == oracle.requant_s8(acc, scale, bias)).all()


def test_gather_gemm_oracle(oracle):
    rng = np.random.default_rng(9)
    a = rng.standard_normal((300, 16)).astype(np.float16)
    b = rng.standard_normal((24, 16)).astype(np.float16)
    ai = rng.permutation(300)[:200].astype(np.int32)
    ci = rng.permutation(250)[:200].astype(np.int32)
    c = np.zeros((250, 24), np.float16)
    oracle.gemm_shuffle_ac(a, b, c, ai, ci)
    want = np.zeros((250, 24), np.float32)
    want[ci] = a[ai].astype(np.float32) @ b.T.astype(np.float32)
    np.testing.assert_allclose(c.astype(np.float32), want, rtol=2e-3, atol=2e-3)
    a2 = rng.standard_normal((300, 24)).astype(np.float16)
    bi = rng.permutation(300)[:200].astype(np.int32)
    c2 = oracle.gemm_shuffle_ab(a2, a, np.zeros((24, 16), np.float16), ai, bi)
    want2 = a2[ai].astype(np.float32).T @ a[bi].astype(np.float32)
    np.testing.assert_allclose(c2.astype(np.float32), want2, rtol=5e-3, atol=5e-2)


def test_contract_mirror_matches_reference(oracle):
    """GemmAlgoDesp / ConvAlgoDesp of the package reproduce the reference's name strings,
    supported(), workspace sizes, mnk and tile counts (golden values from its headers)."""
    from cumm_b200.tensorview.gemm import (ConvAlgoDesp, GemmAlgoDesp, ShuffleStrideType,
                                           get_spconv_logical_tile_count, implicit_gemm_mnk)
    recs = json.loads((GOLD / "contract.json").read_text())
    assert len(recs) >= 20
    for rec in recs:
        f = rec["fields"]

        def fill(d):
            d.dtype_a, d.dtype_b, d.dtype_c, d.dacc, d.dcomp = f["dtype_a"], f["dtype_b"], f["dtype_c"], f["dacc"], f["dcomp"]
            d.trans_a, d.trans_b, d.trans_c = bool(f["trans_a"]), bool(f["trans_b"]), bool(f["trans_c"])
            d.tile_shape, d.warp_tile_shape, d.tensorop = list(f["tile_shape"]), list(f["warp_tile_shape"]), list(f["tensorop"])
            d.num_stage = f["num_stage"]
            d.split_k_serial, d.split_k_parallel = bool(f["split_k_serial"]), bool(f["split_k_parallel"])
            d.shuffle_type = ShuffleStrideType(f["shuffle_type"])
            d.element_per_access_a, d.element_per_access_b, d.element_per_access_c = f["epa_a"], f["epa_b"], f["epa_c"]
            d.access_per_vector = f["access_per_vector"]
            d.algo = f["algo"]
            return d

        g = fill(GemmAlgoDesp())
        c = fill(ConvAlgoDesp(f["ndim"], f["op_type"]))
        c.mask_sparse, c.increment_k_first = bool(f["mask_sparse"]), bool(f["increment_k_first"])
        c.dynamic_mask, c.is_int8_inference = bool(f["dynamic_mask"]), bool(f["is_int8_inference"])
        assert repr(g) == rec["gemm_repr"]
        assert repr(c) == rec["conv_repr"]
        for pr in rec["probes"]:
            mnk = implicit_gemm_mnk(f["op_type"], pr["N"], pr["C"], pr["K"], pr["kv"])
            assert list(mnk) == pr["mnk"]
            m, n, k = mnk
            tiles = get_spconv_logical_tile_count(m, n, k, f["tile_shape"][0], f["tile_shape"][1], pr["split_k"],
                                                  pr["kv"], f["op_type"])
            assert list(tiles) == pr["tiles"]
            assert int(g.supported(m, n, k)) == pr["gemm_supported"]
            assert int(c.supported(m, n, k, pr["C"], pr["K"], pr["mask_width"])) == pr["conv_supported"]
            if "gemm_workspace" in pr:
                # the reference computes these in 32-bit int and wraps for split-k-parallel at
                # full size; the mirror returns the true byte count, so compare below 2^31 only
                gw = g.query_workspace_size(m, n, k, pr["split_k"])
                cw = c.query_conv_workspace_size(m, n, k, pr["split_k"], pr["kv"])
                if gw < 2 ** 31:
                    assert gw == pr["gemm_workspace"]
                if cw < 2 ** 31:
                    assert cw == pr["conv_workspace"]
