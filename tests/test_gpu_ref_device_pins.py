"""Pins the oracle's two output operators to the reference's own device code.

``oracle/_ref/libref_device.so`` (built by ``make -C oracle ref`` from ``oracle/ref_device_shim.cu``)
instantiates the reference's epilogue functors -- ``multiply_add``, ``multiplies``, ``maximum`` and
the ``NumericArrayConverter`` chain int32 -> float -> int8 / float -> half -- in the order
cumm/gemm/output_op/linear.py:105-144 and :279-360 prescribe, as sm_100a device code.  Here it runs
on the GPU over more than a million random and edge inputs and the C oracle's restatement
(``orc_requant_s8``, ``orc_lincomb_f16``) must agree bit for bit.  The shipped library is not
involved: this checks the checker."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def refdev(cuda_lib, oracle):
    R = oracle.ref_device_lib()
    if R is None:
        pytest.skip("oracle/_ref/libref_device.so was not built (the reference tree was absent at build time)")
    return R


def _ptr(a, typ):
    import ctypes
    return None if a is None else a.ctypes.data_as(typ)


def ref_requant(R, oracle, acc, scale, bias, beta, src, act):
    out = np.empty(acc.shape, np.int8)
    rc = R.ref_dev_requant_s8(acc.size, acc.shape[1], _ptr(acc, oracle.c_i32p), _ptr(scale, oracle.c_f32p),
                              _ptr(bias, oracle.c_f32p), float(beta), _ptr(src, oracle.c_i8p), int(act),
                              _ptr(out, oracle.c_i8p))
    assert rc == 0, f"reference device shim failed with code {rc}"
    return out


def test_int8_requant_matches_reference_device_code(refdev, oracle):
    rng = np.random.default_rng(11)
    K = 128
    rows = 8192 + 64  # > 10^6 elements
    acc = rng.integers(-60_000_000, 60_000_000, (rows, K)).astype(np.int32)  # beyond 2^24: the int->float step rounds
    acc[:2048] = rng.integers(-200_000, 200_000, (2048, K))                   # the usual magnitude
    scale = rng.uniform(1e-3, 1e-2, K).astype(np.float32)
    bias = rng.standard_normal(K).astype(np.float32)
    # rows of edge cases
    e = 8192
    scale_e = scale.copy()
    acc[e:e + 8] = np.arange(-4 * K, 4 * K).reshape(8, K) * 2 + 1             # odd numbers: x.5 ties under scale 0.5
    acc[e + 8] = 2**24 + np.arange(K)                                         # first integers floats cannot hold
    acc[e + 9] = -(2**24) - np.arange(K)
    acc[e + 10] = np.iinfo(np.int32).max - np.arange(K)
    acc[e + 11] = np.iinfo(np.int32).min + np.arange(K)
    acc[e + 12:e + 16] = rng.integers(-300, 300, (4, K))                      # around the saturation bounds
    got_parts, want_parts = [], []
    # (a) plain, (b) ReLU, (c) with an int8 source and beta
    src = rng.integers(-128, 128, (rows, K)).astype(np.int8)
    for beta, s, act in ((0.0, None, 0), (0.0, None, 1), (0.75, src, 0), (-1.5, src, 1)):
        got_parts.append(ref_requant(refdev, oracle, acc, scale, bias, beta, s, act))
        want_parts.append(oracle.requant_s8(acc, scale, bias, beta=beta, src=s, act_type=act))
    # (d) ties: scale 0.5, bias 0 -> every odd accumulator lands on x.5
    half = np.full(K, 0.5, np.float32)
    zero = np.zeros(K, np.float32)
    got_parts.append(ref_requant(refdev, oracle, acc[e:e + 16], half, zero, 0.0, None, 0))
    want_parts.append(oracle.requant_s8(acc[e:e + 16], half, zero))
    # (e) unit scale: saturation at -128 / 127 exactly
    one = np.ones(K, np.float32)
    got_parts.append(ref_requant(refdev, oracle, acc[e + 12:e + 16], one, zero, 0.0, None, 0))
    want_parts.append(oracle.requant_s8(acc[e + 12:e + 16], one, zero))
    # (f) NaN and infinite scales / biases: NaN -> 0, +-inf saturate
    scale_e[:8] = [np.nan, np.inf, -np.inf, 0.0, 1e30, -1e30, 1e-30, np.nan]
    bias_e = bias.copy()
    bias_e[8:12] = [np.nan, np.inf, -np.inf, 1e20]
    got_parts.append(ref_requant(refdev, oracle, acc[:64], scale_e, bias_e, 0.0, None, 0))
    want_parts.append(oracle.requant_s8(acc[:64], scale_e, bias_e))
    n = 0
    for i, (g, w) in enumerate(zip(got_parts, want_parts)):
        bad = np.nonzero(g != w)
        assert len(bad[0]) == 0, (f"case {i}: {len(bad[0])} of {g.size} int8 outputs differ from the reference's device "
                                  f"code; first at {bad[0][0]},{bad[1][0]}: reference {g[bad][0]}, oracle {w[bad][0]}")
        n += g.size
    assert n > 4_000_000


def test_fp16_linear_combination_matches_reference_device_code(refdev, oracle):
    import ctypes
    rng = np.random.default_rng(12)
    n = 1 << 20
    acc = (rng.standard_normal(n) * np.exp(rng.uniform(-18, 12, n))).astype(np.float32)  # subnormal halves to overflow
    acc[:4096] = np.arange(4096, dtype=np.float32) * 0.25 + 2048.0                          # exact ties at 2048..3072
    acc[4096:4104] = [0.0, -0.0, 65504.0, 65520.0, -65520.0, 6e-8, 2.98e-8, 1e-10]
    src = (rng.standard_normal(n) * 4).astype(np.float16)
    c_u16p = oracle.c_u16p

    def ref(alpha, beta, s, act):
        out = np.empty(n, np.uint16)
        rc = refdev.ref_dev_lincomb_f16(n, _ptr(acc, oracle.c_f32p), float(alpha), float(beta),
                                        None if s is None else _ptr(s.view(np.uint16), c_u16p), int(act),
                                        _ptr(out, c_u16p))
        assert rc == 0, f"reference device shim failed with code {rc}"
        return out

    for alpha, beta, s, act in ((1.0, 0.0, None, 0), (0.37, 0.0, None, 1), (1.0, 1.0, src, 0), (0.5, -0.25, src, 1)):
        got = ref(alpha, beta, s, act)
        want = oracle.lincomb_f16(acc, alpha, beta, s, act_type=act).view(np.uint16)
        bad = np.nonzero(got != want)[0]
        assert len(bad) == 0, (f"alpha={alpha} beta={beta} act={act}: {len(bad)} of {n} fp16 outputs differ; first at "
                               f"{bad[0]}: acc={acc[bad[0]]!r} reference 0x{got[bad[0]]:04x} oracle 0x{want[bad[0]]:04x}")
