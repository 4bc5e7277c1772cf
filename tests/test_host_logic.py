"""Host-side logic that needs no GPU: the operator mirror's validation (the reference's
prologue checks), shape extraction, the C-ABI library's exported symbols, kernel tables."""
import ctypes
import re
from pathlib import Path

import numpy as np
import pytest

import helpers as H
from cumm_b200 import _lib
from cumm_b200 import tensorview as tv
from cumm_b200.conv.main import ConvMainUnitTest
from cumm_b200.gemm.main import GemmMainUnitTest
from cumm_b200.tensorview.gemm import (Activation, ConvAlgoDesp, ConvOpType, ConvParams, GemmAlgoDesp, GemmParams,
                                       ShuffleStrideType, _conv_args, _gemm_args)

ROOT = Path(__file__).resolve().parent.parent


def fake(shape, dtype, ptr=0x7f0000001000):
    """A device-tensor stand-in: shapes and dtypes are all the host logic looks at."""
    return tv.from_blob(ptr, shape, dtype, 0)


def test_library_exports_every_declared_symbol():
    header = (ROOT / "include" / "cumm_b200.h").read_text()
    declared = set(re.findall(r"\b(cb2_[a-z0-9_]+)\s*\(", header))
    assert declared, "no declarations found"
    L = ctypes.CDLL(str(_lib.LIB_PATH))
    for name in sorted(declared):
        assert hasattr(L, name), f"{name} declared in include/cumm_b200.h but not exported"
    assert declared >= set(_lib.EXPORTED_SYMBOLS)
    assert L.cb2_tile_m() == 128


def test_struct_layout_matches_header_field_order():
    header = (ROOT / "include" / "cumm_b200.h").read_text()
    for cname, cls in (("cb2_gemm_args", _lib.GemmArgs), ("cb2_conv_args", _lib.ConvArgs),
                       ("cb2_pairgen_args", _lib.PairgenArgs), ("cb2_peer_allreduce_args", _lib.PeerAllreduceArgs)):
        body = header[header.index("typedef struct " + cname):header.index("} " + cname)]
        body = re.sub(r"/\*.*?\*/", "", body, flags=re.S)
        names = []
        for decl in body.split("{", 1)[1].split(";"):
            decl = decl.strip()
            if not decl:
                continue
            for part in decl.split(","):
                names.append(re.findall(r"[A-Za-z_][A-Za-z0-9_]*", part)[-1])
        assert names == [f[0] for f in cls._fields_], cname


def test_desp_validation_errors():
    d = GemmAlgoDesp()
    with pytest.raises(RuntimeError, match="trans_a, trans_b, trans_c and algo must be set"):
        d.check_valid()
    d = H.gemm_desp(ShuffleStrideType.ShuffleAC)
    d.tensorop = [-1, -1, -1]
    with pytest.raises(RuntimeError, match="tensorop must be set"):
        d.check_valid()
    d = H.gemm_desp(ShuffleStrideType.ShuffleAC)
    d.num_stage = 0
    with pytest.raises(RuntimeError, match="num_stage"):
        repr(d)
    d = H.gemm_desp(ShuffleStrideType.ShuffleAC)
    d2 = d.copy()
    d2.tile_shape[0] = 7
    assert d.tile_shape[0] == 128
    assert d.supported(100, 64, 64) and not d.supported(100, 64, 60)


def test_gemm_params_checks_follow_reference():
    p = GemmParams()
    p.algo_desp = H.gemm_desp(ShuffleStrideType.ShuffleAC)
    with pytest.raises(RuntimeError, match="a,b,c must not empty"):
        p.check_valid()
    p.a = fake([100, 64], tv.float16)
    p.b = fake([32, 64], tv.float16)
    p.c = fake([200, 32], tv.float16)
    assert p.algo_desp.dtype_a == tv.float16
    with pytest.raises(RuntimeError, match="a_inds,c_inds tensor must not empty"):
        p.check_valid()
    p.a_inds = fake([50], tv.int32)
    p.c_inds = fake([50], tv.int32)
    args = _gemm_args(p)
    assert (args.m, args.n, args.k) == (50, 32, 64)
    assert (args.stride_A, args.stride_B, args.stride_C) == (64, 64, 32)
    assert args.rows_A == 100
    # d of another dtype is refused (params.h:381-385)
    with pytest.raises(RuntimeError, match="d dtype must equal to c"):
        p.d = fake([200, 32], tv.float32)
    # a bias vector must have n entries
    p.d = fake([31], tv.float16)
    with pytest.raises(RuntimeError, match="valid bias"):
        _gemm_args(p)
    p.d = fake([32], tv.float16)
    assert _gemm_args(p).d_is_vector == 1
    # misaligned contiguous dim -> invalid argument
    p.b = fake([32, 60], tv.float16)
    p.a = fake([100, 60], tv.float16)
    with pytest.raises(ValueError, match="misaligned"):
        _gemm_args(p)
    # ShuffleAB needs trans_a and !trans_b
    q = GemmParams()
    q.algo_desp = H.gemm_desp(ShuffleStrideType.ShuffleAB, trans_a=False, trans_b=False)
    q.a, q.b, q.c = fake([100, 64], tv.float16), fake([100, 32], tv.float16), fake([64, 32], tv.float16)
    q.a_inds, q.b_inds = fake([70], tv.int32), fake([70], tv.int32)
    with pytest.raises(RuntimeError, match="shuffle AB must be nt"):
        _gemm_args(q)
    q.algo_desp.trans_a = True
    a = _gemm_args(q)
    assert (a.m, a.n, a.k) == (64, 32, 70)


def conv_params(op, N=1000, n_in=1000, C=64, K=32, kv=27, int8=False):
    p = ConvParams(3, op)
    p.conv_algo_desp = H.conv_desp(op, C, K, int8_inference=int8)
    dt = tv.int8 if int8 else tv.float16
    p.input = fake([n_in, C], dt)
    p.weight = fake([K, kv, C], dt)
    p.output = fake([N, K], dt)
    rows = n_in if op == ConvOpType.BackwardInput else N
    p.indices = fake([kv, rows], tv.int32)
    p.mask = fake([rows], tv.uint32)
    p.mask_argsort = fake([rows], tv.int32)
    return p


def test_conv_args_role_mapping_and_checks():
    p = conv_params(ConvOpType.Forward)
    a = _conv_args(p)
    assert (a.N, a.C, a.K, a.kernel_volume) == (1000, 64, 32, 27)
    assert a.ptr_A == p.input.data_ptr() and a.ptr_B == p.weight.data_ptr() and a.ptr_C == p.output.data_ptr()
    assert a.ptr_D == p.output.data_ptr() and a.d_is_bias == 0
    p.bias = fake([32], tv.float16, 0x7f0000009000)
    a = _conv_args(p)
    assert a.ptr_D == 0x7f0000009000 and a.d_is_bias == 1
    p.output_add = fake([1000, 32], tv.float16)
    with pytest.raises(ValueError, match="only int8 inference support output_add"):
        _conv_args(p)
    # backward input: a = dout, c = din; N comes from the table and must match input rows
    p = conv_params(ConvOpType.BackwardInput, N=900, n_in=1000)
    a = _conv_args(p)
    assert a.ptr_A == p.output.data_ptr() and a.ptr_C == p.input.data_ptr() and a.N == 1000 and a.rows_A == 900
    p.indices = fake([27, 999], tv.int32)
    with pytest.raises(RuntimeError, match="input.dim"):
        _conv_args(p)
    # backward weight: needs mask_width, a = dout, b = input, c = dW
    p = conv_params(ConvOpType.BackwardWeight)
    with pytest.raises(RuntimeError, match="mask_width"):
        _conv_args(p)
    p.mask_width = 128
    p.split_k_slices = 32
    a = _conv_args(p)
    assert a.ptr_A == p.output.data_ptr() and a.ptr_B == p.input.data_ptr() and a.ptr_C == p.weight.data_ptr()
    # int8 needs scale and bias
    p = conv_params(ConvOpType.Forward, C=64, K=32, int8=True)
    with pytest.raises(RuntimeError, match="both scale and bias"):
        _conv_args(p)
    p.scale, p.bias = fake([32], tv.float32), fake([32], tv.float32)
    a = _conv_args(p)
    assert a.is_int8_inference == 1 and a.d_is_bias == 0
    # missing tables
    p = conv_params(ConvOpType.Forward)
    p.mask = None
    with pytest.raises(RuntimeError, match="mask empty"):
        _conv_args(p)
    # split-k on an algo without it
    p = conv_params(ConvOpType.Forward)
    p.split_k_slices = 4
    with pytest.raises(RuntimeError, match="splitk"):
        _conv_args(p)
    # misaligned channels
    p = conv_params(ConvOpType.Forward, C=60)
    with pytest.raises(RuntimeError, match="not supported"):
        _conv_args(p)


def test_kernel_tables_and_static_helpers():
    gd = GemmMainUnitTest.get_all_algo_desp()
    cd = ConvMainUnitTest.get_all_conv_algo_desp()
    assert len({repr(d) for d in gd}) == len(gd) and len({repr(d) for d in cd}) == len(cd)
    assert all(d.algo == "Blackwell" and d.min_arch == (10, 0) for d in gd + cd)
    assert any(d.is_int8_inference for d in cd) and any(d.op_type == ConvOpType.BackwardWeight for d in cd)
    assert GemmMainUnitTest.extract_mnk([100, 64], [32, 64], False, True, False, 1, [50], [], [50]) == (50, 32, 64)
    assert GemmMainUnitTest.extract_mnk([100, 64], [100, 32], True, False, False, 2, [70], [70]) == (64, 32, 70)
    assert GemmMainUnitTest.extract_mnk([128, 64], [64, 128], False, False, False) == (128, 128, 64)
    assert ConvMainUnitTest.extract_mnk(2, 150000, 128, 128, 27) == (128, 3456, 150000)
    assert [GemmMainUnitTest.align_to_power2(v) for v in (1, 2, 3, 8, 9, 1000)] == [1, 2, 4, 8, 16, 1024]
    table = {64 | (64 << 20) | (32 << 40): [3], 128 | (128 << 20) | (32 << 40): [5, 6]}
    pick = GemmMainUnitTest.simple_select_tile_shape
    assert pick(100, 100, 20, [32, 64, 128], [64, 128], [32], table, False) == [5, 6]
    assert pick(50, 50, 20, [32, 64, 128], [64, 128], [32], table, True) == [3]
    assert pick(10, 10, 10, [32], [32], [8], table, False) == []


def test_missing_library_fails_loudly(monkeypatch, tmp_path):
    monkeypatch.setattr(_lib, "_lib", None)
    monkeypatch.setattr(_lib, "LIB_PATH", tmp_path / "nope.so")
    with pytest.raises(RuntimeError, match="no CPU fallback"):
        _lib.load()


def test_table_builder_workspace_size_is_a_host_function():
    """cb2_pairgen_workspace_size needs no GPU: geometry checks and the size arithmetic only."""
    L = ctypes.CDLL(str(_lib.LIB_PATH))
    L.cb2_pairgen_workspace_size.restype = ctypes.c_size_t
    L.cb2_pairgen_workspace_size.argtypes = [ctypes.POINTER(_lib.PairgenArgs)]

    def size(n_in, subm, stride=(1, 1, 1), ksize=(3, 3, 3), grid=(41, 1600, 1408), batch=1):
        a = _lib.PairgenArgs()
        a.n_in, a.batch_size, a.subm = n_in, batch, int(subm)
        for name, vals in (("grid", grid), ("ksize", ksize), ("stride", stride), ("pad", (1, 1, 1)), ("dil", (1, 1, 1))):
            for i in range(3):
                getattr(a, name)[i] = vals[i]
        return L.cb2_pairgen_workspace_size(ctypes.byref(a))

    s1, s2 = size(150000, True), size(300000, True)
    assert 0 < s1 < s2
    assert size(150000, False, stride=(2, 2, 2)) > s1  # the strided case also holds the output set and lists
    assert size(150000, True, stride=(2, 2, 2)) == 0   # a submanifold convolution has stride 1
    assert size(150000, True, ksize=(3, 3, 5)) > size(150000, True)   # kernel volume 45: two mask words per row
    assert size(150000, True, ksize=(5, 5, 6)) == 0    # kernel volume 150 > 128
    assert size(150000, True, grid=(0, 10, 10)) == 0
    assert size(150000, True, batch=0) == 0


def test_peer_allreduce_buffer_size_is_a_host_function():
    L = ctypes.CDLL(str(_lib.LIB_PATH))
    L.cb2_peer_allreduce_buffer_size.restype = ctypes.c_size_t
    L.cb2_peer_allreduce_buffer_size.argtypes = [ctypes.c_longlong, ctypes.c_int]
    numel = 128 * 27 * 128
    # control block, then per call parity: one receive slot per GPU of one shard each, and one result array;
    # every float travels beside a copy of the call number (8 bytes per float)
    one = L.cb2_peer_allreduce_buffer_size(numel, 1)
    assert one == 8192 + 2 * numel * 8 + 2 * numel * 8
    shard = numel * 8 // 8
    assert shard % 256 == 0
    assert L.cb2_peer_allreduce_buffer_size(numel, 8) == 8192 + 2 * 8 * shard + 2 * numel * 8
    assert L.cb2_peer_allreduce_buffer_size(numel + 2, 8) == 0  # not a multiple of 4
    assert L.cb2_peer_allreduce_buffer_size(numel, 17) == 0
    assert L.cb2_peer_allreduce_buffer_size(0, 2) == 0


def test_kernel_table_comes_from_the_library():
    """get_all_algo_desp / get_all_conv_algo_desp read cb2_enumerate_*_desps (no GPU needed)."""
    from cumm_b200.conv.main import ConvMainUnitTest
    from cumm_b200.gemm.main import GemmMainUnitTest
    from cumm_b200.tensorview.gemm import ConvOpType, ShuffleStrideType
    L = ctypes.CDLL(str(_lib.LIB_PATH))
    for fn in (L.cb2_enumerate_gemm_desps, L.cb2_enumerate_conv_desps):
        fn.restype = ctypes.c_int
        fn.argtypes = [ctypes.POINTER(_lib.KernelDesp), ctypes.c_int]
    assert L.cb2_enumerate_gemm_desps(None, 0) == 18 and L.cb2_enumerate_conv_desps(None, 0) == 24
    two = (_lib.KernelDesp * 2)()
    assert L.cb2_enumerate_conv_desps(two, 2) == 24  # the count, whatever the capacity
    assert two[0].op_type == 0 and list(two[0].tile_shape) == [128, 64, 64] and two[1].tile_shape[2] == 128
    gemm = GemmMainUnitTest.get_all_algo_desp()
    conv = ConvMainUnitTest.get_all_conv_algo_desp()
    assert len(gemm) == 18 and len(conv) == 24
    assert sum(d.shuffle_type == ShuffleStrideType.ShuffleAB for d in gemm) == 2
    assert all(d.trans_a and not d.trans_b and d.split_k_serial for d in gemm if d.shuffle_type == ShuffleStrideType.ShuffleAB)
    assert sum(bool(d.is_int8_inference) for d in conv) == 4 and sum(bool(d.dynamic_mask) for d in conv) == 12
    assert {tuple(d.tile_shape) for d in conv if d.op_type == ConvOpType.BackwardWeight} == {(128, 64, 128), (128, 128, 128)}
    names = {d.__repr__() for d in conv} | {d.__repr__() for d in gemm}
    assert len(names) == 42, "every variant has its own algorithm name"
    assert all(n.startswith("Blackwell_") for n in names)


def test_nvrtc_entry_points_throw_without_a_module(monkeypatch):
    """cumm/tensorview_bind.py:147-149,164-166: run_nvrtc_* need a run-time-compiled kernel."""
    import cumm_b200.tensorview.gemm as G
    monkeypatch.delenv("CUMM_B200_NVRTC_USES_PREBUILT", raising=False)
    with pytest.raises(RuntimeError, match="you must use nvrtc kernel to run conv"):
        G._nvrtc_gate(G.NVRTCParams(), "conv")
    with pytest.raises(RuntimeError, match="you must use nvrtc kernel to run gemm"):
        G._nvrtc_gate(G.NVRTCParams(), "gemm")
    p = G.NVRTCParams()
    p.cumodule = object()
    with pytest.raises(RuntimeError, match="not loaded by this library"):
        G._nvrtc_gate(p, "gemm")
    monkeypatch.setattr(G, "NVRTC_ENTRY_POINTS_USE_PREBUILT", True)
    G._nvrtc_gate(G.NVRTCParams(), "conv")  # opted in: no error


def test_kernel_timer_names_follow_the_namespace_stack():
    """tv::CUDAKernelTimer naming rules (cuda_profiler.h:225-300), without touching a GPU."""
    from cumm_b200.tensorview import CUDAKernelTimer
    t = CUDAKernelTimer(True)
    t.push("layer1")
    t.push("Blackwell_x")
    assert t._unique("start") == "layer1.Blackwell_x.start" and t._unique("") == "layer1.Blackwell_x"
    name = t.insert_pair("", "start", "stop")
    assert name == "layer1.Blackwell_x" and t.has_pair("")
    with pytest.raises(RuntimeError, match="already exists"):
        t.insert_pair("", "start", "stop")
    t.pop()
    t.pop()
    with pytest.raises(RuntimeError, match="empty namespaces"):
        t.pop()
    off = CUDAKernelTimer(False)
    off.push("x")
    off.record("start")
    assert off.insert_pair("", "a", "b") == "" and off._events == {}
