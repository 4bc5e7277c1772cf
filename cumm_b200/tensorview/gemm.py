"""Operator surface of the sparse-conv hot path: the names exported by the reference's
``cumm.tensorview.gemm`` (cumm/tensorview/gemm.py:15-20) with the fields, defaults and
checks of ``include/tensorview/gemm/core/params.h``.

    GemmAlgoDesp, ConvAlgoDesp      kernel selector records       params.h:24-164, 166-327
    GemmParams, ConvParams          per-call argument records     params.h:329-390, 392-428
    ConvOpType, ShuffleStrideType, Activation, ConvMode, ConvIterAlgo, ConvLayoutType
                                    include/tensorview/gemm/core/constants.h:18-56
    run_nvrtc_gemm_kernel, run_nvrtc_conv_kernel
                                    cumm/tensorview_bind.py:134-167

The reference's kernels are generated per descriptor; here a descriptor is matched to one of
a small set of hand-written sm_100a kernels (algo name ``"Blackwell"``), and a descriptor no
kernel fits raises ``RuntimeError`` exactly like the reference's "can't find any suitable
algo" (cumm/gemm/main.py:1323-1333).  There is no CPU path.
"""
from __future__ import annotations

import ctypes
import enum
from typing import List, Optional, Tuple

from . import as_view, dtype_short_str, itemsize, unknown
from .. import _lib


class ConvOpType(enum.IntEnum):
    Forward = 0
    BackwardInput = 1
    BackwardWeight = 2
    # C++ spellings
    kForward = 0
    kBackwardInput = 1
    kBackwardWeight = 2


class ConvMode(enum.IntEnum):
    Convolution = 0
    CrossCorrelation = 1


class ConvIterAlgo(enum.IntEnum):
    Analytic = 0
    Optimized = 1


class ConvLayoutType(enum.IntEnum):
    ChannelFirst = 0
    ChannelLast = 1
    SpatialFirst = 2


class ShuffleStrideType(enum.IntEnum):
    NoShuffle = 0
    ShuffleAC = 1
    ShuffleAB = 2


class Activation(enum.IntEnum):
    None_ = 0
    ReLU = 1
    Sigmoid = 2
    LeakyReLU = 3


class NVRTCParams:
    """Placeholder for the reference's run-time-compiled kernel handle
    (include/tensorview/gemm/core/nvrtc_bases.h:21-32).  Kernels here are prebuilt, so the
    record only keeps the fields for interface compatibility."""

    def __init__(self):
        self.cumodule = None
        self.kernel_name = ""
        self.init_kernel_name = ""
        self.constant_name = ""
        self.param_size = -1
        self.param_storage = None
        self.param_storage_cpu = None
        self.num_threads = -1
        self.smem_size = -1
        self.mode = 0


def _div_up(a: int, b: int) -> int:
    return (a + b - 1) // b


class GemmAlgoDesp:
    """params.h:24-164."""

    def __init__(self):
        self.dtype_a = unknown
        self.dtype_b = unknown
        self.dtype_c = unknown
        self.trans_a_ = -1
        self.trans_b_ = -1
        self.trans_c_ = -1
        self.tile_shape = [-1, -1, -1]
        self.warp_tile_shape = [-1, -1, -1]
        self.num_stage = -1
        self.dacc = unknown
        self.dcomp = unknown
        self.algo = ""
        self.tensorop = [-1, -1, -1]
        self.split_k_serial_ = 0
        self.split_k_parallel_ = 0
        self.shuffle_type = ShuffleStrideType.NoShuffle
        self.element_per_access_a = -1
        self.element_per_access_b = -1
        self.element_per_access_c = -1
        self.access_per_vector = 1
        self.is_nvrtc = False
        self.min_arch = (0, 0)

    # bool properties over int storage (cumm/tensorview_bind.py:233-310)
    @property
    def trans_a(self) -> bool:
        return self.trans_a_ == 1

    @trans_a.setter
    def trans_a(self, v: bool):
        self.trans_a_ = 1 if v else 0

    @property
    def trans_b(self) -> bool:
        return self.trans_b_ == 1

    @trans_b.setter
    def trans_b(self, v: bool):
        self.trans_b_ = 1 if v else 0

    @property
    def trans_c(self) -> bool:
        return self.trans_c_ == 1

    @trans_c.setter
    def trans_c(self, v: bool):
        self.trans_c_ = 1 if v else 0

    @property
    def split_k_serial(self) -> bool:
        return self.split_k_serial_ == 1

    @split_k_serial.setter
    def split_k_serial(self, v: bool):
        self.split_k_serial_ = 1 if v else 0

    @property
    def split_k_parallel(self) -> bool:
        return self.split_k_parallel_ == 1

    @split_k_parallel.setter
    def split_k_parallel(self, v: bool):
        self.split_k_parallel_ = 1 if v else 0

    def check_valid(self) -> None:
        """params.h:83-108."""
        if self.trans_a_ == -1 or self.trans_b_ == -1 or self.trans_c_ == -1 or not self.algo:
            raise RuntimeError("trans_a, trans_b, trans_c and algo must be set")
        for i in range(3):
            if not (self.tile_shape[i] > 0 and self.warp_tile_shape[i] > 0):
                raise RuntimeError("tile_shape and warp_tile_shape must be set, but they are "
                                   f"{list(self.tile_shape)} {list(self.warp_tile_shape)}")
        if self.algo not in ("Simt", "SimtDP4A", "SimtDP2A"):
            for i in range(3):
                if not self.tensorop[i] > 0:
                    raise RuntimeError(f"tensorop must be set, but they are {list(self.tensorop)}")
        if unknown in (self.dtype_a, self.dtype_b, self.dtype_c):
            raise RuntimeError("dacc and dcomp must be set to valid value")
        if unknown in (self.dacc, self.dcomp):
            raise RuntimeError("dacc and dcomp must be set to valid value")
        if not self.num_stage > 0:
            raise RuntimeError("num_stage must larger than zero")

    def __repr__(self) -> str:
        """Algorithm name string, params.h:56-78."""
        self.check_valid()
        s = self.algo + "_"
        s += "".join(dtype_short_str(d) for d in (self.dtype_a, self.dtype_b, self.dtype_c, self.dacc,
                                                  self.dcomp))
        s += ("n" if self.trans_a else "t") + ("n" if self.trans_b else "t") + ("n" if self.trans_c else "t")
        s += "_m{}n{}k{}".format(*self.tile_shape)
        s += "m{}n{}k{}".format(*self.warp_tile_shape)
        s += f"A{self.access_per_vector}"
        if self.tensorop[0] != -1:
            s += "T{}{}{}".format(*self.tensorop)
        s += f"_{self.num_stage}"
        s += ("1" if self.split_k_serial else "0") + ("1" if self.split_k_parallel else "0")
        if self.shuffle_type != ShuffleStrideType.NoShuffle:
            s += f"_S{int(self.shuffle_type)}"
        return s

    def copy(self):
        import copy
        return copy.deepcopy(self)

    def query_workspace_size(self, m: int, n: int, k: int, split_k_slices: int) -> int:
        """params.h:115-132 (the reference's formula, a pure function of the record)."""
        tiles = (_div_up(m, self.tile_shape[0]), _div_up(n, self.tile_shape[1]), split_k_slices)
        if split_k_slices > 1:
            if self.split_k_serial:
                return 4 * tiles[0] * tiles[1]
            if self.split_k_parallel:
                return itemsize(self.dacc) * m * n * tiles[2]
            raise ValueError("not impemented")
        return 0

    def supported(self, m: int, n: int, k: int) -> bool:
        """params.h:133-149: contiguous dims divisible by the access widths."""
        lda = m if self.trans_a else k
        ldb = k if self.trans_b else n
        ldc = m if self.trans_c else n
        return self.supported_ldx(lda, ldb, ldc)

    def supported_ldx(self, lda: int, ldb: int, ldc: int) -> bool:
        res = True
        if self.element_per_access_a > 0:
            res &= lda % self.element_per_access_a == 0
        if self.element_per_access_b > 0:
            res &= ldb % self.element_per_access_b == 0
        if self.element_per_access_c > 0:
            res &= ldc % self.element_per_access_c == 0
        return bool(res)


def conv_iwo_012_to_abc(op_type) -> List[int]:
    """include/tensorview/gemm/core/utils.h:93-106."""
    op_type = int(op_type)
    if op_type == ConvOpType.Forward:
        return [0, 1, 2]
    if op_type == ConvOpType.BackwardInput:
        return [2, 1, 0]
    if op_type == ConvOpType.BackwardWeight:
        return [1, 2, 0]
    raise RuntimeError(f"unknown op type {op_type}")


def gemm_abc_012_to_iwo(op_type) -> List[int]:
    """include/tensorview/gemm/core/utils.h:108-122."""
    op_type = int(op_type)
    if op_type == ConvOpType.Forward:
        return [0, 1, 2]
    if op_type == ConvOpType.BackwardInput:
        return [2, 1, 0]
    if op_type == ConvOpType.BackwardWeight:
        return [2, 0, 1]
    raise RuntimeError(f"unknown op type {op_type}")


def implicit_gemm_mnk(op_type, N: int, C: int, K: int, kernel_volume: int) -> Tuple[int, int, int]:
    """include/tensorview/gemm/core/utils.h:62-92, mask-sparse branch."""
    op_type = int(op_type)
    if op_type == ConvOpType.Forward:
        return (N, K, C * kernel_volume)
    if op_type == ConvOpType.BackwardInput:
        return (N, C, K * kernel_volume)
    if op_type == ConvOpType.BackwardWeight:
        return (K, C * kernel_volume, N)
    raise RuntimeError(f"unknown op type {op_type}")


def get_spconv_logical_tile_count(m, n, k, tile_m, tile_n, split_k_slices, kv, op_type):
    """include/tensorview/gemm/core/utils.h:39-60."""
    if int(op_type) == ConvOpType.BackwardWeight:
        C = n // kv
        gy = _div_up(C, tile_n) * kv
    else:
        gy = _div_up(n, tile_n)
    return (_div_up(m, tile_m), gy, split_k_slices)


class ConvAlgoDesp(GemmAlgoDesp):
    """params.h:166-327."""

    def __init__(self, ndim: int, op_type):
        super().__init__()
        self.ndim = int(ndim)
        self.op_type = ConvOpType(int(op_type))
        self.iter_algo = ConvIterAlgo.Optimized
        self.layout_i = ConvLayoutType.ChannelLast
        self.layout_w = ConvLayoutType.ChannelLast
        self.layout_o = ConvLayoutType.ChannelLast
        self.interleave_i = 1
        self.interleave_w = 1
        self.interleave_o = 1
        self.mask_sparse = False
        self.increment_k_first = False
        self.dynamic_mask = False
        self.is_int8_inference = False
        self.conv2gemm_inds = conv_iwo_012_to_abc(op_type)
        self.gemm2conv_inds = gemm_abc_012_to_iwo(op_type)

    conv_iwo_012_to_abc = staticmethod(conv_iwo_012_to_abc)
    gemm_abc_012_to_iwo = staticmethod(gemm_abc_012_to_iwo)

    def __repr__(self) -> str:
        """params.h:191-224."""
        s = GemmAlgoDesp.__repr__(self)
        s += f"_C{self.ndim}{int(self.op_type)}{int(self.iter_algo)}"

        def lay(l, inter):
            t = "F" if l == ConvLayoutType.ChannelFirst else "L"
            return t + (str(inter) if inter > 1 else "")

        s += lay(self.layout_i, self.interleave_i) + lay(self.layout_w, self.interleave_w) + \
            lay(self.layout_o, self.interleave_o)
        if self.mask_sparse:
            s += "_" + ("SK" if self.increment_k_first else "SF")
        if self.dynamic_mask:
            s += "D"
        if self.is_int8_inference:
            s += "_S8"
        return s

    @property
    def dtype_input(self) -> int:
        return (self.dtype_a, self.dtype_b, self.dtype_c)[self.conv2gemm_inds[0]]

    @property
    def dtype_weight(self) -> int:
        return (self.dtype_a, self.dtype_b, self.dtype_c)[self.conv2gemm_inds[1]]

    @property
    def dtype_output(self) -> int:
        return (self.dtype_a, self.dtype_b, self.dtype_c)[self.conv2gemm_inds[2]]

    def supported(self, m: int, n: int, k: int, C: Optional[int] = None, K: Optional[int] = None,
                  mask_width: int = -1) -> bool:
        """params.h:266-285."""
        res = GemmAlgoDesp.supported(self, m, n, k)
        if C is None or K is None:
            return res
        if self.mask_sparse:
            if self.op_type == ConvOpType.Forward:
                res &= C % self.element_per_access_a == 0
            elif self.op_type == ConvOpType.BackwardInput:
                res &= K % self.element_per_access_a == 0
            else:
                res &= mask_width % self.tile_shape[2] == 0
                res &= K % self.element_per_access_a == 0
                res &= C % self.element_per_access_b == 0
        return bool(res)

    def query_conv_workspace_size(self, m: int, n: int, k: int, split_k_slices: int, kv: int) -> int:
        """params.h:286-307 (the reference's formula)."""
        if not self.mask_sparse:
            return self.query_workspace_size(m, n, k, split_k_slices)
        tiles = get_spconv_logical_tile_count(m, n, k, self.tile_shape[0], self.tile_shape[1],
                                              split_k_slices, kv, self.op_type)
        if split_k_slices > 1:
            if self.split_k_serial:
                return 4 * tiles[0] * tiles[1]
            if self.split_k_parallel:
                return itemsize(self.dacc) * m * n * tiles[2]
            raise ValueError("not impemented")
        return 0

    def supported_ldx_conv(self, ldi: int, ldw: int, ldo: int) -> bool:
        """params.h:308-326."""
        epas = (self.element_per_access_a, self.element_per_access_b, self.element_per_access_c)
        res = True
        for ld, which in ((ldi, 0), (ldw, 1), (ldo, 2)):
            epa = epas[self.conv2gemm_inds[which]]
            if epa > 0:
                res &= ld % epa == 0
        return bool(res)


class GemmParams:
    """params.h:329-390.  Tensors may be ``torch.Tensor`` (CUDA) or ``tensorview.Tensor``."""

    def __init__(self, timer=None):
        self.algo_desp = GemmAlgoDesp()
        self._a = None
        self._b = None
        self._c = None
        self._d = None
        self.split_k_slices = 1
        self.workspace = None
        self.a_inds = None
        self.b_inds = None
        self.c_inds = None
        self.alpha = 1.0
        self.beta = 0.0
        self.act_alpha = 0.0  # the reference leaves these uninitialised (params.h:343-344)
        self.act_beta = 0.0
        self.act_type = Activation.None_
        self.stream = 0
        self.timer = timer
        self.nvrtc_params = NVRTCParams()
        self.max_ctas = 0  # not in the reference: see ConvParams.max_ctas

    # setters copy the dtype into the descriptor (params.h:366-388)
    @property
    def a(self):
        return self._a

    @a.setter
    def a(self, v):
        self._a = v
        t = as_view(v)
        if t is not None:
            self.algo_desp.dtype_a = t.dtype

    @property
    def b(self):
        return self._b

    @b.setter
    def b(self, v):
        self._b = v
        t = as_view(v)
        if t is not None:
            self.algo_desp.dtype_b = t.dtype

    @property
    def c(self):
        return self._c

    @c.setter
    def c(self, v):
        self._c = v
        t = as_view(v)
        if t is not None:
            self.algo_desp.dtype_c = t.dtype

    @property
    def d(self):
        return self._d

    @d.setter
    def d(self, v):
        tc, td = as_view(self._c), as_view(v)
        if tc is not None and td is not None and tc.dtype != td.dtype:
            raise RuntimeError("d dtype must equal to c")
        self._d = v

    def check_valid(self) -> None:
        """params.h:353-365."""
        self.algo_desp.check_valid()
        if as_view(self.a) is None or as_view(self.b) is None or as_view(self.c) is None:
            raise RuntimeError("a,b,c must not empty")
        if self.algo_desp.shuffle_type == ShuffleStrideType.ShuffleAC:
            if as_view(self.c_inds) is None:
                raise RuntimeError("a_inds,c_inds tensor must not empty")
        elif self.algo_desp.shuffle_type == ShuffleStrideType.ShuffleAB:
            if as_view(self.a_inds) is None or as_view(self.b_inds) is None:
                raise RuntimeError("a_inds,b_inds tensor must not empty")


class ConvParams:
    """params.h:392-428."""

    def __init__(self, ndim: int, op_type, timer=None):
        self.conv_algo_desp = ConvAlgoDesp(ndim, op_type)
        self.input = None
        self.weight = None
        self.output = None
        self.output_add = None
        self.bias = None
        self.scale = None
        self.split_k_slices = 1
        self.padding: List[int] = []
        self.stride: List[int] = []
        self.dilation: List[int] = []
        self.alpha = 1.0
        self.beta = 0.0
        self.act_alpha = 0.0
        self.act_beta = 0.0
        self.act_type = Activation.None_
        self.mask_width = -1
        self.mask_filter = 0xFFFFFFFF
        self.reverse_mask = False
        self.verbose = False
        self.mask_int_count = 1
        self.timer = timer
        self.workspace = None
        self.mask = None
        self.mask_argsort = None
        self.indices = None
        self.mask_output = None
        self.stream = 0
        self.nvrtc_params = NVRTCParams()
        # Not in the reference: upper bound on the CTAs of the launch (0 = one per SM), for calls
        # that run side by side on different streams (``cb2_conv_args.max_ctas``).
        self.max_ctas = 0


# --------------------------------------------------------------------------------------
# dispatch
# --------------------------------------------------------------------------------------
_WORKSPACES = {}


def _workspace_for(device: int, stream: int, nbytes: int, user_ws):
    """The reference's callee allocates scratch when the caller passes none
    (cumm/gemm/nvrtc_code.py:137-140).  Here a per-(device, stream) buffer is cached so no
    allocation happens on the steady-state path.  Calls on one stream that rely on it share
    the buffer; they are ordered by the stream, and the weight-gradient kernel waits for its
    predecessor before it touches the workspace, so they do not race.  Callers that run weight
    gradients on several streams at once pass their own ``workspace`` (or use
    :func:`prepare_conv`, which gives every call its own)."""
    t = as_view(user_ws)
    if t is not None and t.nbytes() >= nbytes and t.data_ptr() % 256 == 0:
        return t.data_ptr(), t.nbytes()
    if t is not None and t.nbytes() < nbytes:
        raise RuntimeError(f"workspace at least {nbytes} bytes.")
    import torch
    key = (device, stream)
    buf = _WORKSPACES.get(key)
    if buf is None or buf.numel() < nbytes:
        buf = torch.empty(nbytes, dtype=torch.uint8, device=f"cuda:{device}")
        _WORKSPACES[key] = buf
    return buf.data_ptr(), buf.numel()


def _ptr(t):
    return None if t is None else ctypes.c_void_p(t.data_ptr())


def _gemm_args(params: GemmParams) -> _lib.GemmArgs:
    """Shape extraction of the reference's GEMM prologue (cumm/gemm/nvrtc_code.py:34-146)."""
    params.check_valid()
    desp = params.algo_desp
    a, b, c = as_view(params.a), as_view(params.b), as_view(params.c)
    d = as_view(params.d)
    for t in (a, b, c):
        if t.ndim != 2:
            raise RuntimeError(f"a, b, c must be 2-D, got {t.shape}")
    if not (a.device == b.device == c.device):
        raise RuntimeError("a, b, c must be on the same device")
    ta, tb, tc = desp.trans_a, desp.trans_b, desp.trans_c
    if tc:
        ta, tb = (not tb), (not ta)
        a, b = b, a
    a_inds, b_inds, c_inds = as_view(params.a_inds), as_view(params.b_inds), as_view(params.c_inds)
    if not (desp.split_k_serial or desp.split_k_parallel) and params.split_k_slices > 1:
        raise RuntimeError("algo don't support splitk but you provide split_k_slices > 1.")
    args = _lib.GemmArgs()
    if desp.shuffle_type == ShuffleStrideType.ShuffleAC:
        if ta:
            raise RuntimeError("a of shuffle AB must be row major")
        m = a_inds.dim(0) if a_inds is not None else a.dim(0)
        k = a.dim(int(not ta))
        k2 = b.dim(int(tb))
        n = b.dim(int(not tb))
        if c.dim(1) != (m if tc else n):
            raise RuntimeError(f"c shape {c.shape} does not match [-1, {n}]")
        args.indiceA = _ptr(a_inds)
        args.indiceBorC = _ptr(c_inds)
    elif desp.shuffle_type == ShuffleStrideType.ShuffleAB:
        if not (ta and not tb):
            raise RuntimeError("shuffle AB must be nt, i.e. backward weight")
        m = a.dim(int(ta))
        k = a_inds.dim(0)
        k2 = b_inds.dim(0)
        n = b.dim(int(not tb))
        if list(c.shape) != ([n, m] if tc else [m, n]):
            raise RuntimeError(f"c shape {c.shape} does not match [{m}, {n}]")
        args.indiceA = _ptr(a_inds)
        args.indiceBorC = _ptr(b_inds)
    else:
        m = a.dim(int(ta))
        k = a.dim(int(not ta))
        k2 = b.dim(int(tb))
        n = b.dim(int(not tb))
        if list(c.shape) != ([n, m] if tc else [m, n]):
            raise RuntimeError(f"c shape {c.shape} does not match [{m}, {n}]")
    if not desp.supported(m, n, k):
        raise ValueError("this m, n, k isn't supported due to misaligned contiguous dim.")
    if k != k2:
        raise ValueError("error: k of a and b differ")
    if d is not None and d.ndim == 1 and d.dim(0) != n:
        raise RuntimeError("d must be a valid bias")
    args.m, args.n, args.k = m, n, k
    args.ptr_A, args.ptr_B, args.ptr_C = _ptr(a), _ptr(b), _ptr(c)
    args.ptr_D = _ptr(d)
    args.stride_A, args.stride_B, args.stride_C = a.stride(0), b.stride(0), c.stride(0)
    args.stride_D = 0 if (d is None or d.ndim == 1) else d.stride(0)
    args.d_is_vector = 1 if (d is not None and d.ndim == 1) else 0
    args.alpha, args.beta = float(params.alpha), float(params.beta)
    args.act_alpha, args.act_beta = float(params.act_alpha), float(params.act_beta)
    args.act_type = int(params.act_type)
    args.split_k_slices = int(params.split_k_slices)
    args.dtype_a, args.dtype_b, args.dtype_c = desp.dtype_a, desp.dtype_b, desp.dtype_c
    args.trans_a, args.trans_b, args.trans_c = int(ta), int(tb), 0
    args.shuffle_type = int(desp.shuffle_type)
    args.rows_A = a.dim(0)
    args.rows_B = b.dim(0)
    # The descriptor selects the kernel: tile_shape = [rows, columns, reduction] of one CTA tile.
    if desp.tile_shape[0] != 128:
        raise RuntimeError(f"can't find any suitable algo: tile_shape[0] = {desp.tile_shape[0]} (the sm_100a "
                           "kernels work on 128-row tiles)")
    args.tile_n = int(desp.tile_shape[1])
    args.tile_k = int(desp.tile_shape[2]) if desp.shuffle_type != ShuffleStrideType.ShuffleAB else 0
    args.max_ctas = int(getattr(params, "max_ctas", 0))
    args._device = c.device
    return args


def run_gemm(params: GemmParams) -> None:
    """What ``GemmMainUnitTest.matmul2`` does (cumm/gemm/main.py:1178-1335): validate,
    pick a kernel for the descriptor, launch on ``params.stream``."""
    L = _lib.load()
    args = _gemm_args(params)
    need = L.cb2_gemm_workspace_size(ctypes.byref(args))
    if need:
        ptr, nbytes = _workspace_for(args._device, int(params.stream), need, params.workspace)
        args.workspace, args.workspace_bytes = ptr, nbytes
    import torch
    from . import _TimerGuard
    with torch.cuda.device(args._device), _TimerGuard(params.algo_desp.__repr__(), params.timer, int(params.stream)):
        _lib.raise_for(L.cb2_gemm_run(ctypes.byref(args), ctypes.c_void_p(int(params.stream))))


def _conv_args(params: ConvParams) -> _lib.ConvArgs:
    """Shape extraction of the reference's conv prologue (cumm/conv/nvrtc_code.py:20-196)."""
    desp = params.conv_algo_desp
    desp.check_valid()
    if not desp.mask_sparse:
        raise RuntimeError("a dense convolution has no flat argument record of its own: run_conv routes it "
                           "through cumm_b200.dense")
    inp, weight, output = as_view(params.input), as_view(params.weight), as_view(params.output)
    if inp is None or weight is None or output is None:
        raise RuntimeError("input, weight, output must not empty")
    if inp.ndim != 2 or output.ndim != 2 or weight.ndim != 3:
        raise RuntimeError("error: mask-sparse conv takes 2-D input/output and 3-D [K, kv, C] weight")
    if not (desp.split_k_serial or desp.split_k_parallel) and params.split_k_slices > 1:
        raise RuntimeError("algo don't support splitk but you provide split_k_slices > 1.")
    output_add, bias, scale = as_view(params.output_add), as_view(params.bias), as_view(params.scale)
    indices, mask, mask_argsort = as_view(params.indices), as_view(params.mask), as_view(params.mask_argsort)
    mask_output = as_view(params.mask_output)
    K = weight.dim(0)
    C = inp.dim(1)
    if output.dim(1) != K:
        raise RuntimeError("error: output channels do not match the weight")
    if weight.dim(2) != C:
        raise RuntimeError("error: input channels do not match the weight")
    if not desp.is_int8_inference:
        if output_add is not None:
            raise ValueError("only int8 inference support output_add not empty ")
    else:
        if bias is None or scale is None:
            raise RuntimeError("int8 inference must have both scale and bias")
    if output_add is not None:
        if output_add.dtype != output.dtype or list(output_add.shape) != list(output.shape):
            raise RuntimeError("output and output_add must have same dtype and shape")
    op = desp.op_type
    if op == ConvOpType.BackwardWeight:
        if not (params.mask_width > 0 and params.mask_width % desp.tile_shape[2] == 0):
            raise RuntimeError("error: mask_width must be a positive multiple of tile_shape[2]")
    if indices is None:
        raise RuntimeError("error: indices empty")
    if mask is None:
        raise RuntimeError("error: mask empty")
    if mask_argsort is None:
        raise RuntimeError("error: mask_argsort empty")
    kv = weight.dim(1)
    if indices.ndim != 2 or indices.dim(0) != kv:
        raise RuntimeError(f"indices shape {indices.shape} does not match [{kv}, -1]")
    N = indices.dim(1)
    # Kernel volumes above 32: ceil(kv / 32) mask words per row / per reduced-mask chunk (the
    # reference's dynamic-mask kernels, cumm/gemm/blockmma/mma.py:78-270, which compute the same
    # count from the kernel volume, cumm/conv/kernel.py:829,935).
    mask_words = _div_up(kv, 32)
    if kv > 128:
        raise RuntimeError(f"kernel volume {kv}: the kernels handle up to 128 filter offsets")
    if kv > 32 and not desp.dynamic_mask:
        raise RuntimeError(f"kernel volume {kv} needs a dynamic-mask descriptor (ConvAlgoDesp.dynamic_mask)")
    if op in (ConvOpType.BackwardWeight, ConvOpType.Forward):
        if N != output.dim(0):
            raise RuntimeError("error: indices.dim(1) must equal output.dim(0)")
    else:
        if N != inp.dim(0):
            raise RuntimeError("error: indices.dim(1) must equal input.dim(0)")
    m, n, k = implicit_gemm_mnk(op, N, C, K, kv)
    if not desp.supported(m, n, k, C, K, params.mask_width):
        raise RuntimeError("error: problem not supported by this descriptor (alignment)")
    tensors = (inp, weight, output)
    inv = gemm_abc_012_to_iwo(op)
    a_t, b_t, c_t = tensors[inv[0]], tensors[inv[1]], tensors[inv[2]]
    for t in (inp, weight, output):
        expect = 1
        for i in reversed(range(t.ndim)):
            if t.stride(i) != expect and t.dim(i) != 1:
                raise RuntimeError("input, weight and output must be contiguous")
            expect *= t.dim(i)
    args = _lib.ConvArgs()
    args.ptr_A, args.ptr_B, args.ptr_C = _ptr(a_t), _ptr(b_t), _ptr(c_t)
    # source operand selection, cumm/conv/nvrtc_code.py:78-90
    if output_add is None:
        if desp.is_int8_inference or bias is None:
            args.ptr_D = _ptr(c_t)
        else:
            args.ptr_D = _ptr(bias)
    else:
        args.ptr_D = _ptr(output_add)
    args.d_is_bias = 1 if (bias is not None and not desp.is_int8_inference and output_add is None) else 0
    args.bias_pointer = _ptr(bias)
    args.scale_pointer = _ptr(scale)
    args.alpha, args.beta = float(params.alpha), float(params.beta)
    args.act_alpha, args.act_beta = float(params.act_alpha), float(params.act_beta)
    args.act_type = int(params.act_type)
    args.split_k_slices = int(params.split_k_slices)
    args.mask_ptr = _ptr(mask)
    args.mask_out_ptr = _ptr(mask_output)
    args.indice_ptr = _ptr(indices)
    args.mask_argsort_ptr = _ptr(mask_argsort)
    args.mask_filter = int(params.mask_filter) & 0xFFFFFFFF
    args.reverse_mask = int(bool(params.reverse_mask))
    args.mask_width = int(params.mask_width)
    args.ndim, args.N, args.C, args.K = desp.ndim, N, C, K
    args.kernel_volume = kv
    args.mode = int(ConvMode.CrossCorrelation)
    args.groups = 1
    args.op_type = int(op)
    args.dtype_a, args.dtype_b, args.dtype_c = a_t.dtype, b_t.dtype, c_t.dtype
    args.is_int8_inference = int(bool(desp.is_int8_inference))
    args.rows_A = a_t.dim(0)
    args.rows_B = b_t.dim(0)
    args.mask_words = mask.size()
    if op != ConvOpType.BackwardWeight and mask.size() < N * mask_words:
        raise RuntimeError(f"mask has {mask.size()} words, {N * mask_words} needed ({mask_words} per row)")
    if op == ConvOpType.Forward and mask_output is not None:
        if mask_output.size() < _div_up(N, 128) * mask_words:
            raise RuntimeError("mask_output is too small")
    # The descriptor selects the kernel: tile_shape = [rows, columns, reduction] of one CTA tile
    # (for backward weight the reduction runs over rows and is tied to mask_width).
    if desp.tile_shape[0] != 128:
        raise RuntimeError(f"can't find any suitable algo: tile_shape[0] = {desp.tile_shape[0]} (the sm_100a "
                           "kernels work on 128-row tiles)")
    args.tile_n = int(desp.tile_shape[1])
    args.tile_k = int(desp.tile_shape[2]) if op != ConvOpType.BackwardWeight else 0
    args.max_ctas = int(getattr(params, "max_ctas", 0))
    args._device = c_t.device
    return args


def run_conv(params: ConvParams) -> None:
    """What ``ConvMainUnitTest.implicit_gemm2`` does (cumm/conv/main.py:485-745)."""
    if not params.conv_algo_desp.mask_sparse:
        # dense convolution: the same kernels over the neighbour table of the full grid
        from ..dense import run_dense_conv
        return run_dense_conv(params)
    L = _lib.load()
    args = _conv_args(params)
    need = L.cb2_conv_workspace_size(ctypes.byref(args))
    if need:
        ptr, nbytes = _workspace_for(args._device, int(params.stream), need, params.workspace)
        args.workspace, args.workspace_bytes = ptr, nbytes
    import torch
    from . import CUDAKernelTimer, _TimerGuard
    name = params.conv_algo_desp.__repr__()
    # verbose: registers of the kernel and the time of this launch (cumm/conv/main.py:723-729)
    timer = params.timer
    own = None
    if params.verbose and not (timer is not None and getattr(timer, "enable", False)):
        timer = own = CUDAKernelTimer(True)
    with torch.cuda.device(args._device), _TimerGuard(name, timer, int(params.stream)):
        _lib.raise_for(L.cb2_conv_run(ctypes.byref(args), ctypes.c_void_p(int(params.stream))))
    if params.verbose:
        info = _lib.last_launch_info()
        t = (own or timer).get_pair_duration(name)
        print(f"{name} kernel num regs: {info['num_regs']} time: {t}")


# The reference's run_nvrtc_* entry points launch the run-time-compiled module the caller puts
# in ``params.nvrtc_params`` and throw when there is none.  This library ships prebuilt sm_100a
# kernels and loads no foreign modules; a caller that wants those entry points to use the
# prebuilt kernels says so here (or with CUMM_B200_NVRTC_USES_PREBUILT=1 in the environment).
NVRTC_ENTRY_POINTS_USE_PREBUILT = False


def _nvrtc_gate(nvrtc_params, what: str) -> None:
    import os
    if getattr(nvrtc_params, "cumodule", None) is not None:
        raise RuntimeError(f"run-time-compiled modules are not loaded by this library; clear nvrtc_params.cumodule and "
                           f"call the static entry point (matmul2 / implicit_gemm2) to run {what} on the prebuilt kernels")
    if not (NVRTC_ENTRY_POINTS_USE_PREBUILT or os.environ.get("CUMM_B200_NVRTC_USES_PREBUILT") == "1"):
        raise RuntimeError(f"you must use nvrtc kernel to run {what} by this function")


def run_nvrtc_gemm_kernel(params: GemmParams) -> None:
    """cumm/tensorview_bind.py:152-167: validates like ``matmul2``, then requires a
    run-time-compiled kernel in ``params.nvrtc_params`` and throws without one.  Here: the
    same error, unless :data:`NVRTC_ENTRY_POINTS_USE_PREBUILT` opts into the prebuilt kernels."""
    _gemm_args(params)
    _nvrtc_gate(params.nvrtc_params, "gemm")
    run_gemm(params)


def run_nvrtc_conv_kernel(params: ConvParams) -> None:
    """cumm/tensorview_bind.py:134-150; see :func:`run_nvrtc_gemm_kernel`."""
    _conv_args(params)
    _nvrtc_gate(params.nvrtc_params, "conv")
    run_conv(params)


class PreparedCall:
    """A validated call with its flat argument record built once, for launch-bound loops
    (replays, CUDA-graph capture): ``launch()`` only crosses the C ABI.  The record owns its
    tile-ticket counters (``sched_scratch``), so a captured launch shares them with nobody --
    two pairs, used in turn: with programmatic dependent launch a launch may start drawing
    tickets while its predecessor on the stream still runs, and that predecessor can be the
    same call.
    ``static_tables``: the caller promises that the neighbour tables (for the weight gradient:
    the reduced masks) keep their contents while the call is in use; the weight gradient then
    plans its schedule on the first launch only (``reuse_plan``)."""

    def __init__(self, kind: str, args, device: int, stream: int, keep, static_tables: bool = False):
        import torch
        self._kind = kind
        self._args = args
        self._device = device
        self._stream = int(stream)
        self._keep = keep  # tensors whose memory the record points at
        self._tickets = torch.zeros(8, dtype=torch.int32, device=f"cuda:{device}")
        self._turn = 0
        args.sched_scratch = self._tickets.data_ptr()
        self._plan_once = bool(static_tables) and bool(args.workspace)
        L = _lib.load()
        self._fn = L.cb2_conv_run if kind == "conv" else L.cb2_gemm_run

    def launch(self, stream: Optional[int] = None) -> None:
        s = self._stream if stream is None else int(stream)
        self._args.sched_scratch = self._tickets.data_ptr() + 16 * self._turn
        self._turn ^= 1
        rc = self._fn(ctypes.byref(self._args), ctypes.c_void_p(s))
        if rc:
            _lib.raise_for(rc)
        if self._plan_once:
            self._args.reuse_plan = 1


def _attach_workspace(L, args, params, keep, size_fn) -> None:
    need = size_fn(ctypes.byref(args))
    if need:
        t = as_view(params.workspace)
        if t is None or t.nbytes() < need:
            import torch
            ws = torch.empty(need, dtype=torch.uint8, device=f"cuda:{args._device}")
            keep.append(ws)
            args.workspace, args.workspace_bytes = ws.data_ptr(), need
        else:
            keep.append(params.workspace)
            args.workspace, args.workspace_bytes = t.data_ptr(), t.nbytes()


def prepare_conv(params: ConvParams, static_tables: bool = False) -> PreparedCall:
    """Validate ``params`` like :func:`run_conv` and return a replayable call.  The tensors
    in ``params`` must stay alive and in place while the call is in use.  Every prepared call
    has a workspace of its own (two prepared weight gradients may overlap on the GPU)."""
    L = _lib.load()
    args = _conv_args(params)
    keep = [params.input, params.weight, params.output, params.indices, params.mask, params.mask_argsort,
            params.mask_output, params.bias, params.scale, params.output_add]
    _attach_workspace(L, args, params, keep, L.cb2_conv_workspace_size)
    return PreparedCall("conv", args, args._device, params.stream, keep, static_tables)


def prepare_gemm(params: GemmParams, static_tables: bool = False) -> PreparedCall:
    L = _lib.load()
    args = _gemm_args(params)
    keep = [params.a, params.b, params.c, params.d, params.a_inds, params.b_inds, params.c_inds]
    _attach_workspace(L, args, params, keep, L.cb2_gemm_workspace_size)
    return PreparedCall("gemm", args, args._device, params.stream, keep, static_tables)
