"""ctypes binding of the C ABI declared in ``include/cumm_b200.h``.

The shared library is built in-tree (``cumm_b200/libcumm_b200.so``) by ``cumm_b200.build``.
There is no fallback: if the library is missing or a call fails, an exception is raised.
"""
from __future__ import annotations

import ctypes
import os
from pathlib import Path

_HERE = Path(__file__).resolve().parent
# CUMM_B200_LIBRARY: another build of the same library (e.g. one compiled with -DCB2_TRACE)
LIB_PATH = Path(os.environ.get("CUMM_B200_LIBRARY") or _HERE / "libcumm_b200.so")

CB2_OK = 0
CB2_ERR_INVALID_ARG = -1
CB2_ERR_RUNTIME = -2
CB2_ERR_UNSUPPORTED = -3
CB2_ERR_CUDA = -4

EXPORTED_SYMBOLS = (
    "cb2_gemm_run",
    "cb2_conv_run",
    "cb2_gemm_workspace_size",
    "cb2_conv_workspace_size",
    "cb2_tile_m",
    "cb2_last_error",
    "cb2_device_status",
    "cb2_launch_count",
    "cb2_conv_backward_weight_static",
    "cb2_static_scratch_bytes",
    "cb2_static_status",
    "cb2_pairgen_workspace_size",
    "cb2_pairgen_count_outputs",
    "cb2_pairgen_run",
    "cb2_peer_allreduce_buffer_size",
    "cb2_peer_allreduce",
    "cb2_enumerate_gemm_desps",
    "cb2_enumerate_conv_desps",
    "cb2_last_launch_info",
    "cb2_dense_tables_run",
    "cb2_gemm_sequence_workspace_size",
    "cb2_gemm_sequence_run",
)


class GemmArgs(ctypes.Structure):
    """``cb2_gemm_args``."""
    _fields_ = [
        ("m", ctypes.c_int), ("n", ctypes.c_int), ("k", ctypes.c_int),
        ("ptr_A", ctypes.c_void_p), ("ptr_B", ctypes.c_void_p), ("ptr_D", ctypes.c_void_p),
        ("ptr_C", ctypes.c_void_p),
        ("stride_A", ctypes.c_int64), ("stride_B", ctypes.c_int64),
        ("stride_C", ctypes.c_int64), ("stride_D", ctypes.c_int64),
        ("indiceA", ctypes.c_void_p), ("indiceBorC", ctypes.c_void_p), ("indiceD", ctypes.c_void_p),
        ("alpha", ctypes.c_float), ("beta", ctypes.c_float),
        ("act_alpha", ctypes.c_float), ("act_beta", ctypes.c_float),
        ("act_type", ctypes.c_int),
        ("split_k_slices", ctypes.c_int),
        ("workspace", ctypes.c_void_p),
        ("workspace_bytes", ctypes.c_size_t),
        ("dtype_a", ctypes.c_int), ("dtype_b", ctypes.c_int), ("dtype_c", ctypes.c_int),
        ("trans_a", ctypes.c_int), ("trans_b", ctypes.c_int), ("trans_c", ctypes.c_int),
        ("shuffle_type", ctypes.c_int),
        ("d_is_vector", ctypes.c_int),
        ("rows_A", ctypes.c_int), ("rows_B", ctypes.c_int),
        ("tile_n", ctypes.c_int), ("tile_k", ctypes.c_int),
        ("sched_scratch", ctypes.c_void_p), ("max_ctas", ctypes.c_int), ("reuse_plan", ctypes.c_int),
    ]


class ConvArgs(ctypes.Structure):
    """``cb2_conv_args``."""
    _fields_ = [
        ("ptr_A", ctypes.c_void_p), ("ptr_B", ctypes.c_void_p), ("ptr_D", ctypes.c_void_p),
        ("ptr_C", ctypes.c_void_p),
        ("alpha", ctypes.c_float), ("beta", ctypes.c_float),
        ("act_alpha", ctypes.c_float), ("act_beta", ctypes.c_float),
        ("act_type", ctypes.c_int),
        ("split_k_slices", ctypes.c_int),
        ("workspace", ctypes.c_void_p),
        ("workspace_bytes", ctypes.c_size_t),
        ("mask_ptr", ctypes.c_void_p),
        ("mask_out_ptr", ctypes.c_void_p),
        ("indice_ptr", ctypes.c_void_p),
        ("mask_argsort_ptr", ctypes.c_void_p),
        ("mask_filter", ctypes.c_uint32),
        ("reverse_mask", ctypes.c_int),
        ("mask_width", ctypes.c_int),
        ("ndim", ctypes.c_int), ("N", ctypes.c_int), ("C", ctypes.c_int), ("K", ctypes.c_int),
        ("kernel_volume", ctypes.c_int),
        ("mode", ctypes.c_int),
        ("groups", ctypes.c_int),
        ("d_is_bias", ctypes.c_int),
        ("bias_pointer", ctypes.c_void_p),
        ("scale_pointer", ctypes.c_void_p),
        ("op_type", ctypes.c_int),
        ("dtype_a", ctypes.c_int), ("dtype_b", ctypes.c_int), ("dtype_c", ctypes.c_int),
        ("is_int8_inference", ctypes.c_int),
        ("rows_A", ctypes.c_int), ("rows_B", ctypes.c_int),
        ("mask_words", ctypes.c_int),
        ("tile_n", ctypes.c_int), ("tile_k", ctypes.c_int),
        ("sched_scratch", ctypes.c_void_p), ("max_ctas", ctypes.c_int), ("reuse_plan", ctypes.c_int),
    ]


class PairgenArgs(ctypes.Structure):
    """``cb2_pairgen_args``."""
    _fields_ = [
        ("in_coords", ctypes.c_void_p),
        ("n_in", ctypes.c_int),
        ("batch_size", ctypes.c_int),
        ("grid", ctypes.c_int * 3),
        ("ksize", ctypes.c_int * 3), ("stride", ctypes.c_int * 3), ("pad", ctypes.c_int * 3), ("dil", ctypes.c_int * 3),
        ("subm", ctypes.c_int),
        ("n_out", ctypes.c_int),
        ("out_coords", ctypes.c_void_p),
        ("indices", ctypes.c_void_p),
        ("mask", ctypes.c_void_p),
        ("mask_argsort", ctypes.c_void_p),
        ("indices_bwd", ctypes.c_void_p),
        ("mask_bwd", ctypes.c_void_p),
        ("mask_argsort_bwd", ctypes.c_void_p),
        ("workspace", ctypes.c_void_p),
        ("workspace_bytes", ctypes.c_size_t),
        ("tile_masks", ctypes.c_void_p),
    ]


class GemmSequenceArgs(ctypes.Structure):
    """``cb2_gemm_sequence_args``."""
    _fields_ = [
        ("calls", ctypes.POINTER(GemmArgs)),
        ("count", ctypes.c_int),
        ("n_out_rows", ctypes.c_int),
        ("workspace", ctypes.c_void_p),
        ("workspace_bytes", ctypes.c_size_t),
        ("reuse_tables", ctypes.c_int),
    ]


class KernelDesp(ctypes.Structure):
    """``cb2_kernel_desp``."""
    _fields_ = [
        ("op_type", ctypes.c_int), ("shuffle_type", ctypes.c_int),
        ("dtype_a", ctypes.c_int), ("dtype_b", ctypes.c_int), ("dtype_c", ctypes.c_int),
        ("dacc", ctypes.c_int), ("dcomp", ctypes.c_int),
        ("trans_a", ctypes.c_int), ("trans_b", ctypes.c_int), ("trans_c", ctypes.c_int),
        ("tile_shape", ctypes.c_int * 3), ("warp_tile_shape", ctypes.c_int * 3), ("tensorop", ctypes.c_int * 3),
        ("num_stage", ctypes.c_int),
        ("element_per_access", ctypes.c_int),
        ("split_k_serial", ctypes.c_int),
        ("mask_sparse", ctypes.c_int), ("increment_k_first", ctypes.c_int), ("is_int8_inference", ctypes.c_int),
        ("min_arch_major", ctypes.c_int), ("min_arch_minor", ctypes.c_int),
        ("dynamic_mask", ctypes.c_int),
    ]


class DenseTablesArgs(ctypes.Structure):
    """``cb2_dense_tables_args``."""
    _fields_ = [
        ("batch", ctypes.c_int),
        ("in_dims", ctypes.c_int * 3), ("out_dims", ctypes.c_int * 3),
        ("ksize", ctypes.c_int * 3), ("stride", ctypes.c_int * 3), ("pad", ctypes.c_int * 3), ("dil", ctypes.c_int * 3),
        ("indices_fwd", ctypes.c_void_p), ("indices_bwd", ctypes.c_void_p),
        ("mask_fwd", ctypes.c_void_p), ("argsort_fwd", ctypes.c_void_p),
        ("mask_bwd", ctypes.c_void_p), ("argsort_bwd", ctypes.c_void_p),
    ]


class PeerAllreduceArgs(ctypes.Structure):
    """``cb2_peer_allreduce_args``."""
    _fields_ = [
        ("peer_buffers", ctypes.POINTER(ctypes.c_void_p)),
        ("rank", ctypes.c_int), ("world", ctypes.c_int),
        ("src", ctypes.c_void_p),
        ("out_f32", ctypes.c_void_p),
        ("out_f16", ctypes.c_void_p),
        ("numel", ctypes.c_longlong),
        ("timeout_ns", ctypes.c_ulonglong),
        ("own_sm_smem_bytes", ctypes.c_int),
    ]


_lib = None


def load() -> ctypes.CDLL:
    """Load the CUDA library; raises if it has not been built."""
    global _lib
    if _lib is not None:
        return _lib
    if not LIB_PATH.exists():
        raise RuntimeError(
            f"{LIB_PATH} is missing: the CUDA extension has not been built "
            "(run `python -c 'import cumm_b200.build as b; b.build()'`). There is no CPU fallback.")
    L = ctypes.CDLL(str(LIB_PATH))
    L.cb2_gemm_run.restype = ctypes.c_int
    L.cb2_gemm_run.argtypes = [ctypes.POINTER(GemmArgs), ctypes.c_void_p]
    L.cb2_conv_run.restype = ctypes.c_int
    L.cb2_conv_run.argtypes = [ctypes.POINTER(ConvArgs), ctypes.c_void_p]
    L.cb2_gemm_workspace_size.restype = ctypes.c_size_t
    L.cb2_gemm_workspace_size.argtypes = [ctypes.POINTER(GemmArgs)]
    L.cb2_conv_workspace_size.restype = ctypes.c_size_t
    L.cb2_conv_workspace_size.argtypes = [ctypes.POINTER(ConvArgs)]
    L.cb2_tile_m.restype = ctypes.c_int
    L.cb2_last_error.restype = ctypes.c_char_p
    L.cb2_device_status.restype = ctypes.c_int
    L.cb2_device_status.argtypes = [ctypes.POINTER(ctypes.c_int)]
    L.cb2_launch_count.restype = ctypes.c_uint64
    L.cb2_conv_backward_weight_static.restype = ctypes.c_int
    L.cb2_conv_backward_weight_static.argtypes = [ctypes.POINTER(ConvArgs), ctypes.c_void_p]
    L.cb2_static_scratch_bytes.restype = ctypes.c_size_t
    L.cb2_static_status.restype = ctypes.c_int
    L.cb2_static_status.argtypes = [ctypes.POINTER(ctypes.c_int)]
    L.cb2_pairgen_workspace_size.restype = ctypes.c_size_t
    L.cb2_pairgen_workspace_size.argtypes = [ctypes.POINTER(PairgenArgs)]
    L.cb2_pairgen_count_outputs.restype = ctypes.c_int
    L.cb2_pairgen_count_outputs.argtypes = [ctypes.POINTER(PairgenArgs), ctypes.POINTER(ctypes.c_int), ctypes.c_void_p]
    L.cb2_pairgen_run.restype = ctypes.c_int
    L.cb2_pairgen_run.argtypes = [ctypes.POINTER(PairgenArgs), ctypes.c_void_p]
    L.cb2_peer_allreduce_buffer_size.restype = ctypes.c_size_t
    L.cb2_peer_allreduce_buffer_size.argtypes = [ctypes.c_longlong, ctypes.c_int]
    L.cb2_peer_allreduce.restype = ctypes.c_int
    L.cb2_peer_allreduce.argtypes = [ctypes.POINTER(PeerAllreduceArgs), ctypes.c_void_p]
    for fn in (L.cb2_enumerate_gemm_desps, L.cb2_enumerate_conv_desps):
        fn.restype = ctypes.c_int
        fn.argtypes = [ctypes.POINTER(KernelDesp), ctypes.c_int]
    L.cb2_gemm_sequence_workspace_size.restype = ctypes.c_size_t
    L.cb2_gemm_sequence_workspace_size.argtypes = [ctypes.POINTER(GemmSequenceArgs)]
    L.cb2_gemm_sequence_run.restype = ctypes.c_int
    L.cb2_gemm_sequence_run.argtypes = [ctypes.POINTER(GemmSequenceArgs), ctypes.c_void_p]
    L.cb2_dense_tables_run.restype = ctypes.c_int
    L.cb2_dense_tables_run.argtypes = [ctypes.POINTER(DenseTablesArgs), ctypes.c_void_p]
    L.cb2_last_launch_info.restype = ctypes.c_int
    L.cb2_last_launch_info.argtypes = [ctypes.POINTER(ctypes.c_int)] * 3
    _lib = L
    return L


def last_error() -> str:
    return load().cb2_last_error().decode("utf-8", "replace")


def raise_for(rc: int) -> None:
    """Translate a return code into the exception class the reference would raise
    (std::invalid_argument -> ValueError, std::runtime_error -> RuntimeError)."""
    if rc == CB2_OK:
        return
    msg = last_error()
    if rc == CB2_ERR_INVALID_ARG:
        raise ValueError(msg)
    raise RuntimeError(msg)


def device_status() -> int:
    """Synchronise the current device and return (and clear) the kernels' status word."""
    v = ctypes.c_int(0)
    raise_for(load().cb2_device_status(ctypes.byref(v)))
    return v.value


def kernel_table(which: str):
    """The library's kernel variants (``cb2_enumerate_gemm_desps`` / ``cb2_enumerate_conv_desps``)."""
    L = load()
    fn = L.cb2_enumerate_conv_desps if which == "conv" else L.cb2_enumerate_gemm_desps
    n = fn(None, 0)
    arr = (KernelDesp * n)()
    fn(arr, n)
    return list(arr)


def last_launch_info() -> dict:
    """Registers per thread, threads per CTA and dynamic shared memory of the last kernel this
    host thread launched through the library (``cb2_last_launch_info``)."""
    r, t, m = ctypes.c_int(0), ctypes.c_int(0), ctypes.c_int(0)
    load().cb2_last_launch_info(ctypes.byref(r), ctypes.byref(t), ctypes.byref(m))
    return {"num_regs": r.value, "num_threads": t.value, "smem_bytes": m.value}


def launch_count() -> int:
    return int(load().cb2_launch_count())
