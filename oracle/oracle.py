"""CPU oracle for the sparse-convolution hot path -- TEST INFRASTRUCTURE ONLY.

Python face of ``sparse_conv_oracle.c`` (loaded with ctypes from ``oracle/_build``) plus
an independent numpy statement of the same operators that follows the reference's own
numpy check loop (cumm/conv/main_real_spconv.py:309-403: for each filter offset, gather
rows, cast fp16->fp32, matmul, scatter-add; cumm/gemm/main_real.py:196-232 for the
gather/scatter GEMM).  The numpy form doubles as the timed CPU baseline, because it runs
on every host core through the BLAS thread pool.

Only ``tests/``, the smoke check and the benchmark's CPU-baseline leg may import this
module.  The shipped package never does.

Parity status: conversions and contract arithmetic are pinned to the reference's own host
headers (``oracle/_ref``, golden vectors in ``tests/golden``); the convolution loops have
no stored vectors in the reference ("parity unpinned" there, see the C file's header).
"""
from __future__ import annotations

import ctypes
import os
import subprocess
from pathlib import Path

import numpy as np

_HERE = Path(__file__).resolve().parent
_LIB = None
_REF = None
_REF_DEV = None

c_i32p = ctypes.POINTER(ctypes.c_int32)
c_u32p = ctypes.POINTER(ctypes.c_uint32)
c_u16p = ctypes.POINTER(ctypes.c_uint16)
c_i8p = ctypes.POINTER(ctypes.c_int8)
c_f32p = ctypes.POINTER(ctypes.c_float)


def build(ref: bool = True) -> None:
    """Compile the C restatement (and the reference host shim when the tree is there)."""
    subprocess.run(["make", "-C", str(_HERE), "-s"], check=True)
    if ref:
        subprocess.run(["make", "-C", str(_HERE), "-s", "ref"], check=True)


def lib() -> ctypes.CDLL:
    global _LIB
    if _LIB is None:
        path = _HERE / "_build" / "liboracle.so"
        if not path.exists():
            build(ref=False)
        L = ctypes.CDLL(str(path))
        L.orc_half_to_float.restype = ctypes.c_float
        L.orc_half_to_float.argtypes = [ctypes.c_uint16]
        L.orc_float_to_half.restype = ctypes.c_uint16
        L.orc_float_to_half.argtypes = [ctypes.c_float]
        L.orc_float_to_s8.restype = ctypes.c_int8
        L.orc_float_to_s8.argtypes = [ctypes.c_float]
        L.orc_build_pairs.restype = ctypes.c_int
        _LIB = L
    return _LIB


def ref_lib():
    """The reference's own host code (None when it was not built in this checkout)."""
    global _REF
    if _REF is None:
        path = _HERE / "_ref" / "libref_host.so"
        if not path.exists():
            return None
        R = ctypes.CDLL(str(path))
        R.ref_float_to_half.restype = ctypes.c_uint16
        R.ref_float_to_half.argtypes = [ctypes.c_float]
        R.ref_half_to_float.restype = ctypes.c_float
        R.ref_half_to_float.argtypes = [ctypes.c_uint16]
        R.ref_float_to_s8.restype = ctypes.c_int
        R.ref_float_to_s8.argtypes = [ctypes.c_float]
        _REF = R
    return _REF


def _p(arr, typ):
    if arr is None:
        return None
    return arr.ctypes.data_as(typ)


def _u16(a):
    a = np.ascontiguousarray(a)
    assert a.dtype == np.float16
    return a.view(np.uint16)


# --------------------------------------------------------------------------------------
# scalar numerics
# --------------------------------------------------------------------------------------
def half_to_float(bits: int) -> float:
    return float(lib().orc_half_to_float(int(bits)))


def float_to_half(x: float) -> int:
    return int(lib().orc_float_to_half(float(x)))


def float_to_s8(x: float) -> int:
    return int(lib().orc_float_to_s8(float(x)))


# --------------------------------------------------------------------------------------
# pair / mask generation (documented convention, see orc_build_pairs)
# --------------------------------------------------------------------------------------
def build_pairs(in_coords, out_coords, grid, ksize, stride, pad, dil):
    in_coords = np.ascontiguousarray(in_coords, np.int32)
    out_coords = np.ascontiguousarray(out_coords, np.int32)
    kv = int(np.prod(ksize))
    n_in, n_out = len(in_coords), len(out_coords)
    indices = np.empty((kv, n_out), np.int32)
    words = (kv + 31) // 32  # kernel volumes above 32: several mask words per row
    mask = np.empty((n_out,) if words == 1 else (n_out, words), np.uint32)
    arr = lambda v: np.ascontiguousarray(v, np.int32)
    g, k, s, p, d = arr(grid), arr(ksize), arr(stride), arr(pad), arr(dil)
    rc = lib().orc_build_pairs(n_in, _p(in_coords, c_i32p), n_out, _p(out_coords, c_i32p),
                               _p(g, c_i32p), _p(k, c_i32p), _p(s, c_i32p), _p(p, c_i32p),
                               _p(d, c_i32p), _p(indices, c_i32p), _p(mask, c_u32p))
    assert rc == 0
    return indices, mask


def regular_out_coords(in_coords, grid, ksize, stride, pad, dil):
    """Output voxel set of a regular (non-submanifold) sparse conv: every output
    coordinate reached by at least one input voxel, ordered by linearised (b,z,y,x)."""
    in_coords = np.asarray(in_coords, np.int64)
    out_grid = [(grid[a] + 2 * pad[a] - dil[a] * (ksize[a] - 1) - 1) // stride[a] + 1
                for a in range(3)]
    keys = []
    for rz in range(ksize[0]):
        for ry in range(ksize[1]):
            for rx in range(ksize[2]):
                r = (rz, ry, rx)
                ok = np.ones(len(in_coords), bool)
                oc = []
                for a in range(3):
                    num = in_coords[:, a + 1] + pad[a] - r[a] * dil[a]
                    ok &= (num % stride[a] == 0)
                    q = num // stride[a]
                    ok &= (q >= 0) & (q < out_grid[a])
                    oc.append(q)
                lin = ((in_coords[:, 0] * out_grid[0] + oc[0]) * out_grid[1] + oc[1]) * out_grid[2] + oc[2]
                keys.append(lin[ok])
    lin = np.unique(np.concatenate(keys))
    x = lin % out_grid[2]
    y = (lin // out_grid[2]) % out_grid[1]
    z = (lin // (out_grid[2] * out_grid[1])) % out_grid[0]
    b = lin // (out_grid[2] * out_grid[1] * out_grid[0])
    return np.stack([b, z, y, x], 1).astype(np.int32), out_grid


def sort_masks(mask):
    """Stable ascending sort of the per-row masks; returns (sorted mask, argsort).  Masks of
    several words compare as one integer whose most significant word is the last one."""
    if mask.ndim == 2:
        order = np.lexsort(tuple(mask[:, w] for w in range(mask.shape[1]))).astype(np.int32)
    else:
        order = np.argsort(mask, kind="stable").astype(np.int32)
    return np.ascontiguousarray(mask[order]), order


def backward_indices(indices, n_in):
    """indices_bwd[f, i] = output row o with indices[f, o] == i, else -1."""
    kv, n_out = indices.shape
    out = np.full((kv, n_in), -1, np.int32)
    for f in range(kv):
        o = np.nonzero(indices[f] >= 0)[0]
        out[f, indices[f, o]] = o.astype(np.int32)
    return out


# --------------------------------------------------------------------------------------
# device-semantics restatements (C)
# --------------------------------------------------------------------------------------
def gemm_shuffle_ac(a, b, c, a_inds, c_inds, trans_b=True, d=None, alpha=1.0, beta=0.0,
                    act_type=0, act_alpha=0.0):
    """C[c_inds[i]] = act(alpha * A[a_inds[i]] @ B' + beta * D[c_inds[i]]); c is updated."""
    m = len(a_inds) if a_inds is not None else a.shape[0]
    k = a.shape[1]
    n = b.shape[0] if trans_b else b.shape[1]
    au, bu, cu = _u16(a), _u16(b), c.view(np.uint16)
    d_is_bias = d is not None and d.ndim == 1
    du = cu if (d is None or d is c) else _u16(d)
    ai = None if a_inds is None else np.ascontiguousarray(a_inds, np.int32)
    ci = None if c_inds is None else np.ascontiguousarray(c_inds, np.int32)
    lib().orc_gemm_shuffle_ac_f16(
        ctypes.c_int(m), ctypes.c_int(n), ctypes.c_int(k), _p(au, c_u16p),
        ctypes.c_int64(a.shape[1]), _p(bu, c_u16p), ctypes.c_int64(b.shape[1]),
        ctypes.c_int(int(trans_b)), _p(cu, c_u16p), ctypes.c_int64(c.shape[1]),
        _p(du, c_u16p), ctypes.c_int64(0 if d_is_bias else (c.shape[1] if d is None else d.shape[1])),
        ctypes.c_int(int(d_is_bias)), _p(ai, c_i32p), _p(ci, c_i32p), ctypes.c_float(alpha),
        ctypes.c_float(beta), ctypes.c_int(act_type), ctypes.c_float(act_alpha))
    return c


def gemm_shuffle_ab(a, b, c, a_inds, b_inds, d=None, alpha=1.0, beta=0.0):
    """C = alpha * A[a_inds].T @ B[b_inds] + beta * D."""
    m, n = a.shape[1], b.shape[1]
    au, bu, cu = _u16(a), _u16(b), c.view(np.uint16)
    du = cu if (d is None or d is c) else _u16(d)
    ai = np.ascontiguousarray(a_inds, np.int32)
    bi = np.ascontiguousarray(b_inds, np.int32)
    lib().orc_gemm_shuffle_ab_f16(
        ctypes.c_int(m), ctypes.c_int(n), ctypes.c_int(len(ai)), _p(au, c_u16p),
        ctypes.c_int64(a.shape[1]), _p(bu, c_u16p), ctypes.c_int64(b.shape[1]),
        _p(cu, c_u16p), ctypes.c_int64(c.shape[1]), _p(du, c_u16p),
        ctypes.c_int64(c.shape[1] if d is None else d.shape[1]), _p(ai, c_i32p), _p(bi, c_i32p),
        ctypes.c_float(alpha), ctypes.c_float(beta), ctypes.c_int(0), ctypes.c_float(0))
    return c


def mask_igemm(a, w, out, indices, mask, mask_argsort, *, is_dgrad=False, d=None,
               mask_out=None, mask_filter=0xFFFFFFFF, reverse_mask=False, tile_m=128,
               alpha=1.0, beta=0.0, act_type=0, act_alpha=0.0):
    """Forward (a = features) or input gradient (a = output gradients) in fp16.
    w is [K_out, kv, C_in]; `out` is updated in place and returned."""
    K_out, kv, C_in = w.shape
    N = indices.shape[1]
    assert indices.shape[0] == kv
    au, wu, ou = _u16(a), _u16(w), out.view(np.uint16)
    d_is_bias = d is not None and d.ndim == 1
    du = ou if (d is None or d is out) else _u16(d)
    idx = np.ascontiguousarray(indices, np.int32)
    mk = np.ascontiguousarray(mask, np.uint32)
    ms = np.ascontiguousarray(mask_argsort, np.int32)
    lib().orc_mask_igemm_f16(
        ctypes.c_int(int(is_dgrad)), ctypes.c_int(N), ctypes.c_int(a.shape[0]),
        ctypes.c_int(C_in), ctypes.c_int(K_out), ctypes.c_int(kv), _p(au, c_u16p),
        _p(wu, c_u16p), _p(ou, c_u16p), _p(du, c_u16p), ctypes.c_int(int(d_is_bias)),
        _p(idx, c_i32p), _p(mk, c_u32p), _p(ms, c_i32p), _p(mask_out, c_u32p),
        ctypes.c_uint32(mask_filter), ctypes.c_int(int(reverse_mask)), ctypes.c_int(tile_m),
        ctypes.c_float(alpha), ctypes.c_float(beta), ctypes.c_int(act_type),
        ctypes.c_float(act_alpha))
    return out


def mask_igemm_wgrad(dout, x, dw, indices, reduced_mask, mask_argsort, *,
                     mask_filter=0xFFFFFFFF, mask_width=128, alpha=1.0, beta=0.0,
                     out_f32=None):
    """dW [K_out, kv, C_in] (fp16 in place, or fp32 into out_f32)."""
    K_out, kv, C_in = dw.shape if out_f32 is None else out_f32.shape
    N = indices.shape[1]
    idx = np.ascontiguousarray(indices, np.int32)
    rm = np.ascontiguousarray(reduced_mask, np.uint32)
    ms = np.ascontiguousarray(mask_argsort, np.int32)
    lib().orc_mask_igemm_wgrad_f16(
        ctypes.c_int(N), ctypes.c_int(C_in), ctypes.c_int(K_out), ctypes.c_int(kv),
        _p(_u16(dout), c_u16p), _p(_u16(x), c_u16p),
        None if dw is None else _p(dw.view(np.uint16), c_u16p), _p(out_f32, c_f32p),
        _p(idx, c_i32p), _p(rm, c_u32p), _p(ms, c_i32p), ctypes.c_uint32(mask_filter),
        ctypes.c_int(mask_width), ctypes.c_float(alpha), ctypes.c_float(beta))
    return dw if out_f32 is None else out_f32


def mask_igemm_s8(x, w, out, scale, bias, indices, mask, mask_argsort, *, output_add=None,
                  mask_out=None, mask_filter=0xFFFFFFFF, tile_m=128, beta=0.0, act_type=0,
                  act_alpha=0.0):
    """int8 inference forward with the fused requantisation epilogue."""
    K_out, kv, C_in = w.shape
    N = indices.shape[1]
    idx = np.ascontiguousarray(indices, np.int32)
    mk = np.ascontiguousarray(mask, np.uint32)
    ms = np.ascontiguousarray(mask_argsort, np.int32)
    x = np.ascontiguousarray(x, np.int8)
    w = np.ascontiguousarray(w, np.int8)
    sc = np.ascontiguousarray(scale, np.float32)
    bi = np.ascontiguousarray(bias, np.float32)
    lib().orc_mask_igemm_s8(
        ctypes.c_int(N), ctypes.c_int(C_in), ctypes.c_int(K_out), ctypes.c_int(kv),
        _p(x, c_i8p), _p(w, c_i8p), _p(out, c_i8p), _p(output_add, c_i8p), _p(sc, c_f32p),
        _p(bi, c_f32p), _p(idx, c_i32p), _p(mk, c_u32p), _p(ms, c_i32p),
        _p(mask_out, c_u32p), ctypes.c_uint32(mask_filter), ctypes.c_int(tile_m),
        ctypes.c_float(beta), ctypes.c_int(act_type), ctypes.c_float(act_alpha))
    return out


def requant_s8(acc, scale, bias, beta=0.0, src=None, act_type=0, act_alpha=0.0):
    acc = np.ascontiguousarray(acc, np.int32)
    rows, K_out = acc.shape
    out = np.empty((rows, K_out), np.int8)
    sc = np.ascontiguousarray(scale, np.float32)
    bi = np.ascontiguousarray(bias, np.float32)
    lib().orc_requant_s8(ctypes.c_int(rows), ctypes.c_int(K_out), _p(acc, c_i32p),
                         _p(sc, c_f32p), _p(bi, c_f32p), ctypes.c_float(beta),
                         _p(src, c_i8p), ctypes.c_int(act_type), ctypes.c_float(act_alpha),
                         _p(out, c_i8p))
    return out


def lincomb_f16(acc, alpha=1.0, beta=0.0, src=None, act_type=0, act_alpha=0.0):
    """fp16 output operator on an fp32 accumulator array (any shape); ``src`` fp16 or None."""
    acc = np.ascontiguousarray(acc, np.float32)
    out = np.empty(acc.shape, np.float16)
    sb = None if src is None else _u16(np.ascontiguousarray(src, np.float16))
    lib().orc_lincomb_f16(ctypes.c_longlong(acc.size), _p(acc, c_f32p), ctypes.c_float(alpha), ctypes.c_float(beta),
                          _p(sb, c_u16p), ctypes.c_int(act_type), ctypes.c_float(act_alpha),
                          _p(out.view(np.uint16), c_u16p))
    return out


def ref_device_lib():
    """The reference's own epilogue functors compiled as device code (``oracle/ref_device_shim.cu``);
    None when it was not built in this checkout.  Calling into it needs a GPU."""
    global _REF_DEV
    if _REF_DEV is None:
        path = _HERE / "_ref" / "libref_device.so"
        if not path.exists():
            return None
        R = ctypes.CDLL(str(path))
        R.ref_dev_requant_s8.restype = ctypes.c_int
        R.ref_dev_requant_s8.argtypes = [ctypes.c_longlong, ctypes.c_int, c_i32p, c_f32p, c_f32p, ctypes.c_float,
                                         c_i8p, ctypes.c_int, c_i8p]
        R.ref_dev_lincomb_f16.restype = ctypes.c_int
        R.ref_dev_lincomb_f16.argtypes = [ctypes.c_longlong, c_f32p, ctypes.c_float, ctypes.c_float, c_u16p,
                                          ctypes.c_int, c_u16p]
        _REF_DEV = R
    return _REF_DEV


# --------------------------------------------------------------------------------------
# numpy statement (the reference's own check loop), also the timed CPU baseline
# --------------------------------------------------------------------------------------
def np_pairs(indices):
    """Per-offset (in_idx, out_idx) pair lists = non-negative entries in ascending out."""
    pairs = []
    for f in range(indices.shape[0]):
        o = np.nonzero(indices[f] >= 0)[0]
        pairs.append((indices[f, o], o))
    return pairs


def np_forward(x, w, indices, out_dtype=np.float32):
    """out[o] = sum_f x[idx[f,o]] @ w[:, f, :].T in fp32 (cumm/conv/main_real_spconv.py:309-329)."""
    K_out, kv, C_in = w.shape
    out = np.zeros((indices.shape[1], K_out), np.float32)
    for f, (i_idx, o_idx) in enumerate(np_pairs(indices)):
        if len(o_idx) == 0:
            continue
        out[o_idx] += x[i_idx].astype(np.float32) @ w[:, f, :].T.astype(np.float32)
    return out.astype(out_dtype)


def np_dgrad(dout, w, indices, n_in):
    """din[i] = sum_f dout[o] @ w[:, f, :] over pairs (i, o) (main_real_spconv.py:349-369)."""
    K_out, kv, C_in = w.shape
    din = np.zeros((n_in, C_in), np.float32)
    for f, (i_idx, o_idx) in enumerate(np_pairs(indices)):
        if len(o_idx) == 0:
            continue
        # pairs are unique in i for a fixed offset, so fancy += is safe
        din[i_idx] += dout[o_idx].astype(np.float32) @ w[:, f, :].astype(np.float32)
    return din


def np_wgrad(dout, x, indices):
    """dW[:, f, :] = dout[o].T @ x[i] over pairs (main_real_spconv.py:377-396)."""
    K_out, C_in = dout.shape[1], x.shape[1]
    kv = indices.shape[0]
    dw = np.zeros((K_out, kv, C_in), np.float32)
    for f, (i_idx, o_idx) in enumerate(np_pairs(indices)):
        if len(o_idx) == 0:
            continue
        dw[:, f, :] = dout[o_idx].astype(np.float32).T @ x[i_idx].astype(np.float32)
    return dw


def np_forward_s8_acc(x, w, indices):
    """Exact int32 accumulators through float64 BLAS (|acc| <= 27*128*127^2 < 2^53)."""
    K_out, kv, C_in = w.shape
    acc = np.zeros((indices.shape[1], K_out), np.float64)
    for f, (i_idx, o_idx) in enumerate(np_pairs(indices)):
        if len(o_idx) == 0:
            continue
        acc[o_idx] += x[i_idx].astype(np.float64) @ w[:, f, :].T.astype(np.float64)
    return acc.astype(np.int64).astype(np.int32)


def np_dense_gemm_tiled(a, b, tile=(64, 64, 32)):
    """Single-threaded tile-loop restatement of the data flow of the reference's CPU
    simulator GEMM (cumm/gemm/kernel.py:1025-1180: one block per 64x64 output tile, the
    k-loop in steps of 32, fp32 accumulation, fp16 store).  Stand-in for the simulator,
    which cannot be imported without its code generator."""
    m, k = a.shape
    n = b.shape[1]
    tm, tn, tk = tile
    c = np.zeros((m, n), np.float16)
    for bm in range(0, m, tm):
        for bn in range(0, n, tn):
            acc = np.zeros((min(tm, m - bm), min(tn, n - bn)), np.float32)
            for bk in range(0, k, tk):
                acc += a[bm:bm + tm, bk:bk + tk].astype(np.float32) @ \
                    b[bk:bk + tk, bn:bn + tn].astype(np.float32)
            c[bm:bm + tm, bn:bn + tn] = acc.astype(np.float16)
    return c
