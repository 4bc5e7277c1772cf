"""Dense (non-mask) convolution behind ``ConvParams``: ``conv_algo_desp.mask_sparse == False``.

The reference's dense implicit-GEMM kernels take channels-last tensors -- input
``[N, *spatial, C]``, weight ``[K, *kernel, C]``, output ``[N, *out_spatial, K]`` -- with
``padding`` / ``stride`` / ``dilation`` per axis (cumm/conv/nvrtc_code.py:49-64, iterators
cumm/conv/input_iters.py:2353; harness cumm/conv/main_real.py:41-231, checked against
``torch.nn.functional.conv{1,2,3}d``).  Here a dense convolution is the sparse one whose voxels
fill the grid: ``cb2_dense_tables_run`` writes the neighbour table of the geometry on the GPU
(the reference's coordinate rule, in = out * stride - pad + r * dilation), every row carries every
filter offset, rows keep their order, and the three operators run through the same sm_100a
row-gather kernels.  Tables are cached per geometry and device."""
from __future__ import annotations

import ctypes
from typing import Dict, List, Tuple

from . import _lib
from .tensorview import as_view

_TABLES: Dict[Tuple, dict] = {}


def _geometry(params):
    """(batch, in_dims, out_dims, ksize, stride, pad, dil, C, K), each spatial list padded to 3 axes."""
    from .tensorview.gemm import ConvOpType
    desp = params.conv_algo_desp
    ndim = int(desp.ndim)
    inp, weight, output = as_view(params.input), as_view(params.weight), as_view(params.output)
    if inp is None or weight is None or output is None:
        raise RuntimeError("input, weight, output must not empty")
    for t, what in ((inp, "input"), (weight, "weight"), (output, "output")):
        if t.ndim != ndim + 2:
            raise RuntimeError(f"error: a dense {ndim}-d convolution takes {ndim + 2}-d channels-last tensors; {what} is {t.shape}")
    def lst(v, default):
        v = list(v) if v else [default] * ndim
        if len(v) != ndim:
            raise RuntimeError(f"error: padding, stride and dilation need {ndim} entries")
        return [int(x) for x in v]
    pad, stride, dil = lst(params.padding, 0), lst(params.stride, 1), lst(params.dilation, 1)
    batch, C, K = inp.dim(0), inp.dim(ndim + 1), weight.dim(0)
    in_dims = [inp.dim(1 + a) for a in range(ndim)]
    ksize = [weight.dim(1 + a) for a in range(ndim)]
    if weight.dim(ndim + 1) != C or output.dim(ndim + 1) != K or output.dim(0) != batch:
        raise RuntimeError("error: channel or batch extents of input, weight and output do not match")
    out_dims = []
    for a in range(ndim):
        span = in_dims[a] + 2 * pad[a] - dil[a] * (ksize[a] - 1) - 1
        if span < 0:
            raise RuntimeError(f"error: the kernel does not fit the input on axis {a}")
        out_dims.append(span // stride[a] + 1)
        if output.dim(1 + a) != out_dims[a]:
            raise RuntimeError(f"error: output extent {output.dim(1 + a)} on axis {a}, expected {out_dims[a]}")
    lead = 3 - ndim
    ext = lambda v, fill: [fill] * lead + list(v)
    return (batch, ext(in_dims, 1), ext(out_dims, 1), ext(ksize, 1), ext(stride, 1), ext(pad, 0), ext(dil, 1), C, K)


def _tables(device: int, geom, stream: int) -> dict:
    import torch
    batch, in_dims, out_dims, ksize, stride, pad, dil, _, _ = geom
    key = (device, batch, tuple(in_dims), tuple(out_dims), tuple(ksize), tuple(stride), tuple(pad), tuple(dil))
    t = _TABLES.get(key)
    if t is not None:
        return t
    n_in = batch * in_dims[0] * in_dims[1] * in_dims[2]
    n_out = batch * out_dims[0] * out_dims[1] * out_dims[2]
    kv = ksize[0] * ksize[1] * ksize[2]
    words = (kv + 31) // 32
    dev = f"cuda:{device}"
    i32 = lambda *shape: torch.empty(shape, dtype=torch.int32, device=dev)
    t = dict(n_in=n_in, n_out=n_out, kv=kv, words=words,
             indices_fwd=i32(kv, n_out), indices_bwd=i32(kv, n_in),
             mask_fwd=i32(n_out, words) if words > 1 else i32(n_out), argsort_fwd=i32(n_out),
             mask_bwd=i32(n_in, words) if words > 1 else i32(n_in), argsort_bwd=i32(n_in))
    tiles = (n_out + 127) // 128
    a = _lib.DenseTablesArgs()
    a.batch = batch
    for name, vals in (("in_dims", in_dims), ("out_dims", out_dims), ("ksize", ksize), ("stride", stride),
                       ("pad", pad), ("dil", dil)):
        arr = getattr(a, name)
        for i in range(3):
            arr[i] = int(vals[i])
    for name in ("indices_fwd", "indices_bwd", "mask_fwd", "argsort_fwd", "mask_bwd", "argsort_bwd"):
        setattr(a, name, t[name].data_ptr())
    with torch.cuda.device(device):
        _lib.raise_for(_lib.load().cb2_dense_tables_run(ctypes.byref(a), ctypes.c_void_p(int(stream))))
    # the reduced masks of the weight gradient: every tile carries every offset
    t["tile_masks"] = t["mask_fwd"][:tiles].clone()
    _TABLES[key] = t
    return t


def run_dense_conv(params) -> None:
    """Forward / backward input / backward weight of a dense convolution (see the module text)."""
    from .tensorview.gemm import ConvOpType, ConvParams, run_conv
    desp = params.conv_algo_desp
    geom = _geometry(params)
    C, K = geom[7], geom[8]
    inp, weight, output = params.input, params.weight, params.output
    device = as_view(output).device
    t = _tables(device, geom, int(params.stream))
    d = desp.copy()
    d.mask_sparse = True
    d.increment_k_first = True
    d.dynamic_mask = t["kv"] > 32
    q = ConvParams(desp.ndim, desp.op_type, params.timer)
    q.conv_algo_desp = d
    q.input = inp.view(t["n_in"], C)
    q.weight = weight.view(K, t["kv"], C)
    q.output = output.view(t["n_out"], K)
    q.bias, q.scale, q.output_add = params.bias, params.scale, None
    if params.output_add is not None:
        q.output_add = params.output_add.view(t["n_out"], K)
    q.alpha, q.beta = params.alpha, params.beta
    q.act_alpha, q.act_beta, q.act_type = params.act_alpha, params.act_beta, params.act_type
    q.split_k_slices = params.split_k_slices
    q.workspace, q.stream, q.verbose = params.workspace, params.stream, params.verbose
    q.max_ctas = getattr(params, "max_ctas", 0)
    op = ConvOpType(int(desp.op_type))
    if op == ConvOpType.BackwardInput:
        q.indices, q.mask, q.mask_argsort = t["indices_bwd"], t["mask_bwd"], t["argsort_bwd"]
    else:
        q.indices, q.mask_argsort = t["indices_fwd"], t["argsort_fwd"]
        if op == ConvOpType.BackwardWeight:
            q.mask, q.mask_width = t["tile_masks"], 128
        else:
            q.mask = t["mask_fwd"]
    run_conv(q)
