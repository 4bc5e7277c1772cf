"""Neighbour tables built on the GPU (``cb2_pairgen_*`` of the C ABI): the step before the
convolution calls, replacing the host generator of :mod:`cumm_b200.workloads` in a pipeline.

The convention is the one :func:`cumm_b200.workloads.build_tables` documents and the tests compare
bit for bit: offsets in (z, y, x) row-major order, ``indices [kv, n_out]`` with -1 for a missing
neighbour, masks sorted ascending with a stable sort, active outputs of a strided convolution
ordered by their linearised (batch, z, y, x).  Kernel volumes above 32 (up to 128) give masks
``[n, words]`` (word w = offsets 32w .. 32w+31) sorted as one integer whose last word is the most
significant, for the ``dynamic_mask`` kernels."""
from __future__ import annotations

import ctypes
from typing import Optional, Sequence

from . import _lib
from .layer import DeviceTables


def build_tables_gpu(in_coords, batch_size: int, grid: Sequence[int], ksize=(3, 3, 3), stride=(1, 1, 1),
                     pad: Optional[Sequence[int]] = None, dil=(1, 1, 1), subm: bool = True, backward: bool = True,
                     stream: int = 0, return_out_coords: bool = False):
    """``in_coords``: int32 CUDA tensor [n_in, 4] (batch, z, y, x), unique rows.  Returns a
    :class:`cumm_b200.layer.DeviceTables` (``num_pairs`` is left at -1: counting would cost a
    synchronisation nobody needs), and the output coordinates when asked for."""
    import torch
    if not (in_coords.is_cuda and in_coords.dtype == torch.int32 and in_coords.dim() == 2 and in_coords.shape[1] == 4
            and in_coords.is_contiguous()):
        raise RuntimeError("in_coords must be a contiguous int32 CUDA tensor of shape [n, 4]")
    if pad is None:
        pad = tuple(k // 2 for k in ksize)
    L = _lib.load()
    dev = in_coords.device
    n_in = int(in_coords.shape[0])
    kv = int(ksize[0] * ksize[1] * ksize[2])
    a = _lib.PairgenArgs()
    a.in_coords = in_coords.data_ptr()
    a.n_in, a.batch_size, a.subm = n_in, int(batch_size), int(bool(subm))
    for name, vals in (("grid", grid), ("ksize", ksize), ("stride", stride), ("pad", pad), ("dil", dil)):
        arr = getattr(a, name)
        for i in range(3):
            arr[i] = int(vals[i])
    with torch.cuda.device(dev):
        need = L.cb2_pairgen_workspace_size(ctypes.byref(a))
        if need == 0:
            raise ValueError(_lib.last_error() or "bad geometry")
        ws = torch.empty(need, dtype=torch.uint8, device=dev)
        a.workspace, a.workspace_bytes = ws.data_ptr(), need
        n_out = ctypes.c_int(0)
        _lib.raise_for(L.cb2_pairgen_count_outputs(ctypes.byref(a), ctypes.byref(n_out), ctypes.c_void_p(stream)))
        n_out = n_out.value
        a.n_out = n_out
        out_coords = in_coords if subm else torch.empty((n_out, 4), dtype=torch.int32, device=dev)
        indices = torch.empty((kv, n_out), dtype=torch.int32, device=dev)
        words = (kv + 31) // 32
        wide = (words,) if words > 1 else ()
        mask = torch.empty((n_out,) + wide, dtype=torch.int32, device=dev)
        argsort = torch.empty((n_out,), dtype=torch.int32, device=dev)
        a.out_coords = 0 if subm else out_coords.data_ptr()
        a.indices, a.mask, a.mask_argsort = indices.data_ptr(), mask.data_ptr(), argsort.data_ptr()
        ibwd = mbwd = abwd = None
        if backward:
            ibwd = torch.empty((kv, n_in), dtype=torch.int32, device=dev)
            mbwd = torch.empty((n_in,) + wide, dtype=torch.int32, device=dev)
            abwd = torch.empty((n_in,), dtype=torch.int32, device=dev)
            a.indices_bwd, a.mask_bwd, a.mask_argsort_bwd = ibwd.data_ptr(), mbwd.data_ptr(), abwd.data_ptr()
        mask_output = torch.zeros(((n_out + 127) // 128,) + wide, dtype=torch.int32, device=dev)
        a.tile_masks = mask_output.data_ptr()
        _lib.raise_for(L.cb2_pairgen_run(ctypes.byref(a), ctypes.c_void_p(stream)))
    # the kernels enqueued above still read the workspace: it lives as long as the tables do
    tables = DeviceTables(n_in, n_out, kv, indices, mask, argsort, ibwd, mbwd, abwd, mask_output, -1, keep=ws)
    return (tables, out_coords) if return_out_coords else tables
