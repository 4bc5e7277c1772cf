"""A layer's sequence of gather-GEMM-scatter calls in one launch (``cb2_gemm_sequence_run``).

The reference's callers run a native (non-mask) sparse convolution as one ``GemmParams`` call
per filter offset, each accumulating into the output with beta = 1
(cumm/gemm/main_real.py:196-232).  At spconv sizes 26 of the 27 calls of a 3x3x3 layer move a
few hundred rows: the sequence is launch-bound by construction.  ``prepare_gemm_sequence`` takes
the same list of ``GemmParams`` and runs it as ONE launch: the pair lists are scattered into the
neighbour table of one convolution (once: the table depends on the lists only) and the
mask-convolution kernel does the rest.  Sums are taken in fp32 over all offsets and rounded once,
where the call-by-call sequence rounds after every call: results agree to a few fp16 ulps."""
from __future__ import annotations

import ctypes
from typing import Optional, Sequence

from . import _lib
from .tensorview import as_view
from .tensorview.gemm import GemmParams, _gemm_args


class PreparedGemmSequence:
    """``launch()`` enqueues the whole sequence; the tensors of the calls must stay alive and in
    place, and the pair lists must keep their contents (the tables are built on the first launch)."""

    def __init__(self, params: Sequence[GemmParams], n_out_rows: Optional[int] = None, stream: int = 0):
        import torch
        if not params:
            raise ValueError("empty sequence")
        L = _lib.load()
        args = [_gemm_args(p) for p in params]
        self._calls = (_lib.GemmArgs * len(args))(*args)
        self._keep = [[p.a, p.b, p.c, p.a_inds, p.c_inds] for p in params]
        c = as_view(params[0].c)
        self._device = c.device
        self._stream = int(stream or params[0].stream)
        a = _lib.GemmSequenceArgs()
        a.calls = ctypes.cast(self._calls, ctypes.POINTER(_lib.GemmArgs))
        a.count = len(args)
        a.n_out_rows = int(c.dim(0) if n_out_rows is None else n_out_rows)
        need = L.cb2_gemm_sequence_workspace_size(ctypes.byref(a))
        if need == 0:
            raise ValueError("a sequence holds 1 to 32 calls")
        self._ws = torch.empty(need, dtype=torch.uint8, device=f"cuda:{self._device}")
        a.workspace, a.workspace_bytes = self._ws.data_ptr(), need
        self._args = a
        self._L = L

    def launch(self, stream: Optional[int] = None) -> None:
        s = self._stream if stream is None else int(stream)
        rc = self._L.cb2_gemm_sequence_run(ctypes.byref(self._args), ctypes.c_void_p(s))
        if rc:
            _lib.raise_for(rc)
        self._args.reuse_tables = 1


def prepare_gemm_sequence(params: Sequence[GemmParams], n_out_rows: Optional[int] = None,
                          stream: int = 0) -> PreparedGemmSequence:
    return PreparedGemmSequence(params, n_out_rows, stream)
