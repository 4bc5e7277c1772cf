"""One sparse-conv layer's three launches (forward, input gradient, weight gradient) wired
through the operator surface, with device-resident neighbour tables.  This is the caller's
side of the hot path in miniature: it only fills ``ConvParams`` records the way the
reference's harness does (cumm/conv/main_real_spconv.py:228-293) and keeps the prepared
calls so a training step can be replayed or captured in a CUDA graph."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import numpy as np

from .conv.main import TILE_M
from .tensorview import float16, float32, int8, int32
from .tensorview.gemm import (ConvAlgoDesp, ConvOpType, ConvParams, PreparedCall, prepare_conv)
from .workloads import ConvTables


def default_tile(op, C: int, K: int, int8_inference: bool = False):
    """The tile shape used when nothing has been tuned: the narrowest column tile that covers the
    output width and the narrowest reduction tile that covers the reduction width."""
    op = ConvOpType(int(op))
    n_width = K if op == ConvOpType.Forward else C
    red = C if op == ConvOpType.Forward else K
    tile_n = 64 if n_width <= 64 else 128
    if op == ConvOpType.BackwardWeight or int8_inference:
        tile_k = 128
    else:
        tile_k = 64 if red <= 64 else 128
    return [TILE_M, tile_n, tile_k]


def make_desp(op, int8_inference: bool = False, C: int = 128, K: int = 128, tile=None) -> ConvAlgoDesp:
    d = ConvAlgoDesp(3, op)
    if int8_inference:
        d.dtype_a = d.dtype_b = d.dtype_c = int8
        d.dacc, d.dcomp = int32, float32
        epa = 16
    else:
        d.dtype_a = d.dtype_b = d.dtype_c = float16
        d.dacc = d.dcomp = float32
        epa = 8
    d.trans_a, d.trans_b, d.trans_c = {ConvOpType.Forward: (False, True, False),
                                       ConvOpType.BackwardInput: (False, False, False),
                                       ConvOpType.BackwardWeight: (True, False, False)}[ConvOpType(int(op))]
    d.tile_shape = list(tile) if tile is not None else default_tile(op, C, K, int8_inference)
    d.warp_tile_shape = list(d.tile_shape)
    d.tensorop = [128, d.tile_shape[1], 32 if int8_inference else 16]
    d.num_stage = 3
    d.algo = "Blackwell"
    d.split_k_serial = int(op) == ConvOpType.BackwardWeight
    d.element_per_access_a = d.element_per_access_b = d.element_per_access_c = epa
    d.mask_sparse = True
    d.increment_k_first = True
    d.is_int8_inference = int8_inference
    return d


@dataclass
class DeviceTables:
    """Neighbour tables on the device (masks as int32 bit patterns)."""
    n_in: int
    n_out: int
    kv: int
    indices: "torch.Tensor"
    mask: "torch.Tensor"
    mask_argsort: "torch.Tensor"
    indices_bwd: "torch.Tensor"
    mask_bwd: "torch.Tensor"
    mask_argsort_bwd: "torch.Tensor"
    mask_output: "torch.Tensor"
    num_pairs: int
    keep: object = None  # memory that kernels still in flight read (the builder's workspace)

    def clone(self) -> "DeviceTables":
        """A copy with its own device tensors (benchmarks rotate over such copies)."""
        def c(t):
            return None if t is None else t.clone()
        return DeviceTables(self.n_in, self.n_out, self.kv, c(self.indices), c(self.mask), c(self.mask_argsort),
                            c(self.indices_bwd), c(self.mask_bwd), c(self.mask_argsort_bwd), c(self.mask_output),
                            self.num_pairs)

    @staticmethod
    def from_host(tb: ConvTables, device) -> "DeviceTables":
        import torch

        def up(a):
            if a.dtype == np.uint32:
                a = a.view(np.int32)
            return torch.from_numpy(np.ascontiguousarray(a)).to(device)

        # per-tile OR of the sorted masks: what the forward pass reports and the weight gradient reads
        mo = up(np.bitwise_or.reduceat(tb.mask, np.arange(0, max(tb.n_out, 1), TILE_M))[:(tb.n_out + TILE_M - 1) // TILE_M]
                if tb.n_out else np.zeros(0, np.uint32))
        return DeviceTables(tb.n_in, tb.n_out, tb.kv, up(tb.indices), up(tb.mask), up(tb.mask_argsort),
                            up(tb.indices_bwd), up(tb.mask_bwd), up(tb.mask_argsort_bwd), mo, tb.num_pairs)


class SparseConvLayer:
    """Prepared forward / backward-input / backward-weight calls over fixed buffers."""

    def __init__(self, tables: DeviceTables, weight, x, out, dout=None, din=None, dw=None, stream: int = 0,
                 tiles=None, cta_shares=None):
        """``tiles``: optional {ConvOpType: tile_shape} (e.g. from the tuner); ops without an entry
        use :func:`default_tile`.  ``cta_shares``: optional {ConvOpType: CTAs} bounding each launch
        (``max_ctas``), for a caller that runs the three ops side by side on three streams.
        The tables are fixed for the life of the layer, so the weight gradient plans once."""
        self.t = tables
        shares = dict(cta_shares or {})
        tiles = dict(tiles or {})
        K, C = int(weight.shape[0]), int(weight.shape[2])
        self.fwd: Optional[PreparedCall] = None
        self.dgrad: Optional[PreparedCall] = None
        self.wgrad: Optional[PreparedCall] = None
        int8_inf = str(x.dtype).endswith("int8")
        p = ConvParams(3, ConvOpType.Forward)
        p.conv_algo_desp = make_desp(ConvOpType.Forward, int8_inf, C, K, tiles.get(ConvOpType.Forward))
        p.input, p.weight, p.output = x, weight, out
        p.indices, p.mask, p.mask_argsort = tables.indices, tables.mask, tables.mask_argsort
        p.mask_output = tables.mask_output
        p.stream = stream
        p.max_ctas = int(shares.get(ConvOpType.Forward, 0))
        self.fwd_params = p
        if not int8_inf:
            self.fwd = prepare_conv(p, static_tables=True)
        if dout is not None and din is not None:
            q = ConvParams(3, ConvOpType.BackwardInput)
            q.conv_algo_desp = make_desp(ConvOpType.BackwardInput, False, C, K, tiles.get(ConvOpType.BackwardInput))
            q.input, q.weight, q.output = din, weight, dout
            q.indices, q.mask, q.mask_argsort = tables.indices_bwd, tables.mask_bwd, tables.mask_argsort_bwd
            q.stream = stream
            q.max_ctas = int(shares.get(ConvOpType.BackwardInput, 0))
            self.dgrad = prepare_conv(q, static_tables=True)
        if dout is not None and dw is not None:
            r = ConvParams(3, ConvOpType.BackwardWeight)
            r.conv_algo_desp = make_desp(ConvOpType.BackwardWeight, False, C, K, tiles.get(ConvOpType.BackwardWeight))
            r.input, r.weight, r.output = x, dw, dout
            r.indices, r.mask, r.mask_argsort = tables.indices, tables.mask_output, tables.mask_argsort
            r.mask_width = TILE_M
            r.split_k_slices = 32
            r.stream = stream
            r.max_ctas = int(shares.get(ConvOpType.BackwardWeight, 0))
            self.wgrad = prepare_conv(r, static_tables=True)

    def prepare_int8(self, scale, bias) -> None:
        self.fwd_params.scale, self.fwd_params.bias = scale, bias
        self.fwd = prepare_conv(self.fwd_params, static_tables=True)
