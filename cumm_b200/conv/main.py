"""``ConvMainUnitTest``: the static entry points of the reference's sparse-conv dispatcher
(cumm/conv/main.py:469-1050) over the sm_100a kernels."""
from __future__ import annotations

from typing import List, Sequence, Tuple

from ..tensorview import float16, float32, int8, int32
from ..tensorview.gemm import (ConvAlgoDesp, ConvOpType, ConvParams, implicit_gemm_mnk, run_conv)

TILE_M = 128

# (trans_a, trans_b, trans_c) per op, cumm/conv/params.py:61-69
_TRANS = {ConvOpType.Forward: (False, True, False),
          ConvOpType.BackwardInput: (False, False, False),
          ConvOpType.BackwardWeight: (True, False, False)}


def _desp(op: ConvOpType, tile_n: int, tile_k: int, int8_inference: bool = False) -> ConvAlgoDesp:
    d = ConvAlgoDesp(3, op)
    if int8_inference:
        d.dtype_a = d.dtype_b = d.dtype_c = int8
        d.dacc, d.dcomp = int32, float32
        epa = 16
    else:
        d.dtype_a = d.dtype_b = d.dtype_c = float16
        d.dacc = d.dcomp = float32
        epa = 8
    d.trans_a, d.trans_b, d.trans_c = _TRANS[op]
    tm = TILE_M
    d.tile_shape = [tm, tile_n, tile_k]
    d.warp_tile_shape = [tm, tile_n, tile_k]
    d.tensorop = [128, tile_n, 32 if int8_inference else 16]
    d.num_stage = 3
    d.algo = "Blackwell"
    d.split_k_serial = op == ConvOpType.BackwardWeight
    d.element_per_access_a = d.element_per_access_b = d.element_per_access_c = epa
    d.mask_sparse = True
    d.increment_k_first = True
    d.is_int8_inference = int8_inference
    d.min_arch = (10, 0)
    return d


class ConvMainUnitTest:
    @staticmethod
    def get_all_conv_algo_desp() -> List[ConvAlgoDesp]:
        """cumm/conv/main.py:985-1050.  The reference ships an empty conv kernel list and lets
        its caller supply tile shapes (cumm/conv/main.py:236-239); the sm_100a kernels have a
        fixed 128-row tile and pick the channel tiling from C and K, so the table is short."""
        out = []
        for op in (ConvOpType.Forward, ConvOpType.BackwardInput):
            for tn in (64, 128):
                for tk in (64, 128):
                    out.append(_desp(op, tn, tk))
        for tn in (64, 128):
            out.append(_desp(ConvOpType.BackwardWeight, tn, 128))
            out.append(_desp(ConvOpType.Forward, tn, 128, int8_inference=True))
        return out

    @staticmethod
    def extract_mnk(op_type: int, N: int, C: int, K: int, kernel_volume: int, in_prod: int = -1,
                    out_prod: int = -1, mask_sparse: bool = True) -> Tuple[int, int, int]:
        """cumm/conv/main.py:469-482 -> include/tensorview/gemm/core/utils.h:62-92."""
        if not mask_sparse:
            raise RuntimeError("only mask-sparse implicit GEMM is built")
        return implicit_gemm_mnk(op_type, N, C, K, kernel_volume)

    @staticmethod
    def implicit_gemm2(params: ConvParams) -> None:
        """cumm/conv/main.py:485-745."""
        run_conv(params)
