"""``ConvMainUnitTest``: the static entry points of the reference's sparse-conv dispatcher
(cumm/conv/main.py:469-1050) over the sm_100a kernels."""
from __future__ import annotations

from typing import List, Sequence, Tuple

from ..tensorview.gemm import (ConvAlgoDesp, ConvOpType, ConvParams, implicit_gemm_mnk, run_conv)

TILE_M = 128

def _from_record(r) -> ConvAlgoDesp:
    """A descriptor from one ``cb2_kernel_desp`` record of the library's kernel table."""
    d = ConvAlgoDesp(3, ConvOpType(r.op_type))
    d.dtype_a, d.dtype_b, d.dtype_c = r.dtype_a, r.dtype_b, r.dtype_c
    d.dacc, d.dcomp = r.dacc, r.dcomp
    d.trans_a, d.trans_b, d.trans_c = bool(r.trans_a), bool(r.trans_b), bool(r.trans_c)
    d.tile_shape = list(r.tile_shape)
    d.warp_tile_shape = list(r.warp_tile_shape)
    d.tensorop = list(r.tensorop)
    d.num_stage = r.num_stage
    d.algo = "Blackwell"
    d.split_k_serial = bool(r.split_k_serial)
    d.element_per_access_a = d.element_per_access_b = d.element_per_access_c = r.element_per_access
    d.mask_sparse = bool(r.mask_sparse)
    d.increment_k_first = bool(r.increment_k_first)
    d.is_int8_inference = bool(r.is_int8_inference)
    d.dynamic_mask = bool(r.dynamic_mask)
    d.min_arch = (r.min_arch_major, r.min_arch_minor)
    return d


class ConvMainUnitTest:
    @staticmethod
    def get_all_conv_algo_desp() -> List[ConvAlgoDesp]:
        """cumm/conv/main.py:985-1050.  The reference ships an empty conv kernel list and lets
        its caller supply tile shapes (cumm/conv/main.py:236-239); the sm_100a kernels have a
        fixed 128-row tile and pick the channel tiling from C and K, so the table is short.  It is
        read from the library (``cb2_enumerate_conv_desps``)."""
        from .. import _lib
        return [_from_record(r) for r in _lib.kernel_table("conv")]

    @staticmethod
    def extract_mnk(op_type: int, N: int, C: int, K: int, kernel_volume: int, in_prod: int = -1,
                    out_prod: int = -1, mask_sparse: bool = True) -> Tuple[int, int, int]:
        """cumm/conv/main.py:469-482 -> include/tensorview/gemm/core/utils.h:62-92."""
        if not mask_sparse:
            # dense convolution (include/tensorview/gemm/core/utils.h:62-92): batch times the output
            # positions (forward, backward weight) or the input positions (backward input)
            prod = in_prod if int(op_type) == int(ConvOpType.BackwardInput) else out_prod
            if prod < 0:
                raise RuntimeError("a dense convolution needs in_prod / out_prod")
            N = N * prod
        return implicit_gemm_mnk(op_type, N, C, K, kernel_volume)

    @staticmethod
    def implicit_gemm2(params: ConvParams) -> None:
        """cumm/conv/main.py:485-745."""
        run_conv(params)
