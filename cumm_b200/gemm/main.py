"""``GemmMainUnitTest``: the static entry points of the reference's GEMM dispatcher
(cumm/gemm/main.py:916-1335) over the sm_100a kernels."""
from __future__ import annotations

from typing import Dict, List, Sequence, Tuple

from ..tensorview.gemm import GemmAlgoDesp, GemmParams, ShuffleStrideType, run_gemm

TILE_M = 128


def _from_record(r) -> GemmAlgoDesp:
    """A descriptor from one ``cb2_kernel_desp`` record of the library's kernel table."""
    d = GemmAlgoDesp()
    d.dtype_a, d.dtype_b, d.dtype_c = r.dtype_a, r.dtype_b, r.dtype_c
    d.dacc, d.dcomp = r.dacc, r.dcomp
    d.trans_a, d.trans_b, d.trans_c = bool(r.trans_a), bool(r.trans_b), bool(r.trans_c)
    d.tile_shape = list(r.tile_shape)
    d.warp_tile_shape = list(r.warp_tile_shape)  # one tcgen05 instruction stream per CTA tile
    d.tensorop = list(r.tensorop)
    d.num_stage = r.num_stage
    d.algo = "Blackwell"
    d.shuffle_type = ShuffleStrideType(r.shuffle_type)
    d.split_k_serial = bool(r.split_k_serial)
    d.element_per_access_a = d.element_per_access_b = d.element_per_access_c = r.element_per_access
    d.min_arch = (r.min_arch_major, r.min_arch_minor)
    return d


class GemmMainUnitTest:
    """Stateless; every method is static like the reference's pybind class."""

    @staticmethod
    def get_all_algo_desp() -> List[GemmAlgoDesp]:
        """cumm/gemm/main.py:916-965.  The kernel table, read from the library
        (``cb2_enumerate_gemm_desps``): row-gather GEMMs (ShuffleAC / dense) with B given as
        [n,k] or [k,n], and the gather-gather weight-gradient GEMM (ShuffleAB)."""
        from .. import _lib
        return [_from_record(r) for r in _lib.kernel_table("gemm")]

    @staticmethod
    def extract_mnk(a_shape: Sequence[int], b_shape: Sequence[int], trans_a: bool, trans_b: bool,
                    trans_c: bool, shuffle_type: int = 0, a_inds_shape: Sequence[int] = (),
                    b_inds_shape: Sequence[int] = (), c_inds_shape: Sequence[int] = ()) -> Tuple[int, int, int]:
        """cumm/gemm/main.py:969-1027."""
        a_shape, b_shape = list(a_shape), list(b_shape)
        if trans_c:
            trans_a, trans_b = (not trans_b), (not trans_a)
            a_shape, b_shape = b_shape, a_shape
        if shuffle_type == ShuffleStrideType.ShuffleAC:
            if trans_a:
                raise RuntimeError("a of shuffle AB must be row major")
            if not len(c_inds_shape):
                raise RuntimeError("c_inds must not empty")
            m = a_inds_shape[0] if len(a_inds_shape) else a_shape[0]
            k = a_shape[int(not trans_a)]
            n = b_shape[int(not trans_b)]
        elif shuffle_type == ShuffleStrideType.ShuffleAB:
            if not (len(a_inds_shape) and len(b_inds_shape)):
                raise RuntimeError("a_inds and c_inds must not empty")
            if not (trans_a and not trans_b):
                raise RuntimeError("shuffle AB must be nt, i.e. backward weight")
            m = a_shape[int(trans_a)]
            k = a_inds_shape[0]
            n = b_shape[int(not trans_b)]
        else:
            m = a_shape[int(trans_a)]
            k = a_shape[int(not trans_a)]
            n = b_shape[int(not trans_b)]
        return int(m), int(n), int(k)

    @staticmethod
    def align_to_power2(val: int) -> int:
        """cumm/gemm/main.py:1030-1049: smallest power of two >= val (val itself if it is one)."""
        r = 0
        ones = 1 if val & 1 else 0
        while True:
            val >>= 1
            if not val:
                break
            r += 1
            if val & 1:
                ones += 1
        return 1 << r if ones == 1 else 1 << (r + 1)

    @staticmethod
    def device_synchronize() -> None:
        import torch
        torch.cuda.synchronize()

    @staticmethod
    def stream_synchronize(stream: int) -> None:
        import torch
        torch.cuda.ExternalStream(int(stream)).synchronize() if stream else torch.cuda.current_stream().synchronize()

    @staticmethod
    def simple_select_tile_shape(m: int, n: int, k: int, tile_ms: Sequence[int], tile_ns: Sequence[int],
                                 tile_ks: Sequence[int], tile_shape_to_algos: Dict[int, List[int]],
                                 large_k_first: bool) -> List[int]:
        """cumm/gemm/main.py:1074-1134: smallest listed tile >= (m, n, k) by lower bound,
        then scan downwards for a tile that has kernels."""
        import bisect

        def target(vals, x):
            i = bisect.bisect_left(list(vals), x)
            return min(i, len(vals) - 1)

        im, in_, ik = target(tile_ms, m), target(tile_ns, n), target(tile_ks, k)

        def key(tm, tn, tk):
            return tm | (tn << 20) | (tk << 40)

        if large_k_first:
            order = ((a, b, c) for c in range(ik, -1, -1) for b in range(in_, -1, -1) for a in range(im, -1, -1))
        else:
            order = ((a, b, c) for a in range(im, -1, -1) for b in range(in_, -1, -1) for c in range(ik, -1, -1))
        for a, b, c in order:
            hit = tile_shape_to_algos.get(key(tile_ms[a], tile_ns[b], tile_ks[c]))
            if hit is not None:
                return list(hit)
        return []

    @staticmethod
    def matmul2(params: GemmParams) -> None:
        """cumm/gemm/main.py:1178-1335."""
        run_gemm(params)
