"""Tile-shape tuner: picks the descriptor (kernel variant) by measured time and remembers it.

The reference's tuner lives in its caller (spconv) on top of the lists this package mirrors
(``GemmMainUnitTest.get_all_algo_desp`` / ``ConvMainUnitTest.get_all_conv_algo_desp``,
cumm/gemm/main.py:916-965, cumm/conv/main.py:985-1050): it runs every supported descriptor on
the real tensors, times it with events and keeps the fastest per problem key.  This module does
the same over the sm_100a kernels, where a descriptor's ``tile_shape`` selects the variant:
``tile_shape[1]`` = output columns of one CTA tile (64 | 128), ``tile_shape[2]`` = reduction
elements per pipeline stage (fp16: 64 | 128).

The choice is cached per (operation, dtypes, C, K, kernel volume, size bucket, device name) in
memory and, when a path is given, in a JSON file, so that a tuned process does not measure
again.  Timing uses CUDA events around back-to-back launches of the prepared call on the
caller's own tensors (outputs are overwritten: tune before the values matter, or on scratch).
"""
from __future__ import annotations

import json
import os
import threading
from pathlib import Path
from typing import Callable, Dict, Iterable, List, Optional, Sequence, Tuple

from .conv.main import ConvMainUnitTest
from .gemm.main import GemmMainUnitTest
from .tensorview import as_view
from .tensorview.gemm import (ConvAlgoDesp, ConvOpType, ConvParams, GemmAlgoDesp, GemmParams, ShuffleStrideType,
                              implicit_gemm_mnk, prepare_conv, prepare_gemm)

CACHE_ENV = "CUMM_B200_TUNE_CACHE"
_FORMAT = 1


def size_bucket(n: int) -> int:
    """Problems within a factor of two in rows share a choice: ceil(log2(n)), 0 for n <= 1."""
    return 0 if n <= 1 else int(n - 1).bit_length()


def conv_key(desp: ConvAlgoDesp, N: int, C: int, K: int, kv: int, device_name: str) -> str:
    return "conv|op{}|a{}b{}c{}|i8{}|C{}|K{}|kv{}|n{}|{}".format(
        int(desp.op_type), int(desp.dtype_a), int(desp.dtype_b), int(desp.dtype_c), int(bool(desp.is_int8_inference)),
        C, K, kv, size_bucket(N), device_name)


def gemm_key(desp: GemmAlgoDesp, m: int, n: int, k: int, device_name: str) -> str:
    return "gemm|s{}|ta{}tb{}|a{}b{}c{}|m{}|n{}|k{}|{}".format(
        int(desp.shuffle_type), int(bool(desp.trans_a)), int(bool(desp.trans_b)), int(desp.dtype_a), int(desp.dtype_b),
        int(desp.dtype_c), size_bucket(m), n if desp.shuffle_type != ShuffleStrideType.ShuffleAB else size_bucket(n),
        k if desp.shuffle_type != ShuffleStrideType.ShuffleAB else size_bucket(k), device_name)


def conv_candidates(desp: ConvAlgoDesp) -> List[Tuple[int, int, int]]:
    """Tile shapes of the listed descriptors for this operation and dtype family."""
    out = []
    for d in ConvMainUnitTest.get_all_conv_algo_desp():
        if int(d.op_type) == int(desp.op_type) and bool(d.is_int8_inference) == bool(desp.is_int8_inference) \
                and int(d.dtype_a) == int(desp.dtype_a):
            t = tuple(int(v) for v in d.tile_shape)
            if t not in out:
                out.append(t)
    return out


def gemm_candidates(desp: GemmAlgoDesp) -> List[Tuple[int, int, int]]:
    out = []
    for d in GemmMainUnitTest.get_all_algo_desp():
        if int(d.shuffle_type) == int(desp.shuffle_type) and bool(d.trans_a) == bool(desp.trans_a) \
                and bool(d.trans_b) == bool(desp.trans_b) and int(d.dtype_a) == int(desp.dtype_a):
            t = tuple(int(v) for v in d.tile_shape)
            if t not in out:
                out.append(t)
    return out


def _cuda_timer(launch: Callable[[], None], stream: int, warmup: int, reps: int) -> float:
    """Median microseconds per launch over ``reps`` batches of four back-to-back launches."""
    import torch
    s = torch.cuda.ExternalStream(stream) if stream else torch.cuda.current_stream()
    for _ in range(warmup):
        launch()
    s.synchronize()
    times = []
    for _ in range(reps):
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record(s)
        for _ in range(4):
            launch()
        b.record(s)
        s.synchronize()
        times.append(a.elapsed_time(b) * 1e3 / 4)
    times.sort()
    return times[len(times) // 2]


class Tuner:
    """Measured selection with a persisted cache.  ``timer(launch, stream, warmup, reps) -> us`` can
    be replaced (the CPU tests pass a table of made-up times)."""

    def __init__(self, cache_path: Optional[str] = None, timer: Optional[Callable] = None, warmup: int = 2,
                 reps: int = 5, device_name: Optional[str] = None):
        self._path = Path(cache_path or os.environ.get(CACHE_ENV, "")) if (cache_path or os.environ.get(CACHE_ENV)) \
            else None
        self._timer = timer or _cuda_timer
        self._warmup, self._reps = warmup, reps
        self._device_name = device_name
        self._lock = threading.Lock()
        self._cache: Dict[str, dict] = {}
        self.measurements = 0  # candidates timed by this object (0 when everything came from the cache)
        if self._path is not None and self._path.exists():
            self._load()

    # ---------------------------------------------------------------- cache
    def _load(self) -> None:
        try:
            blob = json.loads(self._path.read_text())
        except (OSError, ValueError):
            return  # an unreadable cache is the same as none
        if isinstance(blob, dict) and blob.get("format") == _FORMAT and isinstance(blob.get("entries"), dict):
            self._cache.update(blob["entries"])

    def _save(self) -> None:
        if self._path is None:
            return
        self._path.parent.mkdir(parents=True, exist_ok=True)
        tmp = self._path.with_suffix(self._path.suffix + ".tmp")
        tmp.write_text(json.dumps({"format": _FORMAT, "entries": self._cache}, indent=1, sort_keys=True))
        os.replace(tmp, self._path)

    def cached(self, key: str) -> Optional[Tuple[int, int, int]]:
        e = self._cache.get(key)
        return tuple(e["tile_shape"]) if e else None

    def entries(self) -> Dict[str, dict]:
        return dict(self._cache)

    def _device(self) -> str:
        if self._device_name is None:
            import torch
            self._device_name = torch.cuda.get_device_name(torch.cuda.current_device()).replace(" ", "_")
        return self._device_name

    # ---------------------------------------------------------------- selection
    def _select(self, key: str, candidates: Sequence[Tuple[int, int, int]], make_launch, stream: int):
        with self._lock:
            hit = self.cached(key)
            if hit is not None and hit in [tuple(c) for c in candidates]:
                return hit
            results = []
            for tile in candidates:
                try:
                    launch = make_launch(tile)
                except (RuntimeError, ValueError):
                    continue  # this variant does not support the problem (alignment, workspace, ...)
                us = float(self._timer(launch, stream, self._warmup, self._reps))
                self.measurements += 1
                results.append((us, tuple(tile)))
            if not results:
                raise RuntimeError("can't find any suitable algo: no listed tile shape supports this problem")
            results.sort()
            best_us, best = results[0]
            self._cache[key] = {"tile_shape": list(best), "us": best_us,
                                "tried": {"x".join(map(str, t)): us for us, t in results}}
            self._save()
            return best

    def tune_conv(self, params: ConvParams) -> ConvAlgoDesp:
        """Returns a copy of ``params.conv_algo_desp`` with the fastest listed tile shape for this
        problem (measured on ``params``'s own tensors unless cached); ``params`` is left as it is."""
        desp = params.conv_algo_desp
        inp, weight = as_view(params.input), as_view(params.weight)
        indices = as_view(params.indices)
        if inp is None or weight is None or indices is None:
            raise RuntimeError("input, weight, indices must not empty")
        K, kv, C = weight.dim(0), weight.dim(1), weight.dim(2)
        N = indices.dim(1)
        key = conv_key(desp, N, C, K, kv, self._device())
        saved = (list(desp.tile_shape), list(desp.warp_tile_shape))

        def make_launch(tile):
            desp.tile_shape = [tile[0], tile[1], tile[2] if int(desp.op_type) != int(ConvOpType.BackwardWeight)
                               else saved[0][2]]
            desp.warp_tile_shape = list(desp.tile_shape)
            return prepare_conv(params).launch

        try:
            best = self._select(key, conv_candidates(desp), make_launch, int(params.stream))
        finally:
            desp.tile_shape, desp.warp_tile_shape = saved
        out = desp.copy()
        out.tile_shape = [best[0], best[1], best[2] if int(desp.op_type) != int(ConvOpType.BackwardWeight)
                          else saved[0][2]]
        out.warp_tile_shape = list(out.tile_shape)
        out.tensorop = [128, out.tile_shape[1], out.tensorop[2]]
        return out

    def tune_gemm(self, params: GemmParams) -> GemmAlgoDesp:
        desp = params.algo_desp
        a, b = as_view(params.a), as_view(params.b)
        if a is None or b is None:
            raise RuntimeError("a, b must not empty")
        a_inds = as_view(params.a_inds)
        m, n, k = GemmMainUnitTest.extract_mnk(a.shape, b.shape, desp.trans_a, desp.trans_b, desp.trans_c,
                                               int(desp.shuffle_type), a_inds.shape if a_inds is not None else [],
                                               as_view(params.b_inds).shape if params.b_inds is not None else [],
                                               as_view(params.c_inds).shape if params.c_inds is not None else [])
        key = gemm_key(desp, m, n, k, self._device())
        saved = (list(desp.tile_shape), list(desp.warp_tile_shape))

        def make_launch(tile):
            desp.tile_shape = list(tile)
            desp.warp_tile_shape = list(tile)
            return prepare_gemm(params).launch

        try:
            best = self._select(key, gemm_candidates(desp), make_launch, int(params.stream))
        finally:
            desp.tile_shape, desp.warp_tile_shape = saved
        out = desp.copy()
        out.tile_shape = list(best)
        out.warp_tile_shape = list(best)
        out.tensorop = [128, best[1], out.tensorop[2]]
        return out
