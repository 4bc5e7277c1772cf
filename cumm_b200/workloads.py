"""Seeded synthetic sparse-convolution workloads (host side, numpy).

Stands in for voxelised LiDAR scenes: voxel coordinates are sampled uniformly without
replacement in a (z, y, x) grid, and the per-offset neighbour table, per-row neighbour
masks and the mask sort are derived from them.  The kernels consume these tables in the
layout the reference's callers hand over (``indices [kv, N]`` in original row order with
-1 for a missing neighbour, ``mask [N]`` in *sorted* order, ``mask_argsort [N]``).

Convention (the reference leaves pair generation to its caller): cross-correlation,
``in = out*stride - pad + r*dilation`` per axis as in the reference's dense convolution
iterators (cumm/conv/input_iters.py:2666,2684); filter offset ``f`` is the row-major index
of ``(r_z, r_y, r_x)``; ``mask`` bit ``f`` is set iff ``indices[f, o] >= 0``; the mask sort
is a stable ascending sort of the mask values.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Sequence

import numpy as np

GRID = (41, 1600, 1408)


@dataclass
class ConvTables:
    """Neighbour tables of one sparse-conv layer."""
    n_in: int
    n_out: int
    kv: int
    indices: np.ndarray        # [kv, n_out] int32, -1 = no pair   (forward direction)
    mask: np.ndarray           # [n_out] uint32, sorted ascending ([n_out, words] when kv > 32)
    mask_argsort: np.ndarray   # [n_out] int32
    indices_bwd: np.ndarray    # [kv, n_in] int32                  (input-gradient direction)
    mask_bwd: np.ndarray       # [n_in] uint32, sorted
    mask_argsort_bwd: np.ndarray
    out_coords: np.ndarray     # [n_out, 4] (b, z, y, x)
    num_pairs: int


def sample_coords(n: int, seed, grid: Sequence[int] = GRID, batch: int = 0) -> np.ndarray:
    """`n` unique voxel coordinates, uniform in `grid`; rows are (b, z, y, x) int32."""
    rng = np.random.default_rng(seed)
    lin = rng.choice(int(np.prod(grid)), n, replace=False)
    z, y, x = np.unravel_index(lin, grid)
    b = np.full_like(z, batch)
    return np.stack([b, z, y, x], 1).astype(np.int32)


def dense_block_coords(side: int, batch: int = 0) -> np.ndarray:
    """All voxels of a solid side^3 cube: the contraction-bound stress input (about 27
    neighbours per voxel).  Not one of the benchmark configurations."""
    z, y, x = np.meshgrid(np.arange(side), np.arange(side), np.arange(side), indexing="ij")
    b = np.full(z.size, batch)
    return np.stack([b, z.ravel(), y.ravel(), x.ravel()], 1).astype(np.int32)


def _linear(coords: np.ndarray, grid) -> np.ndarray:
    c = coords.astype(np.int64)
    return ((c[:, 0] * grid[0] + c[:, 1]) * grid[1] + c[:, 2]) * grid[2] + c[:, 3]


def neighbour_table(in_coords, out_coords, grid, ksize, stride, pad, dil) -> np.ndarray:
    """indices[f, o] by sorted-key lookup (vectorised; no hash table)."""
    keys = _linear(in_coords, grid)
    order = np.argsort(keys, kind="stable")
    skeys = keys[order]
    n_out = len(out_coords)
    kv = int(np.prod(ksize))
    indices = np.full((kv, n_out), -1, np.int32)
    oc = out_coords.astype(np.int64)
    f = 0
    for rz in range(ksize[0]):
        for ry in range(ksize[1]):
            for rx in range(ksize[2]):
                z = oc[:, 1] * stride[0] - pad[0] + rz * dil[0]
                y = oc[:, 2] * stride[1] - pad[1] + ry * dil[1]
                x = oc[:, 3] * stride[2] - pad[2] + rx * dil[2]
                ok = (z >= 0) & (z < grid[0]) & (y >= 0) & (y < grid[1]) & (x >= 0) & (x < grid[2])
                q = ((oc[:, 0] * grid[0] + z) * grid[1] + y) * grid[2] + x
                pos = np.searchsorted(skeys, q)
                pos = np.minimum(pos, len(skeys) - 1)
                hit = ok & (skeys[pos] == q)
                indices[f, hit] = order[pos[hit]].astype(np.int32)
                f += 1
    return indices


def masks_from_indices(indices: np.ndarray) -> np.ndarray:
    """Per-row neighbour masks: [n] for kernel volumes up to 32, else [n, ceil(kv / 32)] with
    word w covering offsets 32w .. 32w+31 (the layout of the reference's dynamic-mask kernels,
    cumm/gemm/blockmma/mma.py:78-270)."""
    kv = indices.shape[0]
    words = (kv + 31) // 32
    mask = np.zeros((indices.shape[1], words), np.uint32)
    for f in range(kv):
        mask[:, f >> 5] |= (indices[f] >= 0).astype(np.uint32) << np.uint32(f & 31)
    return mask[:, 0].copy() if words == 1 else mask


def sort_masks(mask: np.ndarray):
    """Stable ascending sort; masks of several words compare as one integer whose most
    significant word is the last one."""
    if mask.ndim == 2:
        order = np.lexsort(tuple(mask[:, w] for w in range(mask.shape[1]))).astype(np.int32)
    else:
        order = np.argsort(mask, kind="stable").astype(np.int32)
    return np.ascontiguousarray(mask[order]), order


def invert_table(indices: np.ndarray, n_in: int) -> np.ndarray:
    kv = indices.shape[0]
    out = np.full((kv, n_in), -1, np.int32)
    for f in range(kv):
        o = np.nonzero(indices[f] >= 0)[0]
        out[f, indices[f, o]] = o.astype(np.int32)
    return out


def regular_out_coords(in_coords, grid, ksize, stride, pad, dil):
    """Active output voxels of a regular sparse conv, ordered by linearised (b,z,y,x)."""
    ic = in_coords.astype(np.int64)
    og = [(grid[a] + 2 * pad[a] - dil[a] * (ksize[a] - 1) - 1) // stride[a] + 1 for a in range(3)]
    found = []
    for rz in range(ksize[0]):
        for ry in range(ksize[1]):
            for rx in range(ksize[2]):
                r = (rz, ry, rx)
                ok = np.ones(len(ic), bool)
                q = []
                for a in range(3):
                    num = ic[:, a + 1] + pad[a] - r[a] * dil[a]
                    ok &= num % stride[a] == 0
                    v = num // stride[a]
                    ok &= (v >= 0) & (v < og[a])
                    q.append(v)
                lin = ((ic[:, 0] * og[0] + q[0]) * og[1] + q[1]) * og[2] + q[2]
                found.append(lin[ok])
    lin = np.unique(np.concatenate(found))
    x = lin % og[2]
    y = (lin // og[2]) % og[1]
    z = (lin // (og[2] * og[1])) % og[0]
    b = lin // (og[2] * og[1] * og[0])
    return np.stack([b, z, y, x], 1).astype(np.int32), og


def build_tables(in_coords: np.ndarray, grid=GRID, ksize=(3, 3, 3), stride=(1, 1, 1),
                 pad: Optional[Sequence[int]] = None, dil=(1, 1, 1), subm: bool = True) -> ConvTables:
    """Tables for a submanifold (`subm`, outputs = inputs) or regular sparse conv."""
    if pad is None:
        pad = tuple(k // 2 for k in ksize)
    if subm:
        out_coords = in_coords
    else:
        out_coords, _ = regular_out_coords(in_coords, grid, ksize, stride, pad, dil)
    indices = neighbour_table(in_coords, out_coords, grid, ksize, stride, pad, dil)
    mask, order = sort_masks(masks_from_indices(indices))
    ibwd = invert_table(indices, len(in_coords))
    mbwd, obwd = sort_masks(masks_from_indices(ibwd))
    return ConvTables(len(in_coords), len(out_coords), indices.shape[0], indices, mask, order,
                      ibwd, mbwd, obwd, out_coords, int((indices >= 0).sum()))


def concat_scenes(tables: Sequence[ConvTables]) -> ConvTables:
    """Stack independent scenes into one batch: rows are renumbered, masks re-sorted."""
    kv = tables[0].kv
    n_in = sum(t.n_in for t in tables)
    n_out = sum(t.n_out for t in tables)
    indices = np.full((kv, n_out), -1, np.int32)
    io = oo = 0
    for t in tables:
        blk = t.indices.copy()
        blk[blk >= 0] += io
        indices[:, oo:oo + t.n_out] = blk
        io += t.n_in
        oo += t.n_out
    mask, order = sort_masks(masks_from_indices(indices))
    ibwd = invert_table(indices, n_in)
    mbwd, obwd = sort_masks(masks_from_indices(ibwd))
    oc = np.concatenate([t.out_coords for t in tables])
    return ConvTables(n_in, n_out, kv, indices, mask, order, ibwd, mbwd, obwd, oc,
                      int((indices >= 0).sum()))
