"""Seeded synthetic voxel scenes with the shapes, sizes and occupancy statistics of the
workloads this library is measured on.  They stand in for real indoor scans (no dataset is
shipped or reproduced): only geometry statistics matter to the attention path — how many
voxels, how they fall into windows, and how many share a window.

All generators return int32 coordinates ``[N, 4]`` = (batch, z, y, x) with unique rows, plus the
dense grid dims ``(D, H, W)`` the coordinates live in.  numpy's PCG64 generator is used so that
the same seed gives the same scene on every machine.
"""
from __future__ import annotations

from typing import Tuple

import numpy as np

Dims = Tuple[int, int, int]


def uniform_scene(n_voxels: int = 20_000, grid: int = 128, seed: int = 0, batch_index: int = 0):
    """`n_voxels` distinct cells drawn uniformly from a `grid`^3 cube (volume-sparse: most
    windows hold only a few voxels)."""
    rng = np.random.default_rng(seed)
    flat = rng.choice(grid ** 3, size=n_voxels, replace=False)
    z, y, x = np.unravel_index(flat, (grid, grid, grid))
    coords = np.stack([np.full_like(z, batch_index), z, y, x], axis=1).astype(np.int32)
    return coords, (grid, grid, grid)


def _sample_rect(rng, n, origin, u, v):
    """n points uniform on the parallelogram origin + a*u + b*v, a,b in [0,1)."""
    a = rng.random((n, 1))
    b = rng.random((n, 1))
    return origin[None, :] + a * u[None, :] + b * v[None, :]


def room_scene(n_voxels: int = 150_000, seed: int = 0, batch_index: int = 0,
               room_m=(8.0, 8.0, 3.0), voxel_m: float = 0.02, n_boxes: int = 20):
    """A surface-sparse indoor room: floor, four walls and `n_boxes` axis-aligned boxes
    (sides 0.3-2 m, standing on the floor).  Points are sampled uniformly by surface area,
    voxelised at `voxel_m`, de-duplicated, and a uniform subset of exactly `n_voxels`
    occupied cells is kept.  Dense dims are (D,H,W) = (x cells, y cells, z cells) =
    (400, 400, 150) for the default 8 x 8 x 3 m room at 2 cm."""
    rng = np.random.default_rng(seed)
    X, Y, Z = room_m
    rects = []  # (origin, u, v)
    e = np.eye(3)
    rects.append((np.zeros(3), e[0] * X, e[1] * Y))  # floor
    rects.append((np.zeros(3), e[0] * X, e[2] * Z))  # wall y=0
    rects.append((np.array([0, Y - 1e-6, 0]), e[0] * X, e[2] * Z))  # wall y=Y
    rects.append((np.zeros(3), e[1] * Y, e[2] * Z))  # wall x=0
    rects.append((np.array([X - 1e-6, 0, 0]), e[1] * Y, e[2] * Z))  # wall x=X
    for _ in range(n_boxes):
        s = rng.uniform(0.3, 2.0, size=3)
        s[2] = min(s[2], Z - 0.05)
        o = np.array([rng.uniform(0, X - s[0]), rng.uniform(0, Y - s[1]), 0.0])
        sx, sy, sz = e[0] * s[0], e[1] * s[1], e[2] * s[2]
        rects += [(o + sz, sx, sy),  # top
                  (o, sx, sz), (o + sy, sx, sz),  # two faces along x
                  (o, sy, sz), (o + sx, sy, sz)]  # two faces along y
    areas = np.array([np.linalg.norm(np.cross(u, v)) for _, u, v in rects])
    dims = (int(round(X / voxel_m)), int(round(Y / voxel_m)), int(round(Z / voxel_m)))
    cells = np.zeros((0,), dtype=np.int64)
    n_samples = int(n_voxels * 1.4)
    for _ in range(8):
        counts = rng.multinomial(n_samples, areas / areas.sum())
        pts = np.concatenate([_sample_rect(rng, c, *r) for c, r in zip(counts, rects) if c > 0])
        ijk = np.floor(pts / voxel_m).astype(np.int64)
        ijk = np.clip(ijk, 0, np.array(dims) - 1)
        flat = (ijk[:, 0] * dims[1] + ijk[:, 1]) * dims[2] + ijk[:, 2]
        cells = np.unique(np.concatenate([cells, flat]))
        if cells.size >= n_voxels:
            break
    if cells.size < n_voxels:
        raise ValueError("room surface has fewer cells than requested voxels")
    keep = rng.choice(cells.size, size=n_voxels, replace=False)
    flat = cells[np.sort(keep)]
    rng.shuffle(flat)  # voxel order in memory carries no spatial locality
    d0 = flat // (dims[1] * dims[2])
    d1 = (flat // dims[2]) % dims[1]
    d2 = flat % dims[2]
    coords = np.stack([np.full_like(d0, batch_index), d0, d1, d2], axis=1).astype(np.int32)
    return coords, dims


def downsample_scene(coords: np.ndarray, dims: Dims, stride: int = 2):
    """Coordinates of the next Swin stage: unique(coords // stride), as a stride-2 sparse
    convolution would produce."""
    c = coords.astype(np.int64).copy()
    c[:, 1:] //= stride
    nd = tuple((d + stride - 1) // stride for d in dims)
    flat = ((c[:, 0] * nd[0] + c[:, 1]) * nd[1] + c[:, 2]) * nd[2] + c[:, 3]
    _, first = np.unique(flat, return_index=True)
    return c[np.sort(first)].astype(np.int32), nd


def skewed_scene(grid: int = 126, window: int = 9, p_dense: float = 0.5, seed: int = 0, batch_index: int = 0):
    """Skewed-occupancy stress scene: every `window`^3 block of a `grid`^3 cube is either fully
    dense (probability `p_dense`) or holds 1-8 random cells."""
    rng = np.random.default_rng(seed)
    nw = grid // window
    n = window ** 3
    chunks = []
    for wz in range(nw):
        for wy in range(nw):
            for wx in range(nw):
                if rng.random() < p_dense:
                    local = np.arange(n)
                else:
                    local = rng.choice(n, size=int(rng.integers(1, 9)), replace=False)
                lz, ly, lx = np.unravel_index(local, (window, window, window))
                chunks.append(np.stack([wz * window + lz, wy * window + ly, wx * window + lx], axis=1))
    zyx = np.concatenate(chunks)
    rng.shuffle(zyx, axis=0)
    coords = np.concatenate([np.full((zyx.shape[0], 1), batch_index), zyx], axis=1).astype(np.int32)
    return coords, (grid, grid, grid)


def window_stats(coords: np.ndarray, dims: Dims, window: int = 7):
    """Occupancy statistics used in reports: non-empty windows, sum c, sum c^2, max c."""
    pd = [((d + window - 1) // window) for d in dims]
    w = ((coords[:, 0].astype(np.int64) * pd[0] + coords[:, 1] // window) * pd[1] + coords[:, 2] // window) * pd[2] \
        + coords[:, 3] // window
    _, c = np.unique(w, return_counts=True)
    return {"windows": int(c.size), "voxels": int(c.sum()), "sum_c2": int((c.astype(np.int64) ** 2).sum()),
            "c_max": int(c.max()), "c_median": float(np.median(c))}
