"""Seeded inputs shared by the parity tests (CPU tensors; tests move them to the device)."""
from __future__ import annotations

import torch

from oracle import ssw_oracle as O
from sparseswin3d_b200 import scenes


def make_case(n_vox=3000, grid=40, heads=3, head_dim=32, window=(7, 7, 7), shift=(0, 0, 0), seed=0, batch=1,
              table_std=0.5, dims=None):
    """Uniform random voxels in a cube (or `dims`), random qkv and bias table; returns a dict with
    everything the oracle and the CUDA path need."""
    g = torch.Generator().manual_seed(seed)
    import numpy as np

    if dims is None:
        dims = (grid, grid, grid)
    rng = np.random.default_rng(seed)
    per = []
    for b in range(batch):
        flat = rng.choice(dims[0] * dims[1] * dims[2], size=n_vox, replace=False)
        z, y, x = np.unravel_index(flat, dims)
        per.append(np.stack([np.full_like(z, b), z, y, x], 1))
    coords = torch.from_numpy(np.concatenate(per).astype(np.int32))
    idx, Bw, n, ws, ss, dp = O.window_keys(coords, batch, dims, window, shift)
    N = coords.shape[0]
    qkv = torch.randn(N, 3, heads, head_dim, generator=g)
    table = torch.randn((2 * window[0] - 1) * (2 * window[1] - 1) * (2 * window[2] - 1), heads, generator=g) * table_std
    rpi = O.relative_position_index(window)
    mask = O.compute_mask(dp, ws, ss) if any(s > 0 for s in ss) else None
    return dict(coords=coords, dims=dims, batch=batch, window=window, shift=shift, indices=idx, n_windows=Bw, n=n,
                ws=ws, ss=ss, dims_p=dp, qkv=qkv, table=table, rpi=rpi, mask=mask, heads=heads, head_dim=head_dim,
                scale=head_dim ** -0.5)


def rel_err(x: torch.Tensor, ref: torch.Tensor) -> float:
    """max |x - ref| / max(|ref|, rms(ref)) — the tolerance form used for value parity."""
    ref = ref.double()
    x = x.double()
    rms = ref.pow(2).mean().sqrt().clamp_min(1e-30)
    return float(((x - ref).abs() / torch.maximum(ref.abs(), rms)).max()) if ref.numel() else 0.0


def digest_i64(a) -> int:
    """Order-sensitive checksum of an integer array (wraps in int64, deterministically)."""
    import numpy as np

    a = np.asarray(a).reshape(-1).astype(np.int64)
    w = (np.arange(a.size, dtype=np.int64) % 1000003) + 1
    with np.errstate(over="ignore"):
        return int((a * w).sum() & np.int64(2 ** 62 - 1))


def room_crop_case(shift=(0, 0, 0), crop=200, heads=3, head_dim=32, window=(7, 7, 7), seed=0):
    """The x,y < crop corner of the benchmark's 150 000-voxel room (about 36 000 voxels): large and
    surface-sparse like the benchmark scene, and still inside upstream's int32 index domain."""
    import numpy as np

    coords, dims = scenes.room_scene(150_000, seed=seed)
    keep = (coords[:, 1] < crop) & (coords[:, 2] < crop)
    coords = torch.from_numpy(coords[keep].copy())
    dims = (crop, crop, dims[2])
    idx, Bw, n, ws, ss, dp = O.window_keys(coords, 1, dims, window, shift)
    g = torch.Generator().manual_seed(1000 + seed)
    qkv = torch.randn(coords.shape[0], 3, heads, head_dim, generator=g)
    table = torch.randn((2 * window[0] - 1) ** 3, heads, generator=g) * 0.5
    mask = O.compute_mask(dp, ws, ss) if any(s > 0 for s in ss) else None
    return dict(coords=coords, dims=dims, batch=1, window=window, shift=shift, indices=idx, n_windows=Bw, n=n, ws=ws,
                ss=ss, dims_p=dp, qkv=qkv, table=table, rpi=O.relative_position_index(window), mask=mask, heads=heads,
                head_dim=head_dim, scale=head_dim ** -0.5)


def skewed_case(grid=27, shift=(4, 4, 4), heads=6, head_dim=32, seed=3):
    """The skewed-occupancy stress shape at reduced size: window 9^3, half of the windows completely
    full (729 voxels), the rest with 1-8 voxels."""
    window = (9, 9, 9)
    coords_np, dims = scenes.skewed_scene(grid=grid, window=9, p_dense=0.5, seed=seed)
    coords = torch.from_numpy(coords_np)
    idx, Bw, n, ws, ss, dp = O.window_keys(coords, 1, dims, window, shift)
    g = torch.Generator().manual_seed(7 + seed)
    qkv = torch.randn(coords.shape[0], 3, heads, head_dim, generator=g)
    table = torch.randn(17 ** 3, heads, generator=g) * 0.5
    mask = O.compute_mask(dp, ws, ss) if any(s > 0 for s in ss) else None
    return dict(coords=coords, dims=dims, batch=1, window=window, shift=shift, indices=idx, n_windows=Bw, n=n, ws=ws,
                ss=ss, dims_p=dp, qkv=qkv, table=table, rpi=O.relative_position_index(window), mask=mask, heads=heads,
                head_dim=head_dim, scale=head_dim ** -0.5)
