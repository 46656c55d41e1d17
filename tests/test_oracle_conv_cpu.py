"""CPU: the oracle's sparse convolutions (dense conv3d / conv_transpose3d read at the active sites)
against the definition written out as loops over voxels and kernel taps, on tiny scenes."""
import itertools

import torch

from oracle import ssw_oracle as O
from tests.cases import make_case


def _lut(coords):
    return {tuple(c): i for i, c in enumerate(coords.tolist())}


def test_submanifold_definition():
    dims, batch = (5, 6, 4), 2
    coords = make_case(n_vox=40, dims=dims, batch=batch, seed=1)["coords"]
    g = torch.Generator().manual_seed(0)
    x = torch.randn(coords.shape[0], 3, generator=g, dtype=torch.float64)
    w = torch.randn(27, 3, 5, generator=g, dtype=torch.float64)
    bias = torch.randn(5, generator=g, dtype=torch.float64)
    lut = _lut(coords)
    want = bias.repeat(coords.shape[0], 1)
    for i, (b, z, y, xx) in enumerate(coords.tolist()):
        for t, (dz, dy, dx) in enumerate(itertools.product((-1, 0, 1), repeat=3)):
            j = lut.get((b, z + dz, y + dy, xx + dx))
            if j is not None:
                want[i] += x[j] @ w[t]
    got = O.subm_conv3d(x, coords, batch, dims, w, bias)
    assert torch.allclose(got, want, atol=1e-12)


def test_strided_and_inverse_definition():
    dims, batch, k = (7, 6, 5), 1, 2            # 7 and 5 are odd: the last plane has no output cell
    coords = make_case(n_vox=60, dims=dims, batch=batch, seed=2)["coords"]
    g = torch.Generator().manual_seed(1)
    x = torch.randn(60, 4, generator=g, dtype=torch.float64)
    w = torch.randn(8, 4, 6, generator=g, dtype=torch.float64)
    od = [(d - k) // k + 1 for d in dims]
    cells = {}
    for i, (b, z, y, xx) in enumerate(coords.tolist()):
        if z < od[0] * k and y < od[1] * k and xx < od[2] * k:
            cells.setdefault((b, z // k, y // k, xx // k), []).append((i, ((z % k) * k + y % k) * k + xx % k))
    keys = sorted(cells)
    want = torch.stack([sum(x[i] @ w[t] for i, t in cells[c]) for c in keys])
    got, idx, got_od = O.strided_conv3d(x, coords, batch, dims, w)
    assert got_od == od and idx.tolist() == [list(c) for c in keys]
    assert torch.allclose(got, want, atol=1e-12)
    # inverse: every fine voxel gets its parent's row through the tap it occupies; none -> zero
    wi = torch.randn(8, 6, 4, generator=g, dtype=torch.float64)
    pos = {c: m for m, c in enumerate(keys)}
    want_inv = torch.zeros(60, 4, dtype=torch.float64)
    for c, members in cells.items():
        for i, t in members:
            want_inv[i] = got[pos[c]] @ wi[t]
    got_inv = O.inverse_conv3d(got, idx, batch, od, coords, wi)
    assert torch.allclose(got_inv, want_inv, atol=1e-12)
    assert int((want_inv.abs().sum(1) == 0).sum()) > 0      # the scene does have voxels in the dropped planes
