"""CPU: the shared library loads and exports every symbol the public header declares; host-only
entry points (geometry, layouts, workspace sizes, argument validation) behave; no compute call is
made here."""
import ctypes
import re
from pathlib import Path

import pytest
import torch

from oracle import ssw_oracle as O

ROOT = Path(__file__).resolve().parents[1]


def _declared():
    text = (ROOT / "include" / "ssw_b200.h").read_text()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(ssw_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    from sparseswin3d_b200 import _lib

    names = _declared()
    assert len(names) >= 25
    raw = ctypes.CDLL(str(_lib.LIB_PATH))
    missing = [n for n in names if not hasattr(raw, n)]
    assert not missing, missing
    assert _lib.lib.ssw_version() >= 100
    assert _lib.lib.ssw_status_string(-2).decode().startswith("size")


def test_missing_library_fails_loudly(tmp_path, monkeypatch):
    from sparseswin3d_b200 import _lib

    monkeypatch.setattr(_lib, "LIB_PATH", tmp_path / "nope.so")
    with pytest.raises(_lib.NativeLibraryMissing):
        _lib._load()


@pytest.mark.parametrize("dims,window,shift", [
    ((400, 400, 150), (7, 7, 7), (3, 3, 3)), ((128, 128, 128), (7, 7, 7), (0, 0, 0)), ((5, 30, 6), (7, 7, 7), (3, 3, 3)),
    ((126, 126, 126), (9, 9, 9), (4, 4, 4)), ((20, 21, 22), (5, 6, 7), (2, 3, 3))])
def test_geometry_matches_oracle(dims, window, shift):
    from sparseswin3d_b200 import window as W

    g = W.resolve_geometry(2, dims, window, shift)
    ws, ss, dp = O.resolve_geometry(dims, window, shift)
    assert tuple(g.ws) == ws and tuple(g.ss) == ss and tuple(g.dims_p) == dp
    n = ws[0] * ws[1] * ws[2]
    assert g.n_per_window == n
    assert g.n_windows == 2 * (dp[0] // ws[0]) * (dp[1] // ws[1]) * (dp[2] // ws[2])
    assert bool(g.shifted) == any(s > 0 for s in ss)


def test_geometry_and_layout_reject_bad_sizes():
    from sparseswin3d_b200 import _lib
    from sparseswin3d_b200 import window as W

    with pytest.raises(_lib.SswError):
        W.resolve_geometry(1, (0, 4, 4), (7, 7, 7))
    with pytest.raises(_lib.SswError):
        W.resolve_geometry(1, (40, 40, 40), (11, 11, 11))  # 1331 positions: beyond the 10-bit position field
    with pytest.raises(_lib.SswError):
        W.resolve_geometry(64, (2000, 2000, 2000), (7, 7, 7))  # window table leaves int32
    L = _lib.PlanLayout()
    assert _lib.lib.ssw_plan_layout_init(L, 1000, 512, 343, 48, 0) == 0
    assert L.w_cap == 512 and L.plan_ints > 4 * 1000 and L.scratch_ints >= 512 * 12
    assert _lib.lib.ssw_plan_layout_init(L, 1000, 512, 343, 65, 0) != 0
    assert _lib.lib.ssw_plan_layout_init(L, 2 ** 31, 512, 343, 48, 0) != 0
    assert _lib.lib.ssw_argsort_workspace_bytes(1000) >= 12000


def test_cpu_tensors_are_rejected_not_computed_on_cpu():
    from sparseswin3d_b200 import _lib, ops
    from sparseswin3d_b200 import window as W

    g = W.resolve_geometry(1, (16, 16, 16), (7, 7, 7))
    with pytest.raises(_lib.SswError):
        W.bucket_windows(coords=torch.zeros((4, 4), dtype=torch.int32), geom=g)
    with pytest.raises(_lib.SswError):
        ops.flatten_indices(torch.zeros((2, 4), dtype=torch.int32), [4, 4])


def test_default_tile_rows():
    from sparseswin3d_b200 import attention

    assert attention.default_tile_rows(3, 32, torch.float32, (7, 7, 7)) == 48
    for h, hd in ((3, 16), (6, 16), (6, 32), (12, 16), (12, 32), (24, 16)):
        t = attention.default_tile_rows(h, hd, torch.bfloat16, (7, 7, 7))
        assert 8 <= t <= 64
