"""ctypes binding of ``libssw_b200.so`` (the C ABI declared in ``include/ssw_b200.h``).

There is no CPU fallback: if the shared object is missing or fails to load, importing this
module raises, and so does every operator of the package.
"""
from __future__ import annotations

import ctypes as C
from pathlib import Path

_PKG = Path(__file__).resolve().parent
LIB_PATH = _PKG / "libssw_b200.so"

SSW_OK = 0
SSW_F32, SSW_BF16, SSW_F16 = 0, 1, 2
HEADER_INTS = 64
H_N, H_W, H_PACKS, H_ERROR, H_CMAX, H_SUMC2_LO, H_SUMC2_HI, H_TILE = range(8)
H_PACKS_SMALL, H_PADDED = 10, 11
DEV_BAD_COORD, DEV_DUPLICATE, DEV_COO_RANGE, DEV_TIMEOUT, DEV_BAD_PLAN = 1, 2, 4, 8, 16

i32, i64, vp, f32 = C.c_int32, C.c_int64, C.c_void_p, C.c_float
I3 = i32 * 3


class Geometry(C.Structure):
    _fields_ = [("batch", i32), ("dims", I3), ("window", I3), ("shift", I3), ("ws", I3), ("ss", I3),
                ("dims_p", I3), ("nwin", I3), ("n_per_window", i32), ("n_windows", i32), ("shifted", i32)]


class PlanLayout(C.Structure):
    _fields_ = [("n_vox", i64), ("n_windows", i32), ("n_per_window", i32), ("tile_rows", i32), ("w_cap", i32),
                ("pack_cap", i32), ("bitmap_words", i32), ("padded", i32), ("reserved_", i32),
                ("off_header", i64), ("off_perm", i64), ("off_inv_perm", i64), ("off_win_id", i64),
                ("off_win_start", i64), ("off_coo_start", i64), ("off_win_pstart", i64), ("off_pack_win", i64),
                ("off_pack_perm", i64), ("off_pack_meta", i64), ("off_pack_desc", i64), ("off_bins", i64),
                ("plan_ints", i64), ("off_count", i64), ("off_bitmap", i64), ("off_partials", i64),
                ("scratch_ints", i64)]


class NativeLibraryMissing(RuntimeError):
    pass


def _load() -> C.CDLL:
    if not LIB_PATH.exists():
        raise NativeLibraryMissing(
            f"{LIB_PATH} not found: build it with `python -m sparseswin3d_b200.build` "
            "(nvcc, sm_100a). This package has no CPU or PyTorch fallback.")
    lib = C.CDLL(str(LIB_PATH))
    P = C.POINTER
    sig = {
        "ssw_status_string": (C.c_char_p, [C.c_int]),
        "ssw_last_cuda_error": (C.c_char_p, []),
        "ssw_version": (C.c_int, []),
        "ssw_geometry_resolve": (C.c_int, [P(Geometry)]),
        "ssw_window_keys": (C.c_int, [vp, i64, P(Geometry), vp, vp, vp, vp]),
        "ssw_default_tile_rows": (i32, [i32, i32, C.c_int, P(i32)]),
        "ssw_plan_layout_init": (C.c_int, [P(PlanLayout), i64, i32, i32, i32, i32]),
        "ssw_default_padded": (i32, [C.c_int]),
        "ssw_bucket_windows": (C.c_int, [vp, P(Geometry), vp, vp, i32, P(i32), P(PlanLayout), vp, vp, vp]),
        "ssw_bucket_windows_static_capacity": (i64, []),
        "ssw_bucket_windows_static": (C.c_int, [vp, P(Geometry), vp, vp, i32, P(i32), P(PlanLayout), vp, vp]),
        "ssw_attn_fused": (C.c_int, [vp, C.c_int, i32, i32, P(PlanLayout), vp, vp, P(i32), f32, C.c_int, vp, vp, vp]),
        "ssw_attn_fused_multi": (C.c_int, [vp, C.c_int, i32, i32, P(PlanLayout), vp, vp, P(i32), f32, C.c_int, P(vp), i32, vp, vp]),
        "ssw_voxel_grid_build": (C.c_int, [vp, i64, i32, P(i32), vp, vp, vp]),
        "ssw_subm_neighbors": (C.c_int, [vp, i64, i32, P(i32), vp, i32, vp, vp]),
        "ssw_gather_cols": (C.c_int, [vp, C.c_int, i64, i64, i32, i32, vp, vp, vp]),
        "ssw_gather_reduce": (C.c_int, [vp, vp, C.c_int, i64, vp, vp, i64, i64, i32, vp, vp]),
        "ssw_gather_slices": (C.c_int, [vp, C.c_int, i64, i32, i32, i64, vp, vp, vp, vp]),
        "ssw_add_layernorm": (C.c_int, [vp, vp, vp, vp, f32, C.c_int, i64, i32, vp, vp, vp]),
        "ssw_enable_peer_access": (C.c_int, [i32]),
        "ssw_peer_buffer_create": (C.c_int, [i64, P(vp), C.c_char_p]),
        "ssw_peer_buffer_open": (C.c_int, [C.c_char_p, P(vp)]),
        "ssw_peer_buffer_close": (C.c_int, [vp]),
        "ssw_peer_buffer_destroy": (C.c_int, [vp]),
        "ssw_bucket_windows_range": (C.c_int, [vp, P(Geometry), vp, vp, i32, P(i32), P(PlanLayout), vp, vp, i32, i32, vp]),
        "ssw_attn_fused_bwd_workspace_floats": (i64, [i64, i32]),
        "ssw_attn_fused_bwd": (C.c_int, [vp, vp, C.c_int, i32, i32, P(PlanLayout), vp, vp, P(i32), f32, C.c_int, vp, vp, vp, vp]),
        "ssw_flatten_indices": (C.c_int, [vp, i32, i64, P(i32), vp, vp]),
        "ssw_argsort_workspace_bytes": (i64, [i64]),
        "ssw_argsort_i32": (C.c_int, [vp, i64, vp, vp, i64, vp]),
        "ssw_return_inverse_workspace_bytes": (i64, [i64]),
        "ssw_return_inverse": (C.c_int, [vp, i64, i64, vp, vp, vp, vp, i64, vp]),
        "ssw_scan_workspace_bytes": (i64, [i64]),
        "ssw_unique_consecutive_inverse": (C.c_int, [vp, i64, vp, vp, i64, vp]),
        "ssw_qkv_sparse_indices": (C.c_int, [vp, i64, i32, i32, P(PlanLayout), vp, vp, vp, vp, vp, vp]),
        "ssw_coo_plan_workspace_bytes": (i64, [i64]),
        "ssw_coo_block_plan": (C.c_int, [vp, i64, i32, vp, vp, vp, vp, i64, vp]),
        "ssw_coo_matmul": (C.c_int, [C.c_int, C.c_int, vp, vp, i64, vp, i32, vp, vp, i64, i64, vp, vp, vp, vp, vp]),
        "ssw_coo_offsets_from_counts": (C.c_int, [vp, i64, vp, vp, vp, i64, vp]),
        "ssw_coo_matmul_grad": (C.c_int, [C.c_int, C.c_int, vp, vp, vp, vp, i64, i32, vp, vp]),
        "ssw_coo_block_transpose": (C.c_int, [C.c_int, C.c_int, vp, vp, vp, i64, i32, vp, vp]),
        "ssw_softmax_rows_fwd": (C.c_int, [vp, i64, i32, vp, vp, vp, vp]),
        "ssw_softmax_rows_bwd": (C.c_int, [vp, i64, i32, vp, vp, vp, vp, vp]),
        "ssw_coo_add_bias_mask": (C.c_int, [C.c_int, vp, vp, i64, vp, i32, vp, i32, i32, vp, vp]),
        "ssw_debug_graph_edges": (C.c_int, [vp, C.c_char_p, i64, P(i64), P(i64), P(i64)]),
    }
    for name, (res, args) in sig.items():
        fn = getattr(lib, name)  # AttributeError here = header and library disagree
        fn.restype, fn.argtypes = res, args
    return lib


lib = _load()


class SswError(RuntimeError):
    """Raised for any non-zero status of the native library (upstream raises RuntimeError
    through TORCH_CHECK for the same conditions)."""


def check(status: int, what: str) -> None:
    if status != SSW_OK:
        msg = lib.ssw_status_string(status).decode()
        if status in (-4, -5):
            msg += ": " + lib.ssw_last_cuda_error().decode()
        raise SswError(f"{what}: {msg} (status {status})")


def dtype_code(dtype) -> int:
    import torch

    try:
        return {torch.float32: SSW_F32, torch.bfloat16: SSW_BF16, torch.float16: SSW_F16}[dtype]
    except KeyError:
        raise SswError(f"unsupported dtype {dtype}: expected float32, bfloat16 or float16") from None


def ptr(t) -> int:
    return 0 if t is None else t.data_ptr()


def stream_ptr(device=None) -> int:
    import torch

    return torch.cuda.current_stream(device).cuda_stream


def graph_edges(graph) -> dict:
    """Dependency edges of a captured ``torch.cuda.CUDAGraph`` (created with keep_graph=True):
    {"nodes", "edges": [(from, to, "full" | "programmatic", from_port, to_port)], "programmatic"}."""
    buf = C.create_string_buffer(1 << 20)
    nn, ne, npg = i64(), i64(), i64()
    check(lib.ssw_debug_graph_edges(graph.raw_cuda_graph(), buf, len(buf), C.byref(nn), C.byref(ne), C.byref(npg)),
          "ssw_debug_graph_edges")
    edges = []
    for line in buf.value.decode().splitlines():
        a, rest = line.split(" -> ", 1)
        b, kind, fp, tp = rest.rsplit(" ", 3)
        edges.append((a, b, kind, int(fp.split("=")[1]), int(tp.split("=")[1])))
    return {"nodes": nn.value, "edges": edges, "programmatic": npg.value}
