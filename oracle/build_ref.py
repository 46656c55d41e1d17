"""Build the upstream SparseSwin3D extension, unmodified, as a checker for the oracle.

TEST INFRASTRUCTURE ONLY.  Nothing in the product package may import this file or
the library it produces.

The upstream project ships its native code as two files, ``sparse_swin/ops.cpp`` and
``sparse_swin/ops.cu``, and JIT-builds them at import time with
``torch.utils.cpp_extension.load`` (sparse_swin/swin3d_base.py:22-26) from paths that
only exist inside a Pointcept checkout.  This script runs the same kind of build with
explicit paths: the two sources are compiled *where they lie* in a read-only reference
checkout and the output is ``oracle/_ref/custom_ops.so`` plus ninja's scratch files next
to it.  The upstream Python module (``sparse_swin/swin3d_base.py``) is staged beside it,
verbatim, so that the drop-in test can execute upstream's own ``WindowAttentionSparse``
on a machine that has a GPU but no upstream checkout.  ``oracle/_ref/`` is excluded from
version control: nothing of upstream enters this repository's history.

Usage::

    python oracle/build_ref.py --reference /path/to/SparseSwin3D   (or SSW_REFERENCE=...)

The resulting module exposes the ten upstream functions (sparse_swin/ops.cpp:7-18).
Every one of them is CUDA-only, so the module can be *built* on a machine without a
GPU but only *run* on one.
"""
from __future__ import annotations

import argparse
import os
import sys
from pathlib import Path

HERE = Path(__file__).resolve().parent
OUT = HERE / "_ref"


def build(reference: Path, verbose: bool = False) -> Path | None:
    src = reference / "sparse_swin"
    cu, cpp = src / "ops.cu", src / "ops.cpp"
    if not (cu.is_file() and cpp.is_file()):
        return None
    target = OUT / "custom_ops.so"
    if target.is_file() and target.stat().st_mtime >= max(cu.stat().st_mtime, cpp.stat().st_mtime):
        return target
    OUT.mkdir(parents=True, exist_ok=True)
    os.environ.setdefault("TORCH_CUDA_ARCH_LIST", "10.0")
    os.environ.setdefault("MAX_JOBS", "4")
    from torch.utils.cpp_extension import load

    load(
        name="custom_ops",
        sources=[str(cpp), str(cu)],
        extra_cuda_cflags=["--extended-lambda"],
        extra_include_paths=[str(src)],
        build_directory=str(OUT),
        is_python_module=False,  # build only; importing needs a CUDA context for nothing, but keep it lazy
        verbose=verbose,
    )
    return target if target.is_file() else None


def stage_python(reference: Path) -> Path | None:
    """Stage upstream's Python module, byte for byte, as oracle/_ref/upstream_swin3d_base.py."""
    src = reference / "sparse_swin" / "swin3d_base.py"
    if not src.is_file():
        return None
    OUT.mkdir(parents=True, exist_ok=True)
    dst = OUT / "upstream_swin3d_base.py"
    data = src.read_bytes()
    if not dst.is_file() or dst.read_bytes() != data:
        dst.write_bytes(data)
    return dst


def upstream_python_source() -> Path | None:
    """Where upstream's swin3d_base.py can be read from on this machine: the checkout named by
    SSW_REFERENCE, else the staged copy, else None."""
    ref = os.environ.get("SSW_REFERENCE")
    if ref and (Path(ref) / "sparse_swin" / "swin3d_base.py").is_file():
        return Path(ref) / "sparse_swin" / "swin3d_base.py"
    staged = OUT / "upstream_swin3d_base.py"
    return staged if staged.is_file() else None


def load_ref():
    """Import oracle/_ref/custom_ops.so as a Python module (needs a GPU to *call* it)."""
    import importlib.machinery
    import importlib.util

    import torch  # noqa: F401  (libtorch must be loaded first)

    so = OUT / "custom_ops.so"
    if not so.is_file():
        return None
    loader = importlib.machinery.ExtensionFileLoader("custom_ops", str(so))
    spec = importlib.util.spec_from_loader("custom_ops", loader)
    mod = importlib.util.module_from_spec(spec)
    loader.exec_module(mod)
    return mod


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", default=os.environ.get("SSW_REFERENCE"),
                    help="root of an upstream SparseSwin3D checkout (or set SSW_REFERENCE)")
    ap.add_argument("-v", "--verbose", action="store_true")
    a = ap.parse_args()
    if not a.reference:
        print("no upstream checkout given (--reference or SSW_REFERENCE); nothing built")
        sys.exit(0)
    out = build(Path(a.reference), a.verbose)
    staged = stage_python(Path(a.reference))
    print("built" if out else "reference sources not found; nothing built", out or "", staged or "")
    sys.exit(0)
