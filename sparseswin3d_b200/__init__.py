"""sparseswin3d_b200 — sparse 3-D window attention (W-MSA / SW-MSA) for NVIDIA B200 (sm_100a).

The arithmetic lives in ``libssw_b200.so`` (hand-written CUDA behind the C ABI of
``include/ssw_b200.h``); this package is the thin PyTorch-facing host side.  Importing the
operator modules fails loudly when the library has not been built."""
__version__ = "0.1.0"
