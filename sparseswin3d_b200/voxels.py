"""A minimal stand-in for the container upstream's attention receives (an spconv SparseConvTensor
after window_partition_sparse): only the four fields WindowAttentionSparse.forward reads
(swin3d_base.py:654-657) and `replace_feature` (:205-206)."""
from __future__ import annotations

from dataclasses import dataclass, replace
from typing import Tuple

import torch


@dataclass
class WindowedVoxels:
    features: torch.Tensor      # [N, C]
    indices: torch.Tensor       # [N, 2] int32 (window, pos)
    batch_size: int             # all windows of the padded grid, empty ones included
    spatial_shape: Tuple[int]   # (positions per window,)

    def replace_feature(self, new_features: torch.Tensor) -> "WindowedVoxels":
        return replace(self, features=new_features)
