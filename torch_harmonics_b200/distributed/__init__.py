"""Spatially distributed spherical harmonic transforms (polar x azimuth process grid).

Mirrors the SHT-related exports of torch_harmonics/distributed/__init__.py:33-71.
"""

from .distributed_sht import DistributedInverseRealSHT, DistributedInverseRealVectorSHT, DistributedRealSHT, DistributedRealVectorSHT
from .primitives import (
    compute_split_shapes,
    distributed_transpose_azimuth,
    distributed_transpose_polar,
    flatten_and_pad_leading_dims,
    split_tensor_along_dim,
    unpad_and_unflatten_leading_dims,
)
from .utils import (
    azimuth_group,
    azimuth_group_rank,
    azimuth_group_size,
    config,
    finalize,
    init,
    is_distributed_azimuth,
    is_distributed_polar,
    is_initialized,
    polar_group,
    polar_group_rank,
    polar_group_size,
)
