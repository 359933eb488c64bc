"""Spatially distributed spherical harmonic transforms (polar x azimuth process grid).

Mirrors the SHT-, spectral-convolution- and quadrature-related exports of torch_harmonics/distributed/__init__.py:33-71.
"""

from .distributed_quadrature import DistributedQuadratureS2
from .distributed_sht import DistributedInverseRealSHT, DistributedInverseRealVectorSHT, DistributedRealSHT, DistributedRealVectorSHT
from .distributed_spectral_convolution import DistributedSpectralConvS2
from .primitives import (
    compute_split_shapes,
    copy_to_azimuth_region,
    copy_to_polar_region,
    distributed_transpose_azimuth,
    distributed_transpose_polar,
    flatten_and_pad_leading_dims,
    reduce_from_azimuth_region,
    reduce_from_polar_region,
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
