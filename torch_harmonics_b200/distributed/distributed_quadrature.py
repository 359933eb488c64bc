"""Integral over the sphere of a field whose latitude-longitude grid is tiled over the polar x azimuth process grid.

Counterpart of torch_harmonics/distributed/distributed_quadrature.py:42-139: same constructor, the same local
``quad_weight`` buffer (1, 1, nlat_local, nlon_local) float32, the same result on every rank.  The local part of the sum
is one launch of the library's reduction kernel; the partial sums are then added over the two communicators.
"""

import math
from typing import Optional, Tuple

import torch
import torch.nn as nn

from ..quadrature import _Quadrature, clenshaw_curtiss_weights, legendre_gauss_weights, lobatto_weights
from .primitives import compute_split_shapes, reduce_from_azimuth_region, reduce_from_polar_region
from .utils import azimuth_group_rank, azimuth_group_size, polar_group_rank, polar_group_size


class DistributedQuadratureS2(nn.Module):
    """``(..., nlat_local, nlon_local) -> (...)``: the integral (``normalize=True``: the mean) over the whole sphere."""

    def __init__(self, img_shape: Tuple[int], grid: Optional[str] = "equiangular", normalize: Optional[bool] = False):
        super().__init__()
        self.grid = grid
        self.img_shape = img_shape
        self.normalize = normalize
        self.comm_size_polar = polar_group_size()
        self.comm_rank_polar = polar_group_rank()
        self.comm_size_azimuth = azimuth_group_size()
        self.comm_rank_azimuth = azimuth_group_rank()

        nlat, nlon = img_shape
        if grid == "legendre-gauss":
            _, weights = legendre_gauss_weights(nlat, -1, 1)
        elif grid == "lobatto":
            _, weights = lobatto_weights(nlat, -1, 1)
        elif grid == "equiangular":
            _, weights = clenshaw_curtiss_weights(nlat, -1, 1)
        else:
            raise ValueError("Unknown quadrature mode")
        lat = (2 * math.pi / nlon) * weights
        if normalize:
            lat = lat / (4.0 * math.pi)

        # this rank's tile of the grid
        self.lat_shapes = compute_split_shapes(nlat, self.comm_size_polar)
        self.lon_shapes = compute_split_shapes(nlon, self.comm_size_azimuth)
        k0 = sum(self.lat_shapes[: self.comm_rank_polar])
        lat = lat[k0 : k0 + self.lat_shapes[self.comm_rank_polar]]
        nlon_local = self.lon_shapes[self.comm_rank_azimuth]
        quad_weight = lat.unsqueeze(1).tile(1, nlon_local).reshape(1, 1, -1, nlon_local).to(torch.float32).contiguous()
        self.register_buffer("quad_weight", quad_weight, persistent=False)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        if not x.is_cuda:
            raise RuntimeError("DistributedQuadratureS2: expected a CUDA tensor; torch_harmonics_b200 has no CPU path")
        if x.dtype != torch.float32:
            raise TypeError(f"DistributedQuadratureS2: expected dtype torch.float32, got {x.dtype}")
        if x.shape[-2:] != self.quad_weight.shape[-2:]:
            raise RuntimeError(f"Expected local spatial shape {tuple(self.quad_weight.shape[-2:])}, got {tuple(x.shape[-2:])}")
        quad = _Quadrature.apply(x, self.quad_weight[0, 0, :, 0].contiguous())
        if self.comm_size_polar > 1:
            quad = reduce_from_polar_region(quad)
        if self.comm_size_azimuth > 1:
            quad = reduce_from_azimuth_region(quad)
        return quad
