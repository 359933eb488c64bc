"""Latitude quadrature rules in the cos(theta) domain, float64.

Same nodes and weights as torch_harmonics/quadrature.py:176-204 (Gauss-Legendre, numpy ``leggauss``),
:207-267 (Gauss-Lobatto by Newton iteration) and :270-325 (Clenshaw-Curtis by Waldvogel's FFT formula).
"""

import math
from typing import Optional, Tuple

import numpy as np
import torch
import torch.nn as nn


def _rescale(x: torch.Tensor, w: torch.Tensor, a: float, b: float):
    half = (b - a) * 0.5
    return half * x + (b + a) * 0.5, w * half


def legendre_gauss_weights(n: int, a: Optional[float] = -1.0, b: Optional[float] = 1.0) -> Tuple[torch.Tensor, torch.Tensor]:
    x, w = np.polynomial.legendre.leggauss(n)
    return _rescale(torch.as_tensor(x).clone(), torch.as_tensor(w).clone(), a, b)


def lobatto_weights(n: int, a: Optional[float] = -1.0, b: Optional[float] = 1.0, tol: Optional[float] = 1e-16, maxiter: Optional[int] = 100) -> Tuple[torch.Tensor, torch.Tensor]:
    idx = torch.arange(n, dtype=torch.float64)
    t = -torch.cos(math.pi * idx / (n - 1))
    leg = torch.zeros((n, n), dtype=torch.float64)  # leg[:, k] = P_k(t)
    for _ in range(maxiter):
        prev = t
        leg[:, 0] = 1.0
        leg[:, 1] = t
        for k in range(2, n):
            leg[:, k] = ((2 * k - 1) * t * leg[:, k - 1] - (k - 1) * leg[:, k - 2]) / k
        t = prev - (t * leg[:, n - 1] - leg[:, n - 2]) / (n * leg[:, n - 1])
        if float((t - prev).abs().max()) < tol:
            break
    w = 2.0 / ((n * (n - 1)) * leg[:, n - 1] ** 2)
    return _rescale(t, w, a, b)


def clenshaw_curtiss_weights(n: int, a: Optional[float] = -1.0, b: Optional[float] = 1.0) -> Tuple[torch.Tensor, torch.Tensor]:
    if n <= 1:
        raise ValueError(f"n must be greater than 1, got {n}")
    nodes = torch.cos(torch.linspace(math.pi, 0, n, dtype=torch.float64))
    if n == 2:
        w = torch.ones(2, dtype=torch.float64)
    else:
        n1 = n - 1
        odd = torch.arange(1, n1, 2, dtype=torch.float64)
        nodd = odd.numel()
        rest = n1 - nodd
        v = torch.cat([2.0 / odd / (odd - 2.0), 1.0 / odd[-1:], torch.zeros(rest, dtype=torch.float64)])
        v = -v[:-1] - torch.flip(v[1:], dims=(0,))
        g = -torch.ones(n1, dtype=torch.float64)
        g[nodd] += n1
        g[rest] += n1
        g = g / (n1 * n1 - 1 + (n1 % 2))
        w = torch.fft.ifft(v + g).real
        w = torch.cat((w, w[:1]))
    return _rescale(nodes, w, a, b)


def trapezoidal_weights(n: int, a: Optional[float] = -1.0, b: Optional[float] = 1.0, periodic: Optional[bool] = False) -> Tuple[torch.Tensor, torch.Tensor]:
    """Equispaced nodes with trapezoidal weights (torch_harmonics/quadrature.py:140-174)."""
    x = torch.as_tensor(np.linspace(a, b, n, endpoint=not periodic))
    w = (b - a) / (n - 1 + int(periodic)) * torch.ones(n, dtype=x.dtype)
    if not periodic:
        w[0] *= 0.5
        w[-1] *= 0.5
    return x, w


def precompute_longitudes(nlon: int) -> torch.Tensor:
    return torch.linspace(0, 2 * math.pi, nlon + 1, dtype=torch.float64)[:-1]


def _nodes(nlat: int, grid: str):
    if grid == "legendre-gauss":
        return legendre_gauss_weights(nlat, -1, 1)
    if grid == "lobatto":
        return lobatto_weights(nlat, -1, 1)
    if grid == "equiangular":
        return clenshaw_curtiss_weights(nlat, -1, 1)
    raise ValueError("Unknown quadrature mode")


def sht_colatitudes(nlat: int, grid: str):
    """Colatitudes ascending from the north pole, and the rule's weights in the order the SHT
    constructors use them (torch_harmonics/sht.py:124-143).  The rule itself is always evaluated on the
    host; the result follows the ambient default device so that the tables built from it do too."""
    with torch.device("cpu"):
        cost, w = _nodes(nlat, grid)
        tq = torch.flip(torch.arccos(cost), dims=(0,))
    dev = torch.get_default_device()
    return tq.to(dev), w.to(dev)


def precompute_latitudes(nlat: int, grid: Optional[str] = "equiangular"):
    """(colatitudes, weights), both flipped to run north to south (torch_harmonics/quadrature.py:109-137)."""
    cost, w = _nodes(nlat, grid)
    return torch.flip(torch.arccos(cost), dims=(0,)).clone(), torch.flip(w, dims=(0,)).clone()


class _Quadrature(torch.autograd.Function):
    """Integral over the last two axes with latitude weights (already times 2 pi / nlon): one reduction kernel forward;
    the gradient is the weights broadcast along longitude times the incoming gradient."""

    @staticmethod
    def forward(ctx, x, w):
        from . import _lib

        xc = _lib.dense(x)
        nlat, nlon = xc.shape[-2], xc.shape[-1]
        out = torch.empty(xc.shape[:-2], dtype=torch.float32, device=x.device)
        n = out.numel()
        if n:
            with torch.cuda.device(x.device):
                _lib.quadrature(xc, w, out, n, nlat, nlon, torch.cuda.current_stream(x.device).cuda_stream)
        ctx.save_for_backward(w)
        ctx.nlon = nlon
        return out

    @staticmethod
    def backward(ctx, g):
        (w,) = ctx.saved_tensors
        return (g[..., None, None] * w[:, None]).expand(*g.shape, w.shape[0], ctx.nlon), None


class QuadratureS2(nn.Module):
    """Integral of a signal over the sphere, ``(..., nlat, nlon) -> (...)``.

    Counterpart of torch_harmonics/quadrature.py:328-463: same constructor, the same ``quad_weight`` buffer
    (1, 1, nlat, nlon) float32 and the same result; the reduction runs in one CUDA kernel on float32 CUDA input."""

    def __init__(self, img_shape: Tuple[int], grid: Optional[str] = "equiangular", normalize: Optional[bool] = False):
        super().__init__()
        self.grid = grid
        self.normalize = normalize
        if grid == "legendre-gauss":
            _, weights = legendre_gauss_weights(img_shape[0], -1, 1)
        elif grid == "lobatto":
            _, weights = lobatto_weights(img_shape[0], -1, 1)
        elif grid == "equiangular":
            _, weights = clenshaw_curtiss_weights(img_shape[0], -1, 1)
        elif grid == "equiangular-trapezoidal":
            _, weights = trapezoidal_weights(img_shape[0], -1, 1)
        else:
            raise ValueError("Unknown quadrature mode")
        lat = (2 * math.pi / img_shape[1]) * weights
        if normalize:
            lat = lat / (4.0 * math.pi)
        quad_weight = lat.unsqueeze(1).tile(1, img_shape[1]).reshape(1, 1, *img_shape).to(torch.float32).contiguous()
        self.register_buffer("quad_weight", quad_weight, persistent=False)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        if not x.is_cuda:
            raise RuntimeError("QuadratureS2: expected a CUDA tensor; torch_harmonics_b200 has no CPU path")
        if x.dtype != torch.float32:
            raise TypeError(f"QuadratureS2: expected dtype torch.float32, got {x.dtype}")
        if x.shape[-2:] != self.quad_weight.shape[-2:]:
            raise RuntimeError(f"Expected spatial shape {tuple(self.quad_weight.shape[-2:])}, got {tuple(x.shape[-2:])}")
        return _Quadrature.apply(x, self.quad_weight[0, 0, :, 0].contiguous())
