"""Gaussian random fields on the sphere, sampled through the inverse SHT kernels.

Counterpart of ``torch_harmonics.GaussianRandomFieldS2`` (torch_harmonics/random_fields.py:38-147): a mean-zero field
with covariance sigma^2 (-Lap + tau^2 I)^(-alpha), drawn by scaling white spectral noise with the square roots of the
covariance's eigenvalues (Karhunen-Loeve expansion) and synthesising it on an (nlat, 2 nlat) grid.
"""

import torch
import torch.nn as nn

from .sht import InverseRealSHT


class GaussianRandomFieldS2(nn.Module):
    def __init__(self, nlat, alpha=2.0, tau=3.0, sigma=None, radius=1.0, grid="equiangular", dtype=torch.float32):
        super().__init__()
        if dtype != torch.float32:
            raise TypeError("GaussianRandomFieldS2: the transform kernels compute in float32")
        self.nlat = nlat
        if sigma is None:
            if alpha <= 1.0:
                raise ValueError(f"Alpha must be greater than one, got {alpha}.")
            sigma = tau ** (0.5 * (2 * alpha - 2.0))
        self.isht = InverseRealSHT(self.nlat, 2 * self.nlat, grid=grid, norm="backward")
        lmax, mmax = self.isht.lmax, self.isht.mmax
        # square roots of the eigenvalues of the covariance operator, per degree (torch_harmonics/random_fields.py:107-111)
        ll = torch.as_tensor([j * (j + 1) for j in range(lmax)]).view(lmax, 1).repeat(1, mmax)
        sqrt_eig = torch.tril(sigma * (((ll / radius**2) + tau**2) ** (-alpha / 2.0)))
        sqrt_eig[0, 0] = 0.0
        self.register_buffer("sqrt_eig", sqrt_eig.unsqueeze(0).to(torch.float32))

    def forward(self, N, xi=None, generator=None):
        """N samples ``(N, nlat, 2 nlat)``; ``xi`` (N, lmax, mmax) complex64 replaces the internally drawn noise."""
        if xi is None:
            lmax, mmax = self.isht.lmax, self.isht.mmax
            xi = torch.view_as_complex(torch.randn(N, lmax, mmax, 2, device=self.sqrt_eig.device, dtype=torch.float32, generator=generator))
        return self.isht((xi * self.sqrt_eig).contiguous())
