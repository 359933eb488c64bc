"""Timed port of the reference's per-call SHT path (TEST / BASELINE INFRASTRUCTURE ONLY).

The reference's forward methods are a short sequence of torch ops: they run on MKL when the input lives on the
CPU and on cuFFT + cuBLAS when it lives on a GPU.  This module restates that exact op sequence (torch.fft.rfft ->
scale -> transpose -> real/imag copies -> two einsums -> complex; and the mirror image) with float32 tables, so
that ``bench.py`` can time "the reference's path" on the GPU box, where the reference tree itself is not present:
on the host cores (cpu_baseline / --impl reference legs) and, as the incumbent the CUDA kernels replace, on the
same GPU (incumbent_cuda leg).  Tables come from ``oracle.sht_oracle`` (pinned against the reference's buffers) or
are handed in.

Only ``bench.py`` (those baseline legs) and tests import this; nothing in the package does.
"""

import torch

from . import sht_oracle as orc


class CpuShtPort:
    """RealSHT + InverseRealSHT of the reference, ``.float()``-ed, on CPU threads."""

    def __init__(self, nlat, nlon, lmax, mmax, grid="equiangular", norm="ortho", csphase=True, tables=None):
        """``tables`` = (weights (mmax, lmax, nlat), pct (mmax, nlat, lmax)) float32 tensors on the device the port
        shall run on; by default they are built on the CPU by the oracle."""
        if tables is None:
            w, self.lmax, self.mmax = orc.sht_weights(nlat, nlon, lmax, mmax, grid, norm, csphase)
            self.weights = torch.from_numpy(w).float()  # (mmax, lmax, nlat)   torch_harmonics/sht.py:141-146 + .float()
            del w
            p, _, _ = orc.isht_pct(nlat, nlon, lmax, mmax, grid, norm, csphase)
            self.pct = torch.from_numpy(p).float()  # (mmax, nlat, lmax)   torch_harmonics/sht.py:297-301 + .float()
            del p
        else:
            self.weights, self.pct = tables
            self.mmax, self.lmax = self.weights.shape[0], self.weights.shape[1]
        self.nlat, self.nlon = nlat, nlon

    @torch.no_grad()
    def sht(self, x: torch.Tensor) -> torch.Tensor:
        """torch_harmonics/sht.py:171-186 with fft.py:52-68 inlined."""
        X = torch.fft.rfft(x, dim=-1, norm="forward").contiguous()
        have = X.shape[-1]
        if self.mmax > have:
            X = torch.nn.functional.pad(X, (0, self.mmax - have))
        elif self.mmax < have:
            X = X.narrow(-1, 0, self.mmax)
        X = 2.0 * torch.pi * X
        X = X.transpose(-1, -2)
        xr = X.real.contiguous()
        xi = X.imag.contiguous()
        out_re = torch.einsum("...mk,mlk->...lm", xr, self.weights)
        out_im = torch.einsum("...mk,mlk->...lm", xi, self.weights)
        return torch.complex(out_re.contiguous(), out_im.contiguous())

    @torch.no_grad()
    def isht(self, c: torch.Tensor) -> torch.Tensor:
        """torch_harmonics/sht.py:326-342 with fft.py:71-96 inlined."""
        c = c.transpose(-1, -2)
        cr = c.real.contiguous()
        ci = c.imag.contiguous()
        out_re = torch.einsum("...ml,mkl->...km", cr, self.pct)
        out_im = torch.einsum("...ml,mkl->...km", ci, self.pct)
        X = torch.complex(out_re.contiguous(), out_im.contiguous())
        scale = torch.ones(X.shape[-1], dtype=X.real.dtype, device=X.device)
        scale[0] = 0.0
        if self.nlon % 2 == 0 and self.nlon // 2 < X.shape[-1]:
            scale[self.nlon // 2] = 0.0
        X = torch.complex(X.real, X.imag * scale)
        return torch.fft.irfft(X, n=self.nlon, dim=-1, norm="forward").contiguous()
