"""Spectral convolution on the sphere (Driscoll-Healy) on the shtb200 kernels.

Drop-in counterpart of ``torch_harmonics.SpectralConvS2`` (torch_harmonics/spectral_convolution.py:43-247): same
constructor arguments, parameters (``weight`` (groups, in / groups, out / groups, lmax) complex64, optional
``spectral_bias``), sub-modules (``sht``, ``isht``, ``quadrature``) and results.

Without bias the whole layer is ONE library call (``shtb200_spectral_conv``): forward transform, per-degree channel
mixing and inverse transform run back to back on the degree-slab layout the two Legendre contraction kernels share, so the
(batch, channel, l, m) coefficient tensors and the transposes that would build them never exist.  The input gradient is
the same call with the adjoint plans and the conjugated, transposed weights; the weight gradient needs the coefficients
themselves and takes the ordinary transforms.  With bias the layer composes the transform modules the way the reference
does.
"""

import math
from typing import Optional, Tuple

import torch
import torch.nn as nn

from . import _lib
from .quadrature import QuadratureS2
from .sht import InverseRealSHT, RealSHT, _LinearTransform
from .truncation import truncate_sht


class _FusedSpectralConv(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight, layer):
        B, Cin = x.shape[0], x.shape[1]
        G, _, Cog, _ = weight.shape
        Cout = G * Cog
        xc, wc = _lib.dense(x), _lib.dense(weight)
        y = torch.empty(B, Cout, layer.isht.nlat, layer.isht.nlon, dtype=torch.float32, device=x.device)
        with torch.cuda.device(x.device):
            _lib.spectral_conv(layer.sht._op.plan(x.device, False), layer.isht._op.plan(x.device, False), xc, wc, y, B, Cin, Cout, G,
                               torch.cuda.current_stream(x.device).cuda_stream)
        ctx.layer = layer
        ctx.save_for_backward(xc, wc)
        return y

    @staticmethod
    def backward(ctx, gy):
        x, w = ctx.saved_tensors
        layer = ctx.layer
        gy = _lib.dense(gy)
        B, Cin = x.shape[0], x.shape[1]
        G, Cig, Cog, L = w.shape
        Cout = G * Cog
        gx = gw = None
        if ctx.needs_input_grad[0]:
            # x -> y is real-linear: its transpose is the adjoint inverse transform, the conjugated weights with the
            # channel roles swapped, the adjoint forward transform
            wt = _lib.dense(w.conj().permute(0, 2, 1, 3))  # (with one channel per group the permutation is a view: the conjugate must be materialised)
            gx = torch.empty_like(x)
            with torch.cuda.device(x.device):
                _lib.spectral_conv(layer.isht._op.plan(x.device, True), layer.sht._op.plan(x.device, True), gy, wt, gx, B, Cout, Cin, G,
                                   torch.cuda.current_stream(x.device).cuda_stream)
        if ctx.needs_input_grad[1]:
            with torch.no_grad():
                u = layer.sht(x).reshape(B, G, Cig, L, -1)
                gv = _LinearTransform.apply(gy, layer.isht._op, True, (layer.isht.lmax, layer.isht.mmax), torch.complex64, gy.dim() - 2).reshape(B, G, Cog, L, -1)
                gw = torch.einsum("bgixy,bgoxy->giox", u.conj(), gv)
        return gx, gw, None


class SpectralConvS2(nn.Module):
    """``(batch, in_channels, nlat_in, nlon_in) -> (batch, out_channels, nlat_out, nlon_out)``: forward SHT, channel mixing
    with weights that depend on the degree l only, inverse SHT (possibly onto another grid)."""

    def __init__(
        self,
        in_shape: Tuple[int],
        out_shape: Tuple[int],
        in_channels: int,
        out_channels: int,
        num_groups: Optional[int] = 1,
        grid_in: Optional[str] = "equiangular",
        grid_out: Optional[str] = "equiangular",
        bias: Optional[bool] = False,
    ):
        super().__init__()
        if in_channels % num_groups != 0:
            raise ValueError(f"in_channels ({in_channels}) must be divisible by num_groups ({num_groups})")
        if out_channels % num_groups != 0:
            raise ValueError(f"out_channels ({out_channels}) must be divisible by num_groups ({num_groups})")
        self.in_channels = in_channels
        self.out_channels = out_channels
        self.num_groups = num_groups

        # common truncation of the two grids (torch_harmonics/spectral_convolution.py:174-182)
        lmax_in, mmax_in = truncate_sht(in_shape[0], in_shape[1], grid=grid_in)
        lmax_out, mmax_out = truncate_sht(out_shape[0], out_shape[1], grid=grid_out)
        self.lmax = min(min(lmax_in, lmax_out), min(mmax_in, mmax_out))
        self.mmax = self.lmax
        self.sht = RealSHT(*in_shape, grid=grid_in, lmax=self.lmax, mmax=self.mmax)
        self.isht = InverseRealSHT(*out_shape, grid=grid_out, lmax=self.lmax, mmax=self.mmax)

        weight_shape = [num_groups, in_channels // num_groups, out_channels // num_groups, self.lmax]
        scale = math.sqrt(1.0 / (in_channels // num_groups)) * torch.ones(self.lmax, dtype=torch.complex64)
        scale[0] *= math.sqrt(2.0)  # the l = 0 coefficients are real
        self.weight = nn.Parameter(scale * torch.randn(*weight_shape, dtype=torch.complex64))
        if bias:
            self.spectral_bias = nn.Parameter(torch.zeros(1, self.in_channels, self.lmax, self.mmax, dtype=torch.complex64))
            self.quadrature = QuadratureS2(img_shape=in_shape, grid=grid_in, normalize=False)

    # The one-call path mixes the channels with a register-tiled fp32 kernel on the degree slabs; it beats transform +
    # einsum + transform up to about 100 x 100 channels per group (B200, 721 x 1440: 0.64 against 0.70 ms at 73 channels,
    # 0.28 / 0.31 at 32) and loses to the library's complex GEMM beyond (1.32 against 1.14 ms at 128, 3.9 / 2.8 at 256).
    fused_max_channel_product = 10000

    def forward(self, x):
        dtype = x.dtype
        with torch.amp.autocast(device_type=x.device.type, enabled=False):
            x = x.to(torch.float32)
            cig, cog = self.in_channels // self.num_groups, self.out_channels // self.num_groups
            if (not hasattr(self, "spectral_bias") and x.dim() == 4 and x.is_cuda and self.weight.dtype == torch.complex64
                    and cig * cog <= self.fused_max_channel_product):
                return _FusedSpectralConv.apply(x, self.weight, self).to(dtype=dtype)
            if hasattr(self, "spectral_bias"):
                integral = self.quadrature(x)
            x = self.sht(x).contiguous()
        B, C, H, W = x.shape
        if hasattr(self, "spectral_bias"):
            x = x + integral.reshape(B, C, 1, 1) * self.spectral_bias
        x = x.reshape(B, self.num_groups, C // self.num_groups, H, W)
        x = torch.einsum("bgixy,giox->bgoxy", x, self.weight).reshape(B, self.out_channels, H, W).contiguous()
        with torch.amp.autocast(device_type=x.device.type, enabled=False):
            x = self.isht(x)
        return x.to(dtype=dtype)
