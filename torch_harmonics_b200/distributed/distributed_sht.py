"""Spatially distributed SHT modules (scalar and vector) on the shtb200 kernels.

Counterparts of ``DistributedRealSHT`` / ``DistributedInverseRealSHT`` / ``DistributedRealVectorSHT`` /
``DistributedInverseRealVectorSHT`` (torch_harmonics/distributed/distributed_sht.py:51-222, :225-391, :394-555, :558-711): same constructor arguments, attributes
(``comm_size_*``, ``comm_rank_*``, ``lat_shapes``, ``lon_shapes``, ``l_shapes``, ``m_shapes``, ``nlat_local``,
``nlon_local``, ``lmax_local``, ``mmax_local``), local tensor layouts and autograd behaviour.  Latitudes and
degrees are sharded over the polar group, longitudes and orders over the azimuth group; four all-to-all
transposes per direction move between the layouts.  The longitude FFT and the Legendre contraction between the
transposes run through the stage entry points of the C ABI (``shtb200_rfft_modes``, ``shtb200_irfft_modes``,
``shtb200_legendre``).
"""

import ctypes
import math

import torch
import torch.nn as nn

from .. import _lib
from ..legendre import _precompute_dlegpoly, _precompute_legpoly
from ..quadrature import sht_colatitudes
from ..sht import _check, _default_engine, _require
from ..truncation import truncate_sht
from .primitives import (
    _pieces_exchange_in,
    _pieces_exchange_out,
    compute_split_shapes,
    distributed_transpose_azimuth,
    distributed_transpose_polar,
    flatten_and_pad_leading_dims,
    unpad_and_unflatten_leading_dims,
)
from .utils import azimuth_group, azimuth_group_rank, azimuth_group_size, polar_group, polar_group_rank, polar_group_size


def _stream(t):
    return ctypes.c_void_p(torch.cuda.current_stream(t.device).cuda_stream)


def _edge_weights(nmodes, nlon, interior, device):
    """Per-order factors of the FFT adjoints: 1 at m = 0 and Nyquist, ``interior`` elsewhere."""
    w = torch.full((nmodes,), interior, dtype=torch.float32, device=device)
    w[0] = 1.0
    if nlon % 2 == 0 and nlon // 2 < nmodes:
        w[nlon // 2] = 1.0
    return w


def _zero_edge_imag(c, nlon):
    c = c.clone()
    c[..., 0] = torch.complex(c[..., 0].real, torch.zeros_like(c[..., 0].real))
    if nlon % 2 == 0 and nlon // 2 < c.shape[-1]:
        k = nlon // 2
        c[..., k] = torch.complex(c[..., k].real, torch.zeros_like(c[..., k].real))
    return c


class _RfftStage(torch.autograd.Function):
    """(rows, nlon) float32 -> (rows, nmodes) complex64 = scale * rfft(norm="forward"), kept / zero-padded to nmodes."""

    @staticmethod
    def forward(ctx, x, nmodes, scale):
        ctx.nlon, ctx.nmodes, ctx.scale = x.shape[-1], nmodes, scale
        xc = _lib.dense(x)
        out = torch.empty(xc.shape[:-1] + (nmodes,), dtype=torch.complex64, device=x.device)
        rows = xc.numel() // xc.shape[-1] if xc.numel() else 0
        with torch.cuda.device(x.device):
            _lib.check(_lib.load().shtb200_rfft_modes(ctypes.c_void_p(xc.data_ptr()), ctypes.c_void_p(out.data_ptr()), rows, xc.shape[-1], nmodes, scale, _stream(x)), "shtb200_rfft_modes")
        return out

    @staticmethod
    def backward(ctx, g):
        # adjoint: (scale / nlon) * unnormalised c2r of the cotangent with interior bins halved
        w = _edge_weights(ctx.nmodes, ctx.nlon, 0.5, g.device) * (ctx.scale / ctx.nlon)
        return _IrfftStage.apply((g * w).contiguous(), ctx.nlon), None, None


class _IrfftStage(torch.autograd.Function):
    """(rows, nmodes) complex64 -> (rows, nlon) float32: unnormalised c2r, imaginary parts of DC / Nyquist ignored."""

    @staticmethod
    def forward(ctx, c, nlon):
        ctx.nlon, ctx.nmodes = nlon, c.shape[-1]
        cc = _lib.dense(c)
        out = torch.empty(cc.shape[:-1] + (nlon,), dtype=torch.float32, device=c.device)
        rows = cc.numel() // cc.shape[-1] if cc.numel() else 0
        with torch.cuda.device(c.device):
            _lib.check(_lib.load().shtb200_irfft_modes(ctypes.c_void_p(cc.data_ptr()), ctypes.c_void_p(out.data_ptr()), rows, nlon, cc.shape[-1], _stream(c)), "shtb200_irfft_modes")
        return out

    @staticmethod
    def backward(ctx, g):
        # adjoint: unnormalised r2c, interior bins doubled, imaginary parts of DC / Nyquist zeroed
        r = _RfftStage.apply(g.contiguous(), ctx.nmodes, float(ctx.nlon))
        w = _edge_weights(ctx.nmodes, ctx.nlon, 2.0, g.device)
        return _zero_edge_imag(r * w, ctx.nlon), None


class _AzimuthRfft(torch.autograd.Function):
    """The azimuth sandwich of the forward transforms in one step: exchange (fields scattered, longitudes gathered), row
    FFT, exchange (orders scattered, fields gathered) - ``(n, ..., nlon_local)`` float32 -> ``(n, ..., mmax_local)``
    complex64.  The FFT kernel reads the first exchange's receive buffer and writes the second one's send buffer in their
    piece-major form, so no copy sits between the three (the separate transposes concatenate / split one tensor each).
    The backward pass is the chain of the separate, differentiable steps."""

    @staticmethod
    def forward(ctx, x, owner, scale):
        group, A = azimuth_group(), owner.comm_size_azimuth
        n, mid = x.shape[0], tuple(x.shape[1:-1])
        ctx.owner, ctx.scale, ctx.n, ctx.lead = owner, scale, n, -x.dim()
        recv, n_loc = _pieces_exchange_in(_lib.dense(x), owner.lon_shapes, group)
        rows = n_loc
        for s in mid:
            rows *= s
        spec = torch.empty(rows * owner.mmax * 2, dtype=torch.float32, device=x.device)
        with torch.cuda.device(x.device):
            _lib.check(_lib.load().shtb200_rfft_modes_pieces(ctypes.c_void_p(recv.data_ptr()), ctypes.c_void_p(spec.data_ptr()), rows, owner.nlon, owner.mmax, scale, A, A,
                                                              _stream(x)), "shtb200_rfft_modes_pieces")
        return _pieces_exchange_out(spec, n_loc, n, mid + (0,), -1, owner.m_shapes, True, group)

    @staticmethod
    def backward(ctx, g):
        o, lead = ctx.owner, ctx.lead
        g = distributed_transpose_azimuth(g, (lead, -1), o.m_shapes)
        w = _edge_weights(o.mmax, o.nlon, 0.5, g.device) * (ctx.scale / o.nlon)
        g = _IrfftStage.apply((g * w).contiguous(), o.nlon)
        return distributed_transpose_azimuth(g, (-1, lead), compute_split_shapes(ctx.n, o.comm_size_azimuth)), None, None


class _AzimuthIrfft(torch.autograd.Function):
    """The azimuth sandwich of the inverse transforms: exchange (fields scattered, orders gathered), inverse row FFT,
    exchange (longitudes scattered, fields gathered) - ``(n, ..., mmax_local)`` complex64 -> ``(n, ..., nlon_local)``
    float32, piece-major in between like :class:`_AzimuthRfft`."""

    @staticmethod
    def forward(ctx, c, owner):
        group, A = azimuth_group(), owner.comm_size_azimuth
        n, mid = c.shape[0], tuple(c.shape[1:-1])
        ctx.owner, ctx.n, ctx.lead = owner, n, -c.dim()
        recv, n_loc = _pieces_exchange_in(_lib.dense(c), owner.m_shapes, group)
        rows = n_loc
        for s in mid:
            rows *= s
        grid = torch.empty(rows * owner.nlon, dtype=torch.float32, device=c.device)
        with torch.cuda.device(c.device):
            _lib.check(_lib.load().shtb200_irfft_modes_pieces(ctypes.c_void_p(recv.data_ptr()), ctypes.c_void_p(grid.data_ptr()), rows, owner.nlon, owner.mmax, A, A,
                                                               _stream(c)), "shtb200_irfft_modes_pieces")
        return _pieces_exchange_out(grid, n_loc, n, mid + (0,), -1, owner.lon_shapes, False, group)

    @staticmethod
    def backward(ctx, g):
        o, lead = ctx.owner, ctx.lead
        g = distributed_transpose_azimuth(g, (lead, -1), o.lon_shapes)
        r = _RfftStage.apply(g.contiguous(), o.mmax, float(o.nlon))
        r = _zero_edge_imag(r * _edge_weights(o.mmax, o.nlon, 2.0, g.device), o.nlon)
        return distributed_transpose_azimuth(r, (-1, lead), compute_split_shapes(ctx.n, o.comm_size_azimuth)), None


class _LegendreStage(torch.autograd.Function):
    """Contraction with the packed table for the local orders [m0, m0 + mloc): (N, nlat, mloc) <-> (N, lmax, mloc);
    vector plans carry the component axis, (N, 2, nlat, mloc) <-> (N, 2, lmax, mloc)."""

    @staticmethod
    def forward(ctx, x, owner, adjoint, out_rows):
        ctx.owner, ctx.adjoint, ctx.in_rows = owner, adjoint, x.shape[-2]
        xc = _lib.dense(x)
        n, mloc = xc.shape[0], xc.shape[-1]
        out = torch.empty(xc.shape[:-2] + (out_rows, mloc), dtype=torch.complex64, device=x.device)
        if n == 0 or mloc == 0:
            return out
        plan = owner._plan(x.device, adjoint)
        ws = torch.empty(max(plan.legendre_workspace_bytes(n, mloc), 1), dtype=torch.uint8, device=x.device)
        with torch.cuda.device(x.device):
            plan.legendre(xc, out, n, owner._m0, mloc, ws, torch.cuda.current_stream(x.device).cuda_stream)
        return out

    @staticmethod
    def backward(ctx, g):
        return _LegendreStage.apply(g.contiguous(), ctx.owner, not ctx.adjoint, ctx.in_rows), None, None, None


class _PolarLegendre(torch.autograd.Function):
    """The polar sandwich in one step: exchange (fields scattered, latitudes / degrees gathered), contraction, exchange
    (degrees / latitudes scattered, fields gathered) - ``(n, ..., rows_in_local, mloc)`` -> ``(n, ..., rows_out_local, mloc)``
    complex64.  The contraction's fold / unfold and coefficient kernels read the first exchange's receive buffer and write
    the second one's send buffer in their piece-major form (``shtb200_legendre_pieces``): no copy in between.  The backward
    pass is the chain of the separate, differentiable steps."""

    @staticmethod
    def forward(ctx, x, owner, in_splits, out_splits):
        group, P = polar_group(), owner.comm_size_polar
        n, rest, mloc = x.shape[0], list(x.shape[1:]), x.shape[-1]
        ctx.owner, ctx.n, ctx.lead, ctx.in_splits, ctx.out_splits = owner, n, -x.dim(), in_splits, out_splits
        recv, n_loc = _pieces_exchange_in(_lib.dense(x), in_splits, group, axis=-2)
        comp = 1
        for s in rest[:-2]:
            comp *= s
        out = torch.empty(n_loc * comp * sum(out_splits) * mloc * 2, dtype=torch.float32, device=x.device)
        plan = owner._plan(x.device, False)
        ws = torch.empty(max(plan.legendre_workspace_bytes(n_loc, mloc), 1), dtype=torch.uint8, device=x.device)
        with torch.cuda.device(x.device):
            plan.legendre(recv, out, n_loc, owner._m0, mloc, ws, torch.cuda.current_stream(x.device).cuda_stream, in_pieces=P, out_pieces=P)
        return _pieces_exchange_out(out, n_loc, n, rest, -2, out_splits, True, group)

    @staticmethod
    def backward(ctx, g):
        o, lead = ctx.owner, ctx.lead
        g = distributed_transpose_polar(g, (lead, -2), ctx.out_splits)
        g = _LegendreStage.apply(g.contiguous(), o, True, sum(ctx.in_splits))
        return distributed_transpose_polar(g, (-2, lead), compute_split_shapes(ctx.n, o.comm_size_polar)), None, None, None


class _DistributedBase(nn.Module):
    def __init__(self, nlat, nlon, lmax, mmax, grid, norm, csphase):
        super().__init__()
        self.nlat, self.nlon, self.grid, self.norm, self.csphase = nlat, nlon, grid, norm, csphase
        self.engine = _default_engine()
        self._tq, self._quad_w = sht_colatitudes(nlat, grid)  # raises ValueError("Unknown quadrature mode")
        self.comm_size_polar = polar_group_size()
        self.comm_rank_polar = polar_group_rank()
        self.comm_size_azimuth = azimuth_group_size()
        self.comm_rank_azimuth = azimuth_group_rank()
        self.lmax, self.mmax = truncate_sht(nlat, nlon, lmax, mmax, grid)
        self.lat_shapes = compute_split_shapes(self.nlat, self.comm_size_polar)
        self.nlat_local = self.lat_shapes[self.comm_rank_polar]
        self.lon_shapes = compute_split_shapes(self.nlon, self.comm_size_azimuth)
        self.nlon_local = self.lon_shapes[self.comm_rank_azimuth]
        self.l_shapes = compute_split_shapes(self.lmax, self.comm_size_polar)
        self.lmax_local = self.l_shapes[self.comm_rank_polar]
        self.m_shapes = compute_split_shapes(self.mmax, self.comm_size_azimuth)
        self.mmax_local = self.m_shapes[self.comm_rank_azimuth]
        self._m0 = sum(self.m_shapes[: self.comm_rank_azimuth])
        self._plans = {}

    def extra_repr(self):
        return f"nlat={self.nlat}, nlon={self.nlon},\n lmax={self.lmax}, mmax={self.mmax},\n grid={self.grid}, csphase={self.csphase}"

    def _local_table(self):
        """float64 table of this rank's orders [_m0, _m0 + mmax_local) in the reference's layout (built once, in the constructor)."""
        raise NotImplementedError

    def _plan(self, device, adjoint):
        """Plan over this rank's window of orders, packed from the module's own buffer."""
        key = (device.index, adjoint, self.engine)
        pl = self._plans.get(key)
        if pl is None:
            with torch.cuda.device(device):
                t32 = getattr(self, self._table_name).detach().to(device=device, dtype=torch.float32).contiguous()
                pl = _lib.Plan(self._adj_kind if adjoint else self._kind, self.nlat, self.nlon, self.lmax, self.mmax, t32, engine=self.engine,
                               orders=(self._m0, self.mmax_local))
                del t32
            self._plans[key] = pl
        return pl

    # Number of field chunks the inference path pipelines (0 / 1 switches it off) and the smallest local tensor worth it.
    pipeline_chunks = 4
    pipeline_min_bytes = 64 << 20
    last_pipelined = False  # whether the last forward call ran in chunks

    fuse_azimuth_fft = True  # exchange - row FFT - exchange without copies in between, where the row kernels support it

    def _rfft_stages(self, lead):
        """Stages of the forward transforms between the local grid tile and (fields, ..., local orders)."""
        A = self.comm_size_azimuth
        if A > 1 and self.fuse_azimuth_fft and _lib.rows_pieces_supported(self.nlon, self.mmax, A, A):
            return [lambda t, n: _AzimuthRfft.apply(t, self, 2.0 * math.pi)]
        stages = []
        if A > 1:  # fields get sharded over the azimuth group, longitudes become local
            stages.append(lambda t, n: distributed_transpose_azimuth(t, (lead, -1), self.lon_shapes))
        stages.append(lambda t, n: _RfftStage.apply(t, self.mmax, 2.0 * math.pi))
        if A > 1:  # orders get sharded, fields local again
            stages.append(lambda t, n: distributed_transpose_azimuth(t, (-1, lead), compute_split_shapes(n, A)))
        return stages

    fuse_polar_legendre = True  # exchange - contraction - exchange without copies in between

    def _legendre_stages(self, lead, in_splits, out_splits):
        """Stages between (fields, ..., local latitudes | degrees, local orders) and (fields, ..., local degrees | latitudes,
        local orders): ``in_splits`` / ``out_splits`` are the polar group's chunks of the contracted / produced axis."""
        P = self.comm_size_polar
        if P > 1 and self.fuse_polar_legendre:
            return [lambda t, n: _PolarLegendre.apply(t, self, in_splits, out_splits)]
        stages = []
        if P > 1:  # fields get sharded over the polar group, the contracted axis becomes local
            stages.append(lambda t, n: distributed_transpose_polar(t, (lead, -2), in_splits))
        stages.append(lambda t, n: _LegendreStage.apply(t, self, False, sum(out_splits)))
        if P > 1:  # the produced axis gets sharded, fields local again
            stages.append(lambda t, n: distributed_transpose_polar(t, (-2, lead), compute_split_shapes(n, P)))
        return stages

    def _irfft_stages(self, lead):
        """Stages of the inverse transforms between (fields, ..., local orders) and the local grid tile."""
        A = self.comm_size_azimuth
        if A > 1 and self.fuse_azimuth_fft and _lib.rows_pieces_supported(self.nlon, self.mmax, A, A):
            return [lambda t, n: _AzimuthIrfft.apply(t, self)]
        stages = []
        if A > 1:
            stages.append(lambda t, n: distributed_transpose_azimuth(t, (lead, -1), self.m_shapes))
        stages.append(lambda t, n: _IrfftStage.apply(t, self.nlon))
        if A > 1:
            stages.append(lambda t, n: distributed_transpose_azimuth(t, (-1, lead), compute_split_shapes(n, A)))
        return stages

    def _run_stages(self, x, stages):
        """Apply the stage functions ``stage(tensor, nfields)`` to the flattened batch ``x`` (fields on axis 0; ``nfields`` is
        the number of fields of the batch the tensor belongs to, which the gathering transposes need for their split sizes).

        Every stage maps (fields, ...) to (fields, ...) and the fields never mix, so the batch may be cut into chunks that
        run as independent transforms.  When no gradient is recorded and the tensor is large, the chunks are issued stage
        by stage on streams of their own: NCCL executes the all-to-alls in issue order (chunk 0, chunk 1, ... of one
        stage), while the FFT / Legendre kernels of a chunk run on its stream next to the other chunks' exchanges.
        Only grids with ONE distributed axis are pipelined: with two communicators the exchanges of different chunks would
        sit on two NCCL streams whose relative order is not the same on every rank.  And only stage lists that still hold
        separate transposes: what the pipeline hides are their copies; once the exchanges are fused with the kernels
        around them (two stages left) nothing remains to hide - the persistent FFT / Legendre kernels fill the GPU, an
        all-to-all does not run beside them (measured at 1 x 2, 2 048 fields: 18.9 / 18.4 ms plain, 19.5 / 20.4 ms in four
        chunks, no better with 8 to 48 SMs held back for NCCL)."""
        n = x.shape[0]
        gmax = max(self.comm_size_polar, self.comm_size_azimuth)
        nchunks = min(self.pipeline_chunks, n // max(gmax, 1))
        if (gmax == 1 or min(self.comm_size_polar, self.comm_size_azimuth) > 1 or nchunks < 2 or len(stages) < 3 or torch.is_grad_enabled() and x.requires_grad or not x.is_cuda
                or x.numel() * x.element_size() < self.pipeline_min_bytes):
            self.last_pipelined = False
            for st in stages:
                x = st(x, n)
            return x
        self.last_pipelined = True
        main = torch.cuda.current_stream(x.device)
        if not hasattr(self, "_streams") or len(self._streams) < nchunks or self._streams[0].device != x.device:
            self._streams = [torch.cuda.Stream(device=x.device) for _ in range(nchunks)]
        parts = list(torch.tensor_split(x, nchunks, dim=0))
        counts = [p.shape[0] for p in parts]
        for c in range(nchunks):
            self._streams[c].wait_stream(main)
        for st in stages:
            for c in range(nchunks):
                with torch.cuda.stream(self._streams[c]):
                    parts[c] = st(parts[c], counts[c])
        out = torch.empty((n,) + tuple(parts[0].shape[1:]), dtype=parts[0].dtype, device=x.device)
        n0 = 0
        for c in range(nchunks):
            with torch.cuda.stream(self._streams[c]):
                out[n0:n0 + parts[c].shape[0]].copy_(parts[c])
            n0 += parts[c].shape[0]
            main.wait_stream(self._streams[c])
        # (the chunk tensors were allocated on the chunk streams and die here; `out` belongs to the caller's stream)
        return out

    def _apply(self, fn, *args, **kwargs):
        # buffers may move or change dtype: plans built from the old table are dropped
        out = super()._apply(fn, *args, **kwargs)
        for pl in self._plans.values():
            pl.close()
        self._plans.clear()
        return out


class DistributedRealSHT(_DistributedBase):
    """Forward SHT on a local tile: ``(..., nlat_local, nlon_local)`` float32 -> ``(..., lmax_local, mmax_local)`` complex64."""

    _kind, _adj_kind, _table_name = _lib.SHT, _lib.SHT_ADJOINT, "weights"

    def __init__(self, nlat, nlon, lmax=None, mmax=None, grid="equiangular", norm="ortho", csphase=True):
        super().__init__(nlat, nlon, lmax, mmax, grid, norm, csphase)
        # the module keeps this rank's orders only, like the reference (distributed_sht.py:164); only they are computed
        self.register_buffer("weights", self._local_table(), persistent=False)

    def _local_table(self):
        pct = _precompute_legpoly(self.mmax, self.lmax, self._tq, norm=self.norm, csphase=self.csphase, m_first=self._m0, m_count=self.mmax_local)
        return (pct * self._quad_w.to(pct.device)[None, None, :]).contiguous()

    def forward(self, x: torch.Tensor):
        _check(x.dim() >= 3, lambda: f"Expected tensor with at least 3 dimensions but got {x.dim()} instead")
        _check(x.shape[-2] == self.nlat_local, lambda: f"Expected latitudes shape[-2]=={self.nlat_local}, got {x.shape[-2]}")
        _check(x.shape[-1] == self.nlon_local, lambda: f"Expected longitudes shape[-1]=={self.nlon_local}, got {x.shape[-1]}")
        _require(x, torch.float32, "DistributedRealSHT")

        x, lead_shape, lead_size = flatten_and_pad_leading_dims(x, max(self.comm_size_polar, self.comm_size_azimuth))
        stages = self._rfft_stages(-3) + self._legendre_stages(-3, self.lat_shapes, self.l_shapes)
        x = self._run_stages(x, stages)
        return unpad_and_unflatten_leading_dims(x, lead_shape, lead_size)


class DistributedInverseRealSHT(_DistributedBase):
    """Inverse SHT on a local tile: ``(..., lmax_local, mmax_local)`` complex64 -> ``(..., nlat_local, nlon_local)`` float32."""

    _kind, _adj_kind, _table_name = _lib.ISHT, _lib.ISHT_ADJOINT, "pct"

    def __init__(self, nlat, nlon, lmax=None, mmax=None, grid="equiangular", norm="ortho", csphase=True):
        super().__init__(nlat, nlon, lmax, mmax, grid, norm, csphase)
        self.register_buffer("pct", self._local_table(), persistent=False)  # this rank's orders (distributed_sht.py:333)

    def _local_table(self):
        pct = _precompute_legpoly(self.mmax, self.lmax, self._tq, norm=self.norm, inverse=True, csphase=self.csphase, m_first=self._m0, m_count=self.mmax_local)
        return pct.permute(0, 2, 1).contiguous()

    def forward(self, x: torch.Tensor):
        _check(x.dim() >= 3, lambda: f"Expected tensor with at least 3 dimensions but got {x.dim()} instead")
        _check(x.shape[-2] == self.lmax_local, lambda: f"Expected spherical harmonic degrees (lmax) shape[-2]=={self.lmax_local}, got {x.shape[-2]}")
        _check(x.shape[-1] == self.mmax_local, lambda: f"Expected spherical harmonic orders (mmax) shape[-1]=={self.mmax_local}, got {x.shape[-1]}")
        _require(x, torch.complex64, "DistributedInverseRealSHT")

        x, lead_shape, lead_size = flatten_and_pad_leading_dims(x, max(self.comm_size_polar, self.comm_size_azimuth))
        stages = self._legendre_stages(-3, self.l_shapes, self.lat_shapes) + self._irfft_stages(-3)
        x = self._run_stages(x, stages)
        return unpad_and_unflatten_leading_dims(x, lead_shape, lead_size)


class DistributedRealVectorSHT(_DistributedBase):
    """Forward vector SHT on a local tile: ``(..., 2, nlat_local, nlon_local)`` float32 ->
    ``(..., 2, lmax_local, mmax_local)`` complex64 (spheroidal, toroidal)."""

    _kind, _adj_kind, _table_name = _lib.VSHT, _lib.VSHT_ADJOINT, "weights"

    def __init__(self, nlat, nlon, lmax=None, mmax=None, grid="equiangular", norm="ortho", csphase=True):
        super().__init__(nlat, nlon, lmax, mmax, grid, norm, csphase)
        self.register_buffer("weights", self._local_table(), persistent=False)  # this rank's orders only (distributed_sht.py:490)

    def _local_table(self):
        dpct = _precompute_dlegpoly(self.mmax, self.lmax, self._tq, norm=self.norm, csphase=self.csphase, m_first=self._m0, m_count=self.mmax_local)
        # 1 / (l (l + 1)) in float32, like the serial module (torch_harmonics/sht.py:439-441)
        l = torch.arange(0, self.lmax)
        norm_factor = 1.0 / l / (l + 1)
        norm_factor[0] = 1.0
        weights = dpct * self._quad_w.to(dpct.device)[None, None, None, :] * norm_factor.to(dtype=torch.float64, device=dpct.device)[None, None, :, None]
        weights[1] = -1 * weights[1]
        return weights.contiguous()

    def forward(self, x: torch.Tensor):
        _check(x.dim() >= 4, lambda: f"Expected tensor with at least 4 dimensions but got {x.dim()} instead")
        _check(x.shape[-3] == 2, lambda: f"Expected vector field shape[-3]==2, got {x.shape[-3]}")
        _check(x.shape[-2] == self.nlat_local, lambda: f"Expected latitudes shape[-2]=={self.nlat_local}, got {x.shape[-2]}")
        _check(x.shape[-1] == self.nlon_local, lambda: f"Expected longitudes shape[-1]=={self.nlon_local}, got {x.shape[-1]}")
        _require(x, torch.float32, "DistributedRealVectorSHT")

        x, lead_shape, lead_size = flatten_and_pad_leading_dims(x, max(self.comm_size_polar, self.comm_size_azimuth), num_trailing_dims=3)
        stages = self._rfft_stages(-4) + self._legendre_stages(-4, self.lat_shapes, self.l_shapes)
        x = self._run_stages(x, stages)
        return unpad_and_unflatten_leading_dims(x, lead_shape, lead_size, num_trailing_dims=3)


class DistributedInverseRealVectorSHT(_DistributedBase):
    """Inverse vector SHT on a local tile: ``(..., 2, lmax_local, mmax_local)`` complex64 ->
    ``(..., 2, nlat_local, nlon_local)`` float32."""

    _kind, _adj_kind, _table_name = _lib.IVSHT, _lib.IVSHT_ADJOINT, "dpct"

    def __init__(self, nlat, nlon, lmax=None, mmax=None, grid="equiangular", norm="ortho", csphase=True):
        super().__init__(nlat, nlon, lmax, mmax, grid, norm, csphase)
        self.register_buffer("dpct", self._local_table(), persistent=False)  # this rank's orders only (distributed_sht.py:645)

    def _local_table(self):
        dpct = _precompute_dlegpoly(self.mmax, self.lmax, self._tq, norm=self.norm, inverse=True, csphase=self.csphase, m_first=self._m0, m_count=self.mmax_local)
        return dpct.permute(0, 1, 3, 2).contiguous()

    def forward(self, x: torch.Tensor):
        _check(x.dim() >= 4, lambda: f"Expected tensor with at least 4 dimensions but got {x.dim()} instead")
        _check(x.shape[-3] == 2, lambda: f"Expected vector field shape[-3]==2, got {x.shape[-3]}")
        _check(x.shape[-2] == self.lmax_local, lambda: f"Expected spherical harmonic degrees (lmax) shape[-2]=={self.lmax_local}, got {x.shape[-2]}")
        _check(x.shape[-1] == self.mmax_local, lambda: f"Expected spherical harmonic orders (mmax) shape[-1]=={self.mmax_local}, got {x.shape[-1]}")
        _require(x, torch.complex64, "DistributedInverseRealVectorSHT")

        x, lead_shape, lead_size = flatten_and_pad_leading_dims(x, max(self.comm_size_polar, self.comm_size_azimuth), num_trailing_dims=3)
        stages = self._legendre_stages(-4, self.l_shapes, self.lat_shapes) + self._irfft_stages(-4)
        x = self._run_stages(x, stages)
        return unpad_and_unflatten_leading_dims(x, lead_shape, lead_size, num_trailing_dims=3)
