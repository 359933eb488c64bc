"""Spherical harmonic transform modules backed by the shtb200 CUDA library.

Drop-in counterparts of ``torch_harmonics.RealSHT``, ``InverseRealSHT``, ``RealVectorSHT`` and
``InverseRealVectorSHT`` (torch_harmonics/sht.py:41, :189, :345, :498): same constructor arguments,
attributes, buffer names and shapes, tensor layouts, error messages and autograd behaviour.  The forward
methods run hand-written sm_100a kernels through the C ABI in ``include/shtb200.h``; inputs must be CUDA
tensors (float32 on the grid side, complex64 on the spectral side) — there is no CPU or PyTorch fallback.
"""

import itertools
import os
import weakref
from typing import List

import torch
import torch.nn as nn

from . import _lib
from .legendre import _precompute_dlegpoly, _precompute_legpoly
from .quadrature import sht_colatitudes
from .truncation import truncate_sht


def _default_engine():
    return os.environ.get("SHTB200_ENGINE", "auto")


class _ShtOp:
    """A pair of plans (operator, adjoint) created lazily per device from a module's table."""

    def __init__(self, module, kind, adj_kind, table_name, vector):
        # weak: the module owns this object, so a strong reference back would keep the plans (and their packed tables,
        # hundreds of MB of device memory at 721 x 1440) alive until the cycle collector runs
        self._module = weakref.ref(module)
        self.kind, self.adj_kind = kind, adj_kind
        self.table_name = table_name
        self.vector = vector
        self.plans = {}
        _register_op(self)

    @property
    def module(self):
        mod = self._module()
        if mod is None:
            raise RuntimeError("the SHT module of this operator has been deleted")
        return mod

    def plan(self, device, adjoint):
        mod = self.module
        key = (device.index, adjoint, mod.engine)
        pl = self.plans.get(key)
        if pl is None:
            table = getattr(mod, self.table_name)
            with torch.cuda.device(device):
                t32 = table.detach().to(device=device, dtype=torch.float32).contiguous()
                pl = _lib.Plan(self.adj_kind if adjoint else self.kind, mod.nlat, mod.nlon, mod.lmax, mod.mmax, t32, engine=mod.engine)
                del t32
            self.plans[key] = pl
        return pl

    def clear(self):
        for pl in self.plans.values():
            pl.close()
        self.plans.clear()

    def __del__(self):
        try:
            self.clear()
        except Exception:
            pass


def _run(plan, x, out_tail, out_dtype, nfields):
    out = torch.empty(x.shape[: x.dim() - len(out_tail)] + tuple(out_tail), dtype=out_dtype, device=x.device)
    if nfields == 0:
        return out
    nbytes = plan.workspace_bytes(nfields)
    ws = torch.empty(max(nbytes, 1), dtype=torch.uint8, device=x.device)
    with torch.cuda.device(x.device):
        plan.execute(x, out, nfields, ws, torch.cuda.current_stream(x.device).cuda_stream)
    return out


# The transforms are exposed to PyTorch as ONE custom operator, so that modules that use them stay traceable by
# torch.compile (fake implementation for shape / dtype inference, autograd registered on the operator).  Non-tensor
# state (the pair of plans) is looked up through an integer handle.
_OPS = weakref.WeakValueDictionary()
_HANDLES = itertools.count(1)


def _register_op(op):
    op.handle = next(_HANDLES)
    _OPS[op.handle] = op
    return op.handle


@torch.library.custom_op("shtb200::linear_transform", mutates_args=(), device_types="cuda")
def _linear_transform(x: torch.Tensor, handle: int, adjoint: bool, out_tail: List[int], out_complex: bool, lead_dims: int) -> torch.Tensor:
    """y = A x for the real-linear map A of plan pair `handle` (its transpose when `adjoint`)."""
    op = _OPS[handle]
    xc = _lib.dense(x)
    nfields = 1
    for s in xc.shape[:lead_dims]:
        nfields *= s
    return _run(op.plan(xc.device, adjoint), xc, tuple(out_tail), torch.complex64 if out_complex else torch.float32, nfields)


@_linear_transform.register_fake
def _(x, handle, adjoint, out_tail, out_complex, lead_dims):
    return x.new_empty(tuple(x.shape[:lead_dims]) + tuple(out_tail), dtype=torch.complex64 if out_complex else torch.float32)


def _lt_setup(ctx, inputs, output):
    x, handle, adjoint, out_tail, out_complex, lead_dims = inputs
    ctx.handle, ctx.adjoint, ctx.lead_dims = handle, adjoint, lead_dims
    ctx.in_tail, ctx.in_complex = [int(v) for v in x.shape[lead_dims:]], x.is_complex()


def _lt_backward(ctx, g):
    # the gradient is A^T g, realised by the partner plan; differentiating that again lands back on A
    gx = _linear_transform(g, ctx.handle, not ctx.adjoint, ctx.in_tail, ctx.in_complex, ctx.lead_dims)
    return gx, None, None, None, None, None


_linear_transform.register_autograd(_lt_backward, setup_context=_lt_setup)


class _LinearTransform:
    """Call shim with the signature the modules use."""

    @staticmethod
    def apply(x, op, adjoint, out_tail, out_dtype, lead_dims):
        return _linear_transform(x, op.handle, adjoint, [int(v) for v in out_tail], out_dtype == torch.complex64, lead_dims)


def _check(cond, message):
    """torch._check with the reference's messages (RuntimeError), written as a plain branch: the message closures
    refer to the input tensor, which torch.compile does not accept inside torch._check."""
    if not cond:
        raise RuntimeError(message())


def _require(x, dtype, what):
    if not x.is_cuda:
        raise RuntimeError(f"{what}: expected a CUDA tensor; torch_harmonics_b200 has no CPU path")
    if x.dtype != dtype:
        raise TypeError(f"{what}: expected dtype {dtype}, got {x.dtype}")


class _ShtBase(nn.Module):
    _vector = False

    def __init__(self, nlat, nlon, lmax, mmax, grid, norm, csphase):
        super().__init__()
        self.nlat = nlat
        self.nlon = nlon
        self.grid = grid
        self.norm = norm
        self.csphase = csphase
        self.engine = _default_engine()
        # colatitudes (north to south) and quadrature weights; raises ValueError("Unknown quadrature mode")
        self._tq, self._quad_w = sht_colatitudes(nlat, grid)
        self.lmax, self.mmax = truncate_sht(self.nlat, self.nlon, lmax, mmax, self.grid)

    def extra_repr(self):
        return f"nlat={self.nlat}, nlon={self.nlon},\n lmax={self.lmax}, mmax={self.mmax},\n grid={self.grid}, csphase={self.csphase}"

    def _apply(self, fn, *args, **kwargs):
        # buffers may move or change dtype: plans built from the old table are dropped
        out = super()._apply(fn, *args, **kwargs)
        if hasattr(self, "_op"):
            self._op.clear()
        return out

    def close(self):
        """Release the device memory of the plans built so far (they are rebuilt on the next call)."""
        if hasattr(self, "_op"):
            self._op.clear()

    def __getstate__(self):
        state = self.__dict__.copy()
        state.pop("_op", None)
        return state

    def __setstate__(self, state):
        self.__dict__.update(state)
        self._make_op()


class RealSHT(_ShtBase):
    """Forward real SHT: ``(..., nlat, nlon)`` float32 -> ``(..., lmax, mmax)`` complex64.

    Counterpart of torch_harmonics/sht.py:41-186.  ``weights`` is the reference's buffer: Legendre functions
    times quadrature weights, shape (mmax, lmax, nlat), float64, non-persistent.
    """

    def __init__(self, nlat, nlon, lmax=None, mmax=None, grid="equiangular", norm="ortho", csphase=True):
        super().__init__(nlat, nlon, lmax, mmax, grid, norm, csphase)
        pct = _precompute_legpoly(self.mmax, self.lmax, self._tq, norm=self.norm, csphase=self.csphase)
        weights = (pct * self._quad_w.to(pct.device)[None, None, :]).contiguous()
        self.register_buffer("weights", weights, persistent=False)
        self._make_op()

    def _make_op(self):
        self._op = _ShtOp(self, _lib.SHT, _lib.SHT_ADJOINT, "weights", False)

    def forward(self, x: torch.Tensor):
        _check(x.dim() >= 2, lambda: f"Expected tensor with at least 2 dimensions but got {x.dim()} instead")
        _check(x.shape[-2] == self.nlat, lambda: f"Expected latitudes shape[-2]=={self.nlat}, got {x.shape[-2]}")
        _check(x.shape[-1] == self.nlon, lambda: f"Expected longitudes shape[-1]=={self.nlon}, got {x.shape[-1]}")
        _require(x, torch.float32, "RealSHT")
        return _LinearTransform.apply(x, self._op, False, (self.lmax, self.mmax), torch.complex64, x.dim() - 2)


class InverseRealSHT(_ShtBase):
    """Inverse real SHT: ``(..., lmax, mmax)`` complex64 -> ``(..., nlat, nlon)`` float32.

    Counterpart of torch_harmonics/sht.py:189-342.  ``pct`` has shape (mmax, nlat, lmax), float64.
    """

    def __init__(self, nlat, nlon, lmax=None, mmax=None, grid="equiangular", norm="ortho", csphase=True):
        super().__init__(nlat, nlon, lmax, mmax, grid, norm, csphase)
        pct = _precompute_legpoly(self.mmax, self.lmax, self._tq, norm=self.norm, inverse=True, csphase=self.csphase)
        self.register_buffer("pct", pct.permute(0, 2, 1).contiguous(), persistent=False)
        self._make_op()

    def _make_op(self):
        self._op = _ShtOp(self, _lib.ISHT, _lib.ISHT_ADJOINT, "pct", False)

    def forward(self, x: torch.Tensor):
        _check(x.dim() >= 2, lambda: f"Expected tensor with at least 2 dimensions but got {x.dim()} instead")
        _check(x.shape[-2] == self.lmax, lambda: f"Expected spherical harmonic degrees (lmax) shape[-2]=={self.lmax}, got {x.shape[-2]}")
        _check(x.shape[-1] == self.mmax, lambda: f"Expected spherical harmonic orders (mmax) shape[-1]=={self.mmax}, got {x.shape[-1]}")
        _require(x, torch.complex64, "InverseRealSHT")
        return _LinearTransform.apply(x, self._op, False, (self.nlat, self.nlon), torch.float32, x.dim() - 2)


class RealVectorSHT(_ShtBase):
    """Forward vector SHT: ``(..., 2, nlat, nlon)`` float32 -> ``(..., 2, lmax, mmax)`` complex64
    (spheroidal, toroidal).  Counterpart of torch_harmonics/sht.py:345-495; ``weights`` has shape
    (2, mmax, lmax, nlat)."""

    _vector = True

    def __init__(self, nlat, nlon, lmax=None, mmax=None, grid="equiangular", norm="ortho", csphase=True):
        super().__init__(nlat, nlon, lmax, mmax, grid, norm, csphase)
        dpct = _precompute_dlegpoly(self.mmax, self.lmax, self._tq, norm=self.norm, csphase=self.csphase)
        # 1 / (l (l + 1)) is evaluated in float32, as the reference does (integer arange divided into a Python
        # float, torch_harmonics/sht.py:439-441); the rounding is part of the reference's weights
        l = torch.arange(0, self.lmax)
        norm_factor = 1.0 / l / (l + 1)
        norm_factor[0] = 1.0
        weights = dpct * self._quad_w.to(dpct.device)[None, None, None, :] * norm_factor.to(dtype=torch.float64, device=dpct.device)[None, None, :, None]
        weights[1] = -1 * weights[1]
        self.register_buffer("weights", weights.contiguous(), persistent=False)
        self._make_op()

    def _make_op(self):
        self._op = _ShtOp(self, _lib.VSHT, _lib.VSHT_ADJOINT, "weights", True)

    def forward(self, x: torch.Tensor):
        _check(x.dim() >= 3, lambda: f"Expected tensor with at least 3 dimensions but got {x.dim()} instead")
        _check(x.shape[-3] == 2, lambda: f"Expected vector field shape[-3]==2, got {x.shape[-3]}")
        _check(x.shape[-2] == self.nlat, lambda: f"Expected latitudes shape[-2]=={self.nlat}, got {x.shape[-2]}")
        _check(x.shape[-1] == self.nlon, lambda: f"Expected longitudes shape[-1]=={self.nlon}, got {x.shape[-1]}")
        _require(x, torch.float32, "RealVectorSHT")
        return _LinearTransform.apply(x, self._op, False, (2, self.lmax, self.mmax), torch.complex64, x.dim() - 3)


class InverseRealVectorSHT(_ShtBase):
    """Inverse vector SHT: ``(..., 2, lmax, mmax)`` complex64 -> ``(..., 2, nlat, nlon)`` float32.
    Counterpart of torch_harmonics/sht.py:498-649; ``dpct`` has shape (2, mmax, nlat, lmax)."""

    _vector = True

    def __init__(self, nlat, nlon, lmax=None, mmax=None, grid="equiangular", norm="ortho", csphase=True):
        super().__init__(nlat, nlon, lmax, mmax, grid, norm, csphase)
        dpct = _precompute_dlegpoly(self.mmax, self.lmax, self._tq, norm=self.norm, inverse=True, csphase=self.csphase)
        self.register_buffer("dpct", dpct.permute(0, 1, 3, 2).contiguous(), persistent=False)
        self._make_op()

    def _make_op(self):
        self._op = _ShtOp(self, _lib.IVSHT, _lib.IVSHT_ADJOINT, "dpct", True)

    def forward(self, x: torch.Tensor):
        _check(x.dim() >= 3, lambda: f"Expected tensor with at least 3 dimensions but got {x.dim()} instead")
        _check(x.shape[-3] == 2, lambda: f"Expected vector field shape[-3]==2, got {x.shape[-3]}")
        _check(x.shape[-2] == self.lmax, lambda: f"Expected spherical harmonic degrees (lmax) shape[-2]=={self.lmax}, got {x.shape[-2]}")
        _check(x.shape[-1] == self.mmax, lambda: f"Expected spherical harmonic orders (mmax) shape[-1]=={self.mmax}, got {x.shape[-1]}")
        _require(x, torch.complex64, "InverseRealVectorSHT")
        return _LinearTransform.apply(x, self._op, False, (2, self.nlat, self.nlon), torch.float32, x.dim() - 3)
