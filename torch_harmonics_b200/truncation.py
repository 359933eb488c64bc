"""Resolved spectral truncation of an SHT on a given grid.

Same rule as the reference (torch_harmonics/truncation.py:36-73, :93-175): per-grid default degree, Nyquist
default order, then triangular truncation ``lmax = mmax = min(lmax, mmax)``.
"""

import warnings
from typing import Optional, Tuple

_DEFAULT_LMAX = {
    "legendre-gauss": lambda nlat: nlat,
    "lobatto": lambda nlat: nlat - 1,
    "equiangular": lambda nlat: (nlat + 1) // 2,
    "equiangular-trapezoidal": lambda nlat: (nlat + 1) // 2,
}


def _truncate_lmax(nlat: int, grid: Optional[str] = "equiangular") -> int:
    if grid not in _DEFAULT_LMAX:
        raise ValueError(f"Unknown grid type {grid}")
    if grid.startswith("equiangular"):
        warnings.warn(
            "Default SHT truncation changed in v0.9.0: equiangular/equiangular-trapezoidal grids now truncate to (nlat+1)//2. "
            "Specify lmax explicitly to override.",
            UserWarning,
            stacklevel=3,
        )
    return _DEFAULT_LMAX[grid](nlat)


def _truncate_mmax(nlon: int) -> int:
    return nlon // 2 + 1


def truncate_sht(nlat: int, nlon: int, lmax: Optional[int] = None, mmax: Optional[int] = None, grid: Optional[str] = "equiangular") -> Tuple[int, int]:
    """(lmax, mmax), both exclusive upper bounds, after triangular truncation.

    A falsy ``lmax`` / ``mmax`` (None or 0) selects the grid default, as in the reference.
    """
    lmax = lmax or _truncate_lmax(nlat, grid)
    mmax = mmax or _truncate_mmax(nlon)
    tri = min(lmax, mmax)
    return tri, tri
