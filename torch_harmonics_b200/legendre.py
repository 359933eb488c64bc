"""Float64 tables of normalised associated Legendre functions and their theta-derivatives.

The values are those of torch_harmonics/legendre.py:46-116 (``legpoly``) and :151-237
(``_precompute_dlegpoly``): same seeds, recurrences, normalisations (``"ortho"``, ``"schmidt"``, anything
else = four-pi) and Condon-Shortley phase.  The recurrence over the degree is carried degree-major
(one contiguous (order, node) slab per degree) and transposed once at the end.
"""

import math
from typing import Optional

import torch


def clm(l: int, m: int) -> float:
    """Orthonormalisation constant of Y_l^m."""
    return math.sqrt((2 * l + 1) / 4 / math.pi) * math.sqrt(math.factorial(l - m) / math.factorial(l + m))


@torch.no_grad()
def legpoly(mmax: int, lmax: int, x: torch.Tensor, norm: Optional[str] = "ortho", inverse: Optional[bool] = False, csphase: Optional[bool] = True) -> torch.Tensor:
    """(-1)^m c_l^m P_l^m(x), shape (mmax, lmax, len(x)), float64."""
    x = x.to(torch.float64)
    n = max(mmax, lmax)
    tab = torch.zeros((n, n, x.numel()), dtype=torch.float64, device=x.device)  # [degree, order, node]

    scale = 1.0 if norm == "ortho" else math.sqrt(4 * math.pi)
    if inverse:
        scale = 1.0 / scale
    tab[0, 0] = scale / math.sqrt(4 * math.pi)

    one_minus_x2 = (1 + x) * (1 - x)
    for l in range(1, n):
        sectoral = tab[l - 1, l - 1]
        tab[l, l - 1] = math.sqrt(2 * l + 1) * x * sectoral
        tab[l, l] = torch.sqrt((2 * l + 1) * one_minus_x2 / 2 / l) * sectoral

    for l in range(2, n):
        m = torch.arange(0, l - 1, dtype=torch.float64, device=x.device)
        a = torch.sqrt((2 * l - 1) / (l - m) * (2 * l + 1) / (l + m))
        b = torch.sqrt((l + m - 1) / (l - m) * (2 * l + 1) / (2 * l - 3) * (l - m - 1) / (l + m))
        tab[l, : l - 1] = a[:, None] * x[None, :] * tab[l - 1, : l - 1] - b[:, None] * tab[l - 2, : l - 1]

    if norm == "schmidt":
        deg = torch.sqrt(2 * torch.arange(n, dtype=torch.float64, device=x.device) + 1)[:, None, None]
        tab = tab * deg if inverse else tab / deg

    out = tab[:lmax, :mmax].permute(1, 0, 2).contiguous()
    if csphase:
        out[1::2] *= -1
    return out


@torch.no_grad()
def _precompute_legpoly(mmax: int, lmax: int, t: torch.Tensor, norm: Optional[str] = "ortho", inverse: Optional[bool] = False, csphase: Optional[bool] = True) -> torch.Tensor:
    return legpoly(mmax, lmax, torch.cos(t), norm=norm, inverse=inverse, csphase=csphase)


@torch.no_grad()
def _precompute_dlegpoly(mmax: int, lmax: int, t: torch.Tensor, norm: Optional[str] = "ortho", inverse: Optional[bool] = False, csphase: Optional[bool] = True) -> torch.Tensor:
    """Stack of d/dtheta P_l^m(cos theta) and (m / sin theta) P_l^m(cos theta), shape (2, mmax, lmax, len(t))."""
    base = _precompute_legpoly(mmax + 1, lmax + 1, t, norm=norm, inverse=inverse, csphase=False)
    dev = t.device
    m = torch.arange(mmax, dtype=torch.float64, device=dev)[:, None]
    l = torch.arange(lmax, dtype=torch.float64, device=dev)[None, :]
    below = (torch.arange(mmax, device=dev) - 1).clamp(min=0)
    above = torch.arange(mmax, device=dev) + 1
    inside = ((m >= 1) & (m <= l))[..., None]

    out = torch.zeros((2, mmax, lmax, t.numel()), dtype=torch.float64, device=dev)

    lower = torch.sqrt(torch.clamp((l + m) * (l - m + 1), min=0.0))[..., None]
    upper = torch.sqrt(torch.clamp((l - m) * (l + m + 1), min=0.0))[..., None]
    out[0] = inside * 0.5 * (lower * base[below, :lmax] - upper * base[above, :lmax])
    out[0, 0] = -torch.sqrt(l[0] * (l[0] + 1))[:, None] * base[1, :lmax]

    ratio = torch.sqrt((2 * l + 1) / (2 * l + 3))[..., None]
    lower1 = torch.sqrt(torch.clamp((l - m + 1) * (l - m + 2), min=0.0))[..., None]
    upper1 = torch.sqrt((l + m + 1) * (l + m + 2))[..., None]
    out[1] = inside * 0.5 * ratio * (lower1 * base[below, 1 : lmax + 1] + upper1 * base[above, 1 : lmax + 1])

    if norm == "schmidt":
        lv = l[0]
        fix = torch.sqrt((2 * lv + 3) / (2 * lv + 1)) if not inverse else torch.sqrt((2 * lv + 1) / (2 * lv + 3))
        out[1] = out[1] * fix[None, :, None]

    if csphase:
        out[:, 1::2] *= -1
    return out
