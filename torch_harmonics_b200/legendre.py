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
def legpoly(mmax: int, lmax: int, x: torch.Tensor, norm: Optional[str] = "ortho", inverse: Optional[bool] = False, csphase: Optional[bool] = True,
            m_first: int = 0, m_count: Optional[int] = None) -> torch.Tensor:
    """(-1)^m c_l^m P_l^m(x), shape (mmax, lmax, len(x)), float64.

    ``m_first`` / ``m_count`` restrict the orders to the window [m_first, m_first + m_count) (shape (m_count, lmax,
    len(x))): every order runs its own recurrence over the degree, so the window costs its share of the work and
    memory and equals the matching slice of the full table bit for bit."""
    x = x.to(torch.float64)
    n = max(mmax, lmax)
    m1 = mmax if m_count is None else m_first + m_count
    if m_count is None:
        m1 = n  # (the full recurrence carries orders up to max(mmax, lmax) and is cut at the end)
    cnt = m1 - m_first
    tab = torch.zeros((n, cnt, x.numel()), dtype=torch.float64, device=x.device)  # [degree, order - m_first, node]

    scale = 1.0 if norm == "ortho" else math.sqrt(4 * math.pi)
    if inverse:
        scale = 1.0 / scale
    # sectoral chain P_l^l and its neighbour P_l^{l-1}: seeds of the recurrences of all orders
    sectoral = torch.full_like(x, scale / math.sqrt(4 * math.pi))
    if m_first == 0:
        tab[0, 0] = sectoral
    one_minus_x2 = (1 + x) * (1 - x)
    for l in range(1, n):
        if m_first <= l - 1 < m1:
            tab[l, l - 1 - m_first] = math.sqrt(2 * l + 1) * x * sectoral
        sectoral = torch.sqrt((2 * l + 1) * one_minus_x2 / 2 / l) * sectoral
        if m_first <= l < m1:
            tab[l, l - m_first] = sectoral

    for l in range(2, n):
        hi = min(l - 1, m1)
        if hi <= m_first:
            continue
        m = torch.arange(m_first, hi, dtype=torch.float64, device=x.device)
        a = torch.sqrt((2 * l - 1) / (l - m) * (2 * l + 1) / (l + m))
        b = torch.sqrt((l + m - 1) / (l - m) * (2 * l + 1) / (2 * l - 3) * (l - m - 1) / (l + m))
        k = hi - m_first
        tab[l, :k] = a[:, None] * x[None, :] * tab[l - 1, :k] - b[:, None] * tab[l - 2, :k]

    if norm == "schmidt":
        deg = torch.sqrt(2 * torch.arange(n, dtype=torch.float64, device=x.device) + 1)[:, None, None]
        tab = tab * deg if inverse else tab / deg

    keep = (mmax if m_count is None else m1) - m_first
    out = tab[:lmax, :keep].permute(1, 0, 2).contiguous()
    if csphase:
        out[(1 - m_first % 2) % 2 :: 2] *= -1  # odd orders
    return out


@torch.no_grad()
def _precompute_legpoly(mmax: int, lmax: int, t: torch.Tensor, norm: Optional[str] = "ortho", inverse: Optional[bool] = False, csphase: Optional[bool] = True,
                        m_first: int = 0, m_count: Optional[int] = None) -> torch.Tensor:
    return legpoly(mmax, lmax, torch.cos(t), norm=norm, inverse=inverse, csphase=csphase, m_first=m_first, m_count=m_count)


@torch.no_grad()
def _precompute_dlegpoly(mmax: int, lmax: int, t: torch.Tensor, norm: Optional[str] = "ortho", inverse: Optional[bool] = False, csphase: Optional[bool] = True,
                         m_first: int = 0, m_count: Optional[int] = None) -> torch.Tensor:
    """Stack of d/dtheta P_l^m(cos theta) and (m / sin theta) P_l^m(cos theta), shape (2, mmax, lmax, len(t));
    with ``m_first`` / ``m_count`` only the orders of that window, shape (2, m_count, lmax, len(t))."""
    if m_count is None:
        m_first, m_count = 0, mmax
    # orders m - 1 .. m + 1 of the plain functions feed order m of the derivatives
    b0 = max(m_first - 1, 0)
    base = _precompute_legpoly(mmax + 1, lmax + 1, t, norm=norm, inverse=inverse, csphase=False, m_first=b0, m_count=m_first + m_count + 1 - b0)
    dev = t.device
    mi = torch.arange(m_first, m_first + m_count, device=dev)
    m = mi.to(torch.float64)[:, None]
    l = torch.arange(lmax, dtype=torch.float64, device=dev)[None, :]
    below = (mi - 1).clamp(min=0) - b0
    above = mi + 1 - b0
    inside = ((m >= 1) & (m <= l))[..., None]

    out = torch.zeros((2, m_count, lmax, t.numel()), dtype=torch.float64, device=dev)

    lower = torch.sqrt(torch.clamp((l + m) * (l - m + 1), min=0.0))[..., None]
    upper = torch.sqrt(torch.clamp((l - m) * (l + m + 1), min=0.0))[..., None]
    out[0] = inside * 0.5 * (lower * base[below, :lmax] - upper * base[above, :lmax])
    if m_first == 0:
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
        out[:, (1 - m_first % 2) % 2 :: 2] *= -1  # odd orders
    return out
