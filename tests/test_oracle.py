"""Pin the CPU oracle: against outputs of the reference modules (tests/golden/*.npz, produced by
tests/golden/make_golden.py) and against the analytic known answers the reference's own tests
use (torch-harmonics tests/test_sht.py:63-98 closed-form Legendre values, :278-414 known-answer
coefficients, :230-276 cross-norm scaling, :416-473 csphase).  CPU only.
"""

import math
import os
import warnings

import numpy as np
import pytest

from oracle import sht_oracle as orc

GOLD = os.path.join(os.path.dirname(__file__), "golden")


def gold(name):
    return np.load(os.path.join(GOLD, name))


def rel(a, b):
    return orc.max_normalised_error(a, b)


# ---------------------------------------------------------------- tables vs reference buffers


@pytest.mark.parametrize("grid", ["equiangular", "legendre-gauss", "lobatto"])
@pytest.mark.parametrize("norm", ["ortho", "four-pi", "schmidt"])
@pytest.mark.parametrize("cs", [True, False])
def test_tables_match_reference(grid, norm, cs):
    g = gold("tables.npz")
    key = f"{grid}|{norm}|{int(cs)}"
    kw = dict(lmax=9, grid=grid, norm=norm, csphase=cs)
    w, lmax, mmax = orc.sht_weights(12, 24, **kw)
    assert (lmax, mmax) == (9, 9)
    assert w.shape == g[key + "|w"].shape
    assert rel(w, g[key + "|w"]) < 1e-13
    p, _, _ = orc.isht_pct(12, 24, **kw)
    assert rel(p, g[key + "|p"]) < 1e-13
    vw, _, _ = orc.vsht_weights(12, 24, **kw)
    assert rel(vw, g[key + "|vw"]) < 1e-13
    vp, _, _ = orc.ivsht_dpct(12, 24, **kw)
    assert rel(vp, g[key + "|vp"]) < 1e-13


@pytest.mark.parametrize("grid", ["equiangular", "legendre-gauss", "lobatto"])
def test_default_truncation(grid):
    g = gold("tables.npz")
    with warnings.catch_warnings():
        warnings.simplefilter("ignore")
        w, lmax, mmax = orc.sht_weights(33, 64, grid=grid)
    assert [lmax, mmax] == list(g[f"default|{grid}|lm"])
    assert rel(w, g[f"default|{grid}|w"]) < 1e-13


def test_equiangular_default_warns():
    with pytest.warns(UserWarning):
        orc.truncate_sht(33, 64, grid="equiangular")
    assert orc.truncate_sht(64, 128, 64, 65, "equiangular") == (64, 64)
    assert orc.truncate_sht(256, 512, 256, 257, "legendre-gauss") == (256, 256)
    with pytest.raises(ValueError):
        orc.quadrature_nodes(8, "equiangular-trapezoidal")


def test_weight_structure():
    """Exact zeros for l < m and equatorial parity (-1)^(l+m) — the structure the CUDA packing uses."""
    for grid, nlat in (("equiangular", 33), ("legendre-gauss", 32), ("lobatto", 33)):
        w, lmax, mmax = orc.sht_weights(nlat, 64, lmax=20, grid=grid)
        for m in range(mmax):
            assert np.all(w[m, :m] == 0.0)
        l = np.arange(lmax)[None, :, None]
        m = np.arange(mmax)[:, None, None]
        sign = (-1.0) ** (l + m)
        assert np.max(np.abs(w[:, :, ::-1] - sign * w)) < 1e-14
        vw, _, _ = orc.vsht_weights(nlat, 64, lmax=20, grid=grid)
        assert np.max(np.abs(vw[0][:, :, ::-1] + sign * vw[0])) < 1e-13
        assert np.max(np.abs(vw[1][:, :, ::-1] - sign * vw[1])) < 1e-13


# ---------------------------------------------------------------- closed forms (reference tests/test_sht.py:63-98)


def test_legendre_closed_forms():
    t = np.linspace(0.1, 3.0, 17)
    x = np.cos(t)
    s = np.sin(t)
    P = orc.legpoly(4, 4, x, norm="ortho", csphase=True)
    c = lambda l, m: math.sqrt((2 * l + 1) / 4 / math.pi) * math.sqrt(math.factorial(l - m) / math.factorial(l + m))
    assert np.allclose(P[0, 0], c(0, 0), atol=1e-12)
    assert np.allclose(P[0, 1], c(1, 0) * x, atol=1e-12)
    assert np.allclose(P[1, 1], -c(1, 1) * s, atol=1e-12)
    assert np.allclose(P[0, 2], c(2, 0) * 0.5 * (3 * x**2 - 1), atol=1e-12)
    assert np.allclose(P[1, 2], -c(2, 1) * 3 * x * s, atol=1e-12)
    assert np.allclose(P[2, 2], c(2, 2) * 3 * s**2, atol=1e-12)
    assert np.allclose(P[0, 3], c(3, 0) * 0.5 * (5 * x**3 - 3 * x), atol=1e-12)
    assert np.allclose(P[3, 3], -c(3, 3) * 15 * s**3, atol=1e-12)


# ---------------------------------------------------------------- known answers (reference tests/test_sht.py:278-414)


@pytest.mark.parametrize("grid", ["equiangular", "legendre-gauss", "lobatto"])
@pytest.mark.parametrize("norm", ["ortho", "four-pi", "schmidt"])
def test_known_answers(grid, norm):
    nlat, nlon = 32, 64
    w, lmax, mmax = orc.sht_weights(nlat, nlon, lmax=16, grid=grid, norm=norm)
    tq, _ = orc.colatitudes(nlat, grid)
    one = np.ones((nlat, nlon))
    c = orc.sht_forward(one, w)
    exp0 = {"ortho": math.sqrt(4 * math.pi), "four-pi": 4 * math.pi, "schmidt": 4 * math.pi}[norm]
    assert abs(c[0, 0] - exp0) < 1e-9
    c[0, 0] = 0
    assert np.max(np.abs(c)) < 1e-9
    f = np.cos(tq)[:, None] * np.ones((1, nlon))
    c = orc.sht_forward(f, w)
    exp1 = {"ortho": math.sqrt(4 * math.pi / 3), "four-pi": 4 * math.pi / math.sqrt(3), "schmidt": 4 * math.pi / 3}[norm]
    assert abs(c[1, 0] - exp1) < 1e-9
    c[1, 0] = 0
    assert np.max(np.abs(c)) < 1e-9


def test_csphase_flips_odd_m():
    w1, _, _ = orc.sht_weights(16, 32, lmax=12, grid="legendre-gauss", csphase=True)
    w0, _, _ = orc.sht_weights(16, 32, lmax=12, grid="legendre-gauss", csphase=False)
    assert np.allclose(w1[1::2], -w0[1::2]) and np.allclose(w1[0::2], w0[0::2])


def test_roundtrip_fixed_point():
    """isht(sht(.)) is the identity on band-limited signals for Gauss-Legendre (reference
    tests/test_sht.py:108-168, tol 1e-9 in float64)."""
    nlat, nlon = 32, 64
    w, lmax, mmax = orc.sht_weights(nlat, nlon, grid="legendre-gauss")
    p, _, _ = orc.isht_pct(nlat, nlon, grid="legendre-gauss")
    a = orc.random_coeffs((3,), lmax, mmax, seed=7)
    x = orc.sht_inverse(a, p, nlon)
    for _ in range(4):
        x2 = orc.sht_inverse(orc.sht_forward(x, w), p, nlon)
        assert rel(x2, x) < 1e-9
        x = x2


# ---------------------------------------------------------------- per-call math vs reference outputs


def test_cfg1_matches_reference():
    g = gold("cfg1_equiangular_64x128.npz")
    x = np.random.default_rng(0).standard_normal((4, 8, 64, 128))[:2, :2]
    w, lmax, mmax = orc.sht_weights(64, 128, 64, 65, "equiangular")
    p, _, _ = orc.isht_pct(64, 128, 64, 65, "equiangular")
    assert [lmax, mmax] == list(g["lm"])
    c = orc.sht_forward(x, w)
    assert c.shape == (2, 2, 64, 64)
    assert rel(c, g["coeffs"]) < 1e-12
    assert rel(orc.sht_inverse(c, p, 128), g["roundtrip"]) < 1e-12


def test_cfg2_matches_reference():
    g = gold("cfg2_legendre_gauss_256x512.npz")
    a = orc.random_coeffs((2,), 256, 256, seed=1, power=1.0, offset=1.0)[:1]
    w, lmax, mmax = orc.sht_weights(256, 512, 256, 257, "legendre-gauss")
    p, _, _ = orc.isht_pct(256, 512, 256, 257, "legendre-gauss")
    x = orc.sht_inverse(a, p, 512)
    assert rel(x[:, ::4], g["field"]) < 1e-11
    c = orc.sht_forward(x, w)
    assert rel(c[:, ::4], g["coeffs"]) < 1e-11
    assert rel(c, a) < 1e-10  # Gauss-Legendre is exact for band-limited input


@pytest.mark.parametrize("tag,nlat,nlon,lmax,mmax,grid", [
    ("up", 12, 16, 12, 12, "legendre-gauss"),
    ("odd", 13, 25, 10, 10, "lobatto"),
    ("down", 16, 48, 6, 6, "equiangular"),
    ("nyq", 20, 16, 9, 9, "legendre-gauss"),
])
def test_truncation_cases(tag, nlat, nlon, lmax, mmax, grid):
    g = gold("truncation_cases.npz")
    w, L, M = orc.sht_weights(nlat, nlon, lmax, mmax, grid)
    p, _, _ = orc.isht_pct(nlat, nlon, lmax, mmax, grid)
    assert [L, M] == list(g[f"{tag}|lm"])
    rng = np.random.default_rng(50)
    x = rng.standard_normal((2, nlat, nlon))
    cin = rng.standard_normal((2, L, M)) + 1j * rng.standard_normal((2, L, M))
    assert rel(orc.sht_forward(x, w), g[f"{tag}|coeffs"]) < 1e-12
    assert rel(orc.sht_inverse(cin, p, nlon), g[f"{tag}|field"]) < 1e-12


@pytest.mark.parametrize("grid,nlat,nlon,lmax", [("equiangular", 33, 64, 20), ("legendre-gauss", 32, 64, None), ("lobatto", 33, 66, None)])
def test_vector_matches_reference(grid, nlat, nlon, lmax):
    g = gold("vector_small.npz")
    vw, L, M = orc.vsht_weights(nlat, nlon, lmax=lmax, grid=grid)
    vp, _, _ = orc.ivsht_dpct(nlat, nlon, lmax=L, mmax=M, grid=grid)
    assert [L, M] == list(g[f"{grid}|lm"])
    a = orc.random_coeffs((3, 2), L, M, seed=30, power=1.5, offset=1.0, zero_l0=True)
    v = orc.vsht_inverse(a, vp, nlon)
    assert rel(v, g[f"{grid}|field"]) < 1e-11
    assert rel(orc.vsht_forward(v, vw), g[f"{grid}|coeffs"]) < 1e-11


@pytest.mark.parametrize("tag,nlat,nlon,lmax,grid", [("eq", 17, 36, 12, "equiangular"), ("lg", 16, 30, 16, "legendre-gauss")])
def test_adjoints_match_reference_autograd(tag, nlat, nlon, lmax, grid):
    g = gold("autograd_small.npz")
    w, L, M = orc.sht_weights(nlat, nlon, lmax=lmax, grid=grid)
    p, _, _ = orc.isht_pct(nlat, nlon, lmax=lmax, grid=grid)
    assert [L, M] == list(g[f"{tag}|lm"])
    rng = np.random.default_rng(40)
    _x = rng.standard_normal((3, nlat, nlon))
    gy = rng.standard_normal((3, L, M)) + 1j * rng.standard_normal((3, L, M))
    assert rel(orc.sht_forward_vjp(gy, w, nlon), g[f"{tag}|sht_gx"]) < 1e-12
    gx = rng.standard_normal((3, nlat, nlon))
    assert rel(orc.sht_inverse_vjp(gx, p), g[f"{tag}|isht_gc"]) < 1e-12


# ---------------------------------------------------------------- full-size rows (721 x 1440)


@pytest.mark.slow
def test_cfg3_rows_match_reference():
    path = os.path.join(GOLD, "cfg3_equiangular_721x1440.npz")
    if not os.path.exists(path):
        pytest.skip("large fixture not generated")
    g = np.load(path)
    a = orc.random_coeffs((2,), 720, 720, seed=2, offset=25.0, zero_l0=True, mode="grf")
    p, _, _ = orc.isht_pct(721, 1440, 720, 720, "equiangular")
    x = orc.sht_inverse(a, p, 1440)
    del p
    assert np.max(np.abs(x[:, g["rows_k"]] - g["field_rows"])) / float(g["field_absmax"]) < 1e-11
    w, _, _ = orc.sht_weights(721, 1440, 720, 720, "equiangular")
    # the fixture keeps these rows of the reference's buffer in the precision the module held them in
    wtol = 1e-12 if g["weights_rows"].dtype == np.float64 else 2e-7
    assert rel(w[[0, 1, 2, 359, 719]][:, g["rows_l"]][:, :, ::40], g["weights_rows"]) < wtol
    c = orc.sht_forward(x, w)
    assert np.max(np.abs(c[:, g["rows_l"]] - g["coeff_rows"])) / float(g["coeff_absmax"]) < 1e-11
