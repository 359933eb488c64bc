"""CPU-only checks: the shared library builds / loads and exports every symbol the header declares, host-side
precompute of the package matches the oracle, and the product refuses to run without a GPU."""

import ctypes
import os
import re
import warnings

import numpy as np
import pytest
import torch

from oracle import sht_oracle as orc

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def lib():
    from torch_harmonics_b200 import _lib, build

    build.build()
    return _lib.load()


def test_header_symbols_exported(lib):
    hdr = open(os.path.join(ROOT, "include", "shtb200.h")).read()
    hdr = re.sub(r"/\*.*?\*/", "", hdr, flags=re.S)
    names = re.findall(r"\b(shtb200_[a-z0-9_]+)\s*\(", hdr)
    assert len(set(names)) >= 12
    for n in set(names):
        assert hasattr(lib, n), f"{n} declared in include/shtb200.h but not exported"
    assert lib.shtb200_version() >= 100


@pytest.mark.skipif(torch.cuda.is_available(), reason="checks the no-GPU failure mode")
def test_no_cpu_fallback(lib):
    import torch_harmonics_b200 as th

    h = ctypes.c_void_p()
    dummy = (ctypes.c_float * 4)()
    rc = lib.shtb200_plan_create(ctypes.byref(h), 0, 8, 16, 4, 4, ctypes.cast(dummy, ctypes.c_void_p), 0, 0)
    assert rc == -2 and b"no CUDA device" in lib.shtb200_last_error()
    m = th.RealSHT(8, 16, lmax=4, grid="legendre-gauss")
    with pytest.raises(RuntimeError, match="no CPU path"):
        m(torch.zeros(8, 16))
    # argument validation happens before any device work
    assert lib.shtb200_plan_create(ctypes.byref(h), 99, 8, 16, 4, 4, ctypes.cast(dummy, ctypes.c_void_p), 0, 0) == -1
    assert lib.shtb200_plan_create(None, 0, 8, 16, 4, 4, ctypes.cast(dummy, ctypes.c_void_p), 0, 0) == -1
    assert lib.shtb200_workspace_bytes(None, 4) == 0
    assert lib.shtb200_execute(None, None, None, 1, None, 0, None) == -1


@pytest.mark.parametrize("grid", ["equiangular", "legendre-gauss", "lobatto"])
@pytest.mark.parametrize("norm", ["ortho", "four-pi", "schmidt"])
def test_package_tables_match_oracle(grid, norm):
    import torch_harmonics_b200 as th

    kw = dict(lmax=11, grid=grid, norm=norm, csphase=(norm != "four-pi"))
    nlat, nlon = 15, 32
    assert orc.max_normalised_error(th.RealSHT(nlat, nlon, **kw).weights.numpy(), orc.sht_weights(nlat, nlon, **kw)[0]) < 1e-13
    assert orc.max_normalised_error(th.InverseRealSHT(nlat, nlon, **kw).pct.numpy(), orc.isht_pct(nlat, nlon, **kw)[0]) < 1e-13
    assert orc.max_normalised_error(th.RealVectorSHT(nlat, nlon, **kw).weights.numpy(), orc.vsht_weights(nlat, nlon, **kw)[0]) < 1e-13
    assert orc.max_normalised_error(th.InverseRealVectorSHT(nlat, nlon, **kw).dpct.numpy(), orc.ivsht_dpct(nlat, nlon, **kw)[0]) < 1e-13


def test_package_truncation():
    from torch_harmonics_b200.truncation import truncate_sht

    with warnings.catch_warnings():
        warnings.simplefilter("ignore")
        for args in ((33, 64, None, None, "equiangular"), (32, 64, None, None, "legendre-gauss"), (33, 64, None, None, "lobatto"),
                     (64, 128, 64, 65, "equiangular"), (8, 16, 12, 9, "legendre-gauss"), (8, 16, 0, 0, "lobatto")):
            assert truncate_sht(*args) == orc.truncate_sht(*args)
    with pytest.raises(ValueError):
        truncate_sht(8, 16, grid="nope")
    with pytest.warns(UserWarning):
        truncate_sht(8, 16, grid="equiangular")


def test_quadrature_and_random_field_buffers_match_reference():
    """Host-side set-up of QuadratureS2 / GaussianRandomFieldS2 / SpectralConvS2 against buffers of the reference
    (tests/golden/spectral_conv.npz)."""
    import torch_harmonics_b200 as th

    g = np.load(os.path.join(ROOT, "tests", "golden", "spectral_conv.npz"))
    for grid in ("equiangular", "legendre-gauss", "lobatto", "equiangular-trapezoidal"):
        for normalize in (False, True):
            q = th.QuadratureS2((13, 24), grid=grid, normalize=normalize)
            assert q.quad_weight.shape == (1, 1, 13, 24) and q.quad_weight.dtype == torch.float32
            assert np.allclose(q.quad_weight[0, 0, :, 0].numpy(), g[f"quad|{grid}|{int(normalize)}"], rtol=1e-6, atol=0)
    with pytest.raises(ValueError):
        th.QuadratureS2((13, 24), grid="nope")
    with warnings.catch_warnings():
        warnings.simplefilter("ignore")
        grf = th.GaussianRandomFieldS2(16, alpha=2.5, tau=4.0)
        assert [grf.isht.lmax, grf.isht.mmax] == list(g["grf|lm"])
        assert np.allclose(grf.sqrt_eig.numpy(), g["grf|sqrt_eig"], rtol=1e-6)
        with pytest.raises(ValueError):
            th.GaussianRandomFieldS2(16, alpha=1.0)
        conv = th.SpectralConvS2((17, 32), (12, 24), 6, 4, num_groups=2, grid_in="equiangular", grid_out="legendre-gauss", bias=True)
        assert conv.lmax == int(g["groups_resample|lmax"]) and conv.weight.shape == (2, 3, 2, conv.lmax)
        assert conv.spectral_bias.shape == (1, 6, conv.lmax, conv.mmax) and conv.weight.dtype == torch.complex64
        with pytest.raises(ValueError):
            th.SpectralConvS2((17, 32), (17, 32), 6, 4, num_groups=4)


def test_windowed_tables_equal_slices_of_the_full_tables():
    """A distributed rank builds the Legendre tables of its own orders only: bit-identical to the matching slice of the
    full table, scalar and vector, every normalisation."""
    from torch_harmonics_b200.legendre import _precompute_dlegpoly, _precompute_legpoly

    t = torch.linspace(0.01, 3.13, 23, dtype=torch.float64)
    for norm in ("ortho", "schmidt", "four-pi"):
        for inverse in (False, True):
            for cs in (True, False):
                full = _precompute_legpoly(12, 14, t, norm=norm, inverse=inverse, csphase=cs)
                dfull = _precompute_dlegpoly(12, 14, t, norm=norm, inverse=inverse, csphase=cs)
                for first, count in ((0, 5), (3, 4), (5, 7), (11, 1), (0, 12)):
                    assert torch.equal(_precompute_legpoly(12, 14, t, norm=norm, inverse=inverse, csphase=cs, m_first=first, m_count=count), full[first:first + count])
                    assert torch.equal(_precompute_dlegpoly(12, 14, t, norm=norm, inverse=inverse, csphase=cs, m_first=first, m_count=count), dfull[:, first:first + count])
