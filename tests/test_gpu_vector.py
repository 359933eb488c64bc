"""GPU parity of the vector transforms against the reference's outputs (tests/golden/vector_small.npz) and
the float64 oracle, through the module API and the C ABI."""

import os
import warnings

import numpy as np
import pytest

from oracle import sht_oracle as orc
from tests.helpers import TOL, err, make_plan, run_plan

pytestmark = pytest.mark.gpu
GOLD = os.path.join(os.path.dirname(__file__), "golden")


@pytest.mark.parametrize("engine", ["simt", "tcgen05"])
@pytest.mark.parametrize("grid,nlat,nlon,lmax", [("equiangular", 33, 64, 20), ("legendre-gauss", 32, 64, None), ("lobatto", 33, 66, None)])
def test_vector_reference_outputs(grid, nlat, nlon, lmax, engine):
    import torch

    from torch_harmonics_b200 import _lib

    g = np.load(os.path.join(GOLD, "vector_small.npz"))
    with warnings.catch_warnings():
        warnings.simplefilter("ignore")
        vw, L, M = orc.vsht_weights(nlat, nlon, lmax=lmax, grid=grid)
        vp, _, _ = orc.ivsht_dpct(nlat, nlon, lmax=L, mmax=M, grid=grid)
    a = orc.random_coeffs((3, 2), L, M, seed=30, power=1.5, offset=1.0, zero_l0=True)
    ivs = make_plan(_lib.IVSHT, nlat, nlon, L, M, vp, engine)
    vs = make_plan(_lib.VSHT, nlat, nlon, L, M, vw, engine)
    v = run_plan(ivs, a.astype(np.complex64), (3, 2, nlat, nlon), torch.float32, 3)
    assert err(v, g[f"{grid}|field"]) <= TOL
    c = run_plan(vs, g[f"{grid}|field"].astype(np.float32), (3, 2, L, M), torch.complex64, 3)
    assert err(c, g[f"{grid}|coeffs"]) <= TOL
    ll, mm = np.meshgrid(np.arange(L), np.arange(M), indexing="ij")
    assert np.all(c[:, :, ll < mm] == 0)


@pytest.mark.parametrize("tag,nlat,nlon,lmax,grid", [("eq", 17, 36, 12, "equiangular"), ("lg", 16, 30, 16, "legendre-gauss")])
def test_vector_autograd_matches_reference(tag, nlat, nlon, lmax, grid):
    import torch

    import torch_harmonics_b200 as th

    g = np.load(os.path.join(GOLD, "autograd_small.npz"))
    vs = th.RealVectorSHT(nlat, nlon, lmax=lmax, grid=grid).cuda()
    ivs = th.InverseRealVectorSHT(nlat, nlon, lmax=lmax, grid=grid).cuda()
    rng = np.random.default_rng(40)
    # replay the generator exactly as the fixture script drew from it
    L, M = vs.lmax, vs.mmax
    rng.standard_normal((3, nlat, nlon)); rng.standard_normal((3, L, M)); rng.standard_normal((3, L, M)); rng.standard_normal((3, nlat, nlon))
    xv = rng.standard_normal((2, 2, nlat, nlon))
    gv = rng.standard_normal((2, 2, L, M)) + 1j * rng.standard_normal((2, 2, L, M))
    xt = torch.from_numpy(xv).float().cuda().requires_grad_(True)
    vs(xt).backward(torch.from_numpy(gv).to(torch.complex64).cuda())
    assert err(xt.grad.cpu().numpy(), g[f"{tag}|vsht_gx"]) < TOL
    cv = rng.standard_normal((2, 2, L, M)) + 1j * rng.standard_normal((2, 2, L, M))
    gxv = rng.standard_normal((2, 2, nlat, nlon))
    ct = torch.from_numpy(cv).to(torch.complex64).cuda().requires_grad_(True)
    ivs(ct).backward(torch.from_numpy(gxv).float().cuda())
    assert err(ct.grad.cpu().numpy(), g[f"{tag}|ivsht_gc"]) < TOL


def test_vector_module_shapes_and_errors():
    import torch

    import torch_harmonics_b200 as th

    vs = th.RealVectorSHT(32, 64, grid="legendre-gauss").cuda()
    assert vs.weights.shape == (2, 32, 32, 32)
    ivs = th.InverseRealVectorSHT(32, 64, grid="legendre-gauss").cuda()
    assert ivs.dpct.shape == (2, 32, 32, 32)
    x = torch.randn(2, 3, 2, 32, 64, device="cuda")
    c = vs(x)
    assert c.shape == (2, 3, 2, 32, 32)
    assert ivs(c).shape == x.shape
    with pytest.raises(RuntimeError, match="vector field"):
        vs(torch.zeros(3, 32, 64, device="cuda"))


@pytest.mark.parametrize("engine", ["simt", "tcgen05"])
@pytest.mark.parametrize("nlat,nlon,lmax,grid,npairs", [(24, 512, 20, "legendre-gauss", 5), (25, 720, 22, "equiangular", 3), (23, 1440, 16, "legendre-gauss", 6)])
def test_vector_two_pass_longitudes_match_oracle(nlat, nlon, lmax, grid, npairs, engine):
    """Vector transforms on longitudes that take the register-resident two-pass FFT kernels (their emit carries the
    component sign pattern), with pair counts that leave the last block of eight component fields ragged."""
    import torch

    from torch_harmonics_b200 import _lib

    with warnings.catch_warnings():
        warnings.simplefilter("ignore")
        vw, L, M = orc.vsht_weights(nlat, nlon, lmax=lmax, grid=grid)
        vp, _, _ = orc.ivsht_dpct(nlat, nlon, lmax=L, mmax=M, grid=grid)
    rng = np.random.default_rng(nlon)
    x = rng.standard_normal((npairs, 2, nlat, nlon)).astype(np.float32)
    c = run_plan(make_plan(_lib.VSHT, nlat, nlon, L, M, vw, engine), x, (npairs, 2, L, M), torch.complex64, npairs)
    assert err(c, orc.vsht_forward(x.astype(np.float64), vw)) <= TOL
    a = (rng.standard_normal((npairs, 2, L, M)) + 1j * rng.standard_normal((npairs, 2, L, M))).astype(np.complex64)
    v = run_plan(make_plan(_lib.IVSHT, nlat, nlon, L, M, vp, engine), a, (npairs, 2, nlat, nlon), torch.float32, npairs)
    assert err(v, orc.vsht_inverse(a.astype(np.complex128), vp, nlon)) <= TOL
