"""GPU tests of the nn.Module API: the properties the reference's own suite checks (known answers, norms,
csphase, Parseval-type identities, autograd), restated at float32 tolerances, plus the reference's error
behaviour.  Reference: torch-harmonics tests/test_sht.py."""

import math
import os
import warnings

import numpy as np
import pytest

from oracle import sht_oracle as orc
from tests.helpers import TOL, err

pytestmark = pytest.mark.gpu
GOLD = os.path.join(os.path.dirname(__file__), "golden")


def _mods(*a, **k):
    import torch_harmonics_b200 as th

    with warnings.catch_warnings():
        warnings.simplefilter("ignore")
        return th.RealSHT(*a, **k).cuda(), th.InverseRealSHT(*a, **k).cuda()


@pytest.mark.parametrize("grid", ["equiangular", "legendre-gauss", "lobatto"])
@pytest.mark.parametrize("norm", ["ortho", "four-pi", "schmidt"])
def test_known_answers(grid, norm):
    """f = 1 and f = cos(theta): reference tests/test_sht.py:278-414."""
    import torch

    nlat, nlon = 32, 64
    sht, _ = _mods(nlat, nlon, lmax=16, grid=grid, norm=norm)
    tq, _ = orc.colatitudes(nlat, grid)
    one = torch.ones(nlat, nlon, device="cuda")
    c = sht(one).cpu().numpy()
    exp0 = {"ortho": math.sqrt(4 * math.pi), "four-pi": 4 * math.pi, "schmidt": 4 * math.pi}[norm]
    assert abs(c[0, 0] - exp0) < 1e-5 * exp0
    c[0, 0] = 0
    assert np.max(np.abs(c)) < 2e-5 * exp0
    f = torch.from_numpy(np.cos(tq)[:, None] * np.ones((1, nlon))).float().cuda()
    cb = sht(f.expand(3, nlat, nlon)).cpu().numpy()
    c = sht(f).cpu().numpy()
    assert np.array_equal(cb[1], c)  # batched == unbatched
    exp1 = {"ortho": math.sqrt(4 * math.pi / 3), "four-pi": 4 * math.pi / math.sqrt(3), "schmidt": 4 * math.pi / 3}[norm]
    assert abs(c[1, 0] - exp1) < 1e-5 * exp1
    c[1, 0] = 0
    assert np.max(np.abs(c)) < 2e-5 * exp1


def test_cross_norm_and_csphase():
    """four-pi = ortho * sqrt(4 pi), schmidt = ortho * sqrt(4 pi / (2l+1)); csphase flips odd m
    (reference tests/test_sht.py:230-276, :416-473)."""
    import torch

    import torch_harmonics_b200 as th

    nlat, nlon = 32, 64
    x = torch.from_numpy(np.random.default_rng(1).standard_normal((2, nlat, nlon))).float().cuda()
    co = th.RealSHT(nlat, nlon, grid="legendre-gauss", norm="ortho").cuda()(x).cpu().numpy()
    cf = th.RealSHT(nlat, nlon, grid="legendre-gauss", norm="four-pi").cuda()(x).cpu().numpy()
    cs = th.RealSHT(nlat, nlon, grid="legendre-gauss", norm="schmidt").cuda()(x).cpu().numpy()
    l = np.arange(co.shape[-2])[:, None]
    assert err(cf, co * math.sqrt(4 * math.pi)) < TOL
    assert err(cs, co * np.sqrt(4 * math.pi / (2 * l + 1))) < TOL
    cn = th.RealSHT(nlat, nlon, grid="legendre-gauss", csphase=False).cuda()(x).cpu().numpy()
    sign = np.where(np.arange(co.shape[-1]) % 2 == 1, -1.0, 1.0)
    assert err(cn, co * sign) < TOL


@pytest.mark.parametrize("grid,nlat", [("legendre-gauss", 32), ("lobatto", 33), ("equiangular", 33)])
def test_roundtrip_fixed_point_and_parseval(grid, nlat):
    """isht(sht(.)) is a fixed point on band-limited signals (reference tests/test_sht.py:108-168, tol 1e-9 in
    float64; float32 here) and the spectral sum of squares equals the quadrature of f^2 (:475-537)."""
    import torch

    nlon = 64
    sht, isht = _mods(nlat, nlon, lmax=16, grid=grid)
    a = orc.random_coeffs((3,), 16, 16, seed=2)
    x = isht(torch.from_numpy(a).to(torch.complex64).cuda())
    x0 = x.clone()
    for _ in range(4):
        x = isht(sht(x))
    assert err(x.cpu().numpy(), x0.cpu().numpy()) < 2e-5
    c = sht(x0).cpu().numpy().astype(np.complex128)
    spec = np.sum(np.abs(c[..., 0]) ** 2, axis=-1) + 2 * np.sum(np.abs(c[..., 1:]) ** 2, axis=(-1, -2))
    _, w = orc.colatitudes(nlat, grid)
    quad = np.sum(x0.cpu().numpy().astype(np.float64) ** 2 * w[:, None], axis=(-1, -2)) * 2 * np.pi / nlon
    assert np.max(np.abs(spec - quad) / quad) < 1e-4


@pytest.mark.parametrize("tag,nlat,nlon,lmax,grid", [("eq", 17, 36, 12, "equiangular"), ("lg", 16, 30, 16, "legendre-gauss")])
def test_autograd_matches_reference(tag, nlat, nlon, lmax, grid):
    """Input gradients against those the reference's autograd produced (tests/golden/autograd_small.npz)."""
    import torch

    g = np.load(os.path.join(GOLD, "autograd_small.npz"))
    sht, isht = _mods(nlat, nlon, lmax=lmax, grid=grid)
    rng = np.random.default_rng(40)
    x = rng.standard_normal((3, nlat, nlon))
    gy = rng.standard_normal((3, sht.lmax, sht.mmax)) + 1j * rng.standard_normal((3, sht.lmax, sht.mmax))
    xt = torch.from_numpy(x).float().cuda().requires_grad_(True)
    sht(xt).backward(torch.from_numpy(gy).to(torch.complex64).cuda())
    assert err(xt.grad.cpu().numpy(), g[f"{tag}|sht_gx"]) < TOL
    c = orc.random_coeffs((3,), sht.lmax, sht.mmax, seed=41) + 0j
    c[..., :, 0] += 0.3j
    gx = rng.standard_normal((3, nlat, nlon))
    ct = torch.from_numpy(c).to(torch.complex64).cuda().requires_grad_(True)
    isht(ct).backward(torch.from_numpy(gx).float().cuda())
    assert err(ct.grad.cpu().numpy(), g[f"{tag}|isht_gc"]) < TOL
    # a loss through both modules, double-checking the chain
    xt2 = torch.from_numpy(x).float().cuda().requires_grad_(True)
    loss = (isht(sht(xt2)) ** 2).sum()
    loss.backward()
    assert torch.isfinite(xt2.grad).all()


def test_api_surface_and_errors():
    import torch

    import torch_harmonics_b200 as th

    with pytest.warns(UserWarning):
        m = th.RealSHT(33, 64)
    assert (m.lmax, m.mmax) == (17, 17)
    assert m.weights.shape == (17, 17, 33) and m.weights.dtype == torch.float64
    assert "weights" not in m.state_dict()
    assert "nlat=33" in m.extra_repr()
    im = th.InverseRealSHT(33, 64, lmax=17)
    assert im.pct.shape == (17, 33, 17)
    with pytest.raises(ValueError):
        th.RealSHT(16, 32, grid="equiangular-trapezoidal")
    m = m.cuda()
    with pytest.raises(RuntimeError, match="Expected latitudes"):
        m(torch.zeros(2, 32, 64, device="cuda"))
    with pytest.raises(RuntimeError, match="Expected longitudes"):
        m(torch.zeros(2, 33, 63, device="cuda"))
    with pytest.raises(RuntimeError, match="at least 2 dimensions"):
        m(torch.zeros(64, device="cuda"))
    with pytest.raises(RuntimeError, match="no CPU path"):
        m(torch.zeros(33, 64))
    with pytest.raises(TypeError):
        m(torch.zeros(33, 64, device="cuda", dtype=torch.float64))
    # non-contiguous input, extra leading dims, empty batch, float()-ed module
    x = torch.randn(2, 3, 64, 33, device="cuda").transpose(-1, -2)
    y = m(x)
    assert y.shape == (2, 3, 17, 17) and y.is_contiguous() and y.dtype == torch.complex64
    assert torch.equal(y, m(x.contiguous()))
    assert m(torch.zeros(0, 33, 64, device="cuda")).shape == (0, 17, 17)
    y32 = m.float()(x)
    assert err(y32.cpu().numpy(), y.cpu().numpy()) < 1e-6
    with torch.device("cuda"):
        m2 = th.RealSHT(12, 24, lmax=8, grid="legendre-gauss")
    assert m2.weights.is_cuda
    assert m2(torch.ones(12, 24, device="cuda")).shape == (8, 8)


def test_custom_operator_traces_and_matches_eager():
    """The transforms are one torch custom operator: shape inference without running (fake tensors), a full-graph
    torch.compile trace of a module pair, and gradients through the compiled graph equal to the eager ones."""
    import torch

    import torch_harmonics_b200 as th
    from torch_harmonics_b200.sht import _linear_transform

    nlat, nlon = 33, 64
    sht, isht = th.RealSHT(nlat, nlon, grid="equiangular").cuda(), th.InverseRealSHT(nlat, nlon, grid="equiangular").cuda()
    x = torch.randn(3, 2, nlat, nlon, device="cuda", generator=torch.Generator(device="cuda").manual_seed(5))

    # operator-level checks: schema, fake implementation, autograd registration
    torch.library.opcheck(_linear_transform, (x, sht._op.handle, False, [sht.lmax, sht.mmax], True, 2), test_utils=("test_schema", "test_faketensor", "test_autograd_registration"))

    def roundtrip(t):
        return isht(sht(t))

    compiled = torch.compile(roundtrip, fullgraph=True, backend="aot_eager")
    xa = x.clone().requires_grad_(True)
    xb = x.clone().requires_grad_(True)
    ya, yb = roundtrip(xa), compiled(xb)
    assert torch.equal(ya.detach(), yb.detach())
    g = torch.randn_like(ya)
    ya.backward(g)
    yb.backward(g)
    assert torch.equal(xa.grad, xb.grad)


@pytest.mark.parametrize("family", ["scalar", "vector", "distributed"])
def test_autocast_region_leaves_the_transforms_in_float32(family):
    """Inside torch.autocast the transforms still take float32 / complex64 tensors and compute in float32, forward and
    backward (the reference asks callers to guard its modules with autocast(enabled=False), torch_harmonics/sht.py:95-107;
    SpectralConvS2 does so at spectral_convolution.py:226-243): results equal those outside the region bit for bit, and a
    half-precision input is refused rather than silently converted."""
    import torch

    import torch_harmonics_b200 as th
    import torch_harmonics_b200.distributed as thd

    nlat, nlon = 33, 64
    with warnings.catch_warnings():
        warnings.simplefilter("ignore")
        if family == "scalar":
            fwd, inv = th.RealSHT(nlat, nlon, lmax=17).cuda(), th.InverseRealSHT(nlat, nlon, lmax=17).cuda()
            shape = (2, 3, nlat, nlon)
        elif family == "vector":
            fwd, inv = th.RealVectorSHT(nlat, nlon, lmax=17).cuda(), th.InverseRealVectorSHT(nlat, nlon, lmax=17).cuda()
            shape = (2, 2, nlat, nlon)
        else:
            fwd, inv = thd.DistributedRealSHT(nlat, nlon, lmax=17).cuda(), thd.DistributedInverseRealSHT(nlat, nlon, lmax=17).cuda()
            shape = (2, 3, nlat, nlon)
    x = torch.randn(*shape, device="cuda", generator=torch.Generator(device="cuda").manual_seed(3))
    xa = x.clone().requires_grad_(True)
    ya = inv(fwd(xa))
    ya.square().sum().backward()
    xb = x.clone().requires_grad_(True)
    with torch.autocast(device_type="cuda", dtype=torch.bfloat16):
        cb = fwd(xb)
        yb = inv(cb)
        assert cb.dtype == torch.complex64 and yb.dtype == torch.float32
        lin = torch.nn.functional.linear(yb, torch.eye(nlon, device="cuda"))  # an op autocast does convert
        assert lin.dtype == torch.bfloat16
        with pytest.raises(TypeError):
            fwd(x.to(torch.bfloat16))
    yb.square().sum().backward()
    assert torch.equal(ya.detach(), yb.detach())
    assert torch.equal(xa.grad, xb.grad)


def test_module_release_frees_plans():
    """Dropping a module destroys its plans at once (no reference cycle keeps the packed tables alive), and close()
    releases them explicitly; the next call rebuilds them."""
    import gc

    import torch

    sht, _ = _mods(33, 64, lmax=17)
    x = torch.randn(2, 33, 64, device="cuda")
    c0 = sht(x)
    plans = list(sht._op.plans.values())
    assert plans and all(p.handle for p in plans)
    sht.close()
    assert all(p.handle is None for p in plans) and not sht._op.plans
    assert torch.equal(sht(x), c0)
    plans = list(sht._op.plans.values())
    gc.disable()
    try:
        del sht
        assert all(p.handle is None for p in plans)
    finally:
        gc.enable()
