"""GPU parity of the scalar transforms, called through the C ABI (ctypes) on seeded inputs and checked
against the float64 oracle and the committed reference outputs.  Tolerance: max-normalised error <= 1e-5
(``helpers.TOL``), the bound stated for the float32 path."""

import os

import numpy as np
import pytest

from oracle import sht_oracle as orc
from tests.helpers import TOL, err, make_plan, oracle_tables, run_plan

pytestmark = pytest.mark.gpu
GOLD = os.path.join(os.path.dirname(__file__), "golden")

ENGINES = ["simt", "tcgen05"]

# (nlat, nlon, lmax, mmax, grid, nfields): odd / even nlat, odd nlon, nlon with factors 7 and 11,
# mmax above nlon//2+1 (zero-padded orders), tiny and ragged sizes, lmax > nlat
SHAPES = [
    (64, 128, 64, 65, "equiangular", 32),
    (33, 64, 17, 17, "equiangular", 5),
    (32, 64, None, None, "legendre-gauss", 3),
    (33, 66, None, None, "lobatto", 2),
    (13, 25, 10, 10, "lobatto", 1),
    (12, 16, 12, 12, "legendre-gauss", 4),
    (20, 16, 9, 9, "legendre-gauss", 2),
    (16, 48, 6, 6, "equiangular", 7),
    (9, 14, 5, 5, "legendre-gauss", 3),
    (8, 16, 12, 9, "legendre-gauss", 2),
    (91, 180, 90, 90, "equiangular", 9),
    (2, 4, 2, 2, "legendre-gauss", 1),
    # longitudes with a register-resident two-pass FFT (1440 = 40 x 36, 720 = 36 x 20, 512 = 32 x 16), ragged field counts
    (45, 1440, 40, 40, "legendre-gauss", 11),
    (91, 720, 90, 90, "equiangular", 10),
    (40, 512, 40, 40, "legendre-gauss", 9),
]


@pytest.mark.parametrize("engine", ENGINES)
@pytest.mark.parametrize("nlat,nlon,lmax,mmax,grid,nf", SHAPES)
def test_sht_matches_oracle(nlat, nlon, lmax, mmax, grid, nf, engine):
    import torch

    from torch_harmonics_b200 import _lib

    w, p, L, M = oracle_tables(nlat, nlon, lmax, mmax, grid)
    x = np.random.default_rng(nlat * 1000 + nlon).standard_normal((nf, nlat, nlon)).astype(np.float32)
    plan = make_plan(_lib.SHT, nlat, nlon, L, M, w, engine)
    c = run_plan(plan, x, (nf, L, M), torch.complex64, nf)
    ref = orc.sht_forward(x.astype(np.float64), w)
    assert not np.isnan(c).any()
    assert err(c, ref) <= TOL
    # exact zeros above the diagonal, like the reference's dense table produces
    ll, mm = np.meshgrid(np.arange(L), np.arange(M), indexing="ij")
    assert np.all(c[:, ll < mm] == 0)


@pytest.mark.parametrize("engine", ENGINES)
@pytest.mark.parametrize("nlat,nlon,lmax,mmax,grid,nf", SHAPES)
def test_isht_matches_oracle(nlat, nlon, lmax, mmax, grid, nf, engine):
    import torch

    from torch_harmonics_b200 import _lib

    w, p, L, M = oracle_tables(nlat, nlon, lmax, mmax, grid)
    rng = np.random.default_rng(nlat * 1000 + nlon + 1)
    c = (rng.standard_normal((nf, L, M)) + 1j * rng.standard_normal((nf, L, M))).astype(np.complex64)
    plan = make_plan(_lib.ISHT, nlat, nlon, L, M, p, engine)
    x = run_plan(plan, c, (nf, nlat, nlon), torch.float32, nf)
    ref = orc.sht_inverse(c.astype(np.complex128), p, nlon)
    assert not np.isnan(x).any()
    assert err(x, ref) <= TOL


@pytest.mark.parametrize("engine", ENGINES)
@pytest.mark.parametrize("nlat,nlon,lmax,grid", [(17, 36, 12, "equiangular"), (16, 30, 16, "legendre-gauss"), (33, 64, 20, "equiangular")])
def test_adjoints_match_oracle(nlat, nlon, lmax, grid, engine):
    import torch

    from torch_harmonics_b200 import _lib

    w, p, L, M = oracle_tables(nlat, nlon, lmax, None, grid)
    rng = np.random.default_rng(5)
    g = (rng.standard_normal((3, L, M)) + 1j * rng.standard_normal((3, L, M))).astype(np.complex64)
    plan = make_plan(_lib.SHT_ADJOINT, nlat, nlon, L, M, w, engine)
    gx = run_plan(plan, g, (3, nlat, nlon), torch.float32, 3)
    assert err(gx, orc.sht_forward_vjp(g.astype(np.complex128), w, nlon)) <= TOL
    gxx = rng.standard_normal((3, nlat, nlon)).astype(np.float32)
    plan = make_plan(_lib.ISHT_ADJOINT, nlat, nlon, L, M, p, engine)
    gc = run_plan(plan, gxx, (3, L, M), torch.complex64, 3)
    assert err(gc, orc.sht_inverse_vjp(gxx.astype(np.float64), p)) <= TOL


@pytest.mark.parametrize("engine", ENGINES)
def test_cfg1_reference_outputs(engine):
    """Equiangular 64x128, lmax 64, mmax 65 asked (resolves to 64, 64), N(0,1) input of seed 0: coefficients and
    round trip against the reference's own float64 outputs."""
    import torch

    from torch_harmonics_b200 import _lib

    g = np.load(os.path.join(GOLD, "cfg1_equiangular_64x128.npz"))
    x = np.random.default_rng(0).standard_normal((4, 8, 64, 128)).astype(np.float32)
    w, p, L, M = oracle_tables(64, 128, 64, 65, "equiangular")
    assert (L, M) == (64, 64)
    sht = make_plan(_lib.SHT, 64, 128, L, M, w, engine)
    isht = make_plan(_lib.ISHT, 64, 128, L, M, p, engine)
    c = run_plan(sht, x.reshape(32, 64, 128), (32, 64, 64), torch.complex64, 32).reshape(4, 8, 64, 64)
    assert err(c[:2, :2], g["coeffs"]) <= TOL
    rt = run_plan(isht, c.reshape(32, 64, 64), (32, 64, 128), torch.float32, 32).reshape(4, 8, 64, 128)
    assert err(rt[:2, :2], g["roundtrip"]) <= TOL


@pytest.mark.parametrize("engine", ENGINES)
def test_cfg2_reference_outputs(engine):
    """Legendre-Gauss 256x512, (256, 256): band-limited field synthesised from seeded coefficients."""
    import torch

    from torch_harmonics_b200 import _lib

    g = np.load(os.path.join(GOLD, "cfg2_legendre_gauss_256x512.npz"))
    a = orc.random_coeffs((2,), 256, 256, seed=1, power=1.0, offset=1.0)
    w, p, L, M = oracle_tables(256, 512, 256, 257, "legendre-gauss")
    isht = make_plan(_lib.ISHT, 256, 512, L, M, p, engine)
    sht = make_plan(_lib.SHT, 256, 512, L, M, w, engine)
    x = run_plan(isht, a.astype(np.complex64), (2, 256, 512), torch.float32, 2)
    assert err(x[:1, ::4], g["field"]) <= TOL
    c = run_plan(sht, x, (2, 256, 256), torch.complex64, 2)
    assert err(c[:1, ::4], g["coeffs"]) <= TOL
    assert err(c, a) <= 2 * TOL  # exact quadrature: the round trip recovers the coefficients


@pytest.mark.parametrize("tag,nlat,nlon,lmax,mmax,grid", [
    ("up", 12, 16, 12, 12, "legendre-gauss"),
    ("odd", 13, 25, 10, 10, "lobatto"),
    ("down", 16, 48, 6, 6, "equiangular"),
    ("nyq", 20, 16, 9, 9, "legendre-gauss"),
])
@pytest.mark.parametrize("engine", ENGINES)
def test_truncation_reference_outputs(tag, nlat, nlon, lmax, mmax, grid, engine):
    import torch

    from torch_harmonics_b200 import _lib

    g = np.load(os.path.join(GOLD, "truncation_cases.npz"))
    w, p, L, M = oracle_tables(nlat, nlon, lmax, mmax, grid)
    rng = np.random.default_rng(50)
    x = rng.standard_normal((2, nlat, nlon))
    cin = rng.standard_normal((2, L, M)) + 1j * rng.standard_normal((2, L, M))
    c = run_plan(make_plan(_lib.SHT, nlat, nlon, L, M, w, engine), x.astype(np.float32), (2, L, M), torch.complex64, 2)
    assert err(c, g[f"{tag}|coeffs"]) <= TOL
    y = run_plan(make_plan(_lib.ISHT, nlat, nlon, L, M, p, engine), cin.astype(np.complex64), (2, nlat, nlon), torch.float32, 2)
    assert err(y, g[f"{tag}|field"]) <= TOL


@pytest.mark.parametrize("engine", ENGINES)
def test_host_buffer_call_and_errors(engine):
    import ctypes

    import torch

    from torch_harmonics_b200 import _lib

    w, p, L, M = oracle_tables(33, 64, 17, 17, "equiangular")
    plan = make_plan(_lib.SHT, 33, 64, L, M, w, engine)
    x = np.random.default_rng(3).standard_normal((6, 33, 64)).astype(np.float32)
    xt = torch.from_numpy(x).pin_memory()
    out = torch.empty((6, L, M), dtype=torch.complex64).pin_memory()
    plan.execute_host(xt, out, 6)
    assert err(out.numpy(), orc.sht_forward(x.astype(np.float64), w)) <= TOL
    assert plan.last_launch_count == 3
    # empty batch is a no-op; undersized workspace is reported, not overrun
    plan.execute_host(xt, out, 0)
    xd = xt.cuda()
    od = torch.empty((6, L, M), dtype=torch.complex64, device="cuda")
    small = torch.empty(256, dtype=torch.uint8, device="cuda")
    with pytest.raises(_lib.ShtLibraryError, match="workspace too small"):
        plan.execute(xd, od, 6, small, 0)
    lib = _lib.load()
    h = ctypes.c_void_p()
    t = torch.zeros(4, device="cuda")
    assert lib.shtb200_plan_create(ctypes.byref(h), 0, 8, 2 * 37, 4, 4, ctypes.c_void_p(t.data_ptr()), 0, 0) == -1  # prime factor 37
    assert b"prime factor" in lib.shtb200_last_error()
    assert lib.shtb200_plan_create(ctypes.byref(h), 0, 8, 16, 4, 6, ctypes.c_void_p(t.data_ptr()), 0, 0) == -1  # mmax > lmax


def test_linearity_and_batch_independence():
    """Size-independent properties: T(a x + b y) = a T x + b T y, and a field's result does not depend on its batch."""
    import torch

    from torch_harmonics_b200 import _lib

    w, p, L, M = oracle_tables(91, 180, 90, 90, "equiangular")
    plan = make_plan(_lib.SHT, 91, 180, L, M, w)
    rng = np.random.default_rng(9)
    x = rng.standard_normal((4, 91, 180)).astype(np.float32)
    y = rng.standard_normal((4, 91, 180)).astype(np.float32)
    cx = run_plan(plan, x, (4, L, M), torch.complex64, 4)
    cy = run_plan(plan, y, (4, L, M), torch.complex64, 4)
    cz = run_plan(plan, (2 * x - 3 * y).astype(np.float32), (4, L, M), torch.complex64, 4)
    assert err(cz, 2 * cx - 3 * cy) <= TOL
    c1 = run_plan(plan, x[2:3], (1, L, M), torch.complex64, 1)
    assert err(c1, cx[2:3]) <= 1e-6


def _split(n, p):
    q, r = divmod(n, p)
    return [q + (1 if j < r else 0) for j in range(p)]


@pytest.mark.parametrize("nlon,nmodes,nrows,gp,mp", [(1440, 720, 37, 2, 2), (1440, 721, 16, 4, 3), (1440, 100, 1, 8, 1), (720, 361, 50, 4, 8), (720, 400, 21, 1, 7),
                                                    (512, 257, 33, 8, 2), (512, 96, 15, 2, 5)])
def test_piece_major_row_transforms(nlon, nmodes, nrows, gp, mp):
    """Row transforms on piece-major buffers (the receive / send layout of an all-to-all transpose whose last axis is
    gathered / scattered: chunk j of the axis is its own contiguous (nrows, width_j) block) give bit for bit the plain
    transforms' results, rearranged."""
    import ctypes

    import torch

    from torch_harmonics_b200 import _lib

    lib = _lib.load()
    vp = ctypes.c_void_p
    assert lib.shtb200_rows_pieces_supported(nlon, nmodes, gp, mp) == 1
    gen = torch.Generator(device="cuda").manual_seed(nrows)
    x = torch.randn(nrows, nlon, device="cuda", generator=gen)

    def to_pieces(t, p):
        return torch.cat([c.reshape(-1) for c in torch.split(t, _split(t.shape[1], p), dim=1)])

    plain = torch.empty(nrows, nmodes, dtype=torch.complex64, device="cuda")
    assert lib.shtb200_rfft_modes(vp(x.data_ptr()), vp(plain.data_ptr()), nrows, nlon, nmodes, 2.0, None) == 0
    xin = to_pieces(x, gp)
    out = torch.full((nrows * nmodes * 2,), float("nan"), device="cuda")
    assert lib.shtb200_rfft_modes_pieces(vp(xin.data_ptr()), vp(out.data_ptr()), nrows, nlon, nmodes, 2.0, gp, mp, None) == 0
    torch.cuda.synchronize()
    expect = torch.cat([torch.view_as_real(c.contiguous()).reshape(-1) for c in torch.split(plain, _split(nmodes, mp), dim=1)])
    assert torch.equal(out, expect)

    c = torch.view_as_complex(torch.randn(nrows, nmodes, 2, device="cuda", generator=gen))
    plain_y = torch.empty(nrows, nlon, device="cuda")
    assert lib.shtb200_irfft_modes(vp(c.data_ptr()), vp(plain_y.data_ptr()), nrows, nlon, nmodes, None) == 0
    cin = torch.cat([torch.view_as_real(p.contiguous()).reshape(-1) for p in torch.split(c, _split(nmodes, mp), dim=1)])
    y = torch.full((nrows * nlon,), float("nan"), device="cuda")
    assert lib.shtb200_irfft_modes_pieces(vp(cin.data_ptr()), vp(y.data_ptr()), nrows, nlon, nmodes, mp, gp, None) == 0
    torch.cuda.synchronize()
    assert torch.equal(y, to_pieces(plain_y, gp))


def test_piece_major_row_transforms_unsupported_shapes():
    import ctypes

    import torch

    from torch_harmonics_b200 import _lib

    lib = _lib.load()
    # no two-pass kernel for nlon; pieces that are not equal multiples of four longitudes; more pieces than orders
    for nlon, nmodes, gp, mp in ((64, 33, 2, 2), (1440, 720, 7, 1), (720, 361, 16, 1), (512, 257, 1, 300)):
        assert lib.shtb200_rows_pieces_supported(nlon, nmodes, gp, mp) == 0
    x = torch.zeros(4, 64, device="cuda")
    out = torch.zeros(4 * 33 * 2, device="cuda")
    rc = lib.shtb200_rfft_modes_pieces(ctypes.c_void_p(x.data_ptr()), ctypes.c_void_p(out.data_ptr()), 4, 64, 33, 1.0, 2, 2, None)
    assert rc != 0 and "piece-major" in lib.shtb200_last_error().decode()


def test_sm_limit_changes_grids_not_results():
    """``shtb200_set_sm_limit`` caps the SMs the persistent kernels are sized for (room for collectives running beside
    them); results are bit for bit those of the unlimited launch, and the setter returns the previous cap."""
    import torch

    from torch_harmonics_b200 import _lib

    nlat, nlon = 91, 720
    w, p, L, M = oracle_tables(nlat, nlon, 90, 90, "equiangular")
    gen = torch.Generator(device="cuda").manual_seed(2)
    x = torch.randn(40, nlat, nlon, device="cuda", generator=gen)
    fwd, inv = make_plan(_lib.SHT, nlat, nlon, L, M, w, "auto"), make_plan(_lib.ISHT, nlat, nlon, L, M, p, "auto")

    def roundtrip():
        c = torch.empty(40, L, M, dtype=torch.complex64, device="cuda")
        y = torch.empty_like(x)
        ws = torch.empty(max(fwd.workspace_bytes(40), inv.workspace_bytes(40)), dtype=torch.uint8, device="cuda")
        fwd.execute(x, c, 40, ws, 0)
        inv.execute(c, y, 40, ws, 0)
        torch.cuda.synchronize()
        return c, y

    assert _lib.set_sm_limit(0) == 0
    c0, y0 = roundtrip()
    try:
        assert _lib.set_sm_limit(24) == 0
        c1, y1 = roundtrip()
        assert _lib.set_sm_limit(1) == 24
        c2, y2 = roundtrip()
    finally:
        _lib.set_sm_limit(0)
    assert torch.equal(c0, c1) and torch.equal(y0, y1) and torch.equal(c0, c2) and torch.equal(y0, y2)


@pytest.mark.parametrize("pieces_in,pieces_out", [(2, 2), (3, 4), (1, 5), (4, 1)])
def test_piece_major_legendre_stage(pieces_in, pieces_out):
    """The contraction stage on piece-major tensors (row axis in balanced chunks, chunk j its own contiguous
    (fields, rows_j, orders) block: what the polar all-to-all delivers and takes) equals the plain stage bit for bit,
    rearranged - scalar and vector plans, both directions, orders that do not start at 0."""
    import torch

    from torch_harmonics_b200 import _lib

    nlat, nlon, grid = 33, 64, "equiangular"
    w, p, L, M = oracle_tables(nlat, nlon, 20, 20, grid)
    vw, _, _ = orc.vsht_weights(nlat, nlon, lmax=20, mmax=20, grid=grid)
    vp, _, _ = orc.ivsht_dpct(nlat, nlon, lmax=20, mmax=20, grid=grid)
    nf, m0, mloc = 5, 3, 11
    gen = torch.Generator(device="cuda").manual_seed(9)

    def to_pieces(t, n):  # t: (fields, [2,] rows, orders) complex
        return torch.cat([torch.view_as_real(c.contiguous()).reshape(-1) for c in torch.split(t, _split(t.shape[-2], n), dim=-2)])

    for kind, table, comp, rows_in, rows_out in ((_lib.SHT, w, (), nlat, L), (_lib.ISHT, p, (), L, nlat), (_lib.VSHT, vw, (2,), nlat, L), (_lib.IVSHT, vp, (2,), L, nlat)):
        plan = make_plan(kind, nlat, nlon, L, M, table, "auto")
        x = torch.view_as_complex(torch.randn((nf,) + comp + (rows_in, mloc, 2), device="cuda", generator=gen))
        ws = torch.empty(plan.legendre_workspace_bytes(nf, mloc), dtype=torch.uint8, device="cuda")
        plain = torch.full((nf,) + comp + (rows_out, mloc), float("nan"), dtype=torch.complex64, device="cuda")
        plan.legendre(x, plain, nf, m0, mloc, ws, 0)
        out = torch.full((plain.numel() * 2,), float("nan"), device="cuda")
        plan.legendre(to_pieces(x, pieces_in), out, nf, m0, mloc, ws, 0, in_pieces=pieces_in, out_pieces=pieces_out)
        torch.cuda.synchronize()
        assert torch.equal(out, to_pieces(plain, pieces_out)), kind
    with pytest.raises(_lib.ShtLibraryError, match="piece counts"):
        plan.legendre(x, plain, nf, m0, mloc, ws, 0, in_pieces=L + 1, out_pieces=1)


@pytest.mark.parametrize("engine", ENGINES)
def test_stage_entry_points(engine):
    """rfft / irfft row transforms and the stand-alone Legendre stage used by the distributed modules
    (the latter on a window of orders that does not start at m = 0)."""
    import ctypes

    import torch

    from torch_harmonics_b200 import _lib

    lib = _lib.load()
    rng = np.random.default_rng(11)
    # (the last six take the two-pass row kernels: full and ragged items of 16 rows, odd row counts, fewer and more
    # modes than nlon / 2 + 1)
    for nlon, nmodes, nrows in ((64, 33, 37), (30, 12, 5), (25, 13, 8), (16, 12, 3), (1440, 720, 48), (1440, 721, 37), (1440, 100, 1),
                                (720, 361, 16), (720, 400, 21), (512, 257, 50), (512, 96, 15)):
        x = rng.standard_normal((nrows, nlon)).astype(np.float32)
        xd = torch.from_numpy(x).cuda()
        out = torch.empty((nrows, nmodes), dtype=torch.complex64, device="cuda")
        rc = lib.shtb200_rfft_modes(ctypes.c_void_p(xd.data_ptr()), ctypes.c_void_p(out.data_ptr()), nrows, nlon, nmodes, 2 * np.pi, None)
        assert rc == 0
        torch.cuda.synchronize()
        assert err(out.cpu().numpy(), 2 * np.pi * orc.rfft_modes(x.astype(np.float64), nmodes)) <= TOL
        c = (rng.standard_normal((nrows, nmodes)) + 1j * rng.standard_normal((nrows, nmodes))).astype(np.complex64)
        cd = torch.from_numpy(c).cuda()
        y = torch.empty((nrows, nlon), dtype=torch.float32, device="cuda")
        rc = lib.shtb200_irfft_modes(ctypes.c_void_p(cd.data_ptr()), ctypes.c_void_p(y.data_ptr()), nrows, nlon, nmodes, None)
        assert rc == 0
        torch.cuda.synchronize()
        assert err(y.cpu().numpy(), orc.irfft_modes(c.astype(np.complex128), nlon)) <= TOL

    # rows that are not 16-byte aligned take the general kernels
    nlon, nmodes, nrows = 720, 300, 9
    x = rng.standard_normal((nrows * nlon + 1,)).astype(np.float32)
    xd = torch.from_numpy(x).cuda()[1:].view(nrows, nlon)
    out = torch.empty((nrows, nmodes), dtype=torch.complex64, device="cuda")
    assert lib.shtb200_rfft_modes(ctypes.c_void_p(xd.data_ptr()), ctypes.c_void_p(out.data_ptr()), nrows, nlon, nmodes, 1.0, None) == 0
    torch.cuda.synchronize()
    assert err(out.cpu().numpy(), orc.rfft_modes(x[1:].reshape(nrows, nlon).astype(np.float64), nmodes)) <= TOL
    yd = torch.empty((nrows * nlon + 1,), dtype=torch.float32, device="cuda")[1:].view(nrows, nlon)
    assert lib.shtb200_irfft_modes(ctypes.c_void_p(out.data_ptr()), ctypes.c_void_p(yd.data_ptr()), nrows, nlon, nmodes, None) == 0
    torch.cuda.synchronize()
    assert err(yd.cpu().numpy(), orc.irfft_modes(out.cpu().numpy().astype(np.complex128), nlon)) <= TOL

    nlat, nlon, grid = 33, 64, "equiangular"
    w, p, L, M = oracle_tables(nlat, nlon, 20, 20, grid)
    nf, m0, mloc = 3, 5, 9
    Xc = (rng.standard_normal((nf, nlat, mloc)) + 1j * rng.standard_normal((nf, nlat, mloc))).astype(np.complex64)
    plan = make_plan(_lib.SHT, nlat, nlon, L, M, w, engine)
    xd = torch.from_numpy(Xc).cuda()
    out = torch.full((nf, L, mloc), float("nan"), dtype=torch.complex64, device="cuda")
    ws = torch.empty(plan.legendre_workspace_bytes(nf, mloc), dtype=torch.uint8, device="cuda")
    plan.legendre(xd, out, nf, m0, mloc, ws, 0)
    torch.cuda.synchronize()
    ref = np.einsum("nkm,mlk->nlm", Xc.astype(np.complex128), w[m0:m0 + mloc])
    assert err(out.cpu().numpy(), ref) <= TOL
    plan = make_plan(_lib.ISHT, nlat, nlon, L, M, p, engine)
    c = (rng.standard_normal((nf, L, mloc)) + 1j * rng.standard_normal((nf, L, mloc))).astype(np.complex64)
    cd = torch.from_numpy(c).cuda()
    out = torch.full((nf, nlat, mloc), float("nan"), dtype=torch.complex64, device="cuda")
    ws = torch.empty(plan.legendre_workspace_bytes(nf, mloc), dtype=torch.uint8, device="cuda")
    plan.legendre(cd, out, nf, m0, mloc, ws, 0)
    torch.cuda.synchronize()
    ref = np.einsum("nlm,mkl->nkm", c.astype(np.complex128), p[m0:m0 + mloc])
    assert err(out.cpu().numpy(), ref) <= TOL

    # plans that hold a window of orders only (what one azimuth rank of the distributed transforms keeps), called on the
    # whole window and on a part of it
    from torch_harmonics_b200 import _lib as L_

    for kind, table, rows_in, rows_out, spec in ((L_.SHT, w, nlat, L, "nkm,mlk->nlm"), (L_.ISHT, p, L, nlat, "nlm,mkl->nkm")):
        t32 = torch.from_numpy(np.ascontiguousarray(table[m0:m0 + mloc])).to(device="cuda", dtype=torch.float32)
        wplan = L_.Plan(kind, nlat, nlon, L, M, t32, engine=engine, orders=(m0, mloc))
        for a, n in ((m0, mloc), (m0 + 2, 4)):
            xin = (rng.standard_normal((nf, rows_in, n)) + 1j * rng.standard_normal((nf, rows_in, n))).astype(np.complex64)
            out = torch.full((nf, rows_out, n), float("nan"), dtype=torch.complex64, device="cuda")
            ws = torch.empty(wplan.legendre_workspace_bytes(nf, n), dtype=torch.uint8, device="cuda")
            wplan.legendre(torch.from_numpy(xin).cuda(), out, nf, a, n, ws, 0)
            torch.cuda.synchronize()
            assert err(out.cpu().numpy(), np.einsum(spec, xin.astype(np.complex128), table[a:a + n])) <= TOL
        with pytest.raises(L_.ShtLibraryError, match="inside the plan"):
            wplan.legendre(torch.from_numpy(xin).cuda(), out, nf, m0 - 1, 2, ws, 0)
        assert wplan.workspace_bytes(nf) == 0  # whole-transform calls refuse a window plan


@pytest.mark.parametrize("engine", ENGINES)
def test_host_buffer_call_pipelined_chunks(engine):
    """More fields than one chunk: the host-buffer entry point uploads, transforms and downloads chunks of fields on
    three streams; the result must equal the device-resident call (same kernels on the same numbers), in both directions."""
    import torch

    from torch_harmonics_b200 import _lib

    nlat, nlon, nf = 33, 64, 21  # chunk schedule 2, 6, 8, 3, 2
    w, p, L, M = oracle_tables(nlat, nlon, 17, 17, "equiangular")
    rng = np.random.default_rng(11)
    x = rng.standard_normal((nf, nlat, nlon)).astype(np.float32)
    pf, pi = make_plan(_lib.SHT, nlat, nlon, L, M, w, engine), make_plan(_lib.ISHT, nlat, nlon, L, M, p, engine)
    xh = torch.from_numpy(x).pin_memory()
    ch = torch.empty((nf, L, M), dtype=torch.complex64).pin_memory()
    pf.execute_host(xh, ch, nf)
    cd = run_plan(pf, x, (nf, L, M), torch.complex64, nf)
    assert err(ch.numpy(), cd) <= 1e-7
    assert err(cd, orc.sht_forward(x.astype(np.float64), w)) <= TOL
    yh = torch.empty((nf, nlat, nlon), dtype=torch.float32).pin_memory()
    pi.execute_host(ch, yh, nf)
    yd = run_plan(pi, cd, (nf, nlat, nlon), torch.float32, nf)
    assert err(yh.numpy(), yd) <= 1e-7


@pytest.mark.parametrize("engine", ENGINES)
def test_tall_grid_polar_extent_is_clamped(engine):
    """A grid with more than 16 blocks of 32 folded latitudes (nlat = 1601) whose high orders vanish over more than
    half of them: the first live block of those orders lies beyond what the FFT kernels' 4-bit field can carry, so
    plan creation must clamp the extent (skip fewer rows), not fail, and the results must be those of the full
    contraction.  The table is synthetic (the C ABI takes any table with the Legendre tables' equatorial parity):
    W[m, l, k] = sin(theta_k)^(24 m) * cos(theta_k)^((l + m) % 2) * (1 + l / lmax), zero for l < m."""
    import torch

    from torch_harmonics_b200 import _lib

    nlat, nlon, L, M = 1601, 192, 96, 96
    theta = (np.arange(nlat) + 0.5) * np.pi / nlat  # symmetric about the equator
    s, c = np.sin(theta), np.cos(theta)
    m = np.arange(M)[:, None, None]
    l = np.arange(L)[None, :, None]
    w = (s[None, None, :] ** (24.0 * m)) * np.where((l + m) % 2 == 1, c[None, None, :], 1.0) * (1.0 + l / L) * (l >= m)
    # the extent the plan derives: first row reaching 1e-14 of the row's maximum, in 32-row blocks
    first = np.array([np.argmax(np.abs(w[mm, L - 1]) >= 1e-14 * np.abs(w[mm, L - 1]).max()) for mm in range(M)])
    assert first.max() // 32 > 15, "the case must reach beyond block 15 to exercise the clamp"
    rng = np.random.default_rng(77)
    x = rng.standard_normal((3, nlat, nlon)).astype(np.float32)
    plan = make_plan(_lib.SHT, nlat, nlon, L, M, w, engine)
    cf = run_plan(plan, x, (3, L, M), torch.complex64, 3)
    assert err(cf, orc.sht_forward(x.astype(np.float64), w)) <= TOL
    # synthesis with the transposed table
    pt = np.ascontiguousarray(w.transpose(0, 2, 1))
    cin = (rng.standard_normal((3, L, M)) + 1j * rng.standard_normal((3, L, M))).astype(np.complex64)
    plan = make_plan(_lib.ISHT, nlat, nlon, L, M, pt, engine)
    y = run_plan(plan, cin, (3, nlat, nlon), torch.float32, 3)
    assert err(y, orc.sht_inverse(cin.astype(np.complex128), pt, nlon)) <= TOL
