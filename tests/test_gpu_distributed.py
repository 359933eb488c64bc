"""GPU tests of the distributed SHT modules: with no process groups registered they must equal the serial modules
(this exercises the stage entry points on one GPU); with two or four GPUs the tiles computed under NCCL must equal
the matching tiles of the serial result, forward and input gradient (torch-harmonics
tests/test_distributed_sht.py:109-349)."""

import os
import socket
import warnings

import numpy as np
import pytest

from oracle import sht_oracle as orc
from tests.helpers import TOL, err

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("nlat,nlon,lmax,grid", [(33, 64, 17, "equiangular"), (32, 64, None, "legendre-gauss"), (91, 180, 90, "equiangular")])
def test_single_rank_equals_serial(nlat, nlon, lmax, grid):
    import torch

    import torch_harmonics_b200 as th
    import torch_harmonics_b200.distributed as thd

    with warnings.catch_warnings():
        warnings.simplefilter("ignore")
        sht, isht = th.RealSHT(nlat, nlon, lmax=lmax, grid=grid).cuda(), th.InverseRealSHT(nlat, nlon, lmax=lmax, grid=grid).cuda()
        dsht, disht = thd.DistributedRealSHT(nlat, nlon, lmax=lmax, grid=grid).cuda(), thd.DistributedInverseRealSHT(nlat, nlon, lmax=lmax, grid=grid).cuda()
        w, L, M = orc.sht_weights(nlat, nlon, lmax=lmax, grid=grid)
    assert dsht.nlat_local == nlat and dsht.mmax_local == sht.mmax and dsht.weights.shape == sht.weights.shape
    x = torch.randn(2, 3, nlat, nlon, device="cuda", generator=torch.Generator(device="cuda").manual_seed(0))
    xa = x.clone().requires_grad_(True)
    xb = x.clone().requires_grad_(True)
    ca, cb = sht(xa), dsht(xb)
    assert err(cb.detach().cpu().numpy(), orc.sht_forward(x.cpu().numpy().astype(np.float64), w)) <= TOL
    assert err(cb.detach().cpu().numpy(), ca.detach().cpu().numpy()) <= 2e-6
    g = torch.randn_like(ca)
    ca.backward(g)
    cb.backward(g)
    assert err(xb.grad.cpu().numpy(), xa.grad.cpu().numpy()) <= 2e-6
    c1 = ca.detach().clone().requires_grad_(True)
    c2 = ca.detach().clone().requires_grad_(True)
    ya, yb = isht(c1), disht(c2)
    assert err(yb.detach().cpu().numpy(), ya.detach().cpu().numpy()) <= 2e-6
    gy = torch.randn_like(ya)
    ya.backward(gy)
    yb.backward(gy)
    assert err(c2.grad.cpu().numpy(), c1.grad.cpu().numpy()) <= 2e-6


@pytest.mark.parametrize("nlat,nlon,lmax,grid", [(33, 64, 17, "equiangular"), (32, 64, None, "legendre-gauss")])
def test_single_rank_vector_equals_serial(nlat, nlon, lmax, grid):
    import torch

    import torch_harmonics_b200 as th
    import torch_harmonics_b200.distributed as thd

    with warnings.catch_warnings():
        warnings.simplefilter("ignore")
        vsht, ivsht = th.RealVectorSHT(nlat, nlon, lmax=lmax, grid=grid).cuda(), th.InverseRealVectorSHT(nlat, nlon, lmax=lmax, grid=grid).cuda()
        dv, div = thd.DistributedRealVectorSHT(nlat, nlon, lmax=lmax, grid=grid).cuda(), thd.DistributedInverseRealVectorSHT(nlat, nlon, lmax=lmax, grid=grid).cuda()
        w, L, M = orc.vsht_weights(nlat, nlon, lmax=lmax, grid=grid)
    assert dv.weights.shape == vsht.weights.shape and div.dpct.shape == ivsht.dpct.shape
    x = torch.randn(2, 3, 2, nlat, nlon, device="cuda", generator=torch.Generator(device="cuda").manual_seed(1))
    xa = x.clone().requires_grad_(True)
    xb = x.clone().requires_grad_(True)
    ca, cb = vsht(xa), dv(xb)
    assert err(cb.detach().cpu().numpy(), orc.vsht_forward(x.cpu().numpy().astype(np.float64), w)) <= TOL
    assert err(cb.detach().cpu().numpy(), ca.detach().cpu().numpy()) <= 2e-6
    g = torch.randn_like(ca)
    ca.backward(g)
    cb.backward(g)
    assert err(xb.grad.cpu().numpy(), xa.grad.cpu().numpy()) <= 2e-6
    c1 = ca.detach().clone().requires_grad_(True)
    c2 = ca.detach().clone().requires_grad_(True)
    ya, yb = ivsht(c1), div(c2)
    assert err(yb.detach().cpu().numpy(), ya.detach().cpu().numpy()) <= 2e-6
    gy = torch.randn_like(ya)
    ya.backward(gy)
    yb.backward(gy)
    assert err(c2.grad.cpu().numpy(), c1.grad.cpu().numpy()) <= 2e-6


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _tile(t, dim_h, dim_w, gh, gw, rh, rw):
    import torch_harmonics_b200.distributed as thd

    return thd.split_tensor_along_dim(thd.split_tensor_along_dim(t, dim_h, gh)[rh], dim_w, gw)[rw].contiguous()


# (nlat, nlon, lmax, leading dims, grid): the reference's parameter list (tests/test_distributed_sht.py:109-163) -- even and odd
# nlat (uneven 17 + 16 latitude split), default / reduced / enlarged lmax (8, 9, 64, 65), batches smaller than the process
# groups (the leading dimension is zero-padded up to the group size), plus a 91 x 180 grid and a lobatto grid
SCALAR_CASES = [
    (32, 64, None, (32, 8), "equiangular"),
    (32, 64, None, (32, 8), "legendre-gauss"),
    (33, 64, None, (1, 10), "equiangular"),
    (33, 64, None, (1, 10), "legendre-gauss"),
    (8, 16, None, (1, 10), "equiangular"),
    (32, 64, None, (1, 1), "equiangular"),
    (32, 64, None, (1, 1), "legendre-gauss"),
    (32, 64, None, (1, 2), "equiangular"),
    (24, 512, 20, (2, 3), "legendre-gauss"),  # a longitude count the copy-free azimuth path serves
    (32, 64, 8, (4, 8), "equiangular"),
    (33, 64, 9, (1, 10), "equiangular"),
    (33, 64, 8, (1, 10), "legendre-gauss"),
    (32, 64, 64, (4, 8), "legendre-gauss"),
    (33, 64, 65, (1, 10), "equiangular"),
    (33, 64, 9, (3,), "lobatto"),
    (91, 180, 90, (4, 2), "equiangular"),
]
VECTOR_CASES = [
    (32, 64, None, (4, 8), "equiangular"),
    (33, 64, None, (1, 10), "legendre-gauss"),
    (32, 64, None, (1, 1), "equiangular"),
    (32, 64, None, (1, 2), "equiangular"),
    (24, 512, 20, (2, 3), "equiangular"),
    (33, 64, 9, (1, 10), "equiangular"),
    (32, 64, 64, (2, 3), "legendre-gauss"),
    (33, 64, 65, (1, 10), "equiangular"),
]


def _init_grid(rank, world, port, gh, gw):
    import torch
    import torch.distributed as dist

    import torch_harmonics_b200.distributed as thd

    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    rh, rw = rank // gw, rank % gw
    az = pol = None
    for r in range(gh):  # rows share a polar index -> azimuth groups
        grp = dist.new_group([r * gw + c for c in range(gw)])
        if r == rh:
            az = grp
    for c in range(gw):  # columns share an azimuth index -> polar groups
        grp = dist.new_group([r * gw + c for r in range(gh)])
        if c == rw:
            pol = grp
    thd.init(pol if gh > 1 else None, az if gw > 1 else None)
    return rh, rw


def _finish(ok, msgs):
    import torch
    import torch.distributed as dist

    import torch_harmonics_b200.distributed as thd

    flag = torch.tensor([0 if ok else 1], device="cuda")
    dist.all_reduce(flag)
    thd.finalize()
    dist.destroy_process_group()
    assert int(flag.item()) == 0, "; ".join(msgs) or "another rank failed"


def _dist_worker(rank, world, port, gh, gw):
    """Every rank computes the serial transform of the whole (seeded) batch and the distributed transform of its tile;
    the tile must equal the serial result's tile AND the float64 oracle's, forward and input gradient, both directions."""
    import torch

    import torch_harmonics_b200 as th
    import torch_harmonics_b200.distributed as thd

    rh, rw = _init_grid(rank, world, port, gh, gw)
    ok = True
    msgs = []

    def tile(t):
        return _tile(t, -2, -1, gh, gw, rh, rw)

    for vector, cases in ((False, SCALAR_CASES), (True, VECTOR_CASES)):
        for nlat, nlon, lmax, lead, grid in cases:
            with warnings.catch_warnings():
                warnings.simplefilter("ignore")
                if vector:
                    sht, isht = th.RealVectorSHT(nlat, nlon, lmax=lmax, grid=grid).cuda(), th.InverseRealVectorSHT(nlat, nlon, lmax=lmax, grid=grid).cuda()
                    dsht, disht = thd.DistributedRealVectorSHT(nlat, nlon, lmax=lmax, grid=grid).cuda(), thd.DistributedInverseRealVectorSHT(nlat, nlon, lmax=lmax, grid=grid).cuda()
                    w, _, _ = orc.vsht_weights(nlat, nlon, lmax=lmax, grid=grid)
                    p, _, _ = orc.ivsht_dpct(nlat, nlon, lmax=lmax, grid=grid)
                else:
                    sht, isht = th.RealSHT(nlat, nlon, lmax=lmax, grid=grid).cuda(), th.InverseRealSHT(nlat, nlon, lmax=lmax, grid=grid).cuda()
                    dsht, disht = thd.DistributedRealSHT(nlat, nlon, lmax=lmax, grid=grid).cuda(), thd.DistributedInverseRealSHT(nlat, nlon, lmax=lmax, grid=grid).cuda()
                    w, _, _ = orc.sht_weights(nlat, nlon, lmax=lmax, grid=grid)
                    p, _, _ = orc.isht_pct(nlat, nlon, lmax=lmax, grid=grid)
            if min(sht.lmax, nlat) < gh or min(sht.mmax, nlon) < gw:
                continue  # a chunk would be empty on this grid (the reference refuses such splits too)
            comp = (2,) if vector else ()
            gen = torch.Generator(device="cuda").manual_seed(333)  # same numbers on every rank
            x = torch.randn(*lead, *comp, nlat, nlon, device="cuda", generator=gen)
            gc = torch.randn(*lead, *comp, sht.lmax, sht.mmax, device="cuda", generator=gen, dtype=torch.complex64)
            xs = x.clone().requires_grad_(True)
            cs = sht(xs)
            cs.backward(gc)
            xl = tile(x).requires_grad_(True)
            cl = dsht(xl)
            cl.backward(tile(gc))
            xn = x.double().cpu().numpy()
            c64 = torch.from_numpy(orc.vsht_forward(xn, w) if vector else orc.sht_forward(xn, w)).cuda()
            e0 = float((cl.detach() - tile(c64)).abs().max()) / float(c64.abs().max())
            e1 = float((cl.detach() - tile(cs.detach())).abs().max()) / float(cs.detach().abs().max())
            e2 = float((xl.grad - tile(xs.grad)).abs().max()) / float(xs.grad.abs().max())
            c0 = cs.detach().clone().requires_grad_(True)
            ys = isht(c0)
            gy = torch.randn(ys.shape, device="cuda", generator=gen)
            ys.backward(gy)
            cloc = tile(cs.detach()).requires_grad_(True)
            yl = disht(cloc)
            yl.backward(tile(gy))
            cn = cs.detach().to(torch.complex128).cpu().numpy()
            y64 = torch.from_numpy(orc.vsht_inverse(cn, p, nlon) if vector else orc.sht_inverse(cn, p, nlon)).cuda()
            e3 = float((yl.detach() - tile(ys.detach())).abs().max()) / float(ys.detach().abs().max())
            e4 = float((cloc.grad - tile(c0.grad)).abs().max()) / float(c0.grad.abs().max())
            e5 = float((yl.detach() - tile(y64)).abs().max()) / float(y64.abs().max())
            if max(e1, e2, e3, e4) > 3e-6 or max(e0, e5) > TOL:
                ok = False
                msgs.append(f"rank {rank} {'vector ' if vector else ''}{nlat}x{nlon} lmax={lmax} {lead} {grid}: oracle {e0:.2e} {e5:.2e} serial {e1:.2e} {e2:.2e} {e3:.2e} {e4:.2e}")
    # inference path: without a gradient to record, large batches are cut into chunks whose all-to-alls and kernels overlap on
    # streams of their own (forced here by dropping the size limit; grids with one distributed axis only).  The chunks pair
    # the latitude rows differently inside the row FFT (two real rows share one complex transform), so the results agree to
    # rounding, not bit for bit.
    with warnings.catch_warnings():
        warnings.simplefilter("ignore")
        dsht, disht = thd.DistributedRealSHT(33, 64, lmax=17).cuda(), thd.DistributedInverseRealSHT(33, 64, lmax=17).cuda()
    x = torch.randn(37, 3, 33, 64, device="cuda", generator=torch.Generator(device="cuda").manual_seed(5))
    xl = tile(x)
    with torch.no_grad():
        dsht.pipeline_chunks = disht.pipeline_chunks = 0
        c_plain = dsht(xl)
        y_plain = disht(c_plain)
        dsht.pipeline_chunks, dsht.pipeline_min_bytes = 4, 0
        disht.pipeline_chunks, disht.pipeline_min_bytes = 3, 0
        # (stage lists whose exchanges are fused with the kernels around them are not pipelined: keep the transposes separate)
        dsht.fuse_polar_legendre = disht.fuse_polar_legendre = dsht.fuse_azimuth_fft = disht.fuse_azimuth_fft = False
        c_pipe = dsht(xl)
        y_pipe = disht(c_pipe)
    torch.cuda.synchronize()
    if min(gh, gw) == 1 and not (dsht.last_pipelined and disht.last_pipelined):
        ok = False
        msgs.append(f"rank {rank}: the pipelined path did not run")
    # (a rank's tile of coefficients can lie entirely above the diagonal l >= m and be all zeros)
    ep = max(float((c_pipe - c_plain).abs().max() / c_plain.abs().max().clamp_min(1e-30)),
             float((y_pipe - y_plain).abs().max() / y_plain.abs().max().clamp_min(1e-30)))
    if not ep <= 2e-6:
        ok = False
        msgs.append(f"rank {rank}: pipelined inference path differs from the plain path by {ep:.2e}")
    # exchange - kernel - exchange on piece-major buffers (no copies in between; azimuth: row FFT, polar: contraction) against
    # the separate steps: same kernels, same arithmetic, so the results are equal bit for bit - scalar and vector
    from torch_harmonics_b200 import _lib

    assert gw == 1 or _lib.rows_pieces_supported(512, 20, gw, gw)
    gen = torch.Generator(device="cuda").manual_seed(6)
    for vector in (False, True):
        with warnings.catch_warnings():
            warnings.simplefilter("ignore")
            if vector:
                dsht, disht = thd.DistributedRealVectorSHT(24, 512, lmax=20).cuda(), thd.DistributedInverseRealVectorSHT(24, 512, lmax=20).cuda()
            else:
                dsht, disht = thd.DistributedRealSHT(24, 512, lmax=20).cuda(), thd.DistributedInverseRealSHT(24, 512, lmax=20).cuda()
        xl = tile(torch.randn((5, 2, 24, 512) if vector else (5, 24, 512), device="cuda", generator=gen))
        with torch.no_grad():
            c_f = dsht(xl)
            y_f = disht(c_f)
            dsht.fuse_azimuth_fft = disht.fuse_azimuth_fft = dsht.fuse_polar_legendre = disht.fuse_polar_legendre = False
            c_s = dsht(xl)
            y_s = disht(c_s)
        if not (torch.equal(c_f, c_s) and torch.equal(y_f, y_s)):
            ok = False
            msgs.append(f"rank {rank}: copy-free {'vector ' if vector else ''}path differs from the separate steps")
    if rank == 0:
        print(f"distributed parity {gh}x{gw}: {len(SCALAR_CASES)} scalar + {len(VECTOR_CASES)} vector cases + pipelined path, ok={ok}", flush=True)
    _finish(ok, msgs)


def _cfg5_worker(rank, world, port, gh, gw):
    """721 x 1440, lmax = mmax = 720 (uneven 361 + 360 latitude split on a polar group of two): two fields with N(0,1)
    coefficients of seed 4, fewer than the ranks of the larger group.  Tiles against rows of the reference's own float64
    results (committed fixture) and against the serial transform."""
    import torch

    import torch_harmonics_b200 as th
    import torch_harmonics_b200.distributed as thd

    rh, rw = _init_grid(rank, world, port, gh, gw)
    g = np.load(os.path.join(os.path.dirname(__file__), "golden", "cfg5_equiangular_721x1440.npz"))
    a = torch.from_numpy(orc.random_coeffs((2,), 720, 720, seed=4, power=0.0)).to(torch.complex64).cuda()
    with warnings.catch_warnings():
        warnings.simplefilter("ignore")
        with torch.device("cuda"):
            sht, isht = th.RealSHT(721, 1440, lmax=720, mmax=720), th.InverseRealSHT(721, 1440, lmax=720, mmax=720)
            dsht, disht = thd.DistributedRealSHT(721, 1440, lmax=720, mmax=720), thd.DistributedInverseRealSHT(721, 1440, lmax=720, mmax=720)
    x = isht(a)
    cs = sht(x)
    rs = isht(cs)
    cl = dsht(_tile(x, -2, -1, gh, gw, rh, rw))
    rl = disht(cl)
    cmax, fmax = float(g["coeff_absmax"]), float(g["field_absmax"])
    e_ser_c = float((cl - _tile(cs, -2, -1, gh, gw, rh, rw)).abs().max()) / cmax
    e_ser_r = float((rl - _tile(rs, -2, -1, gh, gw, rh, rw)).abs().max()) / fmax
    l0, m0 = sum(dsht.l_shapes[:rh]), sum(dsht.m_shapes[:rw])
    k0, j0 = sum(dsht.lat_shapes[:rh]), sum(dsht.lon_shapes[:rw])
    e_ref_c = e_ref_r = 0.0
    for i, l in enumerate(g["rows_l"]):
        if l0 <= l < l0 + dsht.lmax_local:
            ref = torch.from_numpy(g["coeff_rows"][:, i, m0:m0 + dsht.mmax_local]).cuda()
            e_ref_c = max(e_ref_c, float((cl[:, l - l0, :].to(torch.complex128) - ref).abs().max()) / cmax)
    for i, k in enumerate(g["rows_k"]):
        if k0 <= k < k0 + dsht.nlat_local:
            ref = torch.from_numpy(g["roundtrip_rows"][:, i, j0:j0 + dsht.nlon_local]).cuda()
            e_ref_r = max(e_ref_r, float((rl[:, k - k0, :].double() - ref).abs().max()) / fmax)
    ok = max(e_ser_c, e_ser_r) <= 3e-6 and e_ref_c <= TOL and e_ref_r <= 2 * TOL
    msgs = [] if ok else [f"rank {rank}: serial {e_ser_c:.2e} {e_ser_r:.2e} reference rows {e_ref_c:.2e} {e_ref_r:.2e}"]
    print(f"cfg5 tile {gh}x{gw} rank {rank} ({dsht.nlat_local}x{dsht.nlon_local} -> {dsht.lmax_local}x{dsht.mmax_local}): vs serial {e_ser_c:.2e} {e_ser_r:.2e}, vs reference rows {e_ref_c:.2e} {e_ref_r:.2e}", flush=True)
    _finish(ok, msgs)


# (in_shape, out_shape, batch, channels, groups, grid_in, grid_out, bias): torch-harmonics
# tests/test_distributed_spectral_convolution.py:92-121 (incl. fewer channels than the polar group), plus a grouped case
SPECTRAL_CONV_CASES = [
    ((64, 128), (64, 128), 4, 8, 1, "equiangular", "equiangular", False),
    ((65, 128), (65, 128), 4, 8, 1, "equiangular", "equiangular", False),
    ((64, 128), (32, 64), 4, 8, 1, "equiangular", "equiangular", False),
    ((65, 128), (33, 64), 4, 8, 1, "equiangular", "equiangular", False),
    ((33, 64), (65, 128), 4, 8, 1, "equiangular", "equiangular", False),
    ((64, 128), (64, 128), 4, 8, 1, "equiangular", "legendre-gauss", False),
    ((64, 128), (64, 128), 1, 1, 1, "equiangular", "equiangular", False),
    ((64, 128), (64, 128), 1, 2, 1, "equiangular", "legendre-gauss", False),
    ((64, 128), (64, 128), 4, 8, 1, "equiangular", "equiangular", True),
    ((65, 128), (33, 64), 4, 8, 1, "equiangular", "equiangular", True),
    ((33, 64), (65, 128), 4, 8, 1, "equiangular", "equiangular", True),
    ((65, 128), (65, 128), 4, 8, 1, "equiangular", "legendre-gauss", True),
    ((64, 128), (64, 128), 1, 2, 1, "equiangular", "equiangular", True),
    ((64, 128), (32, 64), 2, 8, 2, "legendre-gauss", "equiangular", True),
]


def _spectral_conv_worker(rank, world, port, gh, gw):
    """DistributedSpectralConvS2 and DistributedQuadratureS2 against the serial modules with the same (seeded) parameters:
    output tile, input-gradient tile, and the weight / bias gradients (a rank's weight gradient covers its own orders only,
    so it is summed over the azimuth group before the comparison, as training code has to)."""
    import torch
    import torch.distributed as dist

    import torch_harmonics_b200 as th
    import torch_harmonics_b200.distributed as thd

    rh, rw = _init_grid(rank, world, port, gh, gw)
    ok, msgs = True, []

    def rel(a, b):
        return float((a - b).abs().max()) / max(float(b.abs().max()), 1e-30)

    for in_shape, out_shape, B, C, G, grid_in, grid_out, bias in SPECTRAL_CONV_CASES:
        torch.manual_seed(333)  # same parameters and data on every rank
        with warnings.catch_warnings():
            warnings.simplefilter("ignore")
            serial = th.SpectralConvS2(in_shape, out_shape, C, C, num_groups=G, grid_in=grid_in, grid_out=grid_out, bias=bias).cuda()
            if serial.lmax < gh or serial.mmax < gw:
                continue
            local = thd.DistributedSpectralConvS2(in_shape, out_shape, C, C, num_groups=G, grid_in=grid_in, grid_out=grid_out, bias=bias).cuda()
        l0, m0 = sum(local.l_shapes[:rh]), sum(local.m_shapes[:rw])
        with torch.no_grad():
            local.weight.copy_(serial.weight[..., l0:l0 + local.lmax_local])
            if bias:
                serial.spectral_bias.copy_(torch.randn(serial.spectral_bias.shape, dtype=torch.complex64, device="cuda"))
                local.spectral_bias.copy_(serial.spectral_bias[..., l0:l0 + local.lmax_local, m0:m0 + local.mmax_local])
        x = torch.randn(B, C, *in_shape, device="cuda")
        xs = x.clone().requires_grad_(True)
        ys = serial(xs)
        gy = torch.randn_like(ys)
        ys.backward(gy)
        xl = _tile(x, -2, -1, gh, gw, rh, rw).clone().requires_grad_(True)
        yl = local(xl)
        yl.backward(_tile(gy, -2, -1, gh, gw, rh, rw).contiguous())
        errs = {"out": rel(yl.detach(), _tile(ys.detach(), -2, -1, gh, gw, rh, rw)), "gx": rel(xl.grad, _tile(xs.grad, -2, -1, gh, gw, rh, rw))}
        gw_loc = torch.view_as_real(local.weight.grad.contiguous()).clone()
        if gw > 1:
            dist.all_reduce(gw_loc, group=thd.azimuth_group())
        errs["gweight"] = rel(torch.view_as_complex(gw_loc), serial.weight.grad[..., l0:l0 + local.lmax_local])
        if bias:
            errs["gbias"] = rel(local.spectral_bias.grad, serial.spectral_bias.grad[..., l0:l0 + local.lmax_local, m0:m0 + local.mmax_local])
            q_s = th.QuadratureS2(in_shape, grid=grid_in, normalize=True).cuda()(x)
            q_l = thd.DistributedQuadratureS2(in_shape, grid=grid_in, normalize=True).cuda()(xl.detach())
            errs["quadrature"] = float((q_l - q_s).abs().max()) / max(float(q_s.abs().max()), 1e-30)
        if max(errs.values()) > TOL:
            ok = False
            msgs.append(f"rank {rank} {in_shape}->{out_shape} B={B} C={C} G={G} {grid_in}/{grid_out} bias={bias}: " + " ".join(f"{k} {v:.2e}" for k, v in errs.items()))
    if rank == 0:
        print(f"distributed spectral convolution / quadrature {gh}x{gw}: {len(SPECTRAL_CONV_CASES)} cases, ok={ok}", flush=True)
    _finish(ok, msgs)


GRIDS = [(1, 2), (2, 1), (2, 2), (2, 4), (4, 2)]


@pytest.mark.parametrize("gh,gw", GRIDS)
def test_multi_gpu_equals_serial(gh, gw):
    import torch
    import torch.multiprocessing as mp

    if torch.cuda.device_count() < gh * gw:
        pytest.skip(f"needs {gh * gw} GPUs")
    mp.spawn(_dist_worker, args=(gh * gw, _free_port(), gh, gw), nprocs=gh * gw, join=True)


@pytest.mark.parametrize("gh,gw", [(1, 2), (2, 1), (2, 2), (2, 4)])
def test_multi_gpu_spectral_conv_equals_serial(gh, gw):
    import torch
    import torch.multiprocessing as mp

    if torch.cuda.device_count() < gh * gw:
        pytest.skip(f"needs {gh * gw} GPUs")
    mp.spawn(_spectral_conv_worker, args=(gh * gw, _free_port(), gh, gw), nprocs=gh * gw, join=True)


@pytest.mark.parametrize("gh,gw", [(1, 2), (2, 2), (2, 4)])
def test_multi_gpu_cfg5_reference_rows(gh, gw):
    import torch
    import torch.multiprocessing as mp

    if torch.cuda.device_count() < gh * gw:
        pytest.skip(f"needs {gh * gw} GPUs")
    mp.spawn(_cfg5_worker, args=(gh * gw, _free_port(), gh, gw), nprocs=gh * gw, join=True)
