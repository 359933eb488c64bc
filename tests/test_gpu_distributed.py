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


def _dist_worker(rank, world, port, gh, gw):
    import torch
    import torch.distributed as dist

    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    import torch_harmonics_b200 as th
    import torch_harmonics_b200.distributed as thd

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
    ok = True
    msgs = []
    for nlat, nlon, lmax, grid, lead in ((33, 64, 17, "equiangular", (2, 5)), (32, 64, None, "legendre-gauss", (1, 1)), (33, 64, 9, "lobatto", (3,)), (91, 180, 90, "equiangular", (4, 2))):
        with warnings.catch_warnings():
            warnings.simplefilter("ignore")
            sht, isht = th.RealSHT(nlat, nlon, lmax=lmax, grid=grid).cuda(), th.InverseRealSHT(nlat, nlon, lmax=lmax, grid=grid).cuda()
            dsht, disht = thd.DistributedRealSHT(nlat, nlon, lmax=lmax, grid=grid).cuda(), thd.DistributedInverseRealSHT(nlat, nlon, lmax=lmax, grid=grid).cuda()
        gen = torch.Generator(device="cuda").manual_seed(7)
        x = torch.randn(*lead, nlat, nlon, device="cuda", generator=gen)
        gc = torch.randn(*lead, sht.lmax, sht.mmax, device="cuda", generator=gen, dtype=torch.complex64)
        xs = x.clone().requires_grad_(True)
        cs = sht(xs)
        cs.backward(gc)
        xl = _tile(x, -2, -1, gh, gw, rh, rw).requires_grad_(True)
        cl = dsht(xl)
        cl.backward(_tile(gc, -2, -1, gh, gw, rh, rw))
        scale = float(cs.detach().abs().max())
        e1 = float((cl.detach() - _tile(cs.detach(), -2, -1, gh, gw, rh, rw)).abs().max()) / scale
        e2 = float((xl.grad - _tile(xs.grad, -2, -1, gh, gw, rh, rw)).abs().max()) / float(xs.grad.abs().max())
        c0 = cs.detach().clone().requires_grad_(True)
        ys = isht(c0)
        gy = torch.randn(ys.shape, device="cuda", generator=gen)  # same numbers on every rank
        ys.backward(gy)
        cloc = _tile(cs.detach(), -2, -1, gh, gw, rh, rw).requires_grad_(True)
        yl = disht(cloc)
        yl.backward(_tile(gy, -2, -1, gh, gw, rh, rw))
        e3 = float((yl.detach() - _tile(ys.detach(), -2, -1, gh, gw, rh, rw)).abs().max()) / float(ys.abs().max())
        e4 = float((cloc.grad - _tile(c0.grad, -2, -1, gh, gw, rh, rw)).abs().max()) / float(c0.grad.abs().max())
        if max(e1, e2, e3, e4) > 3e-6:
            ok = False
            msgs.append(f"rank {rank} {nlat}x{nlon} {grid}: {e1:.2e} {e2:.2e} {e3:.2e} {e4:.2e}")
    # vector transforms: (..., 2, lat, lon) tiles
    for nlat, nlon, lmax, grid, lead in ((33, 64, 17, "equiangular", (2, 3)), (32, 64, None, "legendre-gauss", (1,))):
        with warnings.catch_warnings():
            warnings.simplefilter("ignore")
            vsht, ivsht = th.RealVectorSHT(nlat, nlon, lmax=lmax, grid=grid).cuda(), th.InverseRealVectorSHT(nlat, nlon, lmax=lmax, grid=grid).cuda()
            dv, div = thd.DistributedRealVectorSHT(nlat, nlon, lmax=lmax, grid=grid).cuda(), thd.DistributedInverseRealVectorSHT(nlat, nlon, lmax=lmax, grid=grid).cuda()
        gen = torch.Generator(device="cuda").manual_seed(11)
        x = torch.randn(*lead, 2, nlat, nlon, device="cuda", generator=gen)
        gc = torch.randn(*lead, 2, vsht.lmax, vsht.mmax, device="cuda", generator=gen, dtype=torch.complex64)
        xs = x.clone().requires_grad_(True)
        cs = vsht(xs)
        cs.backward(gc)
        xl = _tile(x, -2, -1, gh, gw, rh, rw).requires_grad_(True)
        cl = dv(xl)
        cl.backward(_tile(gc, -2, -1, gh, gw, rh, rw))
        e1 = float((cl.detach() - _tile(cs.detach(), -2, -1, gh, gw, rh, rw)).abs().max()) / float(cs.detach().abs().max())
        e2 = float((xl.grad - _tile(xs.grad, -2, -1, gh, gw, rh, rw)).abs().max()) / float(xs.grad.abs().max())
        c0 = cs.detach().clone().requires_grad_(True)
        ys = ivsht(c0)
        gy = torch.randn(ys.shape, device="cuda", generator=gen)
        ys.backward(gy)
        cloc = _tile(cs.detach(), -2, -1, gh, gw, rh, rw).requires_grad_(True)
        yl = div(cloc)
        yl.backward(_tile(gy, -2, -1, gh, gw, rh, rw))
        e3 = float((yl.detach() - _tile(ys.detach(), -2, -1, gh, gw, rh, rw)).abs().max()) / float(ys.abs().max())
        e4 = float((cloc.grad - _tile(c0.grad, -2, -1, gh, gw, rh, rw)).abs().max()) / float(c0.grad.abs().max())
        if max(e1, e2, e3, e4) > 3e-6:
            ok = False
            msgs.append(f"rank {rank} vector {nlat}x{nlon} {grid}: {e1:.2e} {e2:.2e} {e3:.2e} {e4:.2e}")
    flag = torch.tensor([0 if ok else 1], device="cuda")
    dist.all_reduce(flag)
    thd.finalize()
    dist.destroy_process_group()
    assert int(flag.item()) == 0, "; ".join(msgs) or "another rank failed"


@pytest.mark.parametrize("gh,gw", [(1, 2), (2, 1), (2, 2)])
def test_multi_gpu_equals_serial(gh, gw):
    import torch
    import torch.multiprocessing as mp

    if torch.cuda.device_count() < gh * gw:
        pytest.skip(f"needs {gh * gw} GPUs")
    mp.spawn(_dist_worker, args=(gh * gw, _free_port(), gh, gw), nprocs=gh * gw, join=True)
