"""Shared helpers of the GPU parity tests: oracle tables -> C-ABI plans, error measure."""

import warnings

import numpy as np

from oracle import sht_oracle as orc

TOL = 1e-5  # max-normalised error bound on coefficients / fields (float32 path vs float64 oracle)


def err(a, b):
    return orc.max_normalised_error(a, b)


def oracle_tables(nlat, nlon, lmax, mmax, grid, norm="ortho", csphase=True):
    with warnings.catch_warnings():
        warnings.simplefilter("ignore")
        w, L, M = orc.sht_weights(nlat, nlon, lmax, mmax, grid, norm, csphase)
        p, _, _ = orc.isht_pct(nlat, nlon, lmax, mmax, grid, norm, csphase)
    return w, p, L, M


def make_plan(kind, nlat, nlon, L, M, table64, engine="simt"):
    import torch

    from torch_harmonics_b200 import _lib

    t = torch.from_numpy(np.ascontiguousarray(table64)).to(device="cuda", dtype=torch.float32).contiguous()
    return _lib.Plan(kind, nlat, nlon, L, M, t, engine=engine)


def run_plan(plan, x_np, out_shape, out_dtype, nfields):
    """Device-buffer call through the C ABI."""
    import torch

    x = torch.from_numpy(np.ascontiguousarray(x_np)).cuda()
    out = torch.full(out_shape, float("nan"), dtype=out_dtype, device="cuda")
    ws = torch.empty(max(plan.workspace_bytes(nfields), 1), dtype=torch.uint8, device="cuda")
    plan.execute(x, out, nfields, ws, torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    plan.device_status()  # raises if a kernel gave up on a bounded wait
    return out.cpu().numpy()
