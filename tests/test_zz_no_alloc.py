"""The allocation-free entry point (``shtb200_execute_static_scratch``) against the regular one.

Who needs it: a caller that may not allocate device memory when the transform is due (inside a stream capture, in
a serving loop with a fixed memory plan, as a plug-in with a fixed budget).  The call keeps its scratch in an array
built into the library, shared by all calls.  Checked here, through the C ABI: same results as ``shtb200_execute``
on two calls in a row (the second one finds the first one's leftovers in the scratch), both directions, and a clear
refusal when the request does not fit.  This file sorts last so that a failure here cannot hide other tests.
"""

import ctypes

import numpy as np
import pytest

from tests.helpers import make_plan, oracle_tables, run_plan

pytestmark = pytest.mark.gpu


def _static_call(lib, plan, x, out, nfields):
    import torch

    return lib.shtb200_execute_static_scratch(plan.handle, ctypes.c_void_p(x.data_ptr()), ctypes.c_void_p(out.data_ptr()), nfields, ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))


def test_static_scratch_matches_regular_entry_point():
    import torch

    from torch_harmonics_b200 import _lib

    lib = _lib.load()
    lib.shtb200_execute_static_scratch.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int, ctypes.c_void_p]
    lib.shtb200_execute_static_scratch.restype = ctypes.c_int
    lib.shtb200_static_scratch_bytes.restype = ctypes.c_size_t
    cap = lib.shtb200_static_scratch_bytes()
    assert cap == 32 * 1024 * 1024

    nlat, nlon = 91, 180
    w, p, L, M = oracle_tables(nlat, nlon, 90, 90, "equiangular")
    sht = make_plan(_lib.SHT, nlat, nlon, L, M, w, "auto")
    isht = make_plan(_lib.ISHT, nlat, nlon, L, M, p, "auto")
    rng = np.random.default_rng(123)
    for nf in (7, 3):  # two calls in a row per direction; the second is smaller, so stale data lies beyond what it writes
        assert sht.workspace_bytes(nf) <= cap and isht.workspace_bytes(nf) <= cap
        x = rng.standard_normal((nf, nlat, nlon)).astype(np.float32)
        ref = run_plan(sht, x, (nf, L, M), torch.complex64, nf)
        xd = torch.from_numpy(x).cuda()
        out = torch.full((nf, L, M), float("nan"), dtype=torch.complex64, device="cuda")
        assert _static_call(lib, sht, xd, out, nf) == 0, lib.shtb200_last_error()
        torch.cuda.synchronize()
        sht.device_status()
        got = out.cpu().numpy()
        assert np.max(np.abs(got - ref)) <= 1e-6 * np.max(np.abs(ref))

        c = (rng.standard_normal((nf, L, M)) + 1j * rng.standard_normal((nf, L, M))).astype(np.complex64)
        refx = run_plan(isht, c, (nf, nlat, nlon), torch.float32, nf)
        cd = torch.from_numpy(c).cuda()
        outx = torch.full((nf, nlat, nlon), float("nan"), dtype=torch.float32, device="cuda")
        assert _static_call(lib, isht, cd, outx, nf) == 0, lib.shtb200_last_error()
        torch.cuda.synchronize()
        gotx = outx.cpu().numpy()
        assert np.max(np.abs(gotx - refx)) <= 1e-6 * np.max(np.abs(refx))

    # a request that does not fit is refused with the sizes in the message, and nothing runs
    big = 4000
    assert sht.workspace_bytes(big) > cap
    xd = torch.zeros(1, device="cuda")
    rc = lib.shtb200_execute_static_scratch(sht.handle, ctypes.c_void_p(xd.data_ptr()), ctypes.c_void_p(xd.data_ptr()), big, None)
    assert rc == -3
    msg = lib.shtb200_last_error().decode()
    assert "built-in array holds" in msg and str(cap) in msg
    # profiling (which creates events) and the allocation-free call exclude each other
    sht.set_profiling(True)
    assert lib.shtb200_execute_static_scratch(sht.handle, ctypes.c_void_p(xd.data_ptr()), ctypes.c_void_p(xd.data_ptr()), 1, None) == -1
    sht.set_profiling(False)
