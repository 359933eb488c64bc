"""Full-size GPU checks at 721 x 1440, lmax = mmax = 720 (the benchmark shape): outputs against rows of the
reference's own float64 results (tests/golden/cfg3_*.npz, cfg4_*.npz) and size-independent properties
(linearity, batch independence, agreement of the two contraction engines).  Tolerance: max-normalised error <= 1e-5."""

import os
import warnings

import numpy as np
import pytest

from oracle import sht_oracle as orc
from tests.helpers import TOL

pytestmark = pytest.mark.gpu
GOLD = os.path.join(os.path.dirname(__file__), "golden")


def _scalar_modules():
    import torch

    import torch_harmonics_b200 as th

    with warnings.catch_warnings():
        warnings.simplefilter("ignore")
        with torch.device("cuda"):
            sht = th.RealSHT(721, 1440, lmax=720, mmax=720, grid="equiangular", norm="ortho")
            isht = th.InverseRealSHT(721, 1440, lmax=720, mmax=720, grid="equiangular", norm="ortho")
    return sht, isht


def test_cfg3_rows_against_reference():
    import torch

    g = np.load(os.path.join(GOLD, "cfg3_equiangular_721x1440.npz"))
    a = orc.random_coeffs((2,), 720, 720, seed=2, offset=25.0, zero_l0=True, mode="grf")
    sht, isht = _scalar_modules()
    at = torch.from_numpy(a).to(torch.complex64).cuda()
    x = isht(at)
    xs = x.cpu().numpy()
    fmax, cmax = float(g["field_absmax"]), float(g["coeff_absmax"])
    assert np.max(np.abs(xs[:, g["rows_k"]] - g["field_rows"])) / fmax <= TOL
    # analysis of the reference's field itself is not stored in full; analyse ours (equal to it within TOL)
    c = sht(x)
    cs = c.cpu().numpy()
    assert np.max(np.abs(cs[:, g["rows_l"]] - g["coeff_rows"])) / cmax <= 2 * TOL
    ll, mm = np.meshgrid(np.arange(720), np.arange(720), indexing="ij")
    assert np.all(cs[:, ll < mm] == 0)
    rt = isht(c).cpu().numpy()
    assert np.max(np.abs(rt[:, g["rows_k"]] - g["roundtrip_rows"])) / fmax <= 2 * TOL
    # the reference's own round trip departs from the input by about 1.3e-3 at this shape; ours must do the same
    ours = orc.max_normalised_error(rt, xs)
    assert abs(ours - float(g["ref_roundtrip_vs_input"])) < 2e-4


def test_cfg3_properties_and_engines_agree():
    import torch

    sht, isht = _scalar_modules()
    gen = torch.Generator(device="cuda").manual_seed(5)
    x = torch.randn(3, 721, 1440, device="cuda", generator=gen)
    y = torch.randn(3, 721, 1440, device="cuda", generator=gen)
    cx, cy = sht(x), sht(y)
    cz = sht(1.5 * x - 0.25 * y)
    ref = 1.5 * cx - 0.25 * cy
    assert float((cz - ref).abs().max() / ref.abs().max()) <= TOL
    # one field alone gives the same numbers as inside a batch
    c1 = sht(x[1:2])
    assert float((c1 - cx[1:2]).abs().max() / cx.abs().max()) <= 1e-6
    # the two contraction engines agree far inside the tolerance
    sht.engine = "simt"
    sht._op.clear()
    cs = sht(x)
    assert float((cs - cx).abs().max() / cx.abs().max()) <= 3e-6
    # synthesis is linear too
    sht.engine = "auto"
    sht._op.clear()
    f1, f2 = isht(cx), isht(cy)
    f3 = isht(2.0 * cx + cy)
    assert float((f3 - (2.0 * f1 + f2)).abs().max() / f3.abs().max()) <= TOL


def test_cfg4_vector_rows_against_reference():
    import torch

    import torch_harmonics_b200 as th

    g = np.load(os.path.join(GOLD, "cfg4_vector_721x1440.npz"))
    a = orc.random_coeffs((1, 2), 720, 720, seed=3, power=1.5, offset=1.0, zero_l0=True)
    with warnings.catch_warnings():
        warnings.simplefilter("ignore")
        with torch.device("cuda"):
            ivs = th.InverseRealVectorSHT(721, 1440, lmax=720, mmax=720, grid="equiangular")
            vs = th.RealVectorSHT(721, 1440, lmax=720, mmax=720, grid="equiangular")
    v = ivs(torch.from_numpy(a).to(torch.complex64).cuda())
    vn = v.cpu().numpy()
    assert np.max(np.abs(vn[:, :, g["rows_k"]] - g["field_rows"])) / float(g["field_absmax"]) <= TOL
    c = vs(v).cpu().numpy()
    assert np.max(np.abs(c[:, :, g["rows_l"]] - g["coeff_rows"])) / float(g["coeff_absmax"]) <= 2 * TOL
