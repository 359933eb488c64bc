"""Generate the golden fixtures in this directory from the reference implementation itself.

Run once on a machine that has a checkout of the reference (torch-harmonics); its path is a required argument
(or the environment variable ``TORCH_HARMONICS_REFERENCE``):

    python tests/golden/make_golden.py --reference /path/to/torch-harmonics [--skip-large] [--only NAME ...]

The reference package's ``__init__`` imports compiled extensions that are not built there, so the
SHT submodules (pure torch) are imported through synthetic package objects.  Inputs come from
``oracle.sht_oracle.random_coeffs`` / numpy PCG64 so that the tests can regenerate them anywhere;
only the reference's OUTPUTS (float64 path) are stored.
"""

import argparse
import importlib
import os
import sys
import types
import warnings

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)
from oracle import sht_oracle as orc  # noqa: E402


def import_reference(path):
    for name, sub in (("torch_harmonics", "torch_harmonics"), ("torch_harmonics.distributed", "torch_harmonics/distributed")):
        mod = types.ModuleType(name)
        mod.__path__ = [os.path.join(path, sub)]
        sys.modules[name] = mod
    sht = importlib.import_module("torch_harmonics.sht")
    # names the reference's own modules import from the package root
    for name in ("RealSHT", "InverseRealSHT", "RealVectorSHT", "InverseRealVectorSHT"):
        setattr(sys.modules["torch_harmonics"], name, getattr(sht, name))
    return sht


def t64(a):
    return torch.from_numpy(np.ascontiguousarray(a))


def tables(ref):
    out = {}
    for grid in ("equiangular", "legendre-gauss", "lobatto"):
        for norm in ("ortho", "four-pi", "schmidt"):
            for cs in (True, False):
                key = f"{grid}|{norm}|{int(cs)}"
                nlat, nlon, lmax = 12, 24, 9
                out[key + "|w"] = ref.RealSHT(nlat, nlon, lmax=lmax, grid=grid, norm=norm, csphase=cs).weights.numpy()
                out[key + "|p"] = ref.InverseRealSHT(nlat, nlon, lmax=lmax, grid=grid, norm=norm, csphase=cs).pct.numpy()
                out[key + "|vw"] = ref.RealVectorSHT(nlat, nlon, lmax=lmax, grid=grid, norm=norm, csphase=cs).weights.numpy()
                out[key + "|vp"] = ref.InverseRealVectorSHT(nlat, nlon, lmax=lmax, grid=grid, norm=norm, csphase=cs).dpct.numpy()
    # default truncation + odd nlat
    for grid in ("equiangular", "legendre-gauss", "lobatto"):
        m = ref.RealSHT(33, 64, grid=grid)
        out[f"default|{grid}|w"] = m.weights.numpy()
        out[f"default|{grid}|lm"] = np.array([m.lmax, m.mmax])
    np.savez_compressed(os.path.join(HERE, "tables.npz"), **out)


def cfg1(ref):
    """Equiangular 64x128, lmax=64, mmax=65 asked -> (64, 64); iid N(0,1) input, seed 0."""
    rng = np.random.default_rng(0)
    x = rng.standard_normal((4, 8, 64, 128))
    sht = ref.RealSHT(64, 128, lmax=64, mmax=65, grid="equiangular", norm="ortho")
    isht = ref.InverseRealSHT(64, 128, lmax=64, mmax=65, grid="equiangular", norm="ortho")
    c = sht(t64(x))
    rt = isht(c)
    c32 = sht.float()(t64(x).float())
    np.savez_compressed(
        os.path.join(HERE, "cfg1_equiangular_64x128.npz"),
        lm=np.array([sht.lmax, sht.mmax]),
        coeffs=c.numpy()[:2, :2],
        roundtrip=rt.numpy()[:2, :2],
        coeffs_fp32_err=np.array(orc.max_normalised_error(c32.numpy(), c.numpy())),
    )


def cfg2(ref):
    """Legendre-Gauss 256x512, lmax=256, mmax=257 asked -> (256, 256); band-limited, seed 1."""
    a = orc.random_coeffs((2,), 256, 256, seed=1, power=1.0, offset=1.0)
    sht = ref.RealSHT(256, 512, lmax=256, mmax=257, grid="legendre-gauss", norm="ortho")
    isht = ref.InverseRealSHT(256, 512, lmax=256, mmax=257, grid="legendre-gauss", norm="ortho")
    x = isht(t64(a))
    c = sht(x)
    np.savez_compressed(
        os.path.join(HERE, "cfg2_legendre_gauss_256x512.npz"),
        lm=np.array([sht.lmax, sht.mmax]),
        field=x.numpy()[:1, ::4, :],
        coeffs=c.numpy()[:1, ::4, :],
    )


ROWS_K = np.array([0, 1, 2, 179, 180, 359, 360, 361, 540, 718, 719, 720])
ROWS_L = np.array([0, 1, 2, 3, 100, 101, 359, 360, 361, 600, 718, 719])


def cfg3(ref):
    """Equiangular 721x1440, lmax=mmax=720; spectrum (l(l+1)+25)^-2, seed 2; two fields."""
    a = orc.random_coeffs((2,), 720, 720, seed=2, offset=25.0, zero_l0=True, mode="grf")
    sht = ref.RealSHT(721, 1440, lmax=720, mmax=720, grid="equiangular", norm="ortho")
    isht = ref.InverseRealSHT(721, 1440, lmax=720, mmax=720, grid="equiangular", norm="ortho")
    x = isht(t64(a))
    c = sht(x)
    rt = isht(c)
    x32 = x.float()
    c32 = sht.float()(x32)
    rt32 = isht.float()(c32)
    np.savez_compressed(
        os.path.join(HERE, "cfg3_equiangular_721x1440.npz"),
        rows_k=ROWS_K,
        rows_l=ROWS_L,
        field_rows=x.numpy()[:, ROWS_K, :],
        coeff_rows=c.numpy()[:, ROWS_L, :],
        roundtrip_rows=rt.numpy()[:, ROWS_K, :],
        field_absmax=np.array(float(x.abs().max())),
        coeff_absmax=np.array(float(c.abs().max())),
        ref_fp32_coeff_err=np.array(orc.max_normalised_error(c32.numpy(), c.numpy())),
        ref_fp32_roundtrip_err=np.array(orc.max_normalised_error(rt32.numpy(), rt.numpy())),
        ref_roundtrip_vs_input=np.array(orc.max_normalised_error(rt.numpy(), x.numpy())),
        weights_rows=sht.weights.numpy()[[0, 1, 2, 359, 719]][:, ROWS_L][:, :, ::40],
    )


def cfg5(ref):
    """Equiangular 721x1440, lmax=mmax=720; N(0,1) coefficients (band-limited fields), seed 4; two fields of the
    global batch.  The spatially distributed transforms must reproduce the serial reference on every rank's tile
    (tests/test_distributed_sht.py:109-163), so the serial reference's rows are the fixture."""
    a = orc.random_coeffs((2,), 720, 720, seed=4, power=0.0)
    sht = ref.RealSHT(721, 1440, lmax=720, mmax=720, grid="equiangular", norm="ortho")
    isht = ref.InverseRealSHT(721, 1440, lmax=720, mmax=720, grid="equiangular", norm="ortho")
    x = isht(t64(a))
    c = sht(x)
    rt = isht(c)
    np.savez_compressed(
        os.path.join(HERE, "cfg5_equiangular_721x1440.npz"),
        rows_k=ROWS_K,
        rows_l=ROWS_L,
        field_rows=x.numpy()[:, ROWS_K, :],
        coeff_rows=c.numpy()[:, ROWS_L, :],
        roundtrip_rows=rt.numpy()[:, ROWS_K, :],
        field_absmax=np.array(float(x.abs().max())),
        coeff_absmax=np.array(float(c.abs().max())),
    )


SPECTRAL_CONV_CASES = [
    # tag, in_shape, out_shape, in_channels, out_channels, groups, grid_in, grid_out, bias
    ("plain", (17, 32), (17, 32), 6, 4, 1, "equiangular", "equiangular", False),
    ("groups_resample", (17, 32), (12, 24), 6, 4, 2, "equiangular", "legendre-gauss", False),
    ("bias", (16, 32), (16, 32), 4, 4, 2, "legendre-gauss", "legendre-gauss", True),
]


def spectral_conv_inputs(tag, in_shape, cin, cout, groups, lmax, out_shape):
    """Seeded inputs of one spectral-convolution case (the tests regenerate them with the same calls)."""
    rng = np.random.default_rng(sum(map(ord, tag)))
    w = 0.3 * (rng.standard_normal((groups, cin // groups, cout // groups, lmax)) + 1j * rng.standard_normal((groups, cin // groups, cout // groups, lmax)))
    b = np.tril(0.1 * (rng.standard_normal((1, cin, lmax, lmax)) + 1j * rng.standard_normal((1, cin, lmax, lmax))))
    b[..., 0] = b[..., 0].real
    x = rng.standard_normal((2, cin) + tuple(in_shape))
    gy = rng.standard_normal((2, cout) + tuple(out_shape))
    return w.astype(np.complex64), b.astype(np.complex64), x.astype(np.float32), gy.astype(np.float32)


def spectral_conv(ref):
    """SpectralConvS2 (outputs, input / weight / bias gradients), QuadratureS2 weights and GaussianRandomFieldS2 samples of
    the reference.  The reference wraps its channel contraction in torch.compile; it is run eagerly here."""
    import torch._dynamo

    torch._dynamo.config.disable = True
    sc = importlib.import_module("torch_harmonics.spectral_convolution")
    rf = importlib.import_module("torch_harmonics.random_fields")
    quad = importlib.import_module("torch_harmonics.quadrature")
    out = {}
    for tag, ishape, oshape, cin, cout, groups, gin, gout, bias in SPECTRAL_CONV_CASES:
        layer = sc.SpectralConvS2(ishape, oshape, cin, cout, num_groups=groups, grid_in=gin, grid_out=gout, bias=bias)
        w, b, x, gy = spectral_conv_inputs(tag, ishape, cin, cout, groups, layer.lmax, oshape)
        layer.weight.data = torch.from_numpy(w)
        if bias:
            layer.spectral_bias.data = torch.from_numpy(b)
        xt = torch.from_numpy(x).requires_grad_(True)
        y = layer(xt)
        y.backward(torch.from_numpy(gy))
        out[f"{tag}|lmax"] = np.array(layer.lmax)
        out[f"{tag}|y"] = y.detach().numpy()
        out[f"{tag}|gx"] = xt.grad.numpy()
        out[f"{tag}|gw"] = layer.weight.grad.numpy()
        if bias:
            out[f"{tag}|gb"] = layer.spectral_bias.grad.numpy()
    for grid in ("equiangular", "legendre-gauss", "lobatto", "equiangular-trapezoidal"):
        for normalize in (False, True):
            q = quad.QuadratureS2((13, 24), grid=grid, normalize=normalize)
            out[f"quad|{grid}|{int(normalize)}"] = q.quad_weight[0, 0, :, 0].numpy()
    grf = rf.GaussianRandomFieldS2(16, alpha=2.5, tau=4.0)
    rng = np.random.default_rng(99)
    xi = (rng.standard_normal((3, grf.isht.lmax, grf.isht.mmax)) + 1j * rng.standard_normal((3, grf.isht.lmax, grf.isht.mmax))).astype(np.complex64)
    out["grf|lm"] = np.array([grf.isht.lmax, grf.isht.mmax])
    out["grf|sqrt_eig"] = grf.sqrt_eig.numpy()
    out["grf|u"] = grf(3, xi=torch.from_numpy(xi)).numpy()
    np.savez_compressed(os.path.join(HERE, "spectral_conv.npz"), **out)


def vector_small(ref):
    out = {}
    for grid, nlat, nlon in (("equiangular", 33, 64), ("legendre-gauss", 32, 64), ("lobatto", 33, 66)):
        vs = ref.RealVectorSHT(nlat, nlon, grid=grid) if grid != "equiangular" else ref.RealVectorSHT(nlat, nlon, lmax=20, grid=grid)
        ivs = ref.InverseRealVectorSHT(nlat, nlon, lmax=vs.lmax, mmax=vs.mmax, grid=grid)
        a = orc.random_coeffs((3, 2), vs.lmax, vs.mmax, seed=30, power=1.5, offset=1.0, zero_l0=True)
        v = ivs(t64(a))
        c = vs(v)
        out[f"{grid}|lm"] = np.array([vs.lmax, vs.mmax])
        out[f"{grid}|field"] = v.numpy()
        out[f"{grid}|coeffs"] = c.numpy()
    np.savez_compressed(os.path.join(HERE, "vector_small.npz"), **out)


def cfg4(ref):
    """Vector 721x1440; gradient + curl of two scalar random fields, amplitude (l+1)^-1.5, seed 3."""
    a = orc.random_coeffs((1, 2), 720, 720, seed=3, power=1.5, offset=1.0, zero_l0=True)
    ivs = ref.InverseRealVectorSHT(721, 1440, lmax=720, mmax=720, grid="equiangular")
    vs = ref.RealVectorSHT(721, 1440, lmax=720, mmax=720, grid="equiangular")
    v = ivs(t64(a))
    c = vs(v)
    np.savez_compressed(
        os.path.join(HERE, "cfg4_vector_721x1440.npz"),
        rows_k=ROWS_K,
        rows_l=ROWS_L,
        field_rows=v.numpy()[:, :, ROWS_K, :],
        coeff_rows=c.numpy()[:, :, ROWS_L, :],
        field_absmax=np.array(float(v.abs().max())),
        coeff_absmax=np.array(float(c.abs().max())),
    )


def autograd_small(ref):
    """Input gradients produced by the reference's autograd (scalar + vector, odd and even nlat)."""
    out = {}
    for tag, nlat, nlon, lmax, grid in (("eq", 17, 36, 12, "equiangular"), ("lg", 16, 30, 16, "legendre-gauss")):
        sht = ref.RealSHT(nlat, nlon, lmax=lmax, grid=grid)
        isht = ref.InverseRealSHT(nlat, nlon, lmax=lmax, grid=grid)
        rng = np.random.default_rng(40)
        x = rng.standard_normal((3, nlat, nlon))
        g = rng.standard_normal((3, sht.lmax, sht.mmax)) + 1j * rng.standard_normal((3, sht.lmax, sht.mmax))
        xt = t64(x).requires_grad_(True)
        y = sht(xt)
        y.backward(t64(g))
        out[f"{tag}|sht_gx"] = xt.grad.numpy()
        c = orc.random_coeffs((3,), sht.lmax, sht.mmax, seed=41) + 0j
        c[..., :, 0] += 0.3j  # non-zero Im at m=0: the gradient there must vanish
        gx = rng.standard_normal((3, nlat, nlon))
        ct = t64(c).requires_grad_(True)
        yy = isht(ct)
        yy.backward(t64(gx))
        out[f"{tag}|isht_gc"] = ct.grad.numpy()
        out[f"{tag}|lm"] = np.array([sht.lmax, sht.mmax])
        # vector
        vs = ref.RealVectorSHT(nlat, nlon, lmax=lmax, grid=grid)
        ivs = ref.InverseRealVectorSHT(nlat, nlon, lmax=lmax, grid=grid)
        xv = rng.standard_normal((2, 2, nlat, nlon))
        gv = rng.standard_normal((2, 2, vs.lmax, vs.mmax)) + 1j * rng.standard_normal((2, 2, vs.lmax, vs.mmax))
        xvt = t64(xv).requires_grad_(True)
        vs(xvt).backward(t64(gv))
        out[f"{tag}|vsht_gx"] = xvt.grad.numpy()
        cv = rng.standard_normal((2, 2, vs.lmax, vs.mmax)) + 1j * rng.standard_normal((2, 2, vs.lmax, vs.mmax))
        gxv = rng.standard_normal((2, 2, nlat, nlon))
        cvt = t64(cv).requires_grad_(True)
        ivs(cvt).backward(t64(gxv))
        out[f"{tag}|ivsht_gc"] = cvt.grad.numpy()
    np.savez_compressed(os.path.join(HERE, "autograd_small.npz"), **out)


def truncation_cases(ref):
    """rfft/irfft mode padding and truncation: mmax above and below nlon//2+1, odd nlon."""
    out = {}
    for tag, nlat, nlon, lmax, mmax, grid in (
        ("up", 12, 16, 12, 12, "legendre-gauss"),  # mmax 12 > nlon//2+1 = 9
        ("odd", 13, 25, 10, 10, "lobatto"),
        ("down", 16, 48, 6, 6, "equiangular"),
        ("nyq", 20, 16, 9, 9, "legendre-gauss"),  # keeps the Nyquist bin m = 8
    ):
        sht = ref.RealSHT(nlat, nlon, lmax=lmax, mmax=mmax, grid=grid)
        isht = ref.InverseRealSHT(nlat, nlon, lmax=lmax, mmax=mmax, grid=grid)
        rng = np.random.default_rng(50)
        x = rng.standard_normal((2, nlat, nlon))
        c = sht(t64(x))
        cin = rng.standard_normal((2, sht.lmax, sht.mmax)) + 1j * rng.standard_normal((2, sht.lmax, sht.mmax))
        y = isht(t64(cin))
        out[f"{tag}|lm"] = np.array([sht.lmax, sht.mmax])
        out[f"{tag}|coeffs"] = c.numpy()
        out[f"{tag}|field"] = y.numpy()
    np.savez_compressed(os.path.join(HERE, "truncation_cases.npz"), **out)


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", default=os.environ.get("TORCH_HARMONICS_REFERENCE"), required="TORCH_HARMONICS_REFERENCE" not in os.environ)
    ap.add_argument("--skip-large", action="store_true")
    ap.add_argument("--only", nargs="*", default=None, help="names of the generator functions to run (default: all)")
    args = ap.parse_args()
    warnings.simplefilter("ignore")
    torch.set_grad_enabled(True)
    ref = import_reference(args.reference)
    small = [tables, cfg1, cfg2, vector_small, autograd_small, truncation_cases, spectral_conv]
    large = [cfg3, cfg4, cfg5]
    for fn in small + ([] if args.skip_large else large):
        if args.only is None or fn.__name__ in args.only:
            fn(ref)
    print("golden fixtures written to", HERE)
