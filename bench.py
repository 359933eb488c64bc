#!/usr/bin/env python
"""Benchmark of the SHT hot path: 721x1440 (lmax = mmax = 720) forward + inverse transform of 73 fields.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

One "step" = RealSHT followed by InverseRealSHT on a batch of 73 synthetic fields (per GPU; ranks are
independent replicas, no data-path collective).  Prints ONE JSON line (rank 0).

  value          fields that went through forward AND inverse per second, inputs resident in HBM.  The K-step block
                 is repeated until at least half a second of device time has been measured; the MEDIAN block is
                 reported (max over ranks), so that the clock sampler sees the whole timed region.
  e2e            the same through the host-buffer C-ABI call, host<->device copies inside the timed region
  roofline       the slowest kernel of the step, from CUDA events recorded between the kernels
  cpu_baseline   CPU port of the reference's torch path on this box's host cores, bounded sample
  module_api     the same round trip through RealSHT.forward / InverseRealSHT.forward (allocation + dispatch included)
  incumbent_cuda the reference's op sequence (torch.fft + einsum = cuFFT + cuBLAS) on the same GPU, TF32 off and on:
                 the kernels this library replaces (1 GPU only)
  configs        fields/s and roofline fractions of the other single-GPU workloads: 256x512 legendre-gauss with 1024
                 fields, the vector transforms with 104 (u, v) pairs, 2048 fields on one GPU (1 GPU only)
  spectral_conv  SpectralConvS2 at the benchmark grid: the fused library call against the composed layer (1 GPU only)
  setup          seconds to build the modules' tables on the GPU and to pack them into plans
  spatial        N > 1 only: DistributedRealSHT / DistributedInverseRealSHT on a polar x azimuth process grid
                 (1x2, 2x2, 2x4) at 721x1440: per-rank parity against the serial transform and the reference's rows,
                 forward / inverse / round-trip fields/s, all-to-all bytes and GB/s
"""

import argparse
import datetime
import json
import os
import subprocess
import sys
import tempfile
import time
import warnings

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

NLAT, NLON, LMAX, MMAX = 721, 1440, 720, 720
METRIC = "721x1440 SHT fwd+inv fields/sec"
MIN_TIMED_S = 0.5


def peaks():
    """(HBM GB/s, dense TF32 TFLOP/s = half the measured bf16 figure, where the numbers come from)."""
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        try:
            d = json.load(open(p))
            return float(d["hbm_gbs"]), float(d["bf16_tflops"]) / 2.0, "measured"
        except Exception:
            pass
    return 6650.0, 1590.0 / 2.0, "fallback"


class ClockSampler:
    """Samples nvidia-smi clocks / throttle reasons of one GPU while the timed region runs."""

    Q = "clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap"

    def __init__(self, index):
        self.index = index
        self.proc = None
        self.path = None

    def start(self):
        try:
            fd, self.path = tempfile.mkstemp(suffix=".csv")
            os.close(fd)
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", str(self.index), f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "20"],
                stdout=open(self.path, "w"), stderr=subprocess.DEVNULL,
            )
            time.sleep(0.15)  # let the first sample land before the timed region starts
        except Exception:
            self.proc = None

    def stop(self):
        out = {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        if self.proc is None:
            return out
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        sm, reasons, mx, pw = [], set(), None, []
        try:
            for line in open(self.path):
                f = [t.strip() for t in line.split(",")]
                if len(f) < 7:
                    continue
                try:
                    sm.append(float(f[0]))
                    mx = float(f[1])
                    pw.append(float(f[2]))
                except ValueError:
                    continue
                for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[3:7]):
                    if v.lower().startswith("active"):
                        reasons.add(name)
            os.unlink(self.path)
        except Exception:
            pass
        if sm:
            sm.sort()
            out.update(sm_mhz=sm[len(sm) // 2], sm_max_mhz=mx, reasons=sorted(reasons), samples=len(sm), power_w_max=max(pw) if pw else None)
        return out


def synthetic_coeffs(nfields, seed, lmax=LMAX, mmax=MMAX, device="cpu", spectrum="grf"):
    """Coefficients of synthetic band-limited fields: lower triangular, real m = 0 column.  spectrum "grf": amplitude
    1 / (l (l + 1) + 25) with the l = 0 term zeroed (a Gaussian random field); "white": N(0, 1) coefficients."""
    g = torch.Generator(device=device).manual_seed(seed)
    re = torch.randn(nfields, lmax, mmax, generator=g, device=device)
    im = torch.randn(nfields, lmax, mmax, generator=g, device=device)
    l = torch.arange(lmax, dtype=torch.float32, device=device)
    amp = torch.ones_like(l)
    if spectrum == "grf":
        amp = 1.0 / (l * (l + 1) + 25.0)
        amp[0] = 0.0
    mask = torch.tril(torch.ones(lmax, mmax, device=device))
    c = torch.complex(re, im) * (amp[:, None] * mask)
    c[..., :, 0] = torch.complex(c[..., :, 0].real, torch.zeros_like(c[..., :, 0].real))
    return c.contiguous()


def timed_blocks(fn, steps, barrier, min_seconds=MIN_TIMED_S, max_blocks=400, agree=None):
    """Run blocks of `steps` calls of fn, each bracketed by CUDA events on the current stream, until about min_seconds
    of device time have been measured.  The number of blocks is fixed after the first one (with `agree`, a max over the
    ranks, so that every rank passes the same number of barriers).  Returns (median block seconds, number of blocks)."""

    def one():
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        barrier()
        e0.record()
        for _ in range(steps):
            fn()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / 1e3

    times = [one()]
    n = int(min(max_blocks, max(1, -(-min_seconds // max(times[0], 1e-6)))))
    if agree is not None:
        n = int(agree(n))
    for _ in range(n - 1):
        times.append(one())
    times.sort()
    return times[len(times) // 2], len(times)


def triangle(lmax, mmax):
    return sum(max(lmax - m, 0) for m in range(mmax))


def transform_bound(nf, nlat, nlon, lmax, mmax, vector=False):
    """Whole-transform roofline of one direction (seconds): input + output + triangular fp32 table at HBM speed, and
    the algorithmic flops of the Legendre contraction at the dense TF32 rate; the slower one is the bound."""
    hbm, tf32, src = peaks()
    T = triangle(lmax, mmax)
    comp = 2 if vector else 1
    t_mem = (nf * comp * (nlat * nlon * 4 + lmax * mmax * 8) + comp * 4 * nlat * T) / (hbm * 1e9)
    t_tc = nf * (32 if vector else 8) * nlat * T / (tf32 * 1e12)
    return t_mem, t_tc, src


def kernel_bytes(nf, table_fwd_bytes, table_inv_bytes, slabs):
    """Algorithmic bytes each kernel of a step must move (reads + writes), by kernel name."""
    Kh = (NLAT + 1) // 2
    T = triangle(LMAX, MMAX)
    ncols = 2 * nf
    grid = nf * NLAT * NLON * 4
    operand = 2 * MMAX * ncols * Kh * 4
    tri = T * ncols * 4
    return {
        "fft_analysis": grid + operand,
        "legendre_analysis": operand + table_fwd_bytes + slabs * ncols * 32 * 4,
        "unpack_coeffs": slabs * ncols * 32 * 4 + nf * LMAX * MMAX * 8,
        "pack_coeffs": tri + slabs * ncols * 32 * 4,
        "legendre_synthesis": slabs * ncols * 32 * 4 + table_inv_bytes + operand,
        "fft_synthesis": operand + grid,
    }


# DRAM traffic (dram__bytes_read.sum + dram__bytes_write.sum) of one launch, copied from the committed ncu summaries:
# (bytes, fields in the captured launch, True if the traffic grows in proportion to the number of fields, capture).
# The FFT and transpose kernels only stream per-field data; the Legendre kernels also read the packed table once per
# launch, so their figure holds for the captured field count only.
NCU_TRAFFIC = {  # kernel: (dram bytes read + written per launch, fields of the capture, scales with the field count, summary under profiles/, commit captured at)
    "fft_analysis": (133.01e6 + 58.22e6, 32, True, "fft_twopass_kernels_32fields", "03be9b6"),
    "fft_synthesis": (98.70e6 + 83.60e6, 32, True, "fft_twopass_kernels_32fields", "03be9b6"),
    "pack_coeffs": (67.86e6 + 26.99e6, 32, True, "coeff_slab_transpose_32fields", "03be9b6"),
    "unpack_coeffs": (72.29e6 + 77.22e6, 32, True, "coeff_slab_transpose_32fields", "03be9b6"),
    "legendre_analysis": (611.81e6 + 135.42e6, 73, False, "legendre_tc_kernel_73fields", "03be9b6"),
    "legendre_synthesis": (561.63e6 + 188.40e6, 73, False, "legendre_tc_kernel_73fields", "03be9b6"),
}


def measured_traffic(kernel, nf):
    b, n, scales = NCU_TRAFFIC[kernel][:3]
    if scales:
        return b * nf / n
    return b if nf == n else None


def build_scalar(dev, nlat, nlon, lmax, mmax, grid, engine):
    import torch_harmonics_b200 as th

    with warnings.catch_warnings():
        warnings.simplefilter("ignore")
        with torch.device(dev):
            sht = th.RealSHT(nlat, nlon, lmax=lmax, mmax=mmax, grid=grid, norm="ortho")
            isht = th.InverseRealSHT(nlat, nlon, lmax=lmax, mmax=mmax, grid=grid, norm="ortho")
    sht.engine = isht.engine = engine
    return sht, isht


def local_barrier():
    torch.cuda.synchronize()


def config_record(dev, name, engine, barrier):
    """One of the other single-GPU workloads: device-resident forward / inverse / round trip through the C ABI."""
    import torch_harmonics_b200 as th

    if name == "cfg2":
        nlat, nlon, lmax, mmax, grid, nf, vector, spectrum = 256, 512, 256, 256, "legendre-gauss", 1024, False, "pow"
    elif name == "cfg4":
        nlat, nlon, lmax, mmax, grid, nf, vector, spectrum = NLAT, NLON, LMAX, MMAX, "equiangular", 104, True, "pow15"
    else:  # cfg5 on one GPU
        nlat, nlon, lmax, mmax, grid, nf, vector, spectrum = NLAT, NLON, LMAX, MMAX, "equiangular", 2048, False, "white"
    with warnings.catch_warnings():
        warnings.simplefilter("ignore")
        with torch.device(dev):
            if vector:
                fwd = th.RealVectorSHT(nlat, nlon, lmax=lmax, mmax=mmax, grid=grid)
                inv = th.InverseRealVectorSHT(nlat, nlon, lmax=lmax, mmax=mmax, grid=grid)
            else:
                fwd = th.RealSHT(nlat, nlon, lmax=lmax, mmax=mmax, grid=grid)
                inv = th.InverseRealSHT(nlat, nlon, lmax=lmax, mmax=mmax, grid=grid)
    fwd.engine = inv.engine = engine
    p_f, p_i = fwd._op.plan(dev, False), inv._op.plan(dev, False)
    for mod, nm in ((fwd, "weights"), (inv, "dpct" if vector else "pct")):
        setattr(mod, nm, torch.empty(0))
    torch.cuda.empty_cache()
    comp = 2 if vector else 1
    # synthetic band-limited input, generated on the device in chunks
    c = torch.empty(nf * comp, lmax, mmax, dtype=torch.complex64, device=dev)
    l = torch.arange(lmax, dtype=torch.float32, device=dev)
    amp = {"pow": 1.0 / (l + 1.0), "pow15": (l + 1.0) ** -1.5, "white": torch.ones_like(l)}[spectrum]
    if spectrum == "pow15":
        amp[0] = 0.0
    g = torch.Generator(device=dev).manual_seed({"cfg2": 1, "cfg4": 3}.get(name, 4))
    mask = torch.tril(torch.ones(lmax, mmax, device=dev)) * amp[:, None]
    for i0 in range(0, nf * comp, 128):
        i1 = min(i0 + 128, nf * comp)
        blk = torch.complex(torch.randn(i1 - i0, lmax, mmax, generator=g, device=dev), torch.randn(i1 - i0, lmax, mmax, generator=g, device=dev)) * mask
        blk[..., 0] = torch.complex(blk[..., 0].real, torch.zeros_like(blk[..., 0].real))
        c[i0:i1] = blk
    stream = torch.cuda.current_stream().cuda_stream
    ws = torch.empty(max(p_f.workspace_bytes(nf), p_i.workspace_bytes(nf)), dtype=torch.uint8, device=dev)
    x = torch.empty(nf * comp, nlat, nlon, device=dev)
    c2 = torch.empty_like(c)
    x2 = torch.empty_like(x)
    p_i.execute(c, x, nf, ws, stream)

    def fwd_fn():
        p_f.execute(x, c2, nf, ws, stream)

    def inv_fn():
        p_i.execute(c2, x2, nf, ws, stream)

    def step():
        fwd_fn()
        inv_fn()

    for _ in range(3):
        step()
    torch.cuda.synchronize()
    p_f.device_status()
    p_i.device_status()
    k = 5 if nf * nlat > 200000 else 20
    t_step, nb = timed_blocks(step, k, barrier, 0.25)
    t_fwd, _ = timed_blocks(fwd_fn, k, barrier, 0.15)
    t_inv, _ = timed_blocks(inv_fn, k, barrier, 0.15)
    p_f.set_profiling(True)
    p_i.set_profiling(True)
    kt = {}
    for _ in range(3):
        fwd_fn()
        for n, t in zip(["fft_analysis", "legendre_analysis", "unpack_coeffs"], p_f.last_kernel_times()):
            kt[n] = kt.get(n, 0.0) + t / 3
        inv_fn()
        for n, t in zip(["pack_coeffs", "legendre_synthesis", "fft_synthesis"], p_i.last_kernel_times()):
            kt[n] = kt.get(n, 0.0) + t / 3
    p_f.set_profiling(False)
    p_i.set_profiling(False)
    t_mem, t_tc, src = transform_bound(nf, nlat, nlon, lmax, mmax, vector)
    bound = max(t_mem, t_tc)
    rec = {
        "workload": f"{grid} {nlat}x{nlon}, lmax={lmax}, mmax={mmax}, {nf} {'(u,v) pairs' if vector else 'fields'}" + (" (vector transforms)" if vector else ""),
        "fields_per_s": nf * k / t_step, "fwd_fields_per_s": nf * k / t_fwd, "inv_fields_per_s": nf * k / t_inv,
        "ms_per_step": 1e3 * t_step / k, "fwd_ms": 1e3 * t_fwd / k, "inv_ms": 1e3 * t_inv / k,
        "transform_roofline": {
            "t_mem_ms_per_direction": 1e3 * t_mem, "t_tc_ms_per_direction": 1e3 * t_tc, "bound": "hbm" if t_mem >= t_tc else "tensor",
            "fwd_frac": bound / (t_fwd / k), "inv_frac": bound / (t_inv / k), "roundtrip_frac": 2 * bound / (t_step / k), "peak_source": src,
        },
        "kernel_ms": kt, "launches_per_step": p_f.last_launch_count + p_i.last_launch_count,
    }
    del p_f, p_i, fwd, inv, c, c2, x, x2, ws
    torch.cuda.empty_cache()
    return rec


def spectral_conv_record(dev, engine, barrier):
    """SpectralConvS2 at the benchmark grid (73 -> 73 channels, default truncation lmax = 361): the single fused library call
    against the same layer composed of the transform modules and a torch einsum, as the reference composes it."""
    import torch_harmonics_b200 as th

    C = 73
    with warnings.catch_warnings():
        warnings.simplefilter("ignore")
        with torch.device(dev):
            layer = th.SpectralConvS2((NLAT, NLON), (NLAT, NLON), C, C)
    layer.sht.engine = layer.isht.engine = engine
    x = torch.randn(1, C, NLAT, NLON, device=dev, generator=torch.Generator(device=dev).manual_seed(5))

    def composed():
        c = layer.sht(x).reshape(1, 1, C, layer.lmax, layer.mmax)
        return layer.isht(torch.einsum("bgixy,giox->bgoxy", c, layer.weight).reshape(1, C, layer.lmax, layer.mmax).contiguous())

    with torch.no_grad():
        y, yc = layer(x), composed()
        diff = float((y - yc).abs().max() / yc.abs().max())
        t_f, _ = timed_blocks(lambda: layer(x), 10, barrier, 0.2)
        t_c, _ = timed_blocks(composed, 10, barrier, 0.2)
    rec = {
        "workload": f"SpectralConvS2 {NLAT}x{NLON} -> {NLAT}x{NLON}, {C} -> {C} channels, 1 group, lmax = mmax = {layer.lmax}, batch 1, no bias",
        "fused_ms": 1e3 * t_f / 10, "composed_ms": 1e3 * t_c / 10, "fused_fields_per_s": C * 10 / t_f, "composed_fields_per_s": C * 10 / t_c,
        "fused_vs_composed_diff": diff, "fused_launches": 6,
        "note": "fused = one library call, coefficients stay in the degree-slab layout (no (.., l, m) tensor, no transposes); composed = RealSHT, torch.einsum, InverseRealSHT",
    }
    del layer, x, y, yc
    torch.cuda.empty_cache()
    return rec


def incumbent_record(dev, sht, isht, x, c_ours, x2_ours, barrier):
    """The reference's per-call op sequence on CUDA tensors (torch.fft -> cuFFT, einsum -> cuBLAS) with float32 dense
    tables, timed with CUDA events like the reference's own benchmark (3 warm-up calls, then the timed ones):
    the incumbent this library replaces.  Baseline only."""
    from oracle.cpu_port import CpuShtPort

    port = CpuShtPort(NLAT, NLON, LMAX, MMAX, tables=(sht.weights.to(dev).float().contiguous(), isht.pct.to(dev).float().contiguous()))
    nf = x.shape[0]
    rec = {"sample": f"{nf} fields, forward then inverse, dense float32 tables (mmax, lmax, nlat) / (mmax, nlat, lmax); torch {torch.__version__}"}
    old = torch.backends.cuda.matmul.allow_tf32
    try:
        for tag, allow in (("tf32_off", False), ("tf32_on", True)):
            torch.backends.cuda.matmul.allow_tf32 = allow
            for _ in range(3):
                c = port.sht(x)
                y = port.isht(c)
            t_f, _ = timed_blocks(lambda: port.sht(x), 5, barrier, 0.2)
            t_i, _ = timed_blocks(lambda: port.isht(c), 5, barrier, 0.2)
            rec[tag] = {
                "fwd_ms": 1e3 * t_f / 5, "inv_ms": 1e3 * t_i / 5, "fields_per_s": nf / ((t_f + t_i) / 5),
                "coeff_diff_vs_ours": float((c - c_ours).abs().max() / c_ours.abs().max()),
                "roundtrip_diff_vs_ours": float((y - x2_ours).abs().max() / x2_ours.abs().max()),
            }
            del c, y
    finally:
        torch.backends.cuda.matmul.allow_tf32 = old
    del port
    torch.cuda.empty_cache()
    return rec


def spatial_record(dev, rank, world, engine, nfields, p_f, p_i):
    """DistributedRealSHT / DistributedInverseRealSHT on a polar x azimuth grid of `world` ranks at 721 x 1440."""
    import numpy as np
    import torch.distributed as dist

    import torch_harmonics_b200.distributed as thd
    from torch_harmonics_b200.distributed import primitives as prim

    grids = {2: (1, 2), 4: (2, 2), 8: (2, 4)}
    if world not in grids:
        return {"skipped": f"no process grid defined for {world} ranks"}
    gh, gw = grids[world]
    rh, rw = rank // gw, rank % gw
    az = pol = None
    for r in range(gh):  # ranks of one row share the polar index: an azimuth group
        grp = dist.new_group([r * gw + c for c in range(gw)])
        if r == rh:
            az = grp
    for c in range(gw):
        grp = dist.new_group([r * gw + c for r in range(gh)])
        if c == rw:
            pol = grp
    thd.init(pol if gh > 1 else None, az if gw > 1 else None)
    with warnings.catch_warnings():
        warnings.simplefilter("ignore")
        with torch.device(dev):
            dsht = thd.DistributedRealSHT(NLAT, NLON, lmax=LMAX, mmax=MMAX, grid="equiangular")
            disht = thd.DistributedInverseRealSHT(NLAT, NLON, lmax=LMAX, mmax=MMAX, grid="equiangular")
    dsht.engine = disht.engine = engine

    def tile(t):
        return thd.split_tensor_along_dim(thd.split_tensor_along_dim(t, -2, gh)[rh], -1, gw)[rw].contiguous()

    def allmax(v):
        t = torch.tensor([v], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    stream = torch.cuda.current_stream().cuda_stream
    B = 8
    C = max(nfields // B, 1)
    nf = B * C
    chunk = min(nf, 128)
    ws = torch.empty(max(p_f.workspace_bytes(chunk), p_i.workspace_bytes(chunk)), dtype=torch.uint8, device=dev)
    # the global batch (N(0,1) coefficients, seed 4) is synthesised chunk by chunk by the SERIAL plans on every rank;
    # each rank keeps its own tile of the field, of the serial coefficients and of the serial round trip
    xl = torch.empty(nf, dsht.nlat_local, dsht.nlon_local, device=dev)
    cl_ser = torch.empty(nf, dsht.lmax_local, dsht.mmax_local, dtype=torch.complex64, device=dev)
    rl_ser = torch.empty_like(xl)
    cmax = xmax = 0.0
    for i0 in range(0, nf, chunk):
        n = min(chunk, nf - i0)
        a = synthetic_coeffs(n, 4000 + i0, device=dev, spectrum="white")
        xg = torch.empty(n, NLAT, NLON, device=dev)
        cg = torch.empty(n, LMAX, MMAX, dtype=torch.complex64, device=dev)
        rg = torch.empty_like(xg)
        p_i.execute(a, xg, n, ws, stream)
        p_f.execute(xg, cg, n, ws, stream)
        p_i.execute(cg, rg, n, ws, stream)
        xl[i0:i0 + n], cl_ser[i0:i0 + n], rl_ser[i0:i0 + n] = tile(xg), tile(cg), tile(rg)
        cmax, xmax = max(cmax, float(cg.abs().max())), max(xmax, float(rg.abs().max()))
        del a, xg, cg, rg
    del ws
    torch.cuda.empty_cache()
    xl = xl.view(B, C, dsht.nlat_local, dsht.nlon_local)

    cl = dsht(xl)
    yl = disht(cl)
    torch.cuda.synchronize()
    err_fwd = allmax(float((cl.reshape(nf, *cl.shape[-2:]) - cl_ser).abs().max()) / cmax)
    err_rt = allmax(float((yl.reshape(nf, *yl.shape[-2:]) - rl_ser).abs().max()) / xmax)
    del cl_ser, rl_ser

    # two fields of the same kind against rows of the reference's own float64 results (committed fixture); the batch of
    # two is smaller than the process groups, which exercises the zero padding of the leading dimension
    err_fix_c = err_fix_rt = None
    fix = os.path.join(ROOT, "tests", "golden", "cfg5_equiangular_721x1440.npz")
    if os.path.exists(fix):
        from oracle import sht_oracle as orc  # checker only: regenerates the fixture's seeded input

        g = np.load(fix)
        a = torch.from_numpy(orc.random_coeffs((2,), LMAX, MMAX, seed=4, power=0.0)).to(torch.complex64).to(dev)
        ws2 = torch.empty(max(p_f.workspace_bytes(2), p_i.workspace_bytes(2)), dtype=torch.uint8, device=dev)
        xg = torch.empty(2, NLAT, NLON, device=dev)
        p_i.execute(a, xg, 2, ws2, stream)
        cf = dsht(tile(xg).unsqueeze(0))
        rf = disht(cf)
        torch.cuda.synchronize()
        l0, m0 = sum(dsht.l_shapes[:rh]), sum(dsht.m_shapes[:rw])
        k0, j0 = sum(dsht.lat_shapes[:rh]), sum(dsht.lon_shapes[:rw])
        ec = er = 0.0
        for i, l in enumerate(g["rows_l"]):
            if l0 <= l < l0 + dsht.lmax_local:
                ref = torch.from_numpy(g["coeff_rows"][:, i, m0:m0 + dsht.mmax_local]).to(dev)
                ec = max(ec, float((cf[0, :, l - l0, :].to(torch.complex128) - ref).abs().max()))
        for i, k in enumerate(g["rows_k"]):
            if k0 <= k < k0 + dsht.nlat_local:
                ref = torch.from_numpy(g["roundtrip_rows"][:, i, j0:j0 + dsht.nlon_local]).to(dev)
                er = max(er, float((rf[0, :, k - k0, :].double() - ref).abs().max()))
        err_fix_c = allmax(ec) / float(g["coeff_absmax"])
        err_fix_rt = allmax(er) / float(g["field_absmax"])
        del ws2, xg, cf, rf, a

    def barrier():
        torch.cuda.synchronize()
        dist.barrier()
        torch.cuda.synchronize()

    def fwd():
        return dsht(xl)

    def inv():
        return disht(cl)

    def step():
        return disht(dsht(xl))

    for _ in range(3):
        step()
    k = 3
    t_step, _ = timed_blocks(step, k, barrier, 0.3, 40, agree=allmax)
    t_fwd, _ = timed_blocks(fwd, k, barrier, 0.2, 40, agree=allmax)
    t_inv, _ = timed_blocks(inv, k, barrier, 0.2, 40, agree=allmax)
    t_step, t_fwd, t_inv = allmax(t_step), allmax(t_fwd), allmax(t_inv)
    was_pipelined = bool(dsht.last_pipelined or disht.last_pipelined)
    # all-to-all volume and time of one forward and one inverse call (unpipelined, so that the events bracket the exchanges only)
    chunks = dsht.pipeline_chunks
    dsht.pipeline_chunks = disht.pipeline_chunks = 0
    t_fwd_plain, _ = timed_blocks(fwd, k, barrier, 0.0, 1, agree=allmax)
    t_inv_plain, _ = timed_blocks(inv, k, barrier, 0.0, 1, agree=allmax)
    t_fwd_plain, t_inv_plain = allmax(t_fwd_plain), allmax(t_inv_plain)
    barrier()
    prim.exchange_log_start()
    fwd()
    log_f = prim.exchange_log_stop()
    barrier()
    prim.exchange_log_start()
    inv()
    log_i = prim.exchange_log_stop()
    dsht.pipeline_chunks = disht.pipeline_chunks = chunks

    def a2a(log):
        sent, recv, ms = sum(v[0] for v in log), sum(v[1] for v in log), sum(v[2] for v in log)
        return {"exchanges": len(log), "sent_bytes_per_rank_max": allmax(sent), "received_bytes_per_rank_max": allmax(recv), "ms_in_all_to_all_max": allmax(ms),
                "gbs_per_direction_min": -allmax(-(sent / (ms * 1e-3) / 1e9 if ms > 0 else 0.0))}

    af, ai = a2a(log_f), a2a(log_i)
    hbm, _, src = peaks()
    # per-rank bound of one direction: the rank's share of input, output and packed table at HBM speed, against the bytes
    # it must send at the nominal NVLink rate (900 GB/s per direction)
    T_loc = sum(max(LMAX - m, 0) for m in range(dsht.mmax_local))  # azimuth rank 0 holds the longest orders
    t_local = (nf * (NLAT * NLON * 4 + LMAX * MMAX * 8) / world + 4 * NLAT * T_loc) / (hbm * 1e9)
    t_link_f, t_link_i = af["sent_bytes_per_rank_max"] / 900e9, ai["sent_bytes_per_rank_max"] / 900e9
    rec = {
        "grid": f"{gh}x{gw} (polar x azimuth)", "workload": f"equiangular {NLAT}x{NLON}, lmax=mmax={LMAX}, global batch [{B}, {C}] = {nf} fields, N(0,1) coefficients (seed 4)",
        "local_tile": [dsht.nlat_local, dsht.nlon_local, dsht.lmax_local, dsht.mmax_local],
        "err_forward_vs_serial": err_fwd, "err_roundtrip_vs_serial": err_rt, "err_forward_vs_reference_rows": err_fix_c, "err_roundtrip_vs_reference_rows": err_fix_rt,
        "tolerance": 1e-5, "parity_ok": bool(max(err_fwd, err_rt, err_fix_c or 0.0, err_fix_rt or 0.0) <= 1e-5),
        "fwd_fields_per_s": nf * k / t_fwd, "inv_fields_per_s": nf * k / t_inv, "roundtrip_fields_per_s": nf * k / t_step,
        "fwd_ms": 1e3 * t_fwd / k, "inv_ms": 1e3 * t_inv / k, "roundtrip_ms": 1e3 * t_step / k,
        "fwd_ms_unpipelined": 1e3 * t_fwd_plain / k, "inv_ms_unpipelined": 1e3 * t_inv_plain / k,
        "pipelined": was_pipelined,
        "all_to_all_forward": af, "all_to_all_inverse": ai,
        "bound": {
            "t_local_hbm_ms": 1e3 * t_local, "t_nvlink_fwd_ms": 1e3 * t_link_f, "t_nvlink_inv_ms": 1e3 * t_link_i, "nvlink_gbs_per_direction": 900.0,
            "fwd_frac": max(t_local, t_link_f) / (t_fwd / k), "inv_frac": max(t_local, t_link_i) / (t_inv / k), "peak_source": src,
        },
    }
    thd.finalize()
    return rec


def run_ours(args):
    import torch.distributed as dist

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the SHT kernels have no CPU path")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        # a short collective timeout: a rank that falls out of step ends the run within minutes instead of holding the GPUs
        dist.init_process_group("nccl", device_id=dev, timeout=datetime.timedelta(seconds=240))

    if args.record:
        # one of the side records alone (the small, reproducible command the profile summaries of these workloads name);
        # prints that record, not the headline line
        if world > 1:
            raise SystemExit("--record is a single-GPU option")

        def barrier1():
            torch.cuda.synchronize()

        rec = spectral_conv_record(dev, args.engine, barrier1) if args.record == "spectral_conv" else config_record(dev, args.record, args.engine, barrier1)
        print(json.dumps({"record": args.record, **rec}), flush=True)
        return

    nf = args.nfields
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    sht, isht = build_scalar(dev, NLAT, NLON, LMAX, MMAX, "equiangular", args.engine)
    torch.cuda.synchronize()
    t1 = time.perf_counter()
    p_f = sht._op.plan(dev, False)
    p_i = isht._op.plan(dev, False)
    torch.cuda.synchronize()
    t2 = time.perf_counter()
    # construction: float64 tables of both modules built on the device (torch ops), then packed into the two plans
    setup = {"tables_s": t1 - t0, "plans_s": t2 - t1, "note": "RealSHT + InverseRealSHT constructors on the GPU, then table packing and polar-extent scan of both plans"}

    coeffs = synthetic_coeffs(nf, seed=2 + rank).to(dev)
    stream = torch.cuda.current_stream().cuda_stream
    ws = torch.empty(max(p_f.workspace_bytes(nf), p_i.workspace_bytes(nf)), dtype=torch.uint8, device=dev)
    x = torch.empty(nf, NLAT, NLON, device=dev)
    c = torch.empty(nf, LMAX, MMAX, dtype=torch.complex64, device=dev)
    x2 = torch.empty_like(x)
    p_i.execute(coeffs, x, nf, ws, stream)  # the synthetic input fields (outside any timed region)
    torch.cuda.synchronize()

    def fwd():
        p_f.execute(x, c, nf, ws, stream)

    def inv():
        p_i.execute(c, x2, nf, ws, stream)

    def step():
        fwd()
        inv()

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def maxr(v):
        if world == 1:
            return v
        t = torch.tensor([v], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    warm = max(args.warmup, 3)
    for _ in range(warm):
        step()
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    t_step, nblocks = timed_blocks(step, args.steps, barrier, agree=maxr)
    t_fwd, _ = timed_blocks(fwd, args.steps, barrier, 0.2, agree=maxr)
    t_inv, _ = timed_blocks(inv, args.steps, barrier, 0.2, agree=maxr)
    barrier()
    clocks = sampler.stop() if rank == 0 else None
    p_f.device_status()
    p_i.device_status()

    # per-kernel times from events recorded between the launches (separate pass, not the timed one)
    names_f = ["fft_analysis", "legendre_analysis", "unpack_coeffs"]
    names_i = ["pack_coeffs", "legendre_synthesis", "fft_synthesis"]
    kt = {n: 0.0 for n in names_f + names_i}
    p_f.set_profiling(True)
    p_i.set_profiling(True)
    reps = 10
    for _ in range(reps):
        fwd()
        for n, t in zip(names_f, p_f.last_kernel_times()):
            kt[n] += t / reps
        inv()
        for n, t in zip(names_i, p_i.last_kernel_times()):
            kt[n] += t / reps
    p_f.set_profiling(False)
    p_i.set_profiling(False)

    # the same round trip through the module API (output allocation and operator dispatch inside the timed region)
    def module_step():
        return isht(sht(x))

    for _ in range(3):
        module_step()
    t_mod, _ = timed_blocks(module_step, args.steps, barrier, 0.2, agree=maxr)

    # end to end through the host-buffer entry point (pinned host memory, copies inside the timed region); this rank's
    # thread runs on (and first-touches the pinned pages from) the CPUs NVML reports as local to its GPU
    host_cpus, numa = bind_near_gpu(dev)
    xh = x.cpu().pin_memory()
    ch = torch.empty(nf, LMAX, MMAX, dtype=torch.complex64).pin_memory()
    xh2 = torch.empty(nf, NLAT, NLON).pin_memory()

    def e2e_step():
        p_f.execute_host(xh, ch, nf, stream)
        p_i.execute_host(ch, xh2, nf, stream)

    for _ in range(2):
        e2e_step()
    e2e_steps = max(1, min(args.steps, 10))
    t_e2e, _ = timed_blocks(e2e_step, e2e_steps, barrier, 0.0, agree=maxr)
    # what the copies alone cost on this box with all ranks copying at once: the same bytes up and down on two streams,
    # no kernels.  e2e can not be faster than this; where the two agree the host side (PCIe / host memory) is the bound.
    xd, cd = torch.empty_like(x), torch.empty_like(c)
    s_up, s_dn = torch.cuda.Stream(), torch.cuda.Stream()

    def copy_step():
        cur = torch.cuda.current_stream()
        s_up.wait_stream(cur)
        s_dn.wait_stream(cur)
        with torch.cuda.stream(s_up):
            xd.copy_(xh, non_blocking=True)
            cd.copy_(ch, non_blocking=True)
        with torch.cuda.stream(s_dn):
            ch.copy_(c, non_blocking=True)
            xh2.copy_(x2, non_blocking=True)
        cur.wait_stream(s_up)
        cur.wait_stream(s_dn)

    copy_step()
    t_copy, _ = timed_blocks(copy_step, e2e_steps, barrier, 0.0, agree=maxr)
    del xd, cd
    if host_cpus:
        os.sched_setaffinity(0, host_cpus)

    t_step, t_fwd, t_inv, t_e2e, t_mod, t_copy_max = maxr(t_step), maxr(t_fwd), maxr(t_inv), maxr(t_e2e), maxr(t_mod), maxr(t_copy)
    xb, cb = x.numel() * 4, c.numel() * 8

    extras = {}
    if world == 1 and not args.quick:
        try:
            extras["incumbent_cuda"] = incumbent_record(dev, sht, isht, x, c, x2, barrier)
        except Exception as e:  # a failing side record must not take the headline down with it
            extras["incumbent_cuda"] = {"error": repr(e)[:300]}
    # the dense float64 tables are not needed once the plans hold the packed copies
    sht.weights = torch.empty(0)
    isht.pct = torch.empty(0)
    del xh, ch, xh2
    torch.cuda.empty_cache()
    if world == 1 and not args.quick:
        cfgs = {}
        for name in ("cfg2", "cfg4", "cfg5_one_gpu"):
            try:
                cfgs[name] = config_record(dev, name, args.engine, barrier)
            except Exception as e:
                cfgs[name] = {"error": repr(e)[:300]}
                torch.cuda.empty_cache()
        extras["configs"] = cfgs
        try:
            extras["spectral_conv"] = spectral_conv_record(dev, args.engine, barrier)
        except Exception as e:
            extras["spectral_conv"] = {"error": repr(e)[:300]}
            torch.cuda.empty_cache()
    if world > 1 and not args.no_spatial:
        try:
            extras["spatial"] = spatial_record(dev, rank, world, args.engine, args.spatial_fields, p_f, p_i)
        except Exception as e:
            # every rank takes the same branch only if the failure is collective; report what this rank saw
            extras["spatial"] = {"error": repr(e)[:300]}

    if rank == 0:
        peak, _, peak_src = peaks()
        slabs = sum(-(-((LMAX - m - p + 1) // 2) // 32) for m in range(MMAX) for p in range(2) if LMAX - m - p > 0)
        kb = kernel_bytes(nf, p_f.table_bytes, p_i.table_bytes, slabs)
        dom = max(kt, key=lambda n: kt[n])
        ach = kb[dom] / (kt[dom] * 1e-3) / 1e9 if kt[dom] > 0 else 0.0
        t_mem, t_tc, _ = transform_bound(nf, NLAT, NLON, LMAX, MMAX)
        k = args.steps
        line = {
            "metric": METRIC,
            "value": nf * world * k / t_step,
            "unit": "fields/s",
            "n_gpus": world,
            "steps": k,
            "warmup": warm,
            "ms_per_step": 1e3 * t_step / k,
            "higher_is_better": True,
            "scaling": "weak",
            "vs_baseline": None,
            "dtype": "f32",
            "data": "synthetic",
            "config": {
                "workload": f"cfg3: equiangular {NLAT}x{NLON}, lmax=mmax={LMAX}, {nf} fields per GPU, RealSHT then InverseRealSHT",
                "fields_per_gpu": nf, "engine": args.engine, "sharding": "replicas (fields split across GPUs, no collective)",
                "l2": "inputs (303 MB per direction) exceed the 126 MB L2; no explicit flush",
                "arithmetic": "fp32 FFT; Legendre contraction fp32 (simt) or split-TF32 with fp32 accumulation (tcgen05)",
                "timing": f"median of {nblocks} blocks of {k} steps (blocks repeated until {MIN_TIMED_S} s of device time), CUDA events, max over ranks",
            },
            "timed_blocks": nblocks,
            "fwd_fields_per_s": nf * world * k / t_fwd,
            "inv_fields_per_s": nf * world * k / t_inv,
            "transform_roofline": {
                "t_mem_ms_per_direction": 1e3 * t_mem, "t_tc_ms_per_direction": 1e3 * t_tc, "fwd_frac": t_mem / (t_fwd / k), "inv_frac": t_mem / (t_inv / k),
                "roundtrip_frac": 2 * t_mem / (t_step / k), "peak_source": peak_src,
            },
            "kernel_ms": kt,
            "kernel_hbm_frac": {n: (kb[n] / (kt[n] * 1e-3) / 1e9 / peak if kt[n] > 0 else None) for n in kt},
            "roofline": {
                "kernel": dom, "bound": "hbm", "achieved": ach, "peak": peak, "unit": "GB/s", "frac": ach / peak,
                "traffic": measured_traffic(dom, nf), "peak_source": peak_src, "algorithmic_bytes": kb[dom],
                "traffic_source": f"ncu capture '{NCU_TRAFFIC[dom][3]}' of this kernel (kernels as of commit {NCU_TRAFFIC[dom][4]}), scaled by the field count where it is proportional",
            },
            "e2e": {
                "value": nf * world * e2e_steps / t_e2e, "unit": "fields/s",
                "h2d_bytes_per_step": xb + cb, "d2h_bytes_per_step": cb + xb, "steps": e2e_steps,
                "h2d_gbs_per_rank": (xb + cb) * e2e_steps / t_e2e / 1e9, "d2h_gbs_per_rank": (xb + cb) * e2e_steps / t_e2e / 1e9,
                "host_binding": numa,
                "copies_only": {
                    "fields_per_s": nf * world * e2e_steps / t_copy_max, "gbs_per_direction_per_rank": (xb + cb) * e2e_steps / t_copy_max / 1e9,
                    "note": "the step's host<->device copies alone (both directions at once, no kernels), all ranks at the same time: the host-side ceiling of e2e on this box",
                },
            },
            "module_api": {"value": nf * world * k / t_mod, "unit": "fields/s", "ms_per_step": 1e3 * t_mod / k,
                           "note": "RealSHT.forward then InverseRealSHT.forward on device tensors: output and workspace allocation and operator dispatch included"},
            "setup": setup,
            "gpu_launches": 6 * k * nblocks,
            "clocks": clocks,
        }
        line.update(extras)
        if world == 1 and not args.no_cpu_baseline:
            line["cpu_baseline"] = cpu_baseline(args.cpu_fields, 3)
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def bind_near_gpu(dev):
    """Restrict this process to the CPUs NVML lists as local to `dev` (a query; nothing on the GPU changes).

    Returns (the previous CPU set or None, a record for the bench line).  Pinned buffers allocated afterwards are first
    touched from those CPUs, so they land on the GPU's NUMA node when the kernel's default policy applies."""
    try:
        import pynvml

        pynvml.nvmlInit()
        idx = dev.index if dev.index is not None else torch.cuda.current_device()
        try:  # by UUID: NVML's index order need not be CUDA's
            h = pynvml.nvmlDeviceGetHandleByUUID(("GPU-" + str(torch.cuda.get_device_properties(idx).uuid)).encode())
        except Exception:
            h = pynvml.nvmlDeviceGetHandleByIndex(idx)
        words = -(-(os.cpu_count() or 1) // 64)
        mask = pynvml.nvmlDeviceGetCpuAffinity(h, max(words, 1))
        near = {64 * w + b for w, v in enumerate(mask) for b in range(64) if (int(v) >> b) & 1}
        before = os.sched_getaffinity(0)
        use = near & before
        if not use:
            return None, {"bound": False, "why": "no CPU local to the GPU is in this process's CPU set", "cpus_allowed": len(before)}
        os.sched_setaffinity(0, use)
        return before, {"bound": True, "cpus_local_to_gpu": len(near), "cpus_used": len(use), "cpus_allowed": len(before)}
    except Exception as e:  # no NVML, or affinity not permitted: run unbound and say so
        return None, {"bound": False, "why": repr(e)[:120]}


def cpu_baseline(nfields, steps, warmup=1):
    """The reference's torch CPU path (float32 tables), restated in oracle/cpu_port.py, on all host threads."""
    from oracle.cpu_port import CpuShtPort

    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    port = CpuShtPort(NLAT, NLON, LMAX, MMAX, "equiangular", "ortho")
    x = port.isht(synthetic_coeffs(nfields, seed=2))
    for _ in range(warmup):
        port.isht(port.sht(x))
    t0 = time.perf_counter()
    for _ in range(steps):
        port.isht(port.sht(x))
    dt = time.perf_counter() - t0
    return {
        "value": nfields * steps / dt, "unit": "fields/s", "cores": torch.get_num_threads(), "kind": "port",
        "sample": f"{steps} round trips (RealSHT + InverseRealSHT) of {nfields} fields of the same 721x1440 workload, float32 tables, torch CPU ops",
        "ms_per_field": 1e3 * dt / (nfields * steps),
    }


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if rank != 0:
        return
    nf = args.cpu_fields
    steps = max(1, min(args.steps, 5))
    warm = 1
    from oracle.cpu_port import CpuShtPort

    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    port = CpuShtPort(NLAT, NLON, LMAX, MMAX, "equiangular", "ortho")
    x = port.isht(synthetic_coeffs(nf, seed=2))
    for _ in range(warm):
        port.isht(port.sht(x))
    t0 = time.perf_counter()
    for _ in range(steps):
        port.isht(port.sht(x))
    dt = time.perf_counter() - t0
    val = nf * steps / dt
    sample = f"each step = RealSHT + InverseRealSHT of {nf} fields (bounded sample of the 73-field batch), float32 tables, torch CPU ops on {torch.get_num_threads()} threads"
    print(json.dumps({
        "impl": "reference", "metric": METRIC, "value": val, "unit": "fields/s", "n_gpus": world, "steps": steps, "warmup": warm,
        "ms_per_step": 1e3 * dt / steps, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": f"cfg3: equiangular {NLAT}x{NLON}, lmax=mmax={LMAX}; CPU port of the reference's torch path", "fields_per_step": nf},
        "cpu_baseline": {"value": val, "unit": "fields/s", "cores": torch.get_num_threads(), "kind": "port", "sample": sample},
        "e2e": {"value": val, "unit": "fields/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }), flush=True)


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=100)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--nfields", type=int, default=73)
    ap.add_argument("--engine", default=os.environ.get("SHTB200_ENGINE", "auto"), choices=["auto", "simt", "tcgen05"])
    ap.add_argument("--cpu-fields", type=int, default=8)
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--quick", action="store_true", help="headline, e2e and roofline only: skip the incumbent and the other workloads")
    ap.add_argument("--no-spatial", action="store_true", help="N > 1: skip the spatially distributed transforms")
    ap.add_argument("--record", default=None, choices=["cfg2", "cfg4", "cfg5_one_gpu", "spectral_conv"], help="run one side record alone and print it")
    ap.add_argument("--spatial-fields", type=int, default=2048, help="global batch of the spatially distributed run")
    a = ap.parse_args()
    if a.impl == "reference":
        run_reference(a)
    else:
        run_ours(a)
