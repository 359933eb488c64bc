#!/usr/bin/env python
"""Benchmark of the SHT hot path: 721x1440 (lmax = mmax = 720) forward + inverse transform of 73 fields.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

One "step" = RealSHT followed by InverseRealSHT on a batch of 73 synthetic fields (per GPU; ranks are
independent replicas, no data-path collective).  Prints ONE JSON line (rank 0).  `value` counts fields that
went through forward AND inverse per second with inputs resident in HBM; `e2e` is the same through the
host-buffer C-ABI call with host<->device copies inside the timed region; `roofline` describes the slowest
kernel of the step from CUDA-event timings taken between the kernels; `cpu_baseline` times the CPU port of
the reference's torch path on this box's host cores on a bounded sample.
"""

import argparse
import json
import os
import subprocess
import sys
import tempfile
import threading
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

NLAT, NLON, LMAX, MMAX = 721, 1440, 720, 720
METRIC = "721x1440 SHT fwd+inv fields/sec"


def peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        try:
            d = json.load(open(p))
            return float(d["hbm_gbs"]), "measured"
        except Exception:
            pass
    return 6650.0, "fallback"


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
        sm, reasons, mx = [], set(), None
        try:
            for line in open(self.path):
                f = [t.strip() for t in line.split(",")]
                if len(f) < 7:
                    continue
                try:
                    sm.append(float(f[0]))
                    mx = float(f[1])
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
            out.update(sm_mhz=sm[len(sm) // 2], sm_max_mhz=mx, reasons=sorted(reasons), samples=len(sm))
        return out


def synthetic_coeffs(nfields, seed):
    """Gaussian random field coefficients with spectrum (l(l+1)+25)^-2, lower triangular, real m = 0 column."""
    g = torch.Generator().manual_seed(seed)
    re = torch.randn(nfields, LMAX, MMAX, generator=g)
    im = torch.randn(nfields, LMAX, MMAX, generator=g)
    l = torch.arange(LMAX, dtype=torch.float32)
    amp = 1.0 / (l * (l + 1) + 25.0)
    amp[0] = 0.0
    mask = torch.tril(torch.ones(LMAX, MMAX))
    c = torch.complex(re, im) * (amp[:, None] * mask)
    c[..., :, 0] = torch.complex(c[..., :, 0].real, torch.zeros_like(c[..., :, 0].real))
    return c.contiguous()


def time_steps(fn, steps, stream_sync):
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    stream_sync()
    e0.record()
    for _ in range(steps):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / 1e3


def kernel_bytes(nf, table_fwd_bytes, table_inv_bytes, slabs):
    """Algorithmic bytes each kernel of a step must move (reads + writes), by kernel name."""
    Kh = (NLAT + 1) // 2
    T = sum(max(LMAX - m, 0) for m in range(MMAX))
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


# DRAM traffic (dram__bytes_read.sum + dram__bytes_write.sum) of one launch, from the ncu captures summarised under
# profiles/: (bytes, fields in the captured launch, True if the traffic grows in proportion to the number of fields).
# The FFT and transpose kernels only stream per-field data; the Legendre kernels also read the packed table once per
# launch, so their figure holds for the captured field count only.
NCU_TRAFFIC = {
    "fft_analysis": (132.96e6 + 64.42e6, 32, True),
    "fft_synthesis": (98.66e6 + 87.81e6, 32, True),
    "pack_coeffs": (67.86e6 + 26.12e6, 32, True),
    "unpack_coeffs": (72.31e6 + 78.94e6, 32, True),
    "legendre_analysis": (611.80e6 + 135.90e6, 73, False),
    "legendre_synthesis": (551.98e6 + 198.46e6, 73, False),
}


def measured_traffic(kernel, nf):
    b, n, scales = NCU_TRAFFIC[kernel]
    if scales:
        return b * nf / n
    return b if nf == n else None


def run_ours(args):
    import torch.distributed as dist

    import torch_harmonics_b200 as th

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the SHT kernels have no CPU path")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)

    nf = args.nfields
    import warnings

    with warnings.catch_warnings():
        warnings.simplefilter("ignore")
        with torch.device(dev):
            sht = th.RealSHT(NLAT, NLON, lmax=LMAX, mmax=MMAX, grid="equiangular", norm="ortho")
            isht = th.InverseRealSHT(NLAT, NLON, lmax=LMAX, mmax=MMAX, grid="equiangular", norm="ortho")
    sht.engine = isht.engine = args.engine
    p_f = sht._op.plan(dev, False)
    p_i = isht._op.plan(dev, False)
    # the dense float64 tables are not needed once the plans hold the packed copies
    sht.weights = torch.empty(0)
    isht.pct = torch.empty(0)
    torch.cuda.empty_cache()

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

    for _ in range(max(args.warmup, 3)):
        step()
    # clocks are sampled from before the timed round-trip loop until the separately timed forward / inverse loops end
    # (all three run the same kernels back to back; a single loop of 20 steps is shorter than one sampling period)
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    t_step = time_steps(step, args.steps, barrier)
    t_fwd = time_steps(fwd, args.steps, barrier)
    t_inv = time_steps(inv, args.steps, barrier)
    barrier()
    clocks = sampler.stop() if rank == 0 else None

    # per-kernel times from events recorded between the launches (separate pass, not the timed one)
    names_f = ["fft_analysis", "legendre_analysis", "unpack_coeffs"]
    names_i = ["pack_coeffs", "legendre_synthesis", "fft_synthesis"]
    kt = {n: 0.0 for n in names_f + names_i}
    p_f.set_profiling(True)
    p_i.set_profiling(True)
    reps = 5
    for _ in range(reps):
        fwd()
        for n, t in zip(names_f, p_f.last_kernel_times()):
            kt[n] += t / reps
        inv()
        for n, t in zip(names_i, p_i.last_kernel_times()):
            kt[n] += t / reps
    p_f.set_profiling(False)
    p_i.set_profiling(False)

    # end to end through the host-buffer entry point (pinned host memory, copies inside the timed region)
    xh = x.cpu().pin_memory()
    ch = torch.empty(nf, LMAX, MMAX, dtype=torch.complex64).pin_memory()
    xh2 = torch.empty(nf, NLAT, NLON).pin_memory()

    def e2e_step():
        p_f.execute_host(xh, ch, nf, stream)
        p_i.execute_host(ch, xh2, nf, stream)

    for _ in range(2):
        e2e_step()
    e2e_steps = max(1, min(args.steps, 10))
    t_e2e = time_steps(e2e_step, e2e_steps, barrier)

    def maxr(v):
        if world == 1:
            return v
        t = torch.tensor([v], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    t_step, t_fwd, t_inv, t_e2e = maxr(t_step), maxr(t_fwd), maxr(t_inv), maxr(t_e2e)

    if rank == 0:
        peak, peak_src = peaks()
        slabs = sum(-(-((LMAX - m - p + 1) // 2) // 32) for m in range(MMAX) for p in range(2) if LMAX - m - p > 0)
        kb = kernel_bytes(nf, p_f.table_bytes, p_i.table_bytes, slabs)
        dom = max(kt, key=lambda n: kt[n])
        ach = kb[dom] / (kt[dom] * 1e-3) / 1e9 if kt[dom] > 0 else 0.0
        # whole-transform roofline of one direction: input + output + triangular fp32 table, at HBM speed
        T = sum(max(LMAX - m, 0) for m in range(MMAX))
        t_mem = (nf * (NLAT * NLON * 4 + LMAX * MMAX * 8) + 4 * NLAT * T) / (peak * 1e9)
        xb, cb = x.numel() * 4, c.numel() * 8
        line = {
            "metric": METRIC,
            "value": nf * world * args.steps / t_step,
            "unit": "fields/s",
            "n_gpus": world,
            "steps": args.steps,
            "warmup": max(args.warmup, 3),
            "ms_per_step": 1e3 * t_step / args.steps,
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
            },
            "fwd_fields_per_s": nf * world * args.steps / t_fwd,
            "inv_fields_per_s": nf * world * args.steps / t_inv,
            "transform_roofline": {
                "t_mem_ms_per_direction": 1e3 * t_mem, "fwd_frac": t_mem / (t_fwd / args.steps), "inv_frac": t_mem / (t_inv / args.steps),
                "roundtrip_frac": 2 * t_mem / (t_step / args.steps), "peak_source": peak_src,
            },
            "kernel_ms": kt,
            "roofline": {
                "kernel": dom, "bound": "hbm", "achieved": ach, "peak": peak, "unit": "GB/s", "frac": ach / peak,
                "traffic": measured_traffic(dom, nf), "peak_source": peak_src, "algorithmic_bytes": kb[dom],
                "traffic_source": "ncu capture of this kernel (profiles/), scaled by the field count where it is proportional",
            },
            "e2e": {
                "value": nf * world * e2e_steps / t_e2e, "unit": "fields/s",
                "h2d_bytes_per_step": xb + cb, "d2h_bytes_per_step": cb + xb, "steps": e2e_steps,
            },
            "gpu_launches": 6 * args.steps,
            "clocks": clocks,
        }
        if world == 1 and not args.no_cpu_baseline:
            line["cpu_baseline"] = cpu_baseline(args.cpu_fields, 3)
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


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
    a = ap.parse_args()
    if a.impl == "reference":
        run_reference(a)
    else:
        run_ours(a)
