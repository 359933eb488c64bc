"""ctypes binding of ``libshtb200.so`` (the C ABI declared in ``include/shtb200.h``).

There is no CPU path: if the shared library is missing, or a plan is asked for without a CUDA
device, the calls raise.
"""

import ctypes
import os
import threading

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "lib", "libshtb200.so")

# enum shtb200_kind
SHT, ISHT, SHT_ADJOINT, ISHT_ADJOINT, VSHT, IVSHT, VSHT_ADJOINT, IVSHT_ADJOINT = range(8)
# enum shtb200_engine
ENGINE_AUTO, ENGINE_SIMT, ENGINE_TCGEN05 = range(3)
ENGINES = {"auto": ENGINE_AUTO, "simt": ENGINE_SIMT, "tcgen05": ENGINE_TCGEN05}

_lock = threading.Lock()
_lib = None


class ShtLibraryError(RuntimeError):
    pass


def load():
    """Load the library once; raise ``ShtLibraryError`` if it has not been built."""
    global _lib
    with _lock:
        if _lib is not None:
            return _lib
        if not os.path.exists(LIB_PATH):
            raise ShtLibraryError(
                f"{LIB_PATH} not found: build it with `python -m torch_harmonics_b200.build` (needs nvcc); " "there is no CPU or PyTorch fallback for the SHT kernels"
            )
        lib = ctypes.CDLL(LIB_PATH)
        vp, ci, cs, cll = ctypes.c_void_p, ctypes.c_int, ctypes.c_size_t, ctypes.c_longlong
        lib.shtb200_version.restype = ci
        lib.shtb200_last_error.restype = ctypes.c_char_p
        lib.shtb200_plan_create.argtypes = [ctypes.POINTER(vp), ci, ci, ci, ci, ci, vp, ci, ci]
        lib.shtb200_plan_create.restype = ci
        lib.shtb200_plan_create_orders.argtypes = [ctypes.POINTER(vp), ci, ci, ci, ci, ci, ci, vp, ci, ci]
        lib.shtb200_plan_create_orders.restype = ci
        lib.shtb200_plan_destroy.argtypes = [vp]
        lib.shtb200_plan_destroy.restype = ci
        lib.shtb200_workspace_bytes.argtypes = [vp, ci]
        lib.shtb200_workspace_bytes.restype = cs
        lib.shtb200_execute.argtypes = [vp, vp, vp, ci, vp, cs, vp]
        lib.shtb200_execute.restype = ci
        lib.shtb200_execute_host.argtypes = [vp, vp, vp, ci, vp]
        lib.shtb200_execute_host.restype = ci
        lib.shtb200_plan_info.argtypes = [vp] + [ctypes.POINTER(ci)] * 6
        lib.shtb200_plan_info.restype = ci
        lib.shtb200_last_launch_count.argtypes = [vp]
        lib.shtb200_last_launch_count.restype = ci
        lib.shtb200_plan_set_profiling.argtypes = [vp, ci]
        lib.shtb200_plan_set_profiling.restype = ci
        lib.shtb200_last_kernel_times.argtypes = [vp, ctypes.POINTER(ctypes.c_float), ci]
        lib.shtb200_last_kernel_times.restype = ci
        lib.shtb200_device_status.argtypes = [vp]
        lib.shtb200_device_status.restype = ci
        lib.shtb200_plan_table_bytes.argtypes = [vp]
        lib.shtb200_plan_table_bytes.restype = cs
        lib.shtb200_rfft_modes.argtypes = [vp, vp, cll, ci, ci, ctypes.c_float, vp]
        lib.shtb200_rfft_modes.restype = ci
        lib.shtb200_irfft_modes.argtypes = [vp, vp, cll, ci, ci, vp]
        lib.shtb200_irfft_modes.restype = ci
        lib.shtb200_set_sm_limit.argtypes = [ci]
        lib.shtb200_set_sm_limit.restype = ci
        lib.shtb200_rows_pieces_supported.argtypes = [ci, ci, ci, ci]
        lib.shtb200_rows_pieces_supported.restype = ci
        lib.shtb200_rfft_modes_pieces.argtypes = [vp, vp, cll, ci, ci, ctypes.c_float, ci, ci, vp]
        lib.shtb200_rfft_modes_pieces.restype = ci
        lib.shtb200_irfft_modes_pieces.argtypes = [vp, vp, cll, ci, ci, ci, ci, vp]
        lib.shtb200_irfft_modes_pieces.restype = ci
        lib.shtb200_legendre.argtypes = [vp, vp, vp, ci, ci, ci, vp, cs, vp]
        lib.shtb200_legendre.restype = ci
        lib.shtb200_legendre_pieces.argtypes = [vp, vp, vp, ci, ci, ci, ci, ci, vp, cs, vp]
        lib.shtb200_legendre_pieces.restype = ci
        lib.shtb200_legendre_workspace_bytes.argtypes = [vp, ci, ci]
        lib.shtb200_legendre_workspace_bytes.restype = cs
        lib.shtb200_spectral_conv_workspace_bytes.argtypes = [vp, vp, ci, ci, ci, ci]
        lib.shtb200_spectral_conv_workspace_bytes.restype = cs
        lib.shtb200_spectral_conv.argtypes = [vp, vp, vp, vp, vp, ci, ci, ci, ci, vp, cs, vp]
        lib.shtb200_spectral_conv.restype = ci
        lib.shtb200_quadrature.argtypes = [vp, vp, vp, cll, ci, ci, vp]
        lib.shtb200_quadrature.restype = ci
        _lib = lib
        return lib


def check(rc, what):
    if rc != 0:
        msg = load().shtb200_last_error().decode("utf-8", "replace")
        raise ShtLibraryError(f"{what} failed (code {rc}): {msg}")


def dense(t):
    """``t`` as plain contiguous memory, ready for ``data_ptr()``: ``contiguous()`` alone keeps the lazy conjugate / negative
    bits of a tensor that already is contiguous (``w.conj()``, ``z.conj().imag``), and the raw memory then holds the
    unconjugated values."""
    return t.contiguous().resolve_conj().resolve_neg()


def set_sm_limit(nsm):
    """Cap the SMs the persistent kernels size their grids for (0 = no cap); returns the previous cap."""
    return load().shtb200_set_sm_limit(int(nsm))


def rows_pieces_supported(nlon, nmodes, grid_pieces, mode_pieces):
    """Whether the row transforms take piece-major buffers for this shape (``shtb200_rows_pieces_supported``)."""
    return bool(load().shtb200_rows_pieces_supported(nlon, nmodes, grid_pieces, mode_pieces))


def spectral_conv(analysis, synthesis, x, weight, y, batch, cin, cout, groups, stream):
    """SHT -> per-degree channel mixing -> inverse SHT on device tensors (``shtb200_spectral_conv``)."""
    import torch

    lib = load()
    nbytes = lib.shtb200_spectral_conv_workspace_bytes(analysis.handle, synthesis.handle, batch, cin, cout, groups)
    if nbytes == 0:
        check(-1, "shtb200_spectral_conv_workspace_bytes")
    ws = torch.empty(nbytes, dtype=torch.uint8, device=x.device)
    rc = lib.shtb200_spectral_conv(
        analysis.handle, synthesis.handle, ctypes.c_void_p(x.data_ptr()), ctypes.c_void_p(weight.data_ptr()), ctypes.c_void_p(y.data_ptr()),
        batch, cin, cout, groups, ctypes.c_void_p(ws.data_ptr()), nbytes, ctypes.c_void_p(stream),
    )
    check(rc, "shtb200_spectral_conv")


def quadrature(x, lat_weights, out, nfields, nlat, nlon, stream):
    rc = load().shtb200_quadrature(ctypes.c_void_p(x.data_ptr()), ctypes.c_void_p(lat_weights.data_ptr()), ctypes.c_void_p(out.data_ptr()), nfields, nlat, nlon, ctypes.c_void_p(stream))
    check(rc, "shtb200_quadrature")


class Plan:
    """Owner of one ``shtb200_plan``."""

    def __init__(self, kind, nlat, nlon, lmax, mmax, table_f32_cuda, engine="auto", orders=None):
        """``orders = (m_first, m_count)`` builds a plan for that window of orders from a table that holds them only
        (``shtb200_plan_create_orders``); such a plan serves :meth:`legendre` alone."""
        import torch

        lib = load()
        if not table_f32_cuda.is_cuda or table_f32_cuda.dtype != torch.float32 or not table_f32_cuda.is_contiguous():
            raise ShtLibraryError("the Legendre table must be a contiguous float32 CUDA tensor")
        self.kind = kind
        self.device = table_f32_cuda.device
        self.handle = ctypes.c_void_p()
        torch.cuda.synchronize(self.device)
        if orders is None:
            rc = lib.shtb200_plan_create(
                ctypes.byref(self.handle), kind, nlat, nlon, lmax, mmax, ctypes.c_void_p(table_f32_cuda.data_ptr()), self.device.index or 0, ENGINES[engine]
            )
        else:
            rc = lib.shtb200_plan_create_orders(
                ctypes.byref(self.handle), kind, nlat, nlon, lmax, int(orders[0]), int(orders[1]), ctypes.c_void_p(table_f32_cuda.data_ptr()), self.device.index or 0, ENGINES[engine]
            )
        check(rc, "shtb200_plan_create")

    def workspace_bytes(self, nfields):
        return load().shtb200_workspace_bytes(self.handle, nfields)

    def execute(self, inp, out, nfields, workspace, stream):
        rc = load().shtb200_execute(
            self.handle, ctypes.c_void_p(inp.data_ptr()), ctypes.c_void_p(out.data_ptr()), nfields, ctypes.c_void_p(workspace.data_ptr()), workspace.numel(), ctypes.c_void_p(stream)
        )
        check(rc, "shtb200_execute")

    def execute_host(self, inp, out, nfields, stream=0):
        rc = load().shtb200_execute_host(self.handle, ctypes.c_void_p(inp.data_ptr()), ctypes.c_void_p(out.data_ptr()), nfields, ctypes.c_void_p(stream))
        check(rc, "shtb200_execute_host")

    def legendre_workspace_bytes(self, nfields, mloc):
        return load().shtb200_legendre_workspace_bytes(self.handle, nfields, mloc)

    def legendre(self, inp, out, nfields, m0, mloc, workspace, stream, in_pieces=1, out_pieces=1):
        """The contraction stage alone; ``in_pieces`` / ``out_pieces`` > 1: the row axis of the input / output is stored
        piece-major (``shtb200_legendre_pieces``)."""
        rc = load().shtb200_legendre_pieces(
            self.handle, ctypes.c_void_p(inp.data_ptr()), ctypes.c_void_p(out.data_ptr()), nfields, m0, mloc, in_pieces, out_pieces,
            ctypes.c_void_p(workspace.data_ptr()), workspace.numel(), ctypes.c_void_p(stream)
        )
        check(rc, "shtb200_legendre_pieces")

    def device_status(self):
        """Synchronise and raise if a kernel of this plan gave up on a bounded wait."""
        check(load().shtb200_device_status(self.handle), "shtb200_device_status")

    def set_profiling(self, on):
        check(load().shtb200_plan_set_profiling(self.handle, 1 if on else 0), "shtb200_plan_set_profiling")

    def last_kernel_times(self):
        """Milliseconds of each kernel of the last ``execute`` (needs ``set_profiling(True)``)."""
        buf = (ctypes.c_float * 8)()
        n = load().shtb200_last_kernel_times(self.handle, buf, 8)
        if n < 0:
            check(n, "shtb200_last_kernel_times")
        return [buf[i] for i in range(n)]

    @property
    def last_launch_count(self):
        return load().shtb200_last_launch_count(self.handle)

    @property
    def table_bytes(self):
        return load().shtb200_plan_table_bytes(self.handle)

    def close(self):
        if getattr(self, "handle", None) is not None and self.handle:
            try:
                load().shtb200_plan_destroy(self.handle)
            finally:
                self.handle = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass
