/*
 * shtb200 — C ABI of the B200 (sm_100a) spherical-harmonic-transform kernels.
 *
 * torch-harmonics has no FFI for this path: its SHT is a sequence of torch ops inside
 * nn.Module.forward.  This header is the boundary a binding would target instead; each entry
 * point names the reference method it replaces (paths relative to the torch-harmonics tree).
 * Plain pointers and sizes only; no torch types.  All pointers named *_dev are CUDA device
 * pointers on the plan's device; `stream` is a cudaStream_t passed as void* (NULL = default).
 *
 * Every function returns 0 on success and a negative SHTB200_E* code on failure;
 * shtb200_last_error() returns a human-readable message for the calling thread's last failure.
 */
#ifndef SHTB200_H
#define SHTB200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define SHTB200_OK 0
#define SHTB200_EINVAL -1     /* bad argument (shape, null pointer, unsupported nlon factor ...) */
#define SHTB200_ECUDA -2      /* a CUDA runtime / driver call failed */
#define SHTB200_EWORKSPACE -3 /* workspace too small */
#define SHTB200_EDEVICE -4    /* kernel reported a device-side error (bounded wait ran out ...) */

/* What a plan computes.  The two ADJOINT kinds are the vector-Jacobian products autograd
 * derives for the reference modules (they reuse the other direction's kernels with this
 * direction's table). */
enum shtb200_kind {
    SHTB200_SHT = 0,          /* RealSHT.forward              torch_harmonics/sht.py:151-186 */
    SHTB200_ISHT = 1,         /* InverseRealSHT.forward       torch_harmonics/sht.py:306-342 */
    SHTB200_SHT_ADJOINT = 2,  /* d/dx of RealSHT.forward:  grad (.., lmax, mmax) c64 -> (.., nlat, nlon) */
    SHTB200_ISHT_ADJOINT = 3, /* d/dc of InverseRealSHT.forward: grad (.., nlat, nlon) -> (.., lmax, mmax) c64 */
    SHTB200_VSHT = 4,         /* RealVectorSHT.forward        torch_harmonics/sht.py:454-495 */
    SHTB200_IVSHT = 5,        /* InverseRealVectorSHT.forward torch_harmonics/sht.py:606-649 */
    SHTB200_VSHT_ADJOINT = 6,
    SHTB200_IVSHT_ADJOINT = 7
};

/* Which Legendre contraction kernel a plan launches. */
enum shtb200_engine {
    SHTB200_ENGINE_AUTO = 0,   /* tensor-core kernel when the shape allows it */
    SHTB200_ENGINE_SIMT = 1,   /* fp32 CUDA-core contraction */
    SHTB200_ENGINE_TCGEN05 = 2 /* tcgen05 split-TF32 contraction, TMA-fed, TMEM accumulators */
};

typedef struct shtb200_plan shtb200_plan;

int shtb200_version(void);
const char *shtb200_last_error(void);

/*
 * Create a plan on CUDA device `device`.
 *
 * `table_dev` is the module's Legendre table in the reference's own dense layout, float32, on the device:
 *   SHT, ISHT_ADJOINT   : RealSHT.weights-like   (mmax, lmax, nlat)         sht.py:141-146
 *   ISHT, SHT_ADJOINT   : InverseRealSHT.pct-like (mmax, nlat, lmax)        sht.py:297-301
 *     (for the ADJOINT kinds pass the table of the module being differentiated: SHT_ADJOINT takes
 *      `weights` (mmax, lmax, nlat), ISHT_ADJOINT takes `pct` (mmax, nlat, lmax))
 *   VSHT / IVSHT (+ adjoints): (2, mmax, lmax, nlat) / (2, mmax, nlat, lmax) sht.py:438-449, 597-601
 * The table is repacked (l >= m band only, folded about the equator) into the plan; the caller may
 * free it afterwards.  nlon must factor into primes <= 31 (2, 3, 5 take the fast butterflies).
 * Replaces the constructors' buffer set-up, sht.py:113-146, 269-301, 411-449, 569-601.
 */
int shtb200_plan_create(shtb200_plan **plan, int kind, int nlat, int nlon, int lmax, int mmax, const float *table_dev, int device, int engine);
/*
 * The same for a WINDOW of orders m_first .. m_first + m_count - 1: `table_dev` holds those orders only ((m_count, lmax, nlat),
 * (m_count, nlat, lmax), or the vector layouts with m_count in place of mmax).  This is what one azimuth rank of the spatially
 * distributed transforms keeps (torch_harmonics/distributed/distributed_sht.py:164, :333, :490, :645 slice the tables the same
 * way).  Such a plan serves shtb200_legendre only (first order m0 >= m_first); the whole-transform calls refuse it.
 */
int shtb200_plan_create_orders(shtb200_plan **plan, int kind, int nlat, int nlon, int lmax, int m_first, int m_count, const float *table_dev, int device, int engine);
int shtb200_plan_destroy(shtb200_plan *plan);

/* Bytes of device scratch a call on `nfields` 2-D fields needs (vector kinds: nfields = number of (u,v) pairs). */
size_t shtb200_workspace_bytes(const shtb200_plan *plan, int nfields);

/*
 * Run the plan: `in_dev` -> `out_dev`, both contiguous, on `nfields` fields.
 *   grid -> spectral kinds (SHT, ISHT_ADJOINT, VSHT, IVSHT_ADJOINT):
 *        in  float32   [nfields, (2,) nlat, nlon]
 *        out complex64 [nfields, (2,) lmax, mmax]   (interleaved re, im; exact zeros where l < m)
 *   spectral -> grid kinds (ISHT, SHT_ADJOINT, IVSHT, VSHT_ADJOINT): the reverse.
 * `workspace_dev` must hold shtb200_workspace_bytes(plan, nfields) bytes and be 256-byte aligned.
 * Work is enqueued on `stream`; the call does not synchronise.  A plan is not re-entrant: calls on the same plan from
 * several host threads must be serialised by the caller (different plans may be used concurrently).
 * Replaces RealSHT.forward / InverseRealSHT.forward / RealVectorSHT.forward /
 * InverseRealVectorSHT.forward (sht.py:151-186, 306-342, 454-495, 606-649) and their autograd.
 */
int shtb200_execute(shtb200_plan *plan, const void *in_dev, void *out_dev, int nfields, void *workspace_dev, size_t workspace_bytes, void *stream);

/*
 * Same transform on HOST buffers: copies `in_host` to the device, runs, copies the result back and
 * synchronises `stream`.  Device staging buffers are kept in the plan and grown on demand.  The fields are
 * processed in chunks of eight: upload, kernels and download of successive chunks overlap on three streams (the
 * copies run on streams owned by the plan; give pinned host memory, pageable memory serialises the copies).
 * This is the call a host-side caller of the reference's CPU path would switch to.  The staging buffers, copy streams
 * and events belong to the plan, so two host-buffer calls on one plan must not overlap.
 */
int shtb200_execute_host(shtb200_plan *plan, const void *in_host, void *out_host, int nfields, void *stream);

/*
 * shtb200_execute for callers that are not allowed to allocate device memory (no counterpart in the reference).
 * Same transform and arguments as shtb200_execute, minus the workspace: the scratch is a device array of
 * SHTB200_STATIC_SCRATCH_BYTES built into the library, so the call itself performs no cudaMalloc / cudaFree and calls
 * no allocating library routine.  Meant for hosts that cannot allocate at call time: code inside a stream capture,
 * latency-bound serving loops with a fixed memory plan, plug-ins with a fixed device budget.
 *   - fails with SHTB200_EWORKSPACE (and says how much was needed) when shtb200_workspace_bytes(plan, nfields)
 *     exceeds SHTB200_STATIC_SCRATCH_BYTES; fails with SHTB200_EINVAL while per-kernel profiling is switched on;
 *   - the first call on each device looks up the array's device address (cudaGetSymbolAddress); make that first call
 *     before any stream capture begins;
 *   - all calls on a device share the one array and it keeps whatever the previous call left in it: the transform
 *     overwrites everything it later reads, so nothing has to be cleared between calls, but two calls that overlap
 *     on the GPU (different streams, no dependency) race on it — serialise them;
 *   - every GPU that loads the library holds the array until the process exits.
 * The plan must have been created (that step allocates) before the phase in which allocation is forbidden.
 */
#define SHTB200_STATIC_SCRATCH_BYTES (32u * 1024u * 1024u)
size_t shtb200_static_scratch_bytes(void);
int shtb200_execute_static_scratch(shtb200_plan *plan, const void *in_dev, void *out_dev, int nfields, void *stream);

/*
 * Spectral convolution on the sphere in one call: forward SHT of `batch * in_channels` fields, per-degree complex channel
 * mixing  out[b, g, o, l, m] = sum_i weight[g, i, o, l] * in[b, g, i, l, m]  within `num_groups` channel groups, inverse SHT
 * of the `batch * out_channels` results.  Replaces SpectralConvS2.forward without bias,
 * torch_harmonics/spectral_convolution.py:203-247 (sht :227, reshape + einsum "bgixy,giox->bgoxy" :236-239, isht :242).
 *   analysis  : a SHTB200_SHT plan (grid nlat_in x nlon_in); synthesis: a SHTB200_ISHT plan (grid nlat_out x nlon_out, which
 *               may differ); both with the same lmax and mmax, on the same device
 *   x_dev     : float32 [batch, in_channels, nlat_in, nlon_in]       y_dev: float32 [batch, out_channels, nlat_out, nlon_out]
 *   weight_dev: complex64 [num_groups, in_channels / num_groups, out_channels / num_groups, lmax]
 * The coefficients stay in the degree-slab layout both contraction kernels share: the (.., l, m) coefficient arrays and
 * the two transposes around them are never produced.  The adjoint kinds may be passed as well (SHTB200_ISHT_ADJOINT as
 * `analysis`, SHTB200_SHT_ADJOINT as `synthesis`): with the conjugated, (in, out)-swapped weights that is the input gradient.
 */
size_t shtb200_spectral_conv_workspace_bytes(const shtb200_plan *analysis, const shtb200_plan *synthesis, int batch, int in_channels, int out_channels, int num_groups);
int shtb200_spectral_conv(shtb200_plan *analysis, shtb200_plan *synthesis, const float *x_dev, const void *weight_dev, float *y_dev, int batch, int in_channels,
                          int out_channels, int num_groups, void *workspace_dev, size_t workspace_bytes, void *stream);

/*
 * Integral over the sphere: out[f] = sum_k lat_weights[k] * sum_j x[f, k, j] for `nfields` fields; pass the latitude
 * quadrature weights times 2 pi / nlon (divided by 4 pi for the normalised variant).  Runs on the current device.
 * Replaces QuadratureS2.forward, torch_harmonics/quadrature.py:447-463.
 */
int shtb200_quadrature(const float *x_dev, const float *lat_weights_dev, float *out_dev, long long nfields, int nlat, int nlon, void *stream);

/* Introspection used by the tests and the benchmark. */
int shtb200_plan_info(const shtb200_plan *plan, int *nlat, int *nlon, int *lmax, int *mmax, int *kind, int *engine);
/* Kernel launches the last shtb200_execute on this plan enqueued. */
int shtb200_last_launch_count(const shtb200_plan *plan);
/*
 * Per-kernel device timing of one execute call.  With profiling on, shtb200_execute records a CUDA event on
 * `stream` before its first kernel and after each kernel; shtb200_last_kernel_times waits for the last of them
 * and writes the elapsed milliseconds between consecutive events into ms[0..capacity), returning how many it
 * wrote.  Order for grid -> spectral kinds: longitude FFT, Legendre contraction, coefficient unpacking; for
 * spectral -> grid kinds: coefficient packing, Legendre contraction, longitude FFT.  (No counterpart in the
 * reference, which times whole calls in benchmarks/bench.py:60-86.)
 */
int shtb200_plan_set_profiling(shtb200_plan *plan, int on);
int shtb200_last_kernel_times(shtb200_plan *plan, float *ms, int capacity);
/*
 * Synchronise with the plan's device and report whether any kernel launched for this plan gave up on one of
 * its bounded waits (returns SHTB200_EDEVICE once, then clears the flag).  No counterpart in the reference.
 */
int shtb200_device_status(shtb200_plan *plan);
/* Total bytes of packed Legendre table held by the plan. */
size_t shtb200_plan_table_bytes(const shtb200_plan *plan);

/*
 * Stage entry points used by the spatially distributed transforms, where all-to-all transposes
 * sit between the longitude FFT and the Legendre contraction (torch_harmonics/distributed/distributed_sht.py:172-222, 341-391).
 *   shtb200_rfft_modes : float32 [nrows, nlon] -> complex64 [nrows, nmodes] = scale * rfft(x, norm="forward"), pass scale = 2*pi
 *                        (rfft(norm="forward") * 2 pi, keep/zero-pad to nmodes: fft.py:52-68 + sht.py:171)
 *   shtb200_irfft_modes: complex64 [nrows, nmodes] -> float32 [nrows, nlon], Im of DC/Nyquist ignored (fft.py:71-96)
 *   shtb200_legendre   : the plan's contraction alone.  Analysis kinds: complex64 [nfields, nlat, mloc]
 *                        (m fastest) -> complex64 [nfields, lmax, mloc]; synthesis kinds the reverse.  `m0` is
 *                        the first global order held locally and `mloc` the number of local orders.
 *                        Vector kinds (distributed_sht.py:497-555, 651-711): nfields counts (theta, phi) pairs and both
 *                        tensors carry the component axis, [nfields, 2, nlat, mloc] <-> [nfields, 2, lmax, mloc].
 * shtb200_rfft_modes / shtb200_irfft_modes take no plan: they run on the calling thread's CURRENT device (their tables
 * are built on first use and cached per (nlon, device) until the process exits).
 */
int shtb200_rfft_modes(const float *in_dev, void *out_dev, long long nrows, int nlon, int nmodes, float scale, void *stream);
int shtb200_irfft_modes(const void *in_dev, float *out_dev, long long nrows, int nlon, int nmodes, void *stream);
/*
 * Process-wide cap on the number of SMs the library's persistent kernels (FFT, Legendre contraction) size their grids for;
 * 0 removes it.  Returns the previous value.  For callers that run NCCL collectives beside these kernels on other streams:
 * a persistent kernel sized for the whole GPU leaves a collective's CTAs nowhere to run until it ends.  Takes effect at the
 * next launch; results do not depend on it.
 */
int shtb200_set_sm_limit(int nsm);
/*
 * The same two transforms on PIECE-MAJOR buffers, the form in which an all-to-all transpose receives / sends a tensor whose
 * last axis is gathered / scattered (torch_harmonics/distributed/primitives.py:227-289: the chunks of the split axis
 * travel as separate contiguous blocks): an axis of length n in P pieces is cut into balanced chunks (the first n % P one
 * longer, as compute_split_shapes does) and chunk j is stored as its own contiguous [nrows, width_j] block, the blocks one
 * after the other.  `grid_pieces` describes the longitude axis of the real buffer, `mode_pieces` the order axis of the
 * complex buffer; 1 means plain rows.  The distributed forward transform then needs no copy between the exchange that
 * gathers the longitudes, the FFT and the exchange that scatters the orders (and the inverse likewise).
 * shtb200_rows_pieces_supported returns 1 where these calls apply (nlon with a two-pass kernel: 1440, 720, 512; the
 * longitude pieces equal and a multiple of four wide), else 0 - the caller then transposes through plain rows.
 */
int shtb200_rows_pieces_supported(int nlon, int nmodes, int grid_pieces, int mode_pieces);
int shtb200_rfft_modes_pieces(const float *in_dev, void *out_dev, long long nrows, int nlon, int nmodes, float scale, int grid_pieces, int mode_pieces, void *stream);
int shtb200_irfft_modes_pieces(const void *in_dev, float *out_dev, long long nrows, int nlon, int nmodes, int mode_pieces, int grid_pieces, void *stream);
int shtb200_legendre(shtb200_plan *plan, const void *in_dev, void *out_dev, int nfields, int m0, int mloc, void *workspace_dev, size_t workspace_bytes, void *stream);
/*
 * shtb200_legendre on piece-major tensors (see shtb200_rfft_modes_pieces): the ROW axis (second to last: latitude or
 * degree) of the input is stored in `in_pieces` balanced chunks, chunk j as its own contiguous [fields, rows_j, mloc]
 * block ([fields, 2, rows_j, mloc] for the vector kinds), and the output is written the same way in `out_pieces` chunks -
 * the layouts in which the polar all-to-all delivers the latitudes and takes the degrees (and the other way round for the
 * inverse transforms), so that no copy sits between those exchanges and the contraction.  1 / 1 is shtb200_legendre.
 */
int shtb200_legendre_pieces(shtb200_plan *plan, const void *in_dev, void *out_dev, int nfields, int m0, int mloc, int in_pieces, int out_pieces, void *workspace_dev,
                            size_t workspace_bytes, void *stream);
size_t shtb200_legendre_workspace_bytes(const shtb200_plan *plan, int nfields, int mloc);

#ifdef __cplusplus
}
#endif
#endif /* SHTB200_H */
