// C ABI of the shtb200 library: plan life cycle and the execute entry points.
// Host-side glue only; the kernels live in fft_kernels.cu, legendre_*.cu and pack_kernels.cu.

#include <math.h>
#include <string.h>

#include <algorithm>
#include <atomic>
#include <mutex>

#include "common.cuh"

struct shtb200_plan : public shtb200::Plan {};

namespace shtb200 {

static thread_local std::string g_last_error;

void set_error(const std::string &msg) { g_last_error = msg; }
int fail(int code, const std::string &msg) {
    g_last_error = msg;
    return code;
}

namespace {

bool is_analysis(int kind) { return kind == SHTB200_SHT || kind == SHTB200_ISHT_ADJOINT || kind == SHTB200_VSHT || kind == SHTB200_IVSHT_ADJOINT; }
bool is_vector(int kind) { return kind >= SHTB200_VSHT; }

template <typename T>
int upload(T **dst, const std::vector<T> &src) {
    SHT_CUDA_CHECK(cudaMalloc(dst, sizeof(T) * std::max<size_t>(src.size(), 1)));
    if (!src.empty()) SHT_CUDA_CHECK(cudaMemcpy(*dst, src.data(), sizeof(T) * src.size(), cudaMemcpyHostToDevice));
    return SHTB200_OK;
}

struct DeviceGuard {
    int prev = -1;
    bool ok = false;
    explicit DeviceGuard(int dev) {
        if (cudaGetDevice(&prev) == cudaSuccess && cudaSetDevice(dev) == cudaSuccess) ok = true;
    }
    ~DeviceGuard() {
        if (prev >= 0) cudaSetDevice(prev);
    }
};

size_t align256(size_t b) { return (b + 255) / 256 * 256; }

struct WsLayout {
    size_t op_bytes = 0;  // analysis: X; synthesis: packed coefficients
    size_t y_bytes = 0;   // synthesis: latitude-row operand of the FFT
    size_t extra_bytes = 0;
    size_t total() const { return align256(op_bytes) + align256(y_bytes) + align256(extra_bytes); }
};

// (m0 = first order of the call, an actual order inside the plan's window)
WsLayout ws_layout(const Plan &pl, int nfields, int m0, int mloc) {
    WsLayout w;
    m0 -= pl.m_base;
    const size_t ncols = (size_t)(pl.vector ? 4 : 2) * nfields;
    const size_t ncp = (size_t)col_pitch((long long)ncols);  // row pitch of the column-contiguous operands
    if (pl.analysis) {
        w.op_bytes = (size_t)2 * mloc * round_up(pl.Ka, kBK) * ncp * sizeof(float);
        w.y_bytes = (size_t)(pl.group_b0[2 * (m0 + mloc)] - pl.group_b0[2 * m0]) * ncols * kBK * sizeof(float);  // degree slabs
    } else {
        const long long slabs = pl.group_b0[2 * (m0 + mloc)] - pl.group_b0[2 * m0];
        w.op_bytes = (size_t)slabs * ncols * kBK * sizeof(float);
        w.y_bytes = (size_t)2 * mloc * round_up(pl.Kh, kBK) * ncp * sizeof(float);
    }
    return w;
}

GemmParams gemm_params(const Plan &pl, int nfields, int m0, int mloc, const float *B, float *out) {
    GemmParams gp{};
    gp.A = pl.d_table;
    gp.B = B;
    gp.a_pitch = pl.a_pitch;
    gp.a_dx = pl.a_dx;
    gp.a_kext = pl.a_kext;
    gp.ncols = (pl.vector ? 4 : 2) * nfields;
    gp.items = pl.d_items;
    gp.nitems = (int)pl.items.size();
    gp.out = out;
    gp.lmax = pl.lmax;
    gp.mmax_out = mloc;
    gp.m0 = m0;
    gp.m_base = pl.m_base;
    const int ml = m0 - pl.m_base;  // first order of the call inside the plan's window
    if (pl.analysis) {
        gp.b_mn = 1;
        gp.b_krows = pl.Ka;
        gp.b_groups = 2 * mloc;
        gp.b_pitch = col_pitch(gp.ncols);
        gp.b_dx = kBK;
        gp.b_kext = pl.Ka;
        gp.b_unit0 = 2 * ml;
        // The contraction leaves degree slabs; a tiled transpose turns them into (field, l, m).  Writing (field, l, m) from
        // the epilogue instead (8-byte stores, a whole coefficient array apart per column) was measured on the
        // scalar transform at 73 fields: contraction 0.30 ms instead of 0.16 + 0.08 ms.
        gp.mode = EPI_SLABS;
        gp.slab0 = pl.d_gb0;
        gp.slab_unit0 = pl.group_b0[2 * ml];
    } else {
        gp.b_pitch = kBK;
        gp.b_dx = 0;
        gp.b_kext = kBK;
        gp.b_unit0 = pl.group_b0[2 * ml];
        gp.mode = EPI_LATROWS;
        gp.out_ld = col_pitch(gp.ncols);
        gp.out_groups = 2 * mloc;
    }
    return gp;
}

void mark(Plan &pl, cudaStream_t st) {
    if (!pl.profiling || pl.nev >= 8) return;
    if (!pl.ev[pl.nev] && cudaEventCreate(&pl.ev[pl.nev]) != cudaSuccess) return;
    cudaEventRecord(pl.ev[pl.nev++], st);
}

int run_gemm(Plan &pl, const GemmParams &gp, cudaStream_t st) {
    bool tc = false;
    if (pl.engine == SHTB200_ENGINE_TCGEN05) {
        if (!gemm_tc_supported(pl, gp)) return fail(SHTB200_EINVAL, "tcgen05 engine requested but the shape is not supported by it");
        tc = true;
    } else if (pl.engine == SHTB200_ENGINE_AUTO) {
        tc = gemm_tc_supported(pl, gp);
    }
    pl.last_launches += 1;
    return tc ? launch_gemm_tc(pl, gp, st) : launch_gemm_simt(gp, st);
}

// Y slices of groups that contain no degree at all are never produced by the contraction.
int clear_empty_groups(const Plan &pl, float *Y, int ncols, int m0, int mloc, cudaStream_t st) {
    m0 -= pl.m_base;
    for (int g = 2 * m0; g < 2 * (m0 + mloc); ++g) {
        if (pl.group_kblocks[g] == 0) {
            const size_t ncp = (size_t)col_pitch(ncols);
            // the group's 64-byte pieces, one per (latitude, 16-column panel), lie a whole panel row (2 mloc pieces) apart
            SHT_CUDA_CHECK(cudaMemset2DAsync(Y + y_off(g - 2 * m0, 0, 0, 2 * mloc, (long long)ncp), sizeof(float) * 16 * 2 * mloc, 0, sizeof(float) * 16, (size_t)pl.Kh * (ncp / 16), st));
        }
    }
    return SHTB200_OK;
}

int execute_full(Plan &pl, const void *in, void *out, int nfields, void *ws, size_t ws_bytes, cudaStream_t st) {
    if (pl.window) return fail(SHTB200_EINVAL, "a plan created for a window of orders serves shtb200_legendre only");
    if (nfields < 0) return fail(SHTB200_EINVAL, "nfields must be >= 0");
    pl.last_launches = 0;
    if (nfields == 0) return SHTB200_OK;
    if (!in || !out) return fail(SHTB200_EINVAL, "null input or output pointer");
    WsLayout w = ws_layout(pl, nfields, 0, pl.mmax);
    if (ws_bytes < w.total() || (!ws && w.total() > 0)) return fail(SHTB200_EWORKSPACE, "workspace too small: need " + std::to_string(w.total()) + " bytes");
    if (((uintptr_t)ws & 255) != 0) return fail(SHTB200_EINVAL, "workspace must be 256-byte aligned");
    int rc;
    pl.nev = 0;
    mark(pl, st);
    if (pl.analysis) {
        float *X = reinterpret_cast<float *>(ws);
        float *Z = reinterpret_cast<float *>(reinterpret_cast<char *>(ws) + align256(w.op_bytes));
        if ((rc = launch_fft_analysis(pl, reinterpret_cast<const float *>(in), X, nfields, st))) return rc;
        mark(pl, st);
        pl.last_launches += 1;
        GemmParams gp = gemm_params(pl, nfields, 0, pl.mmax, X, Z);
        if ((rc = run_gemm(pl, gp, st))) return rc;
        mark(pl, st);
        // (a vector pair's four columns are the (re, im) pairs of its two output fields: the same slab layout with twice the fields)
        if ((rc = launch_unpack_coeffs(pl, Z, reinterpret_cast<float2 *>(out), nfields, 0, pl.mmax, 1, st))) return rc;
        pl.last_launches += 1;
        mark(pl, st);
    } else {
        float *Ct = reinterpret_cast<float *>(ws);
        float *Y = reinterpret_cast<float *>(reinterpret_cast<char *>(ws) + align256(w.op_bytes));
        const int ncols = (pl.vector ? 4 : 2) * nfields;
        if ((rc = launch_pack_coeffs(pl, reinterpret_cast<const float2 *>(in), Ct, nfields, 0, pl.mmax, 1, st))) return rc;
        if ((rc = clear_empty_groups(pl, Y, ncols, 0, pl.mmax, st))) return rc;
        mark(pl, st);
        GemmParams gp = gemm_params(pl, nfields, 0, pl.mmax, Ct, Y);
        if ((rc = run_gemm(pl, gp, st))) return rc;
        mark(pl, st);
        if ((rc = launch_fft_synthesis(pl, Y, reinterpret_cast<float *>(out), nfields, st))) return rc;
        mark(pl, st);
        pl.last_launches += 2;
    }
    return SHTB200_OK;
}

int grow(void **p, size_t *have, size_t need) {
    if (*have >= need) return SHTB200_OK;
    if (*p) cudaFree(*p);
    *p = nullptr;
    *have = 0;
    SHT_CUDA_CHECK(cudaMalloc(p, need));
    *have = need;
    return SHTB200_OK;
}

}  // namespace
}  // namespace shtb200

using namespace shtb200;

namespace shtb200 {
static std::atomic<int> g_sm_limit{0};
int effective_sms(int sm_count) {
    const int lim = g_sm_limit.load(std::memory_order_relaxed);
    return lim > 0 ? std::min(sm_count, lim) : sm_count;
}
}  // namespace shtb200

extern "C" {

int shtb200_version(void) { return 100; }

const char *shtb200_last_error(void) { return g_last_error.c_str(); }

}  // extern "C"

// `mmax` orders starting at `m_base`; `window` marks a plan that serves the Legendre stage only
static int plan_create_impl(shtb200_plan **plan_out, int kind, int nlat, int nlon, int lmax, int m_base, int mmax, bool window, const float *table_dev, int device,
                            int engine) {
    if (!plan_out) return fail(SHTB200_EINVAL, "plan_out is null");
    *plan_out = nullptr;
    if (kind < SHTB200_SHT || kind > SHTB200_IVSHT_ADJOINT) return fail(SHTB200_EINVAL, "unknown plan kind");
    if (engine < SHTB200_ENGINE_AUTO || engine > SHTB200_ENGINE_TCGEN05) return fail(SHTB200_EINVAL, "unknown engine");
    if (nlat < 2 || nlon < 2 || lmax < 1 || mmax < 1) return fail(SHTB200_EINVAL, "nlat, nlon >= 2 and lmax, mmax >= 1 required");
    if (m_base < 0 || m_base + mmax > lmax) return fail(SHTB200_EINVAL, "mmax must not exceed lmax (triangular truncation)");
    if (!table_dev) return fail(SHTB200_EINVAL, "table_dev is null");
    int ndev = 0;
    if (cudaGetDeviceCount(&ndev) != cudaSuccess || ndev == 0) return fail(SHTB200_ECUDA, "no CUDA device available: this library has no CPU path");
    if (device < 0 || device >= ndev) return fail(SHTB200_EINVAL, "device index out of range");
    DeviceGuard guard(device);
    if (!guard.ok) return fail(SHTB200_ECUDA, "cudaSetDevice failed");

    shtb200_plan *pl = new shtb200_plan();
    pl->kind = kind;
    pl->engine = engine;
    pl->device = device;
    pl->nlat = nlat;
    pl->nlon = nlon;
    pl->lmax = lmax;
    pl->mmax = mmax;
    pl->m_base = m_base;
    pl->window = window;
    pl->analysis = is_analysis(kind);
    pl->vector = is_vector(kind);
    pl->ncomp = pl->vector ? 2 : 1;
    pl->Kh = (nlat + 1) / 2;
    pl->Ka = pl->ncomp * pl->Kh;
    pl->Lh = (lmax + 1) / 2;
    pl->negate_seg1 = (kind == SHTB200_VSHT_ADJOINT || kind == SHTB200_IVSHT_ADJOINT) ? 1 : 0;
    if (cudaDeviceGetAttribute(&pl->sm_count, cudaDevAttrMultiProcessorCount, device) != cudaSuccess || pl->sm_count < 1) {
        delete pl;
        return fail(SHTB200_ECUDA, "cannot read the multiprocessor count");
    }

    int rc;

    // per-order scale applied inside the FFT kernels
    std::vector<float> ms(mmax);
    {
        for (int ml = 0; ml < mmax; ++ml) {
            const int m = m_base + ml;
            const bool edge = (m == 0) || (2 * m == nlon);
            double s = 1.0;
            switch (kind) {
                case SHTB200_SHT: case SHTB200_VSHT: s = 2.0 * M_PI / nlon; break;                       // sht.py:171
                case SHTB200_ISHT: case SHTB200_IVSHT: s = 1.0; break;                                     // irfft(norm="forward")
                case SHTB200_SHT_ADJOINT: case SHTB200_VSHT_ADJOINT: s = (2.0 * M_PI / nlon) * (edge ? 1.0 : 0.5); break;
                case SHTB200_ISHT_ADJOINT: case SHTB200_IVSHT_ADJOINT: s = edge ? 1.0 : 2.0; break;
            }
            ms[ml] = (float)s;
        }
        if ((rc = upload(&pl->d_mscale, ms))) { shtb200_plan_destroy(pl); return rc; }
        pl->zero_imag_edges = (kind == SHTB200_ISHT_ADJOINT || kind == SHTB200_IVSHT_ADJOINT) ? 1 : 0;
    }

    // groups g = 2 m + p
    const int ngroups = 2 * mmax;
    pl->group_rows.assign(ngroups, 0);
    for (int m = 0; m < mmax; ++m)
        for (int p = 0; p < 2; ++p) {
            int cnt = lmax - (m_base + m) - p;
            pl->group_rows[2 * m + p] = cnt > 0 ? (cnt + 1) / 2 : 0;
        }
    // Polar extent of every group, in whole 32-row blocks.  The cut-off is far below what fp32 keeps next to the
    // largest entry of the same degree, so the result is the one the full contraction would give.
    pl->group_krow0.assign(ngroups, 0);
    if (kind == SHTB200_SHT || kind == SHTB200_ISHT) {
        std::vector<int> first;
        if ((rc = launch_polar_extent(*pl, table_dev, 1e-14f, &first))) { shtb200_plan_destroy(pl); return rc; }
        // The FFT kernels carry the extent as a 4-bit block index per group: blocks beyond 15 are not skipped (skipping
        // fewer rows is always correct; the contraction and the FFT kernels read the same clamped value).
        for (int g = 0; g < ngroups; ++g) pl->group_krow0[g] = std::min(std::min(first[g], std::max(pl->Kh - 1, 0)) / kBK, kMaxPolarBlock) * kBK;
    }
    // (a window plan never runs a longitude transform)
    if (!window && ((rc = build_fft_plan(nlon, mmax, pl->analysis ? kFftSplit : kFftPacked, pl->group_krow0.data(), &pl->fft, &pl->d_tw, &pl->d_perm)) ||
                    (rc = build_twopass_tables(*pl, ms)))) {
        shtb200_plan_destroy(pl);
        return rc;
    }
    pl->group_a0.assign(ngroups + 1, 0);
    pl->group_kblocks.assign(ngroups, 0);
    pl->group_b0.assign(ngroups + 1, 0);
    std::vector<int> kb0(ngroups, 0);
    if (pl->analysis) {
        pl->a_pitch = round_up(pl->Ka, 8);
        pl->a_dx = kBK;
        pl->a_kext = pl->Ka;
        for (int g = 0; g < ngroups; ++g) {
            pl->group_a0[g + 1] = pl->group_a0[g] + pl->group_rows[g];
            // degree slabs of the contraction's output (same layout the synthesis side reads)
            pl->group_kblocks[g] = ceil_div(pl->group_rows[g], kBK);
            pl->group_b0[g + 1] = pl->group_b0[g] + pl->group_kblocks[g];
        }
        pl->total_b_slabs = pl->group_b0[ngroups];
        pl->table_floats = (size_t)(pl->group_a0[ngroups] + kItemRowsMax) * pl->a_pitch;
        const int kblocks = ceil_div(pl->Ka, kBK);
        for (int g = 0; g < ngroups; ++g)
            for (int r0 = 0; r0 < pl->group_rows[g]; r0 += kItemRowsMax) {
                GemmItem it{};
                it.a_y0 = (int)(pl->group_a0[g] + r0);
                it.a_dy = 0;
                it.b_y0 = g;
                it.b_dy = 0;
                it.kfirst = pl->group_krow0[g] / kBK;
                it.kblocks = kblocks - it.kfirst;
                it.rows = std::min(kItemRowsMax, pl->group_rows[g] - r0);
                it.m = m_base + (g >> 1);
                it.p = g & 1;
                it.r0 = r0;
                pl->items.push_back(it);
            }
    } else {
        pl->a_pitch = kBK;
        pl->a_dx = 0;
        pl->a_kext = kBK;
        for (int g = 0; g < ngroups; ++g) {
            int nb = ceil_div(pl->group_rows[g], kBK);
            if (pl->vector) {
                kb0[g] = ceil_div(pl->group_rows[g ^ 1], kBK);
                nb += kb0[g];
            }
            pl->group_kblocks[g] = nb;
            pl->group_a0[g + 1] = pl->group_a0[g] + (long long)nb * pl->Kh;
            pl->group_b0[g + 1] = pl->group_b0[g] + nb;
        }
        pl->total_b_slabs = pl->group_b0[ngroups];
        pl->table_floats = (size_t)(pl->group_a0[ngroups] + kItemRowsMax) * kBK;
        for (int g = 0; g < ngroups; ++g) {
            if (pl->group_kblocks[g] == 0) continue;
            for (int r0 = pl->group_krow0[g]; r0 < pl->Kh; r0 += kItemRowsMax) {
                GemmItem it{};
                it.a_y0 = (int)(pl->group_a0[g] + r0);
                it.a_dy = pl->Kh;
                it.b_y0 = (int)pl->group_b0[g];
                it.b_dy = 1;
                it.kblocks = pl->group_kblocks[g];
                it.rows = std::min(kItemRowsMax, pl->Kh - r0);
                it.m = m_base + (g >> 1);
                it.p = g & 1;
                it.r0 = r0;
                pl->items.push_back(it);
            }
        }
    }
    if (pl->group_a0[ngroups] + kItemRowsMax > 0x7fffffffLL) { shtb200_plan_destroy(pl); return fail(SHTB200_EINVAL, "table too large for 32-bit row indices"); }
    // Heaviest groups first; the row tiles of one group stay adjacent so that CTAs working on them at the same
    // time share the group's operand through L2 instead of fetching it from HBM again later.
    {
        std::vector<long long> gwork(ngroups, 0);
        for (const GemmItem &it : pl->items) gwork[2 * (it.m - m_base) + it.p] += (long long)it.kblocks * it.rows;
        std::stable_sort(pl->items.begin(), pl->items.end(), [&gwork, m_base](const GemmItem &a, const GemmItem &b) {
            const int ga = 2 * (a.m - m_base) + a.p, gb = 2 * (b.m - m_base) + b.p;
            if (gwork[ga] != gwork[gb]) return gwork[ga] > gwork[gb];
            if (ga != gb) return ga < gb;
            return a.r0 < b.r0;
        });
    }

    if ((rc = upload(&pl->d_items, pl->items)) || (rc = upload(&pl->d_ga0, pl->group_a0)) || (rc = upload(&pl->d_gb0, pl->group_b0)) ||
        (rc = upload(&pl->d_grows, pl->group_rows)) || (rc = upload(&pl->d_gkb, pl->group_kblocks)) || (rc = upload(&pl->d_gkb0, kb0)) ||
        (rc = upload(&pl->d_krow0, pl->group_krow0))) {
        shtb200_plan_destroy(pl);
        return rc;
    }
    if (pl->analysis && !pl->vector && !pl->window) {  // degree classes of the slabs (see Plan::d_cls_off)
        std::vector<std::vector<int>> cls(pl->lmax);
        for (int g = 0; g < ngroups; ++g)
            for (int rb = 0; rb < pl->group_kblocks[g]; ++rb) {
                const int l0 = (g >> 1) + (g & 1) + 2 * kBK * rb;  // (< lmax: a slab exists only for a degree below lmax)
                cls[l0].push_back((int)(pl->group_b0[g] + rb));
            }
        std::vector<int> off(pl->lmax + 1, 0), slabs;
        for (int l0 = 0; l0 < pl->lmax; ++l0) {
            slabs.insert(slabs.end(), cls[l0].begin(), cls[l0].end());
            off[l0 + 1] = (int)slabs.size();
        }
        if (slabs.empty()) slabs.push_back(0);
        if ((rc = upload(&pl->d_cls_off, off)) || (rc = upload(&pl->d_cls_slab, slabs))) {
            shtb200_plan_destroy(pl);
            return rc;
        }
    }
    if (cudaMalloc(&pl->d_err, sizeof(int)) != cudaSuccess || cudaMemset(pl->d_err, 0, sizeof(int)) != cudaSuccess) {
        shtb200_plan_destroy(pl);
        return fail(SHTB200_ECUDA, "error word allocation failed");
    }
    cudaError_t e = cudaMalloc(&pl->d_table, sizeof(float) * pl->table_floats);
    if (e == cudaSuccess) e = cudaMemset(pl->d_table, 0, sizeof(float) * pl->table_floats);
    if (e != cudaSuccess) { shtb200_plan_destroy(pl); return fail(SHTB200_ECUDA, std::string("table allocation: ") + cudaGetErrorString(e)); }
    if ((rc = launch_pack_table(*pl, table_dev, 0))) { shtb200_plan_destroy(pl); return rc; }
    *plan_out = pl;
    return SHTB200_OK;
}

extern "C" {

int shtb200_plan_create(shtb200_plan **plan_out, int kind, int nlat, int nlon, int lmax, int mmax, const float *table_dev, int device, int engine) {
    if (mmax > lmax) return fail(SHTB200_EINVAL, "mmax must not exceed lmax (triangular truncation)");
    return plan_create_impl(plan_out, kind, nlat, nlon, lmax, 0, mmax, false, table_dev, device, engine);
}

int shtb200_plan_create_orders(shtb200_plan **plan_out, int kind, int nlat, int nlon, int lmax, int m_first, int m_count, const float *table_dev, int device, int engine) {
    return plan_create_impl(plan_out, kind, nlat, nlon, lmax, m_first, m_count, true, table_dev, device, engine);
}

int shtb200_plan_destroy(shtb200_plan *pl) {
    if (!pl) return SHTB200_OK;
    DeviceGuard guard(pl->device);
    cudaFree(pl->d_tw);
    cudaFree(pl->d_perm);
    cudaFree(pl->d_mscale);
    cudaFree(pl->d_tp_blob);
    cudaFree(pl->d_table);
    cudaFree(pl->d_items);
    cudaFree(pl->d_ga0);
    cudaFree(pl->d_gb0);
    cudaFree(pl->d_grows);
    cudaFree(pl->d_gkb);
    cudaFree(pl->d_gkb0);
    cudaFree(pl->d_cls_off);
    cudaFree(pl->d_cls_slab);
    if (pl->copy_in) cudaStreamDestroy(pl->copy_in);
    if (pl->copy_out) cudaStreamDestroy(pl->copy_out);
    for (cudaEvent_t e : pl->ev_up) cudaEventDestroy(e);
    for (cudaEvent_t e : pl->ev_done) cudaEventDestroy(e);
    cudaFree(pl->stage_in);
    cudaFree(pl->stage_out);
    cudaFree(pl->stage_ws);
    cudaFree(pl->d_krow0);
    cudaFree(pl->d_err);
    for (auto &e : pl->ev)
        if (e) cudaEventDestroy(e);
    delete pl;
    return SHTB200_OK;
}

size_t shtb200_workspace_bytes(const shtb200_plan *pl, int nfields) {
    if (!pl || nfields <= 0 || pl->window) return 0;
    return ws_layout(*pl, nfields, 0, pl->mmax).total();
}

int shtb200_execute(shtb200_plan *pl, const void *in_dev, void *out_dev, int nfields, void *workspace_dev, size_t workspace_bytes, void *stream) {
    if (!pl) return fail(SHTB200_EINVAL, "plan is null");
    DeviceGuard guard(pl->device);
    if (!guard.ok) return fail(SHTB200_ECUDA, "cudaSetDevice failed");
    return execute_full(*pl, in_dev, out_dev, nfields, workspace_dev, workspace_bytes, (cudaStream_t)stream);
}

int shtb200_execute_host(shtb200_plan *pl, const void *in_host, void *out_host, int nfields, void *stream) {
    if (!pl) return fail(SHTB200_EINVAL, "plan is null");
    if (pl->window) return fail(SHTB200_EINVAL, "a plan created for a window of orders serves shtb200_legendre only");
    if (nfields < 0) return fail(SHTB200_EINVAL, "nfields must be >= 0");
    if (nfields == 0) return SHTB200_OK;
    if (!in_host || !out_host) return fail(SHTB200_EINVAL, "null host pointer");
    DeviceGuard guard(pl->device);
    if (!guard.ok) return fail(SHTB200_ECUDA, "cudaSetDevice failed");
    cudaStream_t st = (cudaStream_t)stream;
    const size_t comp = pl->vector ? 2 : 1;
    const size_t grid_bytes = (size_t)nfields * comp * pl->nlat * pl->nlon * sizeof(float);
    const size_t spec_bytes = (size_t)nfields * comp * pl->lmax * pl->mmax * sizeof(float2);
    const size_t in_bytes = pl->analysis ? grid_bytes : spec_bytes;
    const size_t out_bytes = pl->analysis ? spec_bytes : grid_bytes;
    // Fields are independent, so the transform is pipelined over chunks of fields: the upload of chunk i + 1, the
    // kernels of chunk i and the download of chunk i - 1 run at the same time on three streams (both PCIe directions busy).
    // Chunks of eight fields, except at both ends: the first upload and the last download have nothing to hide behind,
    // so the first and the last chunk are short (two fields).
    const int chunk = std::min(nfields, 8);
    std::vector<int> sizes;
    {
        int left = nfields;
        if (left > 16) { sizes.push_back(2); sizes.push_back(6); left -= 8; }
        while (left > 10) { sizes.push_back(8); left -= 8; }
        if (left > 2 && nfields > 16) { sizes.push_back(left - 2); left = 2; }
        while (left > 0) { sizes.push_back(std::min(left, chunk)); left -= sizes.back(); }
    }
    const int nchunks = (int)sizes.size();
    const size_t ws_bytes = shtb200_workspace_bytes(pl, chunk);
    int rc;
    if ((rc = grow(&pl->stage_in, &pl->stage_in_bytes, in_bytes)) || (rc = grow(&pl->stage_out, &pl->stage_out_bytes, out_bytes)) ||
        (rc = grow(&pl->stage_ws, &pl->stage_ws_bytes, ws_bytes)))
        return rc;
    if (!pl->copy_in) SHT_CUDA_CHECK(cudaStreamCreateWithFlags(&pl->copy_in, cudaStreamNonBlocking));
    if (!pl->copy_out) SHT_CUDA_CHECK(cudaStreamCreateWithFlags(&pl->copy_out, cudaStreamNonBlocking));
    while ((int)pl->ev_up.size() < nchunks + 1) {
        cudaEvent_t a = nullptr, b = nullptr;
        SHT_CUDA_CHECK(cudaEventCreateWithFlags(&a, cudaEventDisableTiming));
        pl->ev_up.push_back(a);
        SHT_CUDA_CHECK(cudaEventCreateWithFlags(&b, cudaEventDisableTiming));
        pl->ev_done.push_back(b);
    }
    const size_t in_per = in_bytes / nfields, out_per = out_bytes / nfields;
    // the copy streams start after whatever the caller already queued on `stream`
    SHT_CUDA_CHECK(cudaEventRecord(pl->ev_up[nchunks], st));
    SHT_CUDA_CHECK(cudaStreamWaitEvent(pl->copy_in, pl->ev_up[nchunks], 0));
    int launches = 0;
    for (int i = 0, f0 = 0; i < nchunks; f0 += sizes[i], ++i) {
        const int nf = sizes[i];
        char *din = reinterpret_cast<char *>(pl->stage_in) + (size_t)f0 * in_per;
        char *dout = reinterpret_cast<char *>(pl->stage_out) + (size_t)f0 * out_per;
        SHT_CUDA_CHECK(cudaMemcpyAsync(din, reinterpret_cast<const char *>(in_host) + (size_t)f0 * in_per, (size_t)nf * in_per, cudaMemcpyHostToDevice, pl->copy_in));
        SHT_CUDA_CHECK(cudaEventRecord(pl->ev_up[i], pl->copy_in));
        SHT_CUDA_CHECK(cudaStreamWaitEvent(st, pl->ev_up[i], 0));
        if ((rc = execute_full(*pl, din, dout, nf, pl->stage_ws, pl->stage_ws_bytes, st))) return rc;
        launches += pl->last_launches;
        SHT_CUDA_CHECK(cudaEventRecord(pl->ev_done[i], st));
        SHT_CUDA_CHECK(cudaStreamWaitEvent(pl->copy_out, pl->ev_done[i], 0));
        SHT_CUDA_CHECK(cudaMemcpyAsync(reinterpret_cast<char *>(out_host) + (size_t)f0 * out_per, dout, (size_t)nf * out_per, cudaMemcpyDeviceToHost, pl->copy_out));
    }
    pl->last_launches = launches;
    SHT_CUDA_CHECK(cudaStreamSynchronize(pl->copy_out));
    SHT_CUDA_CHECK(cudaStreamSynchronize(st));
    return SHTB200_OK;
}

namespace {
struct ConvLayout {
    size_t op, zin, zout, wsplit;  // [X / Y (shared)][Z in][Z out][split weights]
    size_t total() const { return align256(op) + align256(zin) + align256(zout) + align256(wsplit); }
};
int conv_layout(const Plan &pa, const Plan &ps, int batch, int cin, int cout, int ngroups, ConvLayout *out) {
    if (pa.window || ps.window) return fail(SHTB200_EINVAL, "a plan created for a window of orders serves shtb200_legendre only");
    if (pa.vector || ps.vector || !pa.analysis || ps.analysis) return fail(SHTB200_EINVAL, "spectral convolution needs a scalar analysis plan and a scalar synthesis plan");
    if (pa.lmax != ps.lmax || pa.mmax != ps.mmax) return fail(SHTB200_EINVAL, "the two plans of a spectral convolution must share lmax and mmax");
    if (pa.device != ps.device) return fail(SHTB200_EINVAL, "the two plans of a spectral convolution must live on the same device");
    if (batch < 1 || cin < 1 || cout < 1 || ngroups < 1 || cin % ngroups || cout % ngroups) return fail(SHTB200_EINVAL, "bad (batch, channels, groups)");
    if ((long long)batch * std::max(cin, cout) > 0x3fffffffLL) return fail(SHTB200_EINVAL, "too many fields");
    const WsLayout wa = ws_layout(pa, batch * cin, 0, pa.mmax), wsyn = ws_layout(ps, batch * cout, 0, ps.mmax);
    out->op = std::max(wa.op_bytes, wsyn.y_bytes);
    out->zin = wa.y_bytes;
    out->zout = wsyn.op_bytes;
    out->wsplit = slab_mix_weight_bytes(cin, cout, ngroups, pa.lmax);
    return SHTB200_OK;
}
}  // namespace

size_t shtb200_spectral_conv_workspace_bytes(const shtb200_plan *analysis, const shtb200_plan *synthesis, int batch, int in_channels, int out_channels, int num_groups) {
    ConvLayout L{};
    if (!analysis || !synthesis || conv_layout(*analysis, *synthesis, batch, in_channels, out_channels, num_groups, &L)) return 0;
    return L.total();
}

int shtb200_spectral_conv(shtb200_plan *analysis, shtb200_plan *synthesis, const float *x_dev, const void *weight_dev, float *y_dev, int batch, int in_channels,
                          int out_channels, int num_groups, void *workspace_dev, size_t workspace_bytes, void *stream) {
    if (!analysis || !synthesis) return fail(SHTB200_EINVAL, "plan is null");
    if (!x_dev || !weight_dev || !y_dev) return fail(SHTB200_EINVAL, "null pointer");
    Plan &pa = *analysis, &ps = *synthesis;
    ConvLayout L{};
    int rc;
    if ((rc = conv_layout(pa, ps, batch, in_channels, out_channels, num_groups, &L))) return rc;
    if (workspace_bytes < L.total() || !workspace_dev) return fail(SHTB200_EWORKSPACE, "workspace too small: need " + std::to_string(L.total()) + " bytes");
    if (((uintptr_t)workspace_dev & 255) != 0) return fail(SHTB200_EINVAL, "workspace must be 256-byte aligned");
    DeviceGuard guard(pa.device);
    if (!guard.ok) return fail(SHTB200_ECUDA, "cudaSetDevice failed");
    cudaStream_t st = (cudaStream_t)stream;
    char *base = reinterpret_cast<char *>(workspace_dev);
    float *XY = reinterpret_cast<float *>(base);
    float *Zin = reinterpret_cast<float *>(base + align256(L.op));
    float *Zout = reinterpret_cast<float *>(base + align256(L.op) + align256(L.zin));
    float2 *Wsplit = reinterpret_cast<float2 *>(base + align256(L.op) + align256(L.zin) + align256(L.zout));
    const int nin = batch * in_channels, nout = batch * out_channels;
    pa.last_launches = ps.last_launches = 0;
    // analysis: longitude FFT, Legendre contraction into the degree slabs
    if ((rc = launch_fft_analysis(pa, x_dev, XY, nin, st))) return rc;
    {
        GemmParams gp = gemm_params(pa, nin, 0, pa.mmax, XY, Zin);
        if ((rc = run_gemm(pa, gp, st))) return rc;
    }
    // per-degree channel mixing, slabs to slabs
    if ((rc = launch_slab_mix(pa, Zin, Zout, reinterpret_cast<const float2 *>(weight_dev), Wsplit, batch, in_channels, out_channels, num_groups, st))) return rc;
    // synthesis: Legendre contraction from the slabs, longitude FFT
    if ((rc = clear_empty_groups(ps, XY, 2 * nout, 0, ps.mmax, st))) return rc;
    {
        GemmParams gp = gemm_params(ps, nout, 0, ps.mmax, Zout, XY);
        if ((rc = run_gemm(ps, gp, st))) return rc;
    }
    if ((rc = launch_fft_synthesis(ps, XY, y_dev, nout, st))) return rc;
    pa.last_launches = 6;  // FFT, contraction, weight split, mixing, contraction, FFT
    return SHTB200_OK;
}

int shtb200_quadrature(const float *x_dev, const float *lat_weights_dev, float *out_dev, long long nfields, int nlat, int nlon, void *stream) {
    if (nfields < 0 || nlat < 1 || nlon < 1) return fail(SHTB200_EINVAL, "bad quadrature shape");
    if (nfields == 0) return SHTB200_OK;
    if (!x_dev || !lat_weights_dev || !out_dev) return fail(SHTB200_EINVAL, "null pointer");
    return launch_quadrature(x_dev, lat_weights_dev, out_dev, nfields, nlat, nlon, (cudaStream_t)stream);
}

int shtb200_plan_info(const shtb200_plan *pl, int *nlat, int *nlon, int *lmax, int *mmax, int *kind, int *engine) {
    if (!pl) return fail(SHTB200_EINVAL, "plan is null");
    if (nlat) *nlat = pl->nlat;
    if (nlon) *nlon = pl->nlon;
    if (lmax) *lmax = pl->lmax;
    if (mmax) *mmax = pl->mmax;
    if (kind) *kind = pl->kind;
    if (engine) *engine = pl->engine;
    return SHTB200_OK;
}

int shtb200_last_launch_count(const shtb200_plan *pl) { return pl ? pl->last_launches : 0; }

int shtb200_plan_set_profiling(shtb200_plan *pl, int on) {
    if (!pl) return fail(SHTB200_EINVAL, "plan is null");
    pl->profiling = on ? 1 : 0;
    pl->nev = 0;
    return SHTB200_OK;
}

int shtb200_last_kernel_times(shtb200_plan *pl, float *ms, int capacity) {
    if (!pl || !ms) return fail(SHTB200_EINVAL, "null argument");
    if (pl->nev < 2) return 0;
    DeviceGuard guard(pl->device);
    if (cudaEventSynchronize(pl->ev[pl->nev - 1]) != cudaSuccess) return fail(SHTB200_ECUDA, "event synchronise failed");
    int n = 0;
    for (int i = 0; i + 1 < pl->nev && n < capacity; ++i, ++n) {
        if (cudaEventElapsedTime(&ms[n], pl->ev[i], pl->ev[i + 1]) != cudaSuccess) return fail(SHTB200_ECUDA, "event elapsed time failed");
    }
    return n;
}

int shtb200_device_status(shtb200_plan *pl) {
    if (!pl) return fail(SHTB200_EINVAL, "plan is null");
    DeviceGuard guard(pl->device);
    int v = 0;
    cudaError_t e = cudaMemcpy(&v, pl->d_err, sizeof(int), cudaMemcpyDeviceToHost);  // waits for the work enqueued so far
    if (e != cudaSuccess) return fail(SHTB200_ECUDA, std::string("device status: ") + cudaGetErrorString(e));
    if (v != 0) {
        cudaMemset(pl->d_err, 0, sizeof(int));
        return fail(SHTB200_EDEVICE, "a kernel gave up on a bounded wait (device error word " + std::to_string(v) + ")");
    }
    return SHTB200_OK;
}

size_t shtb200_plan_table_bytes(const shtb200_plan *pl) { return pl ? pl->table_floats * sizeof(float) : 0; }

int shtb200_rfft_modes(const float *in_dev, void *out_dev, long long nrows, int nlon, int nmodes, float scale, void *stream) {
    if (nrows < 0 || nlon < 2 || nmodes < 1) return fail(SHTB200_EINVAL, "bad rfft shape");
    if (nrows == 0) return SHTB200_OK;
    if (!in_dev || !out_dev) return fail(SHTB200_EINVAL, "null pointer");
    return launch_rfft_modes(in_dev, reinterpret_cast<float2 *>(out_dev), nrows, nlon, nmodes, scale, 1, 1, (cudaStream_t)stream);
}

int shtb200_set_sm_limit(int nsm) {
    const int before = g_sm_limit.exchange(nsm > 0 ? nsm : 0);
    return before;
}

int shtb200_rows_pieces_supported(int nlon, int nmodes, int grid_pieces, int mode_pieces) { return rows_pieces_supported(nlon, nmodes, grid_pieces, mode_pieces) ? 1 : 0; }

int shtb200_rfft_modes_pieces(const float *in_dev, void *out_dev, long long nrows, int nlon, int nmodes, float scale, int grid_pieces, int mode_pieces, void *stream) {
    if (nrows < 0 || nlon < 2 || nmodes < 1 || grid_pieces < 1 || mode_pieces < 1) return fail(SHTB200_EINVAL, "bad rfft shape");
    if (nrows == 0) return SHTB200_OK;
    if (!in_dev || !out_dev) return fail(SHTB200_EINVAL, "null pointer");
    return launch_rfft_modes(in_dev, reinterpret_cast<float2 *>(out_dev), nrows, nlon, nmodes, scale, grid_pieces, mode_pieces, (cudaStream_t)stream);
}

int shtb200_irfft_modes_pieces(const void *in_dev, float *out_dev, long long nrows, int nlon, int nmodes, int mode_pieces, int grid_pieces, void *stream) {
    if (nrows < 0 || nlon < 2 || nmodes < 1 || grid_pieces < 1 || mode_pieces < 1) return fail(SHTB200_EINVAL, "bad irfft shape");
    if (nrows == 0) return SHTB200_OK;
    if (!in_dev || !out_dev) return fail(SHTB200_EINVAL, "null pointer");
    return launch_irfft_modes(reinterpret_cast<const float2 *>(in_dev), out_dev, nrows, nlon, nmodes, mode_pieces, grid_pieces, (cudaStream_t)stream);
}

int shtb200_irfft_modes(const void *in_dev, float *out_dev, long long nrows, int nlon, int nmodes, void *stream) {
    if (nrows < 0 || nlon < 2 || nmodes < 1) return fail(SHTB200_EINVAL, "bad irfft shape");
    if (nrows == 0) return SHTB200_OK;
    if (!in_dev || !out_dev) return fail(SHTB200_EINVAL, "null pointer");
    return launch_irfft_modes(reinterpret_cast<const float2 *>(in_dev), out_dev, nrows, nlon, nmodes, 1, 1, (cudaStream_t)stream);
}

size_t shtb200_legendre_workspace_bytes(const shtb200_plan *pl, int nfields, int mloc) {
    if (!pl || nfields <= 0 || mloc <= 0) return 0;
    // sized for the worst first order (the plan's first order holds the longest groups)
    return ws_layout(*pl, nfields, pl->m_base, std::min(mloc, pl->mmax)).total();
}

int shtb200_legendre(shtb200_plan *pl, const void *in_dev, void *out_dev, int nfields, int m0, int mloc, void *workspace_dev, size_t workspace_bytes, void *stream) {
    return shtb200_legendre_pieces(pl, in_dev, out_dev, nfields, m0, mloc, 1, 1, workspace_dev, workspace_bytes, stream);
}

int shtb200_legendre_pieces(shtb200_plan *pl, const void *in_dev, void *out_dev, int nfields, int m0, int mloc, int in_pieces, int out_pieces, void *workspace_dev,
                            size_t workspace_bytes, void *stream) {
    if (!pl) return fail(SHTB200_EINVAL, "plan is null");
    {
        const int rows_in = pl->analysis ? pl->nlat : pl->lmax, rows_out = pl->analysis ? pl->lmax : pl->nlat;
        if (in_pieces < 1 || out_pieces < 1 || in_pieces > rows_in || out_pieces > rows_out || in_pieces > 64 || out_pieces > 64)
            return fail(SHTB200_EINVAL, "bad piece counts: between 1 and min(64, length of the row axis)");
    }
    if (nfields < 0 || mloc < 0 || m0 < pl->m_base || m0 + mloc > pl->m_base + pl->mmax) return fail(SHTB200_EINVAL, "bad (nfields, m0, mloc): the orders must lie inside the plan");
    pl->last_launches = 0;
    if (nfields == 0 || mloc == 0) return SHTB200_OK;
    if (!in_dev || !out_dev) return fail(SHTB200_EINVAL, "null pointer");
    DeviceGuard guard(pl->device);
    if (!guard.ok) return fail(SHTB200_ECUDA, "cudaSetDevice failed");
    cudaStream_t st = (cudaStream_t)stream;
    WsLayout w = ws_layout(*pl, nfields, m0, mloc);
    if (workspace_bytes < w.total() || !workspace_dev) return fail(SHTB200_EWORKSPACE, "workspace too small: need " + std::to_string(w.total()) + " bytes");
    if (((uintptr_t)workspace_dev & 255) != 0) return fail(SHTB200_EINVAL, "workspace must be 256-byte aligned");
    int rc;
    if (pl->analysis) {
        float *X = reinterpret_cast<float *>(workspace_dev);
        float *Z = reinterpret_cast<float *>(reinterpret_cast<char *>(workspace_dev) + align256(w.op_bytes));
        if ((rc = launch_fold_modes(*pl, reinterpret_cast<const float2 *>(in_dev), X, nfields, m0, mloc, in_pieces, st))) return rc;
        {
            GemmParams gp = gemm_params(*pl, nfields, m0, mloc, X, Z);
            if ((rc = run_gemm(*pl, gp, st))) return rc;
            if ((rc = launch_unpack_coeffs(*pl, Z, reinterpret_cast<float2 *>(out_dev), nfields, m0, mloc, out_pieces, st))) return rc;
        }
        pl->last_launches += 2;
    } else {
        float *Ct = reinterpret_cast<float *>(workspace_dev);
        float *Y = reinterpret_cast<float *>(reinterpret_cast<char *>(workspace_dev) + align256(w.op_bytes));
        if ((rc = launch_pack_coeffs(*pl, reinterpret_cast<const float2 *>(in_dev), Ct, nfields, m0, mloc, in_pieces, st))) return rc;
        if ((rc = clear_empty_groups(*pl, Y, (pl->vector ? 4 : 2) * nfields, m0, mloc, st))) return rc;
        GemmParams gp = gemm_params(*pl, nfields, m0, mloc, Ct, Y);
        if ((rc = run_gemm(*pl, gp, st))) return rc;
        if ((rc = launch_unfold_modes(*pl, Y, reinterpret_cast<float2 *>(out_dev), nfields, m0, mloc, out_pieces, st))) return rc;
        pl->last_launches += 2;
    }
    return SHTB200_OK;
}

}  // extern "C"
