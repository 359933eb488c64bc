// Shared declarations of the shtb200 library: plan object, device-side descriptors, launch helpers.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

#include <string>
#include <vector>

#include "../../include/shtb200.h"

namespace shtb200 {

// ------------------------------------------------------------------------------------------------
// error plumbing
// ------------------------------------------------------------------------------------------------
void set_error(const std::string &msg);
int fail(int code, const std::string &msg);

#define SHT_CUDA_CHECK(expr)                                                                              \
    do {                                                                                                  \
        cudaError_t _e = (expr);                                                                          \
        if (_e != cudaSuccess) {                                                                          \
            return ::shtb200::fail(SHTB200_ECUDA, std::string(#expr) + ": " + cudaGetErrorString(_e));    \
        }                                                                                                 \
    } while (0)

// ------------------------------------------------------------------------------------------------
// longitude FFT plan (device view passed by value to the kernels)
// ------------------------------------------------------------------------------------------------
constexpr int kMaxFftStages = 24;

struct FftPlanDev {
    int n;                        // nlon
    int nstages;                  // number of radix passes
    int radix[kMaxFftStages];     // radix of pass s (decimation in frequency order)
    int sublen[kMaxFftStages];    // length L of the sub-transforms pass s splits (L_0 = n, L_{s+1} = L_s / radix_s)
    int twoff[kMaxFftStages];     // offset of pass s's twiddle table inside tw
    int tw_pass_total;            // entries of all per-pass tables together (padded to an even count)
    // Geometry of one transform in shared memory.  Split layout (analysis kernel; re array | im array of floats): the
    // imaginary parts start `io` floats after the real parts, transforms lie `ts` floats apart (ts = 4 mod 32 spreads
    // the transforms of a CTA over the banks), np = 0.  Interleaved layout (synthesis and stage kernels): transforms lie
    // `np` float2 apart, io = ts = 0.
    int io, ts, np;
    int tab_bytes;                // size of the blob [tw | bfly | perm | eorder] that starts at tw (a multiple of 16)
    const float2 *tw;             // per-pass tables: entry (q - 1) * L/R + j of pass s = exp(-2 pi i q j / L_s), from double
    const float2 *tw_full;        // n roots of unity exp(-2 pi i k / n) (generic prime-radix butterflies only)
    const unsigned short *perm;   // perm[k] = slot of output bin k after the in-place DIF passes
    // Thread -> butterfly assignment of each pass, ordered so that the 16 lanes that share a shared-memory wavefront
    // touch 16 different 8-byte bank pairs: entry i of pass s = (first leg's slot) | (twiddle index j) << 16.
    const unsigned *bfly;
    int bfoff[kMaxFftStages];
    int bf_total;
    // Order in which the retained longitudinal orders are emitted / gathered (a permutation of [0, eorder_len)), chosen
    // so that the lanes of one wavefront read different banks of the permuted spectrum; null = natural order.
    const unsigned short *eorder;
    int eorder_len;
};

// ------------------------------------------------------------------------------------------------
// Legendre contraction: one work item = one (order m, parity p) group x one block of table rows.
//
// Operands are addressed generically so that both packings share the kernels:
//   element (row r, contraction index k) of an operand with origin row y0 lives at
//       base[(y0 + (k / BK) * dy + r) * pitch + (k / BK) * dx + k % BK]
//   "row-packed" (dx = BK, dy = 0): plain row-major rows, contraction index contiguous along a row;
//   "block-packed" (dx = 0, dy = rows of a block): one [rows x BK] slab per BK-wide slice of k.
// ------------------------------------------------------------------------------------------------
constexpr int kBK = 32;  // contraction slice width (floats): one 128-byte swizzle row
constexpr int kMaxPolarBlock = 15;  // largest first-live latitude block a group may carry (a 4-bit field in the FFT tables)

struct GemmItem {
    int a_y0;      // first table row of this item
    int a_dy;      // block-packed: rows per k-slab of this group; row-packed: 0
    int b_y0;      // operand origin of this group in units of ncols rows (group index, or first k-slab of the group)
    int b_dy;      // block-packed: 1 (ncols rows per k-slab); row-packed: 0
    int kblocks;   // number of BK-wide slices of the contraction index
    int rows;      // valid table rows in this item (<= kItemRowsMax)
    int m;         // spherical harmonic order
    int p;         // parity of l - m handled by this group (0 / 1)
    int r0;        // index of the item's first row inside its group
    int kfirst;    // contraction slices skipped at the front of this group: slice i of the item is slice kfirst + i of the operands
};
constexpr int kItemRowsMax = 128;  // one 128-row tensor-core tile

// How a finished tile leaves the contraction kernel.
enum EpilogueMode : int {
    EPI_LATROWS = 1,  // synthesis: rows are folded latitudes k'      -> float Y[y_off(group, k', col)] (out_ld = padded column count)
    EPI_SLABS = 2,    // analysis: rows are degrees -> float Z[(slab0[g] + r / 32) * ncols + col][r % 32], the same
                      // degree-slab layout the synthesis contraction reads its coefficients from
};

struct GemmParams {
    const float *A;       // packed Legendre table
    const float *B;       // packed operand (FFT output / packed coefficients)
    long long a_pitch;    // floats per table row
    long long b_pitch;    // floats per operand row
    int a_dx, b_dx;       // see above
    int a_kext, b_kext;   // valid extent of the inner (k) axis of a row (reads beyond it yield 0)
    int b_mn;             // 1: B is column-contiguous, element (col, k) of group u at B[blocked_row(u - b_unit0, k, b_groups) * b_pitch + col]
    int b_krows;          // b_mn: valid contraction indices per group
    int b_groups;         // b_mn: groups held in B
    int ncols;            // columns of the product = 2 * nfields (4 * pairs for vector kinds)
    long long b_unit0;    // operand origin (same units as GemmItem::b_y0) of the first order held in B
    const GemmItem *items;
    int nitems;
    int mode;             // EpilogueMode
    float *out;           // destination
    int lmax, mmax_out;   // degrees; number of orders of the call (mloc)
    int m0;               // first order stored in out (orders outside [m0, m0 + mmax_out) are skipped)
    int m_base;           // first order the plan holds: slab0 is indexed by 2 (m - m_base) + p
    long long out_ld;     // EPI_LATROWS: padded column count of Y
    int out_groups;       // EPI_LATROWS: groups held in Y
    const long long *slab0;  // EPI_SLABS: first slab of every group (device array, 2 * mmax + 1 entries)
    long long slab_unit0;    // EPI_SLABS: slab0 of the first order held in the output
};

// ------------------------------------------------------------------------------------------------
// the plan
// ------------------------------------------------------------------------------------------------
struct Plan {
    int kind = 0, engine = 0, device = 0;
    int sm_count = 0;  // multiprocessors of `device` (grid size of the persistent contraction kernel)
    int nlat = 0, nlon = 0, lmax = 0, mmax = 0;
    // A plan may hold a window of orders only (the spatially distributed transforms contract the orders of one azimuth
    // rank): m_base = first order of the window, mmax = number of orders in it.  Group arrays are indexed by the local
    // group 2 (m - m_base) + p; GemmItem::m and every degree computation use the actual order m.
    int m_base = 0;
    bool window = false;  // created for a window: only the Legendre stage entry point accepts the plan
    int Kh = 0;   // folded latitude count, (nlat + 1) / 2
    int Ka = 0;   // contraction length of the analysis kinds, ncomp * Kh
    int Lh = 0;   // largest number of degrees of one parity, (lmax + 1) / 2
    bool analysis = false;  // grid -> spectral
    bool vector = false;
    int ncomp = 1;          // latitude-axis multiplicity of the contraction (vector: 2 tables side by side)

    // FFT
    FftPlanDev fft{};
    float2 *d_tw = nullptr;
    unsigned short *d_perm = nullptr;
    float *d_mscale = nullptr;  // per-order scale applied in the FFT kernel (2 pi / nlon, adjoint weights ...)
    int zero_imag_edges = 0;    // analysis adjoint: force Im = 0 at m = 0 and Nyquist
    // two-pass FFT kernels (scalar kinds, nlon = R1 * R2 with a built factorisation): their table blob
    bool twopass = false;
    unsigned char *d_tp_blob = nullptr;
    int tp_blob_bytes = 0, tp_mpad = 0;

    // packed table
    float *d_table = nullptr;
    size_t table_floats = 0;
    long long a_pitch = 0;
    int a_dx = 0, a_kext = 0;
    std::vector<int> group_rows;      // rows (degrees) in group g = 2 m + p
    std::vector<long long> group_a0;  // first table row of group g
    std::vector<int> group_kblocks;   // synthesis: BK-slabs of group g
    std::vector<long long> group_b0;  // synthesis: first operand row of group g, per unit column (multiply by ncols)
    long long total_b_slabs = 0;      // synthesis: sum of kblocks over groups

    std::vector<GemmItem> items;      // host copy, longest first
    GemmItem *d_items = nullptr;
    // device copies of the per-group arrays
    long long *d_ga0 = nullptr, *d_gb0 = nullptr;
    int *d_grows = nullptr, *d_gkb = nullptr, *d_gkb0 = nullptr;
    int negate_seg1 = 0;              // vector adjoints: the m/sin(theta) table enters with the opposite sign
    // scalar analysis plans: degree classes of the slabs.  Lane i of slab (g = 2 m + p, rb) holds degree m + p + 64 rb + 2 i,
    // so all slabs with the same l0 = m + p + 64 rb carry the same 32 degrees; class l0 lists them
    // (d_cls_slab[d_cls_off[l0] .. d_cls_off[l0 + 1])).  A kernel that applies per-degree weights loads them once per class.
    int *d_cls_off = nullptr, *d_cls_slab = nullptr;

    // host-call staging
    void *stage_in = nullptr, *stage_out = nullptr, *stage_ws = nullptr;
    size_t stage_in_bytes = 0, stage_out_bytes = 0, stage_ws_bytes = 0;
    // host-buffer entry point: copy streams and per-chunk events of its upload / compute / download pipeline
    cudaStream_t copy_in = nullptr, copy_out = nullptr;
    std::vector<cudaEvent_t> ev_up, ev_done;

    int last_launches = 0;
    // First folded latitude row (a multiple of 32) of each group that the contraction touches: towards the pole the
    // associated Legendre functions of high order vanish faster than fp32 can represent next to the row's largest value
    // (see launch_polar_extent), so analysis never reads the operand rows above it and synthesis never writes them.
    std::vector<int> group_krow0;
    int *d_krow0 = nullptr;
    int *d_err = nullptr;             // device error word raised by kernels whose bounded waits ran out

    // optional per-kernel timing (cudaEvents recorded between the launches of one execute call)
    int profiling = 0;
    cudaEvent_t ev[8] = {};
    int nev = 0;
};

// ------------------------------------------------------------------------------------------------
// kernel launchers (defined in the .cu files)
// ------------------------------------------------------------------------------------------------
// mmax_emit > 0 also builds the emit order for that many retained orders (the SHT kernels); 0 leaves it out
enum { kFftRows = 0, kFftSplit = 1, kFftPacked = 2 };  // shared-memory layout the tables are built for (see FftPlanDev)
// krow0 (2 mmax_emit entries, may be null): first latitude row of every (order, parity) group that the contraction touches
int build_fft_plan(int nlon, int mmax_emit, int layout, const int *krow0, FftPlanDev *out, float2 **d_tw, unsigned short **d_perm);

// analysis: rows of x -> folded, order-major operand X[blocked_row(group, k)][col] (row pitch col_pitch(ncols))
int launch_fft_analysis(const Plan &pl, const float *x, float *X, int nfields, cudaStream_t st);
// synthesis: Y[blocked_row(group, k')][col] -> rows of x
int launch_fft_synthesis(const Plan &pl, const float *Y, float *x, int nfields, cudaStream_t st);
// Process-wide cap on the SMs the persistent kernels size their grids for (shtb200_set_sm_limit; 0 = none): a caller that
// overlaps NCCL collectives with these kernels leaves the collective's CTAs somewhere to run.
int effective_sms(int sm_count);

// balanced split of n into P pieces (the first n % P one longer): the piece that holds index i -> (first index, width)
__host__ __device__ __forceinline__ void piece_of(int i, int n, int P, int *start, int *width) {
    const int q = n / P, rem = n - q * P;
    int s = 0, w = q + (rem > 0 ? 1 : 0);
    for (int j = 1; j < P && i >= s + w; ++j) {
        s += w;
        w = q + (j < rem ? 1 : 0);
    }
    *start = s;
    *width = w;
}

// A (nF, R, mloc) tensor whose row axis travels through an all-to-all in P pieces is stored "piece-major": piece j is its
// own contiguous (nF, width_j, mloc) block, the blocks one after the other.  row index (in units of mloc) of (F, row):
struct RowPieces {
    int P = 1, nF = 0;
};
__device__ __forceinline__ size_t piece_row(const RowPieces rp, int F, int R, int row) {
    if (rp.P == 1) return (size_t)F * R + row;
    int s0, w;
    piece_of(row, R, rp.P, &s0, &w);
    return (size_t)rp.nF * s0 + (size_t)F * w + (row - s0);
}

// register-resident two-pass kernels (fft_twopass.cu); the launchers above pick them when the plan has their tables
bool twopass_supported(int nlon, int *r1, int *r2);
int build_twopass_tables(Plan &pl, const std::vector<float> &mscale);
int launch_fft_analysis_twopass(const Plan &pl, const float *x, float *X, int nfields, cudaStream_t st);
int launch_fft_synthesis_twopass(const Plan &pl, const float *Y, float *x, int nfields, cudaStream_t st);
// the same kernels as plain batched row transforms (stage entry points, no plan)
struct TwoPassRows {
    const unsigned char *blob = nullptr;  // pass twiddles (build_twopass_rows_tables)
    int blob_bytes = 0, sm_count = 0;
    int *d_err = nullptr;  // device error word for bounded waits that ran out
};
int build_twopass_rows_tables(int nlon, unsigned char **d_blob, int *bytes);
bool rows_pieces_supported(int nlon, int nmodes, int grid_pieces, int mode_pieces);
int launch_rows_twopass(const TwoPassRows &tr, bool forward, const void *in, void *out, long long nrows, int nlon, int nmodes, float scale, int grid_pieces,
                        int mode_pieces, cudaStream_t st);
// plain row transforms for the distributed stages
int launch_rfft_modes(const float *in, float2 *out, long long nrows, int nlon, int nmodes, float scale, int grid_pieces, int mode_pieces, cudaStream_t st);
int launch_irfft_modes(const float2 *in, float *out, long long nrows, int nlon, int nmodes, int mode_pieces, int grid_pieces, cudaStream_t st);

int launch_gemm_simt(const GemmParams &gp, cudaStream_t st);
int launch_gemm_tc(const Plan &pl, const GemmParams &gp, cudaStream_t st);
bool gemm_tc_supported(const Plan &pl, const GemmParams &gp);

// table / operand packing
int launch_pack_table(Plan &pl, const float *table, cudaStream_t st);
// first_row[2 m + p] = first folded latitude k' at which any degree l = m + p + 2 r of the dense table reaches `rel` times
// that degree's largest magnitude over all latitudes (Kh if none does)
int launch_polar_extent(const Plan &pl, const float *table, float rel, std::vector<int> *first_row);
// (m0 = first order of the call, an actual order: m_base <= m0, m0 + mloc <= m_base + mmax)
// pieces: the (field, row, order) side is piece-major along its row axis (RowPieces above); 1 = plain
int launch_pack_coeffs(const Plan &pl, const float2 *c, float *Ct, int nfields, int m0, int mloc, int pieces, cudaStream_t st);
int launch_unpack_coeffs(const Plan &pl, const float *Z, float2 *c, int nfields, int m0, int mloc, int pieces, cudaStream_t st);
int launch_fold_modes(const Plan &pl, const float2 *Xc, float *X, int nfields, int m0, int mloc, int pieces, cudaStream_t st);
int launch_unfold_modes(const Plan &pl, const float *Y, float2 *Xc, int nfields, int m0, int mloc, int pieces, cudaStream_t st);  // honours group_krow0

// spectral convolution on the degree slabs, spherical quadrature (spectral_conv.cu)
size_t slab_mix_weight_bytes(int cin, int cout, int ngroups, int lmax);
int launch_slab_mix(const Plan &pl, const float *Zin, float *Zout, const float2 *weight, float2 *wsplit, int batch, int cin, int cout, int ngroups, cudaStream_t st);
int launch_quadrature(const float *x, const float *w, float *out, long long nfields, int nlat, int nlon, cudaStream_t st);

// Row of (group, k) in the column-contiguous operands X and Y: 32-row blocks of k are outermost, then the group,
// then k inside the block.  CTAs of the FFT kernels that run at the same time work on neighbouring k for ALL groups,
// so with this order they fill / read one contiguous region of HBM instead of 2 * mmax far-apart ones, and the
// 32 x columns tile the contraction loads per k-step is one contiguous piece.
__host__ __device__ inline long long blocked_row(long long group, int k, int ngroups) { return (((long long)(k >> 5) * ngroups + group) << 5) + (k & 31); }

// Offset (floats) of element (group, k', column) of the synthesis operand Y, stored in panels of 16 columns (eight
// fields): Y[k'][column / 16][group][column % 16], `ncp` = padded column count (a multiple of 32).  The synthesis FFT
// works on one latitude pair of eight fields at a time and needs, of every group, exactly those 16 columns: with this order
// its whole input is ONE contiguous region of ngroups x 64 bytes.  The contraction's epilogue produces 64-byte pieces
// (16 columns of one latitude row) anyway, which it scatters into the panels.
__host__ __device__ inline size_t y_off(long long group, int k, int col, int ngroups, long long ncp) {
    return ((((size_t)k * (size_t)(ncp >> 4) + (size_t)(col >> 4)) * (size_t)ngroups + (size_t)group) << 4) + (size_t)(col & 15);
}

inline int ceil_div(int a, int b) { return (a + b - 1) / b; }
// Row pitch (floats) of the column-contiguous operands: whole 128-byte lines, so that the 64-byte runs the FFT kernels
// write and read never straddle two lines.
inline long long col_pitch(long long ncols) { return (ncols + 31) / 32 * 32; }
inline long long round_up(long long a, long long b) { return (a + b - 1) / b * b; }

}  // namespace shtb200
