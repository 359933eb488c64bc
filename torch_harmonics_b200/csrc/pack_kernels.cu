// Repacking kernels around the Legendre contraction.
//
//  * pack_table_*   : once per plan, dense reference-layout Legendre table -> triangular (l >= m),
//                     parity-split, equator-folded operand of the contraction.
//  * pack_coeffs    : synthesis, per call: coefficients (field, l, m) -> order-major operand with the
//                     degree index contiguous (replaces the transpose + real/imag split copies of
//                     torch_harmonics/sht.py:326-328 and :630-633).
//  * fold / unfold  : distributed stages: plain complex (field, k, m) <-> folded order-major operand.

#include <algorithm>
#include <string>

#include "common.cuh"

namespace shtb200 {

namespace {

struct TableView {
    const float *t;
    int mmax, lmax, nlat;
    int mkl;    // 0: (.., m, l, k)   1: (.., m, k, l)
    int mbase;  // order of the table's first row block (the table holds orders mbase .. mbase + mmax - 1)
    // m: index into the table (order minus mbase)
    __device__ float at(int seg, int m, int l, int k) const {
        size_t base = (size_t)seg * mmax * lmax * nlat;
        return mkl ? t[base + ((size_t)m * nlat + k) * lmax + l] : t[base + ((size_t)m * lmax + l) * nlat + k];
    }
};

// One CTA per order m, one warp per degree l at a time: the degree's largest magnitude over the northern latitudes, then
// the first latitude that reaches rel times it; the minimum over the degrees of each parity is the group's answer.
__global__ void polar_extent_kernel(TableView tv, int Kh, float rel, int *first_row) {
    const int m = blockIdx.x;  // index inside the plan's window of orders
    __shared__ int s_first[2];
    if (threadIdx.x < 2) s_first[threadIdx.x] = Kh;
    __syncthreads();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = blockDim.x >> 5;
    for (int l = m + tv.mbase + warp; l < tv.lmax; l += nwarps) {
        float mx = 0.f;
        for (int k = lane; k < Kh; k += 32) mx = fmaxf(mx, fabsf(tv.at(0, m, l, k)));
        for (int o = 16; o; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
        int first = Kh;
        if (mx > 0.f)
            for (int k = lane; k < Kh && first == Kh; k += 32)
                if (fabsf(tv.at(0, m, l, k)) >= rel * mx) first = k;
        for (int o = 16; o; o >>= 1) first = min(first, __shfl_xor_sync(0xffffffffu, first, o));
        if (lane == 0) atomicMin(&s_first[(l - m - tv.mbase) & 1], first);
    }
    __syncthreads();
    if (threadIdx.x < 2) first_row[2 * m + threadIdx.x] = s_first[threadIdx.x];
}

// rows = degrees, contraction index = folded latitude (row-packed): A[a0[g] + r][seg * Kh + k'], zero beyond
__global__ void pack_table_rows_kernel(TableView tv, float *A, const long long *a0, const int *grows, int ngroups, int ncomp, int Kh, int pitch, int negate_seg1) {
    const int g = blockIdx.y;
    const int m = g >> 1, p = g & 1;
    const int rows = grows[g];
    const long long total = (long long)rows * pitch;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
        const int r = (int)(i / pitch), c = (int)(i - (long long)r * pitch);
        const int seg = c / Kh, k = c - seg * Kh;
        const int l = m + tv.mbase + p + 2 * r;
        // scalar and the m/sin(theta) table share parity p with the rows; the d/dtheta table (seg 0 of a
        // vector plan) has the opposite parity but is addressed the same way: the fold is chosen by the FFT kernel
        float v = 0.f;
        if (seg < ncomp) v = tv.at(ncomp == 2 ? seg : 0, m, l, k);
        if (negate_seg1 && seg == 1) v = -v;
        A[(a0[g] + r) * pitch + c] = v;
    }
}

// rows = folded latitudes, contraction index = degree (block-packed): A[a0[g] + kb * Kh + k'][kk]
// scalar: one segment, degrees of parity p.  vector: segment 0 = d/dtheta table with degrees of parity 1 - p,
// segment 1 = m/sin(theta) table with degrees of parity p.
__global__ void pack_table_blocks_kernel(TableView tv, float *A, const long long *a0, const int *gkb, const int *gkb0, int ngroups, int ncomp, int Kh,
                                         int lmax, int negate_seg1) {
    const int g = blockIdx.y;
    const int m = g >> 1, p = g & 1;
    const int nkb = gkb[g];
    const int nkb0 = gkb0[g];  // slabs of segment 0 (0 for scalar)
    const long long total = (long long)nkb * Kh * kBK;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
        const int kk = (int)(i % kBK);
        const long long t = i / kBK;
        const int k = (int)(t % Kh);
        const int kb = (int)(t / Kh);
        int seg, r, par;
        if (ncomp == 2 && kb < nkb0) { seg = 0; r = kb * kBK + kk; par = 1 - p; }
        else { seg = ncomp == 2 ? 1 : 0; r = (kb - nkb0) * kBK + kk; par = p; }
        const int l = m + tv.mbase + par + 2 * r;
        float v = 0.f;
        if (l < lmax) v = tv.at(seg, m, l, k);
        if (negate_seg1 && seg == 1) v = -v;
        A[(a0[g] + (long long)kb * Kh + k) * kBK + kk] = v;
    }
}

// Ct[((b0[g] - b0[2 m0]) + kb) * ncols + col][kk]
__global__ void pack_coeffs_kernel(const float2 *__restrict__ c, float *__restrict__ Ct, const long long *b0, const int *gkb, const int *gkb0, int ncols,
                                   int lmax, int mloc, int m0, int mbase, int vector, RowPieces rp) {
    const int gl = blockIdx.y;             // group inside the call's orders
    const int m = m0 + (gl >> 1), p = gl & 1;
    const int g = gl + 2 * (m0 - mbase);   // group inside the plan
    const int nkb = gkb[g], nkb0 = gkb0[g];
    const long long base = (b0[g] - b0[2 * (m0 - mbase)]) * ncols;
    const long long total = (long long)nkb * ncols * kBK;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
        const int kk = (int)(i % kBK);
        const long long t = i / kBK;
        const int col = (int)(t % ncols);
        const int kb = (int)(t / ncols);
        float v = 0.f;
        if (!vector) {
            const int l = m + p + 2 * (kb * kBK + kk);
            if (l < lmax) {
                float2 z = c[piece_row(rp, col >> 1, lmax, l) * mloc + (m - m0)];
                v = (col & 1) ? z.y : z.x;
            }
        } else {
            const int pair = col >> 2, cc = col & 3;
            const bool s0 = kb < nkb0;
            const int l = s0 ? m + (1 - p) + 2 * (kb * kBK + kk) : m + p + 2 * ((kb - nkb0) * kBK + kk);
            if (l < lmax) {
                // which component / part / sign feeds (column cc, segment): torch_harmonics/sht.py:638-643
                int comp, im;
                float sg;
                if (s0) {  // d/dtheta table
                    comp = (cc < 2) ? 0 : 1; im = cc & 1; sg = (cc < 2) ? 1.f : -1.f;
                } else {   // m / sin(theta) table
                    comp = (cc < 2) ? 1 : 0; im = 1 - (cc & 1); sg = (cc == 0 || cc == 2) ? -1.f : 1.f;
                }
                float2 z = c[piece_row(rp, pair * 2 + comp, lmax, l) * mloc + (m - m0)];
                v = sg * (im ? z.y : z.x);
            }
        }
        Ct[(base + (long long)kb * ncols + col) * kBK + kk] = v;
    }
}

// Scalar fast path, both directions: tiled transpose between the coefficient array c[field][l][mi] (order index mi
// contiguous, order m = m0 + mi) and the degree-slab layout S[(slab0[g] + r / 32) * ncols + 2 field + re/im][r % 32] with
// g = 2 m + p and r = (l - m - p) / 2.
//
// A CTA takes 32 orders x ONE slab index sb (32 consecutive r of both parities of each order) of one field.  On the
// slab side that is, per (order, parity), two adjacent 128-byte rows (re, im) moved as float4 per thread; in the
// coefficient array it is the band 64 sb <= l - m < 64 sb + 64, i.e. 95 rows l of which every one is touched as one
// contiguous run of up to 32 complex values (8-byte accesses, a warp per row).  The tile passes through shared memory
// as T[l - lbase][mi ^ swz(l - lbase)] (float2); the column swizzle makes the strided scalar accesses of the slab side
// hit 32 different banks.
//
// TO_SLABS = false additionally writes the exact zeros of the l < m triangle: the part next to the diagonal from the
// sb = 0 tiles, the full 32-order row segments above it from extra tiles (blockIdx.y >= nsb).
// TO_SLABS = true writes the zero padding of the last slab of every group (degrees l >= lmax read as zero).
constexpr int kTileRows = 96;
__device__ __forceinline__ int tile_swz(int ll) { return 2 * ((ll >> 3) & 7) + (ll & 1); }

template <bool TO_SLABS>
__global__ void __launch_bounds__(256) coeff_slab_transpose_kernel(float2 *__restrict__ c, float *__restrict__ S, const long long *__restrict__ slab0,
                                                                   const int *__restrict__ gkb, int ncols, int lmax, int mloc, int m0, int nsb, int mbase, RowPieces rp) {
    __shared__ float2 T[kTileRows][32];
    const int mb0 = blockIdx.x * 32, f = blockIdx.z;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int mi_l = mb0 + lane;  // order index of this lane on the coefficient side

    if ((int)blockIdx.y >= nsb) {
        // rows entirely above the diagonal for all 32 orders: l < m0 + mb0
        if (TO_SLABS) return;
        const int t = blockIdx.y - nsb;
        const int hi = m0 + mb0 - 64 * t, lo = max(hi - 64, 0);
        for (int l = lo + warp; l < min(hi, lmax); l += 8)
            if (mi_l < mloc) c[piece_row(rp, f, lmax, l) * mloc + mi_l] = make_float2(0.f, 0.f);
        return;
    }
    const int sb = blockIdx.y;
    // the first order of the tile has the longest groups: nothing to do beyond them (except the zeros next to the diagonal)
    if (sb > 0 && sb >= gkb[2 * (m0 - mbase + mb0)]) return;
    const int lbase = m0 + mb0 + 64 * sb;  // degree of tile row 0

    if (TO_SLABS) {
        // all twelve loads of a thread are in flight before the first store
        float2 v[kTileRows / 8];
        const int d0 = warp - lane, lrem = lmax - lbase - warp;  // d = l - m - 64 sb; rows left below lmax (row ll = warp, then 8 further per step)
        const bool colok = mi_l < mloc;
#pragma unroll
        for (int it = 0; it < kTileRows / 8; ++it) {
            const int d = d0 + 8 * it;
            v[it] = make_float2(0.f, 0.f);
            if (colok && d >= 0 && d < 64 && 8 * it < lrem) v[it] = __ldg(c + piece_row(rp, f, lmax, lbase + warp + 8 * it) * mloc + mi_l);
        }
#pragma unroll
        for (int it = 0; it < kTileRows / 8; ++it) {
            const int ll = warp + 8 * it;
            T[ll][lane ^ tile_swz(ll)] = v[it];
        }
        __syncthreads();
    }
    // slab side: a warp moves both parities of one order per step: lane = (parity, re/im, quad of r)
    {
        const int q = lane & 7, ri = (lane >> 3) & 1, p = lane >> 4;
        float4 x[4];
        float *srow[4];
        bool have[4];
#pragma unroll
        for (int it = 0; it < 4; ++it) {
            const int ml = warp + 8 * it, mi = mb0 + ml;
            have[it] = false;
            srow[it] = S;
            if (mi < mloc) {
                const int g = 2 * (m0 - mbase + mi) + p;  // group inside the plan
                have[it] = sb < gkb[g];
                srow[it] = S + ((size_t)(slab0[g] - slab0[2 * (m0 - mbase)] + sb) * ncols + 2 * f + ri) * kBK + 4 * q;
            }
        }
        if (!TO_SLABS) {
#pragma unroll
            for (int it = 0; it < 4; ++it) {
                x[it] = make_float4(0.f, 0.f, 0.f, 0.f);
                if (have[it]) x[it] = __ldg(reinterpret_cast<const float4 *>(srow[it]));
            }
        }
#pragma unroll
        for (int it = 0; it < 4; ++it) {
            const int ml = warp + 8 * it;
            const int ll0 = ml + p + 8 * q;  // tile row of the first of this thread's four degrees (rows ll0, +2, +4, +6)
            if (TO_SLABS) {
                if (have[it]) {
                    float v[4];
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        const int ll = ll0 + 2 * i;
                        v[i] = reinterpret_cast<const float *>(&T[ll][ml ^ tile_swz(ll)])[ri];
                    }
                    *reinterpret_cast<float4 *>(srow[it]) = make_float4(v[0], v[1], v[2], v[3]);
                }
            } else if (mb0 + ml < mloc) {
                const float v[4] = {x[it].x, x[it].y, x[it].z, x[it].w};
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const int ll = ll0 + 2 * i;
                    reinterpret_cast<float *>(&T[ll][ml ^ tile_swz(ll)])[ri] = v[i];
                }
            }
        }
    }
    if (!TO_SLABS) {
        __syncthreads();
        const int d0 = warp - lane, lrem = lmax - lbase - warp;
        if (mi_l < mloc) {
#pragma unroll
            for (int it = 0; it < kTileRows / 8; ++it) {
                const int ll = warp + 8 * it, d = d0 + 8 * it;
                if (8 * it >= lrem) break;
                float2 *crow = c + piece_row(rp, f, lmax, lbase + ll) * mloc + mi_l;
                if (d >= 0 && d < 64) *crow = T[ll][lane ^ tile_swz(ll)];
                else if (d < 0 && sb == 0) *crow = make_float2(0.f, 0.f);  // l < m
            }
        }
    }
}

// Vector synthesis: the same tiled transpose from c[(pair, component)][l][mi] into the two-segment slabs the vector
// contraction reads, Ct[(b0[g] + kb) * ncols + 4 pair + cc][kk].  For group g = 2 m + p the first kb0[g] slabs (segment 0,
// contracted with the d/dtheta table) hold the degrees of parity 1 - p, the others (segment 1, m / sin(theta) table) the
// degrees of parity p.  A degree l = m + pi + 2 r of component `comp` therefore lands in
//     segment 0 of group 2 m + (1 - pi):  columns 2 comp + (re, im),            sign - for the phi component,
//     segment 1 of group 2 m + pi:        columns 2 (1 - comp) + (im, re),      sign - for the imaginary part
// (component / part / sign pattern of torch_harmonics/sht.py:638-643).  One CTA: 32 orders x one slab index x one component field.
__global__ void __launch_bounds__(256) coeff_slab_transpose_vec_kernel(const float2 *__restrict__ c, float *__restrict__ S, const long long *__restrict__ b0,
                                                                       const int *__restrict__ gkb, const int *__restrict__ gkb0, int ncols, int lmax, int mloc,
                                                                       int m0, int mbase, RowPieces rp) {
    __shared__ float2 T[kTileRows][32];
    const int mb0 = blockIdx.x * 32, sb = blockIdx.y, cf = blockIdx.z;  // cf = 2 pair + component
    const int pair = cf >> 1, comp = cf & 1;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int mi_l = mb0 + lane;
    const int lbase = m0 + mb0 + 64 * sb;
    if (lbase >= lmax) return;  // no degree of this band exists for any order of the tile
    {
        float2 v[kTileRows / 8];
        const int d0 = warp - lane, lrem = lmax - lbase - warp;
        const bool colok = mi_l < mloc;
#pragma unroll
        for (int it = 0; it < kTileRows / 8; ++it) {
            const int d = d0 + 8 * it;
            v[it] = make_float2(0.f, 0.f);
            if (colok && d >= 0 && d < 64 && 8 * it < lrem) v[it] = __ldg(c + piece_row(rp, cf, lmax, lbase + warp + 8 * it) * mloc + mi_l);
        }
#pragma unroll
        for (int it = 0; it < kTileRows / 8; ++it) {
            const int ll = warp + 8 * it;
            T[ll][lane ^ tile_swz(ll)] = v[it];
        }
        __syncthreads();
    }
    // lane = (parity pi of l - m, re / im, quad of r): four consecutive r per store, two destinations
    const int q = lane & 7, ri = (lane >> 3) & 1, pi = lane >> 4;
    const float sa = comp ? -1.f : 1.f, sbn = ri ? -1.f : 1.f;
#pragma unroll
    for (int it = 0; it < 4; ++it) {
        const int ml = warp + 8 * it, mi = mb0 + ml;
        if (mi >= mloc) continue;
        const int gm = 2 * (m0 - mbase + mi);  // group of parity 0 of this order inside the plan
        const int ga = gm + (1 - pi), gb = gm + pi;
        float v[4];
        const int ll0 = ml + pi + 8 * q;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int ll = ll0 + 2 * i;
            v[i] = reinterpret_cast<const float *>(&T[ll][ml ^ tile_swz(ll)])[ri];
        }
        const long long base = b0[2 * (m0 - mbase)];
        if (sb < gkb0[ga])  // segment 0 of group ga
            *reinterpret_cast<float4 *>(S + ((size_t)(b0[ga] - base + sb) * ncols + 4 * pair + 2 * comp + ri) * kBK + 4 * q) = make_float4(sa * v[0], sa * v[1], sa * v[2], sa * v[3]);
        if (sb < gkb[gb] - gkb0[gb])  // segment 1 of group gb
            *reinterpret_cast<float4 *>(S + ((size_t)(b0[gb] - base + gkb0[gb] + sb) * ncols + 4 * pair + 2 * (1 - comp) + (1 - ri)) * kBK + 4 * q) =
                make_float4(sbn * v[0], sbn * v[1], sbn * v[2], sbn * v[3]);
    }
}

// Xc (field, k, mloc) complex -> X[blocked_row(2 mi + p, k')][2 f + ri] (row pitch ncp); rows k' >= Kh of the last
// 32-row block are written as zeros.  The input is contiguous along the orders, the output along the fields: a CTA moves
// a 32 (orders) x 32 (fields) tile of one folded latitude through shared memory, so that both sides see 256-byte runs.
__global__ void __launch_bounds__(256) fold_modes_kernel(const float2 *__restrict__ Xc, float *__restrict__ X, int nfields, int nlat, int Kh, int ncp, int mloc,
                                                         RowPieces rp) {
    __shared__ float2 E[32][33], O[32][33];
    const int mi0 = blockIdx.x * 32, k = blockIdx.y, f0 = blockIdx.z * 32;
    const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
    if (k < Kh) {
        const int ks = nlat - 1 - k;
        const int mi = mi0 + tx;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int f = f0 + ty + 8 * i;
            float2 e = make_float2(0.f, 0.f), o = e;
            if (f < nfields && mi < mloc) {
                const float2 a = __ldg(Xc + piece_row(rp, f, nlat, k) * mloc + mi);
                e = a;
                if (ks != k) {
                    const float2 b = __ldg(Xc + piece_row(rp, f, nlat, ks) * mloc + mi);
                    e = make_float2(a.x + b.x, a.y + b.y);
                    o = make_float2(a.x - b.x, a.y - b.y);
                }
            }
            E[ty + 8 * i][tx] = e;
            O[ty + 8 * i][tx] = o;
        }
    }
    __syncthreads();
    const int f = f0 + tx;
    if (f >= nfields) return;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int mi = mi0 + ty + 8 * i;
        if (mi >= mloc) continue;
        const float2 e = k < Kh ? E[tx][ty + 8 * i] : make_float2(0.f, 0.f), o = k < Kh ? O[tx][ty + 8 * i] : make_float2(0.f, 0.f);
        *reinterpret_cast<float2 *>(X + (size_t)blocked_row(2 * mi, k, 2 * mloc) * ncp + 2 * f) = e;
        *reinterpret_cast<float2 *>(X + (size_t)blocked_row(2 * mi + 1, k, 2 * mloc) * ncp + 2 * f) = o;
    }
}

// Vector analysis: Xc (pair, component, k, mloc) complex -> the two-segment operand the vector contraction reads
// (the layout fft_analysis_kernel<.., 2, ..> emits): columns 4 f .. 4 f + 3 feed (s_re, s_im, t_re, t_im); rows
// k' < Kh contract against the d/dtheta table and carry the fold of parity 1 - p, rows Kh + k' against the
// m/sin(theta) table with the fold of parity p; signs as in torch_harmonics/sht.py:488-493.
__global__ void fold_modes_vec_kernel(const float2 *__restrict__ Xc, float *__restrict__ X, int npairs, int nlat, int Kh, int ncp, int mloc, RowPieces rp) {
    const int Ka = 2 * Kh, Kr = (Ka + kBK - 1) / kBK * kBK;
    const int ngroups = 2 * mloc;
    const long long total = (long long)mloc * (Kh + (Kr - Ka)) * npairs;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
        const int f = (int)(i % npairs);
        const long long t = i / npairs;
        const int k = (int)(t % (Kh + (Kr - Ka)));
        const int mi = (int)(t / (Kh + (Kr - Ka)));
        if (k >= Kh) {  // rows that pad the contraction length to a multiple of 32
            const int kk = Ka + (k - Kh);
            for (int p = 0; p < 2; ++p) *reinterpret_cast<float4 *>(X + (size_t)blocked_row(2 * mi + p, kk, ngroups) * ncp + 4 * f) = make_float4(0.f, 0.f, 0.f, 0.f);
            continue;
        }
        const int ks = nlat - 1 - k;
        float2 e[2], o[2];
        for (int comp = 0; comp < 2; ++comp) {
            const float2 a = Xc[piece_row(rp, 2 * f + comp, nlat, k) * mloc + mi];
            e[comp] = a;
            o[comp] = make_float2(0.f, 0.f);
            if (ks != k) {
                const float2 b = Xc[piece_row(rp, 2 * f + comp, nlat, ks) * mloc + mi];
                e[comp] = make_float2(a.x + b.x, a.y + b.y);
                o[comp] = make_float2(a.x - b.x, a.y - b.y);
            }
        }
        for (int p = 0; p < 2; ++p) {
            const float2 *fa = p ? e : o, *fb = p ? o : e;
            *reinterpret_cast<float4 *>(X + (size_t)blocked_row(2 * mi + p, k, ngroups) * ncp + 4 * f) = make_float4(fa[0].x, fa[0].y, -fa[1].x, -fa[1].y);
            *reinterpret_cast<float4 *>(X + (size_t)blocked_row(2 * mi + p, Kh + k, ngroups) * ncp + 4 * f) = make_float4(-fb[1].y, fb[1].x, -fb[0].y, fb[0].x);
        }
    }
}

// Y[y_off(2 mi + p, k', 2 f + ri)] -> Xc (field, k, mloc) complex, the same tiling the other way round
// (rows above krow0[2 (m0 + mi) + p] were not produced by the contraction: they count as zeros; m0 here = first order of
// the call relative to the plan's first order)
__global__ void __launch_bounds__(256) unfold_modes_kernel(const float *__restrict__ Y, float2 *__restrict__ Xc, int nfields, int nlat, int Kh, int ncp, int mloc,
                                                           const int *__restrict__ krow0, int m0, RowPieces rp) {
    __shared__ float2 E[32][33], O[32][33];
    const int mi0 = blockIdx.x * 32, k = blockIdx.y, f0 = blockIdx.z * 32;
    const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
    {
        const int f = f0 + tx;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int mi = mi0 + ty + 8 * i;
            float2 e = make_float2(0.f, 0.f), o = e;
            if (f < nfields && mi < mloc) {
                if (k >= krow0[2 * (m0 + mi)]) e = __ldg(reinterpret_cast<const float2 *>(Y + y_off(2 * mi, k, 2 * f, 2 * mloc, ncp)));
                if (k >= krow0[2 * (m0 + mi) + 1]) o = __ldg(reinterpret_cast<const float2 *>(Y + y_off(2 * mi + 1, k, 2 * f, 2 * mloc, ncp)));
            }
            E[ty + 8 * i][tx] = e;
            O[ty + 8 * i][tx] = o;
        }
    }
    __syncthreads();
    const int mi = mi0 + tx;
    if (mi >= mloc) return;
    const int ks = nlat - 1 - k;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int f = f0 + ty + 8 * i;
        if (f >= nfields) continue;
        const float2 e = E[tx][ty + 8 * i], o = O[tx][ty + 8 * i];
        Xc[piece_row(rp, f, nlat, k) * mloc + mi] = make_float2(e.x + o.x, e.y + o.y);
        if (ks != k) Xc[piece_row(rp, f, nlat, ks) * mloc + mi] = make_float2(e.x - o.x, e.y - o.y);
    }
}

}  // namespace

static int grid_x_for(long long total) {
    long long b = (total + 255) / 256;
    if (b < 1) b = 1;
    if (b > 4096) b = 4096;
    return (int)b;
}

int launch_pack_table(Plan &pl, const float *table, cudaStream_t st) {
    const int ngroups = 2 * pl.mmax;
    TableView tv{table, pl.mmax, pl.lmax, pl.nlat, 0, pl.m_base};
    // dense layout handed over by the caller: (.., m, k, l) for the tables of the inverse modules
    tv.mkl = (pl.kind == SHTB200_ISHT || pl.kind == SHTB200_ISHT_ADJOINT || pl.kind == SHTB200_IVSHT || pl.kind == SHTB200_IVSHT_ADJOINT) ? 1 : 0;
    dim3 grid(64, ngroups);
    if (pl.analysis) {
        pack_table_rows_kernel<<<grid, 256, 0, st>>>(tv, pl.d_table, pl.d_ga0, pl.d_grows, ngroups, pl.ncomp, pl.Kh, (int)pl.a_pitch, pl.negate_seg1);
    } else {
        pack_table_blocks_kernel<<<grid, 256, 0, st>>>(tv, pl.d_table, pl.d_ga0, pl.d_gkb, pl.d_gkb0, ngroups, pl.ncomp, pl.Kh, pl.lmax, pl.negate_seg1);
    }
    SHT_CUDA_CHECK(cudaGetLastError());
    SHT_CUDA_CHECK(cudaStreamSynchronize(st));
    return SHTB200_OK;
}

int launch_polar_extent(const Plan &pl, const float *table, float rel, std::vector<int> *first_row) {
    const int ngroups = 2 * pl.mmax;
    first_row->assign(ngroups, 0);
    if (pl.mmax == 0) return SHTB200_OK;
    TableView tv{table, pl.mmax, pl.lmax, pl.nlat, 0, pl.m_base};
    tv.mkl = (pl.kind == SHTB200_ISHT || pl.kind == SHTB200_ISHT_ADJOINT || pl.kind == SHTB200_IVSHT || pl.kind == SHTB200_IVSHT_ADJOINT) ? 1 : 0;
    int *d = nullptr;
    SHT_CUDA_CHECK(cudaMalloc(&d, sizeof(int) * ngroups));
    polar_extent_kernel<<<pl.mmax, 256>>>(tv, pl.Kh, rel, d);
    cudaError_t e = cudaGetLastError();
    if (e == cudaSuccess) e = cudaMemcpy(first_row->data(), d, sizeof(int) * ngroups, cudaMemcpyDeviceToHost);
    cudaFree(d);
    if (e != cudaSuccess) return fail(SHTB200_ECUDA, std::string("polar extent: ") + cudaGetErrorString(e));
    return SHTB200_OK;
}

// `pieces` (all four launchers): the (field, row, order) tensor is piece-major along its row axis (see RowPieces); 1 = plain
int launch_pack_coeffs(const Plan &pl, const float2 *c, float *Ct, int nfields, int m0, int mloc, int pieces, cudaStream_t st) {
    const int ncols = (pl.vector ? 4 : 2) * nfields;
    if (mloc == 0 || ncols == 0) return SHTB200_OK;
    RowPieces rp;
    rp.P = pieces;
    rp.nF = pl.vector ? 2 * nfields : nfields;
    if (!pl.vector && nfields <= 65535) {
        const int nsb = ceil_div(pl.Lh, kBK);  // slabs of the longest group
        dim3 grid(ceil_div(mloc, 32), nsb, nfields);
        coeff_slab_transpose_kernel<true><<<grid, 256, 0, st>>>(const_cast<float2 *>(c), Ct, pl.d_gb0, pl.d_gkb, ncols, pl.lmax, mloc, m0, nsb, pl.m_base, rp);
        SHT_CUDA_CHECK(cudaGetLastError());
        return SHTB200_OK;
    }
    if (pl.vector && 2 * nfields <= 65535) {
        dim3 grid(ceil_div(mloc, 32), ceil_div(pl.Lh, kBK), 2 * nfields);
        coeff_slab_transpose_vec_kernel<<<grid, 256, 0, st>>>(c, Ct, pl.d_gb0, pl.d_gkb, pl.d_gkb0, ncols, pl.lmax, mloc, m0, pl.m_base, rp);
        SHT_CUDA_CHECK(cudaGetLastError());
        return SHTB200_OK;
    }
    const long long per_group = (long long)ceil_div(pl.Lh, kBK) * pl.ncomp * ncols * kBK;
    dim3 grid(grid_x_for(per_group), 2 * mloc);
    pack_coeffs_kernel<<<grid, 256, 0, st>>>(c, Ct, pl.d_gb0, pl.d_gkb, pl.d_gkb0, ncols, pl.lmax, mloc, m0, pl.m_base, pl.vector ? 1 : 0, rp);
    SHT_CUDA_CHECK(cudaGetLastError());
    return SHTB200_OK;
}

int launch_unpack_coeffs(const Plan &pl, const float *Z, float2 *c, int nfields, int m0, int mloc, int pieces, cudaStream_t st) {
    if (mloc == 0 || nfields == 0) return SHTB200_OK;
    if (pl.vector) nfields *= 2;  // a vector pair is two output fields (spheroidal, toroidal) side by side
    RowPieces rp;
    rp.P = pieces;
    rp.nF = nfields;
    if (nfields > 65535) return fail(SHTB200_EINVAL, "too many fields in one call (limit 65535)");
    const int nsb = ceil_div(pl.Lh, kBK);
    // extra tile rows for the degrees above the diagonal of the last order block: l < m0 + 32 (blocks - 1)
    const int nzero = ceil_div(std::min(m0 + 32 * (ceil_div(mloc, 32) - 1), pl.lmax), 64);
    dim3 grid(ceil_div(mloc, 32), nsb + nzero, nfields);
    coeff_slab_transpose_kernel<false><<<grid, 256, 0, st>>>(c, const_cast<float *>(Z), pl.d_gb0, pl.d_gkb, 2 * nfields, pl.lmax, mloc, m0, nsb, pl.m_base, rp);
    SHT_CUDA_CHECK(cudaGetLastError());
    return SHTB200_OK;
}

int launch_fold_modes(const Plan &pl, const float2 *Xc, float *X, int nfields, int m0, int mloc, int pieces, cudaStream_t st) {
    (void)m0;
    RowPieces rp;
    rp.P = pieces;
    rp.nF = pl.vector ? 2 * nfields : nfields;
    if (pl.vector) {
        const int pad = (int)(round_up(pl.Ka, kBK) - pl.Ka);
        const long long total = (long long)mloc * nfields * (pl.Kh + pad);
        if (total == 0) return SHTB200_OK;
        fold_modes_vec_kernel<<<grid_x_for(total), 256, 0, st>>>(Xc, X, nfields, pl.nlat, pl.Kh, (int)col_pitch(4 * nfields), mloc, rp);
        SHT_CUDA_CHECK(cudaGetLastError());
        return SHTB200_OK;
    }
    if (mloc == 0 || nfields == 0) return SHTB200_OK;
    if (ceil_div(nfields, 32) > 65535) return fail(SHTB200_EINVAL, "too many fields in one call");
    dim3 grid(ceil_div(mloc, 32), (unsigned)round_up(pl.Kh, kBK), ceil_div(nfields, 32));
    fold_modes_kernel<<<grid, 256, 0, st>>>(Xc, X, nfields, pl.nlat, pl.Kh, (int)col_pitch(2 * nfields), mloc, rp);
    SHT_CUDA_CHECK(cudaGetLastError());
    return SHTB200_OK;
}

int launch_unfold_modes(const Plan &pl, const float *Y, float2 *Xc, int nfields, int m0, int mloc, int pieces, cudaStream_t st) {
    // a vector pair is two complex fields side by side (theta, phi): same kernel on 2 x nfields fields
    const int nf = pl.vector ? 2 * nfields : nfields;
    RowPieces rp;
    rp.P = pieces;
    rp.nF = nf;
    if (nf == 0 || mloc == 0) return SHTB200_OK;
    if (ceil_div(nf, 32) > 65535) return fail(SHTB200_EINVAL, "too many fields in one call");
    dim3 grid(ceil_div(mloc, 32), pl.Kh, ceil_div(nf, 32));
    unfold_modes_kernel<<<grid, 256, 0, st>>>(Y, Xc, nf, pl.nlat, pl.Kh, (int)col_pitch(2 * nf), mloc, pl.d_krow0, m0 - pl.m_base, rp);
    SHT_CUDA_CHECK(cudaGetLastError());
    return SHTB200_OK;
}

}  // namespace shtb200
