// Longitude transforms of the SHT for nlon = R1 * R2 (1440 = 40 * 36, 720 = 36 * 20, 512 = 32 * 16): register-resident
// two-pass FFT kernels.
//
// A persistent CTA (two per SM) works through (field block, latitude pair) items.  An item = eight fields x one
// pair of rows (k', nlat-1-k'), i.e. eight complex transforms of z = north + i south.  R1 threads carry one transform,
// the eight transforms of an item sit in the eight low lane positions (lane & 7), so that whatever a quarter-warp
// writes to / reads from the contraction operand for one order m is one contiguous 64-byte run of 8 fields.
//
// Analysis, per item:
//   rows -> shared memory as bulk asynchronous copies (issued for item i + 1 while item i is being emitted);
//   pass 1: thread (t, j < R2) reads its R1 strided samples z[j + R2 r] into registers, radix-R1 transform, twiddles
//           w_n^{q j}, result q goes to slot R2 q + j of an exchange area that overlays the rows (every thread has
//           read before any thread writes);
//   pass 2: thread (t, q < R1) reads the R2 contiguous slots of sub-transform q, radix-R2 transform: it now holds the
//           bins q + R1 i in registers.  The mirror bins n - m that separating the two real rows needs sit in the thread
//           that owns q' = R1 - q, which is placed 16 lanes away in the same warp: one shuffle per bin;
//   emit:   even / odd folds of every retained order go straight from registers to X[blocked_row(2 m + p, k')].
// The exchange area is the only shared-memory round trip of a transform (the three-pass kernel makes three, plus one
// for the emit).  Synthesis is the mirror image and ends with bulk copies of the finished rows to global memory.
//
// Replaces torch_harmonics/fft.py:52-68, :71-96 and the scale / transpose / real-imag split passes at
// torch_harmonics/sht.py:171-176 and :337-340 for the grids it supports; other grids and the vector transforms
// take the general mixed-radix kernels.

#include <math.h>

#include <vector>

#include "common.cuh"
#include "fft_butterflies.cuh"
#include "tc_ptx.cuh"

namespace shtb200 {

namespace {

constexpr int kNT = 8;  // transforms per item (fields per CTA)

template <int R1, int R2>
struct TwoPass {
    static constexpr int N = R1 * R2;
    // floats between the transforms of an item.  As rows: real array at 0, imaginary array at N.  As exchange area
    // (float2 units, stride TS / 2): slot(q, j) = R2 q + (j + (q & 1)) mod R2, i.e. the blocks of odd q are rotated by
    // one slot.  TS = 4 mod 32, TS / 2 = 2 mod 16 and that rotation keep the accesses of both passes free of bank
    // conflicts for the lane arrangement described at the kernels (the two q of a half-warp are one even, one odd).
    static constexpr int TS = ((2 * N + 2 - 4 + 31) / 32) * 32 + 4;
    static constexpr int NTW = (R1 - 1) * R2;  // pass twiddles, entry (q - 1) R2 + j = exp(-2 pi i q j / n)
    static constexpr int THREADS = kNT * R1;
    static_assert(R1 % 4 == 0 && R2 <= R1 && R2 % 2 == 0, "thread arrangement");
    static_assert(TS % 4 == 0 && TS / 2 >= N, "row copies need 16-byte aligned targets; the exchange area needs N slots");
};

// sub-transform index q owned in pass 2 by slot s (0..3) of warp w: an even q, an odd q, and their mirrors R1 - q
// 16 lanes further (q = 0 and q = R1 / 2 mirror themselves and share a slot pair)
template <int R1>
__device__ __forceinline__ int q_of(int w, int s) {
    return s == 0 ? 2 * w : s == 1 ? 2 * w + 1 : s == 2 ? (w == 0 ? R1 / 2 : R1 - 2 * w) : R1 - 1 - 2 * w;
}

// CTA-wide wait for phase `parity` of an mbarrier; false (for all threads alike) when it did not complete in about a second
__device__ __forceinline__ bool cta_wait(uint32_t bar, uint32_t parity, int *err, int code) {
    bool ok = ptx::mbar_try_wait(bar, parity) != 0;
    if (!ok) {
        const long long t0 = clock64();
        for (uint32_t it = 1; !ok; ++it) {
            ok = ptx::mbar_try_wait(bar, parity) != 0;
            if (!ok && (it & 63u) == 0u && clock64() - t0 > 2000000000ll) break;
        }
    }
    if (__syncthreads_or(ok ? 0 : 1)) {
        if (threadIdx.x == 0 && err) atomicExch(err, code);
        return false;
    }
    return true;
}

// thread index read through a volatile statement, so that values derived from it are recomputed where they are used
// instead of being kept in registers across the butterflies
__device__ __forceinline__ int tid_now() {
    int x;
    asm volatile("mov.u32 %0, %%tid.x;" : "=r"(x));
    return x;
}

struct TwoPassArgs {
    const float *grid_in;   // analysis: x (nfields, nlat, n)
    float *grid_out;        // synthesis: x
    float *op;              // analysis: X (written); synthesis: Y (read)
    const unsigned char *blob;  // [twiddles float2 x NTW][mscale float x mpad][kfirst u8 x mpad], 16-byte granular
    int blob_bytes, mpad;
    int nlat, Kh, nfields, ncp, mmax, zero_imag_edges;
    int kpad;               // analysis: zero rows appended to the operand (contraction length rounded up to 32)
    int *err;
    // ROWS kernels (plain batched rfft / irfft of `nrows` rows, an item = 16 consecutive rows = 8 transforms of
    // row 2 t + i row (2 t + 1)): spectra (nrows, nmodes) complex, `scale` multiplies the forward spectra
    const float2 *rows_in;
    float2 *rows_out;
    long long nrows;
    int nmodes;
    float scale;
    // ROWS kernels, piece-major buffers (what an all-to-all transpose sends / receives, see distributed/primitives.py):
    // the longitude (grid_pieces) or order (mode_pieces) axis is cut into balanced pieces (the first n % P pieces one longer)
    // and piece j is stored as its own contiguous (nrows, width_j) block, the blocks one after the other.  1 = plain rows.
    int grid_pieces, mode_pieces;
};

// ROWS: transforms of item `it` that have at least one row
__device__ __forceinline__ int rows_nvalid(long long nrows, int it) {
    const long long left = nrows - 16LL * it;
    return left >= 16 ? kNT : (int)((left + 1) >> 1);
}

// item -> (latitude pair, first field): full field blocks first (k' slowest), the ragged last block at the end, so that
// the CTAs' last round is made of the light items
__device__ __forceinline__ void decode_item(int it, int Kh, int nfields, int *kn, int *f0, int *nvalid) {
    const int nfull = nfields / kNT;
    const int nmain = Kh * nfull;
    if (it < nmain) {
        *kn = it / nfull;
        *f0 = (it - *kn * nfull) * kNT;
        *nvalid = kNT;
    } else {
        *kn = it - nmain;
        *f0 = nfull * kNT;
        *nvalid = nfields - *f0;
    }
}

// Register arrays are filled unconditionally (idle lanes read valid but meaningless addresses and only their stores are
// predicated): an array that is initialised under a condition counts as live around the whole item loop, and the two
// passes' arrays would then not share registers.  Thread coordinates are re-derived in every phase for the same reason.
// VEC = 2: the transforms of an item are the (theta, phi) components of four vector fields; a.nfields counts component
// fields (2 per pair).  The operand then has two row segments per group, k' against the d/dtheta table with the fold of
// parity 1 - p and Kh + k' against the m / sin(theta) table with the fold of parity p, and four columns per pair that
// carry the sign pattern of torch_harmonics/sht.py:488-493:
//     rows k'     : ( Re X0,  Im X0, -Re X1, -Im X1)        rows Kh + k' : (-Im X1,  Re X1, -Im X0,  Re X0)
// (X0 = theta component, X1 = phi component): every thread still writes 8-byte pieces of its own transform only.
// ROWS: the same two passes as a plain batched rfft (distributed stage, torch_harmonics/distributed/distributed_sht.py:197):
// the emit writes the two rows' spectra A and B instead of their folds.
template <int R1, int R2, int VEC, bool ROWS>
__global__ void __launch_bounds__(TwoPass<R1, R2>::THREADS, 2) fft_analysis_twopass_kernel(const TwoPassArgs a) {
    using TP = TwoPass<R1, R2>;
    constexpr int N = TP::N, TS = TP::TS, TS2 = TP::TS / 2;
    extern __shared__ __align__(16) float smem_tp[];
    unsigned char *blob_s = reinterpret_cast<unsigned char *>(smem_tp + kNT * TS);
    const uint32_t bar_tab = ptx::smem_u32(blob_s + a.blob_bytes), bar_rows = bar_tab + 8;
    const int nfb = (a.nfields + kNT - 1) / kNT;
    const int nitems = ROWS ? (int)((a.nrows + 15) >> 4) : a.Kh * nfb;

    // rows of the last 32-row block beyond the contraction length: the contraction reads them, they must be zeros
    for (int z = blockIdx.x; z < a.kpad * nfb; z += gridDim.x) {
        const int kk = VEC * a.Kh + z / nfb, f0 = (z % nfb) * kNT, ngroups = 2 * a.mmax;
        for (int i = threadIdx.x; i < ngroups * 4; i += blockDim.x) {
            const int g = i >> 2, c = 2 * f0 + 4 * (i & 3);
            if (c < 2 * a.nfields) *reinterpret_cast<float4 *>(a.op + (size_t)blocked_row(g, kk, ngroups) * a.ncp + c) = make_float4(0.f, 0.f, 0.f, 0.f);
        }
    }
    if ((int)blockIdx.x >= nitems) return;

    auto issue_rows = [&](int it) {  // thread 0: the rows of item `it` (row k' -> real array, its mirror -> imaginary array)
        if (ROWS) {
            const long long r0 = 16LL * it;
            const int nr = (int)min(16LL, a.nrows - r0);
            ptx::mbar_arrive_expect_tx(bar_rows, N * 4u * (uint32_t)nr);
            if (a.grid_pieces == 1) {
                for (int u = 0; u < nr; ++u)
                    ptx::bulk_load(ptx::smem_u32(smem_tp + (u >> 1) * TS + (u & 1) * N), a.grid_in + (size_t)(r0 + u) * N, N * 4u, bar_rows);
            } else {  // a row is one segment in every piece (widths are multiples of 4 floats: checked by the launcher)
                const int q = N / a.grid_pieces, rem = N - q * a.grid_pieces;
                for (int j = 0, s0 = 0; j < a.grid_pieces; ++j) {
                    const int w = q + (j < rem ? 1 : 0);
                    const float *pj = a.grid_in + (size_t)a.nrows * s0 + (size_t)r0 * w;
                    for (int u = 0; u < nr; ++u)
                        ptx::bulk_load(ptx::smem_u32(smem_tp + (u >> 1) * TS + (u & 1) * N + s0), pj + (size_t)u * w, w * 4u, bar_rows);
                    s0 += w;
                }
            }
            return;
        }
        int kn, f0, nvalid;
        decode_item(it, a.Kh, a.nfields, &kn, &f0, &nvalid);
        const int ks = a.nlat - 1 - kn;
        ptx::mbar_arrive_expect_tx(bar_rows, 2u * N * 4u * (uint32_t)nvalid);
        for (int u = 0; u < nvalid; ++u) {
            const float *f = a.grid_in + (size_t)(f0 + u) * a.nlat * N;
            ptx::bulk_load(ptx::smem_u32(smem_tp + u * TS), f + (size_t)kn * N, N * 4u, bar_rows);
            ptx::bulk_load(ptx::smem_u32(smem_tp + u * TS + N), f + (size_t)ks * N, N * 4u, bar_rows);
        }
    };
    if (threadIdx.x == 0) {
        ptx::mbar_init(bar_tab, 1);
        ptx::mbar_init(bar_rows, 1);
        ptx::fence_barrier_init();
        ptx::mbar_arrive_expect_tx(bar_tab, (uint32_t)a.blob_bytes);
        ptx::bulk_load(ptx::smem_u32(blob_s), a.blob, (uint32_t)a.blob_bytes, bar_tab);
        issue_rows(blockIdx.x);
    }
    __syncthreads();  // barrier initialisation visible to everybody who polls
    if (!cta_wait(bar_tab, 0, a.err, 0x0F7F0011)) return;

    uint32_t phase = 0;
    for (int it = blockIdx.x; it < nitems; it += gridDim.x) {
        if (!cta_wait(bar_rows, phase, a.err, 0x0F7F0012)) return;
        phase ^= 1u;
        if (ROWS && 16LL * it + 16 > a.nrows && (a.nrows & 1)) {  // odd row count: the last transform's second row is zeros
            float *im = smem_tp + (rows_nvalid(a.nrows, it) - 1) * TS + N;
            for (int i = threadIdx.x; i < N; i += blockDim.x) im[i] = 0.f;
            __syncthreads();
        }

        // ---- pass 1: R2 butterflies of radix R1 per transform (lane = 8 slot + transform, butterfly j = 4 warp + slot) ----
        {
            const int tid = tid_now();
            const int t = tid & 7, j = 4 * (tid >> 5) + ((tid >> 3) & 3);
            int kn, f0, nvalid;
            if (ROWS) nvalid = rows_nvalid(a.nrows, it);
            else decode_item(it, a.Kh, a.nfields, &kn, &f0, &nvalid);
            const bool work = t < nvalid && j < R2;
            float2 v[R1];
            {
                const float *re = smem_tp + t * TS + min(j, R2 - 1), *im = re + N;
#pragma unroll
                for (int r = 0; r < R1; ++r) v[r] = make_float2(re[R2 * r], im[R2 * r]);
            }
            __syncthreads();  // every sample is in registers: the rows may be overwritten by the exchange area
            Dft<R1, false>::run(v);
            if (work) {
                float2 *ex = reinterpret_cast<float2 *>(smem_tp) + t * TS2;
                float2 *ex0 = ex + j, *ex1 = ex + (j + 1 == R2 ? 0 : j + 1);  // slot of j in the blocks of even / odd q
                const float2 *tw = reinterpret_cast<const float2 *>(blob_s) + j;
                ex0[0] = v[0];
#pragma unroll
                for (int qq = 1; qq < R1; ++qq) ((qq & 1) ? ex1 : ex0)[R2 * qq] = cmul(v[qq], tw[(qq - 1) * R2]);
            }
        }
        __syncthreads();

        // ---- pass 2: R1 butterflies of radix R2 per transform (sub-transform q = q_of(warp, slot)) ----
        float2 u[R2];
        {
            const int tid = tid_now();
            const int t = tid & 7, q = q_of<R1>(tid >> 5, (tid >> 3) & 3);
            const float2 *ex = reinterpret_cast<const float2 *>(smem_tp) + t * TS2 + R2 * q;
            const float2 *exr = ex + (q & 1);  // element r of the block sits at slot (r + (q & 1)) mod R2
#pragma unroll
            for (int r = 0; r < R2 - 1; ++r) u[r] = exr[r];
            u[R2 - 1] = ex[(q & 1) ? 0 : R2 - 1];
        }
        ptx::fence_proxy_async_smem();  // generic accesses to the area are ordered before the bulk copies that refill it
        __syncthreads();
        if (tid_now() == 0 && it + (int)gridDim.x < nitems) issue_rows(it + gridDim.x);  // lands while this item is emitted
        Dft<R2, false>::run(u);

        if (ROWS) {
            // ---- emit: spectra of the two real rows packed in z = row a + i row b: A = (z_m + conj z_{n-m}) / 2,
            // B = (z_m - conj z_{n-m}) / (2 i) ----
            const int tid = tid_now();
            const int t = tid & 7, q = q_of<R1>(tid >> 5, (tid >> 3) & 3);
            const long long ra = 16LL * it + 2 * t;
            const bool va = ra < a.nrows, vb = ra + 1 < a.nrows;
            const int mtop = min(a.nmodes, N / 2 + 1);
            const bool plain = a.mode_pieces == 1;
            float2 *oa = a.rows_out + (size_t)ra * a.nmodes, *ob = oa + a.nmodes;
            const float sc = 0.5f * a.scale;
            // where order m of row r goes: plain rows, or the (nrows, width) block of the piece that holds m
            auto slot = [&](int m, float2 **pa, float2 **pb) {
                if (plain) {
                    *pa = oa + m;
                    *pb = ob + m;
                } else {
                    int s0, w;
                    piece_of(m, a.nmodes, a.mode_pieces, &s0, &w);
                    *pa = a.rows_out + (size_t)a.nrows * s0 + (size_t)ra * w + (m - s0);
                    *pb = *pa + w;
                }
            };
#pragma unroll
            for (int i = 0; i <= R2 / 2; ++i) {
                const int m = q + R1 * i;
                const float2 give = u[R2 - 1 - i];
                float2 got;
                got.x = __shfl_xor_sync(0xffffffffu, give.x, 16);
                got.y = __shfl_xor_sync(0xffffffffu, give.y, 16);
                if (m >= mtop) continue;
                const float2 zm = u[i];
                const float2 zn = (q == 0) ? u[(R2 - i) % R2] : (q == R1 / 2) ? give : got;
                float2 *pa, *pb;
                slot(m, &pa, &pb);
                if (va) *pa = make_float2(sc * (zm.x + zn.x), sc * (zm.y - zn.y));
                if (vb) *pb = make_float2(sc * (zm.y + zn.y), sc * (zn.x - zm.x));
            }
            for (int m = mtop + (tid >> 3); m < a.nmodes; m += TP::THREADS >> 3) {  // beyond the Nyquist frequency: zeros
                float2 *pa, *pb;
                slot(m, &pa, &pb);
                if (va) *pa = make_float2(0.f, 0.f);
                if (vb) *pb = make_float2(0.f, 0.f);
            }
        } else {
            // ---- emit: bins q + R1 i, i <= R2 / 2, are the retained orders; their mirrors come from the partner lane ----
            const int tid = tid_now();
            const int t = tid & 7, q = q_of<R1>(tid >> 5, (tid >> 3) & 3);
            int kn, f0, nvalid;
            decode_item(it, a.Kh, a.nfields, &kn, &f0, &nvalid);
            const bool active = t < nvalid;
            const int ngroups = 2 * a.mmax;
            const int mtop = min(a.mmax, N / 2 + 1);
            const float *ms_s = reinterpret_cast<const float *>(blob_s + sizeof(float2) * TP::NTW);
            const unsigned char *kf_s = reinterpret_cast<const unsigned char *>(ms_s + a.mpad);
            const float sc0 = (a.nlat - 1 - kn == kn) ? 0.25f : 0.5f;  // odd nlat: the equator row is its own mirror image and counts once
            float *xb = a.op + ((size_t)(kn >> 5) * ngroups * 32 + (kn & 31)) * a.ncp + 2 * (f0 + t);
            const int k2 = a.Kh + kn;  // VEC = 2: row of the second segment
            float *xb2 = a.op + ((size_t)(k2 >> 5) * ngroups * 32 + (k2 & 31)) * a.ncp + 2 * (f0 + t);
            const size_t gstride = (size_t)32 * a.ncp;  // floats between the rows of consecutive groups
#pragma unroll
            for (int i = 0; i <= R2 / 2; ++i) {
                const int m = q + R1 * i;
                const float2 give = u[R2 - 1 - i];
                float2 got;
                got.x = __shfl_xor_sync(0xffffffffu, give.x, 16);
                got.y = __shfl_xor_sync(0xffffffffu, give.y, 16);
                if (!active || m >= mtop) continue;
                const float2 zm = u[i];
                const float2 zn = (q == 0) ? u[(R2 - i) % R2] : (q == R1 / 2) ? give : got;
                // spectra of the two real rows packed in z = north + i south: A = (z_m + conj z_{n-m}) / 2,
                // B = (z_m - conj z_{n-m}) / (2 i); even fold = A + B, odd fold = A - B
                const float sc = sc0 * ms_s[m];
                const float ar = zm.x + zn.x, ai = zm.y - zn.y, br = zm.y + zn.y, bi = zn.x - zm.x;
                const bool edge = a.zero_imag_edges && (m == 0 || 2 * m == N);
                const float2 e = make_float2(sc * (ar + br), edge ? 0.f : sc * (ai + bi));
                const float2 o = make_float2(sc * (ar - br), edge ? 0.f : sc * (ai - bi));
                if (VEC == 1) {
                    const int kf = kf_s[m];  // (the contraction does not read rows above the group's polar extent)
                    float *pe = xb + (size_t)(2 * m) * gstride;
                    if (kn >= (kf & 15) * kBK) *reinterpret_cast<float2 *>(pe) = e;
                    if (kn >= (kf >> 4) * kBK) *reinterpret_cast<float2 *>(pe + gstride) = o;
                } else {
                    const int comp = t & 1;
                    const float sg = comp ? -1.f : 1.f;
                    // own columns inside the pair's four: the first segment at 2 comp, the second at 2 (1 - comp)
                    float *p0 = xb + (size_t)(2 * m) * gstride;                    // rows k'
                    float *p1 = xb2 + (2 - 4 * comp) + (size_t)(2 * m) * gstride;  // rows Kh + k'
                    // group 2 m (p = 0): first segment takes the odd fold, second the even one; group 2 m + 1 the other way
                    *reinterpret_cast<float2 *>(p0) = make_float2(sg * o.x, sg * o.y);
                    *reinterpret_cast<float2 *>(p1) = make_float2(-e.y, e.x);
                    *reinterpret_cast<float2 *>(p0 + gstride) = make_float2(sg * e.x, sg * e.y);
                    *reinterpret_cast<float2 *>(p1 + gstride) = make_float2(-o.y, o.x);
                }
            }
            // orders beyond the Nyquist frequency (mmax > n / 2 + 1) are zeros
            for (int m = mtop + (tid >> 3); m < a.mmax; m += TP::THREADS >> 3) {
                if (active) {
                    float *pe = xb + (size_t)(2 * m) * gstride;
                    *reinterpret_cast<float2 *>(pe) = make_float2(0.f, 0.f);
                    *reinterpret_cast<float2 *>(pe + gstride) = make_float2(0.f, 0.f);
                    if (VEC == 2) {
                        pe = xb2 + (size_t)(2 * m) * gstride;
                        *reinterpret_cast<float2 *>(pe) = make_float2(0.f, 0.f);
                        *reinterpret_cast<float2 *>(pe + gstride) = make_float2(0.f, 0.f);
                    }
                }
            }
        }
    }
}

// ROWS: plain batched irfft of (nrows, nmodes) spectra (distributed stage, torch_harmonics/distributed/distributed_sht.py:385).
template <int R1, int R2, bool ROWS>
__global__ void __launch_bounds__(TwoPass<R1, R2>::THREADS, 2) fft_synthesis_twopass_kernel(const TwoPassArgs a) {
    using TP = TwoPass<R1, R2>;
    constexpr int N = TP::N, TS = TP::TS, TS2 = TP::TS / 2;
    constexpr int CH = 5;  // orders whose loads are in flight together (measured: more in flight, or asking the next item's rows into L2 ahead of time, is slower)
    extern __shared__ __align__(16) float smem_tp[];
    unsigned char *blob_s = reinterpret_cast<unsigned char *>(smem_tp + kNT * TS);
    const uint32_t bar_tab = ptx::smem_u32(blob_s + a.blob_bytes);
    const int nitems = ROWS ? (int)((a.nrows + 15) >> 4) : a.Kh * ((a.nfields + kNT - 1) / kNT);
    if ((int)blockIdx.x >= nitems) return;

    if (threadIdx.x == 0) {
        ptx::mbar_init(bar_tab, 1);
        ptx::fence_barrier_init();
        ptx::mbar_arrive_expect_tx(bar_tab, (uint32_t)a.blob_bytes);
        ptx::bulk_load(ptx::smem_u32(blob_s), a.blob, (uint32_t)a.blob_bytes, bar_tab);
    }
    __syncthreads();
    if (!cta_wait(bar_tab, 0, a.err, 0x0F7F0021)) return;

    for (int it = blockIdx.x; it < nitems; it += gridDim.x) {
        // ---- gather the even / odd parts of the retained orders, rebuild the Hermitian spectrum of north + i south ----
        float2 u[R2];
        {
            const int tid = tid_now();
            const int t = tid & 7, q = q_of<R1>(tid >> 5, (tid >> 3) & 3);
            int kn = 0, f0 = 0, nvalid = 0;
            if (!ROWS) decode_item(it, a.Kh, a.nfields, &kn, &f0, &nvalid);
            const bool active = ROWS || t < nvalid;
            const int ngroups = 2 * a.mmax;
            const int mtop = min(ROWS ? a.nmodes : a.mmax, N / 2 + 1);
            const float *ms_s = reinterpret_cast<const float *>(blob_s + sizeof(float2) * TP::NTW);
            const unsigned char *kf_s = reinterpret_cast<const unsigned char *>(ms_s + a.mpad);
            // this item's panel of Y (latitude kn, fields f0 .. f0 + 7): one contiguous region, 16 floats per group
            const float *yb = ROWS ? nullptr : a.op + y_off(0, kn, 2 * (f0 + t), ngroups, a.ncp);
            const size_t gstride = 16;
            // ROWS: the spectra of rows 2 t and 2 t + 1 of the item
            const long long ra = 16LL * it + 2 * t;
            const bool va = ROWS && ra < a.nrows, vb = ROWS && ra + 1 < a.nrows;
            const float2 *ia = ROWS ? a.rows_in + (size_t)ra * a.nmodes : nullptr, *ib = ia + (ROWS ? a.nmodes : 0);
            // the loads of CH orders are issued before the first of them is used
#pragma unroll
            for (int r = 0; r < R2; ++r) u[r] = make_float2(0.f, 0.f);
#pragma unroll
            for (int i0 = 0; i0 <= R2 / 2; i0 += CH) {
                float2 ev[CH], ov[CH];
#pragma unroll
                for (int c = 0; c < CH; ++c) {
                    const int i = i0 + c, m = q + R1 * i;
                    ev[c] = ov[c] = make_float2(0.f, 0.f);
                    if (i <= R2 / 2 && active && m < mtop) {
                        if (ROWS) {
                            const float2 *pa = ia + m, *pb = ib + m;
                            if (a.mode_pieces != 1) {
                                int s0, w;
                                piece_of(m, a.nmodes, a.mode_pieces, &s0, &w);
                                pa = a.rows_in + (size_t)a.nrows * s0 + (size_t)ra * w + (m - s0);
                                pb = pa + w;
                            }
                            if (va) ev[c] = __ldg(pa);
                            if (vb) ov[c] = __ldg(pb);
                        } else {
                            const int kf = kf_s[m];  // (rows above the group's polar extent were not produced: zeros)
                            const float *pe = yb + (size_t)(2 * m) * gstride;
                            if (kn >= (kf & 15) * kBK) ev[c] = __ldg(reinterpret_cast<const float2 *>(pe));
                            if (kn >= (kf >> 4) * kBK) ov[c] = __ldg(reinterpret_cast<const float2 *>(pe + gstride));
                        }
                    }
                }
                // bin m -> register i.  Bin n - m -> register R2 - 1 - i of the thread that owns R1 - q, i.e. of the partner
                // lane (of this thread itself for q = R1 / 2); for q = 0 it is this thread's register R2 - i.  DC and Nyquist
                // have no mirror bin.  Orders that are not retained contribute zeros.
#pragma unroll
                for (int c = 0; c < CH; ++c) {
                    const int i = i0 + c, m = q + R1 * i;
                    if (i > R2 / 2) continue;
                    // north row spectrum A = even + odd, south row spectrum B = even - odd; Z_m = A + i B, Z_{n-m} = conj A + i conj B
                    // (ROWS: the two loads are A and B themselves, unscaled)
                    const float sc = ROWS ? 1.f : (active && m < mtop) ? ms_s[m] : 0.f;
                    const float ar = ROWS ? ev[c].x : sc * (ev[c].x + ov[c].x), ai = ROWS ? ev[c].y : sc * (ev[c].y + ov[c].y);
                    const float br = ROWS ? ov[c].x : sc * (ev[c].x - ov[c].x), bi = ROWS ? ov[c].y : sc * (ev[c].y - ov[c].y);
                    const bool edge = (m == 0) || (2 * m == N);  // imaginary parts of DC / Nyquist are dropped
                    const float2 zm = edge ? make_float2(ar, br) : make_float2(ar - bi, ai + br);
                    const float2 zn = edge ? make_float2(0.f, 0.f) : make_float2(ar + bi, br - ai);
                    float2 got;
                    got.x = __shfl_xor_sync(0xffffffffu, zn.x, 16);
                    got.y = __shfl_xor_sync(0xffffffffu, zn.y, 16);
                    // every assignment is unconditional (a select with the old value), so that the register array never looks
                    // conditionally initialised; for q = 0 register R2 - 1 - i first takes a placeholder and the next order fills it
                    if (i < R2 / 2) {
                        u[i] = zm;
                        u[R2 - 1 - i] = (q == R1 / 2) ? zn : got;
                        if (i >= 1) u[R2 - i] = (q == 0) ? zn : u[R2 - i];
                    } else {
                        u[i] = (q == 0) ? zm : u[i];  // order R1 R2 / 2 = n / 2 exists for q = 0 only
                    }
                }
            }
        }
        Dft<R2, true>::run(u);

        // the rows of the previous item must have left shared memory before the area is written again
        if (tid_now() == 0) ptx::bulk_wait_read_all();
        __syncthreads();
        {
            const int tid = tid_now();
            const int t = tid & 7, q = q_of<R1>(tid >> 5, (tid >> 3) & 3);
            float2 *ex = reinterpret_cast<float2 *>(smem_tp) + t * TS2 + R2 * q;
            float2 *exr = ex + (q & 1);
#pragma unroll
            for (int r = 0; r < R2 - 1; ++r) exr[r] = u[r];
            ex[(q & 1) ? 0 : R2 - 1] = u[R2 - 1];
        }
        __syncthreads();

        // ---- inverse of pass 1: conjugate twiddles, radix R1, samples j + R2 r ----
        {
            const int tid = tid_now();
            const int t = tid & 7, j = 4 * (tid >> 5) + ((tid >> 3) & 3);
            const int jc = min(j, R2 - 1);
            float2 v[R1];
            {
                const float2 *ex = reinterpret_cast<const float2 *>(smem_tp) + t * TS2;
                const float2 *ex0 = ex + jc, *ex1 = ex + (jc + 1 == R2 ? 0 : jc + 1);
                const float2 *tw = reinterpret_cast<const float2 *>(blob_s) + jc;
                v[0] = ex0[0];
#pragma unroll
                for (int qq = 1; qq < R1; ++qq) v[qq] = cmulc(((qq & 1) ? ex1 : ex0)[R2 * qq], tw[(qq - 1) * R2]);
            }
            __syncthreads();  // the exchange area has been read: the rows may be written over it
            Dft<R1, true>::run(v);
            if (j < R2) {
                float *re = smem_tp + t * TS + j, *im = re + N;
#pragma unroll
                for (int r = 0; r < R1; ++r) {
                    re[R2 * r] = v[r].x;
                    im[R2 * r] = v[r].y;
                }
            }
        }
        ptx::fence_proxy_async_smem();  // the rows are visible to the bulk copies that follow
        __syncthreads();
        if (ROWS) {
            if (tid_now() == 0) {
                const long long r0 = 16LL * it;
                const int nr = (int)min(16LL, a.nrows - r0);
                if (a.grid_pieces == 1) {
                    for (int w = 0; w < nr; ++w)
                        ptx::bulk_store(a.grid_out + (size_t)(r0 + w) * N, ptx::smem_u32(smem_tp + (w >> 1) * TS + (w & 1) * N), N * 4u);
                } else {
                    const int q = N / a.grid_pieces, rem = N - q * a.grid_pieces;
                    for (int j = 0, s0 = 0; j < a.grid_pieces; ++j) {
                        const int wd = q + (j < rem ? 1 : 0);
                        float *pj = a.grid_out + (size_t)a.nrows * s0 + (size_t)r0 * wd;
                        for (int w = 0; w < nr; ++w)
                            ptx::bulk_store(pj + (size_t)w * wd, ptx::smem_u32(smem_tp + (w >> 1) * TS + (w & 1) * N + s0), wd * 4u);
                        s0 += wd;
                    }
                }
                ptx::bulk_commit();
            }
        } else if (tid_now() == 0) {
            int kn, f0, nvalid;
            decode_item(it, a.Kh, a.nfields, &kn, &f0, &nvalid);
            const int ks = a.nlat - 1 - kn;
            for (int w = 0; w < nvalid; ++w) {
                float *f = a.grid_out + (size_t)(f0 + w) * a.nlat * N;
                ptx::bulk_store(f + (size_t)kn * N, ptx::smem_u32(smem_tp + w * TS), N * 4u);
                if (ks != kn) ptx::bulk_store(f + (size_t)ks * N, ptx::smem_u32(smem_tp + w * TS + N), N * 4u);
            }
            ptx::bulk_commit();
        }
    }
    if (tid_now() == 0) ptx::bulk_wait_read_all();  // shared memory stays allocated until the last rows have been read
}

// nfields: scalar fields, or (theta, phi) pairs of a vector plan (two component fields each)
template <int R1, int R2>
int launch_twopass(const Plan &pl, bool analysis, const float *in, float *out, int nfields, cudaStream_t st) {
    using TP = TwoPass<R1, R2>;
    const int vec = pl.vector ? 2 : 1;
    nfields *= vec;  // component fields from here on
    TwoPassArgs a{};
    a.blob = pl.d_tp_blob;
    a.blob_bytes = pl.tp_blob_bytes;
    a.mpad = pl.tp_mpad;
    a.nlat = pl.nlat;
    a.Kh = pl.Kh;
    a.nfields = nfields;
    a.ncp = (int)col_pitch(2 * nfields);
    a.mmax = pl.mmax;
    a.zero_imag_edges = pl.zero_imag_edges;
    a.err = pl.d_err;
    const size_t smem = sizeof(float) * kNT * TP::TS + (size_t)pl.tp_blob_bytes + 32;
    if (smem > 113 * 1024) return fail(SHTB200_EINVAL, "two-pass FFT tables do not fit two CTAs per SM");
    const int nitems = pl.Kh * ceil_div(nfields, kNT);
    const int grid = std::min(2 * effective_sms(pl.sm_count), nitems);
    if (analysis) {
        a.grid_in = in;
        a.op = out;
        a.kpad = (int)(round_up(pl.Ka, kBK) - pl.Ka);
        if (vec == 2) {
            SHT_CUDA_CHECK(cudaFuncSetAttribute(fft_analysis_twopass_kernel<R1, R2, 2, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
            fft_analysis_twopass_kernel<R1, R2, 2, false><<<grid, TP::THREADS, smem, st>>>(a);
        } else {
            SHT_CUDA_CHECK(cudaFuncSetAttribute(fft_analysis_twopass_kernel<R1, R2, 1, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
            fft_analysis_twopass_kernel<R1, R2, 1, false><<<grid, TP::THREADS, smem, st>>>(a);
        }
    } else {
        a.op = const_cast<float *>(in);
        a.grid_out = out;
        SHT_CUDA_CHECK(cudaFuncSetAttribute(fft_synthesis_twopass_kernel<R1, R2, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        fft_synthesis_twopass_kernel<R1, R2, false><<<grid, TP::THREADS, smem, st>>>(a);
    }
    SHT_CUDA_CHECK(cudaGetLastError());
    return SHTB200_OK;
}

}  // namespace

// The factorisation nlon = R1 * R2 the two-pass kernels are built for (0 when there is none).
bool twopass_supported(int nlon, int *r1, int *r2) {
#ifdef SHTB200_DISABLE_TWOPASS  // build-time switch for A/B measurements against the general kernels
    return false;
#endif
    // nlon = R1 * R2 with R2 <= R1 <= 40 (the radices are carried in registers), R1 a multiple of 4, R2 even
    static const int splits[][3] = {{1440, 40, 36}, {720, 36, 20}, {512, 32, 16}};
    for (const auto &sp : splits)
        if (nlon == sp[0]) {
            *r1 = sp[1];
            *r2 = sp[2];
            return true;
        }
    return false;
}

// Tables of the two-pass kernels: [pass twiddles][per-order scale][first live latitude block of the even (low nibble) /
// odd (high nibble) group of each order], one device blob copied to shared memory once per CTA.
int build_twopass_tables(Plan &pl, const std::vector<float> &mscale) {
    int r1 = 0, r2 = 0;
    pl.twopass = false;
    if (!twopass_supported(pl.nlon, &r1, &r2)) return SHTB200_OK;
    const int n = pl.nlon, ntw = (r1 - 1) * r2;
    const int mpad = (int)round_up(pl.mmax, 16);
    std::vector<unsigned char> blob(sizeof(float2) * ntw + sizeof(float) * mpad + mpad, 0);
    float2 *tw = reinterpret_cast<float2 *>(blob.data());
    for (int q = 1; q < r1; ++q)
        for (int j = 0; j < r2; ++j) {
            const double ang = -2.0 * M_PI * (double)((long long)q * j % n) / (double)n;
            tw[(q - 1) * r2 + j] = make_float2((float)cos(ang), (float)sin(ang));
        }
    float *ms = reinterpret_cast<float *>(blob.data() + sizeof(float2) * ntw);
    unsigned char *kf = blob.data() + sizeof(float2) * ntw + sizeof(float) * mpad;
    for (int m = 0; m < pl.mmax; ++m) {
        ms[m] = mscale[m];
        kf[m] = (unsigned char)((pl.group_krow0[2 * m] / kBK) | ((pl.group_krow0[2 * m + 1] / kBK) << 4));
    }
    blob.resize(round_up((long long)blob.size(), 16));
    SHT_CUDA_CHECK(cudaMalloc(&pl.d_tp_blob, blob.size()));
    SHT_CUDA_CHECK(cudaMemcpy(pl.d_tp_blob, blob.data(), blob.size(), cudaMemcpyHostToDevice));
    pl.tp_blob_bytes = (int)blob.size();
    pl.tp_mpad = mpad;
    pl.twopass = true;
    return SHTB200_OK;
}

// Both need 16-byte aligned rows (bulk copies): the caller falls back to the general kernels otherwise.
static int dispatch_twopass(const Plan &pl, bool analysis, const float *in, float *out, int nfields, cudaStream_t st) {
    switch (pl.nlon) {
        case 1440: return launch_twopass<40, 36>(pl, analysis, in, out, nfields, st);
        case 720: return launch_twopass<36, 20>(pl, analysis, in, out, nfields, st);
        case 512: return launch_twopass<32, 16>(pl, analysis, in, out, nfields, st);
    }
    return fail(SHTB200_EINVAL, "no two-pass FFT kernel for this nlon");
}

int launch_fft_analysis_twopass(const Plan &pl, const float *x, float *X, int nfields, cudaStream_t st) { return dispatch_twopass(pl, true, x, X, nfields, st); }

int launch_fft_synthesis_twopass(const Plan &pl, const float *Y, float *x, int nfields, cudaStream_t st) { return dispatch_twopass(pl, false, Y, x, nfields, st); }

// ---- plain batched row transforms (stage entry points) ----

// Pass twiddles alone, as a device blob for the ROWS kernels.
int build_twopass_rows_tables(int nlon, unsigned char **d_blob, int *bytes) {
    int r1 = 0, r2 = 0;
    *d_blob = nullptr;
    *bytes = 0;
    if (!twopass_supported(nlon, &r1, &r2)) return SHTB200_OK;
    std::vector<float2> tw((size_t)(r1 - 1) * r2 + 1);  // (+1: keeps the blob a multiple of 16 bytes for odd counts)
    for (int q = 1; q < r1; ++q)
        for (int j = 0; j < r2; ++j) {
            const double ang = -2.0 * M_PI * (double)((long long)q * j % nlon) / (double)nlon;
            tw[(size_t)(q - 1) * r2 + j] = make_float2((float)cos(ang), (float)sin(ang));
        }
    const size_t nbytes = (size_t)round_up((long long)(sizeof(float2) * (size_t)(r1 - 1) * r2), 16);
    SHT_CUDA_CHECK(cudaMalloc(d_blob, nbytes));
    SHT_CUDA_CHECK(cudaMemcpy(*d_blob, tw.data(), nbytes, cudaMemcpyHostToDevice));
    *bytes = (int)nbytes;
    return SHTB200_OK;
}

template <int R1, int R2>
static int launch_rows(const TwoPassRows &tr, bool forward, const void *in, void *out, long long nrows, int nmodes, float scale, int grid_pieces, int mode_pieces,
                       cudaStream_t st) {
    using TP = TwoPass<R1, R2>;
    TwoPassArgs a{};
    a.blob = tr.blob;
    a.blob_bytes = tr.blob_bytes;
    a.err = tr.d_err;
    a.nrows = nrows;
    a.nmodes = nmodes;
    a.scale = scale;
    a.grid_pieces = grid_pieces;
    a.mode_pieces = mode_pieces;
    const size_t smem = sizeof(float) * kNT * TP::TS + (size_t)tr.blob_bytes + 32;
    const long long nitems = (nrows + 15) / 16;
    if (nitems > 0x7fffffffLL) return fail(SHTB200_EINVAL, "too many rows");
    const int grid = (int)std::min<long long>(2LL * effective_sms(tr.sm_count), nitems);
    if (forward) {
        a.grid_in = static_cast<const float *>(in);
        a.rows_out = static_cast<float2 *>(out);
        SHT_CUDA_CHECK(cudaFuncSetAttribute(fft_analysis_twopass_kernel<R1, R2, 1, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        fft_analysis_twopass_kernel<R1, R2, 1, true><<<grid, TP::THREADS, smem, st>>>(a);
    } else {
        a.rows_in = static_cast<const float2 *>(in);
        a.grid_out = static_cast<float *>(out);
        SHT_CUDA_CHECK(cudaFuncSetAttribute(fft_synthesis_twopass_kernel<R1, R2, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        fft_synthesis_twopass_kernel<R1, R2, true><<<grid, TP::THREADS, smem, st>>>(a);
    }
    SHT_CUDA_CHECK(cudaGetLastError());
    return SHTB200_OK;
}

// Piece-major buffers need every piece of the longitude axis to be a multiple of four floats wide (bulk copies move whole
// 16-byte units) and both splits non-empty.
bool rows_pieces_supported(int nlon, int nmodes, int grid_pieces, int mode_pieces) {
    int r1, r2;
    if (!twopass_supported(nlon, &r1, &r2)) return false;
    if (grid_pieces < 1 || mode_pieces < 1 || grid_pieces > 64 || mode_pieces > 64 || nmodes < mode_pieces || nlon < grid_pieces) return false;
    if (grid_pieces > 1 && ((nlon / grid_pieces) % 4 != 0 || nlon % grid_pieces != 0)) return false;
    return true;
}

// forward: in = (nrows, nlon) real, out = (nrows, nmodes) complex; else the other way round.  Rows must be 16-byte aligned.
int launch_rows_twopass(const TwoPassRows &tr, bool forward, const void *in, void *out, long long nrows, int nlon, int nmodes, float scale, int grid_pieces,
                        int mode_pieces, cudaStream_t st) {
    switch (nlon) {
        case 1440: return launch_rows<40, 36>(tr, forward, in, out, nrows, nmodes, scale, grid_pieces, mode_pieces, st);
        case 720: return launch_rows<36, 20>(tr, forward, in, out, nrows, nmodes, scale, grid_pieces, mode_pieces, st);
        case 512: return launch_rows<32, 16>(tr, forward, in, out, nrows, nmodes, scale, grid_pieces, mode_pieces, st);
    }
    return fail(SHTB200_EINVAL, "no two-pass FFT kernel for this nlon");
}

}  // namespace shtb200
