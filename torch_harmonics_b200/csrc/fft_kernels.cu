// Longitude transforms of the SHT: shared-memory mixed-radix FFT kernels.
//
// Analysis (grid -> order-major operand of the Legendre contraction), per CTA:
//   * one pair of latitude rows (k', nlat-1-k') of each of eight fields arrives as bulk asynchronous copies
//     (cp.async.bulk, one per row) straight into the real array / imaginary array of a split-complex transform
//     buffer: z_j = x_north + i x_south.  One complex transform of z yields the spectra of both real rows at once;
//     no thread touches the rows on their way in, and the tables come with them on the same mbarrier.
//   * an in-place decimation-in-frequency FFT of length nlon runs in shared memory, two warps per transform
//     (in-register butterflies of radix 2..16; any other prime factor <= 31 goes through a generic butterfly);
//     a host-built table assigns butterflies to threads so that every pass is free of bank conflicts,
//   * the retained orders m < mmax are separated into the two rows' spectra, folded about the equator (even = north
//     + south, odd = north - south: what the parity-split Legendre tables contract with) and written, already
//     transposed, into the contraction's operand layout X[blocked_row(2 m + parity, k')][column = 2 field + re/im]
//     (columns contiguous; a CTA covers eight consecutive fields so that every write is a full 64-byte run).
// Synthesis is the mirror image on interleaved (re, im) buffers: gather the two parities, rebuild the Hermitian
// spectrum of (north + i south), decimation-in-time inverse FFT, coalesced float4 row stores.
//
// Replaces torch_harmonics/fft.py:52-68 (rfft wrapper), :71-96 (irfft wrapper) and the
// scale / transpose / real-imag split passes at torch_harmonics/sht.py:171-176 and :337-340.

#include <math.h>
#include <stdlib.h>
#include <string.h>

#include <algorithm>
#include <mutex>
#include <vector>

#include "common.cuh"
#include "fft_butterflies.cuh"
#include "fft_consts.cuh"
#include "tc_ptx.cuh"

namespace shtb200 {


// ------------------------------------------------------------------------------------------------
// host: factorisation, twiddles, output permutation
// ------------------------------------------------------------------------------------------------
namespace {

// Radices with in-register butterflies (2..5 direct, the others as products of two of those).
const int kFastRadices[] = {16, 15, 12, 10, 9, 8, 6, 5, 4, 3, 2};

// Cost of one pass of radix r over a transform of length ntot carried by 64 threads: rounds of butterflies times the
// work of one butterfly (~ r log2 r).  Radices that leave the last round of a pass half empty, or that need many
// registers, lose: for 1440 this ranks 8.12.15 ahead of 16.10.9, which measures 4 % faster in the analysis kernel.
double pass_cost(int ntot, int r) {
    const int rounds = (ntot / r + 63) / 64;
    return rounds * r * log2((double)r);
}

// Split n (a divisor of ntot) into fast radices: fewest passes; then a split that contains an odd radix (it goes last,
// where an even radix would make the unit-stride pass and the final gather conflict on shared-memory banks); then the
// cheapest one by pass_cost.
std::vector<int> best_split(int n, int ntot, std::vector<std::vector<int>> &memo, std::vector<char> &done) {
    if (n == 1) return {};
    if (done[n]) return memo[n];
    std::vector<int> best;
    bool have = false;
    auto odd = [](const std::vector<int> &v) { for (int x : v) if (x & 1) return 1; return 0; };
    auto cost = [ntot](const std::vector<int> &v) { double c = 0; for (int x : v) c += pass_cost(ntot, x); return c; };
    for (int r : kFastRadices) {
        if (n % r) continue;
        std::vector<int> cand = best_split(n / r, ntot, memo, done);
        if (n / r != 1 && cand.empty()) continue;  // remainder not factorable with fast radices
        cand.insert(cand.begin(), r);
        bool better = !have || cand.size() < best.size();
        if (have && cand.size() == best.size()) better = odd(cand) > odd(best) || (odd(cand) == odd(best) && cost(cand) < cost(best));
        if (better) { best = cand; have = true; }
    }
    done[n] = 1;
    memo[n] = best;
    return best;
}

// Shared memory serves a warp's 32-bit accesses in one wavefront when the 32 lanes touch 32 different banks (word index
// mod 32), and a 64-bit access as two wavefronts of 16 lanes that must touch 16 different bank pairs (index mod 16 in
// 8-byte units); every further distinct address on a used bank costs one more wavefront.
// Order the butterflies of a pass (first-leg slot `off`, twiddle index j) so that each run of `width` consecutive
// threads is conflict-free on the data (width 32: split re / im arrays of floats; width 16: interleaved float2) and
// each half-warp on the float2 twiddle table.  All legs of a butterfly are shifted by the same amount, so one check
// covers them all.
std::vector<unsigned> order_butterflies(int n, int L, int R, int width) {
    const int Ls = L / R, nb = n / R;
    std::vector<std::vector<unsigned>> bucket(width);
    for (int b = 0; b < n / L; ++b)
        for (int j = 0; j < Ls; ++j) bucket[(b * L + j) % width].push_back((unsigned)(b * L + j) | ((unsigned)j << 16));
    std::vector<unsigned> out;
    out.reserve(nb);
    std::vector<int> cls(width);
    while ((int)out.size() < nb) {
        for (int c = 0; c < width; ++c) cls[c] = c;
        std::stable_sort(cls.begin(), cls.end(), [&](int a, int b) { return bucket[a].size() > bucket[b].size(); });
        // the run is filled as `width / 16` half-warps, each with its own twiddle bank pairs
        const int halves = width / 16;
        std::vector<std::vector<unsigned>> half(halves);
        std::vector<std::vector<int>> jslot(halves, std::vector<int>(16, -1));
        int taken = 0;
        for (int ci = 0; ci < width && taken < width; ++ci) {
            std::vector<unsigned> &bk = bucket[cls[ci]];
            bool placed = false;
            for (size_t i = 0; i < bk.size() && !placed; ++i) {
                const int j = (int)(bk[i] >> 16);
                for (int h = 0; h < halves && !placed; ++h) {
                    if ((int)half[h].size() >= 16) continue;
                    if (jslot[h][j % 16] >= 0 && jslot[h][j % 16] != j) continue;  // another twiddle on the same bank pair
                    jslot[h][j % 16] = j;
                    half[h].push_back(bk[i]);
                    bk.erase(bk.begin() + (long)i);
                    placed = true;
                    ++taken;
                }
            }
        }
        // nothing conflict-free left for this run: fill it from the fullest classes
        while (taken < width && (int)out.size() + taken < nb) {
            int best = -1;
            for (int c = 0; c < width; ++c)
                if (!bucket[c].empty() && (best < 0 || bucket[c].size() > bucket[best].size())) best = c;
            if (best < 0) break;
            for (int h = 0; h < halves; ++h)
                if ((int)half[h].size() < 16) { half[h].push_back(bucket[best].front()); break; }
            bucket[best].erase(bucket[best].begin());
            ++taken;
        }
        // full half-warps first, so that only the very last one of the pass may be ragged
        for (int h = 0; h < halves; ++h)
            if ((int)half[h].size() == 16) out.insert(out.end(), half[h].begin(), half[h].end());
        for (int h = 0; h < halves; ++h)
            if ((int)half[h].size() != 16) out.insert(out.end(), half[h].begin(), half[h].end());
    }
    return out;
}

// Order of the retained orders m < mmax for the emit / gather loops of the SHT kernels.  `lanes` adjacent lanes share
// an order, lane c of them touching transforms 2c and 2c+1, which lie `stride` units apart (floats in the split
// layout, where a wavefront is the 32 lanes of a warp; float2 in the interleaved layout, where it is 16 lanes).
// Both spectrum slots an order touches (bin m and bin n - m) must avoid the banks of the other orders of the wavefront.
std::vector<unsigned short> order_emit(int n, int mmax, int stride, int lanes, int width, const std::vector<unsigned short> &perm) {
    const int per = width / lanes;
    auto mask = [&](int m, int which) {
        const int k = which == 0 ? (m < n ? m : 0) : ((n - m % n) % n);
        unsigned mk = 0;
        for (int c = 0; c < lanes; ++c) mk |= 1u << ((2 * c * stride + perm[k]) % width);
        return mk;
    };
    std::vector<unsigned short> out;
    out.reserve(mmax);
    size_t first = 0;
    std::vector<char> used(mmax, 0);
    while ((int)out.size() < mmax) {
        while (used[first]) ++first;
        int cnt = 1;
        unsigned u0 = mask((int)first, 0), u1 = mask((int)first, 1);
        used[first] = 1;
        out.push_back((unsigned short)first);
        // look a bounded distance ahead so that neighbouring orders (neighbouring rows of the operand) stay together
        for (size_t i = first + 1; i < (size_t)mmax && i < first + 512 && cnt < per; ++i) {
            if (used[i]) continue;
            const unsigned s0 = mask((int)i, 0), s1 = mask((int)i, 1);
            if ((s0 & u0) || (s1 & u1)) continue;
            u0 |= s0;
            u1 |= s1;
            used[i] = 1;
            out.push_back((unsigned short)i);
            ++cnt;
        }
        for (size_t i = first + 1; i < (size_t)mmax && cnt < per; ++i) {
            if (used[i]) continue;
            used[i] = 1;
            out.push_back((unsigned short)i);
            ++cnt;
        }
    }
    return out;
}

}  // namespace

int build_fft_plan(int nlon, int mmax_emit, int layout, const int *krow0, FftPlanDev *out, float2 **d_tw, unsigned short **d_perm) {
    if (nlon < 2 || nlon > 65535) return fail(SHTB200_EINVAL, "nlon must be in [2, 65535]");
    // strip prime factors 7..31 (generic butterflies), split the rest into fast radices
    std::vector<int> slow;
    int n = nlon;
    for (int p = 7; p <= 31; p += 2) {
        if (p % 3 == 0 || p % 5 == 0) continue;
        while (n % p == 0) { slow.push_back(p); n /= p; }
    }
    {
        int r = n;
        while (r % 2 == 0) r /= 2;
        while (r % 3 == 0) r /= 3;
        while (r % 5 == 0) r /= 5;
        if (r != 1) return fail(SHTB200_EINVAL, "nlon has a prime factor larger than 31");
    }
    std::vector<std::vector<int>> memo(n + 1);
    std::vector<char> done(n + 1, 0);
    std::vector<int> rad = best_split(n, nlon, memo, done);
    // largest radices first; an odd radix last keeps the unit-stride pass free of bank conflicts
    std::sort(rad.begin(), rad.end(), [](int a, int b) { return a > b; });
    for (size_t i = 0; i + 1 < rad.size(); ++i)
        if (rad.back() % 2 == 0 && rad[i] % 2 == 1) { std::swap(rad[i], rad.back()); break; }
    rad.insert(rad.begin(), slow.begin(), slow.end());
    if ((int)rad.size() > kMaxFftStages) return fail(SHTB200_EINVAL, "nlon has too many factors");

    FftPlanDev fp{};
    fp.n = nlon;
    fp.nstages = (int)rad.size();
    int L = nlon;
    std::vector<float2> tw;
    for (int s = 0; s < fp.nstages; ++s) {
        const int R = rad[s], Ls = L / R;
        fp.radix[s] = R;
        fp.sublen[s] = L;
        fp.twoff[s] = (int)tw.size();
        // pass table: entry (q - 1) * Ls + j = exp(-2 pi i q j / L); none for the last pass (Ls = 1)
        if (Ls > 1)
            for (int q = 1; q < R; ++q)
                for (int j = 0; j < Ls; ++j) {
                    double a = -2.0 * M_PI * (double)((long long)q * j % L) / (double)L;
                    tw.push_back(make_float2((float)cos(a), (float)sin(a)));
                }
        L = Ls;
    }
    if (tw.size() & 1) tw.push_back(make_float2(0.f, 0.f));  // keeps what follows the pass tables 16-byte aligned
    fp.tw_pass_total = (int)tw.size();
    // output bin k = q1 + R1 (q2 + R2 (...)) ends at slot q1 n/R1 + q2 n/(R1 R2) + ...
    std::vector<unsigned short> perm(nlon);
    for (int k = 0; k < nlon; ++k) {
        int kk = k, stride = nlon, pos = 0;
        for (int s = 0; s < fp.nstages; ++s) {
            stride /= rad[s];
            pos += (kk % rad[s]) * stride;
            kk /= rad[s];
        }
        perm[k] = (unsigned short)pos;
    }
    // thread -> butterfly tables of all passes, and the emit order; they share one allocation with perm:
    // [bfly u32 x bf_total][perm u16 x n][eorder u16 x mmax_emit]
    std::vector<unsigned> bfly;
    L = nlon;
    for (int s = 0; s < fp.nstages; ++s) {
        fp.bfoff[s] = (int)bfly.size();
        std::vector<unsigned> o = order_butterflies(nlon, L, rad[s], layout == kFftSplit ? 32 : 16);
        {  // every butterfly of the pass exactly once
            std::vector<unsigned> chk(o);
            std::sort(chk.begin(), chk.end(), [](unsigned a, unsigned b) { return (a & 0xffffu) < (b & 0xffffu); });
            const int Ls = L / rad[s];
            bool okp = (int)chk.size() == nlon / rad[s];
            for (size_t i = 0; okp && i < chk.size(); ++i) okp = (int)(chk[i] & 0xffffu) == (int)(i / Ls) * L + (int)(i % Ls) && (int)(chk[i] >> 16) == (int)(i % Ls);
            if (!okp) return fail(SHTB200_EINVAL, "butterfly order is not a permutation");
        }
        bfly.insert(bfly.end(), o.begin(), o.end());
        L /= rad[s];
    }
    fp.bf_total = (int)bfly.size();
    std::vector<unsigned short> eorder;
    if (layout == kFftSplit) {
        fp.io = (nlon + 3) / 4 * 4;
        fp.ts = 2 * fp.io;
        fp.ts += ((4 - fp.ts % 32) + 32) % 32;
        if (mmax_emit > 0) eorder = order_emit(nlon, mmax_emit, fp.ts, 4, 32, perm);
    } else if (layout == kFftPacked) {
        // with a pitch that is a multiple of 128 bytes the same bin of all transforms would fall on one bank pair
        fp.np = nlon + 2;
        if (mmax_emit > 0) eorder = order_emit(nlon, mmax_emit, fp.np, 4, 16, perm);
    } else {
        fp.np = nlon;
    }
    {
        std::vector<unsigned short> chk(eorder);
        std::sort(chk.begin(), chk.end());
        for (size_t i = 0; i < chk.size(); ++i)
            if (chk[i] != i) return fail(SHTB200_EINVAL, "emit order is not a permutation");
    }
    fp.eorder_len = (int)eorder.size();
    // One device allocation: the tables the kernels keep in shared memory as one 16-byte granular blob
    //   [pass twiddles float2 x tw_pass_total][bfly u32 x bf_total][perm u16 x n][eorder u16 x eorder_len]
    //   [kfirst u8 x eorder_len: first 32-row latitude block of the even (low nibble) / odd (high nibble) group of
    //    each order that the contraction touches][pad]
    // followed by the n roots of unity the generic prime-radix butterflies read from global memory.
    const size_t o_bf = sizeof(float2) * tw.size();
    const size_t o_perm = o_bf + sizeof(unsigned) * bfly.size();
    const size_t o_eo = o_perm + sizeof(unsigned short) * perm.size();
    const size_t o_kf = o_eo + sizeof(unsigned short) * eorder.size();
    const size_t tab_bytes = (o_kf + eorder.size() + 15) / 16 * 16;
    std::vector<unsigned char> tab(tab_bytes + sizeof(float2) * nlon, 0);
    memcpy(tab.data(), tw.data(), sizeof(float2) * tw.size());
    memcpy(tab.data() + o_bf, bfly.data(), sizeof(unsigned) * bfly.size());
    memcpy(tab.data() + o_perm, perm.data(), sizeof(unsigned short) * perm.size());
    if (!eorder.empty()) memcpy(tab.data() + o_eo, eorder.data(), sizeof(unsigned short) * eorder.size());
    if (krow0)
        for (size_t m = 0; m < eorder.size(); ++m) {
            const int b0 = krow0[2 * m] / kBK, b1 = krow0[2 * m + 1] / kBK;
            if (b0 > kMaxPolarBlock || b1 > kMaxPolarBlock) return fail(SHTB200_EINVAL, "polar extent was not clamped to the 4-bit block index");
            tab[o_kf + m] = (unsigned char)(b0 | (b1 << 4));
        }
    {
        float2 *roots = reinterpret_cast<float2 *>(tab.data() + tab_bytes);
        for (int k = 0; k < nlon; ++k) {
            double a = -2.0 * M_PI * (double)k / (double)nlon;
            roots[k] = make_float2((float)cos(a), (float)sin(a));
        }
    }
    unsigned char *d_blob = nullptr;
    SHT_CUDA_CHECK(cudaMalloc(&d_blob, tab.size()));
    SHT_CUDA_CHECK(cudaMemcpy(d_blob, tab.data(), tab.size(), cudaMemcpyHostToDevice));
    *d_tw = reinterpret_cast<float2 *>(d_blob);
    *d_perm = nullptr;
    fp.tab_bytes = (int)tab_bytes;
    fp.tw = reinterpret_cast<const float2 *>(d_blob);
    fp.tw_full = reinterpret_cast<const float2 *>(d_blob + tab_bytes);
    fp.bfly = reinterpret_cast<const unsigned *>(d_blob + o_bf);
    fp.perm = reinterpret_cast<const unsigned short *>(d_blob + o_perm);
    fp.eorder = eorder.empty() ? nullptr : reinterpret_cast<const unsigned short *>(d_blob + o_eo);
    *out = fp;
    return SHTB200_OK;
}

// Two views of a transform in shared memory: interleaved (re, im) pairs, or the real parts and the imaginary parts
// as two separate arrays.  The SHT kernels use the second: a pair of latitude rows copied from global memory as it is
// IS north + i south in that form, so the rows move between global and shared memory as bulk copies.
struct CxPacked {
    float2 *p;
    __device__ __forceinline__ float2 ld(int i) const { return p[i]; }
    __device__ __forceinline__ void st(int i, float2 v) const { p[i] = v; }
};
struct CxSplit {
    float *re, *im;
    __device__ __forceinline__ float2 ld(int i) const { return make_float2(re[i], im[i]); }
    __device__ __forceinline__ void st(int i, float2 v) const {
        re[i] = v.x;
        im[i] = v.y;
    }
};

// One butterfly of a pass.  Forward (decimation in frequency): transform, then the pass twiddles w_L^{q j};
// inverse (decimation in time): conjugate twiddles first, then the conjugate transform.  `tw` points at the
// table entry of (q = 1, this j); consecutive q are `twstr` entries apart.  Legs at d[base + r * str].
template <int R, bool INV, class D>
__device__ __forceinline__ void butterfly(const D &d, int base, int str, const float2 *tw, int twstr, bool has_tw) {
    float2 v[R];
    if (!INV) {
#pragma unroll
        for (int r = 0; r < R; ++r) v[r] = d.ld(base + r * str);
        Dft<R, false>::run(v);
        d.st(base, v[0]);
        if (has_tw) {
#pragma unroll
            for (int q = 1; q < R; ++q) d.st(base + q * str, cmul(v[q], tw[(q - 1) * twstr]));
        } else {
#pragma unroll
            for (int q = 1; q < R; ++q) d.st(base + q * str, v[q]);
        }
    } else {
        v[0] = d.ld(base);
        if (has_tw) {
#pragma unroll
            for (int r = 1; r < R; ++r) v[r] = cmulc(d.ld(base + r * str), tw[(r - 1) * twstr]);
        } else {
#pragma unroll
            for (int r = 1; r < R; ++r) v[r] = d.ld(base + r * str);
        }
        Dft<R, true>::run(v);
#pragma unroll
        for (int q = 0; q < R; ++q) d.st(base + q * str, v[q]);
    }
}

// Prime radix above 5: plain O(R^2) transform with the order-n roots of unity read from global memory.
template <bool INV, class D>
__device__ void generic_butterfly(const D &d, int base, int R, int str, const float2 *tw, int twstr, bool has_tw, const float2 *__restrict__ roots, int n) {
    float2 v[31], y[31];
    const int step = n / R;
    for (int r = 0; r < R; ++r) {
        float2 z = d.ld(base + r * str);
        if (INV && has_tw && r) z = cmulc(z, tw[(r - 1) * twstr]);
        v[r] = z;
    }
    for (int q = 0; q < R; ++q) {
        float2 acc = v[0];
        int idx = 0;
        for (int r = 1; r < R; ++r) {
            idx += q;
            if (idx >= R) idx -= R;
            float2 w = __ldg(roots + idx * step);
            acc = cadd(acc, INV ? cmulc(v[r], w) : cmul(v[r], w));
        }
        y[q] = acc;
    }
    for (int q = 0; q < R; ++q) {
        float2 z = y[q];
        if (!INV && has_tw && q) z = cmul(z, tw[(q - 1) * twstr]);
        d.st(base + q * str, z);
    }
}

// Barrier among the G warps that share one transform (named barrier `id`; plain __syncwarp when G = 1).
template <int G>
__device__ __forceinline__ void group_sync(int id) {
    if (G == 1) __syncwarp();
    else asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(32 * G) : "memory");
}

// All passes of ONE transform of length n, carried by G warps (in place, group barrier between passes).
// `lane` is the thread's index inside the group.  Forward: natural order in, bin k at slot perm[k] out.
// Inverse: bin k at slot perm[k] in, natural order out.
template <bool INV, int G, class D>
__device__ void fft_group(const D &d, const FftPlanDev &fp, const float2 *tw_s, int lane, int bar_id) {
    const int n = fp.n;
    for (int ss = 0; ss < fp.nstages; ++ss) {
        const int s = INV ? fp.nstages - 1 - ss : ss;
        const int R = fp.radix[s];
        const int L = fp.sublen[s];
        const int Ls = L / R;  // stride between butterfly legs
        const int nb = n / R;  // butterflies in this pass
        const bool has_tw = Ls > 1;
        const float2 *tw = tw_s + fp.twoff[s];
        const unsigned *bt = reinterpret_cast<const unsigned *>(tw_s + fp.tw_pass_total) + fp.bfoff[s];
        for (int i = lane; i < nb; i += 32 * G) {
            const unsigned e = bt[i];
            const int j = (int)(e >> 16);
            const int b = (int)(e & 0xffffu);
            switch (R) {
                case 16: butterfly<16, INV>(d, b, Ls, tw + j, Ls, has_tw); break;
                case 15: butterfly<15, INV>(d, b, Ls, tw + j, Ls, has_tw); break;
                case 12: butterfly<12, INV>(d, b, Ls, tw + j, Ls, has_tw); break;
                case 10: butterfly<10, INV>(d, b, Ls, tw + j, Ls, has_tw); break;
                case 9: butterfly<9, INV>(d, b, Ls, tw + j, Ls, has_tw); break;
                case 8: butterfly<8, INV>(d, b, Ls, tw + j, Ls, has_tw); break;
                case 6: butterfly<6, INV>(d, b, Ls, tw + j, Ls, has_tw); break;
                case 5: butterfly<5, INV>(d, b, Ls, tw + j, Ls, has_tw); break;
                case 4: butterfly<4, INV>(d, b, Ls, tw + j, Ls, has_tw); break;
                case 3: butterfly<3, INV>(d, b, Ls, tw + j, Ls, has_tw); break;
                case 2: butterfly<2, INV>(d, b, Ls, tw + j, Ls, has_tw); break;
                default: generic_butterfly<INV>(d, b, R, Ls, tw + j, Ls, has_tw, fp.tw_full, n);
            }
        }
        group_sync<G>(bar_id);
    }
}

// shared memory of the SHT kernels: [NW transforms x ts floats (re array | im array)][table blob: pass twiddles |
// thread -> butterfly tables u32 | n u16 perm | u16 emit order][8-byte mbarrier]; the stage kernels keep NW x n float2.
// plain copy of the blob by all threads of the CTA (callers synchronise afterwards)
__device__ __forceinline__ void load_tables(const FftPlanDev &fp, float2 *tw_s) {
    const uint4 *src = reinterpret_cast<const uint4 *>(fp.tw);
    uint4 *dst = reinterpret_cast<uint4 *>(tw_s);
    for (int i = threadIdx.x; i < fp.tab_bytes / 16; i += blockDim.x) dst[i] = __ldg(src + i);
}

// The same copy as ONE asynchronous bulk transfer issued by thread 0, so that it runs under the row loads instead of
// in front of them.  tables_begin() is called by every thread before the CTA's first barrier, tables_wait() by every
// thread at a point all threads reach: it is a CTA-wide barrier and returns false (for all threads alike) when the
// copy did not land within about a second, in which case the kernel reports through *err and leaves.
__device__ __forceinline__ void tables_begin(const FftPlanDev &fp, float2 *tw_s, uint32_t bar) {
    if (threadIdx.x == 0) {
        ptx::mbar_init(bar, 1);
        ptx::fence_barrier_init();
        ptx::mbar_arrive_expect_tx(bar, (uint32_t)fp.tab_bytes);
        ptx::bulk_load(ptx::smem_u32(tw_s), fp.tw, (uint32_t)fp.tab_bytes, bar);
    }
}
__device__ __forceinline__ bool tables_wait(uint32_t bar, int *err) {
    __syncthreads();  // the barrier's initialisation is visible to every thread that polls it
    bool ok = ptx::mbar_try_wait(bar, 0) != 0;
    if (!ok) {
        const long long t0 = clock64();
        for (uint32_t it = 1; !ok; ++it) {
            ok = ptx::mbar_try_wait(bar, 0) != 0;
            if (!ok && (it & 63u) == 0u && clock64() - t0 > 2000000000ll) break;
        }
    }
    if (__syncthreads_or(ok ? 0 : 1)) {
        if (threadIdx.x == 0 && err) atomicExch(err, 0x0F7F0001);
        return false;
    }
    return true;
}

// ------------------------------------------------------------------------------------------------
// analysis kernel
// ------------------------------------------------------------------------------------------------
// grid: (ceil(nfields / (NW / VEC)), Kh), block: NW transforms x G warps.  A CTA takes ONE pair of latitude rows
// (k', nlat-1-k') of NW / VEC consecutive fields (VEC = 1: scalar fields; VEC = 2: (theta, phi) component pairs), so
// that what it emits for an order m is one contiguous run of 2 NW floats along the column axis of the operand.
//
// Operand layout (column-contiguous):  X[blocked_row(2 m + p, kk)][col],  row pitch ncp floats, kk < Ka = VEC * Kh.
//   scalar:  kk = k',  col = 2 f + (re, im);  p = 0 holds the even fold, p = 1 the odd fold.
//   vector:  col = 4 f + c;  kk = k' contracts against the d/dtheta table and carries the fold of parity 1 - p,
//            kk = Kh + k' contracts against the m/sin(theta) table and carries the fold of parity p; the four
//            columns c follow the sign pattern of torch_harmonics/sht.py:488-493:
//              c0 (s_re): [ Re X0 | -Im X1 ]   c1 (s_im): [ Im X0 |  Re X1 ]
//              c2 (t_re): [-Re X1 | -Im X0 ]   c3 (t_im): [-Im X1 |  Re X0 ]
template <int NW, int VEC, int G>
__global__ void __launch_bounds__(32 * NW * G, (NW * G >= 16) ? 2 : 1) fft_analysis_kernel(const float *__restrict__ x, float *__restrict__ X, FftPlanDev fp,
                                                                                            int nlat, int Kh, int nfields, int ncp, int mmax,
                                                                                            const float *__restrict__ mscale, int zero_imag_edges, int bulk_rows, int *err) {
    extern __shared__ __align__(16) float smem_f[];
    const int n = fp.n;
    constexpr int NF = NW / VEC;                    // fields (or component pairs) per CTA
    constexpr int GT = 32 * G;                      // threads per transform
    const int TS = fp.ts, IO = fp.io;
    float *data = smem_f;
    float2 *tw_s = reinterpret_cast<float2 *>(smem_f + (size_t)NW * TS);
    const unsigned short *perm_s = reinterpret_cast<const unsigned short *>(reinterpret_cast<const unsigned *>(tw_s + fp.tw_pass_total) + fp.bf_total);

    const int kn = blockIdx.y;
    const int f0 = blockIdx.x * NF;  // field blocks vary fastest: CTAs that complete each other's 128-byte lines run together
    const int t = threadIdx.x / GT, lane = threadIdx.x % GT;  // transform index, index inside its group
    const int Ka = VEC * Kh;
    const int ngroups = 2 * mmax;
    if (kn >= Kh) {
        // rows of the last 32-row block beyond the contraction length: the contraction reads them, they must be zeros
        const int kk = Ka + (kn - Kh);
        for (int i = threadIdx.x; i < ngroups * (2 * NW / 4); i += blockDim.x) {
            const int g = i / (2 * NW / 4), c = (i - g * (2 * NW / 4)) * 4;
            if (2 * VEC * f0 + c < 2 * VEC * nfields) *reinterpret_cast<float4 *>(X + (size_t)blocked_row(g, kk, ngroups) * ncp + 2 * VEC * f0 + c) = make_float4(0.f, 0.f, 0.f, 0.f);
        }
        return;
    }
    const int ks = nlat - 1 - kn;
    const bool self = (ks == kn);  // odd nlat: the equator row is its own mirror image

    // ---- tables and rows arrive as bulk copies: row kn of a field is the real array of its transform, row ks the
    // imaginary array (z = north + i south; the fold into even / odd parts happens when the spectrum is emitted) ----
    const uint32_t tab_bar = ptx::smem_u32(reinterpret_cast<unsigned char *>(tw_s) + fp.tab_bytes);
    const int nvalid = min(NW, (nfields - f0) * VEC);  // transforms of this CTA that carry a field
    if (threadIdx.x == 0) {
        ptx::mbar_init(tab_bar, 1);
        ptx::fence_barrier_init();
        const uint32_t row_bytes = (uint32_t)n * 4u;
        ptx::mbar_arrive_expect_tx(tab_bar, (uint32_t)fp.tab_bytes + (bulk_rows ? 2u * row_bytes * (uint32_t)nvalid : 0u));
        ptx::bulk_load(ptx::smem_u32(tw_s), fp.tw, (uint32_t)fp.tab_bytes, tab_bar);
        if (bulk_rows) {
            for (int u = 0; u < nvalid; ++u) {
                const size_t row0 = (size_t)((f0 + u / VEC) * VEC + u % VEC) * nlat;
                ptx::bulk_load(ptx::smem_u32(data + (size_t)u * TS), x + (row0 + kn) * n, row_bytes, tab_bar);
                ptx::bulk_load(ptx::smem_u32(data + (size_t)u * TS + IO), x + (row0 + ks) * n, row_bytes, tab_bar);
            }
        }
    }
    {
        float *re = data + (size_t)t * TS, *im = re + IO;
        if (t >= nvalid) {
            for (int j = lane; j < n; j += GT) re[j] = im[j] = 0.f;
        } else if (!bulk_rows) {  // row starts not 16-byte aligned: plain loads
            const size_t row0 = (size_t)((f0 + t / VEC) * VEC + t % VEC) * nlat;
            const float *rn = x + (row0 + kn) * n, *rs = x + (row0 + ks) * n;
            for (int j = lane; j < n; j += GT) {
                re[j] = __ldg(rn + j);
                im[j] = __ldg(rs + j);
            }
        }
    }
    if (!tables_wait(tab_bar, err)) return;  // (CTA-wide barrier: rows in place as well)

    if (t < nvalid) {  // (a transform without a field holds zeros and stays zeros)
        float *re = data + (size_t)t * TS;
        fft_group<false, G>(CxSplit{re, re + IO}, fp, tw_s, lane, 1 + t);
    }
    __syncthreads();

    // ---- emit the retained orders ----
    // NW / 2 adjacent lanes share one order: lane c of them handles transforms 2c, 2c+1, i.e. one 16-byte piece of the
    // 2 NW floats an (order, fold) run is made of, so that a run leaves the SM as ONE contiguous request.
    const int nyq = n / 2;
    constexpr int LPM = NW / 2;  // lanes per order
    const int c = threadIdx.x % LPM;
    const unsigned short *eo_s = (fp.eorder && fp.eorder_len == mmax) ? perm_s + n : nullptr;
    const unsigned char *kf_s = eo_s ? reinterpret_cast<const unsigned char *>(eo_s + mmax) : nullptr;
    for (int i = threadIdx.x / LPM; i < mmax; i += blockDim.x / LPM) {
        const int m = eo_s ? eo_s[i] : i;
        float e[4], o[4];  // (re, im) of the even / odd fold of transforms 2c, 2c+1
        if (m <= nyq) {
            // spectra of the two real rows packed in z = north + i south: A = (z_m + conj z_{n-m}) / 2,
            // B = (z_m - conj z_{n-m}) / (2 i); even fold = A + B, odd fold = A - B (the equator row counts once)
            const float sc = (self ? 0.25f : 0.5f) * mscale[m];
            const int pm = perm_s[m];
            const int pn = perm_s[m == 0 ? 0 : n - m];
            const bool edge = zero_imag_edges && (m == 0 || (2 * m == n));
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                const float *dre = data + (size_t)(2 * c + h) * TS, *dim = dre + IO;
                const float zmx = dre[pm], zmy = dim[pm], znx = dre[pn], zny = dim[pn];
                const float ar = zmx + znx, ai = zmy - zny, br = zmy + zny, bi = znx - zmx;
                e[2 * h] = sc * (ar + br);
                e[2 * h + 1] = edge ? 0.f : sc * (ai + bi);
                o[2 * h] = sc * (ar - br);
                o[2 * h + 1] = edge ? 0.f : sc * (ai - bi);
            }
        } else {
#pragma unroll
            for (int u = 0; u < 4; ++u) e[u] = o[u] = 0.f;
        }
        if (VEC == 1) {
            // columns 2 (f0 + 2c), ..: (re, im) of two consecutive fields
            const int col = 2 * f0 + 4 * c;
            if (col < 2 * nfields) {  // (columns past the last field pad the row pitch: nobody reads them)
                // (the contraction does not read rows above the group's polar extent)
                const int kf = kf_s ? kf_s[m] : 0;
                if (kn >= (kf & 15) * kBK) *reinterpret_cast<float4 *>(X + (size_t)blocked_row(2 * m, kn, ngroups) * ncp + col) = make_float4(e[0], e[1], e[2], e[3]);
                if (kn >= (kf >> 4) * kBK) *reinterpret_cast<float4 *>(X + (size_t)blocked_row(2 * m + 1, kn, ngroups) * ncp + col) = make_float4(o[0], o[1], o[2], o[3]);
            }
        } else {
            // transforms 2c (theta component X0) and 2c + 1 (phi component X1) of pair f0 + c: four columns 4 (f0 + c)..
            const int col = 4 * (f0 + c);
            if (col < 4 * nfields) {
#pragma unroll
                for (int p = 0; p < 2; ++p) {
                    const float *fa = p ? e : o;  // d/dtheta rows take the fold of parity 1 - p
                    const float *fb = p ? o : e;  // m/sin(theta) rows take the fold of parity p
                    *reinterpret_cast<float4 *>(X + (size_t)blocked_row(2 * m + p, kn, ngroups) * ncp + col) = make_float4(fa[0], fa[1], -fa[2], -fa[3]);
                    *reinterpret_cast<float4 *>(X + (size_t)blocked_row(2 * m + p, Kh + kn, ngroups) * ncp + col) = make_float4(-fb[3], fb[2], -fb[1], fb[0]);
                }
            }
        }
    }
}

// ------------------------------------------------------------------------------------------------
// synthesis kernel
// ------------------------------------------------------------------------------------------------
// Y[y_off(2 m + p, k', col)] (16-column panels, see y_off) holds the even (p = 0) / odd (p = 1) latitude parts of order m;
// col = 2 f + (re, im) for scalar fields, 4 f + (theta re, theta im, phi re, phi im) for vector pairs: in both
// cases transform u of the CTA reads columns 2 u, 2 u + 1 past the CTA's first column.
template <int NW, int VEC, int G>
__global__ void __launch_bounds__(32 * NW * G, (NW * G >= 16) ? 2 : 1) fft_synthesis_kernel(const float *__restrict__ Y, float *__restrict__ x, FftPlanDev fp,
                                                                                             int nlat, int Kh, int nfields, int ncp, int mmax,
                                                                                             const float *__restrict__ mscale, int vec4ok, int *err) {
    extern __shared__ float2 smem[];
    const int n = fp.n;
    constexpr int NF = NW / VEC;
    constexpr int GT = 32 * G;
    const int np = fp.np;
    float2 *data = smem;
    float2 *tw_s = data + (size_t)NW * np;
    const unsigned short *perm_s = reinterpret_cast<const unsigned short *>(reinterpret_cast<const unsigned *>(tw_s + fp.tw_pass_total) + fp.bf_total);

    const int kn = blockIdx.y;
    const int f0 = blockIdx.x * NF;
    const int colbase = 2 * VEC * f0;
    const int t = threadIdx.x / GT, lane = threadIdx.x % GT;
    const uint32_t tab_bar = ptx::smem_u32(reinterpret_cast<unsigned char *>(tw_s) + fp.tab_bytes);
    tables_begin(fp, tw_s, tab_bar);
    if (!tables_wait(tab_bar, err)) return;

    const int nyq = n / 2;
    const int mtop = min(mmax, nyq + 1);
    // bins that no retained order (or its mirror image) fills
    {
        const int nzero = n - 2 * mtop + 1;
        for (int i = threadIdx.x; i < NW * nzero; i += blockDim.x) {
            const int u = i / nzero, m = mtop + (i - u * nzero);
            data[(size_t)u * np + perm_s[m]] = make_float2(0.f, 0.f);
        }
    }
    // NW / 2 adjacent lanes share one order; lane c reads the 16-byte piece of both runs that holds transforms 2c, 2c+1.
    // The loads of three orders are issued before the first of them is consumed.
    {
        constexpr int LPM = NW / 2;
        constexpr int NB = 3;
        const int c = threadIdx.x % LPM;
        const int col = colbase + 4 * c;
        const int step = blockDim.x / LPM;
        const unsigned short *eo_s = (fp.eorder && fp.eorder_len == mmax) ? perm_s + n : nullptr;
        const unsigned char *kf_s = eo_s ? reinterpret_cast<const unsigned char *>(eo_s + mmax) : nullptr;
        for (int i0 = threadIdx.x / LPM; i0 < mmax; i0 += NB * step) {
            int mm[NB];
            float4 av[NB], bv[NB];
#pragma unroll
            for (int u = 0; u < NB; ++u) {
                const int i = i0 + u * step;
                int m = -1;
                if (i < mmax) {
                    m = eo_s ? eo_s[i] : i;
                    if (m >= mtop) m = -1;
                }
                mm[u] = m;
                av[u] = bv[u] = make_float4(0.f, 0.f, 0.f, 0.f);
                if (m >= 0 && col < 2 * VEC * nfields) {
                    // (the contraction does not produce rows above the group's polar extent: they are zeros)
                    const int kf = kf_s ? kf_s[m] : 0;
                    if (kn >= (kf & 15) * kBK) av[u] = __ldg(reinterpret_cast<const float4 *>(Y + y_off(2 * m, kn, col, 2 * mmax, ncp)));
                    if (kn >= (kf >> 4) * kBK) bv[u] = __ldg(reinterpret_cast<const float4 *>(Y + y_off(2 * m + 1, kn, col, 2 * mmax, ncp)));
                }
            }
#pragma unroll
            for (int u = 0; u < NB; ++u) {
                const int m = mm[u];
                if (m < 0) continue;
                const float sc = mscale[m];
                const bool edge = (m == 0) || (2 * m == n);
                const int pm = perm_s[m];
                const int pn = perm_s[m == 0 ? 0 : n - m];
                const float e[4] = {av[u].x, av[u].y, av[u].z, av[u].w}, o[4] = {bv[u].x, bv[u].y, bv[u].z, bv[u].w};
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                    // north row spectrum A = even + odd, south row spectrum B = even - odd; Z = A + i B
                    const float ar = sc * (e[2 * h] + o[2 * h]), ai = sc * (e[2 * h + 1] + o[2 * h + 1]);
                    const float br = sc * (e[2 * h] - o[2 * h]), bi = sc * (e[2 * h + 1] - o[2 * h + 1]);
                    float2 *dd = data + (size_t)(2 * c + h) * np;
                    if (edge) {
                        dd[pm] = make_float2(ar, br);  // imaginary parts of DC / Nyquist are dropped
                    } else {
                        dd[pm] = make_float2(ar - bi, ai + br);
                        dd[pn] = make_float2(ar + bi, br - ai);
                    }
                }
            }
        }
    }
    __syncthreads();

    if (f0 + t / VEC < nfields) fft_group<true, G>(CxPacked{data + (size_t)t * np}, fp, tw_s, lane, 1 + t);  // (rows of a transform without a field are not stored)

    // ---- each group stores its own pair of rows ----
    {
        const int f = f0 + t / VEC, comp = t % VEC;
        if (f < nfields) {
            const int ks = nlat - 1 - kn;
            const float2 *src = data + (size_t)t * np;
            float *rn = x + ((size_t)(f * VEC + comp) * nlat + kn) * n;
            float *rs = x + ((size_t)(f * VEC + comp) * nlat + ks) * n;
            if ((n % 4 == 0) && vec4ok) {
                for (int j = lane; j < n / 4; j += GT) {
                    const float4 *s4 = reinterpret_cast<const float4 *>(src + 4 * j);
                    const int sw = (lane >> 2) & 1;  // same bank-conflict-free chunk order as on the analysis side
                    const float4 c0 = s4[sw], c1 = s4[sw ^ 1];
                    const float4 a = sw ? c1 : c0, b = sw ? c0 : c1;
                    reinterpret_cast<float4 *>(rn)[j] = make_float4(a.x, a.z, b.x, b.z);
                    if (ks != kn) reinterpret_cast<float4 *>(rs)[j] = make_float4(a.y, a.w, b.y, b.w);
                }
            } else {
                for (int j = lane; j < n; j += GT) {
                    rn[j] = src[j].x;
                    if (ks != kn) rs[j] = src[j].y;
                }
            }
        }
    }
}

// ------------------------------------------------------------------------------------------------
// plain row transforms (distributed stages): two real rows share one complex transform, one transform per warp
// ------------------------------------------------------------------------------------------------
template <int NW>
__global__ void __launch_bounds__(32 * NW) rfft_rows_kernel(const float *__restrict__ in, float2 *__restrict__ out, FftPlanDev fp, long long nrows, int nmodes,
                                                            float scale) {
    extern __shared__ float2 smem[];
    const int n = fp.n;
    float2 *data = smem;
    float2 *tw_s = data + (size_t)NW * n;
    const unsigned short *perm_s = reinterpret_cast<const unsigned short *>(reinterpret_cast<const unsigned *>(tw_s + fp.tw_pass_total) + fp.bf_total);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    load_tables(fp, tw_s);
    const long long r0 = (long long)blockIdx.x * (2 * NW);
    {
        const long long ra = r0 + 2 * warp, rb = ra + 1;
        float2 *dst = data + (size_t)warp * n;
        for (int j = lane; j < n; j += 32) {
            float a = ra < nrows ? in[ra * n + j] : 0.f;
            float b = rb < nrows ? in[rb * n + j] : 0.f;
            dst[j] = make_float2(a, b);
        }
    }
    __syncthreads();
    fft_group<false, 1>(CxPacked{data + (size_t)warp * n}, fp, tw_s, lane, 0);
    const int nyq = n / 2;
    {
        const long long ra = r0 + 2 * warp, rb = ra + 1;
        const float2 *src = data + (size_t)warp * n;
        for (int m = lane; m < nmodes; m += 32) {
            float2 A = make_float2(0.f, 0.f), B = A;
            if (m <= nyq) {
                float2 zm = src[perm_s[m]];
                float2 zn = src[perm_s[m == 0 ? 0 : n - m]];
                A = make_float2(0.5f * scale * (zm.x + zn.x), 0.5f * scale * (zm.y - zn.y));
                B = make_float2(0.5f * scale * (zm.y + zn.y), -0.5f * scale * (zm.x - zn.x));
            }
            if (ra < nrows) out[ra * nmodes + m] = A;
            if (rb < nrows) out[rb * nmodes + m] = B;
        }
    }
}

template <int NW>
__global__ void __launch_bounds__(32 * NW) irfft_rows_kernel(const float2 *__restrict__ in, float *__restrict__ out, FftPlanDev fp, long long nrows, int nmodes) {
    extern __shared__ float2 smem[];
    const int n = fp.n;
    float2 *data = smem;
    float2 *tw_s = data + (size_t)NW * n;
    const unsigned short *perm_s = reinterpret_cast<const unsigned short *>(reinterpret_cast<const unsigned *>(tw_s + fp.tw_pass_total) + fp.bf_total);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    load_tables(fp, tw_s);
    float2 *dd = data + (size_t)warp * n;
    for (int j = lane; j < n; j += 32) dd[j] = make_float2(0.f, 0.f);
    __syncthreads();
    const long long r0 = (long long)blockIdx.x * (2 * NW);
    const long long ra = r0 + 2 * warp, rb = ra + 1;
    const int nyq = n / 2;
    const int mtop = min(nmodes, nyq + 1);
    for (int m = lane; m < mtop; m += 32) {
        float2 A = ra < nrows ? in[ra * nmodes + m] : make_float2(0.f, 0.f);
        float2 B = rb < nrows ? in[rb * nmodes + m] : make_float2(0.f, 0.f);
        if (m == 0 || 2 * m == n) {
            dd[perm_s[m]] = make_float2(A.x, B.x);
        } else {
            dd[perm_s[m]] = make_float2(A.x - B.y, A.y + B.x);
            dd[perm_s[n - m]] = make_float2(A.x + B.y, B.x - A.y);
        }
    }
    __syncwarp();
    fft_group<true, 1>(CxPacked{dd}, fp, tw_s, lane, 0);
    for (int j = lane; j < n; j += 32) {
        if (ra < nrows) out[ra * n + j] = dd[j].x;
        if (rb < nrows) out[rb * n + j] = dd[j].y;
    }
}

// ------------------------------------------------------------------------------------------------
// launchers
// ------------------------------------------------------------------------------------------------
static size_t fft_smem_bytes(int nffts, const FftPlanDev &fp) {
    const size_t data = fp.ts ? (size_t)nffts * fp.ts * sizeof(float) : (size_t)nffts * fp.np * sizeof(float2);
    return data + (size_t)fp.tab_bytes + 16;
}

template <typename K>
static int set_smem(K kernel, size_t bytes) {
    if (bytes > 227 * 1024) return fail(SHTB200_EINVAL, "nlon too large for the shared-memory FFT");
    SHT_CUDA_CHECK(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes));
    return SHTB200_OK;
}

constexpr int kGroupWarps = 2;  // warps that share one transform

// transforms per CTA: 8 when two such CTAs fit one SM, else 4, else 2
static int pick_warps(const FftPlanDev &fp, int vec) {
    for (int nw = 8; nw > 2 * vec; nw /= 2)
        if (fft_smem_bytes(nw, fp) <= 110 * 1024) return nw;
    return 2 * vec;
}

int launch_fft_analysis(const Plan &pl, const float *x, float *X, int nfields, cudaStream_t st) {
    if (pl.twopass && (((uintptr_t)x | (uintptr_t)X) & 15) == 0) return launch_fft_analysis_twopass(pl, x, X, nfields, st);
    const int vec = pl.vector ? 2 : 1;
    const int NW = pick_warps(pl.fft, vec);
    const int ncp = (int)col_pitch((pl.vector ? 4 : 2) * nfields);
    // one CTA row per latitude pair plus the zero rows that pad the contraction length to a multiple of 32
    dim3 grid(ceil_div(nfields, NW / vec), pl.Kh + (int)(round_up(pl.Ka, kBK) - pl.Ka));
    size_t smem = fft_smem_bytes(NW, pl.fft);
    const int al = (int)((((uintptr_t)x & 15) == 0) && (pl.fft.n % 4 == 0));
    int rc;
#define LAUNCH_A(WW, VV)                                                                                                                    \
    do {                                                                                                                                    \
        if ((rc = set_smem(fft_analysis_kernel<WW, VV, kGroupWarps>, smem)) != 0) return rc;                                                \
        fft_analysis_kernel<WW, VV, kGroupWarps><<<grid, 32 * WW * kGroupWarps, smem, st>>>(x, X, pl.fft, pl.nlat, pl.Kh, nfields, ncp,     \
                                                                                            pl.mmax, pl.d_mscale, pl.zero_imag_edges, al, pl.d_err); \
    } while (0)
    if (vec == 1) {
        if (NW == 8) LAUNCH_A(8, 1);
        else if (NW == 4) LAUNCH_A(4, 1);
        else LAUNCH_A(2, 1);
    } else {
        if (NW == 8) LAUNCH_A(8, 2);
        else LAUNCH_A(4, 2);
    }
#undef LAUNCH_A
    SHT_CUDA_CHECK(cudaGetLastError());
    return SHTB200_OK;
}

int launch_fft_synthesis(const Plan &pl, const float *Y, float *x, int nfields, cudaStream_t st) {
    if (pl.twopass && (((uintptr_t)x | (uintptr_t)Y) & 15) == 0) return launch_fft_synthesis_twopass(pl, Y, x, nfields, st);
    const int vec = pl.vector ? 2 : 1;
    const int NW = pick_warps(pl.fft, vec);
    const int ncp = (int)col_pitch((pl.vector ? 4 : 2) * nfields);
    dim3 grid(ceil_div(nfields, NW / vec), pl.Kh);
    size_t smem = fft_smem_bytes(NW, pl.fft);
    const int al = (int)((((uintptr_t)x & 15) == 0) && (pl.fft.n % 4 == 0));
    int rc;
#define LAUNCH_S(WW, VV)                                                                                                                 \
    do {                                                                                                                                 \
        if ((rc = set_smem(fft_synthesis_kernel<WW, VV, kGroupWarps>, smem)) != 0) return rc;                                            \
        fft_synthesis_kernel<WW, VV, kGroupWarps><<<grid, 32 * WW * kGroupWarps, smem, st>>>(Y, x, pl.fft, pl.nlat, pl.Kh, nfields, ncp, \
                                                                                             pl.mmax, pl.d_mscale, al, pl.d_err); \
    } while (0)
    if (vec == 1) {
        if (NW == 8) LAUNCH_S(8, 1);
        else if (NW == 4) LAUNCH_S(4, 1);
        else LAUNCH_S(2, 1);
    } else {
        if (NW == 8) LAUNCH_S(8, 2);
        else LAUNCH_S(4, 2);
    }
#undef LAUNCH_S
    SHT_CUDA_CHECK(cudaGetLastError());
    return SHTB200_OK;
}

// The stage entry points build their own FFT tables, cached per (nlon, device) for the life of the process.
struct CachedFft {
    int n = 0, device = -1;
    FftPlanDev fp{};
    float2 *tw = nullptr;
    unsigned short *perm = nullptr;
    TwoPassRows rows;        // two-pass kernels' tables (blob == nullptr: no such kernel for this nlon)
    int *h_err = nullptr;    // pinned copy of rows.d_err, refreshed after every launch and looked at by the next call
};
static std::mutex g_cache_mutex;
static std::vector<CachedFft> g_cache;

// Tables for `nlon` on the CURRENT device (the stage calls run on the caller's current device and stream).
static int cached_fft(int nlon, FftPlanDev *fp, TwoPassRows *rows, int **h_err) {
    int dev = 0;
    SHT_CUDA_CHECK(cudaGetDevice(&dev));
    std::lock_guard<std::mutex> lock(g_cache_mutex);
    for (const CachedFft &c : g_cache)
        if (c.n == nlon && c.device == dev) {
            *fp = c.fp;
            *rows = c.rows;
            *h_err = c.h_err;
            return SHTB200_OK;
        }
    CachedFft c;
    int rc = build_fft_plan(nlon, 0, kFftRows, nullptr, &c.fp, &c.tw, &c.perm);
    if (rc) return rc;
    unsigned char *blob = nullptr;
    if ((rc = build_twopass_rows_tables(nlon, &blob, &c.rows.blob_bytes)) != 0) return rc;
    if (blob) {
        c.rows.blob = blob;
        SHT_CUDA_CHECK(cudaDeviceGetAttribute(&c.rows.sm_count, cudaDevAttrMultiProcessorCount, dev));
        SHT_CUDA_CHECK(cudaMalloc(&c.rows.d_err, sizeof(int)));
        SHT_CUDA_CHECK(cudaMemset(c.rows.d_err, 0, sizeof(int)));
        SHT_CUDA_CHECK(cudaHostAlloc(&c.h_err, sizeof(int), cudaHostAllocDefault));
        *c.h_err = 0;
    }
    c.n = nlon;
    c.device = dev;
    g_cache.push_back(c);
    *fp = c.fp;
    *rows = c.rows;
    *h_err = c.h_err;
    return SHTB200_OK;
}

// Two-pass row transforms when there is a kernel for nlon and the rows are 16-byte aligned; *done says whether it ran.
// A bounded wait that ran out inside an earlier launch shows in the pinned copy of the error word: the next call fails.
static int rows_twopass(const TwoPassRows &rows, int *h_err, bool forward, const void *in, void *out, long long nrows, int nlon, int nmodes, float scale,
                        int grid_pieces, int mode_pieces, cudaStream_t st, bool *done) {
    *done = false;
    const void *grid = forward ? in : out;
    if (!rows.blob || ((uintptr_t)grid & 15) != 0) return SHTB200_OK;
    if ((grid_pieces != 1 || mode_pieces != 1) && !rows_pieces_supported(nlon, nmodes, grid_pieces, mode_pieces)) return SHTB200_OK;
    if (*reinterpret_cast<volatile int *>(h_err) != 0) {
        const int v = *h_err;
        *h_err = 0;
        cudaMemsetAsync(rows.d_err, 0, sizeof(int), st);
        return fail(SHTB200_EDEVICE, "a row-transform kernel gave up on a bounded wait (device error word " + std::to_string(v) + ")");
    }
    int rc = launch_rows_twopass(rows, forward, in, out, nrows, nlon, nmodes, scale, grid_pieces, mode_pieces, st);
    if (rc) return rc;
    SHT_CUDA_CHECK(cudaMemcpyAsync(h_err, rows.d_err, sizeof(int), cudaMemcpyDeviceToHost, st));
    *done = true;
    return SHTB200_OK;
}

// grid_pieces / mode_pieces != 1: piece-major buffers (two-pass kernels only; SHTB200_EINVAL where they do not apply)
int launch_rfft_modes(const float *in, float2 *out, long long nrows, int nlon, int nmodes, float scale, int grid_pieces, int mode_pieces, cudaStream_t st) {
    FftPlanDev fp;
    TwoPassRows rows;
    int *h_err = nullptr;
    int rc = cached_fft(nlon, &fp, &rows, &h_err);
    if (rc) return rc;
    if (nrows == 0) return SHTB200_OK;
    bool done = false;
    if ((rc = rows_twopass(rows, h_err, true, in, out, nrows, nlon, nmodes, scale / (float)nlon, grid_pieces, mode_pieces, st, &done)) != 0 || done) return rc;
    if (grid_pieces != 1 || mode_pieces != 1) return fail(SHTB200_EINVAL, "piece-major row transforms need a two-pass kernel for nlon, 16-byte aligned buffers and pieces that are multiples of four longitudes");
    constexpr int NW = 4;
    size_t smem = fft_smem_bytes(NW, fp);
    if ((rc = set_smem(rfft_rows_kernel<NW>, smem)) != 0) return rc;
    long long blocks = (nrows + 2 * NW - 1) / (2 * NW);
    rfft_rows_kernel<NW><<<(unsigned)blocks, 32 * NW, smem, st>>>(in, out, fp, nrows, nmodes, scale / (float)nlon);  // rfft(norm="forward") carries 1/nlon
    SHT_CUDA_CHECK(cudaGetLastError());
    return SHTB200_OK;
}

int launch_irfft_modes(const float2 *in, float *out, long long nrows, int nlon, int nmodes, int mode_pieces, int grid_pieces, cudaStream_t st) {
    FftPlanDev fp;
    TwoPassRows rows;
    int *h_err = nullptr;
    int rc = cached_fft(nlon, &fp, &rows, &h_err);
    if (rc) return rc;
    if (nrows == 0) return SHTB200_OK;
    bool done = false;
    if ((rc = rows_twopass(rows, h_err, false, in, out, nrows, nlon, nmodes, 1.f, grid_pieces, mode_pieces, st, &done)) != 0 || done) return rc;
    if (grid_pieces != 1 || mode_pieces != 1) return fail(SHTB200_EINVAL, "piece-major row transforms need a two-pass kernel for nlon, 16-byte aligned buffers and pieces that are multiples of four longitudes");
    constexpr int NW = 4;
    size_t smem = fft_smem_bytes(NW, fp);
    if ((rc = set_smem(irfft_rows_kernel<NW>, smem)) != 0) return rc;
    long long blocks = (nrows + 2 * NW - 1) / (2 * NW);
    irfft_rows_kernel<NW><<<(unsigned)blocks, 32 * NW, smem, st>>>(in, out, fp, nrows, nmodes);
    SHT_CUDA_CHECK(cudaGetLastError());
    return SHTB200_OK;
}

}  // namespace shtb200
