// Longitude transforms of the SHT: shared-memory mixed-radix FFT kernels.
//
// Analysis (grid -> order-major operand of the Legendre contraction), per CTA:
//   * P pairs of latitude rows (k', nlat-1-k') of one field are loaded with coalesced float4 reads
//     and folded about the equator: z_j = (x_north + x_south) + i (x_north - x_south).  The even /
//     odd combinations are what the parity-split Legendre tables contract with, and one complex
//     transform of z yields the spectra of both real rows at once.
//   * an in-place decimation-in-frequency FFT of length nlon runs in shared memory (radix 4, 2, 3, 5
//     butterflies; any other prime factor <= 31 goes through a generic butterfly),
//   * only the retained orders m < mmax are written, already transposed into the contraction's
//     operand layout X[group = 2 m + parity][column = 2 field + re/im][k'] (k' contiguous).
// Synthesis is the mirror image: gather the two parities, rebuild the Hermitian spectrum of
// (north + i south), decimation-in-time inverse FFT, coalesced float4 row stores.
//
// Replaces torch_harmonics/fft.py:52-68 (rfft wrapper), :71-96 (irfft wrapper) and the
// scale / transpose / real-imag split passes at torch_harmonics/sht.py:171-176 and :337-340.

#include <math.h>

#include <vector>

#include "common.cuh"

namespace shtb200 {

// ------------------------------------------------------------------------------------------------
// host: factorisation, twiddles, output permutation
// ------------------------------------------------------------------------------------------------
int build_fft_plan(int nlon, FftPlanDev *out, float2 **d_tw, unsigned short **d_perm) {
    if (nlon < 2 || nlon > 65535) return fail(SHTB200_EINVAL, "nlon must be in [2, 65535]");
    std::vector<int> rad;
    int n = nlon;
    while (n % 4 == 0) { rad.push_back(4); n /= 4; }
    while (n % 2 == 0) { rad.push_back(2); n /= 2; }
    while (n % 3 == 0) { rad.push_back(3); n /= 3; }
    while (n % 5 == 0) { rad.push_back(5); n /= 5; }
    for (int p = 7; p <= 31 && n > 1; p += 2) {
        while (n % p == 0) { rad.push_back(p); n /= p; }
    }
    if (n != 1) return fail(SHTB200_EINVAL, "nlon has a prime factor larger than 31");
    if ((int)rad.size() > kMaxFftStages) return fail(SHTB200_EINVAL, "nlon has too many factors");

    FftPlanDev fp{};
    fp.n = nlon;
    fp.nstages = (int)rad.size();
    int L = nlon;
    for (int s = 0; s < fp.nstages; ++s) {
        fp.radix[s] = rad[s];
        fp.sublen[s] = L;
        L /= rad[s];
    }
    std::vector<float2> tw(nlon);
    for (int k = 0; k < nlon; ++k) {
        double a = -2.0 * M_PI * (double)k / (double)nlon;
        tw[k] = make_float2((float)cos(a), (float)sin(a));
    }
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
    SHT_CUDA_CHECK(cudaMalloc(d_tw, sizeof(float2) * nlon));
    SHT_CUDA_CHECK(cudaMalloc(d_perm, sizeof(unsigned short) * nlon));
    SHT_CUDA_CHECK(cudaMemcpy(*d_tw, tw.data(), sizeof(float2) * nlon, cudaMemcpyHostToDevice));
    SHT_CUDA_CHECK(cudaMemcpy(*d_perm, perm.data(), sizeof(unsigned short) * nlon, cudaMemcpyHostToDevice));
    fp.tw = *d_tw;
    fp.perm = *d_perm;
    *out = fp;
    return SHTB200_OK;
}

// ------------------------------------------------------------------------------------------------
// device: butterflies
// ------------------------------------------------------------------------------------------------
__device__ __forceinline__ float2 cmul(float2 a, float2 b) { return make_float2(a.x * b.x - a.y * b.y, a.x * b.y + a.y * b.x); }
__device__ __forceinline__ float2 cmulc(float2 a, float2 b) {  // a * conj(b)
    return make_float2(a.x * b.x + a.y * b.y, a.y * b.x - a.x * b.y);
}
__device__ __forceinline__ float2 cadd(float2 a, float2 b) { return make_float2(a.x + b.x, a.y + b.y); }
__device__ __forceinline__ float2 csub(float2 a, float2 b) { return make_float2(a.x - b.x, a.y - b.y); }
// multiply by -i (forward) or +i (inverse)
template <bool INV>
__device__ __forceinline__ float2 rot(float2 a) {
    return INV ? make_float2(-a.y, a.x) : make_float2(a.y, -a.x);
}

template <bool INV>
__device__ __forceinline__ void dft2(float2 *v) {
    float2 a = v[0], b = v[1];
    v[0] = cadd(a, b);
    v[1] = csub(a, b);
}

template <bool INV>
__device__ __forceinline__ void dft3(float2 *v) {
    const float s = 0.86602540378443864676f;
    float2 t = cadd(v[1], v[2]);
    float2 d = rot<INV>(csub(v[1], v[2]));  // -+ i (v1 - v2)
    float2 h = make_float2(v[0].x - 0.5f * t.x, v[0].y - 0.5f * t.y);
    v[0] = cadd(v[0], t);
    v[1] = make_float2(h.x + s * d.x, h.y + s * d.y);
    v[2] = make_float2(h.x - s * d.x, h.y - s * d.y);
}

template <bool INV>
__device__ __forceinline__ void dft4(float2 *v) {
    float2 t0 = cadd(v[0], v[2]), t1 = csub(v[0], v[2]);
    float2 t2 = cadd(v[1], v[3]), t3 = rot<INV>(csub(v[1], v[3]));
    v[0] = cadd(t0, t2);
    v[2] = csub(t0, t2);
    v[1] = cadd(t1, t3);
    v[3] = csub(t1, t3);
}

template <bool INV>
__device__ __forceinline__ void dft5(float2 *v) {
    const float c1 = 0.30901699437494742410f, c2 = -0.80901699437494742410f;
    const float s1 = 0.95105651629515357212f, s2 = 0.58778525229247312917f;
    float2 a1 = cadd(v[1], v[4]), a2 = cadd(v[2], v[3]);
    float2 b1 = csub(v[1], v[4]), b2 = csub(v[2], v[3]);
    float2 p1 = make_float2(v[0].x + c1 * a1.x + c2 * a2.x, v[0].y + c1 * a1.y + c2 * a2.y);
    float2 p2 = make_float2(v[0].x + c2 * a1.x + c1 * a2.x, v[0].y + c2 * a1.y + c1 * a2.y);
    float2 q1 = rot<INV>(make_float2(s1 * b1.x + s2 * b2.x, s1 * b1.y + s2 * b2.y));
    float2 q2 = rot<INV>(make_float2(s2 * b1.x - s1 * b2.x, s2 * b1.y - s1 * b2.y));
    v[0] = make_float2(v[0].x + a1.x + a2.x, v[0].y + a1.y + a2.y);
    v[1] = cadd(p1, q1);
    v[4] = csub(p1, q1);
    v[2] = cadd(p2, q2);
    v[3] = csub(p2, q2);
}

// Any other prime radix: plain O(R^2) DFT with twiddles taken from the length-n table.
template <bool INV>
__device__ void dft_generic(float2 *v, int R, const float2 *tw, int n) {
    float2 y[31];
    const int step = n / R;
    for (int q = 0; q < R; ++q) {
        float2 acc = v[0];
        int idx = 0;
        for (int r = 1; r < R; ++r) {
            idx += q;
            if (idx >= R) idx -= R;
            float2 w = tw[idx * step];
            acc = cadd(acc, INV ? cmulc(v[r], w) : cmul(v[r], w));
        }
        y[q] = acc;
    }
    for (int q = 0; q < R; ++q) v[q] = y[q];
}

// One decimation-in-frequency butterfly of radix R on d[0], d[str], ..., then the inter-stage twiddles
// w_L^{j q}; `twstep` = j * (n / L).
template <int R>
__device__ __forceinline__ void dif_butterfly(float2 *d, int str, int twstep, const float2 *tw) {
    float2 v[R];
#pragma unroll
    for (int r = 0; r < R; ++r) v[r] = d[r * str];
    if (R == 2) dft2<false>(v);
    if (R == 3) dft3<false>(v);
    if (R == 4) dft4<false>(v);
    if (R == 5) dft5<false>(v);
    d[0] = v[0];
    if (twstep) {
#pragma unroll
        for (int q = 1; q < R; ++q) d[q * str] = cmul(v[q], tw[q * twstep]);
    } else {
#pragma unroll
        for (int q = 1; q < R; ++q) d[q * str] = v[q];
    }
}

// Decimation-in-time butterfly of the inverse transform: conjugate twiddles first, then conjugate DFT.
template <int R>
__device__ __forceinline__ void dit_butterfly(float2 *d, int str, int twstep, const float2 *tw) {
    float2 v[R];
    v[0] = d[0];
    if (twstep) {
#pragma unroll
        for (int r = 1; r < R; ++r) v[r] = cmulc(d[r * str], tw[r * twstep]);
    } else {
#pragma unroll
        for (int r = 1; r < R; ++r) v[r] = d[r * str];
    }
    if (R == 2) dft2<true>(v);
    if (R == 3) dft3<true>(v);
    if (R == 4) dft4<true>(v);
    if (R == 5) dft5<true>(v);
#pragma unroll
    for (int q = 0; q < R; ++q) d[q * str] = v[q];
}

__device__ void generic_butterfly(float2 *d, int R, int str, int twstep, const float2 *tw, int n, bool inverse) {
    float2 v[31];
    if (!inverse) {
        for (int r = 0; r < R; ++r) v[r] = d[r * str];
        dft_generic<false>(v, R, tw, n);
        d[0] = v[0];
        for (int q = 1; q < R; ++q) d[q * str] = twstep ? cmul(v[q], tw[(q * twstep) % n]) : v[q];
    } else {
        v[0] = d[0];
        for (int r = 1; r < R; ++r) v[r] = twstep ? cmulc(d[r * str], tw[(r * twstep) % n]) : d[r * str];
        dft_generic<true>(v, R, tw, n);
        for (int q = 0; q < R; ++q) d[q * str] = v[q];
    }
}

// All passes over `nfft` transforms of length n stored back to back in `data` (in place).
// Forward: natural order in, bin k at slot perm[k] out.  Inverse: bin k at slot perm[k] in, natural order out.
template <bool INV>
__device__ void fft_passes(float2 *data, int nfft, const FftPlanDev &fp, const float2 *tw) {
    const int n = fp.n;
    for (int ss = 0; ss < fp.nstages; ++ss) {
        const int s = INV ? fp.nstages - 1 - ss : ss;
        const int R = fp.radix[s];
        const int L = fp.sublen[s];
        const int Ls = L / R;   // stride between butterfly legs
        const int nb = n / R;   // butterflies per transform
        const int twmul = n / L;
        const int total = nfft * nb;
        for (int i = threadIdx.x; i < total; i += blockDim.x) {
            int q = i / nb;
            int bj = i - q * nb;
            int b = bj / Ls;
            int j = bj - b * Ls;
            float2 *d = data + q * n + b * L + j;
            int twstep = j * twmul;
            if (!INV) {
                switch (R) {
                    case 4: dif_butterfly<4>(d, Ls, twstep, tw); break;
                    case 2: dif_butterfly<2>(d, Ls, twstep, tw); break;
                    case 3: dif_butterfly<3>(d, Ls, twstep, tw); break;
                    case 5: dif_butterfly<5>(d, Ls, twstep, tw); break;
                    default: generic_butterfly(d, R, Ls, twstep, tw, n, false);
                }
            } else {
                switch (R) {
                    case 4: dit_butterfly<4>(d, Ls, twstep, tw); break;
                    case 2: dit_butterfly<2>(d, Ls, twstep, tw); break;
                    case 3: dit_butterfly<3>(d, Ls, twstep, tw); break;
                    case 5: dit_butterfly<5>(d, Ls, twstep, tw); break;
                    default: generic_butterfly(d, R, Ls, twstep, tw, n, true);
                }
            }
        }
        __syncthreads();
    }
}

// shared memory: [P * ncomp * n float2 data][n float2 twiddles][n u16 perm]
__device__ __forceinline__ void load_tables(const FftPlanDev &fp, float2 *tw_s, unsigned short *perm_s) {
    for (int i = threadIdx.x; i < fp.n; i += blockDim.x) {
        tw_s[i] = fp.tw[i];
        perm_s[i] = fp.perm[i];
    }
}

// ------------------------------------------------------------------------------------------------
// analysis kernel
// ------------------------------------------------------------------------------------------------
// grid: (ceil(Kh / P), nfields).  VEC = 1: scalar fields; VEC = 2: (theta, phi) component pairs.
//
// Scalar operand layout   X[(2 m + p) * ncols + 2 f + ri][k'],  p = 0 even fold, p = 1 odd fold.
// Vector operand layout   X[(2 m + p) * ncols + 4 f + c][seg * Kp + k'] with seg 0 contracting against
// the d/dtheta table (fold parity opposite to p) and seg 1 against the m/sin(theta) table (fold parity p);
// the four columns c carry the sign pattern of torch_harmonics/sht.py:488-493:
//   c0 (s_re): [ Re X0 | -Im X1 ]   c1 (s_im): [ Im X0 |  Re X1 ]
//   c2 (t_re): [-Re X1 | -Im X0 ]   c3 (t_im): [-Im X1 |  Re X0 ]
template <int P, int VEC>
__global__ void __launch_bounds__(256) fft_analysis_kernel(const float *__restrict__ x, float *__restrict__ X, FftPlanDev fp, int nlat, int Kh, int Kp,
                                                           int mmax, int ncols, const float *__restrict__ mscale, int zero_imag_edges, int vec4ok) {
    extern __shared__ float2 smem[];
    const int n = fp.n;
    constexpr int NF = P * VEC;
    float2 *data = smem;
    float2 *tw_s = data + (size_t)NF * n;
    unsigned short *perm_s = reinterpret_cast<unsigned short *>(tw_s + n);

    const int f = blockIdx.y;
    const int k0 = blockIdx.x * P;
    load_tables(fp, tw_s, perm_s);

    // ---- load + fold ----
    const bool vec4 = (n % 4 == 0) && vec4ok;
    for (int t = 0; t < NF; ++t) {
        const int q = t % P, comp = t / P;
        const int kn = k0 + q;
        float2 *dst = data + (size_t)t * n;
        if (kn >= Kh) {
            for (int j = threadIdx.x; j < n; j += blockDim.x) dst[j] = make_float2(0.f, 0.f);
            continue;
        }
        const int ks = nlat - 1 - kn;
        const float *rn = x + ((size_t)(f * VEC + comp) * nlat + kn) * n;
        const float *rs = x + ((size_t)(f * VEC + comp) * nlat + ks) * n;
        const bool self = (ks == kn);
        if (vec4) {
            const float4 *rn4 = reinterpret_cast<const float4 *>(rn);
            const float4 *rs4 = reinterpret_cast<const float4 *>(rs);
            for (int j = threadIdx.x; j < n / 4; j += blockDim.x) {
                float4 a = __ldg(rn4 + j);
                float4 b = self ? make_float4(0.f, 0.f, 0.f, 0.f) : __ldg(rs4 + j);
                if (self) {
                    dst[4 * j + 0] = make_float2(a.x, 0.f);
                    dst[4 * j + 1] = make_float2(a.y, 0.f);
                    dst[4 * j + 2] = make_float2(a.z, 0.f);
                    dst[4 * j + 3] = make_float2(a.w, 0.f);
                } else {
                    dst[4 * j + 0] = make_float2(a.x + b.x, a.x - b.x);
                    dst[4 * j + 1] = make_float2(a.y + b.y, a.y - b.y);
                    dst[4 * j + 2] = make_float2(a.z + b.z, a.z - b.z);
                    dst[4 * j + 3] = make_float2(a.w + b.w, a.w - b.w);
                }
            }
        } else {
            for (int j = threadIdx.x; j < n; j += blockDim.x) {
                float a = __ldg(rn + j);
                float b = self ? 0.f : __ldg(rs + j);
                dst[j] = self ? make_float2(a, 0.f) : make_float2(a + b, a - b);
            }
        }
    }
    __syncthreads();

    fft_passes<false>(data, NF, fp, tw_s);

    // ---- emit the retained orders ----
    const int nyq = n / 2;
    for (int m = threadIdx.x; m < mmax; m += blockDim.x) {
        float e_re[NF], e_im[NF], o_re[NF], o_im[NF];
        if (m <= nyq) {
            const float sc = mscale[m];
            const int pm = perm_s[m];
            const int pn = perm_s[m == 0 ? 0 : n - m];
            const bool edge = zero_imag_edges && (m == 0 || (2 * m == n));
#pragma unroll
            for (int t = 0; t < NF; ++t) {
                float2 zm = data[(size_t)t * n + pm];
                float2 zn = data[(size_t)t * n + pn];
                // spectra of the two real rows packed in z = even + i odd
                e_re[t] = 0.5f * sc * (zm.x + zn.x);
                e_im[t] = edge ? 0.f : 0.5f * sc * (zm.y - zn.y);
                o_re[t] = 0.5f * sc * (zm.y + zn.y);
                o_im[t] = edge ? 0.f : -0.5f * sc * (zm.x - zn.x);
            }
        } else {
#pragma unroll
            for (int t = 0; t < NF; ++t) e_re[t] = e_im[t] = o_re[t] = o_im[t] = 0.f;
        }
        if (VEC == 1) {
            float *g0 = X + ((size_t)(2 * m) * ncols + 2 * f) * Kp + k0;
            float *g1 = X + ((size_t)(2 * m + 1) * ncols + 2 * f) * Kp + k0;
#pragma unroll
            for (int q4 = 0; q4 < P; q4 += 4) {
                *reinterpret_cast<float4 *>(g0 + q4) = make_float4(e_re[q4], e_re[q4 + 1], e_re[q4 + 2], e_re[q4 + 3]);
                *reinterpret_cast<float4 *>(g0 + Kp + q4) = make_float4(e_im[q4], e_im[q4 + 1], e_im[q4 + 2], e_im[q4 + 3]);
                *reinterpret_cast<float4 *>(g1 + q4) = make_float4(o_re[q4], o_re[q4 + 1], o_re[q4 + 2], o_re[q4 + 3]);
                *reinterpret_cast<float4 *>(g1 + Kp + q4) = make_float4(o_im[q4], o_im[q4 + 1], o_im[q4 + 2], o_im[q4 + 3]);
            }
        } else {
            // component 0 occupies t in [0, P), component 1 t in [P, 2P)
            const size_t pitch = 2 * (size_t)Kp;
#pragma unroll
            for (int p = 0; p < 2; ++p) {
                float *g = X + ((size_t)(2 * m + p) * ncols + 4 * f) * pitch + k0;
                // seg 0 (d/dtheta table) takes the fold of parity 1 - p, seg 1 the fold of parity p
#pragma unroll
                for (int q = 0; q < P; ++q) {
                    const float x0re_a = p ? e_re[q] : o_re[q], x0im_a = p ? e_im[q] : o_im[q];          // X0, fold 1-p
                    const float x1re_a = p ? e_re[P + q] : o_re[P + q], x1im_a = p ? e_im[P + q] : o_im[P + q];  // X1, fold 1-p
                    const float x0re_b = p ? o_re[q] : e_re[q], x0im_b = p ? o_im[q] : e_im[q];          // X0, fold p
                    const float x1re_b = p ? o_re[P + q] : e_re[P + q], x1im_b = p ? o_im[P + q] : e_im[P + q];  // X1, fold p
                    g[0 * pitch + q] = x0re_a;
                    g[0 * pitch + Kp + q] = -x1im_b;
                    g[1 * pitch + q] = x0im_a;
                    g[1 * pitch + Kp + q] = x1re_b;
                    g[2 * pitch + q] = -x1re_a;
                    g[2 * pitch + Kp + q] = -x0im_b;
                    g[3 * pitch + q] = -x1im_a;
                    g[3 * pitch + Kp + q] = x0re_b;
                }
            }
        }
    }
}

// ------------------------------------------------------------------------------------------------
// synthesis kernel
// ------------------------------------------------------------------------------------------------
// Scalar: Y[(2 m + p) * ncols + 2 f + ri][k'] holds the even (p = 0) / odd (p = 1) latitude parts of order m.
// Vector: Y[(2 m + p) * ncols + 4 f + c][k'] with c = (theta re, theta im, phi re, phi im).
template <int P, int VEC>
__global__ void __launch_bounds__(256) fft_synthesis_kernel(const float *__restrict__ Y, float *__restrict__ x, FftPlanDev fp, int nlat, int Kh, int Kp,
                                                            int mmax, int ncols, const float *__restrict__ mscale, int vec4ok) {
    extern __shared__ float2 smem[];
    const int n = fp.n;
    constexpr int NF = P * VEC;
    float2 *data = smem;
    float2 *tw_s = data + (size_t)NF * n;
    unsigned short *perm_s = reinterpret_cast<unsigned short *>(tw_s + n);

    const int f = blockIdx.y;
    const int k0 = blockIdx.x * P;
    load_tables(fp, tw_s, perm_s);
    for (int i = threadIdx.x; i < NF * n; i += blockDim.x) data[i] = make_float2(0.f, 0.f);
    __syncthreads();

    const int nyq = n / 2;
    const int mtop = min(mmax, nyq + 1);
    for (int i = threadIdx.x; i < mtop * VEC; i += blockDim.x) {
        const int m = i % mtop, comp = i / mtop;
        const float sc = mscale[m];
        const float *ge = Y + ((size_t)(2 * m) * ncols + (2 * VEC) * f + 2 * comp) * Kp + k0;
        const float *go = Y + ((size_t)(2 * m + 1) * ncols + (2 * VEC) * f + 2 * comp) * Kp + k0;
        float er[P], ei[P], orr[P], oi[P];
#pragma unroll
        for (int q4 = 0; q4 < P; q4 += 4) {
            float4 a = *reinterpret_cast<const float4 *>(ge + q4);
            float4 b = *reinterpret_cast<const float4 *>(ge + Kp + q4);
            float4 c = *reinterpret_cast<const float4 *>(go + q4);
            float4 d = *reinterpret_cast<const float4 *>(go + Kp + q4);
            er[q4] = a.x; er[q4 + 1] = a.y; er[q4 + 2] = a.z; er[q4 + 3] = a.w;
            ei[q4] = b.x; ei[q4 + 1] = b.y; ei[q4 + 2] = b.z; ei[q4 + 3] = b.w;
            orr[q4] = c.x; orr[q4 + 1] = c.y; orr[q4 + 2] = c.z; orr[q4 + 3] = c.w;
            oi[q4] = d.x; oi[q4 + 1] = d.y; oi[q4 + 2] = d.z; oi[q4 + 3] = d.w;
        }
        const bool edge = (m == 0) || (2 * m == n);
        const int pm = perm_s[m];
        const int pn = perm_s[m == 0 ? 0 : n - m];
#pragma unroll
        for (int q = 0; q < P; ++q) {
            // north row spectrum A = even + odd, south row spectrum B = even - odd; Z = A + i B
            float ar = sc * (er[q] + orr[q]), ai = sc * (ei[q] + oi[q]);
            float br = sc * (er[q] - orr[q]), bi = sc * (ei[q] - oi[q]);
            float2 *dd = data + (size_t)(comp * P + q) * n;
            if (edge) {
                dd[pm] = make_float2(ar, br);  // imaginary parts of DC / Nyquist are dropped
            } else {
                dd[pm] = make_float2(ar - bi, ai + br);
                dd[pn] = make_float2(ar + bi, br - ai);
            }
        }
    }
    __syncthreads();

    fft_passes<true>(data, NF, fp, tw_s);

    const bool vec4 = (n % 4 == 0) && vec4ok;
    for (int t = 0; t < NF; ++t) {
        const int q = t % P, comp = t / P;
        const int kn = k0 + q;
        if (kn >= Kh) continue;
        const int ks = nlat - 1 - kn;
        const float2 *src = data + (size_t)t * n;
        float *rn = x + ((size_t)(f * VEC + comp) * nlat + kn) * n;
        float *rs = x + ((size_t)(f * VEC + comp) * nlat + ks) * n;
        if (vec4) {
            for (int j = threadIdx.x; j < n / 4; j += blockDim.x) {
                float2 a = src[4 * j], b = src[4 * j + 1], c = src[4 * j + 2], d = src[4 * j + 3];
                reinterpret_cast<float4 *>(rn)[j] = make_float4(a.x, b.x, c.x, d.x);
                if (ks != kn) reinterpret_cast<float4 *>(rs)[j] = make_float4(a.y, b.y, c.y, d.y);
            }
        } else {
            for (int j = threadIdx.x; j < n; j += blockDim.x) {
                rn[j] = src[j].x;
                if (ks != kn) rs[j] = src[j].y;
            }
        }
    }
}

// ------------------------------------------------------------------------------------------------
// plain row transforms (distributed stages): one real row per transform slot, two rows share a complex FFT
// ------------------------------------------------------------------------------------------------
template <int P>
__global__ void __launch_bounds__(256) rfft_rows_kernel(const float *__restrict__ in, float2 *__restrict__ out, FftPlanDev fp, long long nrows, int nmodes,
                                                        float scale) {
    extern __shared__ float2 smem[];
    const int n = fp.n;
    float2 *data = smem;
    float2 *tw_s = data + (size_t)P * n;
    unsigned short *perm_s = reinterpret_cast<unsigned short *>(tw_s + n);
    load_tables(fp, tw_s, perm_s);
    const long long r0 = (long long)blockIdx.x * (2 * P);
    for (int t = 0; t < P; ++t) {
        const long long ra = r0 + 2 * t, rb = ra + 1;
        float2 *dst = data + (size_t)t * n;
        for (int j = threadIdx.x; j < n; j += blockDim.x) {
            float a = ra < nrows ? in[ra * n + j] : 0.f;
            float b = rb < nrows ? in[rb * n + j] : 0.f;
            dst[j] = make_float2(a, b);
        }
    }
    __syncthreads();
    fft_passes<false>(data, P, fp, tw_s);
    const int nyq = n / 2;
    for (int i = threadIdx.x; i < P * nmodes; i += blockDim.x) {
        const int t = i / nmodes, m = i - t * nmodes;
        const long long ra = r0 + 2 * t, rb = ra + 1;
        float2 A = make_float2(0.f, 0.f), B = A;
        if (m <= nyq) {
            float2 zm = data[(size_t)t * n + perm_s[m]];
            float2 zn = data[(size_t)t * n + perm_s[m == 0 ? 0 : n - m]];
            A = make_float2(0.5f * scale * (zm.x + zn.x), 0.5f * scale * (zm.y - zn.y));
            B = make_float2(0.5f * scale * (zm.y + zn.y), -0.5f * scale * (zm.x - zn.x));
        }
        if (ra < nrows) out[ra * nmodes + m] = A;
        if (rb < nrows) out[rb * nmodes + m] = B;
    }
}

template <int P>
__global__ void __launch_bounds__(256) irfft_rows_kernel(const float2 *__restrict__ in, float *__restrict__ out, FftPlanDev fp, long long nrows, int nmodes) {
    extern __shared__ float2 smem[];
    const int n = fp.n;
    float2 *data = smem;
    float2 *tw_s = data + (size_t)P * n;
    unsigned short *perm_s = reinterpret_cast<unsigned short *>(tw_s + n);
    load_tables(fp, tw_s, perm_s);
    for (int i = threadIdx.x; i < P * n; i += blockDim.x) data[i] = make_float2(0.f, 0.f);
    __syncthreads();
    const long long r0 = (long long)blockIdx.x * (2 * P);
    const int nyq = n / 2;
    const int mtop = min(nmodes, nyq + 1);
    for (int i = threadIdx.x; i < P * mtop; i += blockDim.x) {
        const int t = i / mtop, m = i - t * mtop;
        const long long ra = r0 + 2 * t, rb = ra + 1;
        float2 A = ra < nrows ? in[ra * nmodes + m] : make_float2(0.f, 0.f);
        float2 B = rb < nrows ? in[rb * nmodes + m] : make_float2(0.f, 0.f);
        float2 *dd = data + (size_t)t * n;
        if (m == 0 || 2 * m == n) {
            dd[perm_s[m]] = make_float2(A.x, B.x);
        } else {
            dd[perm_s[m]] = make_float2(A.x - B.y, A.y + B.x);
            dd[perm_s[n - m]] = make_float2(A.x + B.y, B.x - A.y);
        }
    }
    __syncthreads();
    fft_passes<true>(data, P, fp, tw_s);
    for (int t = 0; t < P; ++t) {
        const long long ra = r0 + 2 * t, rb = ra + 1;
        const float2 *src = data + (size_t)t * n;
        for (int j = threadIdx.x; j < n; j += blockDim.x) {
            if (ra < nrows) out[ra * n + j] = src[j].x;
            if (rb < nrows) out[rb * n + j] = src[j].y;
        }
    }
}

// ------------------------------------------------------------------------------------------------
// launchers
// ------------------------------------------------------------------------------------------------
static size_t fft_smem_bytes(int nffts, int n) { return (size_t)nffts * n * sizeof(float2) + (size_t)n * sizeof(float2) + (size_t)n * sizeof(unsigned short) + 16; }

template <typename K>
static int set_smem(K kernel, size_t bytes) {
    if (bytes > 227 * 1024) return fail(SHTB200_EINVAL, "nlon too large for the shared-memory FFT");
    SHT_CUDA_CHECK(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes));
    return SHTB200_OK;
}

// pairs of rows per CTA: 8 when it fits comfortably (32-byte runs along k'), else 4
static int pick_pairs(int n, int vec) { return ((size_t)8 * vec * n * sizeof(float2) <= 100 * 1024) ? 8 : 4; }

int launch_fft_analysis(const Plan &pl, const float *x, float *X, int nfields, cudaStream_t st) {
    const int vec = pl.vector ? 2 : 1;
    const int P = pick_pairs(pl.nlon, vec);
    const int ncols = (pl.vector ? 4 : 2) * nfields;
    dim3 grid(pl.Kp / P, nfields);  // covers the row padding [Kh, Kp) too, which must hold zeros
    size_t smem = fft_smem_bytes(P * vec, pl.nlon);
    int rc;
#define LAUNCH_A(PP, VV)                                                                                                           \
    do {                                                                                                                           \
        if ((rc = set_smem(fft_analysis_kernel<PP, VV>, smem)) != 0) return rc;                                                    \
        fft_analysis_kernel<PP, VV><<<grid, 256, smem, st>>>(x, X, pl.fft, pl.nlat, pl.Kh, pl.Kp, pl.mmax, ncols, pl.d_mscale,    \
                                                             pl.zero_imag_edges, (int)(((uintptr_t)x & 15) == 0));                                                  \
    } while (0)
    if (P == 8 && vec == 1) LAUNCH_A(8, 1);
    else if (P == 4 && vec == 1) LAUNCH_A(4, 1);
    else if (P == 8 && vec == 2) LAUNCH_A(8, 2);
    else LAUNCH_A(4, 2);
#undef LAUNCH_A
    SHT_CUDA_CHECK(cudaGetLastError());
    return SHTB200_OK;
}

int launch_fft_synthesis(const Plan &pl, const float *Y, float *x, int nfields, cudaStream_t st) {
    const int vec = pl.vector ? 2 : 1;
    const int P = pick_pairs(pl.nlon, vec);
    const int ncols = (pl.vector ? 4 : 2) * nfields;
    dim3 grid(ceil_div(pl.Kh, P), nfields);
    size_t smem = fft_smem_bytes(P * vec, pl.nlon);
    int rc;
#define LAUNCH_S(PP, VV)                                                                                                    \
    do {                                                                                                                    \
        if ((rc = set_smem(fft_synthesis_kernel<PP, VV>, smem)) != 0) return rc;                                            \
        fft_synthesis_kernel<PP, VV><<<grid, 256, smem, st>>>(Y, x, pl.fft, pl.nlat, pl.Kh, pl.Kp, pl.mmax, ncols, pl.d_mscale, (int)(((uintptr_t)x & 15) == 0)); \
    } while (0)
    if (P == 8 && vec == 1) LAUNCH_S(8, 1);
    else if (P == 4 && vec == 1) LAUNCH_S(4, 1);
    else if (P == 8 && vec == 2) LAUNCH_S(8, 2);
    else LAUNCH_S(4, 2);
#undef LAUNCH_S
    SHT_CUDA_CHECK(cudaGetLastError());
    return SHTB200_OK;
}

// The stage entry points build (and cache per nlon) their own FFT tables.
struct CachedFft {
    int n = 0, device = -1;
    FftPlanDev fp{};
    float2 *tw = nullptr;
    unsigned short *perm = nullptr;
};
static CachedFft g_cache[8];

static int cached_fft(int nlon, FftPlanDev *fp) {
    int dev = 0;
    SHT_CUDA_CHECK(cudaGetDevice(&dev));
    for (auto &c : g_cache)
        if (c.n == nlon && c.device == dev) { *fp = c.fp; return SHTB200_OK; }
    for (auto &c : g_cache)
        if (c.n == 0) {
            int rc = build_fft_plan(nlon, &c.fp, &c.tw, &c.perm);
            if (rc) return rc;
            c.n = nlon;
            c.device = dev;
            *fp = c.fp;
            return SHTB200_OK;
        }
    return fail(SHTB200_EINVAL, "too many distinct nlon values in the stage FFT cache");
}

int launch_rfft_modes(const float *in, float2 *out, long long nrows, int nlon, int nmodes, float scale, cudaStream_t st) {
    FftPlanDev fp;
    int rc = cached_fft(nlon, &fp);
    if (rc) return rc;
    constexpr int P = 4;
    size_t smem = fft_smem_bytes(P, nlon);
    if ((rc = set_smem(rfft_rows_kernel<P>, smem)) != 0) return rc;
    long long blocks = (nrows + 2 * P - 1) / (2 * P);
    if (blocks == 0) return SHTB200_OK;
    rfft_rows_kernel<P><<<(unsigned)blocks, 256, smem, st>>>(in, out, fp, nrows, nmodes, scale / (float)nlon);  // rfft(norm="forward") carries 1/nlon
    SHT_CUDA_CHECK(cudaGetLastError());
    return SHTB200_OK;
}

int launch_irfft_modes(const float2 *in, float *out, long long nrows, int nlon, int nmodes, cudaStream_t st) {
    FftPlanDev fp;
    int rc = cached_fft(nlon, &fp);
    if (rc) return rc;
    constexpr int P = 4;
    size_t smem = fft_smem_bytes(P, nlon);
    if ((rc = set_smem(irfft_rows_kernel<P>, smem)) != 0) return rc;
    long long blocks = (nrows + 2 * P - 1) / (2 * P);
    if (blocks == 0) return SHTB200_OK;
    irfft_rows_kernel<P><<<(unsigned)blocks, 256, smem, st>>>(in, out, fp, nrows, nmodes);
    SHT_CUDA_CHECK(cudaGetLastError());
    return SHTB200_OK;
}

}  // namespace shtb200
