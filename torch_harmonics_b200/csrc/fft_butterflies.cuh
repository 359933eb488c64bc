// In-register discrete Fourier transforms of small size (the butterflies of the longitude FFT kernels).
#pragma once

#include <cuda_runtime.h>

#include "fft_consts.cuh"

namespace shtb200 {

// ------------------------------------------------------------------------------------------------
// device: butterflies (complex values as float2; adds use the packed two-lane fp32 instructions of sm_100)
// ------------------------------------------------------------------------------------------------
__device__ __forceinline__ float2 cadd(float2 a, float2 b) { return __fadd2_rn(a, b); }
__device__ __forceinline__ float2 csub(float2 a, float2 b) { return __ffma2_rn(b, make_float2(-1.f, -1.f), a); }
// a + s * b with a real scalar s
__device__ __forceinline__ float2 caxpy(float s, float2 b, float2 a) { return __ffma2_rn(make_float2(s, s), b, a); }
__device__ __forceinline__ float2 cmul(float2 a, float2 b) { return make_float2(a.x * b.x - a.y * b.y, a.x * b.y + a.y * b.x); }
__device__ __forceinline__ float2 cmulc(float2 a, float2 b) {  // a * conj(b)
    return make_float2(a.x * b.x + a.y * b.y, a.y * b.x - a.x * b.y);
}
// multiply by -i (forward) or +i (inverse)
template <bool INV>
__device__ __forceinline__ float2 rot(float2 a) {
    return INV ? make_float2(-a.y, a.x) : make_float2(a.y, -a.x);
}

template <int R, bool INV>
struct Dft;

template <bool INV>
struct Dft<2, INV> {
    static __device__ __forceinline__ void run(float2 *v) {
        float2 a = v[0], b = v[1];
        v[0] = cadd(a, b);
        v[1] = csub(a, b);
    }
};

template <bool INV>
struct Dft<3, INV> {
    static __device__ __forceinline__ void run(float2 *v) {
        const float s = 0.86602540378443864676f;
        float2 t = cadd(v[1], v[2]);
        float2 d = rot<INV>(csub(v[1], v[2]));
        float2 h = caxpy(-0.5f, t, v[0]);
        v[0] = cadd(v[0], t);
        v[1] = caxpy(s, d, h);
        v[2] = caxpy(-s, d, h);
    }
};

template <bool INV>
struct Dft<4, INV> {
    static __device__ __forceinline__ void run(float2 *v) {
        float2 t0 = cadd(v[0], v[2]), t1 = csub(v[0], v[2]);
        float2 t2 = cadd(v[1], v[3]), t3 = rot<INV>(csub(v[1], v[3]));
        v[0] = cadd(t0, t2);
        v[2] = csub(t0, t2);
        v[1] = cadd(t1, t3);
        v[3] = csub(t1, t3);
    }
};

template <bool INV>
struct Dft<5, INV> {
    static __device__ __forceinline__ void run(float2 *v) {
        const float c1 = 0.30901699437494742410f, c2 = -0.80901699437494742410f;
        const float s1 = 0.95105651629515357212f, s2 = 0.58778525229247312917f;
        float2 a1 = cadd(v[1], v[4]), a2 = cadd(v[2], v[3]);
        float2 b1 = csub(v[1], v[4]), b2 = csub(v[2], v[3]);
        float2 p1 = caxpy(c2, a2, caxpy(c1, a1, v[0]));
        float2 p2 = caxpy(c1, a2, caxpy(c2, a1, v[0]));
        float2 q1 = rot<INV>(caxpy(s2, b2, make_float2(s1 * b1.x, s1 * b1.y)));
        float2 q2 = rot<INV>(caxpy(-s1, b2, make_float2(s2 * b1.x, s2 * b1.y)));
        v[0] = cadd(v[0], cadd(a1, a2));
        v[1] = cadd(p1, q1);
        v[4] = csub(p1, q1);
        v[2] = cadd(p2, q2);
        v[3] = csub(p2, q2);
    }
};

// multiply by exp(-+ 2 pi i k / R) with compile-time (R, k) after unrolling
template <int R, bool INV>
__device__ __forceinline__ float2 mul_root(float2 z, int k) {
    k %= R;
    if (k == 0) return z;
    if (4 * k == R) return rot<INV>(z);
    if (2 * k == R) return make_float2(-z.x, -z.y);
    if (4 * k == 3 * R) return rot<!INV>(z);
    const float c = RootTab<R>::c(k);
    const float s = INV ? RootTab<R>::s(k) : -RootTab<R>::s(k);
    return make_float2(z.x * c - z.y * s, z.x * s + z.y * c);
}

// R = R1 * R2 in registers: R2 transforms of size R1 over the strided inputs, constant twiddles, R1 transforms of
// size R2; results returned in natural order.
template <int R1, int R2, bool INV>
struct DftComposite {
    static __device__ __forceinline__ void run(float2 *v) {
        constexpr int R = R1 * R2;
        float2 w[R];
#pragma unroll
        for (int n2 = 0; n2 < R2; ++n2) {
            float2 t[R1];
#pragma unroll
            for (int n1 = 0; n1 < R1; ++n1) t[n1] = v[n1 * R2 + n2];
            Dft<R1, INV>::run(t);
#pragma unroll
            for (int k1 = 0; k1 < R1; ++k1) w[k1 * R2 + n2] = mul_root<R, INV>(t[k1], k1 * n2);
        }
#pragma unroll
        for (int k1 = 0; k1 < R1; ++k1) {
            float2 t[R2];
#pragma unroll
            for (int n2 = 0; n2 < R2; ++n2) t[n2] = w[k1 * R2 + n2];
            Dft<R2, INV>::run(t);
#pragma unroll
            for (int k2 = 0; k2 < R2; ++k2) v[k1 + R1 * k2] = t[k2];
        }
    }
};
template <bool INV> struct Dft<6, INV> : DftComposite<2, 3, INV> {};
template <bool INV> struct Dft<8, INV> : DftComposite<2, 4, INV> {};
template <bool INV> struct Dft<9, INV> : DftComposite<3, 3, INV> {};
template <bool INV> struct Dft<10, INV> : DftComposite<2, 5, INV> {};
template <bool INV> struct Dft<12, INV> : DftComposite<3, 4, INV> {};
template <bool INV> struct Dft<15, INV> : DftComposite<3, 5, INV> {};
template <bool INV> struct Dft<16, INV> : DftComposite<4, 4, INV> {};

template <bool INV> struct Dft<20, INV> : DftComposite<4, 5, INV> {};
template <bool INV> struct Dft<32, INV> : DftComposite<4, 8, INV> {};
template <bool INV> struct Dft<36, INV> : DftComposite<4, 9, INV> {};
template <bool INV> struct Dft<40, INV> : DftComposite<8, 5, INV> {};

}  // namespace shtb200
