// Degree-wise channel mixing of spherical harmonic coefficients in the degree-slab layout, the middle step of a
// spectral convolution (SHT -> per-degree complex channel contraction -> inverse SHT).
//
// The analysis contraction leaves its result as slabs  S[(slab0[g] + r / 32) * ncols + 2 field + re/im][r % 32]
// (g = 2 m + parity, degree l = m + parity + 2 r) and the synthesis contraction reads exactly that layout, so a caller
// that mixes channels degree by degree can stay in it: the coefficient arrays (field, l, m) and the two transposes that
// produce / consume them never exist.  Mixing touches every (slab row, r) column independently:
//     out[b, o, l, m] = sum_i  W[g, i, o, l] * in[b, g, i, l, m]        (complex, weights shared by all orders m)
// Replaces torch_harmonics/spectral_convolution.py:236-239 (reshape + einsum "bgixy,giox->bgoxy" + reshape) together
// with the (field, l, m) tensors around it.

#include "common.cuh"

namespace shtb200 {

namespace {

constexpr int kMixCo = 4;        // output channels per thread
constexpr int kMixWarps = 8;     // warps per CTA: a CTA produces kMixWarps * kMixCo = 32 output channels of one slab
constexpr int kMixTile = kMixCo * kMixWarps;
constexpr int kMixCiChunk = 256; // input channels staged in shared memory at a time (64 KiB)

// W [G][Cig][Cog][L] complex -> Wp [2][G][Cig][Cog][Lh2]: entry h of parity par = W[.., 2 h + par] (0 beyond L).  All
// degrees of one slab have the same parity, so with this split the 32 lanes of a warp (32 consecutive r, degrees
// l0 + 2 r) read 32 consecutive weights.
__global__ void split_weights_kernel(const float2 *__restrict__ W, float2 *__restrict__ Wp, long long nrows, int L, int Lh2) {
    const long long total = 2 * nrows * Lh2;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
        const int h = (int)(i % Lh2);
        const long long row = (i / Lh2) % nrows;
        const int par = (int)(i / (Lh2 * nrows));
        const int l = 2 * h + par;
        Wp[i] = l < L ? W[row * L + l] : make_float2(0.f, 0.f);
    }
}

struct MixArgs {
    const float *Zin;
    float *Zout;
    const float2 *Wp;
    const long long *gb0;  // first slab of every group (ngroups + 1 entries)
    const int *grows;      // degrees in every group
    int ngroups, B, Cin, Cout, G, Lh2;
};

// grid: (slabs, B * output tiles); block: kMixWarps warps, lane = r
__global__ void __launch_bounds__(32 * kMixWarps) slab_mix_kernel(const MixArgs a) {
    extern __shared__ float tile[];  // [2 * channels of the chunk][32]
    __shared__ int s_group;
    const long long slab = blockIdx.x;
    if (threadIdx.x == 0) {  // the group this slab belongs to: last g with gb0[g] <= slab
        int lo = 0, hi = a.ngroups;
        while (hi - lo > 1) {
            const int mid = (lo + hi) >> 1;
            if (a.gb0[mid] <= slab) lo = mid;
            else hi = mid;
        }
        s_group = lo;
    }
    __syncthreads();
    const int g = s_group;
    const int m = g >> 1, p = g & 1;
    const int rb = (int)(slab - a.gb0[g]);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int r = rb * 32 + lane;
    const bool valid = r < a.grows[g];
    const int l = m + p + 2 * r;
    const int par = l & 1, h = l >> 1;

    const int Cig = a.Cin / a.G, Cog = a.Cout / a.G;
    const int tiles_per_group = (Cog + kMixTile - 1) / kMixTile;
    const int ntile = a.G * tiles_per_group;
    const int b = blockIdx.y / ntile, tl = blockIdx.y % ntile;
    const int cg = tl / tiles_per_group;                          // channel group
    const int co0 = (tl % tiles_per_group) * kMixTile + warp * kMixCo;  // first output channel (inside the group) of this thread
    const long long ncols_in = 2LL * a.B * a.Cin, ncols_out = 2LL * a.B * a.Cout;

    float2 acc[kMixCo];
#pragma unroll
    for (int j = 0; j < kMixCo; ++j) acc[j] = make_float2(0.f, 0.f);
    const float *zin = a.Zin + (slab * ncols_in + 2LL * ((long long)b * a.Cin + (long long)cg * Cig)) * kBK;
    for (int c0 = 0; c0 < Cig; c0 += kMixCiChunk) {
        const int nc = min(kMixCiChunk, Cig - c0);
        __syncthreads();
        for (int i = threadIdx.x; i < 2 * nc * (kBK / 4); i += blockDim.x)  // rows are 128 bytes: float4 copies
            reinterpret_cast<float4 *>(tile)[i] = __ldg(reinterpret_cast<const float4 *>(zin + (size_t)2 * c0 * kBK) + i);
        __syncthreads();
        if (valid) {
            const float2 *w = a.Wp + ((((long long)par * a.G + cg) * Cig + c0) * Cog + co0) * a.Lh2 + h;
            for (int ci = 0; ci < nc; ++ci) {
                const float ur = tile[(2 * ci) * kBK + lane], ui = tile[(2 * ci + 1) * kBK + lane];
#pragma unroll
                for (int j = 0; j < kMixCo; ++j) {
                    if (co0 + j < Cog) {
                        const float2 ww = __ldg(w + (long long)j * a.Lh2);
                        acc[j].x = fmaf(ww.x, ur, fmaf(-ww.y, ui, acc[j].x));
                        acc[j].y = fmaf(ww.x, ui, fmaf(ww.y, ur, acc[j].y));
                    }
                }
                w += (long long)Cog * a.Lh2;
            }
        }
    }
    // rows beyond the group's last degree pad the slab: the synthesis contraction reads them, they must be zeros
    float *zout = a.Zout + (slab * ncols_out + 2LL * ((long long)b * a.Cout + (long long)cg * Cog + co0)) * kBK + lane;
#pragma unroll
    for (int j = 0; j < kMixCo; ++j) {
        if (co0 + j < Cog) {
            zout[(2 * j) * kBK] = acc[j].x;      // (zeros when !valid)
            zout[(2 * j + 1) * kBK] = acc[j].y;
        }
    }
}

// The same mixing, register-tiled.  All slabs of one degree class (Plan::d_cls_off) carry the same 32 degrees in their 32
// lanes, so for a lane the class is ONE small complex matrix product  out[co][n] = sum_ci W[ci][co][l] in[ci][n]  over
// the columns n = (slab of the class, batch entry).  A thread (lane = degree) keeps a kTileCo x kTileN block of it in
// registers: every weight it loads serves kTileN columns, every coefficient kTileCo output channels (the kernel above
// reloads the weights for every slab).  Eight warps of a CTA: four along the output channels, two along the columns.
// (Eight output channels per thread were measured slower: 158 registers, one CTA per SM.)
constexpr int kTileCo = 4, kTileN = 4, kWarpsCo = 4, kWarpsN = 2;

struct TiledMixArgs {
    const float *Zin;
    float *Zout;
    const float2 *Wp;
    const int *cls_off, *cls_slab;
    int B, Cin, Cout, G, Lh2, lmax;
};

// grid: (degree classes l0, channel groups x tiles of 16 output channels); block: 8 warps
__global__ void __launch_bounds__(32 * kWarpsCo * kWarpsN) slab_mix_tiled_kernel(const TiledMixArgs a) {
    const int l0 = blockIdx.x;
    const int s_begin = a.cls_off[l0], nslab = a.cls_off[l0 + 1] - s_begin;
    const int ncol = nslab * a.B;
    if (ncol == 0) return;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int wc = warp % kWarpsCo, wn = warp / kWarpsCo;
    const int l = l0 + 2 * lane;
    const bool valid = l < a.lmax;  // lanes beyond the last degree pad the slab: zeros
    const int par = l0 & 1, h = (l0 >> 1) + lane;
    const int Cig = a.Cin / a.G, Cog = a.Cout / a.G;
    const int tiles = (Cog + kTileCo * kWarpsCo - 1) / (kTileCo * kWarpsCo);
    const int cg = blockIdx.y / tiles;
    const int co0 = (blockIdx.y % tiles) * (kTileCo * kWarpsCo) + wc * kTileCo;  // first output channel (inside the group) of this thread
    if (co0 >= Cog) return;
    const long long ncols_in = 2LL * a.B * a.Cin, ncols_out = 2LL * a.B * a.Cout;
    const float2 *wbase = a.Wp + (((long long)par * a.G + cg) * Cig * Cog + co0) * a.Lh2 + h;
    const long long wstep = (long long)Cog * a.Lh2;  // from one input channel to the next

    for (int n0 = wn * kTileN; n0 < ncol; n0 += kTileN * kWarpsN) {
        const float *in[kTileN];
        float *out[kTileN];
#pragma unroll
        for (int t = 0; t < kTileN; ++t) {
            const int n = min(n0 + t, ncol - 1);  // (columns beyond the class repeat the last one; they are not stored)
            const int slab = a.cls_slab[s_begin + n / a.B], b = n % a.B;
            in[t] = a.Zin + ((long long)slab * ncols_in + 2LL * ((long long)b * a.Cin + (long long)cg * Cig)) * kBK + lane;
            out[t] = a.Zout + ((long long)slab * ncols_out + 2LL * ((long long)b * a.Cout + (long long)cg * Cog + co0)) * kBK + lane;
        }
        float2 acc[kTileCo][kTileN];
#pragma unroll
        for (int j = 0; j < kTileCo; ++j)
#pragma unroll
            for (int t = 0; t < kTileN; ++t) acc[j][t] = make_float2(0.f, 0.f);
        if (valid) {
            const float2 *w = wbase;
#pragma unroll 2
            for (int ci = 0; ci < Cig; ++ci) {
                float2 ww[kTileCo], u[kTileN];
#pragma unroll
                for (int j = 0; j < kTileCo; ++j) ww[j] = (co0 + j < Cog) ? __ldg(w + (long long)j * a.Lh2) : make_float2(0.f, 0.f);
#pragma unroll
                for (int t = 0; t < kTileN; ++t) u[t] = make_float2(__ldg(in[t] + (2 * ci) * kBK), __ldg(in[t] + (2 * ci + 1) * kBK));
#pragma unroll
                for (int j = 0; j < kTileCo; ++j)
#pragma unroll
                    for (int t = 0; t < kTileN; ++t) {
                        acc[j][t].x = fmaf(ww[j].x, u[t].x, fmaf(-ww[j].y, u[t].y, acc[j][t].x));
                        acc[j][t].y = fmaf(ww[j].x, u[t].y, fmaf(ww[j].y, u[t].x, acc[j][t].y));
                    }
                w += wstep;
            }
        }
#pragma unroll
        for (int t = 0; t < kTileN; ++t) {
            if (n0 + t >= ncol) continue;
#pragma unroll
            for (int j = 0; j < kTileCo; ++j) {
                if (co0 + j < Cog) {
                    out[t][(2 * j) * kBK] = acc[j][t].x;      // (zeros when !valid)
                    out[t][(2 * j + 1) * kBK] = acc[j][t].y;
                }
            }
        }
    }
}

}  // namespace

size_t slab_mix_weight_bytes(int cin, int cout, int ngroups, int lmax) {
    return sizeof(float2) * 2 * (size_t)(cin / ngroups) * cout * ((lmax + 1) / 2);
}

// Zin: slabs of batch * cin fields; Zout: slabs of batch * cout fields; weight: complex64 [ngroups][cin / ngroups][cout / ngroups][lmax];
// wsplit: scratch of slab_mix_weight_bytes(..) bytes
int launch_slab_mix(const Plan &pl, const float *Zin, float *Zout, const float2 *weight, float2 *wsplit, int batch, int cin, int cout, int ngroups, cudaStream_t st) {
    const int Lh2 = (pl.lmax + 1) / 2;
    const long long nrows = (long long)(cin / ngroups) * cout;  // G * Cig * Cog
    const long long total = 2 * nrows * Lh2;
    split_weights_kernel<<<(unsigned)std::min<long long>((total + 255) / 256, 8192), 256, 0, st>>>(weight, wsplit, nrows, pl.lmax, Lh2);
    SHT_CUDA_CHECK(cudaGetLastError());
#ifndef SHTB200_MIX_UNTILED  // build-time switch for A/B measurements against the slab-by-slab kernel below
    if (pl.d_cls_off) {
        TiledMixArgs t{};
        t.Zin = Zin;
        t.Zout = Zout;
        t.Wp = wsplit;
        t.cls_off = pl.d_cls_off;
        t.cls_slab = pl.d_cls_slab;
        t.B = batch;
        t.Cin = cin;
        t.Cout = cout;
        t.G = ngroups;
        t.Lh2 = Lh2;
        t.lmax = pl.lmax;
        const int tiles = ngroups * ceil_div(cout / ngroups, kTileCo * kWarpsCo);
        if (tiles > 65535) return fail(SHTB200_EINVAL, "too many output channels for one spectral-convolution call");
        dim3 grid((unsigned)pl.lmax, (unsigned)tiles);
        slab_mix_tiled_kernel<<<grid, 32 * kWarpsCo * kWarpsN, 0, st>>>(t);
        SHT_CUDA_CHECK(cudaGetLastError());
        return SHTB200_OK;
    }
#endif
    MixArgs a{};
    a.Zin = Zin;
    a.Zout = Zout;
    a.Wp = wsplit;
    a.gb0 = pl.d_gb0;
    a.grows = pl.d_grows;
    a.ngroups = 2 * pl.mmax;
    a.B = batch;
    a.Cin = cin;
    a.Cout = cout;
    a.G = ngroups;
    a.Lh2 = Lh2;
    const int cog = cout / ngroups, cig = cin / ngroups;
    const int tiles = ngroups * ceil_div(cog, kMixTile);
    if ((long long)batch * tiles > 65535) return fail(SHTB200_EINVAL, "batch x output channels too large for one spectral-convolution call");
    dim3 grid((unsigned)pl.total_b_slabs, (unsigned)(batch * tiles));
    const size_t smem = sizeof(float) * 2 * std::min(cig, kMixCiChunk) * kBK;
    SHT_CUDA_CHECK(cudaFuncSetAttribute(slab_mix_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    slab_mix_kernel<<<grid, 32 * kMixWarps, smem, st>>>(a);
    SHT_CUDA_CHECK(cudaGetLastError());
    return SHTB200_OK;
}

// Integral over the sphere of every field: out[f] = sum_k w[k] * sum_j x[f, k, j]  (w = latitude quadrature weights
// times 2 pi / nlon).  One warp per (field, latitude chunk); replaces torch_harmonics/quadrature.py:447-463.
__global__ void quadrature_kernel(const float *__restrict__ x, const float *__restrict__ w, float *__restrict__ out, long long nfields, int nlat, int nlon) {
    const long long f = blockIdx.x;
    float acc = 0.f;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
    for (int k = warp; k < nlat; k += nw) {
        const float *row = x + ((size_t)f * nlat + k) * nlon;
        float s = 0.f;
        for (int j = lane; j < nlon; j += 32) s += __ldg(row + j);
        acc = fmaf(w[k], s, acc);
    }
    for (int o = 16; o; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
    __shared__ float part[32];
    if (lane == 0) part[warp] = acc;
    __syncthreads();
    if (threadIdx.x == 0) {
        float t = 0.f;
        for (int i = 0; i < nw; ++i) t += part[i];
        out[f] = t;
    }
}

int launch_quadrature(const float *x, const float *w, float *out, long long nfields, int nlat, int nlon, cudaStream_t st) {
    if (nfields == 0) return SHTB200_OK;
    if (nfields > 0x7fffffffLL) return fail(SHTB200_EINVAL, "too many fields");
    quadrature_kernel<<<(unsigned)nfields, 256, 0, st>>>(x, w, out, nfields, nlat, nlon);
    SHT_CUDA_CHECK(cudaGetLastError());
    return SHTB200_OK;
}

}  // namespace shtb200
