// Legendre contraction on the fp32 CUDA cores.
//
// Same work-item list, operand packings and epilogues as the tensor-core kernel; used for shapes
// the tcgen05 path does not take and as an independent on-device cross-check of it.
// Replaces the two torch.einsum calls per direction, torch_harmonics/sht.py:180-181 and :333-334
// (vector: :488-493, :638-643), restricted to the l >= m band and folded about the equator.

#include "common.cuh"

namespace shtb200 {

namespace {

constexpr int TM = 64, TN = 64, TK = 16;

__device__ __forceinline__ float load_operand(const float *base, long long pitch, long long y0, int dy, int dx, int kext, int r, int k) {
    const int kb = k / kBK, kk = k - kb * kBK;
    const int col = kb * dx + kk;
    if (col >= kext) return 0.f;
    return base[(y0 + (long long)kb * dy + r) * pitch + col];
}

__global__ void __launch_bounds__(256) legendre_simt_kernel(GemmParams gp) {
    const GemmItem it = gp.items[blockIdx.x];
    if (it.m < gp.m0 || it.m >= gp.m0 + gp.mmax_out) return;
    const int row0 = blockIdx.z * TM;
    if (row0 >= it.rows) return;
    const int col0 = blockIdx.y * TN;

    __shared__ float As[TK][TM + 4];
    __shared__ float Bs[TK][TN + 4];

    const int tx = threadIdx.x % 16, ty = threadIdx.x / 16;
    float acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;

    const int K = it.kblocks * kBK;
    const long long b_y0 = ((long long)it.b_y0 - gp.b_unit0) * gp.ncols;
    const int b_dy = it.b_dy * gp.ncols;
    const int kbase = it.kfirst * kBK;  // slices skipped at the front of the group
    for (int k0 = kbase; k0 < kbase + K; k0 += TK) {
        // 64 x 16 elements per operand, 256 threads: 4 each; consecutive threads walk k (contiguous in memory)
        for (int e = threadIdx.x; e < TM * TK; e += 256) {
            const int kk = e % TK, r = e / TK;
            const int ra = row0 + r;
            As[kk][r] = (ra < it.rows) ? load_operand(gp.A, gp.a_pitch, it.a_y0, it.a_dy, gp.a_dx, gp.a_kext, ra, k0 + kk) : 0.f;
            const int cb = col0 + r;
            float bv = 0.f;
            if (cb < gp.ncols) {
                if (gp.b_mn) {
                    const int k = k0 + kk;
                    if (k < gp.b_krows) bv = gp.B[blocked_row((long long)it.b_y0 - gp.b_unit0, k, gp.b_groups) * gp.b_pitch + cb];
                } else {
                    bv = load_operand(gp.B, gp.b_pitch, b_y0, b_dy, gp.b_dx, gp.b_kext, cb, k0 + kk);
                }
            }
            Bs[kk][r] = bv;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < TK; ++kk) {
            float a[4], b[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) a[i] = As[kk][ty * 4 + i];
#pragma unroll
            for (int j = 0; j < 4; ++j) b[j] = Bs[kk][tx * 4 + j];
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
        }
        __syncthreads();
    }

#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int r = row0 + ty * 4 + i;
        if (r >= it.rows) continue;
        const int rg = it.r0 + r;  // row index inside the group
        if (gp.mode == EPI_SLABS) {
            const long long slab = gp.slab0[2 * (it.m - gp.m_base) + it.p] - gp.slab_unit0 + (rg >> 5);
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const int c = col0 + tx * 4 + j;
                if (c >= gp.ncols) continue;
                gp.out[((size_t)slab * gp.ncols + c) * kBK + (rg & 31)] = acc[i][j];
            }
        } else {
            const int g = 2 * (it.m - gp.m0) + it.p;
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const int c = col0 + tx * 4 + j;
                if (c >= gp.ncols) continue;
                gp.out[y_off(g, rg, c, gp.out_groups, gp.out_ld)] = acc[i][j];
            }
        }
    }
}

}  // namespace

int launch_gemm_simt(const GemmParams &gp, cudaStream_t st) {
    if (gp.nitems == 0 || gp.ncols == 0) return SHTB200_OK;
    dim3 grid(gp.nitems, ceil_div(gp.ncols, TN), kItemRowsMax / TM);
    legendre_simt_kernel<<<grid, 256, 0, st>>>(gp);
    SHT_CUDA_CHECK(cudaGetLastError());
    return SHTB200_OK;
}

}  // namespace shtb200
