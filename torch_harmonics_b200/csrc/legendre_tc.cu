// Legendre contraction on the 5th-generation tensor cores (tcgen05) with split-TF32 arithmetic.
//
// Per (order m, parity) group the contraction is a real GEMM  D[rows x cols] = A[rows x K] * B[cols x K]^T
// with A the packed Legendre table (rows = degrees for analysis, folded latitudes for synthesis) and B the
// operand produced by the FFT kernel / coefficient packing (cols = 2 x fields).  One persistent CTA per SM
// walks a longest-first list of work units (item, column tile):
//
//   warp 0      TMA producer: cp.async.bulk.tensor loads of up to three 128-row A tiles and one B tile per 16-wide
//               k-step into a 4-deep ring of 64-byte-swizzled shared-memory stages (full/empty mbarriers).
//   warps 2-5   splitter: for each landed stage compute lo = x - tf32_trunc(x) for A and B into one of two "lo"
//               slots (same swizzled layout, so the pass is a straight elementwise sweep).
//   warp 1      MMA issuer: per k-step and A tile three tcgen05.mma chains (A B, A_lo B, A B_lo; the tensor core
//               reads fp32 words as TF32 by dropping the low mantissa bits), fp32 accumulation in TMEM
//               (3 accumulators x up to 160 columns); tcgen05.commit releases stages / lo slots / accumulators.
//   warps 6-9   epilogue: tcgen05.ld of the accumulators, direct stores to the coefficient array (analysis) or the
//               latitude-row operand of the synthesis FFT.
//
// Every mbarrier wait is bounded: when one runs out the CTA raises a device error word and unwinds.
// Replaces torch.einsum -> aten::bmm at torch_harmonics/sht.py:180-181, :333-334 (vector :488-493, :638-643).

#include <cuda.h>
#include <stdlib.h>

#include <algorithm>
#include <mutex>

#include "common.cuh"
#include "tc_ptx.cuh"

namespace shtb200 {

namespace {

constexpr int TK = 16;                 // floats per k-step (one 64-byte swizzle row)
constexpr int TILE_M = 128;
constexpr int MT_MAX = kItemRowsMax / TILE_M;  // 3
constexpr int BN_MAX = 160;
constexpr int NSTAGE = 4;
constexpr int NLO = 2;
constexpr int A_TILE_BYTES = TILE_M * TK * 4;                          // 8 KiB
constexpr int STAGE_BYTES = MT_MAX * A_TILE_BYTES + BN_MAX * TK * 4;   // 34 KiB
constexpr int B_OFF = MT_MAX * A_TILE_BYTES;
constexpr int TMEM_COLS = 512;
constexpr int NTHREADS = 320;
constexpr long long WAIT_LIMIT = 4000000000LL;  // ~2 s of SM clock

constexpr int SMEM_BYTES = (NSTAGE + NLO) * STAGE_BYTES + 1024 /* alignment slack */ + 256 /* barriers */;

struct TcParams {
    GemmParams gp;
    int bn;          // columns per tile (multiple of 16, <= BN_MAX)
    int ntiles;      // column tiles
    int nunits;      // nitems * ntiles
    int ksteps_cap;  // row-packed operands: k-steps that cover the valid extent
    int write_hi;    // also store the TF32-truncated value back (only needed if the tensor core rounded instead of truncating)
    int *err;        // device error word
};

__device__ __forceinline__ float tf32_hi(float x) { return __uint_as_float(__float_as_uint(x) & 0xFFFFE000u); }
__device__ __forceinline__ float tf32_lo(float x) { return x - tf32_hi(x); }

__global__ void __launch_bounds__(NTHREADS, 1)
legendre_tc_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, const TcParams P) {
    extern __shared__ uint8_t smem_raw[];
    const uint32_t base = (ptx::smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t *base_ptr = smem_raw + (base - ptx::smem_u32(smem_raw));
    const uint32_t stage0 = base;
    const uint32_t lo0 = base + NSTAGE * STAGE_BYTES;
    const uint32_t bar0 = base + (NSTAGE + NLO) * STAGE_BYTES;
    // barrier slots (8 bytes each)
    auto bar_full = [&](int s) { return bar0 + 8u * s; };
    auto bar_empty = [&](int s) { return bar0 + 8u * (NSTAGE + s); };
    auto bar_lofull = [&](int c) { return bar0 + 8u * (2 * NSTAGE + c); };
    auto bar_loempty = [&](int c) { return bar0 + 8u * (2 * NSTAGE + NLO + c); };
    const uint32_t bar_accfull = bar0 + 8u * (2 * NSTAGE + 2 * NLO);
    const uint32_t bar_accempty = bar_accfull + 8u;
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(base_ptr + (NSTAGE + NLO) * STAGE_BYTES + 8 * (2 * NSTAGE + 2 * NLO + 2));
    volatile int *abort_flag = reinterpret_cast<volatile int *>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const GemmParams &gp = P.gp;

    if (threadIdx.x == 0) {
        for (int s = 0; s < NSTAGE; ++s) { ptx::mbar_init(bar_full(s), 1); ptx::mbar_init(bar_empty(s), 1); }
        for (int c = 0; c < NLO; ++c) { ptx::mbar_init(bar_lofull(c), 128); ptx::mbar_init(bar_loempty(c), 1); }
        ptx::mbar_init(bar_accfull, 1);
        ptx::mbar_init(bar_accempty, 128);
        *abort_flag = 0;
        ptx::fence_barrier_init();
        ptx::prefetch_tensormap(&tmA);
        ptx::prefetch_tensormap(&tmB);
    }
    if (warp == 1) {
        ptx::tmem_alloc(ptx::smem_u32(tmem_slot), TMEM_COLS);
        ptx::tmem_relinquish();
    }
    ptx::tc_fence_before();
    __syncthreads();
    ptx::tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    const bool row_packed_a = gp.a_dx != 0, row_packed_b = gp.b_dx != 0;

    // ---- decode of work unit u (identical in every role) ----
    struct Unit { GemmItem it; int ntile; int mt; int ksteps; bool skip; };
    auto get_unit = [&](int u) {
        Unit w;
        w.it = gp.items[u / P.ntiles];
        w.ntile = u % P.ntiles;
        w.mt = (w.it.rows + TILE_M - 1) / TILE_M;
        w.ksteps = w.it.kblocks * (kBK / TK);
        if (row_packed_a && w.ksteps > P.ksteps_cap) w.ksteps = P.ksteps_cap;
        w.skip = (w.it.m < gp.m0) || (w.it.m >= gp.m0 + gp.mmax_out);
        return w;
    };

    if (warp == 0) {
        // =========================== TMA producer ===========================
        if (lane == 0) {
            int s = 0;
            uint32_t ph = 0;
            bool ok = true;
            for (int u = blockIdx.x; u < P.nunits && ok; u += gridDim.x) {
                const Unit w = get_unit(u);
                if (w.skip) continue;
                const uint32_t bytes = (uint32_t)(w.mt * A_TILE_BYTES + P.bn * TK * 4);
                const long long by0 = ((long long)w.it.b_y0 - gp.b_unit0) * gp.ncols + (long long)w.ntile * P.bn;
                for (int ks = 0; ks < w.ksteps; ++ks) {
                    if (!(ok = ptx::mbar_wait_bounded(bar_empty(s), ph ^ 1u, abort_flag, WAIT_LIMIT))) break;
                    ptx::mbar_arrive_expect_tx(bar_full(s), bytes);
                    const int kb = (ks * TK) / kBK, kin = (ks * TK) % kBK;
                    const int ax = row_packed_a ? ks * TK : kin;
                    const int ay = w.it.a_y0 + (row_packed_a ? 0 : kb * w.it.a_dy);
                    const uint32_t dst = stage0 + s * STAGE_BYTES;
                    for (int t = 0; t < w.mt; ++t) ptx::tma_load_2d(dst + t * A_TILE_BYTES, &tmA, ax, ay + t * TILE_M, bar_full(s));
                    const int bx = row_packed_b ? ks * TK : kin;
                    const long long by = by0 + (row_packed_b ? 0 : (long long)kb * w.it.b_dy * gp.ncols);
                    ptx::tma_load_2d(dst + B_OFF, &tmB, bx, (int)by, bar_full(s));
                    if (++s == NSTAGE) { s = 0; ph ^= 1u; }
                }
            }
        }
    } else if (warp == 1) {
        // =========================== MMA issuer ===========================
        if (lane == 0) {
            int s = 0, c = 0;
            uint32_t ph = 0, phc = 0, phacc = 0;
            bool ok = true;
            const uint32_t idesc = ptx::idesc_tf32_m128((uint32_t)P.bn);
            for (int u = blockIdx.x; u < P.nunits && ok; u += gridDim.x) {
                const Unit w = get_unit(u);
                if (w.skip) continue;
                // accumulators must have been drained by the epilogue of the previous unit
                if (!(ok = ptx::mbar_wait_bounded(bar_accempty, phacc ^ 1u, abort_flag, WAIT_LIMIT))) break;
                ptx::tc_fence_after();
                for (int ks = 0; ks < w.ksteps; ++ks) {
                    if (!(ok = ptx::mbar_wait_bounded(bar_full(s), ph, abort_flag, WAIT_LIMIT))) break;
                    if (!(ok = ptx::mbar_wait_bounded(bar_lofull(c), phc, abort_flag, WAIT_LIMIT))) break;
                    ptx::tc_fence_after();
                    const uint32_t hi = stage0 + s * STAGE_BYTES, lo = lo0 + c * STAGE_BYTES;
                    const uint64_t bh = ptx::smem_desc_sw64(hi + B_OFF), bl = ptx::smem_desc_sw64(lo + B_OFF);
                    for (int t = 0; t < w.mt; ++t) {
                        const uint64_t ah = ptx::smem_desc_sw64(hi + t * A_TILE_BYTES), al = ptx::smem_desc_sw64(lo + t * A_TILE_BYTES);
                        const uint32_t d = tmem_base + (uint32_t)(t * P.bn);
#pragma unroll
                        for (int k8 = 0; k8 < TK / 8; ++k8) {
                            const uint64_t koff = (uint64_t)((k8 * 32) >> 4);  // 8 TF32 = 32 bytes along the swizzled row
                            ptx::mma_tf32(d, al + koff, bh + koff, idesc, (ks | k8) ? 1u : 0u);  // small terms first
                            ptx::mma_tf32(d, ah + koff, bl + koff, idesc, 1u);
                            ptx::mma_tf32(d, ah + koff, bh + koff, idesc, 1u);
                        }
                    }
                    ptx::tc_commit(bar_empty(s));
                    ptx::tc_commit(bar_loempty(c));
                    if (++s == NSTAGE) { s = 0; ph ^= 1u; }
                    if (++c == NLO) { c = 0; phc ^= 1u; }
                }
                if (!ok) break;
                ptx::tc_commit(bar_accfull);
                phacc ^= 1u;
            }
        }
    } else if (warp < 6) {
        // =========================== splitter (128 threads) ===========================
        const int tid = threadIdx.x - 64;
        int s = 0, c = 0;
        uint32_t ph = 0, phc = 0;
        bool ok = true;
        for (int u = blockIdx.x; u < P.nunits && ok; u += gridDim.x) {
            const Unit w = get_unit(u);
            if (w.skip) continue;
            const int na4 = w.mt * (A_TILE_BYTES / 16), nb4 = P.bn * TK * 4 / 16;
            for (int ks = 0; ks < w.ksteps; ++ks) {
                if (!(ok = ptx::mbar_wait_bounded(bar_full(s), ph, abort_flag, WAIT_LIMIT))) break;
                if (!(ok = ptx::mbar_wait_bounded(bar_loempty(c), phc ^ 1u, abort_flag, WAIT_LIMIT))) break;
                float4 *src = reinterpret_cast<float4 *>(base_ptr + s * STAGE_BYTES);
                float4 *dst = reinterpret_cast<float4 *>(base_ptr + (NSTAGE + c) * STAGE_BYTES);
                for (int i = tid; i < na4; i += 128) {
                    float4 v = src[i];
                    dst[i] = make_float4(tf32_lo(v.x), tf32_lo(v.y), tf32_lo(v.z), tf32_lo(v.w));
                    if (P.write_hi) src[i] = make_float4(tf32_hi(v.x), tf32_hi(v.y), tf32_hi(v.z), tf32_hi(v.w));
                }
                float4 *srcb = src + B_OFF / 16;
                float4 *dstb = dst + B_OFF / 16;
                for (int i = tid; i < nb4; i += 128) {
                    float4 v = srcb[i];
                    dstb[i] = make_float4(tf32_lo(v.x), tf32_lo(v.y), tf32_lo(v.z), tf32_lo(v.w));
                    if (P.write_hi) srcb[i] = make_float4(tf32_hi(v.x), tf32_hi(v.y), tf32_hi(v.z), tf32_hi(v.w));
                }
                ptx::fence_proxy_async_smem();
                ptx::mbar_arrive(bar_lofull(c));
                if (++s == NSTAGE) { s = 0; ph ^= 1u; }
                if (++c == NLO) { c = 0; phc ^= 1u; }
            }
        }
    } else {
        // =========================== epilogue (128 threads) ===========================
        const int q = warp & 3;            // TMEM lane quarter this warp may read
        const int row_in_tile = q * 32 + lane;
        uint32_t phacc = 0;
        bool ok = true;
        for (int u = blockIdx.x; u < P.nunits && ok; u += gridDim.x) {
            const Unit w = get_unit(u);
            if (w.skip) continue;
            if (!(ok = ptx::mbar_wait_bounded(bar_accfull, phacc, abort_flag, WAIT_LIMIT))) break;
            phacc ^= 1u;
            ptx::tc_fence_after();
            const int col0 = w.ntile * P.bn;
            for (int t = 0; t < w.mt; ++t) {
                const int r = t * TILE_M + row_in_tile;     // row inside the item
                const bool rvalid = r < w.it.rows;
                const int rg = w.it.r0 + r;                  // row inside the group
                for (int cc = 0; cc < P.bn; cc += 16) {
                    if (col0 + cc >= gp.ncols) break;        // warp-uniform
                    float v[16];
                    ptx::tmem_ld16(tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(t * P.bn + cc), v);
                    if (!rvalid) continue;
                    if (gp.mode == EPI_COEFFS) {
                        const int l = w.it.m + w.it.p + 2 * rg;
                        float2 *o = reinterpret_cast<float2 *>(gp.out) + (size_t)l * gp.mmax_out + (w.it.m - gp.m0);
                        const size_t fstride = (size_t)gp.lmax * gp.mmax_out;
#pragma unroll
                        for (int j = 0; j < 16; j += 2) {
                            const int col = col0 + cc + j;
                            if (col < gp.ncols) o[(size_t)(col >> 1) * fstride] = make_float2(v[j], v[j + 1]);
                        }
                    } else {
                        const int g = 2 * (w.it.m - gp.m0) + w.it.p;
                        float *o = gp.out + ((size_t)g * gp.ngroups_cols) * gp.out_ld + rg;
#pragma unroll
                        for (int j = 0; j < 16; ++j) {
                            const int col = col0 + cc + j;
                            if (col < gp.ncols) o[(size_t)col * gp.out_ld] = v[j];
                        }
                    }
                }
            }
            ptx::tc_fence_before();
            ptx::mbar_arrive(bar_accempty);
        }
    }

    // ---- teardown ----
    __syncwarp();
    if (*abort_flag) {
        if (threadIdx.x == 0) atomicExch(P.err, 1);
        // leave time for copies and MMAs still in flight before shared / tensor memory are released
        const long long t0 = clock64();
        while (clock64() - t0 < 2000000LL) __nanosleep(1000);
    }
    ptx::tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        ptx::tc_fence_after();
        ptx::tmem_dealloc(tmem_base, TMEM_COLS);
    }
}

// ------------------------------------------------------------------------------------------------
// host side
// ------------------------------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *, const cuuint64_t *, const cuuint32_t *,
                                  const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
    static EncodeTiledFn fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void *p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess && q == cudaDriverEntryPointSuccess) fn = (EncodeTiledFn)p;
    });
    return fn;
}

int make_map(CUtensorMap *tm, const float *base, long long inner, long long rows, long long pitch_floats, int box_rows) {
    EncodeTiledFn fn = encode_fn();
    if (!fn) return fail(SHTB200_ECUDA, "cuTensorMapEncodeTiled not available from the driver");
    cuuint64_t dims[2] = {(cuuint64_t)inner, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)pitch_floats * 4};
    cuuint32_t box[2] = {(cuuint32_t)TK, (cuuint32_t)box_rows};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = fn(tm, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, (void *)base, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_64B,
                    CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail(SHTB200_ECUDA, "cuTensorMapEncodeTiled failed with code " + std::to_string((int)r));
    return SHTB200_OK;
}

}  // namespace

bool gemm_tc_supported(const Plan &pl, const GemmParams &gp) {
    (void)pl;
    if (gp.nitems == 0 || gp.ncols == 0) return false;
    if (((uintptr_t)gp.A & 15) || ((uintptr_t)gp.B & 15)) return false;
    if ((gp.a_pitch % 4) || (gp.b_pitch % 4)) return false;
    return encode_fn() != nullptr;
}

int launch_gemm_tc(const Plan &pl, const GemmParams &gp, cudaStream_t st) {
    static int sm_count = 0;
    if (!sm_count) {
        int dev = 0;
        SHT_CUDA_CHECK(cudaGetDevice(&dev));
        SHT_CUDA_CHECK(cudaDeviceGetAttribute(&sm_count, cudaDevAttrMultiProcessorCount, dev));
        SHT_CUDA_CHECK(cudaFuncSetAttribute(legendre_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES));
    }
    TcParams P{};
    P.gp = gp;
    P.bn = std::min<int>(BN_MAX, (int)round_up(gp.ncols, 16));
    P.ntiles = ceil_div(gp.ncols, P.bn);
    P.nunits = gp.nitems * P.ntiles;
    P.ksteps_cap = ceil_div(gp.a_kext, TK);
    P.err = pl.d_err;
    {
        const char *e = getenv("SHTB200_TC_WRITE_HI");
        P.write_hi = (e && e[0] == '1') ? 1 : 0;
    }

    // extents of the two operands as 2-D row-major tensors
    const bool analysis = gp.mode == EPI_COEFFS;
    long long a_rows, a_inner, b_rows, b_inner;
    if (analysis) {
        a_inner = gp.a_kext;
        a_rows = pl.group_a0.back() + kItemRowsMax;
        b_inner = gp.b_kext;
        b_rows = (long long)2 * gp.mmax_out * gp.ncols;
    } else {
        a_inner = kBK;
        a_rows = pl.group_a0.back() + kItemRowsMax;
        b_inner = kBK;
        b_rows = (pl.group_b0[2 * (gp.m0 + gp.mmax_out)] - pl.group_b0[2 * gp.m0]) * (long long)gp.ncols;
    }
    CUtensorMap tmA, tmB;
    int rc;
    if ((rc = make_map(&tmA, gp.A, a_inner, a_rows, gp.a_pitch, TILE_M))) return rc;
    if ((rc = make_map(&tmB, gp.B, b_inner, b_rows, gp.b_pitch, P.bn))) return rc;

    const int grid = std::min(sm_count, P.nunits);
    legendre_tc_kernel<<<grid, NTHREADS, SMEM_BYTES, st>>>(tmA, tmB, P);
    SHT_CUDA_CHECK(cudaGetLastError());
    return SHTB200_OK;
}

}  // namespace shtb200
