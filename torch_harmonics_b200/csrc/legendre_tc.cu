// Legendre contraction on the 5th-generation tensor cores (tcgen05) with split-TF32 arithmetic.
//
// Per (order m, parity) group the contraction is a real GEMM  D[rows x cols] = A[rows x K] * B[cols x K]^T
// with A the packed Legendre table (rows = degrees for analysis, folded latitudes for synthesis) and B the
// operand produced by the FFT kernel / coefficient packing (cols = 2 x fields).  One persistent CTA per SM
// walks a longest-first list of work units (128-row item, column tile):
//
//   warp 0      TMA producer: cp.async.bulk.tensor loads of one 128 x 32 A tile and one B tile per k-step into a
//               5-deep ring of 128-byte-swizzled shared-memory stages.
//   warps 2-5   A splitter, one warp per tensor-memory lane quarter: a thread reads its row of the landed A tile and
//               stores it twice into a 3-deep ring in TENSOR MEMORY, as it is and as lo = x - tf32_trunc(x)
//               (tcgen05.st), so the table never occupies shared-memory bandwidth again: the MMAs take A from there.
//   warps 6-9   B splitter: lo = x - tf32_trunc(x) of the B tile, written over the region of the stage the A tile came in
//               (same swizzled layout as the B tile, so the pass is a straight elementwise sweep).
//   warp 1      MMA issuer: per k-step three tcgen05.mma chains (A_lo B, A B_lo, A B; the tensor core reads
//               fp32 words as TF32 by dropping the low mantissa bits), fp32 accumulation in one of two
//               tensor-memory accumulators.  It waits on ONE barrier per k-step (both splitters done) and commits to
//               ONE barrier per k-step (MMAs done), which everybody who recycles a stage or an A slot watches.
//   warps 10-17 epilogue: tcgen05.ld of a finished accumulator while the next units are being multiplied,
//               stores to the degree-slab array (analysis) or the latitude-row operand of the synthesis FFT.
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

constexpr int TK = kBK;                // floats per k-step: one 128-byte swizzle row
constexpr int TILE_M = 128;
constexpr int BN_MAX = 160;
constexpr int NSTAGE = 5;              // TMA ring
constexpr int NACC = 2;                // accumulator buffers in tensor memory
constexpr int NATM = 3;                // A slots in tensor memory (raw + lo: 2 x 32 columns each)
constexpr int A_TILE_BYTES = TILE_M * TK * 4;                // 16 KiB
constexpr int B_TILE_BYTES = BN_MAX * TK * 4;                // 20 KiB
// A stage is two 20 KiB regions.  The first receives the A tile (16 KiB); once the A splitter has moved it to tensor
// memory the B splitter overwrites the region with the low-order part of B.  The second holds the B tile as loaded.
// Sharing the region is what buys the fifth stage: the ring's depth times the bytes of a stage has to cover the
// latency from "MMAs done" through the refill (HBM / L2) and both splitters back to "ready".
constexpr int STAGE_BYTES = 2 * B_TILE_BYTES;                // 40 KiB
constexpr int B_OFF = B_TILE_BYTES;
static_assert(A_TILE_BYTES <= B_TILE_BYTES, "the A tile shares the region of B's low-order part");
constexpr int B_BLK_BYTES = 32 * TK * 4;  // column-contiguous B: one 32 (k) x 32 (columns) block, 4 KiB
constexpr int TMEM_COLS = 512;
constexpr int A_TM_COL0 = NACC * BN_MAX;  // first tensor-memory column of the A ring
constexpr int NSPLIT_A = 4, NSPLIT_B = 4, NSPLIT_WARPS = NSPLIT_A + NSPLIT_B, NEPI_WARPS = 8;
constexpr int NTHREADS = 32 * (2 + NSPLIT_WARPS + NEPI_WARPS);  // 576
constexpr long long WAIT_LIMIT = 4000000000LL;                  // ~2 s of SM clock

constexpr int NRING = 15;               // k-steps that own a (ready, done) barrier pair before it is reused: a multiple of NSTAGE and NATM
constexpr int NBARS = 2 * NSTAGE + 2 * NRING + 2 * NACC;
static_assert(NRING % NSTAGE == 0 && NRING % NATM == 0 && NRING >= 2 * NSTAGE, "ring sizes");
constexpr int SMEM_BYTES = NSTAGE * STAGE_BYTES + 1024 /* alignment slack */ + 512 /* barriers */;
static_assert(NACC * BN_MAX + NATM * 2 * TK <= TMEM_COLS, "accumulators and the A ring must fit tensor memory");
static_assert(kItemRowsMax == TILE_M, "one work item = one 128-row tensor-core tile");

struct TcParams {
    GemmParams gp;
    int bn;          // columns per tile (multiple of 16, <= BN_MAX)
    int ntiles;      // column tiles
    int nunits;      // nitems * ntiles
    int ksteps_cap;  // row-packed operands: k-steps that cover the valid extent
    int bblk;        // column-contiguous B: 32-column blocks per tile
    int *err;        // device error word
};

__device__ __forceinline__ float tf32_hi(float x) { return __uint_as_float(__float_as_uint(x) & 0xFFFFE000u); }
__device__ __forceinline__ float tf32_lo(float x) { return x - tf32_hi(x); }

__global__ void __launch_bounds__(NTHREADS, 1)
legendre_tc_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, const __grid_constant__ TcParams P) {
    extern __shared__ uint8_t smem_raw[];
    const uint32_t base = (ptx::smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t *base_ptr = smem_raw + (base - ptx::smem_u32(smem_raw));
    const uint32_t stage0 = base;
    const uint32_t bar0 = base + NSTAGE * STAGE_BYTES;
    // barrier slots (8 bytes each)
    // full[s]: the TMA boxes of ring stage s have landed.  ready[k % NRING]: both splitters are done with k-step k (it
    // implies full).  done[k % NRING]: the MMAs of k-step k have completed; whoever wants to overwrite something k-step
    // k read (stage: k + NSTAGE, tensor-memory A slot: k + NATM) waits for it.  aread[s]: the A splitter has read the A tile of
    // stage s out of shared memory (the B splitter may now overwrite that region).  The MMA thread, which
    // must never leave the tensor pipe idle, thus waits on one barrier and commits to one barrier per k-step.
    auto bar_full = [&](int s) { return bar0 + 8u * s; };
    auto bar_aread = [&](int s) { return bar0 + 8u * (NSTAGE + s); };
    auto bar_ready = [&](int i) { return bar0 + 8u * (2 * NSTAGE + i); };
    auto bar_done = [&](int i) { return bar0 + 8u * (2 * NSTAGE + NRING + i); };
    auto bar_accfull = [&](int a) { return bar0 + 8u * (2 * NSTAGE + 2 * NRING + a); };
    auto bar_accempty = [&](int a) { return bar0 + 8u * (2 * NSTAGE + 2 * NRING + NACC + a); };
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(base_ptr + NSTAGE * STAGE_BYTES + 8 * NBARS);
    volatile int *abort_flag = reinterpret_cast<volatile int *>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const GemmParams &gp = P.gp;

    if (threadIdx.x == 0) {
        for (int s = 0; s < NSTAGE; ++s) { ptx::mbar_init(bar_full(s), 1); ptx::mbar_init(bar_aread(s), NSPLIT_A); }
        for (int i = 0; i < NRING; ++i) { ptx::mbar_init(bar_ready(i), NSPLIT_WARPS); ptx::mbar_init(bar_done(i), 1); }
        for (int a = 0; a < NACC; ++a) { ptx::mbar_init(bar_accfull(a), 1); ptx::mbar_init(bar_accempty(a), NEPI_WARPS); }
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
    struct Unit { GemmItem it; int ntile; int ksteps; bool skip; };
    auto get_unit = [&](int u) {
        Unit w;
        w.it = gp.items[u / P.ntiles];
        w.ntile = u % P.ntiles;
        w.ksteps = w.it.kblocks;
        if (row_packed_a && w.ksteps > P.ksteps_cap - w.it.kfirst) w.ksteps = P.ksteps_cap - w.it.kfirst;
        w.skip = (w.it.m < gp.m0) || (w.it.m >= gp.m0 + gp.mmax_out);
        return w;
    };

    // wait until the MMAs of k-step kc - depth have completed (nothing to wait for during the first `depth` k-steps)
    auto wait_done = [&](int kc, int depth) {
        if (kc < depth) return true;
        const int q = kc - depth;
        return ptx::mbar_wait_bounded(bar_done(q % NRING), (uint32_t)((q / NRING) & 1), abort_flag, WAIT_LIMIT);
    };

    if (warp == 0) {
        // =========================== TMA producer ===========================
        if (lane == 0) {
            int s = 0, kc = 0;
            bool ok = true;
            const uint32_t bytes = (uint32_t)(A_TILE_BYTES + (gp.b_mn ? P.bblk * B_BLK_BYTES : P.bn * TK * 4));
            for (int u = blockIdx.x; u < P.nunits && ok; u += gridDim.x) {
                const Unit w = get_unit(u);
                if (w.skip) continue;
                const long long by0 = gp.b_mn ? ((long long)w.it.b_y0 - gp.b_unit0) * TK  // 32-row block of this group inside a k-step
                                              : ((long long)w.it.b_y0 - gp.b_unit0) * gp.ncols + (long long)w.ntile * P.bn;
                for (int ki = 0; ki < w.ksteps; ++ki) {
                    const int ks = ki + w.it.kfirst;  // slice of the operands
                    if (!(ok = wait_done(kc, NSTAGE))) break;
                    ptx::mbar_arrive_expect_tx(bar_full(s), bytes);
                    const uint32_t dst = stage0 + s * STAGE_BYTES;
                    ptx::tma_load_2d(dst, &tmA, row_packed_a ? ks * TK : 0, w.it.a_y0 + (row_packed_a ? 0 : ks * w.it.a_dy), bar_full(s));
                    if (gp.b_mn) {
                        // 32 contraction rows x 32 columns per box; consecutive boxes hold consecutive column blocks
                        for (int i = 0; i < P.bblk; ++i)
                            ptx::tma_load_2d(dst + B_OFF + i * B_BLK_BYTES, &tmB, w.ntile * P.bn + 32 * i, (int)(by0 + (long long)ks * gp.b_groups * TK), bar_full(s));
                    } else {
                        const long long by = by0 + (row_packed_b ? 0 : (long long)ks * w.it.b_dy * gp.ncols);
                        ptx::tma_load_2d(dst + B_OFF, &tmB, row_packed_b ? ks * TK : 0, (int)by, bar_full(s));
                    }
                    if (++s == NSTAGE) s = 0;
                    ++kc;
                }
            }
        }
    } else if (warp == 1) {
        // =========================== MMA issuer ===========================
        if (lane == 0) {
            int s = 0, a = 0, t = 0, r = 0;
            uint32_t pha = 0, phr = 0;
            bool ok = true;
            const uint32_t idesc = ptx::idesc_tf32_m128((uint32_t)P.bn) | (gp.b_mn ? (1u << 16) : 0u);  // bit 16: B is column (MN) major
            // One MMA consumes 8 contraction indices: 8 columns of A in tensor memory; of B 32 bytes along a K-major row or
            // one 8-row (1 KiB) group of a column-major tile (in the 16-byte units of the descriptor's address field).
            const bool b_mn = gp.b_mn != 0;
            const uint32_t bstep = b_mn ? (1024u >> 4) : (32u >> 4);
            // descriptors of the B tiles: everything but the start address is the same for all of them
            const uint64_t bdesc0 = b_mn ? ptx::smem_desc_sw128_mn(0, B_BLK_BYTES) : ptx::smem_desc_sw128(0);
            const uint32_t b_hi32 = (uint32_t)(bdesc0 >> 32), b_lo_fixed = (uint32_t)bdesc0;
            uint32_t b_raw_lo[NSTAGE], b_lo_lo[NSTAGE];
#pragma unroll
            for (int i = 0; i < NSTAGE; ++i) {
                b_raw_lo[i] = b_lo_fixed | (((stage0 + i * STAGE_BYTES + B_OFF) & 0x3FFFFu) >> 4);
                b_lo_lo[i] = b_lo_fixed | (((stage0 + i * STAGE_BYTES) & 0x3FFFFu) >> 4);
            }
            const uint32_t a_tm0 = tmem_base + (uint32_t)A_TM_COL0;
            for (int u = blockIdx.x; u < P.nunits && ok; u += gridDim.x) {
                const Unit w = get_unit(u);
                if (w.skip) continue;
                // this accumulator buffer must have been drained by the epilogue (NACC units ago)
                if (!(ok = ptx::mbar_wait_bounded(bar_accempty(a), pha ^ 1u, abort_flag, WAIT_LIMIT))) break;
                ptx::tc_fence_after();
                const uint32_t d = tmem_base + (uint32_t)(a * BN_MAX);
                for (int ks = 0; ks < w.ksteps; ++ks) {
                    if (!(ok = ptx::mbar_wait_bounded(bar_ready(r), phr, abort_flag, WAIT_LIMIT))) break;
                    ptx::tc_fence_after();
                    const uint32_t ah = a_tm0 + (uint32_t)(t * 2 * TK);  // A as it is; its low part TK columns further
                    uint32_t brl = b_raw_lo[0], bll = b_lo_lo[0];  // (selects instead of indexed local arrays)
#pragma unroll
                    for (int i = 1; i < NSTAGE; ++i) {
                        brl = (s == i) ? b_raw_lo[i] : brl;
                        bll = (s == i) ? b_lo_lo[i] : bll;
                    }
                    ptx::mma_tf32_kstep32(d, ah, ah + TK, brl, bll, b_hi32, bstep, idesc, ks ? 1u : 0u);
                    ptx::tc_commit(bar_done(r));
                    if (++s == NSTAGE) s = 0;
                    if (++t == NATM) t = 0;
                    if (++r == NRING) { r = 0; phr ^= 1u; }
                }
                if (!ok) break;
                ptx::tc_commit(bar_accfull(a));
                if (++a == NACC) { a = 0; pha ^= 1u; }
            }
        }
    } else if (warp < 2 + NSPLIT_A) {
        // =========================== A splitter: shared memory -> tensor memory ===========================
        const int q = warp & 3;              // tensor-memory lane quarter this warp may write
        const int row = q * 32 + lane;       // row of the A tile = lane of tensor memory
        int s = 0, t = 0, kc = 0;
        uint32_t ph = 0;
        bool ok = true;
        for (int u = blockIdx.x; u < P.nunits && ok; u += gridDim.x) {
            const Unit w = get_unit(u);
            if (w.skip) continue;
            for (int ks = 0; ks < w.ksteps; ++ks) {
                if (!(ok = ptx::mbar_wait_bounded(bar_full(s), ph, abort_flag, WAIT_LIMIT))) break;
                // row `row` of the 128-byte-swizzled tile: 16-byte chunk j sits at position j ^ (row & 7)
                const uint8_t *arow = base_ptr + s * STAGE_BYTES + row * 128;
                float v[TK];
#pragma unroll
                for (int j = 0; j < TK / 4; ++j) {
                    const float4 x = *reinterpret_cast<const float4 *>(arow + ((j ^ (row & 7)) << 4));
                    v[4 * j] = x.x, v[4 * j + 1] = x.y, v[4 * j + 2] = x.z, v[4 * j + 3] = x.w;
                }
                __syncwarp();  // the tile is in registers: its region of the stage may be overwritten
                if (lane == 0) ptx::mbar_arrive(bar_aread(s));
                if (!(ok = wait_done(kc, NATM))) break;
                ptx::tc_fence_after();
                const uint32_t ta = tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(A_TM_COL0 + t * 2 * TK);
                ptx::tmem_st32(ta, v);
#pragma unroll
                for (int j = 0; j < TK; ++j) v[j] = tf32_lo(v[j]);
                ptx::tmem_st32(ta + TK, v);
                ptx::tmem_st_wait();
                ptx::tc_fence_before();
                __syncwarp();  // one arrival per warp
                if (lane == 0) ptx::mbar_arrive(bar_ready(kc % NRING));
                if (++s == NSTAGE) { s = 0; ph ^= 1u; }
                if (++t == NATM) t = 0;
                ++kc;
            }
        }
    } else if (warp < 2 + NSPLIT_WARPS) {
        // =========================== B splitter ===========================
        const int tid = threadIdx.x - 32 * (2 + NSPLIT_A);
        constexpr int NT = 32 * NSPLIT_B;
        int s = 0, kc = 0;
        uint32_t ph = 0;
        bool ok = true;
        const int nb4 = (gp.b_mn ? P.bblk * B_BLK_BYTES : P.bn * TK * 4) / 16;
        for (int u = blockIdx.x; u < P.nunits && ok; u += gridDim.x) {
            const Unit w = get_unit(u);
            if (w.skip) continue;
            for (int ks = 0; ks < w.ksteps; ++ks) {
                if (!(ok = ptx::mbar_wait_bounded(bar_full(s), ph, abort_flag, WAIT_LIMIT))) break;
                float4 *src = reinterpret_cast<float4 *>(base_ptr + s * STAGE_BYTES + B_OFF);
                float4 *dst = reinterpret_cast<float4 *>(base_ptr + s * STAGE_BYTES);  // the region the A tile arrived in
                // all loads of a thread are issued before the first store
                constexpr int PER = (B_TILE_BYTES / 16 + NT - 1) / NT;
                float4 v[PER];
#pragma unroll
                for (int j = 0; j < PER; ++j) {
                    const int i = tid + j * NT;
                    if (i < nb4) v[j] = src[i];
                }
#pragma unroll
                for (int j = 0; j < PER; ++j) v[j] = make_float4(tf32_lo(v[j].x), tf32_lo(v[j].y), tf32_lo(v[j].z), tf32_lo(v[j].w));
                // the A splitter must have taken the A tile out of the region first
                if (!(ok = ptx::mbar_wait_bounded(bar_aread(s), ph, abort_flag, WAIT_LIMIT))) break;
#pragma unroll
                for (int j = 0; j < PER; ++j) {
                    const int i = tid + j * NT;
                    if (i < nb4) dst[i] = v[j];
                }
                ptx::fence_proxy_async_smem();
                __syncwarp();
                if (lane == 0) ptx::mbar_arrive(bar_ready(kc % NRING));
                if (++s == NSTAGE) { s = 0; ph ^= 1u; }
                ++kc;
            }
        }
    } else {
        // =========================== epilogue (two warps per tensor-memory lane quarter) ===========================
        const int ew = warp - (2 + NSPLIT_WARPS);
        const int q = warp & 3;             // lane quarter this warp may read
        const int half = ew >> 2;           // which half of the column chunks this warp handles
        const int row_in_tile = q * 32 + lane;
        int a = 0;
        uint32_t pha = 0;
        bool ok = true;
        const int nchunks = P.bn / 16;
        const int c_begin = half ? (nchunks + 1) / 2 : 0, c_end = half ? nchunks : (nchunks + 1) / 2;
        for (int u = blockIdx.x; u < P.nunits && ok; u += gridDim.x) {
            const Unit w = get_unit(u);
            if (w.skip) continue;
            if (!(ok = ptx::mbar_wait_bounded(bar_accfull(a), pha, abort_flag, WAIT_LIMIT))) break;
            ptx::tc_fence_after();
            const int col0 = w.ntile * P.bn;
            const bool rvalid = row_in_tile < w.it.rows;
            const int rg = w.it.r0 + row_in_tile;  // row inside the group
            const uint32_t trow = tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(a * BN_MAX);
            for (int ch = c_begin; ch < c_end; ++ch) {
                const int cc = ch * 16;
                if (col0 + cc >= gp.ncols) break;  // warp-uniform
                float v[16];
                ptx::tmem_ld16(trow + (uint32_t)cc, v);
                if (gp.mode == EPI_LATROWS) {
                    // A thread holds 16 consecutive columns (64 bytes) of its own row.  Transposing 4 x 4 blocks of 16 bytes inside
                    // every group of 4 lanes lets the 4 lanes store one row's 64 bytes together: one request instead of four.
#pragma unroll
                    for (int bit = 1; bit <= 2; bit <<= 1) {
                        const bool up = (lane & bit) != 0;
#pragma unroll
                        for (int k = 0; k < 4; ++k) {
                            if (k & bit) continue;
#pragma unroll
                            for (int e = 0; e < 4; ++e) {
                                const float send = up ? v[4 * k + e] : v[4 * (k | bit) + e];
                                const float got = __shfl_xor_sync(0xffffffffu, send, bit);
                                if (up) v[4 * k + e] = got;
                                else v[4 * (k | bit) + e] = got;
                            }
                        }
                    }
                    // now v[4 k .. 4 k + 3] = columns 4 (lane & 3) .. of the row of lane (lane & ~3) + k
                    const int g = 2 * (w.it.m - gp.m0) + w.it.p;
                    const int colq = col0 + cc + 4 * (lane & 3);
#pragma unroll
                    for (int k = 0; k < 4; ++k) {
                        const int rr = (q * 32 + (lane & ~3) + k);  // row inside the tile
                        if (rr < w.it.rows && colq < gp.ncols)  // (columns past the last field pad the row pitch: nobody reads them)
                            *reinterpret_cast<float4 *>(gp.out + y_off(g, w.it.r0 + rr, colq, gp.out_groups, gp.out_ld)) =
                                make_float4(v[4 * k], v[4 * k + 1], v[4 * k + 2], v[4 * k + 3]);
                    }
                    continue;
                }
                if (!rvalid) continue;
                if (gp.mode == EPI_SLABS) {
                    const long long slab = gp.slab0[2 * (w.it.m - gp.m_base) + w.it.p] - gp.slab_unit0 + (rg >> 5);
                    float *o = gp.out + (size_t)slab * gp.ncols * kBK + (rg & 31);
#pragma unroll
                    for (int j = 0; j < 16; ++j) {
                        const int col = col0 + cc + j;
                        if (col < gp.ncols) o[(size_t)col * kBK] = v[j];
                    }
                }
            }
            ptx::tc_fence_before();
            __syncwarp();
            if (lane == 0) ptx::mbar_arrive(bar_accempty(a));
            if (++a == NACC) { a = 0; pha ^= 1u; }
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

int make_map(CUtensorMap *tm, const float *base, long long inner, long long rows, long long pitch_floats, int box_rows, bool atom32 = false) {
    if (inner <= 0 || rows <= 0) return fail(SHTB200_EINVAL, "empty operand");
    EncodeTiledFn fn = encode_fn();
    if (!fn) return fail(SHTB200_ECUDA, "cuTensorMapEncodeTiled not available from the driver");
    cuuint64_t dims[2] = {(cuuint64_t)inner, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)pitch_floats * 4};
    cuuint32_t box[2] = {(cuuint32_t)TK, (cuuint32_t)box_rows};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = fn(tm, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, (void *)base, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, atom32 ? CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B : CU_TENSOR_MAP_SWIZZLE_128B,
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
    // The opt-in to large dynamic shared memory is a per-device attribute of the kernel: set it for the current device
    // (the plan's, made current by the caller) on every launch; the SM count is the plan's device's as well.
    SHT_CUDA_CHECK(cudaFuncSetAttribute(legendre_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES));
    const int sm_count = effective_sms(pl.sm_count);
    TcParams P{};
    P.gp = gp;
    P.bn = std::min<int>(BN_MAX, (int)round_up(gp.ncols, 16));
    P.ntiles = ceil_div(gp.ncols, P.bn);
    P.nunits = gp.nitems * P.ntiles;
    P.ksteps_cap = ceil_div(gp.a_kext, TK);
    P.bblk = ceil_div(P.bn, 32);
    P.err = pl.d_err;

    // extents of the two operands as 2-D row-major tensors
    const bool analysis = gp.mode != EPI_LATROWS;
    long long a_rows, a_inner, b_rows, b_inner;
    if (analysis) {
        a_inner = gp.a_kext;
        a_rows = pl.group_a0.back() + kItemRowsMax;
        b_inner = gp.ncols;  // columns beyond it read as zeros
        b_rows = (long long)gp.b_groups * round_up(gp.b_krows, TK);
    } else {
        a_inner = kBK;
        a_rows = pl.group_a0.back() + kItemRowsMax;
        b_inner = kBK;
        b_rows = (pl.group_b0[2 * (gp.m0 - pl.m_base + gp.mmax_out)] - pl.group_b0[2 * (gp.m0 - pl.m_base)]) * (long long)gp.ncols;
    }
    CUtensorMap tmA, tmB;
    int rc;
    if ((rc = make_map(&tmA, gp.A, a_inner, a_rows, gp.a_pitch, TILE_M))) return rc;
    if ((rc = make_map(&tmB, gp.B, b_inner, b_rows, gp.b_pitch, gp.b_mn ? 32 : P.bn, gp.b_mn != 0))) return rc;

    const int grid = std::min(sm_count, P.nunits);
    legendre_tc_kernel<<<grid, NTHREADS, SMEM_BYTES, st>>>(tmA, tmB, P);
    SHT_CUDA_CHECK(cudaGetLastError());
    return SHTB200_OK;
}

}  // namespace shtb200
