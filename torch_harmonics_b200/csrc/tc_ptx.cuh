// Thin inline-PTX wrappers for the Blackwell (sm_100a) features the Legendre kernel uses:
// mbarrier, TMA tiled loads (cp.async.bulk.tensor), tcgen05 MMA / TMEM allocation / TMEM loads.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace shtb200 {
namespace ptx {

__device__ __forceinline__ uint32_t smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }

// ---------------------------------------------------------------- mbarrier
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("{\n\t.reg .b64 st;\n\tmbarrier.arrive.shared::cta.b64 st, [%0];\n\t}" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("{\n\t.reg .b64 st;\n\tmbarrier.arrive.expect_tx.shared::cta.b64 st, [%0], %1;\n\t}" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ uint32_t mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok;
}
// Wait for the phase with the given parity to complete, giving up after `limit_cycles` clock ticks or as soon as
// another thread of the CTA has raised *abort_flag.  Returns false when it gave up (and raises the flag itself).
__device__ __forceinline__ bool mbar_wait_bounded(uint32_t bar, uint32_t parity, volatile int *abort_flag, long long limit_cycles) {
    if (mbar_try_wait(bar, parity)) return true;
    const long long t0 = clock64();
    for (uint32_t it = 1;; ++it) {
        if (mbar_try_wait(bar, parity)) return true;
        if ((it & 255u) == 0u) {
            if (*abort_flag) return false;
            if (clock64() - t0 > limit_cycles) {
                *abort_flag = 1;
                return false;
            }
        }
    }
}

__device__ __forceinline__ void fence_barrier_init() { asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }
__device__ __forceinline__ void fence_proxy_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

// ---------------------------------------------------------------- TMA
__device__ __forceinline__ void prefetch_tensormap(const CUtensorMap *tm) {
    asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(tm)) : "memory");
}
// 2-D tiled load global -> shared, completion counted in bytes on `bar`.  x is the inner (contiguous) coordinate
// and must be a multiple of 4 floats (16 bytes).
__device__ __forceinline__ void tma_load_2d(uint32_t dst_smem, const CUtensorMap *tm, int x, int y, uint32_t bar) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];" ::"r"(dst_smem),
                 "l"(reinterpret_cast<uint64_t>(tm)), "r"(bar), "r"(x), "r"(y)
                 : "memory");
}

// Untiled bulk copy global -> shared; both addresses 16-byte aligned, size a multiple of 16 bytes.
__device__ __forceinline__ void bulk_load(uint32_t dst_smem, const void *src, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst_smem),
                 "l"(reinterpret_cast<uint64_t>(src)), "r"(bytes), "r"(bar)
                 : "memory");
}

// Untiled bulk copy shared -> global (same alignment rules), tracked by the issuing thread's bulk async-group.
__device__ __forceinline__ void bulk_store(void *dst, uint32_t src_smem, uint32_t bytes) {
    asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(reinterpret_cast<uint64_t>(dst)), "r"(src_smem), "r"(bytes) : "memory");
}
__device__ __forceinline__ void bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
// returns once the committed bulk stores of this thread have finished READING shared memory
__device__ __forceinline__ void bulk_wait_read_all() { asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory"); }

// ---------------------------------------------------------------- tcgen05 / TMEM
__device__ __forceinline__ void tmem_alloc(uint32_t slot_smem, uint32_t ncols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(slot_smem), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish() { asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

// D[tmem] (+)= A[smem] * B[smem], 128 x N x 8 TF32, fp32 accumulate.  One thread issues.
__device__ __forceinline__ void mma_tf32(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n\t}" ::"r"(d_tmem),
        "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
}
// Same with the A operand taken from tensor memory: row i of A in lane i, contraction index along the columns.
__device__ __forceinline__ void mma_tf32_ta(uint32_t d_tmem, uint32_t a_tmem, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::tf32 [%0], [%1], %2, %3, p;\n\t}" ::"r"(d_tmem),
        "r"(a_tmem), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
}
// One k-step of the split-TF32 contraction as ONE instruction sequence: 4 slices of 8 contraction indices, each with the
// three products A_lo B, A B_lo, A B (small terms first).  A comes from tensor memory (`a_raw`, `a_lo`: column addresses,
// +8 columns per slice), B from shared memory through descriptors whose high words are equal (`b_hi32`) and whose low
// words (`b_raw_lo32`, `b_lo_lo32`) advance by `b_step` per slice.  `accumulate` = 0 makes the very first product
// overwrite the accumulator.  Written as a single asm block because the issuing thread's scalar instruction latency,
// not the tensor pipe, bounds the issue rate otherwise: this keeps it to two adds per operand and slice.
__device__ __forceinline__ void mma_tf32_kstep32(uint32_t d_tmem, uint32_t a_raw, uint32_t a_lo, uint32_t b_raw_lo32, uint32_t b_lo_lo32, uint32_t b_hi32,
                                                 uint32_t b_step, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t"
        ".reg .pred p0, p1;\n\t"
        ".reg .b32 ar1, ar2, ar3, al1, al2, al3, br1, br2, br3, bl1, bl2, bl3;\n\t"
        ".reg .b64 dr0, dr1, dr2, dr3, dl0, dl1, dl2, dl3;\n\t"
        "setp.ne.b32 p0, %8, 0;\n\t"
        "setp.eq.b32 p1, %8, %8;\n\t"
        "add.u32 ar1, %1, 8;\n\t"
        "add.u32 ar2, %1, 16;\n\t"
        "add.u32 ar3, %1, 24;\n\t"
        "add.u32 al1, %2, 8;\n\t"
        "add.u32 al2, %2, 16;\n\t"
        "add.u32 al3, %2, 24;\n\t"
        "add.u32 br1, %3, %6;\n\t"
        "add.u32 br2, br1, %6;\n\t"
        "add.u32 br3, br2, %6;\n\t"
        "add.u32 bl1, %4, %6;\n\t"
        "add.u32 bl2, bl1, %6;\n\t"
        "add.u32 bl3, bl2, %6;\n\t"
        "mov.b64 dr0, {%3, %5};\n\t"
        "mov.b64 dl0, {%4, %5};\n\t"
        "mov.b64 dr1, {br1, %5};\n\t"
        "mov.b64 dl1, {bl1, %5};\n\t"
        "mov.b64 dr2, {br2, %5};\n\t"
        "mov.b64 dl2, {bl2, %5};\n\t"
        "mov.b64 dr3, {br3, %5};\n\t"
        "mov.b64 dl3, {bl3, %5};\n\t"
        "tcgen05.mma.cta_group::1.kind::tf32 [%0], [%2], dr0, %7, p0;\n\t"
        "tcgen05.mma.cta_group::1.kind::tf32 [%0], [%1], dl0, %7, p1;\n\t"
        "tcgen05.mma.cta_group::1.kind::tf32 [%0], [%1], dr0, %7, p1;\n\t"
        "tcgen05.mma.cta_group::1.kind::tf32 [%0], [al1], dr1, %7, p1;\n\t"
        "tcgen05.mma.cta_group::1.kind::tf32 [%0], [ar1], dl1, %7, p1;\n\t"
        "tcgen05.mma.cta_group::1.kind::tf32 [%0], [ar1], dr1, %7, p1;\n\t"
        "tcgen05.mma.cta_group::1.kind::tf32 [%0], [al2], dr2, %7, p1;\n\t"
        "tcgen05.mma.cta_group::1.kind::tf32 [%0], [ar2], dl2, %7, p1;\n\t"
        "tcgen05.mma.cta_group::1.kind::tf32 [%0], [ar2], dr2, %7, p1;\n\t"
        "tcgen05.mma.cta_group::1.kind::tf32 [%0], [al3], dr3, %7, p1;\n\t"
        "tcgen05.mma.cta_group::1.kind::tf32 [%0], [ar3], dl3, %7, p1;\n\t"
        "tcgen05.mma.cta_group::1.kind::tf32 [%0], [ar3], dr3, %7, p1;\n\t"
        "}" ::"r"(d_tmem),
        "r"(a_raw), "r"(a_lo), "r"(b_raw_lo32), "r"(b_lo_lo32), "r"(b_hi32), "r"(b_step), "r"(idesc), "r"(accumulate)
        : "memory");
}
// 32 lanes x 32 consecutive 32-bit columns <- 32 registers per thread (lane = thread); completion by tmem_st_wait()
__device__ __forceinline__ void tmem_st32(uint32_t taddr, const float *v) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,"
        "%29,%30,%31,%32};" ::"r"(taddr),
        "r"(__float_as_uint(v[0])), "r"(__float_as_uint(v[1])), "r"(__float_as_uint(v[2])), "r"(__float_as_uint(v[3])), "r"(__float_as_uint(v[4])),
        "r"(__float_as_uint(v[5])), "r"(__float_as_uint(v[6])), "r"(__float_as_uint(v[7])), "r"(__float_as_uint(v[8])), "r"(__float_as_uint(v[9])),
        "r"(__float_as_uint(v[10])), "r"(__float_as_uint(v[11])), "r"(__float_as_uint(v[12])), "r"(__float_as_uint(v[13])), "r"(__float_as_uint(v[14])),
        "r"(__float_as_uint(v[15])), "r"(__float_as_uint(v[16])), "r"(__float_as_uint(v[17])), "r"(__float_as_uint(v[18])), "r"(__float_as_uint(v[19])),
        "r"(__float_as_uint(v[20])), "r"(__float_as_uint(v[21])), "r"(__float_as_uint(v[22])), "r"(__float_as_uint(v[23])), "r"(__float_as_uint(v[24])),
        "r"(__float_as_uint(v[25])), "r"(__float_as_uint(v[26])), "r"(__float_as_uint(v[27])), "r"(__float_as_uint(v[28])), "r"(__float_as_uint(v[29])),
        "r"(__float_as_uint(v[30])), "r"(__float_as_uint(v[31]))
        : "memory");
}
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }
// mbarrier arrives once all tcgen05 operations issued so far by this thread have completed
__device__ __forceinline__ void tc_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
// 32 lanes x 16 consecutive 32-bit columns -> 16 registers per thread (lane = thread)
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, float *v) {
    uint32_t r[16];
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]),
                   "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
                 : "r"(taddr)
                 : "memory");
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
    for (int i = 0; i < 16; ++i) v[i] = __uint_as_float(r[i]);
}

// Shared-memory operand descriptor, K-major, 64-byte swizzle (rows of 16 floats; 8-row groups 512 bytes apart).
__device__ __forceinline__ uint64_t smem_desc_sw64(uint32_t smem_addr) {
    uint64_t d = 0;
    d |= (uint64_t)((smem_addr & 0x3FFFFu) >> 4);  // start address, bits [0, 14)
    d |= (uint64_t)1 << 16;                        // leading byte offset (unused with swizzled K-major), bits [16, 30)
    d |= (uint64_t)(512u >> 4) << 32;              // stride byte offset between 8-row groups, bits [32, 46)
    d |= (uint64_t)1 << 46;                        // descriptor version of this architecture, bits [46, 48)
    d |= (uint64_t)4 << 61;                        // layout type SWIZZLE_64B, bits [61, 64)
    return d;
}
// Same for the 128-byte swizzle (rows of 32 floats; 8-row groups 1024 bytes apart).
__device__ __forceinline__ uint64_t smem_desc_sw128(uint32_t smem_addr) {
    uint64_t d = 0;
    d |= (uint64_t)((smem_addr & 0x3FFFFu) >> 4);
    d |= (uint64_t)1 << 16;
    d |= (uint64_t)(1024u >> 4) << 32;
    d |= (uint64_t)1 << 46;
    d |= (uint64_t)2 << 61;  // layout type SWIZZLE_128B
    return d;
}
// Column-contiguous ("MN-major") 32-bit operand: the only layout the tensor core takes for it is the 128-byte
// swizzle with 32-byte atoms (TMA mode SWIZZLE_128B_ATOM_32B).  The tile is a sequence of blocks of 32 columns;
// inside a block each contraction index is one 128-byte row and 4 rows form a 512-byte swizzle group.
// Leading byte offset = distance between column blocks, stride byte offset = distance between 4-row groups.
__device__ __forceinline__ uint64_t smem_desc_sw128_mn(uint32_t smem_addr, uint32_t block_bytes) {
    uint64_t d = 0;
    d |= (uint64_t)((smem_addr & 0x3FFFFu) >> 4);
    d |= (uint64_t)((block_bytes >> 4) & 0x3FFFu) << 16;
    d |= (uint64_t)(512u >> 4) << 32;
    d |= (uint64_t)1 << 46;
    d |= (uint64_t)1 << 61;  // layout type SWIZZLE_128B_BASE32B
    return d;
}
// Instruction descriptor: fp32 accumulator, TF32 x TF32, both K-major, M = 128, N = n.
__device__ __forceinline__ uint32_t idesc_tf32_m128(uint32_t n) { return (1u << 4) | (2u << 7) | (2u << 10) | ((n >> 3) << 17) | ((128u >> 4) << 24); }

}  // namespace ptx
}  // namespace shtb200
