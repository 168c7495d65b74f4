// Inline-PTX building blocks for sm_100a: mbarriers with BOUNDED waits, 1-D bulk async copies
// (TMA engine, no tensor map, one destination CTA), TMEM allocation and tcgen05 MMA / load.
//
// Every wait in this file gives up after a clock budget and reports failure to its caller, so a
// kernel built from these pieces cannot spin forever: the caller sets its abort flag, lets the
// other roles drain, frees its TMEM and returns with an error code in the context's status word.
#pragma once
#include <cuda_runtime.h>

#include <cstdint>

namespace zb {
namespace ptx {

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ bool elect_one() {
    uint32_t pred = 0;
    asm volatile(
        "{\n\t.reg .pred P;\n\telect.sync _|P, 0xffffffff;\n\tselp.b32 %0, 1, 0, P;\n\t}\n"
        : "=r"(pred));
    return pred != 0;
}

// ---------------------------------------------------------------------------- mbarrier
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_fence_init() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("{\n\t.reg .b64 st;\n\tmbarrier.arrive.shared::cta.b64 st, [%0];\n\t}\n" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("{\n\t.reg .b64 st;\n\tmbarrier.arrive.expect_tx.shared::cta.b64 st, [%0], %1;\n\t}\n" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred P;\n\tmbarrier.try_wait.parity.shared::cta.b64 P, [%1], %2, %3;\n\tselp.b32 %0, 1, 0, P;\n\t}\n"
        : "=r"(ok) : "r"(bar), "r"(parity), "r"(2000u) : "memory");   // may suspend the thread for up to ~2 us before reporting "not yet"
    return ok != 0;
}

// About two seconds at 2 GHz; a healthy pipeline waits microseconds.
constexpr long long kWaitBudgetCycles = 4000000000LL;

// Waits for the phase with the given parity.  Returns false when the budget (in SM clock cycles) ran
// out or when another role already raised `*abort_flag` (a shared-memory int).  The production kernels
// use the default budget; the bounded-wait self test passes a budget of microseconds.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag,
                                          long long budget_cycles = kWaitBudgetCycles) {
    if (mbar_try_wait(bar, parity)) return true;
    const long long t0 = clock64();
    const uint32_t check_mask = budget_cycles < (1LL << 24) ? 3u : 255u;   // short budgets look at the clock more often
    uint32_t spins = 0;
    while (true) {
        if (mbar_try_wait(bar, parity)) return true;
        if (++spins > 32) __nanosleep(40);
        if ((spins & check_mask) == 0u) {
            if (*abort_flag) return false;
            if (clock64() - t0 > budget_cycles) { *abort_flag = 1; return false; }
        }
    }
}

// The same wait for roles that are far ahead of the critical path (a loader several stages ahead, an MMA issuer or an
// epilogue warp of a memory-bound kernel): the thread sleeps between polls, so that a waiting warp issues a few
// instructions per microsecond instead of competing for issue slots with the warps that do the arithmetic.
__device__ __forceinline__ bool mbar_wait_sleeping(uint32_t bar, uint32_t parity, volatile int* abort_flag,
                                                   long long budget_cycles = kWaitBudgetCycles) {
    if (mbar_try_wait(bar, parity)) return true;
    const long long t0 = clock64();
    uint32_t polls = 0;
    while (true) {
        __nanosleep(polls < 8u ? 64u : 256u);
        if (mbar_try_wait(bar, parity)) return true;
        if ((++polls & 63u) == 0u) {
            if (*abort_flag) return false;
            if (clock64() - t0 > budget_cycles) { *abort_flag = 1; return false; }
        }
    }
}

// Generic-proxy writes to shared memory (st.shared) must be fenced before the async proxy
// (TMA, tcgen05.mma) reads them.
__device__ __forceinline__ void fence_proxy_async_smem() {
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

// ---------------------------------------------------------------------------- bulk async copy (1-D)
// global -> shared, completion counted in bytes on an mbarrier.  Addresses 16-byte aligned, size a
// multiple of 16.  The destination is this CTA's own shared memory and nothing else.
__device__ __forceinline__ void bulk_g2s(uint32_t dst_smem, const void* src_gmem, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(dst_smem), "l"(src_gmem), "r"(bytes), "r"(bar) : "memory");
}

// shared -> global, as a bulk group of the issuing thread; the group is committed here and waited for, later, by the same
// thread: bulk_wait_read<N> until at most N of its groups still read their shared-memory source, bulk_wait_all until all
// of them are complete.  Writes to the source by other threads need fence_proxy_async_smem and a barrier before the copy.
__device__ __forceinline__ void bulk_s2g(void* dst_gmem, uint32_t src_smem, uint32_t bytes) {
    asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(dst_gmem), "r"(src_smem), "r"(bytes) : "memory");
    asm volatile("cp.async.bulk.commit_group;" ::: "memory");
}
template <int N>
__device__ __forceinline__ void bulk_wait_read() { asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory"); }
__device__ __forceinline__ void bulk_wait_all() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }

// ---------------------------------------------------------------------------- tiled TMA loads
// Box of a tensor map -> this CTA's shared memory (128-byte aligned), completion counted in bytes
// on an mbarrier.  The innermost coordinate times the element size must be a multiple of 16 bytes.
// One destination CTA.  `tmap` is the generic address of a CUtensorMap kernel parameter.
__device__ __forceinline__ void tma_load_3d(uint32_t dst_smem, const void* tmap, int x, int y, int z, uint32_t bar) {
    asm volatile("cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];"
                 ::"r"(dst_smem), "l"(tmap), "r"(x), "r"(y), "r"(z), "r"(bar) : "memory");
}
__device__ __forceinline__ void tma_load_4d(uint32_t dst_smem, const void* tmap, int x, int y, int z, int w, uint32_t bar) {
    asm volatile("cp.async.bulk.tensor.4d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4, %5}], [%6];"
                 ::"r"(dst_smem), "l"(tmap), "r"(x), "r"(y), "r"(z), "r"(w), "r"(bar) : "memory");
}

// ---------------------------------------------------------------------------- TMEM
// One full warp allocates `cols` (power of two >= 32) columns; the base address lands in smem.
__device__ __forceinline__ void tmem_alloc(uint32_t dst_smem, uint32_t cols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(dst_smem), "r"(cols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t cols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tmem_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// ---------------------------------------------------------------------------- descriptors
// Shared-memory matrix descriptor, K-major, no swizzle.  In 16-byte units the operand is
//   ((8, rows/8), 2) : ((1, SBO), LBO)
// i.e. 8 consecutive rows are 8 consecutive 16-byte chunks, the next 8-row group lies SBO bytes
// further, and the second 16-byte K chunk of a 32-byte MMA K step lies LBO bytes further.
__device__ __forceinline__ uint64_t smem_desc_kmajor(uint32_t addr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
    uint64_t d = 0;
    d |= (uint64_t)((addr >> 4) & 0x3FFFu);
    d |= (uint64_t)((lbo_bytes >> 4) & 0x3FFFu) << 16;
    d |= (uint64_t)((sbo_bytes >> 4) & 0x3FFFu) << 32;
    d |= (uint64_t)1 << 46;   // descriptor version for sm_100
    return d;                  // base_offset 0, lbo_mode 0, layout type 0 (no swizzle)
}

// Shared-memory matrix descriptor, MN-major with the 128-byte swizzle: the operand's M (or N) index
// runs along 128-byte rows (128 int8 elements, their 16-byte chunks XOR-swizzled with the row number
// as a TMA load with SWIZZLE_128B writes them), eight consecutive K indices are eight consecutive rows,
// and the next group of eight K indices lies SBO bytes further; LBO is the distance to the next
// 128-element block along M/N.  The tile must start at a 1024-byte boundary.
__device__ __forceinline__ uint64_t smem_desc_mnmajor_sw128(uint32_t addr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
    uint64_t d = 0;
    d |= (uint64_t)((addr >> 4) & 0x3FFFu);
    d |= (uint64_t)((lbo_bytes >> 4) & 0x3FFFu) << 16;
    d |= (uint64_t)((sbo_bytes >> 4) & 0x3FFFu) << 32;
    d |= (uint64_t)1 << 46;   // descriptor version for sm_100
    d |= (uint64_t)2 << 61;   // layout type: 128-byte swizzle
    return d;
}

// Instruction descriptor for kind::i8: int32 accumulator, K-major A and B.
// a_unsigned / b_unsigned choose uint8 (0) or int8 (1) in the format fields.
__host__ __device__ constexpr uint32_t idesc_i8(int M, int N, bool a_signed, bool b_signed) {
    return (2u << 4) | ((a_signed ? 1u : 0u) << 7) | ((b_signed ? 1u : 0u) << 10) |
           ((uint32_t)(N >> 3) << 17) | ((uint32_t)(M >> 4) << 24);
}
// Bit 15 of the instruction descriptor: A is MN-major (its M index is the contiguous one).
constexpr uint32_t kIdescAMnMajor = 1u << 15;

// D[tmem] (+)= A[smem] * B[smem]; issued by ONE thread.
__device__ __forceinline__ void mma_i8(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, bool accumulate) {
    const uint32_t acc = accumulate ? 1u : 0u;
    const uint32_t zero = 0u;
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, {%5, %5, %5, %5}, p;\n\t}\n"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(acc), "r"(zero) : "memory");
}

// The same with the descriptors given as 32-bit halves.  The low half holds the start address (bits 0-13,
// in 16-byte units) and the leading-dimension offset; the issuing thread of a loop over taps, K steps and
// row blocks only ever changes the start address, so it keeps the high halves fixed and advances the low
// ones with single 32-bit adds (shared memory is smaller than 256 KiB: the address field cannot overflow).
// That keeps the instruction count per MMA of a data-dependent loop at a handful; 64-bit descriptor
// arithmetic in such a loop costs more issue time than a 128x64x32 MMA takes to execute.
__device__ __forceinline__ void mma_i8_halves(uint32_t d_tmem, uint32_t a_lo, uint32_t a_hi, uint32_t b_lo, uint32_t b_hi, uint32_t idesc, uint32_t accumulate) {
    const uint32_t zero = 0u;
    asm volatile(
        "{\n\t.reg .pred p;\n\t.reg .b64 da, db;\n\tsetp.ne.b32 p, %6, 0;\n\t"
        "mov.b64 da, {%1, %2};\n\tmov.b64 db, {%3, %4};\n\t"
        "tcgen05.mma.cta_group::1.kind::i8 [%0], da, db, %5, {%7, %7, %7, %7}, p;\n\t}\n"
        ::"r"(d_tmem), "r"(a_lo), "r"(a_hi), "r"(b_lo), "r"(b_hi), "r"(idesc), "r"(accumulate), "r"(zero) : "memory");
}

// Arrives on the mbarrier once every MMA issued so far by this thread has completed.
__device__ __forceinline__ void mma_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}

// 32 lanes x 32 consecutive columns of 32-bit accumulators: thread i of the warp receives the 32
// columns of TMEM lane (lane_base + i).  A warp may only touch the lane quarter (warp_id % 4).
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t* r) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
          "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
          "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr) : "memory");
}

// 32 lanes x 16 consecutive columns.
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t* r) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr) : "memory");
}

__device__ __forceinline__ void named_barrier_sync(uint32_t id, uint32_t threads) {
    asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(threads) : "memory");
}

}  // namespace ptx
}  // namespace zb
