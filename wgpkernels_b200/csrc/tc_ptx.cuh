// Inline-PTX wrappers of the sm_100a machinery the INT8 GEMM is built from: mbarriers with bounded waits, TMA tile loads (never with
// cluster multicast), tensor-memory allocation, tcgen05.mma kind::i8 with its shared-memory and instruction descriptors, tcgen05.ld / st.
#pragma once
#include "common.cuh"

namespace wq {

constexpr int kBM = 128;             // rows of a tile = tensor-memory lanes
constexpr int kStageK = 128;         // bytes (= INT8 elements) of K per stage: one 128-byte swizzle row, one scale block
constexpr int kMmaK = 32;            // K of one tcgen05.mma kind::i8
constexpr int kTmemColumns = 512;    // all of an SM's tensor memory (one CTA per SM)

WQ_DEVICE uint32_t smem_u32(const void* p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }

WQ_DEVICE void mbar_init(uint32_t bar, uint32_t count) { asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count)); }
WQ_DEVICE void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
WQ_DEVICE void mbar_arrive(uint32_t bar) { asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory"); }
// One potentially blocking test of the phase: the hardware may suspend the thread for up to `kSuspendNs` (it resumes as soon as the
// phase completes), so a waiting role does not spend its scheduler's issue slots on polling.
constexpr uint32_t kSuspendNs = 4000;
WQ_DEVICE bool mbar_test(uint32_t bar, uint32_t parity);
WQ_DEVICE bool mbar_try_wait(uint32_t bar, uint32_t parity) {
#ifdef WQ_WAIT_SPIN
    return mbar_test(bar, parity);
#endif
    uint32_t done;
#ifdef WQ_WAIT_NOHINT
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(done)
        : "r"(bar), "r"(parity)
        : "memory");
    return done != 0;
#endif
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(done)
        : "r"(bar), "r"(parity), "r"(kSuspendNs)
        : "memory");
    return done != 0;
}
// Non-blocking test of the phase: the cheap first look (the phase has usually completed by the time a role asks).
WQ_DEVICE bool mbar_test(uint32_t bar, uint32_t parity) {
    uint32_t done;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(done)
        : "r"(bar), "r"(parity)
        : "memory");
    return done != 0;
}

// Waits for the phase of `parity`, for roughly `limit` clocks at most; false when the CTA is aborting or the wait ran out (then `code`
// is recorded in `status` and the abort flag raised).  The common case costs one try_wait (which parks the thread in hardware) and a
// branch; the clock and the abort flag are only looked at every 32 unsuccessful tries.
WQ_DEVICE bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag, int code, int* status, long long limit) {
    long long start = 0;
    for (uint32_t spin = 1;; ++spin) {
        if (mbar_try_wait(bar, parity)) return true;
        if ((spin & 31u) == 0u) {
            if (*abort_flag) return false;
            const long long now = clock64();
            if (spin == 32u) start = now;
            if (now - start > limit) {
                *abort_flag = code;
                atomicCAS(status, 0, code);
                return false;
            }
        }
    }
}

WQ_DEVICE void tma_load_2d(uint32_t dst, const CUtensorMap* map, uint32_t bar, int x, int y) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];" ::"r"(dst), "l"(map),
                 "r"(bar), "r"(x), "r"(y)
                 : "memory");
}
WQ_DEVICE void prefetch_tensormap(const CUtensorMap* map) { asm volatile("prefetch.tensormap [%0];" ::"l"(map) : "memory"); }

WQ_DEVICE void tmem_alloc(uint32_t slot_in_smem, uint32_t columns) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(slot_in_smem), "r"(columns) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
WQ_DEVICE void tmem_dealloc(uint32_t address, uint32_t columns) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(address), "r"(columns) : "memory");
}
WQ_DEVICE void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
WQ_DEVICE void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
// The mbarrier is arrived on once every tcgen05 operation this thread issued before has completed.
WQ_DEVICE void tc_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
// D (tensor memory, 128 lanes x N columns of INT32) = or += A (128 x 32 INT8, smem) * B (N x 32 INT8, smem)^T
WQ_DEVICE void mma_i8(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, p;\n\t}" ::"r"(d_tmem),
        "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}

// Consecutive columns of this thread's lane (a warp reads the 32 lanes of its quarter of tensor memory).
#define WQ_R4(a, i) "=r"(a[i]), "=r"(a[i + 1]), "=r"(a[i + 2]), "=r"(a[i + 3])
WQ_DEVICE void tmem_load_32(uint32_t taddr, int* v) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,"
        "%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
        : WQ_R4(v, 0), WQ_R4(v, 4), WQ_R4(v, 8), WQ_R4(v, 12), WQ_R4(v, 16), WQ_R4(v, 20), WQ_R4(v, 24), WQ_R4(v, 28)
        : "r"(taddr)
        : "memory");
}
WQ_DEVICE void tmem_load_16(uint32_t taddr, int* v) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
                 : WQ_R4(v, 0), WQ_R4(v, 4), WQ_R4(v, 8), WQ_R4(v, 12)
                 : "r"(taddr)
                 : "memory");
}
WQ_DEVICE void tmem_load_8(uint32_t taddr, int* v) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];" : WQ_R4(v, 0), WQ_R4(v, 4) : "r"(taddr) : "memory");
}
#undef WQ_R4
// Completes the loads issued before it (the toolchain tracks tcgen05.ld destinations until this instruction).
WQ_DEVICE void tmem_load_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// v[0..7] into the 8 columns starting at taddr of this thread's lane.
WQ_DEVICE void tmem_store_8(uint32_t taddr, const int* v) {
    asm volatile("tcgen05.st.sync.aligned.32x32b.x8.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};" ::"r"(taddr), "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]),
                 "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7])
                 : "memory");
}
WQ_DEVICE void tmem_store_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

// Shared-memory operand descriptor: K-major rows of 128 bytes, 128-byte swizzle, 8-row groups 1024 bytes apart.
WQ_DEVICE uint64_t smem_descriptor(uint32_t address) {
    uint64_t d = (address & 0x3ffffu) >> 4;       // start address, 16-byte units
    d |= uint64_t(1) << 16;                       // leading byte offset (unused for swizzled K-major layouts)
    d |= uint64_t(1024 >> 4) << 32;               // stride byte offset between 8-row groups
    d |= uint64_t(1) << 46;                       // descriptor version of sm_100
    d |= uint64_t(2) << 61;                       // 128-byte swizzle
    return d;
}
// Instruction descriptor: INT32 accumulator, signed INT8 A and B, both K-major, M = 128, N = n.
__host__ __device__ constexpr uint32_t instruction_descriptor(int n) { return (2u << 4) | (1u << 7) | (1u << 10) | (uint32_t(n >> 3) << 17) | (uint32_t(kBM >> 4) << 24); }

}  // namespace wq
