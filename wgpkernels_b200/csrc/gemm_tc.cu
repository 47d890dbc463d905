// INT8 x INT8 -> INT32 GEMM on the 5th-generation tensor cores of sm_100a (tcgen05.mma kind::i8, accumulators in tensor memory),
// operands staged by TMA (no cluster multicast: every CTA loads its own tiles from its GPU's own memory), warp-specialised:
//
//   warp 0      TMA producer: A (and A_lo) 128 x 128-byte tiles, B BN x 128-byte tiles, 128-byte swizzle, ring of STAGES buffers
//   warp 1      MMA issuer: one elected thread, 4 (x2 with a low part) tcgen05.mma of K = 32 per stage
//   warps 2-3   tensor-memory allocation; gather of per-(n, k-block) weight scales into a shared-memory ring (group-scaled weights)
//   warps 4-11  epilogue: tcgen05.ld of the INT32 sums, promotion to FP32, bias / residual, one rounding, stores
//
// Modes (the arithmetic of wgpkernels/int8/int8_gemm.cu:773-805 and :836-863 of WGPKernels):
//   row      INT32 sums over all K; y = fmaf(float(S) * sa[m], sb[n], bias)
//   exact    hi and lo operands share B; v = fmaf(float(S_lo), 1/254, float(S_hi)); y = fmaf(v * sa[m], sb[n], bias)
//   block    per 128 of K: acc = fmaf(float(S_b), sa[m, b], acc); y = fmaf(acc, sb[n], bias)
//   block+g  acc = fmaf(float(S_b), sa[m, b] * sb[n, b], acc); y = acc + bias
//   exact+g  acc = fmaf(fmaf(float(S_lo_b), 1/254, float(S_hi_b)), sb[n, b], acc); y = fmaf(acc * sa[m], 1, bias)
// then y = fmaf(y, rscale[n], residual[m, n]) and one rounding.  In the per-block modes the tensor cores produce one exact INT32 block
// sum per output and 128 of K into a double-buffered tensor-memory accumulator; the epilogue warps drain a buffer (128 x 256 sums) while
// the MMAs of the next block fill the other one, and keep the FP32 accumulators in registers for the whole tile.
//
// Every wait is bounded: a wait that gives up records a code in a device status word, raises a CTA-wide abort flag and the CTA leaves
// through the common exit (tensor memory is always released).
#include <cuda.h>  // CUtensorMap and its enums only; cuTensorMapEncodeTiled is resolved through the runtime, libcuda is not linked

#include "common.cuh"

namespace wq {

enum Mode : int { kRow = 0, kExact = 1, kBlock = 2, kBlockG = 3, kExactG = 4 };

constexpr int kBM = 128;             // rows of a tile = tensor-memory lanes
constexpr int kStageK = 128;         // bytes (= INT8 elements) of K per stage: one 128-byte swizzle row, one scale block
constexpr int kMmaK = 32;            // K of one tcgen05.mma kind::i8
constexpr int kTmemColumns = 512;    // all of an SM's tensor memory (one CTA per SM)
constexpr int kEpilogueWarps = 8;
constexpr int kRearmWarps = 4;       // one per lane quarter of tensor memory: they put the conversion bias back into drained accumulators
constexpr int kThreads = 32 * (4 + kEpilogueWarps + kRearmWarps);
// Registers per thread after the split (setmaxnreg): 512 threads are launched with 128 each; the control and re-arm warps keep 40 and
// the epilogue warps, which hold a tile's FP32 accumulators, take 216: 256 x 40 + 256 x 216 = all 65536.
constexpr int kSmallRegs = 40, kEpilogueRegs = 216;
constexpr int kScaleRing = 4;        // blocks of gathered weight scales in flight
constexpr long long kWaitLimit = 4000000000ll;  // clocks (about two seconds) before a wait gives up

__device__ int g_status = 0;  // first code of a wait that gave up (wq::Status)

#ifdef WQ_TRACE
// Diagnostic build only: clock stamps of CTA 0 (MMA issuer at slot 0, first epilogue warp at slot 4096), read back by wq8_debug_trace.
__device__ long long g_trace[8192];
#define WQ_STAMP(base, index, field) do { if (blockIdx.x == 0 && (index) < 500) g_trace[(base) + (index) * 8 + (field)] = clock64(); } while (0)
#else
#define WQ_STAMP(base, index, field) do {} while (0)
#endif

// ---- PTX wrappers --------------------------------------------------------------------------------------------------
WQ_DEVICE uint32_t smem_u32(const void* p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }

WQ_DEVICE void mbar_init(uint32_t bar, uint32_t count) { asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count)); }
WQ_DEVICE void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
WQ_DEVICE void mbar_arrive(uint32_t bar) { asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory"); }
// One potentially blocking test of the phase: the hardware may suspend the thread for up to `kSuspendNs` (it resumes as soon as the
// phase completes), so a waiting role does not spend its scheduler's issue slots on polling.
constexpr uint32_t kSuspendNs = 4000;
WQ_DEVICE bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t done;
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

// Waits for the phase of `parity`; false when the CTA is aborting or the wait ran out (then `code` is recorded and the abort flag raised).
WQ_DEVICE bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag, int code) {
    if (mbar_test(bar, parity)) return true;
    const long long start = clock64();
    for (uint32_t spin = 1;; ++spin) {
        if (mbar_try_wait(bar, parity)) return true;
        if ((spin & 15u) == 0u) {
            if (*abort_flag) return false;
            if (clock64() - start > kWaitLimit) {
                *abort_flag = code;
                atomicCAS(&g_status, 0, code);
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

// 32 consecutive columns of this thread's lane (a warp reads the 32 lanes of its quarter of tensor memory).
#define WQ_R4(a, i) "=r"(a[i]), "=r"(a[i + 1]), "=r"(a[i + 2]), "=r"(a[i + 3])
WQ_DEVICE void tmem_load_32(uint32_t taddr, int* v) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,"
        "%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
        : WQ_R4(v, 0), WQ_R4(v, 4), WQ_R4(v, 8), WQ_R4(v, 12), WQ_R4(v, 16), WQ_R4(v, 20), WQ_R4(v, 24), WQ_R4(v, 28)
        : "r"(taddr)
        : "memory");
}
#undef WQ_R4
// Completes the loads issued before it (the toolchain tracks tcgen05.ld destinations until this instruction).
WQ_DEVICE void tmem_load_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

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

// v[0..15] twice into the 32 columns starting at taddr of this thread's lane (sixteen source registers stay resident).
#define WQ_IN4(a, i) "r"(a[i]), "r"(a[i + 1]), "r"(a[i + 2]), "r"(a[i + 3])
WQ_DEVICE void tmem_store_32(uint32_t taddr, const int* v) {
#pragma unroll
    for (int part = 0; part < 2; ++part)
        asm volatile("tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};" ::"r"(taddr + part * 16),
                     WQ_IN4(v, 0), WQ_IN4(v, 4), WQ_IN4(v, 8), WQ_IN4(v, 12)
                     : "memory");
}
#undef WQ_IN4
WQ_DEVICE void tmem_store_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

// Exact INT32 -> FP32 of block sums.  |sum| <= 128 * 127 * 127 < 2^22, so the bits of 1.5 * 2^23 plus the sum are the float
// 1.5 * 2^23 + sum exactly and one subtraction recovers the sum (the conversion instruction issues at a quarter of that rate).
// kFoldBiased: the accumulators in tensor memory START at those bits (the epilogue re-arms every column it drains), so the MMAs
// themselves deliver the biased value and no integer add is needed.  kFoldAdd: the accumulators start at zero and the bits are added here.
constexpr int kBiasBits = 0x4B400000;
#define WQ_B4 kBiasBits, kBiasBits, kBiasBits, kBiasBits
// The re-arming store takes its 16 source registers from here, through volatile loads: values the compiler cannot rebuild with moves in
// front of every store (it would: a move per register and store), so they stay resident for the whole kernel.
__device__ int g_bias_run[16] = {WQ_B4, WQ_B4, WQ_B4, WQ_B4};
#undef WQ_B4
WQ_DEVICE void load_bias_run(int* v) {
#pragma unroll
    for (int j = 0; j < 16; ++j) asm volatile("ld.volatile.global.b32 %0, [%1];" : "=r"(v[j]) : "l"(g_bias_run + j));
}
constexpr float kBiasValue = 12582912.f;
enum Fold : int { kFoldBiased = 0, kFoldAdd = 1 };
template <int FOLD> WQ_DEVICE float block_sum_to_float(int s) {
    if constexpr (FOLD == kFoldAdd) s += kBiasBits;
    return __int_as_float(s) - kBiasValue;
}

template <int MODE, int BN> struct Shape {
    static constexpr bool kHilo = MODE == kExact || MODE == kExactG;
    static constexpr bool kFold = MODE == kBlock || MODE == kBlockG || MODE == kExactG;  // one accumulation per 128 of K
    static constexpr bool kWGroup = MODE == kBlockG || MODE == kExactG;
    static constexpr bool kBlockScales = MODE == kBlock || MODE == kBlockG;              // sa is (M, ceil(K / 128))
    static constexpr int kAccColumns = BN * (kHilo ? 2 : 1);
    static constexpr int kAccBuffers = kTmemColumns / kAccColumns;
    static constexpr int kABytes = kBM * kStageK, kBBytes = BN * kStageK;
    static constexpr int kStageBytes = kABytes * (kHilo ? 2 : 1) + kBBytes;
    static constexpr int kStages = (196 * 1024) / kStageBytes > 6 ? 6 : (196 * 1024) / kStageBytes;
    static constexpr int kEpiColumns = BN / 2;  // columns per epilogue thread (two warpgroups split the tile's columns)
    static constexpr int kRingBytes = kWGroup ? kScaleRing * BN * 4 : 0;
    // Output staging: every epilogue warp owns kStoreBuffers buffers of 32 rows x 32 columns of 16-bit outputs (2 KiB each, 64-byte
    // swizzle) from which the TMA unit writes whole 64-byte row segments; two buffers per warp when shared memory has room for them.
    static constexpr int kStoreTile = 32 * 32 * 2;
    // Column parameters of the tile being finished (weight scale as FP32, bias and residual scale in the output type), shared by the epilogue warps.
    static constexpr int kParamBytes = BN * 8;
    static constexpr int kBarrierBytes = 384;
    static constexpr int kFixedBytes = kStages * kStageBytes + kRingBytes + kParamBytes + kBarrierBytes /* barriers, TMEM slot, abort flag */;
    static constexpr int kStoreBuffers = kFixedBytes + kEpilogueWarps * 2 * kStoreTile <= 227 * 1024 ? 2 : 1;
    static constexpr int kStoreBytes = kEpilogueWarps * kStoreBuffers * kStoreTile;
    static constexpr int kSmemBytes = kFixedBytes + kStoreBytes;
    static_assert(kAccBuffers >= 1 && kStages >= 2, "tile does not fit");
};

struct GemmParams {
    const float* sa;
    const float* sb;
    const void* bias;
    const void* residual;
    const void* rscale;
    void* y;
    int* dump;  // debug: raw block sums (kblocks, M, N)
    int m, n, k;
    int tiles_m, tiles_n;
    int vector_io;  // y, residual, sb, bias and rscale allow 16-byte accesses (N multiple of 8, aligned bases)
    const float* sb_blocks;  // group-scaled weights: the scales regrouped by block, (ceil(K/128), n_pad) with zeros past N
    int n_pad;               // row length of sb_blocks: N rounded up to 256
    int tma_y;      // the output maps describe the destinations: whole 32-column chunks leave through shared memory and the TMA unit
    int wide_store;    // several destinations: the two staging tiles of a warp form one of 32 rows x 64 columns (128-byte rows cross NVLink
                       // in half as many, twice as large writes); the output maps then have 64-column boxes and the 128-byte swizzle
    int destinations;  // copies of the output written by the TMA stores (1, or one per GPU of an N-sharded layer)
    int64_t ld_y, ld_residual;  // row strides in elements of y and of the residual
};

// Up to eight destinations of the output: the same (M, N) block in this GPU's buffer and, for an N-sharded layer, in the buffers of its
// peers (ordinary TMA stores over NVLink; nothing is ever loaded from a peer).
constexpr int kMaxDestinations = 8;
struct OutputMaps { CUtensorMap map[kMaxDestinations]; };

struct TileCoord { int m0, n0; };
// Bands of 16 row tiles are swept over all column tiles, so the CTAs running together share a few A bands and B tiles in L2.
template <int BN> WQ_DEVICE TileCoord tile_origin(int t, int tiles_m, int tiles_n) {
    constexpr int kBand = 16;
    const int width = kBand * tiles_n, first = (t / width) * kBand;
    const int rows = min(tiles_m - first, kBand);
    return {(first + (t % width) % rows) * kBM, ((t % width) / rows) * BN};
}

template <class T, int MODE, int BN, int FOLD, bool DUMP>
__global__ void __launch_bounds__(kThreads, 1)
gemm_i8_tc(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_a_lo, const __grid_constant__ CUtensorMap map_b,
           const __grid_constant__ OutputMaps out_maps, const GemmParams p) {
    using S = Shape<MODE, BN>;
    constexpr int kStages = S::kStages, kAccBuffers = S::kAccBuffers, kEpi = S::kEpiColumns;
    // No static shared memory in this kernel: the dynamic block starts at the CTA's shared window, which is 1024-byte aligned (the
    // 128-byte swizzle of the operand stages needs that); a launch that finds it otherwise reports it and does nothing.
    extern __shared__ __align__(1024) uint8_t smem[];
    if (smem_u32(smem) & 1023u) {
        if (threadIdx.x == 0) atomicCAS(&g_status, 0, int(kStatusSharedAlignment));
        return;
    }
    float* scale_ring = reinterpret_cast<float*>(smem + kStages * S::kStageBytes);
    const uint32_t store_stage = smem_u32(smem + kStages * S::kStageBytes + S::kRingBytes);
    float* store_stage_generic = reinterpret_cast<float*>(smem + kStages * S::kStageBytes + S::kRingBytes);
    uint8_t* params = smem + kStages * S::kStageBytes + S::kRingBytes + S::kStoreBytes;
    float* param_sb = reinterpret_cast<float*>(params);
    T* param_bias = reinterpret_cast<T*>(params + BN * 4);
    T* param_rscale = reinterpret_cast<T*>(params + BN * 6);
    uint64_t* bars = reinterpret_cast<uint64_t*>(params + S::kParamBytes);
    // barrier layout: full[kStages], empty[kStages], acc_full[4], acc_empty[4], ring_full[kScaleRing], ring_empty[kScaleRing], drained[4],
    // params_written, params_consumed; then the TMEM slot and the abort flag
    constexpr int kMaxAcc = 4;
    static_assert(kAccBuffers <= kMaxAcc, "accumulator barriers");
    const uint32_t bar_full = smem_u32(bars), bar_empty = bar_full + 8 * kStages, bar_acc_full = bar_empty + 8 * kStages,
                   bar_acc_empty = bar_acc_full + 8 * kMaxAcc, bar_ring_full = bar_acc_empty + 8 * kMaxAcc,
                   bar_ring_empty = bar_ring_full + 8 * kScaleRing, bar_drained = bar_ring_empty + 8 * kScaleRing,
                   bar_params_written = bar_drained + 8 * kMaxAcc, bar_params_consumed = bar_params_written + 8;
    static_assert(8 * (2 * kStages + 3 * kMaxAcc + 2 * kScaleRing + 2) <= S::kBarrierBytes - 32, "barriers overlap the TMEM slot");
    uint32_t& tmem_slot = *reinterpret_cast<uint32_t*>(reinterpret_cast<uint8_t*>(bars) + S::kBarrierBytes - 32);
    int& abort_word = *reinterpret_cast<int*>(reinterpret_cast<uint8_t*>(bars) + S::kBarrierBytes - 28);
    volatile int* abort_flag = &abort_word;

    constexpr bool kBiased = S::kFold && FOLD == kFoldBiased && !DUMP;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int kblocks = (p.k + kStageK - 1) / kStageK;
    const int tiles = p.tiles_m * p.tiles_n;

    if (threadIdx.x == 0) {
        abort_word = 0;
        for (int s = 0; s < kStages; ++s) {
            mbar_init(bar_full + 8 * s, 1);
            mbar_init(bar_empty + 8 * s, 1);
        }
        for (int s = 0; s < kMaxAcc; ++s) {
            mbar_init(bar_acc_full + 8 * s, 1);
            mbar_init(bar_acc_empty + 8 * s, kBiased ? kRearmWarps : kEpilogueWarps);
            mbar_init(bar_drained + 8 * s, kEpilogueWarps);
        }
        mbar_init(bar_params_written, 32);
        mbar_init(bar_params_consumed, kEpilogueWarps);
        for (int s = 0; s < kScaleRing; ++s) {
            mbar_init(bar_ring_full + 8 * s, 1);
            mbar_init(bar_ring_empty + 8 * s, kEpilogueWarps);
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        prefetch_tensormap(&map_a);
        prefetch_tensormap(&map_b);
        if (S::kHilo) prefetch_tensormap(&map_a_lo);
        if (p.tma_y)
            for (int d = 0; d < p.destinations; ++d) prefetch_tensormap(&out_maps.map[d]);
    }
    if (warp == 2) tmem_alloc(smem_u32(&tmem_slot), kTmemColumns);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = tmem_slot;
    int bias_run[16];
    if constexpr (kBiased) {
        // the re-arm warps put the bias bits into every accumulator column once; from here on they do it after each drain
        if (warp >= 4 + kEpilogueWarps) {
            load_bias_run(bias_run);
            const uint32_t lane_addr = tmem_base + (uint32_t((warp & 3) * 32) << 16);
            for (int column = 0; column < kTmemColumns; column += 32) tmem_store_32(lane_addr + column, bias_run);
            tmem_store_wait();
        }
        tc_fence_before();
        __syncthreads();
        tc_fence_after();
    }

    if (warp < 4) {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(kSmallRegs));
    if (warp == 0) {
        // ---------------- TMA producer ----------------
        if (lane == 0) {
            int stage = 0;
            uint32_t phase = 0;
            bool ok = true;
            for (int t = blockIdx.x; t < tiles && ok; t += gridDim.x) {
                const TileCoord c = tile_origin<BN>(t, p.tiles_m, p.tiles_n);
                for (int kb = 0; kb < kblocks; ++kb) {
                    if (!(ok = mbar_wait(bar_empty + 8 * stage, phase ^ 1u, abort_flag, kTimeoutEmpty))) break;
                    const uint32_t full = bar_full + 8 * stage;
                    const uint32_t dst = smem_u32(smem + stage * S::kStageBytes);
                    mbar_expect_tx(full, S::kStageBytes);
                    tma_load_2d(dst, &map_a, full, kb * kStageK, c.m0);
                    if (S::kHilo) tma_load_2d(dst + S::kABytes, &map_a_lo, full, kb * kStageK, c.m0);
                    tma_load_2d(dst + S::kABytes * (S::kHilo ? 2 : 1), &map_b, full, kb * kStageK, c.n0);
                    if (++stage == kStages) { stage = 0; phase ^= 1u; }
                }
            }
            if (!ok) {
                // aborting: let the copies already issued land before the CTA's shared memory is given back
                for (int s = 0; s < kStages; ++s) {
                    const long long start = clock64();
                    while (!mbar_try_wait(bar_full + 8 * s, 0) && !mbar_try_wait(bar_full + 8 * s, 1) && clock64() - start < 2000000) {}
                }
            }
        }
    } else if (warp == 1) {
        // ---------------- MMA issuer (modes that accumulate over all of K in one buffer) ----------------
        if (!S::kFold && lane == 0) {
            constexpr uint32_t idesc = instruction_descriptor(BN);
            int stage = 0, acc = 0;
            uint32_t phase = 0, acc_phase = 0;
            bool ok = true;
            for (int t = blockIdx.x; t < tiles && ok; t += gridDim.x) {
                for (int kb = 0; kb < kblocks; ++kb) {
                    const bool new_acc = kb == 0;
                    if (new_acc && !(ok = mbar_wait(bar_acc_empty + 8 * acc, acc_phase ^ 1u, abort_flag, kTimeoutTmemEmpty))) break;
                    if (!(ok = mbar_wait(bar_full + 8 * stage, phase, abort_flag, kTimeoutFull))) break;
                    tc_fence_after();
                    const uint32_t a_addr = smem_u32(smem + stage * S::kStageBytes);
                    const uint64_t a_desc = smem_descriptor(a_addr), a_lo_desc = smem_descriptor(a_addr + S::kABytes),
                                   b_desc = smem_descriptor(a_addr + S::kABytes * (S::kHilo ? 2 : 1));
                    const uint32_t d = tmem_base + acc * S::kAccColumns;
#pragma unroll
                    for (int j = 0; j < kStageK / kMmaK; ++j) {
                        const uint32_t accumulate = (new_acc && j == 0) ? 0u : 1u;
                        const uint64_t step = uint64_t(j * kMmaK >> 4);  // start address advances in 16-byte units inside the swizzle row
                        mma_i8(d, a_desc + step, b_desc + step, idesc, accumulate);
                        if (S::kHilo) mma_i8(d + BN, a_lo_desc + step, b_desc + step, idesc, accumulate);
                    }
                    tc_commit(bar_empty + 8 * stage);  // the stage may be refilled once these MMAs have read it
                    if (++stage == kStages) { stage = 0; phase ^= 1u; }
                    if (kb == kblocks - 1) {
                        tc_commit(bar_acc_full + 8 * acc);
                        if (++acc == kAccBuffers) { acc = 0; acc_phase ^= 1u; }
                    }
                }
            }
        }
    }
    if (S::kFold && (warp == 1 || warp == 2)) {
        // ---------------- MMA issuers of the per-block modes: two threads ----------------
        // Block g goes to accumulator buffer g % kAccBuffers (2 buffers of 256 columns, or 4 of 128) and is issued by thread g % 2.  One
        // thread alone spends more time per block on its barrier tests and commits than the four MMAs run; with two, one thread's
        // bookkeeping overlaps the other one's MMAs.
        if (lane == 0) {
            static_assert(!S::kFold || (kStages % 2 == 0 && kAccBuffers % 2 == 0), "two issuers alternate over even numbers of stages and buffers");
            constexpr uint32_t idesc = instruction_descriptor(BN);
            const int me = warp - 1;
            const int total = ((tiles - int(blockIdx.x) + int(gridDim.x) - 1) / int(gridDim.x)) * kblocks;
            int stage = me, acc = me;
            uint32_t phase = 0, acc_phase = 0;
            for (int g = me; g < total; g += 2) {
                const uint32_t d = tmem_base + acc * S::kAccColumns;
                if (!mbar_wait(bar_acc_empty + 8 * acc, acc_phase ^ 1u, abort_flag, kTimeoutTmemEmpty)) break;
                if (!mbar_wait(bar_full + 8 * stage, phase, abort_flag, kTimeoutFull)) break;
                tc_fence_after();
                const uint32_t a_addr = smem_u32(smem + stage * S::kStageBytes);
                const uint64_t a_desc = smem_descriptor(a_addr), a_lo_desc = smem_descriptor(a_addr + S::kABytes),
                               b_desc = smem_descriptor(a_addr + S::kABytes * (S::kHilo ? 2 : 1));
#pragma unroll
                for (int j = 0; j < kStageK / kMmaK; ++j) {
                    const uint32_t accumulate = (!kBiased && j == 0) ? 0u : 1u;
                    const uint64_t step = uint64_t(j * kMmaK >> 4);
                    mma_i8(d, a_desc + step, b_desc + step, idesc, accumulate);
                    if (S::kHilo) mma_i8(d + BN, a_lo_desc + step, b_desc + step, idesc, accumulate);
                }
                tc_commit(bar_empty + 8 * stage);
                tc_commit(bar_acc_full + 8 * acc);
                stage += 2;
                if (stage >= kStages) { stage -= kStages; phase ^= 1u; }
                acc += 2;
                if (acc >= kAccBuffers) { acc -= kAccBuffers; acc_phase ^= 1u; }
            }
        }
    }
    if (warp == 3) {
        // ---------------- column parameters: per tile for the write-out, per block for group-scaled weights ----------------
        // The write-out of a tile needs each column's weight scale, bias and residual scale.  Fetching them there would put a trip to
        // L2 (long, while the operand loads keep it busy) in front of every group of outputs; this warp puts them into shared memory
        // one tile ahead instead: as FP32 weight scale, bias (0 if none) and residual scale (1 if none) in the output type.
        if constexpr (!DUMP) {
            const T* bias = static_cast<const T*>(p.bias);
            const T* rscale = static_cast<const T*>(p.rscale);
            int slot = 0, tile_count = 0;
            uint32_t phase = 0;
            bool ok = true;
            auto stage_params = [&](const TileCoord& c) -> bool {
                if (!p.vector_io) return true;
                // every epilogue warp is done with the previous tile's parameters
                if (tile_count > 0 && !mbar_wait(bar_params_consumed, uint32_t(tile_count - 1) & 1u, abort_flag, kTimeoutParams)) return false;
                for (int i = lane; i < BN; i += 32) {
                    const int col = c.n0 + i;
                    const bool inside = col < p.n;
                    param_sb[i] = !S::kWGroup && inside ? __ldg(p.sb + col) : 0.f;
                    param_bias[i] = bias && inside ? bias[col] : round_one<T>(0.f);
                    param_rscale[i] = rscale && inside ? rscale[col] : round_one<T>(1.f);
                }
                mbar_arrive(bar_params_written);
                ++tile_count;
                return true;
            };
            for (int t = blockIdx.x; t < tiles && ok; t += gridDim.x) {
                const TileCoord c = tile_origin<BN>(t, p.tiles_m, p.tiles_n);
                if constexpr (S::kWGroup) {
                    // the first two blocks' scales go first: the epilogue warps start on them right after the previous tile's write-out
                    const int params_after = (kblocks < 2 ? kblocks : 2) - 1;
                    for (int kb = 0; kb < kblocks && ok; ++kb) {
                        if (!(ok = mbar_wait(bar_ring_empty + 8 * slot, phase ^ 1u, abort_flag, kTimeoutScales))) break;
                        // the tile's BN scales of this block are contiguous in sb_blocks: one bulk copy, up to kScaleRing of them in flight
                        if (lane == 0) {
                            mbar_expect_tx(bar_ring_full + 8 * slot, BN * 4);
                            asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                                             smem_u32(scale_ring + slot * BN)),
                                         "l"(p.sb_blocks + int64_t(kb) * p.n_pad + c.n0), "r"(BN * 4), "r"(bar_ring_full + 8 * slot)
                                         : "memory");
                        }
                        __syncwarp();
                        if (++slot == kScaleRing) { slot = 0; phase ^= 1u; }
                        if (kb == params_after) ok = stage_params(c);
                    }
                } else {
                    ok = stage_params(c);
                }
            }
        }
    }
    } else if (warp >= 4 + kEpilogueWarps) {
        // ---------------- re-arm (accumulators that start at the conversion bias) ----------------
        asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(kSmallRegs));
        if constexpr (kBiased) {
            const uint32_t lane_addr = tmem_base + (uint32_t((warp & 3) * 32) << 16);
            const long long blocks = (long long)((tiles - int(blockIdx.x) + int(gridDim.x) - 1) / int(gridDim.x)) * kblocks;
            int acc = 0;
            uint32_t acc_phase = 0;
            for (long long b = 0; b < blocks; ++b) {
                if (!__all_sync(0xffffffffu, mbar_wait(bar_drained + 8 * acc, acc_phase, abort_flag, kTimeoutTmemEmpty))) break;
                tc_fence_after();
#pragma unroll
                for (int column = 0; column < S::kAccColumns; column += 32) tmem_store_32(lane_addr + acc * S::kAccColumns + column, bias_run);
                tmem_store_wait();
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(bar_acc_empty + 8 * acc);
                if (++acc == kAccBuffers) { acc = 0; acc_phase ^= 1u; }
            }
        }
    } else {
        // ---------------- epilogue ----------------
        asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(kEpilogueRegs));
        const int quarter = warp & 3, half = (warp - 4) >> 2;
        const uint32_t lane_base = uint32_t(quarter * 32) << 16;
        const T* bias = static_cast<const T*>(p.bias);
        const T* residual = static_cast<const T*>(p.residual);
        const T* rscale = static_cast<const T*>(p.rscale);
        T* y = static_cast<T*>(p.y);
        int acc = 0, slot = 0, store_buffer = 0;
        uint32_t acc_phase = 0, ring_phase = 0;
        bool ok = true;
        const uint32_t my_stage = store_stage + (warp - 4) * S::kStoreBuffers * S::kStoreTile;
        int tile_count = 0;  // tiles this CTA has finished: the phase of the parameter hand-over barriers
        float sa_ahead[2] = {0.f, 0.f};
        bool sa_ahead_valid = false;
        for (int t = blockIdx.x; t < tiles && ok; t += gridDim.x) {
            const TileCoord c = tile_origin<BN>(t, p.tiles_m, p.tiles_n);
            const int row = c.m0 + quarter * 32 + lane;
            const bool row_ok = row < p.m;
            const int col0 = c.n0 + half * kEpi;
            const float row_scale = S::kBlockScales ? 1.f : (row_ok ? __ldg(p.sa + row) : 0.f);
            // The tile's column parameters arrive in shared memory from warp 3; false when the CTA aborts.
            auto await_params = [&]() -> bool {
                if (!p.vector_io) return true;
                return __all_sync(0xffffffffu, mbar_wait(bar_params_written, uint32_t(tile_count) & 1u, abort_flag, kTimeoutParams));
            };
            auto params_done = [&]() {
                if (!p.vector_io) return;
                __syncwarp();
                if (lane == 0) mbar_arrive(bar_params_consumed);
                ++tile_count;
            };

            // y values of 32 columns starting at `col`: bias, residual, one rounding, store.  The accumulators of a tile live in registers,
            // so this body is instantiated once per 32 columns of the thread: it is kept short (the tile epilogue runs once per tile and
            // its instructions come from memory each time when the kernel outgrows the instruction cache).
            auto emit = [&](const float* v, int col, int chunk) {
                if (col >= p.n) return;
                T* dst = y + int64_t(row) * p.ld_y + col;
                const T* res = residual && row_ok ? residual + int64_t(row) * p.ld_residual + col : nullptr;
                if (p.vector_io) {
                    // N is a multiple of 8 and every operand 16-byte aligned: eight outputs per step with 128-bit accesses; groups of eight
                    // are whole or absent at the right edge, rows past M are clipped by the TMA store (or skipped by the plain one)
                    const bool staged = p.tma_y != 0;
                    const bool wide = S::kStoreBuffers == 2 && p.wide_store != 0, second = wide && (chunk & 1);
                    const uint32_t stage_tile = wide ? my_stage : my_stage + store_buffer * S::kStoreTile;
                    if (staged && !second) {
                        // the TMA store that last read this buffer must be done with it before the warp writes it again
                        if (lane == 0) {
                            if (wide) asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
                            else asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(S::kStoreBuffers - 1) : "memory");
                        }
                        __syncwarp();
                    }
#pragma unroll
                    for (int j = 0; j < 32; j += 8) {
                        if (col + j >= p.n) break;
                        float scale8[8], bias8[8], out[8];
                        const int ct = col - c.n0 + j;  // column of the tile
                        if constexpr (S::kWGroup) {
#pragma unroll
                            for (int e = 0; e < 8; ++e) scale8[e] = 1.f;
                        } else {
                            const float4 s0 = *reinterpret_cast<const float4*>(param_sb + ct), s1 = *reinterpret_cast<const float4*>(param_sb + ct + 4);
                            scale8[0] = s0.x; scale8[1] = s0.y; scale8[2] = s0.z; scale8[3] = s0.w;
                            scale8[4] = s1.x; scale8[5] = s1.y; scale8[6] = s1.z; scale8[7] = s1.w;
                        }
                        load_eight_plain(param_bias + ct, bias8);
#pragma unroll
                        for (int e = 0; e < 8; ++e) out[e] = fmaf(v[j + e] * row_scale, scale8[e], bias8[e]);
                        if (res) {
                            float res8[8], rs8[8];
                            load_eight_plain(res + j, res8);  // read before this thread overwrites it (y may be the residual)
                            load_eight_plain(param_rscale + ct, rs8);
#pragma unroll
                            for (int e = 0; e < 8; ++e) out[e] = fmaf(out[e], rs8[e], res8[e]);
                        }
                        uint4 packed;
                        packed.x = pack_pair<T>(out[0], out[1]);
                        packed.y = pack_pair<T>(out[2], out[3]);
                        packed.z = pack_pair<T>(out[4], out[5]);
                        packed.w = pack_pair<T>(out[6], out[7]);
                        if (staged) {
                            // row `lane` of the staging tile, 16-byte piece j / 8 at its place in the 64-byte swizzle
                            // (wide: piece 4 (chunk & 1) + j / 8 of a 128-byte row, 128-byte swizzle)
                            const uint32_t piece = wide ? (uint32_t(((chunk & 1) << 2) | (j >> 3)) ^ (uint32_t(lane) & 7u))
                                                        : (uint32_t(j >> 3) ^ ((uint32_t(lane) >> 1) & 3u));
                            asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(stage_tile + lane * (wide ? 128 : 64) + piece * 16), "r"(packed.x),
                                         "r"(packed.y), "r"(packed.z), "r"(packed.w)
                                         : "memory");
                        } else if (row_ok) {
                            *reinterpret_cast<uint4*>(dst + j) = packed;
                        }
                    }
                    // wide: the store leaves with the pair's second chunk, or with the first when the second lies past N
                    if (staged && (!wide || second || col + 32 >= p.n)) {
                        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                        __syncwarp();
                        if (lane == 0) {
                            for (int d = 0; d < p.destinations; ++d)
                                asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%1, %2}], [%3];" ::"l"(&out_maps.map[d]),
                                             "r"(second ? col - 32 : col), "r"(c.m0 + quarter * 32), "r"(stage_tile)
                                             : "memory");
                            asm volatile("cp.async.bulk.commit_group;" ::: "memory");
                        }
                        if (!wide && ++store_buffer == S::kStoreBuffers) store_buffer = 0;
                    }
                    return;
                }
                // Odd N or unaligned operands: one element at a time.  The values go through this thread's 64 bytes of a staging tile
                // (no TMA store is in flight in such a launch), 16 at a time, so that a short loop can index them.
#pragma unroll
                for (int part = 0; part < 32; part += 16) {
                    float* mine = store_stage_generic + ((warp - 4) * S::kStoreBuffers * S::kStoreTile + lane * 64) / 4;
#pragma unroll
                    for (int j = 0; j < 16; ++j) mine[j] = v[part + j];
#pragma unroll 1
                    for (int j = 0; j < 16; ++j) {
                        const int cj = col + part + j;
                        if (row_ok && cj < p.n) {
                            const float col_scale = S::kWGroup ? 1.f : __ldg(p.sb + cj);
                            float value = fmaf(mine[j] * row_scale, col_scale, bias ? as_float(bias[cj]) : 0.f);
                            if (res) value = fmaf(value, rscale ? as_float(rscale[cj]) : 1.f, as_float(res[part + j]));
                            dst[part + j] = round_one<T>(value);
                        }
                    }
                }
            };

            if constexpr (S::kFold) {
                float accf[kEpi];
#pragma unroll
                for (int j = 0; j < kEpi; ++j) accf[j] = 0.f;
                // activation block scales: two blocks ahead in registers
                float sa_now = 0.f, sa_next = 0.f;
                if constexpr (S::kBlockScales && !DUMP) {
                    if (sa_ahead_valid) {  // requested while the previous tile was being written out
                        sa_now = sa_ahead[0];
                        sa_next = sa_ahead[1];
                    } else {
                        const float* sa_row = p.sa + int64_t(row_ok ? row : 0) * kblocks;
                        sa_now = row_ok ? __ldg(sa_row) : 0.f;
                        sa_next = row_ok && kblocks > 1 ? __ldg(sa_row + 1) : 0.f;
                    }
                }
                for (int kb = 0; kb < kblocks; ++kb) {
#ifdef WQ_TRACE
                    const int stamp = (t / int(gridDim.x)) * kblocks + kb;
                    const int tbase = (warp == 4 && lane == 0) ? 4096 : 1 << 30;
#define WQ_ESTAMP(field) do { if (tbase == 4096) WQ_STAMP(4096, stamp, field); } while (0)
#else
#define WQ_ESTAMP(field) do {} while (0)
#endif
                    WQ_ESTAMP(0);
                    float sa_after = 0.f;
                    if constexpr (S::kBlockScales && !DUMP) {
                        if (row_ok && kb + 2 < kblocks) sa_after = __ldg(p.sa + int64_t(row) * kblocks + kb + 2);
                    }
                    if constexpr (S::kWGroup) {
                        if (!(ok = __all_sync(0xffffffffu, mbar_wait(bar_ring_full + 8 * slot, ring_phase, abort_flag, kTimeoutScales)))) break;
                    }
                    if (!(ok = __all_sync(0xffffffffu, mbar_wait(bar_acc_full + 8 * acc, acc_phase, abort_flag, kTimeoutTmemFull)))) break;
                    WQ_ESTAMP(1);
                    tc_fence_after();
                    const uint32_t taddr = tmem_base + lane_base + acc * S::kAccColumns + half * kEpi;
                    const float* ring = scale_ring + slot * BN + half * kEpi;
                    // Two staging buffers of 32 columns.  The buffer in tensor memory is handed back as soon as its last column has been
                    // read (and re-armed), half a drain before the folding ends: the MMAs of the block after next start that much earlier.
                    int hi[2][32], lo[2][32];
                    constexpr int kChunks = kEpi / 32;
                    auto fetch = [&](int chunk) {
                        tmem_load_32(taddr + chunk * 32, hi[chunk & 1]);
                        if (S::kHilo) tmem_load_32(taddr + BN + chunk * 32, lo[chunk & 1]);
                    };
                    auto release = [&]() {
                        // every column of this warp's part of the buffer has been read: it goes back to the MMAs, through the re-arm warps
                        // when the accumulators have to start at the conversion bias again
                        tc_fence_before();
                        __syncwarp();
                        if (lane == 0) mbar_arrive((kBiased ? bar_drained : bar_acc_empty) + 8 * acc);
                    };
                    auto fold = [&](int chunk) {
                        const int* h = hi[chunk & 1];
                        const int* l = lo[chunk & 1];
                        if constexpr (DUMP) {
                            if (row_ok)
#pragma unroll
                                for (int j = 0; j < 32; ++j)
                                    if (col0 + chunk * 32 + j < p.n) p.dump[(int64_t(kb) * p.m + row) * p.n + col0 + chunk * 32 + j] = h[j];
                        } else {
                            // three passes over the chunk, each of 32 independent instructions, converting in place: the dependent
                            // add -> subtract -> multiply-add of one element are never issued back to back
                            float v[32];
#pragma unroll
                            for (int j = 0; j < 32; ++j) v[j] = __int_as_float(FOLD == kFoldAdd ? h[j] + kBiasBits : h[j]);
#pragma unroll
                            for (int j = 0; j < 32; ++j) v[j] -= kBiasValue;
                            if constexpr (MODE == kExactG) {
                                float w[32];
#pragma unroll
                                for (int j = 0; j < 32; ++j) w[j] = __int_as_float(FOLD == kFoldAdd ? l[j] + kBiasBits : l[j]);
#pragma unroll
                                for (int j = 0; j < 32; ++j) w[j] -= kBiasValue;
#pragma unroll
                                for (int j = 0; j < 32; ++j) v[j] = fmaf(w[j], 1.f / 254.f, v[j]);
                            }
#pragma unroll
                            for (int j = 0; j < 32; ++j) {
                                float* a = &accf[chunk * 32 + j];
                                if constexpr (MODE == kBlock) {
                                    *a = fmaf(v[j], sa_now, *a);
                                } else if constexpr (MODE == kBlockG) {
                                    *a = fmaf(v[j], sa_now * ring[chunk * 32 + j], *a);
                                } else {
                                    *a = fmaf(v[j], ring[chunk * 32 + j], *a);
                                }
                            }
                        }
                    };
                    static_assert(kChunks >= 2 && kChunks % 2 == 0, "the drain works on pairs of 32-column chunks");
                    fetch(0);
                    fetch(1);
                    tmem_load_wait();
                    WQ_ESTAMP(2);
                    if (kChunks == 2) release();
#pragma unroll
                    for (int chunk = 0; chunk < kChunks; ++chunk) {
                        fold(chunk);
                        if (chunk + 2 < kChunks) {
                            fetch(chunk + 2);  // into the staging buffer just folded
                            if (chunk & 1) {   // chunks chunk + 1 and chunk + 2 are in flight: complete the pair
                                tmem_load_wait();
                                if (chunk + 2 == kChunks - 1) { WQ_ESTAMP(3); release(); WQ_ESTAMP(4); }
                            }
                        }
                    }
                    if constexpr (S::kWGroup) {
                        __syncwarp();
                        if (lane == 0) mbar_arrive(bar_ring_empty + 8 * slot);
                    }
                    WQ_ESTAMP(5);
                    if (++acc == kAccBuffers) { acc = 0; acc_phase ^= 1u; }
                    if (S::kWGroup && ++slot == kScaleRing) { slot = 0; ring_phase ^= 1u; }
                    sa_now = sa_next;
                    sa_next = sa_after;
                }
                if (!ok) break;
                if constexpr (S::kBlockScales && !DUMP) {
                    // the first two block scales of this thread's row in the next tile: in flight while this tile is written out
                    const int t_next = t + int(gridDim.x);
                    sa_ahead_valid = t_next < tiles;
                    if (sa_ahead_valid) {
                        const int row_next = tile_origin<BN>(t_next, p.tiles_m, p.tiles_n).m0 + quarter * 32 + lane;
                        const float* sa_row = p.sa + int64_t(row_next < p.m ? row_next : 0) * kblocks;
                        sa_ahead[0] = row_next < p.m ? __ldg(sa_row) : 0.f;
                        sa_ahead[1] = row_next < p.m && kblocks > 1 ? __ldg(sa_row + 1) : 0.f;
                    }
                }
#ifdef WQ_TRACE
                if (warp == 4 && lane == 0) WQ_STAMP(4096, (t / int(gridDim.x)) * kblocks + kblocks - 1, 6);
#endif
                if constexpr (!DUMP) {
                    if (!(ok = await_params())) break;
#pragma unroll
                    for (int chunk = 0; chunk < kEpi / 32; ++chunk) emit(&accf[chunk * 32], col0 + chunk * 32, chunk);
                    params_done();
                }
#ifdef WQ_TRACE
                if (warp == 4 && lane == 0) WQ_STAMP(4096, (t / int(gridDim.x)) * kblocks + kblocks - 1, 7);
#endif
            } else {
                if (!(ok = __all_sync(0xffffffffu, mbar_wait(bar_acc_full + 8 * acc, acc_phase, abort_flag, kTimeoutTmemFull)))) break;
                tc_fence_after();
                const uint32_t taddr = tmem_base + lane_base + acc * S::kAccColumns + half * kEpi;
                if (!(ok = await_params())) break;
#pragma unroll 1
                for (int chunk = 0; chunk < kEpi / 32; ++chunk) {
                    int s_hi[32], s_lo[32];
                    tmem_load_32(taddr + chunk * 32, s_hi);
                    if (S::kHilo) tmem_load_32(taddr + BN + chunk * 32, s_lo);
                    tmem_load_wait();
                    float v[32];
#pragma unroll
                    for (int j = 0; j < 32; ++j) {
                        v[j] = float(s_hi[j]);
                        if (S::kHilo) v[j] = fmaf(float(s_lo[j]), 1.f / 254.f, v[j]);
                    }
                    if (chunk == kEpi / 32 - 1) {
                        // all of this warp's columns are in registers: the MMAs of the next tile may overwrite the buffer
                        tc_fence_before();
                        __syncwarp();
                        if (lane == 0) mbar_arrive(bar_acc_empty + 8 * acc);
                    }
                    emit(v, col0 + chunk * 32, chunk);
                }
                params_done();
                if (++acc == kAccBuffers) { acc = 0; acc_phase ^= 1u; }
            }
        }
    }

    // common exit: every role falls through to here, aborting or not
    if (warp >= 4 && warp < 4 + kEpilogueWarps && lane == 0) asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");  // staged outputs
    tc_fence_before();
    __syncthreads();
    if (warp == 2) {
        tc_fence_after();
        tmem_dealloc(tmem_base, kTmemColumns);
    }
}

// Issue-rate probe of the tensor pipe: one CTA per SM issues `iters` groups of four M128 N256 MMAs on resident shared-memory
// operands (no loads, no epilogue), alternating the two accumulator buffers.  KIND 0: kind::i8 (K = 32), 1: kind::f16 with BF16 (K = 16).
template <int KIND>
__global__ void __launch_bounds__(128, 1) mma_peak_probe(int iters, long long* cycles, long long* nanoseconds) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    __shared__ uint32_t tmem_slot;
    __shared__ uint64_t bar;
    __shared__ int abort_word;
    // operands: zeros (the quietest data) or pseudo-random bytes (iters < 0): the tensor pipe's power, and with it the clock, depends on them
    const bool noisy = iters < 0;
    if (noisy) iters = -iters;
    for (int i = threadIdx.x; i < (kBM + 256) * kStageK / 16; i += blockDim.x) {
        uint32_t h = (i * 4 + blockIdx.x * 7919u) * 2654435761u;
        const uint4 v = make_uint4(h, h * 2246822519u, h * 3266489917u, h * 668265263u);
        reinterpret_cast<uint4*>(smem)[i] = noisy ? v : make_uint4(0u, 0u, 0u, 0u);
    }
    if (threadIdx.x == 0) {
        abort_word = 0;
        mbar_init(smem_u32(&bar), 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // the zeroes above are read by the tensor cores
    if (threadIdx.x < 32) tmem_alloc(smem_u32(&tmem_slot), kTmemColumns);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = tmem_slot;
    if (threadIdx.x == 0) {
        // KIND 1: F32 accumulator (1 << 4), BF16 A and B (1 << 7, 1 << 10)
        constexpr uint32_t idesc = KIND == 0 ? instruction_descriptor(256)
                                             : ((1u << 4) | (1u << 7) | (1u << 10) | (uint32_t(256 >> 3) << 17) | (uint32_t(kBM >> 4) << 24));
        const uint64_t a_desc = smem_descriptor(smem_u32(smem)), b_desc = smem_descriptor(smem_u32(smem) + kBM * kStageK);
        long long t0 = clock64(), g0;
        asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(g0));
        for (int i = 0; i < iters; ++i) {
            const uint32_t d = tmem_base + (i & 1) * 256;
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                if (KIND == 0) {
                    mma_i8(d, a_desc + 2 * j, b_desc + 2 * j, idesc, 1u);
                } else {
                    asm volatile(
                        "{\n\t.reg .pred p;\n\t"
                        "setp.ne.b32 p, %4, 0;\n\t"
                        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(d),
                        "l"(a_desc + 2 * j), "l"(b_desc + 2 * j), "r"(idesc), "r"(1u)
                        : "memory");
                }
            }
        }
        tc_commit(smem_u32(&bar));
        mbar_wait(smem_u32(&bar), 0, &abort_word, kTimeoutTmemFull);
        long long t1 = clock64(), g1;
        asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(g1));
        cycles[blockIdx.x] = t1 - t0;
        nanoseconds[blockIdx.x] = g1 - g0;
    }
    tc_fence_before();
    __syncthreads();
    if (threadIdx.x < 32) {
        tc_fence_after();
        tmem_dealloc(tmem_base, kTmemColumns);
    }
}

// ---- host side -------------------------------------------------------------------------------------------------------
using EncodeTiled = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                 const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiled encode_tiled() {
    static EncodeTiled fn = nullptr;
    if (!fn) {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult result;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &result) == cudaSuccess && result == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiled>(p);
    }
    return fn;
}

// (rows, k) row-major INT8 matrix -> tensor map with boxes of `box_rows` rows x 128 bytes, 128-byte swizzle, zero fill outside.
static bool make_map(CUtensorMap* map, const void* base, int rows, int k, int box_rows) {
    EncodeTiled encode = encode_tiled();
    if (!encode) return false;
    const cuuint64_t dims[2] = {cuuint64_t(k), cuuint64_t(rows)};
    const cuuint64_t strides[1] = {cuuint64_t(k)};
    const cuuint32_t box[2] = {cuuint32_t(kStageK), cuuint32_t(box_rows)};
    const cuuint32_t elem[2] = {1, 1};
    return encode(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(base), dims, strides, box, elem, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// (m, n) row-major matrix of 16-bit outputs -> tensor map with boxes of 32 rows x 32 columns, 64-byte swizzle (stores clip at the edges).
// (wide: 32 rows x 64 columns, 128-byte swizzle)
static bool make_output_map(CUtensorMap* map, const void* base, int m, int n, int64_t ld, bool is_bf16, bool wide) {
    EncodeTiled encode = encode_tiled();
    if (!encode) return false;
    const cuuint64_t dims[2] = {cuuint64_t(n), cuuint64_t(m)};
    const cuuint64_t strides[1] = {cuuint64_t(ld) * 2};
    const cuuint32_t box[2] = {wide ? 64u : 32u, 32};
    const cuuint32_t elem[2] = {1, 1};
    return encode(map, is_bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, const_cast<void*>(base), dims, strides, box,
                  elem, CU_TENSOR_MAP_INTERLEAVE_NONE, wide ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_64B, CU_TENSOR_MAP_L2_PROMOTION_NONE,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// Weight scales of group-scaled weights, (N, kblocks) as the caller holds them -> (kblocks, n_pad) with zeros past N, so that the scales
// a tile needs for one block of K are one contiguous run.
__global__ void regroup_weight_scales(const float* __restrict__ sb, float* __restrict__ out, int n, int kblocks, int n_pad) {
    const int64_t total = int64_t(kblocks) * n_pad;
    for (int64_t i = int64_t(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += int64_t(gridDim.x) * blockDim.x) {
        const int kb = int(i / n_pad), col = int(i % n_pad);
        out[i] = col < n ? __ldg(sb + int64_t(col) * kblocks + kb) : 0.f;
    }
}

constexpr int kScalePad = 256;
static int padded_n(int n) { return (n + kScalePad - 1) / kScalePad * kScalePad; }

bool make_byte_matrix_map(CUtensorMap* map, const void* base, int rows, int row_bytes, int box_bytes, int box_rows) {
    EncodeTiled encode = encode_tiled();
    if (!encode) return false;
    const cuuint64_t dims[2] = {cuuint64_t(row_bytes), cuuint64_t(rows)};
    const cuuint64_t strides[1] = {cuuint64_t(row_bytes)};
    const cuuint32_t box[2] = {cuuint32_t(box_bytes), cuuint32_t(box_rows)};
    const cuuint32_t elem[2] = {1, 1};
    return encode(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(base), dims, strides, box, elem, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

struct GemmArgs {
    float* scale_scratch;  // group-scaled weights: (ceil(K/128), padded_n(N)) floats of caller workspace
    const int8_t* a;
    const int8_t* a_lo;
    const float* sa;
    const int8_t* b;
    const float* sb;
    const void* bias;
    const void* residual;
    const void* rscale;
    void* y;
    int* dump;
    int m, n, k, sms;
    void* const* ys = nullptr;  // `count` destinations of the output (host array of device pointers); y when null
    int count = 1;
    int64_t ld_y = 0, ld_residual = 0;  // 0: contiguous (N)
};

template <class T, int MODE, int BN, int FOLD, bool DUMP>
static int launch(const GemmArgs& g, cudaStream_t stream) {
    using S = Shape<MODE, BN>;
    auto kernel = gemm_i8_tc<T, MODE, BN, FOLD, DUMP>;
    static bool configured[64] = {};  // the attribute belongs to a device's copy of the kernel
    int device = 0;
    cudaGetDevice(&device);
    if (device < 0 || device >= 64 || !configured[device]) {
        const cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, S::kSmemBytes);
        if (e != cudaSuccess) return int(e);
        if (device >= 0 && device < 64) configured[device] = true;
    }
    if ((reinterpret_cast<uintptr_t>(g.a) & 15) || (reinterpret_cast<uintptr_t>(g.b) & 15) || (g.a_lo && (reinterpret_cast<uintptr_t>(g.a_lo) & 15)))
        return -2;
    CUtensorMap map_a, map_a_lo, map_b;
    OutputMaps out_maps;
    if (!make_map(&map_a, g.a, g.m, g.k, kBM) || !make_map(&map_b, g.b, g.n, g.k, BN)) return int(cudaErrorNotSupported);
    if (S::kHilo) {
        if (!make_map(&map_a_lo, g.a_lo, g.m, g.k, kBM)) return int(cudaErrorNotSupported);
    } else {
        map_a_lo = map_a;
    }
    GemmParams p{};
    p.sa = g.sa; p.sb = g.sb; p.bias = g.bias; p.residual = g.residual; p.rscale = g.rscale; p.dump = g.dump;
    p.y = g.ys ? g.ys[0] : g.y;
    p.ld_y = g.ld_y ? g.ld_y : g.n;
    p.ld_residual = g.ld_residual ? g.ld_residual : g.n;
    p.destinations = g.ys ? g.count : 1;
    if (p.destinations < 1 || p.destinations > kMaxDestinations) return -2;
    p.m = g.m; p.n = g.n; p.k = g.k;
    p.tiles_m = (g.m + kBM - 1) / kBM;
    p.tiles_n = (g.n + BN - 1) / BN;
    uintptr_t bases = reinterpret_cast<uintptr_t>(p.y) | reinterpret_cast<uintptr_t>(g.residual) | reinterpret_cast<uintptr_t>(g.bias) |
                            reinterpret_cast<uintptr_t>(g.rscale) | (S::kWGroup ? 0 : reinterpret_cast<uintptr_t>(g.sb));
    if (S::kWGroup) {
        if (!g.scale_scratch || (reinterpret_cast<uintptr_t>(g.scale_scratch) & 15)) return -2;
        const int kblocks = (g.k + kStageK - 1) / kStageK;
        p.n_pad = padded_n(g.n);
        p.sb_blocks = g.scale_scratch;
        const int64_t total = int64_t(kblocks) * p.n_pad;
        regroup_weight_scales<<<int((total + 255) / 256 < 1184 ? (total + 255) / 256 : 1184), 256, 0, stream>>>(g.sb, g.scale_scratch, g.n, kblocks, p.n_pad);
    }
    for (int d = 1; d < p.destinations; ++d) bases |= reinterpret_cast<uintptr_t>(g.ys[d]);
    p.vector_io = g.n % 8 == 0 && p.ld_y % 8 == 0 && p.ld_residual % 8 == 0 && (bases & 15) == 0;
    p.tma_y = !DUMP && p.vector_io;
    p.wide_store = S::kStoreBuffers == 2 && p.destinations > 1;
    for (int d = 0; d < kMaxDestinations; ++d) {
        if (p.tma_y && d < p.destinations)
            p.tma_y = make_output_map(&out_maps.map[d], d == 0 ? p.y : g.ys[d], g.m, g.n, p.ld_y, std::is_same<T, bf16>::value, p.wide_store != 0);
        else
            out_maps.map[d] = map_a;
    }
    if (p.destinations > 1 && !p.tma_y) return -2;  // several destinations are only written by the TMA stores
    const int64_t tiles = int64_t(p.tiles_m) * p.tiles_n;
    const int sms = g.sms > 0 ? g.sms : 148;
    const int grid = int(tiles < sms ? tiles : sms);
    kernel<<<grid, kThreads, S::kSmemBytes, stream>>>(map_a, map_a_lo, map_b, out_maps, p);
    return int(cudaGetLastError());
}

template <class T> static int dispatch(const GemmArgs& g, int variant, cudaStream_t stream) {
    switch (variant) {
        case 0: case 2: case 6: return launch<T, kRow, 256, kFoldAdd, false>(g, stream);
        case 1: case 7: return launch<T, kExact, 256, kFoldAdd, false>(g, stream);
        case 10: return launch<T, kBlock, 256, kFoldBiased, false>(g, stream);
        case 11: return launch<T, kBlock, 256, kFoldAdd, false>(g, stream);
        case 12: return launch<T, kBlockG, 256, kFoldBiased, false>(g, stream);
        case 13: return launch<T, kBlockG, 256, kFoldAdd, false>(g, stream);
        case 14: return launch<T, kExactG, 128, kFoldBiased, false>(g, stream);
        case 15: return launch<T, kBlock, 128, kFoldBiased, false>(g, stream);  // tiles of 128 columns: four accumulator buffers
        case 16: return launch<T, kBlock, 128, kFoldAdd, false>(g, stream);
    }
    return -3;
}

}  // namespace wq

using namespace wq;

WQ_API int wq8_gemm(const int8_t* a, const int8_t* a_lo, const float* sa, const int8_t* b, const float* sb, const void* bias, const void* residual,
                    const void* rscale, void* y, int m, int n, int k, int dtype, int variant, int sms, int /*split*/, int* workspace,
                    int* /*counters*/, cudaStream_t stream) {
    if (m <= 0 || n <= 0) return 0;
    if ((variant == 1 || variant == 7 || variant == 14) != (a_lo != nullptr)) return -2;
    if (k <= 0 || k % 16) return -2;
    const GemmArgs g{reinterpret_cast<float*>(workspace), a, a_lo, sa, b, sb, bias, residual, rscale, y, nullptr, m, n, k, sms};
    if (dtype == 0) return dispatch<__half>(g, variant, stream);
    if (dtype == 1) return dispatch<bf16>(g, variant, stream);
    return -1;
}

// wq8_gemm whose output goes to `count` destinations at once (ys: host array of device pointers to the first element of an (M, N)
// block with row stride ld_y; the residual has row stride ld_residual): the rank of an N-sharded layer writes its output columns
// straight into the full-width buffers of all ranks.  Destinations in a peer GPU's memory are written by TMA stores over NVLink.
WQ_API int wq8_gemm_multi(const int8_t* a, const int8_t* a_lo, const float* sa, const int8_t* b, const float* sb, const void* bias,
                          const void* residual, int64_t ld_residual, const void* rscale, void* const* ys, int count, int64_t ld_y, int m, int n,
                          int k, int dtype, int variant, int sms, int* workspace, cudaStream_t stream) {
    if (m <= 0 || n <= 0) return 0;
    if (!ys || count < 1 || count > kMaxDestinations || ld_y < n || (residual && ld_residual < n)) return -2;
    for (int d = 0; d < count; ++d)
        if (!ys[d]) return -2;
    if ((variant == 1 || variant == 7 || variant == 14) != (a_lo != nullptr)) return -2;
    if (k <= 0 || k % 16) return -2;
    GemmArgs g{reinterpret_cast<float*>(workspace), a, a_lo, sa, b, sb, bias, residual, rscale, ys[0], nullptr, m, n, k, sms};
    g.ys = ys;
    g.count = count;
    g.ld_y = ld_y;
    g.ld_residual = residual ? ld_residual : 0;
    if (dtype == 0) return dispatch<__half>(g, variant, stream);
    if (dtype == 1) return dispatch<bf16>(g, variant, stream);
    return -1;
}

// Whole tiles only: no partial sums, no counters.  The variants with group-scaled weights regroup the weight scales by block of K
// into the workspace.
WQ_API void wq8_gemm_workspace(int, int n, int k, int variant, int, int, int64_t* sizes) {
    sizes[0] = sizes[1] = 0;
    if (variant >= 12 && variant <= 14 && n > 0 && k > 0) sizes[0] = int64_t((k + kStageK - 1) / kStageK) * padded_n(n) * 4;
}

WQ_API int wq8_gemm_select(int, int, int, int hilo, int) { return hilo ? 1 : 0; }

// One launch per weight: the quantized input stays in L2 between them (a band of 2048 rows of codes is 10 MB), the values are those of
// wq8_gemm on each weight.  Per-channel weight scales only, as in the reference.
WQ_API int wq8_gemm_segments(const int8_t* a, const int8_t* a_lo, const float* sa, const int8_t* const* bs, const float* const* sbs,
                             const void* const* biases, void* const* ys, int count, int rows, int m, int k, int dtype, int variant, int sms, int split,
                             int* workspace, int* counters, cudaStream_t stream) {
    if (count < 1 || count > 4 || rows <= 0 || rows % 8 || !bs || !sbs || !ys) return -4;
    if (variant >= 12 && variant <= 14) return -4;
    for (int s = 0; s < count; ++s)
        if (!bs[s] || !sbs[s] || !ys[s]) return -4;
    for (int s = 0; s < count; ++s) {
        const int code = wq8_gemm(a, a_lo, sa, bs[s], sbs[s], biases ? biases[s] : nullptr, nullptr, nullptr, ys[s], m, rows, k, dtype, variant, sms, split,
                                  workspace, counters, stream);
        if (code) return code;
    }
    return 0;
}

WQ_API int wq8_debug_block_sums(const int8_t* a, const int8_t* b, int32_t* sums, int m, int n, int k, int sms, cudaStream_t stream) {
    if (m <= 0 || n <= 0) return 0;
    if (k <= 0 || k % 16) return -2;
    const GemmArgs g{nullptr, a, nullptr, nullptr, b, nullptr, nullptr, nullptr, nullptr, nullptr, sums, m, n, k, sms};
    return launch<bf16, kBlock, 256, kFoldAdd, true>(g, stream);
}

// results[0] = tera-operations per second of the whole GPU, results[1] = SM clock in MHz during the probe, results[2] = clocks per MMA group.
WQ_API int wq8_debug_mma_peak(int kind, int iters, int sms, double* results) {
    if (iters == 0 || sms <= 0 || sms > 1024 || (kind != 0 && kind != 1)) return -2;
    long long* buffers = nullptr;
    if (cudaMalloc(&buffers, sizeof(long long) * 2 * sms) != cudaSuccess) return int(cudaGetLastError());
    const int smem_bytes = (kBM + 256) * kStageK + 1024;
    auto kernel = kind == 0 ? mma_peak_probe<0> : mma_peak_probe<1>;
    cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes);
    for (int round = 0; round < 2; ++round) kernel<<<sms, 128, smem_bytes>>>(iters, buffers, buffers + sms);
    int code = int(cudaDeviceSynchronize());
    long long host[2048];
    if (!code) code = int(cudaMemcpy(host, buffers, sizeof(long long) * 2 * sms, cudaMemcpyDeviceToHost));
    cudaFree(buffers);
    if (code) return code;
    double cycles = 0, ns = 0;
    for (int i = 0; i < sms; ++i) { cycles += double(host[i]); ns += double(host[sms + i]); }
    cycles /= sms; ns /= sms;
    const double ops = 2.0 * kBM * 256 * (kind == 0 ? 32 : 16) * 4.0 * (iters < 0 ? -iters : iters) * sms;
    results[0] = ops / (ns * 1e-9) / 1e12;
    results[1] = cycles / ns * 1e3;
    results[2] = cycles / (iters < 0 ? -iters : iters);
    return 0;
}

#ifdef WQ_TRACE
WQ_API int wq8_debug_trace(long long* host_out) {
    if (cudaDeviceSynchronize() != cudaSuccess) return -1;
    return int(cudaMemcpyFromSymbol(host_out, g_trace, sizeof(long long) * 8192));
}
#endif

WQ_API int wq8_debug_status() {
    int code = 0;
    if (cudaDeviceSynchronize() != cudaSuccess) return -1;
    if (cudaMemcpyFromSymbol(&code, g_status, sizeof(int)) != cudaSuccess) return -1;
    const int zero = 0;
    cudaMemcpyToSymbol(g_status, &zero, sizeof(int));
    const int streaming = wq::stream_status_take();  // the weight-streaming kernels keep their own word
    if (streaming < 0) return -1;
    return code ? code : streaming ? 100 + streaming : 0;
}
