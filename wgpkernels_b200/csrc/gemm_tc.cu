// INT8 x INT8 -> INT32 GEMM on the 5th-generation tensor cores of sm_100a (tcgen05.mma kind::i8, accumulators in tensor memory),
// operands staged by TMA (no cluster multicast: every CTA loads its own tiles from its GPU's own memory), warp-specialised:
//
//   warp 0      TMA producer: A (and A_lo) 128 x 128-byte tiles, B BN x 128-byte tiles, 128-byte swizzle, ring of kStages buffers
//   warps 1-2   MMA issue (one elected thread each): 4 (x2 with a low part) tcgen05.mma of K = 32 per stage; warp 2 owns tensor memory
//   warp 3      column parameters of the tile being finished (and the per-block weight scales of group-scaled weights) into shared memory
//   warps 4-19  drain: 16 warps, warp w reads tensor-memory lanes 32 (w % 4) .. + 32 and a quarter of the tile's columns: tcgen05.ld of the
//               INT32 sums, conversion and promotion to FP32 (two-wide FP32 FMAs), bias / residual, one rounding, TMA stores
//
// Modes (the arithmetic of wgpkernels/int8/int8_gemm.cu:773-805 and :836-863 of WGPKernels):
//   row      INT32 sums over all K; y = fmaf(float(S) * sa[m], sb[n], bias)
//   exact    hi and lo operands share B; v = fmaf(float(S_lo), 1/254, float(S_hi)); y = fmaf(v * sa[m], sb[n], bias)
//   block    per 128 of K: acc = fmaf(float(S_b), sa[m, b], acc); y = fmaf(acc, sb[n], bias)
//   block+g  acc = fmaf(float(S_b), sa[m, b] * sb[n, b], acc); y = acc + bias
//   exact+g  acc = fmaf(fmaf(float(S_lo_b), 1/254, float(S_hi_b)), sb[n, b], acc); y = fmaf(acc * sa[m], 1, bias)
// then y = fmaf(y, rscale[n], residual[m, n]) and one rounding.  In the per-block modes the tensor cores produce one exact INT32 block
// sum per output and 128 of K into a multi-buffered tensor-memory accumulator; the drain warps empty a buffer while the MMAs of the
// next block fill another one, and keep the FP32 accumulators in registers for the whole tile (64 per thread).
//
// Every wait is bounded: a wait that gives up records a code in a device status word, raises a CTA-wide abort flag and the CTA leaves
// through the common exit (tensor memory is always released).
#include <cuda.h>  // CUtensorMap and its enums only; cuTensorMapEncodeTiled is resolved through the runtime, libcuda is not linked

#include "tc_ptx.cuh"

namespace wq {

enum Mode : int { kRow = 0, kExact = 1, kBlock = 2, kBlockG = 3, kExactG = 4 };

constexpr int kControlWarps = 4;
// Drain warps: PARTS per lane quarter of tensor memory, each with 1 / PARTS of the tile's columns.  Registers per thread after the split
// (setmaxnreg): the control warps keep few, the drain warps, which hold a tile's FP32 accumulators, take the rest.
//   PARTS = 2:  384 threads launched with 168 registers; control 40, drain 216 (128 accumulators + 2 x 32 staging): 128 x 40 + 256 x 216
//   PARTS = 4:  640 threads launched with 96 registers;  control 32, drain 112 (64 accumulators + 2 x 16 staging):  128 x 32 + 512 x 112
template <int PARTS> struct Roles {
    static_assert(PARTS == 2 || PARTS == 4, "two or four drain warps per lane quarter");
    static constexpr int kDrainWarps = 4 * PARTS;
    static constexpr int kThreads = 32 * (kControlWarps + kDrainWarps);
    static constexpr int kControlRegs = PARTS == 2 ? 40 : 32, kDrainRegs = PARTS == 2 ? 216 : 112;
    static constexpr int kChunk = PARTS == 2 ? 32 : 16;  // columns a drain thread brings in from tensor memory at once
};
constexpr int kScaleRing = 4;        // blocks of gathered weight scales in flight
constexpr int kMaxSegments = 4;      // weights of one launch that share the input (wq8_gemm_segments)
constexpr long long kWaitLimit = 4000000000ll;  // clocks (about two seconds) before a wait gives up

__device__ int g_status = 0;  // first code of a wait that gave up (wq::Status)

WQ_DEVICE bool wait_on(uint32_t bar, uint32_t parity, volatile int* abort_flag, int code) {
    return mbar_wait(bar, parity, abort_flag, code, &g_status, kWaitLimit);
}

// INT32 -> FP32 of the block sums: the conversion instruction (exact: |sum| <= 128 * 127 * 127 < 2^24).  It runs on a pipe of its own,
// beside the FP32 pipe that does the multiply-adds, and needs no preparation of the accumulators: the first MMA of a block overwrites
// its tensor-memory buffer, so a drain warp hands a buffer back as soon as it has read its columns.  (Accumulators that start at
// the bits of 1.5 * 2^23, so that one FP32 subtraction converts, cost more than they save: re-arming a buffer from registers takes a
// register move per column, on the FP32 pipe.)
template <int MODE, int BN, bool WIDE, int PARTS> struct Shape {
    static constexpr int kDrainWarps = Roles<PARTS>::kDrainWarps;
    static constexpr bool kHilo = MODE == kExact || MODE == kExactG;
    static constexpr bool kFold = MODE == kBlock || MODE == kBlockG || MODE == kExactG;  // one accumulation per 128 of K
    static constexpr bool kWGroup = MODE == kBlockG || MODE == kExactG;
    static constexpr bool kBlockScales = MODE == kBlock || MODE == kBlockG;              // sa is (M, ceil(K / 128))
    static constexpr int kAccColumns = BN * (kHilo ? 2 : 1);
    static constexpr int kAccBuffers = kTmemColumns / kAccColumns;
    static constexpr int kABytes = kBM * kStageK, kBBytes = BN * kStageK;
    static constexpr int kStageBytes = kABytes * (kHilo ? 2 : 1) + kBBytes;
    static constexpr int kEpiColumns = BN / PARTS;  // columns per drain thread (PARTS warps split the tile's columns)
    static constexpr int kRingBytes = kWGroup ? kScaleRing * BN * 4 : 0;
    // Output staging: every drain warp owns one buffer of 32 rows x 32 columns of 16-bit outputs (2 KiB, 64-byte swizzle) from which the
    // TMA unit writes whole 64-byte row segments.  kWide (several destinations): 32 rows x 64 columns (4 KiB, 128-byte swizzle), so that
    // rows of 128 bytes cross NVLink; one operand stage less fits then.
    static constexpr bool kWide = WIDE && kEpiColumns >= 64;
    static constexpr int kStoreTile = kWide ? 32 * 64 * 2 : 32 * 32 * 2;
    static constexpr int kStoreBytes = kDrainWarps * kStoreTile;
    // Column parameters of the tile being finished (weight scale and bias as FP32, residual scale in the output type), shared by the drain warps.
    static constexpr int kParamBytes = BN * 10;
    static constexpr int kBarrierBytes = 384;
    static constexpr int kRoom = 227 * 1024 - kStoreBytes - kRingBytes - kParamBytes - kBarrierBytes;
    // The per-block modes are bound by their drain warps, not by the operand feed: three stages serve them better than four (measured:
    // +1.5 % with K = 5120, +5 % with K = 3072; two stages lose 8 %), `row` wants all it can get (four: 2910 TOPS, three: 2710).
    static constexpr int kStageLimit = kFold && BN == 256 ? 3 : 6;  // the 128-channel tiles (smaller stages) keep theirs
    static constexpr int kStagesThatFit = kRoom / kStageBytes > kStageLimit ? kStageLimit : kRoom / kStageBytes;
    // with more than two accumulator buffers the per-block modes take an even number of stages (see the assertion below)
    static constexpr int kStages = kFold && kAccBuffers > 2 ? kStagesThatFit / 2 * 2 : kStagesThatFit;
    static constexpr int kSmemBytes = kStages * kStageBytes + kRingBytes + kStoreBytes + kParamBytes + kBarrierBytes;
    static_assert(kAccBuffers >= 1 && kStages >= 2, "tile does not fit");
    // Per-block modes have two MMA issuers taking the blocks in turn.  With an even number of stages a stage always meets the same
    // issuer.  With an odd one its consecutive fills are awaited by different threads, and a thread that asks for a fill before the one
    // before it has even landed would take the barrier's parity test (one phase bit) for passed.  A thread gets its accumulator buffer
    // back only after the drain has consumed the block kAccBuffers before -- whose operands, and those of every earlier block, had to
    // land first -- at a tile boundary up to 2 kAccBuffers - 1 before, since every tile starts at buffer 0 --, so the fill kStages
    // blocks back has certainly landed when kStages >= 2 kAccBuffers - 1: three stages with two buffers.  (Three stages with the four
    // buffers of the 128-channel tiles did produce a few wrong sums when loads landed out of order under NVLink traffic.)
    static_assert(!kFold || kStages % 2 == 0 || kStages >= 2 * kAccBuffers - 1, "an odd number of stages needs that many to be safe with two issuers");
    static_assert(kEpiColumns % 32 == 0, "a drain thread works on chunks of 16 or 32 and writes out chunks of 32 columns");
};

// Row window of a launch made by one of the *_at entry points: the counter lives on the GPU and is read when the kernel runs (a CUDA
// graph replays the launch while a loop counter advances).  shift = first + counter[0] * step rows of y and of the residual;
// in_first / in_step the same for A, A_lo and their scales; span > 0: rscale holds scale_step values per span of output rows.
struct RowWindow { const long long* counter; long long first, step, span, scale_step, in_first, in_step; };

struct GemmParams {
    const float* sa;
    const float* sb[kMaxSegments];
    const void* bias[kMaxSegments];
    void* y[kMaxSegments];
    const void* residual;
    const void* rscale;
    int* dump;  // debug: raw block sums (kblocks, M, N)
    int m, n, k;    // n: output channels of one segment
    int tiles_m, tiles_n, seg_tiles;  // tiles_n = segments * seg_tiles: a column tile never straddles two segments
    int vector_io;  // y, residual, sb, bias and rscale allow 16-byte accesses (N multiple of 8, aligned bases)
    const float* sb_blocks;  // group-scaled weights: the scales regrouped by block, (ceil(K/128), n_pad) with zeros past N
    int n_pad;               // row length of sb_blocks: N rounded up to 256
    int tma_y;      // the output maps describe the destinations: whole 32-column chunks leave through shared memory and the TMA unit
    int destinations;  // copies of the output written by the TMA stores (1, or one per GPU of an N-sharded layer)
    int tail_rows;     // row window: rows of the last, partial row tile (its A tile is fetched through the *_tail maps), 0 = none
    int64_t ld_y, ld_residual;  // row strides in elements of y and of the residual
    RowWindow window;
};

// Up to eight destinations of the output: the same (M, N) block in this GPU's buffer and, for an N-sharded layer, in the buffers of its
// peers (ordinary TMA stores over NVLink; nothing is ever loaded from a peer).  With segments: map s = the output of weight s.
constexpr int kMaxDestinations = 8;
struct OutputMaps { CUtensorMap map[kMaxDestinations]; };
struct InputMaps { CUtensorMap a, a_lo, a_tail, a_lo_tail; };
struct WeightMaps { CUtensorMap map[kMaxSegments]; };

struct TileCoord { int m0, n0, segment; };
// Bands of 16 row tiles are swept over all column tiles, so the CTAs running together share a few A bands and B tiles in L2.
// Every role computes this once per tile, between two tiles' work: the one general division goes through a reciprocal (exact for the
// tile counts of any launch, far below 2^24), full bands split by shifts, a single weight has segment 0.
template <int BN> WQ_DEVICE TileCoord tile_origin(int t, int tiles_m, int tiles_n, int seg_tiles) {
    constexpr int kBand = 16;
    const int width = kBand * tiles_n;
    int band = __float2int_rz(__int2float_rn(t) * __frcp_rn(__int2float_rn(width)));
    int within = t - band * width;
    if (within < 0) { --band; within += width; }
    if (within >= width) { ++band; within -= width; }
    const int first = band * kBand;
    const int rows = min(tiles_m - first, kBand);
    int column_tile, row_tile;
    if (rows == kBand) {
        column_tile = within >> 4;
        row_tile = within & (kBand - 1);
    } else {
        column_tile = within / rows;
        row_tile = within - column_tile * rows;
    }
    const int segment = column_tile < seg_tiles ? 0 : column_tile / seg_tiles;
    return {(first + row_tile) * kBM, (column_tile - segment * seg_tiles) * BN, segment};
}

WQ_DEVICE float2 as_pair(int a, int b) { return make_float2(__int_as_float(a), __int_as_float(b)); }

template <class T, int MODE, int BN, bool WIDE, bool DUMP, int PARTS>
__global__ void __launch_bounds__(Roles<PARTS>::kThreads, 1)
gemm_i8_tc(const __grid_constant__ InputMaps in_maps, const __grid_constant__ WeightMaps w_maps, const __grid_constant__ OutputMaps out_maps,
           const GemmParams p) {
    using S = Shape<MODE, BN, WIDE, PARTS>;
    constexpr int kStages = S::kStages, kAccBuffers = S::kAccBuffers, kEpi = S::kEpiColumns;
    constexpr int kDrainWarps = Roles<PARTS>::kDrainWarps, kControlRegs = Roles<PARTS>::kControlRegs, kDrainRegs = Roles<PARTS>::kDrainRegs;
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
    float* param_bias = reinterpret_cast<float*>(params + BN * 4);
    T* param_rscale = reinterpret_cast<T*>(params + BN * 8);
    uint64_t* bars = reinterpret_cast<uint64_t*>(params + S::kParamBytes);
    // barrier layout: full[6], empty[6], acc_full[4], acc_empty[4], ring_full[kScaleRing], ring_empty[kScaleRing], params_written,
    // params_consumed; then the TMEM slot and the abort flag
    constexpr int kMaxStages = 6, kMaxAcc = 4;
    static_assert(kAccBuffers <= kMaxAcc && kStages <= kMaxStages, "barrier table");
    const uint32_t bar_full = smem_u32(bars), bar_empty = bar_full + 8 * kMaxStages, bar_acc_full = bar_empty + 8 * kMaxStages,
                   bar_acc_empty = bar_acc_full + 8 * kMaxAcc, bar_ring_full = bar_acc_empty + 8 * kMaxAcc,
                   bar_ring_empty = bar_ring_full + 8 * kScaleRing, bar_params_written = bar_ring_empty + 8 * kScaleRing,
                   bar_params_consumed = bar_params_written + 8;
    static_assert(8 * (2 * kMaxStages + 2 * kMaxAcc + 2 * kScaleRing + 2) <= S::kBarrierBytes - 32, "barriers overlap the TMEM slot");
    uint32_t& tmem_slot = *reinterpret_cast<uint32_t*>(reinterpret_cast<uint8_t*>(bars) + S::kBarrierBytes - 32);
    int& abort_word = *reinterpret_cast<int*>(reinterpret_cast<uint8_t*>(bars) + S::kBarrierBytes - 28);
    volatile int* abort_flag = &abort_word;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int kblocks = (p.k + kStageK - 1) / kStageK;
    const int tiles = p.tiles_m * p.tiles_n;
    // row window of the *_at entry points: where the outputs go and where the inputs come from
    long long out_shift = 0, in_shift = 0;
    if (p.window.counter) {
        const long long count = __ldg(p.window.counter);
        out_shift = p.window.first + count * p.window.step;
        if (p.window.in_first || p.window.in_step) in_shift = p.window.in_first + count * p.window.in_step;
    }

    if (threadIdx.x == 0) {
        abort_word = 0;
        for (int s = 0; s < kMaxStages; ++s) {
            mbar_init(bar_full + 8 * s, 1);
            mbar_init(bar_empty + 8 * s, 1);
        }
        for (int s = 0; s < kMaxAcc; ++s) {
            mbar_init(bar_acc_full + 8 * s, 1);
            mbar_init(bar_acc_empty + 8 * s, kDrainWarps);
        }
        mbar_init(bar_params_written, 32);
        mbar_init(bar_params_consumed, kDrainWarps);
        for (int s = 0; s < kScaleRing; ++s) {
            mbar_init(bar_ring_full + 8 * s, 1);
            mbar_init(bar_ring_empty + 8 * s, kDrainWarps);
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        prefetch_tensormap(&in_maps.a);
        prefetch_tensormap(&w_maps.map[0]);
        if (S::kHilo) prefetch_tensormap(&in_maps.a_lo);
        if (p.tma_y) prefetch_tensormap(&out_maps.map[0]);
    }
    if (warp == 2) tmem_alloc(smem_u32(&tmem_slot), kTmemColumns);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = tmem_slot;

    if (warp < kControlWarps) {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(kControlRegs));
    if (warp == 0) {
        // ---------------- TMA producer ----------------
        if (lane == 0) {
            int stage = 0;
            uint32_t phase = 0;
            bool ok = true;
            for (int t = blockIdx.x; t < tiles && ok; t += gridDim.x) {
                const TileCoord c = tile_origin<BN>(t, p.tiles_m, p.tiles_n, p.seg_tiles);
                // a row window addresses A through maps without a row bound: its last, partial row tile is fetched with a box of just
                // the rows that exist (the other rows of the stage keep stale bytes; their outputs are never stored)
                const bool tail = p.tail_rows && c.m0 + kBM > p.m;
                const CUtensorMap* map_a = tail ? &in_maps.a_tail : &in_maps.a;
                const CUtensorMap* map_a_lo = tail ? &in_maps.a_lo_tail : &in_maps.a_lo;
                const uint32_t bytes = tail ? uint32_t(p.tail_rows * kStageK * (S::kHilo ? 2 : 1) + S::kBBytes) : uint32_t(S::kStageBytes);
                const int a_row = int(in_shift) + c.m0;
                for (int kb = 0; kb < kblocks; ++kb) {
                    if (!(ok = wait_on(bar_empty + 8 * stage, phase ^ 1u, abort_flag, kTimeoutEmpty))) break;
                    const uint32_t full = bar_full + 8 * stage;
                    const uint32_t dst = smem_u32(smem + stage * S::kStageBytes);
                    mbar_expect_tx(full, bytes);
                    tma_load_2d(dst, map_a, full, kb * kStageK, a_row);
                    if (S::kHilo) tma_load_2d(dst + S::kABytes, map_a_lo, full, kb * kStageK, a_row);
                    tma_load_2d(dst + S::kABytes * (S::kHilo ? 2 : 1), &w_maps.map[c.segment], full, kb * kStageK, c.n0);
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
                    if (new_acc && !(ok = wait_on(bar_acc_empty + 8 * acc, acc_phase ^ 1u, abort_flag, kTimeoutTmemEmpty))) break;
                    if (!(ok = wait_on(bar_full + 8 * stage, phase, abort_flag, kTimeoutFull))) break;
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
        // Block kb of a tile goes to accumulator buffer kb % kAccBuffers (2 buffers of 256 columns, or 4 of 128: the drain warps' loop
        // over the blocks is unrolled by the buffers, so every buffer has its own code there); block g of the CTA's sequence is issued
        // by thread g % 2.  One thread alone spends more time per block on its barrier tests and commits than the four MMAs run; with
        // two, one thread's bookkeeping overlaps the other one's MMAs.
        if (lane == 0) {
            static_assert(!S::kFold || (kStages >= 2 && kAccBuffers % 2 == 0), "two issuers alternate over the stages and an even number of buffers");
            constexpr uint32_t idesc = instruction_descriptor(BN);
            const int me = warp - 1;
            const int total = ((tiles - int(blockIdx.x) + int(gridDim.x) - 1) / int(gridDim.x)) * kblocks;
            int stage = me % kStages;
            uint32_t phase = 0;
            int kb = me % kblocks, tile_ordinal = me / kblocks;  // position of block g in the CTA's sequence of tiles
            for (int g = me; g < total; g += 2) {
                // uses of this buffer so far: per tile ceil((kblocks - acc) / kAccBuffers), plus those of this tile
                const int acc = kb % kAccBuffers;
                const int per_tile = acc < kblocks ? (kblocks - acc + kAccBuffers - 1) / kAccBuffers : 0;
                const uint32_t acc_phase = uint32_t(tile_ordinal * per_tile + kb / kAccBuffers) & 1u;
                const uint32_t d = tmem_base + acc * S::kAccColumns;
                if (!wait_on(bar_acc_empty + 8 * acc, acc_phase ^ 1u, abort_flag, kTimeoutTmemEmpty)) break;
                if (!wait_on(bar_full + 8 * stage, phase, abort_flag, kTimeoutFull)) break;
                tc_fence_after();
                const uint32_t a_addr = smem_u32(smem + stage * S::kStageBytes);
                const uint64_t a_desc = smem_descriptor(a_addr), a_lo_desc = smem_descriptor(a_addr + S::kABytes),
                               b_desc = smem_descriptor(a_addr + S::kABytes * (S::kHilo ? 2 : 1));
#pragma unroll
                for (int j = 0; j < kStageK / kMmaK; ++j) {
                    const uint32_t accumulate = j == 0 ? 0u : 1u;  // every block starts a fresh sum
                    const uint64_t step = uint64_t(j * kMmaK >> 4);
                    mma_i8(d, a_desc + step, b_desc + step, idesc, accumulate);
                    if (S::kHilo) mma_i8(d + BN, a_lo_desc + step, b_desc + step, idesc, accumulate);
                }
                tc_commit(bar_empty + 8 * stage);
                tc_commit(bar_acc_full + 8 * acc);
                stage += 2;  // at most one wrap per step (kStages >= 2)
                if (stage >= kStages) { stage -= kStages; phase ^= 1u; }
                kb += 2;
                while (kb >= kblocks) { kb -= kblocks; ++tile_ordinal; }
            }
        }
    }
    if (warp == 3) {
        // ---------------- column parameters: per tile for the write-out, per block for group-scaled weights ----------------
        // The write-out of a tile needs each column's weight scale, bias and residual scale.  Fetching them there would put a trip to
        // L2 (long, while the operand loads keep it busy) in front of every group of outputs; this warp puts them into shared memory
        // one tile ahead instead: weight scale and bias (0 if none) as FP32, residual scale (1 if none) in the output type.
        if constexpr (!DUMP) {
            const T* rscale = static_cast<const T*>(p.rscale);
            int slot = 0, tile_count = 0;
            uint32_t phase = 0;
            bool ok = true;
            auto stage_params = [&](const TileCoord& c) -> bool {
                if (!p.vector_io) return true;
                // every drain warp is done with the previous tile's parameters
                if (tile_count > 0 && !wait_on(bar_params_consumed, uint32_t(tile_count - 1) & 1u, abort_flag, kTimeoutParams)) return false;
                const float* sb = p.sb[c.segment];
                const T* bias = static_cast<const T*>(p.bias[c.segment]);
                for (int i = lane; i < BN; i += 32) {
                    const int col = c.n0 + i;
                    const bool inside = col < p.n;
                    param_sb[i] = !S::kWGroup && inside ? __ldg(sb + col) : 0.f;
                    param_bias[i] = bias && inside ? as_float(bias[col]) : 0.f;
                    param_rscale[i] = rscale && !p.window.span && inside ? rscale[col] : round_one<T>(1.f);
                }
                mbar_arrive(bar_params_written);
                ++tile_count;
                return true;
            };
            for (int t = blockIdx.x; t < tiles && ok; t += gridDim.x) {
                const TileCoord c = tile_origin<BN>(t, p.tiles_m, p.tiles_n, p.seg_tiles);
                if constexpr (S::kWGroup) {
                    // the first two blocks' scales go first: the drain warps start on them right after the previous tile's write-out
                    const int params_after = (kblocks < 2 ? kblocks : 2) - 1;
                    for (int kb = 0; kb < kblocks && ok; ++kb) {
                        if (!(ok = wait_on(bar_ring_empty + 8 * slot, phase ^ 1u, abort_flag, kTimeoutScales))) break;
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
    } else {
        // ---------------- drain ----------------
        asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(kDrainRegs));
        const int quarter = warp & 3, part = (warp - kControlWarps) >> 2;  // lanes 32 quarter .. + 32, columns kEpi part .. + kEpi
        const uint32_t lane_base = uint32_t(quarter * 32) << 16;
        const T* residual = static_cast<const T*>(p.residual);
        const T* rscale = static_cast<const T*>(p.rscale);
        const float* sa = p.sa + in_shift * (S::kBlockScales ? kblocks : 1);
        int acc = 0, slot = 0;              // row / exact: the buffer of the tile being finished
        uint32_t acc_phase = 0, ring_phase = 0;
        uint32_t buffer_phases = 0;         // per-block modes: bit b = phase of buffer b's next use
        bool ok = true;
        const int drain_warp = warp - kControlWarps;
        const uint32_t my_stage = store_stage + drain_warp * S::kStoreTile;
        int tile_count = 0;  // tiles this CTA has finished: the phase of the parameter hand-over barriers
        float sa_ahead[2] = {0.f, 0.f};
        bool sa_ahead_valid = false;
        // the next tile's coordinates are worked out before this tile's write-out, where the arithmetic hides behind the stores
        TileCoord c = tile_origin<BN>(blockIdx.x, p.tiles_m, p.tiles_n, p.seg_tiles), c_next = c;
        for (int t = blockIdx.x; t < tiles && ok; t += gridDim.x, c = c_next) {
            const int row = c.m0 + quarter * 32 + lane;
            const bool row_ok = row < p.m;
            const int col0 = c.n0 + part * kEpi;
            const float row_scale = S::kBlockScales ? 1.f : (row_ok ? __ldg(sa + row) : 0.f);
            T* y = static_cast<T*>(p.y[c.segment]) + out_shift * p.ld_y;
            // The tile's column parameters arrive in shared memory from warp 3; false when the CTA aborts.
            auto await_params = [&]() -> bool {
                if (!p.vector_io) return true;
                return __all_sync(0xffffffffu, wait_on(bar_params_written, uint32_t(tile_count) & 1u, abort_flag, kTimeoutParams));
            };
            auto params_done = [&]() {
                if (!p.vector_io) return;
                __syncwarp();
                if (lane == 0) mbar_arrive(bar_params_consumed);
                ++tile_count;
            };

            // y values of 32 columns starting at `col` (chunk = index of the 32-column chunk among this thread's): bias, residual, one
            // rounding, store.  The accumulators of a tile live in registers, so this body is instantiated once per 32 columns of the
            // thread: it is kept short.
            auto emit = [&](const float* v, int col, int chunk) {
                if (col >= p.n) return;
                T* dst = y + int64_t(row) * p.ld_y + col;
                const T* res = residual && row_ok ? residual + (out_shift + row) * p.ld_residual + col : nullptr;
                if (p.vector_io) {
                    // N is a multiple of 8 and every operand 16-byte aligned: eight outputs per step with 128-bit accesses; groups of eight
                    // are whole or absent at the right edge, rows past M are clipped by the TMA store (or skipped by the plain one)
                    const bool staged = p.tma_y != 0;
                    constexpr bool wide = S::kWide;
                    const bool second = wide && (chunk & 1);
                    if (staged && !second) {
                        // the TMA store that last read this buffer must be done with it before the warp writes it again
                        if (lane == 0) asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
                        __syncwarp();
                    }
                    // residual scales of a row window with spans: per row, straight from memory
                    const T* rs_row = rscale && p.window.span ? rscale + (out_shift + row) / p.window.span * p.window.scale_step : nullptr;
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
                        {
                            const float4 b0 = *reinterpret_cast<const float4*>(param_bias + ct), b1 = *reinterpret_cast<const float4*>(param_bias + ct + 4);
                            bias8[0] = b0.x; bias8[1] = b0.y; bias8[2] = b0.z; bias8[3] = b0.w;
                            bias8[4] = b1.x; bias8[5] = b1.y; bias8[6] = b1.z; bias8[7] = b1.w;
                        }
#pragma unroll
                        for (int e = 0; e < 8; ++e) out[e] = fmaf(v[j + e] * row_scale, scale8[e], bias8[e]);
                        if (res) {
                            float res8[8], rs8[8];
                            load_eight_plain(res + j, res8);  // read before this thread overwrites it (y may be the residual)
                            if (rs_row) load_eight(rs_row + col + j, rs8, true);
                            else load_eight_plain(param_rscale + ct, rs8);
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
                            asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(my_stage + lane * (wide ? 128 : 64) + piece * 16), "r"(packed.x),
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
                            // segments: map s is the output of weight s; else one map per destination of the same output
                            const int first_map = p.destinations > 1 ? 0 : c.segment, maps = p.destinations > 1 ? p.destinations : 1;
                            for (int d = 0; d < maps; ++d)
                                asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%1, %2}], [%3];" ::"l"(&out_maps.map[first_map + d]),
                                             "r"(second ? col - 32 : col), "r"(c.m0 + quarter * 32), "r"(my_stage)
                                             : "memory");
                            asm volatile("cp.async.bulk.commit_group;" ::: "memory");
                        }
                    }
                    return;
                }
                // Odd N or unaligned operands: one element at a time.  The values go through this thread's 64 bytes of the staging tile
                // (no TMA store is in flight in such a launch), 16 at a time, so that a short loop can index them.
                const float* sb = p.sb[c.segment];
                const T* bias = static_cast<const T*>(p.bias[c.segment]);
#pragma unroll
                for (int part16 = 0; part16 < 32; part16 += 16) {
                    float* mine = store_stage_generic + (drain_warp * S::kStoreTile + lane * 64) / 4;
#pragma unroll
                    for (int j = 0; j < 16; ++j) mine[j] = v[part16 + j];
#pragma unroll 1
                    for (int j = 0; j < 16; ++j) {
                        const int cj = col + part16 + j;
                        if (row_ok && cj < p.n) {
                            const float col_scale = S::kWGroup ? 1.f : __ldg(sb + cj);
                            float value = fmaf(mine[j] * row_scale, col_scale, bias ? as_float(bias[cj]) : 0.f);
                            if (res) {
                                const T* rs = rscale && p.window.span ? rscale + (out_shift + row) / p.window.span * p.window.scale_step : rscale;
                                value = fmaf(value, rs ? as_float(rs[cj]) : 1.f, as_float(res[part16 + j]));
                            }
                            dst[part16 + j] = round_one<T>(value);
                        }
                    }
                }
            };

            // The common write-out: a tile that lies inside N, 16-byte accessible operands, one destination reached through its tensor map.
            // Everything a chunk needs beside the accumulators sits in shared memory as FP32 (or arrives as `res`, four 16-byte pieces of the
            // residual row requested a chunk ahead); the outputs are computed with two-wide FP32 instructions and rounded BEFORE the warp waits
            // for the TMA unit to be done reading the staging tile of the previous chunk, so that wait hides behind the arithmetic.
            // Same operations per output, in the same order, as `emit`: the bits do not depend on which of the two writes a tile.
            const bool fast_tile = !S::kWide && p.vector_io && p.tma_y && p.destinations == 1 && c.n0 + BN <= p.n && !(rscale && p.window.span);
            auto emit_fast = [&](const float2* a, int chunk, const uint4* res, bool has_res) {
                const int ct = part * kEpi + chunk * 32;  // first column of the chunk within the tile
                uint32_t packed[16];
#pragma unroll
                for (int g = 0; g < 4; ++g) {  // eight columns
                    float2 o[4];
#pragma unroll
                    for (int h = 0; h < 2; ++h) {
                        float2 v0 = a[4 * g + 2 * h], v1 = a[4 * g + 2 * h + 1];
                        if constexpr (!S::kBlockScales) {
                            v0 = __fmul2_rn(v0, make_float2(row_scale, row_scale));
                            v1 = __fmul2_rn(v1, make_float2(row_scale, row_scale));
                        }
                        const float4 b = *reinterpret_cast<const float4*>(param_bias + ct + 8 * g + 4 * h);
                        if constexpr (S::kWGroup) {
                            o[2 * h] = __fadd2_rn(v0, make_float2(b.x, b.y));
                            o[2 * h + 1] = __fadd2_rn(v1, make_float2(b.z, b.w));
                        } else {
                            const float4 w = *reinterpret_cast<const float4*>(param_sb + ct + 8 * g + 4 * h);
                            o[2 * h] = __ffma2_rn(v0, make_float2(w.x, w.y), make_float2(b.x, b.y));
                            o[2 * h + 1] = __ffma2_rn(v1, make_float2(w.z, w.w), make_float2(b.z, b.w));
                        }
                    }
                    if (has_res) {
                        const uint4 rs = *reinterpret_cast<const uint4*>(param_rscale + ct + 8 * g);
                        const uint32_t rs_raw[4] = {rs.x, rs.y, rs.z, rs.w}, res_raw[4] = {res[g].x, res[g].y, res[g].z, res[g].w};
#pragma unroll
                        for (int e = 0; e < 4; ++e) {
                            float2 scale2, res2;
                            unpack_pair<T>(rs_raw[e], scale2.x, scale2.y);
                            unpack_pair<T>(res_raw[e], res2.x, res2.y);
                            o[e] = __ffma2_rn(o[e], scale2, res2);
                        }
                    }
#pragma unroll
                    for (int e = 0; e < 4; ++e) packed[4 * g + e] = pack_pair<T>(o[e].x, o[e].y);
                }
                // the TMA store that last read this warp's staging tile must be done with it
                if (lane == 0) asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
                __syncwarp();
#pragma unroll
                for (int g = 0; g < 4; ++g) {
                    // row `lane` of the staging tile, 16-byte piece g at its place in the 64-byte swizzle
                    const uint32_t piece = uint32_t(g) ^ ((uint32_t(lane) >> 1) & 3u);
                    asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(my_stage + lane * 64 + piece * 16), "r"(packed[4 * g]),
                                 "r"(packed[4 * g + 1]), "r"(packed[4 * g + 2]), "r"(packed[4 * g + 3])
                                 : "memory");
                }
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                __syncwarp();
                if (lane == 0) {
                    asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%1, %2}], [%3];" ::"l"(&out_maps.map[c.segment]),
                                 "r"(c.n0 + ct), "r"(c.m0 + quarter * 32), "r"(my_stage)
                                 : "memory");
                    asm volatile("cp.async.bulk.commit_group;" ::: "memory");
                }
            };
            // 16-byte piece g of the 32 residual values that belong to chunk `chunk` of this thread's row (plain loads: y may be the residual)
            const T* res_row = residual && row_ok ? residual + (out_shift + row) * p.ld_residual + col0 : nullptr;
            auto fetch_residual = [&](int chunk, uint4* res) {
#pragma unroll
                for (int g = 0; g < 4; ++g) res[g] = *reinterpret_cast<const uint4*>(res_row + chunk * 32 + 8 * g);
            };

            if constexpr (S::kFold) {
                // FP32 accumulators of this thread's kEpi columns, as pairs for the two-wide FP32 instructions
                float2 accf[kEpi / 2];
#pragma unroll
                for (int j = 0; j < kEpi / 2; ++j) accf[j] = make_float2(0.f, 0.f);
                // activation block scales of this thread's row: two blocks ahead in registers (rows past M read row 0's: never stored)
                const float* sa_row = sa + int64_t(row_ok ? row : 0) * kblocks;
                float sa_now = 0.f, sa_next = 0.f;
                if constexpr (S::kBlockScales && !DUMP) {
                    if (sa_ahead_valid) {  // requested while the previous tile was being written out
                        sa_now = sa_ahead[0];
                        sa_next = sa_ahead[1];
                    } else {
                        sa_now = __ldg(sa_row);
                        sa_next = kblocks > 1 ? __ldg(sa_row + 1) : 0.f;
                    }
                }
                // One block of K: wait for its sums, bring them into registers in chunks of 16 columns (two sets of staging registers:
                // chunks 0 and 1 are requested together, every later chunk into the set that has just been folded), hand the buffer back
                // to the MMAs as soon as the last chunk has arrived -- half a drain before the folding ends -- and fold.  BUFFER is a
                // compile-time constant: the loop over the blocks below is unrolled by the buffers.
                auto drain_block = [&](auto buffer_tag, int kb) -> bool {
                    constexpr int BUFFER = decltype(buffer_tag)::value;
                    float sa_after = 0.f;
                    if constexpr (S::kBlockScales && !DUMP) {
                        if (kb + 2 < kblocks) sa_after = __ldg(sa_row + kb + 2);
                    }
                    if constexpr (S::kWGroup) {
                        if (!wait_on(bar_ring_full + 8 * slot, ring_phase, abort_flag, kTimeoutScales)) return false;
                    }
                    if (!wait_on(bar_acc_full + 8 * BUFFER, (buffer_phases >> BUFFER) & 1u, abort_flag, kTimeoutTmemFull)) return false;
                    buffer_phases ^= 1u << BUFFER;
                    tc_fence_after();
                    const uint32_t taddr = tmem_base + lane_base + BUFFER * S::kAccColumns + part * kEpi;
                    const float* ring = scale_ring + slot * BN + part * kEpi;
                    constexpr int CH = Roles<PARTS>::kChunk < kEpi ? Roles<PARTS>::kChunk : kEpi, kChunks = kEpi / CH;
                    int hi[2][CH], lo[2][S::kHilo ? CH : 1];
                    auto fetch = [&](int chunk) {
                        if constexpr (CH == 32) {
                            tmem_load_32(taddr + chunk * CH, hi[chunk & 1]);
                            if constexpr (S::kHilo) tmem_load_32(taddr + BN + chunk * CH, lo[chunk & 1]);
                        } else {
                            tmem_load_16(taddr + chunk * CH, hi[chunk & 1]);
                            if constexpr (S::kHilo) tmem_load_16(taddr + BN + chunk * CH, lo[chunk & 1]);
                        }
                    };
                    auto release = [&]() {
                        // every column of this warp's part of the buffer is in registers: the buffer goes back to the MMAs
                        tc_fence_before();
                        __syncwarp();
                        if (lane == 0) mbar_arrive(bar_acc_empty + 8 * BUFFER);
                    };
                    auto fold = [&](int chunk) {
                        const int* h = hi[chunk & 1];
                        const int* l = lo[chunk & 1];
                        if constexpr (DUMP) {
                            if (row_ok)
#pragma unroll
                                for (int j = 0; j < CH; ++j)
                                    if (col0 + chunk * CH + j < p.n) p.dump[(int64_t(kb) * p.m + row) * p.n + col0 + chunk * CH + j] = h[j];
                        } else {
                            const float2 sa2 = make_float2(sa_now, sa_now);
#pragma unroll
                            for (int j = 0; j < CH / 2; ++j) {
                                float2 v = make_float2(float(h[2 * j]), float(h[2 * j + 1]));
                                float2& a = accf[chunk * (CH / 2) + j];
                                if constexpr (MODE == kBlock) {
                                    a = __ffma2_rn(v, sa2, a);
                                } else {
                                    const float2 w = *reinterpret_cast<const float2*>(ring + chunk * CH + 2 * j);
                                    if constexpr (MODE == kBlockG) {
                                        a = __ffma2_rn(v, __fmul2_rn(sa2, w), a);
                                    } else {
                                        const float2 low = make_float2(float(l[2 * j]), float(l[2 * j + 1]));
                                        v = __ffma2_rn(low, make_float2(1.f / 254.f, 1.f / 254.f), v);
                                        a = __ffma2_rn(v, w, a);
                                    }
                                }
                            }
                        }
                    };
                    fetch(0);
                    if (kChunks > 1) fetch(1);
                    tmem_load_wait();
                    if (kChunks <= 2) release();
#pragma unroll
                    for (int chunk = 0; chunk < kChunks; ++chunk) {
                        fold(chunk);
                        if (chunk + 2 < kChunks) {
                            fetch(chunk + 2);  // into the set just folded
                            if (chunk + 2 == kChunks - 1) {
                                tmem_load_wait();  // every column is in registers
                                release();
                            }
                        }
                    }
                    if constexpr (S::kWGroup) {
                        __syncwarp();
                        if (lane == 0) mbar_arrive(bar_ring_empty + 8 * slot);
                        if (++slot == kScaleRing) { slot = 0; ring_phase ^= 1u; }
                    }
                    sa_now = sa_next;
                    sa_next = sa_after;
                    return true;
                };
                // block kb of the tile uses buffer kb % kAccBuffers (the MMA issuers follow the same rule)
                for (int kb = 0; kb < kblocks && ok; kb += kAccBuffers) {
                    ok = drain_block(std::integral_constant<int, 0>(), kb);
                    if constexpr (kAccBuffers > 1) if (ok && kb + 1 < kblocks) ok = drain_block(std::integral_constant<int, 1>(), kb + 1);
                    if constexpr (kAccBuffers > 2) if (ok && kb + 2 < kblocks) ok = drain_block(std::integral_constant<int, 2>(), kb + 2);
                    if constexpr (kAccBuffers > 3) if (ok && kb + 3 < kblocks) ok = drain_block(std::integral_constant<int, 3>(), kb + 3);
                }
                if (!ok) break;
                const int t_next = t + int(gridDim.x);
                if (t_next < tiles) c_next = tile_origin<BN>(t_next, p.tiles_m, p.tiles_n, p.seg_tiles);
                if constexpr (S::kBlockScales && !DUMP) {
                    // the first two block scales of this thread's row in the next tile: in flight while this tile is written out
                    sa_ahead_valid = t_next < tiles;
                    if (sa_ahead_valid) {
                        const int row_next = c_next.m0 + quarter * 32 + lane;
                        const float* next_row = sa + int64_t(row_next < p.m ? row_next : 0) * kblocks;
                        sa_ahead[0] = __ldg(next_row);
                        sa_ahead[1] = kblocks > 1 ? __ldg(next_row + 1) : 0.f;
                    }
                }
                if constexpr (!DUMP) {
                    if (!(ok = await_params())) break;
                    if (fast_tile) {
                        // the residual of a chunk is requested while the chunk before it is written out, where the registers allow it
                        constexpr bool kResidualAhead = PARTS == 2 && !S::kWGroup;
                        uint4 res[kResidualAhead ? 2 : 1][4];
                        if (kResidualAhead && res_row) fetch_residual(0, res[0]);
#pragma unroll
                        for (int chunk = 0; chunk < kEpi / 32; ++chunk) {
                            if constexpr (kResidualAhead) {
                                if (res_row && chunk + 1 < kEpi / 32) fetch_residual(chunk + 1, res[(chunk + 1) & 1]);
                                emit_fast(&accf[chunk * 16], chunk, res[chunk & 1], res_row != nullptr);
                            } else {
                                if (res_row) fetch_residual(chunk, res[0]);
                                emit_fast(&accf[chunk * 16], chunk, res[0], res_row != nullptr);
                            }
                        }
                    } else
#pragma unroll
                    for (int chunk = 0; chunk < kEpi / 32; ++chunk) {
                        float v[32];
#pragma unroll
                        for (int j = 0; j < 16; ++j) {
                            v[2 * j] = accf[chunk * 16 + j].x;
                            v[2 * j + 1] = accf[chunk * 16 + j].y;
                        }
                        emit(v, col0 + chunk * 32, chunk);
                    }
                    params_done();
                }
            } else {
                if (!(ok = __all_sync(0xffffffffu, wait_on(bar_acc_full + 8 * acc, acc_phase, abort_flag, kTimeoutTmemFull)))) break;
                tc_fence_after();
                const uint32_t taddr = tmem_base + lane_base + acc * S::kAccColumns + part * kEpi;
                if (t + int(gridDim.x) < tiles) c_next = tile_origin<BN>(t + int(gridDim.x), p.tiles_m, p.tiles_n, p.seg_tiles);
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
                    if (fast_tile) {
                        float2 pairs[16];
#pragma unroll
                        for (int j = 0; j < 16; ++j) pairs[j] = make_float2(v[2 * j], v[2 * j + 1]);
                        uint4 res[4];
                        if (res_row) fetch_residual(chunk, res);
                        emit_fast(pairs, chunk, res, res_row != nullptr);
                    } else {
                        emit(v, col0 + chunk * 32, chunk);
                    }
                }
                params_done();
                if (++acc == kAccBuffers) { acc = 0; acc_phase ^= 1u; }
            }
        }
        if (lane == 0) asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");  // staged outputs
    }

    // common exit: every role falls through to here, aborting or not
    tc_fence_before();
    __syncthreads();
    if (warp == 2) {
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
static bool make_map(CUtensorMap* map, const void* base, int64_t rows, int k, int box_rows) {
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

// The same map for other translation units (the few-token tensor-core kernel): (rows, k) bytes, boxes of box_rows x 128 bytes, 128-byte swizzle.
bool make_swizzled_byte_map(CUtensorMap* map, const void* base, int64_t rows, int k, int box_rows) { return make_map(map, base, rows, k, box_rows); }

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
    // several weights of one input (n = output channels of each): per-segment weight, scales, bias and output
    int segments = 1;
    const int8_t* const* seg_b = nullptr;
    const float* const* seg_sb = nullptr;
    const void* const* seg_bias = nullptr;
    void* const* seg_y = nullptr;
    RowWindow window = {nullptr, 0, 0, 0, 0, 0, 0};
};

// Rows a tensor map of a row window may address: the window's position is only known on the GPU.
constexpr int64_t kUnboundedRows = int64_t(1) << 30;

template <class T, int MODE, int BN, bool WIDE, bool DUMP, int PARTS>
static int launch(const GemmArgs& g, cudaStream_t stream) {
    using S = Shape<MODE, BN, WIDE, PARTS>;
    auto kernel = gemm_i8_tc<T, MODE, BN, WIDE, DUMP, PARTS>;
    static bool configured[64] = {};  // the attribute belongs to a device's copy of the kernel
    int device = 0;
    cudaGetDevice(&device);
    if (device < 0 || device >= 64 || !configured[device]) {
        const cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, S::kSmemBytes);
        if (e != cudaSuccess) return int(e);
        if (device >= 0 && device < 64) configured[device] = true;
    }
    if ((reinterpret_cast<uintptr_t>(g.a) & 15) || (g.a_lo && (reinterpret_cast<uintptr_t>(g.a_lo) & 15))) return -2;
    const bool windowed = g.window.counter != nullptr;
    InputMaps in_maps;
    WeightMaps w_maps;
    OutputMaps out_maps;
    GemmParams p{};
    const int64_t a_rows = windowed ? kUnboundedRows : g.m;
    p.tail_rows = windowed ? g.m % kBM : 0;
    if (!make_map(&in_maps.a, g.a, a_rows, g.k, kBM)) return int(cudaErrorNotSupported);
    in_maps.a_lo = in_maps.a_tail = in_maps.a_lo_tail = in_maps.a;
    if (S::kHilo && !make_map(&in_maps.a_lo, g.a_lo, a_rows, g.k, kBM)) return int(cudaErrorNotSupported);
    if (p.tail_rows) {
        if (!make_map(&in_maps.a_tail, g.a, a_rows, g.k, p.tail_rows)) return int(cudaErrorNotSupported);
        if (S::kHilo && !make_map(&in_maps.a_lo_tail, g.a_lo, a_rows, g.k, p.tail_rows)) return int(cudaErrorNotSupported);
    }
    uintptr_t bases = reinterpret_cast<uintptr_t>(g.residual) | reinterpret_cast<uintptr_t>(g.rscale);
    for (int s = 0; s < kMaxSegments; ++s) {
        const bool used = s < g.segments;
        const int8_t* b = !used ? nullptr : g.seg_b ? g.seg_b[s] : g.b;
        p.sb[s] = !used ? nullptr : g.seg_sb ? g.seg_sb[s] : g.sb;
        p.bias[s] = !used ? nullptr : g.seg_bias ? g.seg_bias[s] : g.bias;
        p.y[s] = !used ? nullptr : g.seg_y ? g.seg_y[s] : (g.ys ? g.ys[0] : g.y);
        if (used) {
            if (reinterpret_cast<uintptr_t>(b) & 15) return -2;
            if (!make_map(&w_maps.map[s], b, g.n, g.k, BN)) return int(cudaErrorNotSupported);
            bases |= reinterpret_cast<uintptr_t>(p.y[s]) | reinterpret_cast<uintptr_t>(p.bias[s]) | (S::kWGroup ? 0 : reinterpret_cast<uintptr_t>(p.sb[s]));
        } else {
            w_maps.map[s] = w_maps.map[0];
        }
    }
    p.sa = g.sa; p.residual = g.residual; p.rscale = g.rscale; p.dump = g.dump;
    p.ld_y = g.ld_y ? g.ld_y : g.n;
    p.ld_residual = g.ld_residual ? g.ld_residual : g.n;
    p.destinations = g.ys ? g.count : 1;
    if (p.destinations < 1 || p.destinations > kMaxDestinations || (p.destinations > 1 && g.segments > 1)) return -2;
    p.m = g.m; p.n = g.n; p.k = g.k;
    p.tiles_m = (g.m + kBM - 1) / kBM;
    p.seg_tiles = (g.n + BN - 1) / BN;
    p.tiles_n = p.seg_tiles * g.segments;
    p.window = g.window;
    if (S::kWGroup) {
        if (!g.scale_scratch || (reinterpret_cast<uintptr_t>(g.scale_scratch) & 15)) return -2;
        const int kblocks = (g.k + kStageK - 1) / kStageK;
        p.n_pad = padded_n(g.n);
        p.sb_blocks = g.scale_scratch;
        const int64_t total = int64_t(kblocks) * p.n_pad;
        regroup_weight_scales<<<int((total + 255) / 256 < 1184 ? (total + 255) / 256 : 1184), 256, 0, stream>>>(g.sb, g.scale_scratch, g.n, kblocks, p.n_pad);
    }
    for (int d = 1; d < p.destinations; ++d) bases |= reinterpret_cast<uintptr_t>(g.ys[d]);
    p.vector_io = g.n % 8 == 0 && p.ld_y % 8 == 0 && p.ld_residual % 8 == 0 && (bases & 15) == 0 &&
                  (!g.window.span || g.window.scale_step % 8 == 0);
    // a row window's outputs leave through plain, row-predicated stores: where they go is only known on the GPU
    p.tma_y = !DUMP && p.vector_io && !windowed;
    const bool wide = S::kWide;
    const int maps = p.destinations > 1 ? p.destinations : g.segments;
    for (int d = 0; d < kMaxDestinations; ++d) {
        if (p.tma_y && d < maps)
            p.tma_y = make_output_map(&out_maps.map[d], p.destinations > 1 ? (d == 0 ? p.y[0] : g.ys[d]) : p.y[d], g.m, g.n, p.ld_y,
                                      std::is_same<T, bf16>::value, wide);
        else
            out_maps.map[d] = in_maps.a;
    }
    if (p.destinations > 1 && !p.tma_y) return -2;  // several destinations are only written by the TMA stores
    const int64_t tiles = int64_t(p.tiles_m) * p.tiles_n;
    const int sms = g.sms > 0 ? g.sms : 148;
    const int grid = int(tiles < sms ? tiles : sms);
    kernel<<<grid, Roles<PARTS>::kThreads, S::kSmemBytes, stream>>>(in_maps, w_maps, out_maps, p);
    return int(cudaGetLastError());
}

template <class T, int MODE, int BN, int PARTS = 4> static int launch_width(const GemmArgs& g, cudaStream_t stream) {
    // several destinations: staging tiles with 128-byte rows, one operand stage less
    if (g.ys && g.count > 1) return launch<T, MODE, BN, true, false, PARTS>(g, stream);
    return launch<T, MODE, BN, false, false, PARTS>(g, stream);
}

// Variant numbers keep the reference's meaning of the MODE (row 0 / 2 / 6, exact 1 / 7, block 10 / 11, block+g 12 / 13, exact+g 14);
// the tile shapes are this library's own: 256 output channels per tile, or 128 for variants 13, 15, 16.  Variants 20 and 22 are 10 and 12
// with eight drain warps of 128 columns instead of sixteen of 64: fewer instructions per output, fewer warps to hide latencies with.
template <class T> static int dispatch(const GemmArgs& g, int variant, cudaStream_t stream) {
    switch (variant) {
        case 0: case 2: case 6: return launch_width<T, kRow, 256>(g, stream);
        case 1: case 7: return launch_width<T, kExact, 256>(g, stream);
        case 10: case 11: return launch_width<T, kBlock, 256>(g, stream);
        case 12: return launch_width<T, kBlockG, 256>(g, stream);
        case 13: return launch_width<T, kBlockG, 128>(g, stream);
        case 14: return launch_width<T, kExactG, 128>(g, stream);
        case 15: case 16: return launch_width<T, kBlock, 128>(g, stream);  // tiles of 128 columns: four accumulator buffers
        case 20: return launch_width<T, kBlock, 256, 2>(g, stream);
        case 22: return launch_width<T, kBlockG, 256, 2>(g, stream);
    }
    return -3;
}

static int gemm_entry(GemmArgs& g, int dtype, int variant, cudaStream_t stream) {
    if ((variant == 1 || variant == 7 || variant == 14) != (g.a_lo != nullptr)) return -2;
    if (g.k <= 0 || g.k % 16) return -2;
    if (dtype == 0) return dispatch<__half>(g, variant, stream);
    if (dtype == 1) return dispatch<bf16>(g, variant, stream);
    return -1;
}

}  // namespace wq

using namespace wq;

WQ_API int wq8_gemm(const int8_t* a, const int8_t* a_lo, const float* sa, const int8_t* b, const float* sb, const void* bias, const void* residual,
                    const void* rscale, void* y, int m, int n, int k, int dtype, int variant, int sms, int /*split*/, int* workspace,
                    int* /*counters*/, cudaStream_t stream) {
    if (m <= 0 || n <= 0) return 0;
    GemmArgs g{reinterpret_cast<float*>(workspace), a, a_lo, sa, b, sb, bias, residual, rscale, y, nullptr, m, n, k, sms};
    return gemm_entry(g, dtype, variant, stream);
}

// wq8_gemm on a window of rows whose position is read on the GPU when the kernel runs: the output rows (and those of the residual) start
// at first + counter[0] * step of y; the input rows (A, A_lo and their scales) at in_first + counter[0] * in_step when either is
// non-zero; span > 0: rscale holds scale_step values per span of output rows.
WQ_API int wq8_gemm_at(const int8_t* a, const int8_t* a_lo, const float* sa, const int8_t* b, const float* sb, const void* bias, const void* residual,
                       const void* rscale, void* y, int m, int n, int k, int dtype, int variant, int sms, int /*split*/, int* workspace,
                       int* /*counters*/, const long long* counter, long long first, long long step, long long span, long long scale_step,
                       long long in_first, long long in_step, cudaStream_t stream) {
    if (m <= 0 || n <= 0) return 0;
    if (span < 0) return -2;
    GemmArgs g{reinterpret_cast<float*>(workspace), a, a_lo, sa, b, sb, bias, residual, rscale, y, nullptr, m, n, k, sms};
    g.window = {counter, first, step, counter ? span : 0, scale_step, in_first, in_step};
    return gemm_entry(g, dtype, variant, stream);
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
    GemmArgs g{reinterpret_cast<float*>(workspace), a, a_lo, sa, b, sb, bias, residual, rscale, ys[0], nullptr, m, n, k, sms};
    g.ys = ys;
    g.count = count;
    g.ld_y = ld_y;
    g.ld_residual = residual ? ld_residual : 0;
    return gemm_entry(g, dtype, variant, stream);
}

// Whole tiles only: no partial sums, no counters.  The variants with group-scaled weights regroup the weight scales by block of K
// into the workspace.
WQ_API void wq8_gemm_workspace(int, int n, int k, int variant, int, int, int64_t* sizes) {
    sizes[0] = sizes[1] = 0;
    if (((variant >= 12 && variant <= 14) || variant == 22) && n > 0 && k > 0) sizes[0] = int64_t((k + kStageK - 1) / kStageK) * padded_n(n) * 4;
}

WQ_API int wq8_gemm_select(int, int, int, int hilo, int) { return hilo ? 1 : 0; }

// `count` (1 to 4) linears of one input in ONE launch: the persistent tile schedule walks count x ceil(rows / tile) column tiles per row
// band, each tile taking its weight, scales, bias and output from its segment, so the quantized input is read once for all of them.
// Per-channel weight scales only, no residual, as in the reference.
WQ_API int wq8_gemm_segments(const int8_t* a, const int8_t* a_lo, const float* sa, const int8_t* const* bs, const float* const* sbs,
                             const void* const* biases, void* const* ys, int count, int rows, int m, int k, int dtype, int variant, int sms, int /*split*/,
                             int* workspace, int* /*counters*/, cudaStream_t stream) {
    if (count < 1 || count > kMaxSegments || rows <= 0 || rows % 8 || !bs || !sbs || !ys) return -4;
    if ((variant >= 12 && variant <= 14) || variant == 22) return -4;
    for (int s = 0; s < count; ++s)
        if (!bs[s] || !sbs[s] || !ys[s]) return -4;
    if (m <= 0) return 0;
    const void* no_bias[kMaxSegments] = {nullptr, nullptr, nullptr, nullptr};
    GemmArgs g{reinterpret_cast<float*>(workspace), a, a_lo, sa, bs[0], sbs[0], nullptr, nullptr, nullptr, ys[0], nullptr, m, rows, k, sms};
    g.segments = count;
    g.seg_b = bs;
    g.seg_sb = sbs;
    g.seg_bias = biases ? biases : no_bias;
    g.seg_y = ys;
    return gemm_entry(g, dtype, variant, stream);
}

WQ_API int wq8_debug_block_sums(const int8_t* a, const int8_t* b, int32_t* sums, int m, int n, int k, int sms, cudaStream_t stream) {
    if (m <= 0 || n <= 0) return 0;
    if (k <= 0 || k % 16) return -2;
    const GemmArgs g{nullptr, a, nullptr, nullptr, b, nullptr, nullptr, nullptr, nullptr, nullptr, sums, m, n, k, sms};
    return launch<bf16, kBlock, 256, false, true, 4>(g, stream);
}

// A bounded wait on a barrier that nothing ever completes, with a limit of `clocks`: the kernel must come back, leave `code` in the
// status word and the device usable.  What the tests use to see the give-up path of every wait in this library work, without a fault.
namespace wq {
__global__ void bounded_wait_probe(long long clocks, int code, int* returned) {
    __shared__ uint64_t bar;
    __shared__ int abort_word;
    if (threadIdx.x == 0) {
        abort_word = 0;
        mbar_init(smem_u32(&bar), 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    const bool completed = mbar_wait(smem_u32(&bar), 0, &abort_word, code, &g_status, clocks);
    if (threadIdx.x == 0) *returned = completed ? 1 : 2;
}
}  // namespace wq

WQ_API int wq8_debug_wait_probe(long long clocks, int code, int* returned, cudaStream_t stream) {
    if (clocks <= 0 || clocks > 2000000000ll || !returned) return -2;
    bounded_wait_probe<<<1, 64, 0, stream>>>(clocks, code, returned);
    return int(cudaGetLastError());
}

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
