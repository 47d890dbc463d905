// Few-token weight-only linear (up to 32 tokens) on the 5th-generation tensor cores, with the INT8 weights used as they are.
//
// The few activations are rewritten once per call as three planes of signed 7-bit digits per token and 128 values of K with one power of
// two, x = 2^(E-7) (q0 + q1 / 128 + q2 / 16384) (split_digits; exact for every value within 2^14 of the largest of its 128, rounded to
// nearest below that).  The linear then is an INT8 x INT8 product per 128 of K:
//
//     weights  (128 output channels x 128 of K)   = the M x K operand of tcgen05.mma kind::i8, straight from the checkpoint through TMA
//     digits   (3 planes x TB token slots x 128)  = the N x K operand (TB = 8, 16 or 32 token slots; N = 32, 48 or 96 columns)
//     sums     (128 lanes x N columns, INT32)     in tensor memory, 4 to 8 buffers deep, exact
//
// and four drain warps (one thread per output channel) combine the three planes in FP32, scale by the token's power of two of that run
// and accumulate 8 to 32 FP32 sums per thread -- as little CUDA-core work per weight byte as the job allows, none of it on the weights.
// The kernel is a weight stream: a ring of up to 7 stages of {16 KiB of weights, 4-12 KiB of digits} per SM keeps 20+ MB requested
// ahead of use across the GPU.
//
// Work is spread stream-K style: the (channel tile, K block) pairs are numbered linearly and every CTA takes one contiguous share of
// them, so all SMs stream for the same time whatever N and K are.  A tile whose K range is shared by several CTAs is finished by the
// last one to arrive (a counter per tile): every piece is written to a slot of the caller's scratch, and the last arriver adds the
// pieces in CTA order -- a fixed order, so the result does not depend on timing.  Counters are zero on entry and left zero.
//
// Every wait is bounded (tc_ptx.cuh): a wait that gives up records a code in the status word of the streaming kernels, raises the
// CTA's abort flag, and the CTA leaves through the common exit with tensor memory released.
#include <cuda.h>

#include "tc_ptx.cuh"

namespace wq {

constexpr int kTcThreads = 256;       // warp 0: TMA producer; warp 1: MMA issuer; warp 2: tensor-memory owner; warps 4-7: drain
constexpr int kTcRun = 128;           // values of K sharing one power of two = one K block = one stage
constexpr int kTcChannels = 128;      // output channels of a tile = tensor-memory lanes
constexpr long long kTcWaitLimit = 4000000000ll;
__device__ int g_tc_status = 0;  // first code of a wait of this kernel that gave up (read and cleared by stream_tc_status_take)

template <int TB> struct TcShape {
    static_assert(TB == 8 || TB == 16 || TB == 32, "8, 16 or 32 token slots");
    static constexpr int kColumns = TB == 8 ? 32 : 3 * TB;          // MMA N: the three planes of TB tokens (a multiple of 16)
    static constexpr int kDigitRows = kColumns;                      // rows of the digit matrix (3 TB, padded to 32 for TB = 8)
    static constexpr int kWeightBytes = kTcChannels * kTcRun, kDigitBytes = kColumns * kTcRun;
    static constexpr int kStageBytes = kWeightBytes + kDigitBytes;
    static constexpr int kBarrierBytes = 320;
    static constexpr int kStages = (227 * 1024 - kBarrierBytes) / kStageBytes > 8 ? 8 : (227 * 1024 - kBarrierBytes) / kStageBytes;
    static constexpr int kSmemBytes = kStages * kStageBytes + kBarrierBytes;
    // Accumulator buffers in tensor memory: the hand-over of a buffer (MMA done -> drain reads it -> MMA may overwrite it) takes far longer
    // than a K block's MMAs, so the MMAs run several buffers ahead of the drain.
    static constexpr int kAccBuffers = kColumns <= 48 ? 8 : 4;
    static constexpr int kTmemColumns = kAccBuffers * kColumns <= 256 ? 256 : 512;
    static constexpr int kPieceFloats = kTcChannels * TB;            // partial sums of one piece of a tile
};

// digits: (3 TB [padded to 32 rows for TB = 8], K) int8, row p * TB + t = plane p of token slot t; scales: (K / 128, TB) float = 2^(E-7)
// of (run, token), 0 for empty slots.  One warp per (token slot, run), 4 values per lane.
template <class T, int TB>
__global__ void __launch_bounds__(256) split_digits(const T* x, int64_t ldx, int8_t* __restrict__ digits, float* __restrict__ scales, int m, int k) {
    // the stream kernel that follows may start (its set-up and its first weight loads do not depend on the digits); it waits for this
    // grid to finish before it touches them.  This kernel itself may have started under the tail of the one that produced x.
    dependents_may_start();
    dependency_wait();
    const int lane = threadIdx.x & 31, runs = k / kTcRun;
    const int unit = blockIdx.x * 8 + (threadIdx.x >> 5);
    constexpr int kRows = TcShape<TB>::kDigitRows, kSlots = kRows == 3 * TB ? TB : kRows - 2 * TB;  // TB = 8: 16 slots cover the padding rows
    if (unit >= runs * kSlots) return;
    const int token = unit % kSlots, run = unit / kSlots;
    if (token >= TB) {  // padding rows of the 8-token layout (rows 24 .. 31): zeros
        *reinterpret_cast<uint32_t*>(digits + int64_t(2 * TB + token) * k + run * kTcRun + 4 * lane) = 0u;
        return;
    }
    float v[4] = {0.f, 0.f, 0.f, 0.f};
    if (token < m) {
        const uint2 raw = load_8(x + int64_t(token) * ldx + run * kTcRun + 4 * lane);
        unpack_pair<T>(raw.x, v[0], v[1]);
        unpack_pair<T>(raw.y, v[2], v[3]);
    }
    float amax = fmaxf(fmaxf(fabsf(v[0]), fabsf(v[1])), fmaxf(fabsf(v[2]), fabsf(v[3])));
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, d));
    // amax < 2^E; the digits of v / 2^E in base 128: the first two truncate toward zero (every remainder keeps the sign and is exact in
    // FP32), the last one rounds to nearest: the rewritten value is within 2^(E-22) of v, without a bias toward zero
    int exponent = 0;
    if (amax > 0.f) frexpf(amax, &exponent);
    exponent = max(exponent, -110);  // 2^(7 - E) and 2^(E - 7) stay finite, normal numbers; runs of denormal-sized values become zeros
    const float down = ldexpf(1.f, 7 - exponent);
    uint32_t packed[3] = {0u, 0u, 0u};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        float f = v[j] * down;  // |f| < 128
#pragma unroll
        for (int p = 0; p < 3; ++p) {
            const float digit = p < 2 ? truncf(f) : fminf(fmaxf(rintf(f), -127.f), 127.f);
            packed[p] |= (uint32_t(int(digit)) & 0xffu) << (8 * j);
            f = (f - digit) * 128.f;
        }
    }
#pragma unroll
    for (int p = 0; p < 3; ++p) *reinterpret_cast<uint32_t*>(digits + int64_t(p * TB + token) * k + run * kTcRun + 4 * lane) = packed[p];
    if (lane == 0) scales[run * TB + token] = amax > 0.f ? ldexpf(1.f, exponent - 7) : 0.f;
}

struct TcParams {
    const float* scales;   // (K / 128, TB)
    const float* sw;
    const void* bias;
    const void* residual;
    const void* rscale;
    void* y;
    float* slots;          // 2 pieces of kPieceFloats per CTA
    int* counters;         // one per tile, zero on entry, left zero
    int m, n, k, tiles, kblocks;
};

WQ_DEVICE bool tc_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag) {
    return mbar_wait(bar, parity, abort_flag, 2, &g_tc_status, kTcWaitLimit);
}

// start of CTA c's share of the `total` (tile, K block) pairs among `ctas`
WQ_DEVICE long long share_start(long long c, long long total, long long ctas) { return c * total / ctas; }
// the last CTA whose share starts at or before pair v
WQ_DEVICE long long cta_of_pair(long long v, long long total, long long ctas) { return ((v + 1) * ctas + total - 1) / total - 1; }

template <class T, int TB>
__global__ void __launch_bounds__(kTcThreads, 1)
stream_tc(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_d, const TcParams p) {
    using S = TcShape<TB>;
    constexpr int kStages = S::kStages, N = S::kColumns;
    extern __shared__ __align__(1024) uint8_t smem[];
    if (smem_u32(smem) & 1023u) {
        if (threadIdx.x == 0) atomicCAS(&g_tc_status, 0, 3);
        return;
    }
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + kStages * S::kStageBytes);
    // barriers: full[8], empty[8], acc_full[8], acc_empty[8]; then the TMEM slot, the abort flag and the arrival broadcast
    constexpr int kAcc = S::kAccBuffers;
    const uint32_t bar_full = smem_u32(bars), bar_empty = bar_full + 64, bar_acc_full = bar_empty + 64, bar_acc_empty = bar_acc_full + 64;
    uint32_t& tmem_slot = *reinterpret_cast<uint32_t*>(reinterpret_cast<uint8_t*>(bars) + 256);
    int& abort_word = *reinterpret_cast<int*>(reinterpret_cast<uint8_t*>(bars) + 260);
    int& arrival = *reinterpret_cast<int*>(reinterpret_cast<uint8_t*>(bars) + 264);
    volatile int* abort_flag = &abort_word;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    if (threadIdx.x == 0) {
        abort_word = 0;
        for (int s = 0; s < 8; ++s) {
            mbar_init(bar_full + 8 * s, 1);
            mbar_init(bar_empty + 8 * s, 1);
        }
        for (int s = 0; s < 8; ++s) {
            mbar_init(bar_acc_full + 8 * s, 1);
            mbar_init(bar_acc_empty + 8 * s, 4);
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        prefetch_tensormap(&map_w);
        prefetch_tensormap(&map_d);
    }
    if (warp == 2) tmem_alloc(smem_u32(&tmem_slot), S::kTmemColumns);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = tmem_slot;

    // Launched with programmatic stream serialization behind the digit split: everything above overlapped its tail, and so do the
    // producer's first weight loads; each role waits for the split to finish before it touches the digits or the scales.  (Without
    // that launch attribute the wait returns at once.)

    // this CTA's share of the (tile, K block) pairs
    const long long total = (long long)p.tiles * p.kblocks, ctas = gridDim.x;
    const long long begin = share_start(blockIdx.x, total, ctas), end = share_start(blockIdx.x + 1, total, ctas);

    if (warp == 0) {
        // ---------------- TMA producer ----------------
        if (lane == 0) {
            int stage = 0;
            uint32_t phase = 0;
            bool ok = true;
            // the ring's first fill: the weights go out at once, the digits of the same stages once the split has finished
            const long long first_fill = end - begin < kStages ? end - begin : kStages;
            for (long long i = 0; i < first_fill; ++i) {
                const long long pair = begin + i;
                const int tile = int(pair / p.kblocks), kb = int(pair - (long long)tile * p.kblocks);
                mbar_expect_tx(bar_full + 8 * int(i), S::kStageBytes);
                tma_load_2d(smem_u32(smem + int(i) * S::kStageBytes), &map_w, bar_full + 8 * int(i), kb * kTcRun, tile * kTcChannels);
            }
            dependency_wait();
            for (long long i = 0; i < first_fill; ++i) {
                const int kb = int((begin + i) % p.kblocks);
                tma_load_2d(smem_u32(smem + int(i) * S::kStageBytes) + S::kWeightBytes, &map_d, bar_full + 8 * int(i), kb * kTcRun, 0);
            }
            if (first_fill == kStages) phase = 1u; else stage = int(first_fill);
            for (long long pair = begin + first_fill; pair < end && ok; ++pair) {
                const int tile = int(pair / p.kblocks), kb = int(pair - (long long)tile * p.kblocks);
                if (!(ok = tc_wait(bar_empty + 8 * stage, phase ^ 1u, abort_flag))) break;
                const uint32_t full = bar_full + 8 * stage, dst = smem_u32(smem + stage * S::kStageBytes);
                mbar_expect_tx(full, S::kStageBytes);
                tma_load_2d(dst, &map_w, full, kb * kTcRun, tile * kTcChannels);
                tma_load_2d(dst + S::kWeightBytes, &map_d, full, kb * kTcRun, 0);
                if (++stage == kStages) { stage = 0; phase ^= 1u; }
            }
            if (!ok) {
                for (int s = 0; s < kStages; ++s) {  // aborting: let the copies already issued land before shared memory is given back
                    const long long start = clock64();
                    while (!mbar_try_wait(bar_full + 8 * s, 0) && !mbar_try_wait(bar_full + 8 * s, 1) && clock64() - start < 2000000) {}
                }
            }
        }
    } else if (warp == 1) {
        // ---------------- MMA issuer: every K block is a fresh sum in the next accumulator buffer ----------------
        if (lane == 0) {
            constexpr uint32_t idesc = instruction_descriptor(N);
            int stage = 0;
            uint32_t phase = 0;
            for (long long pair = begin, block = 0; pair < end; ++pair, ++block) {
                const int acc = int(block % kAcc);
                if (!tc_wait(bar_acc_empty + 8 * acc, (uint32_t(block / kAcc) & 1u) ^ 1u, abort_flag)) break;
                if (!tc_wait(bar_full + 8 * stage, phase, abort_flag)) break;
                tc_fence_after();
                const uint32_t w_addr = smem_u32(smem + stage * S::kStageBytes);
                const uint64_t w_desc = smem_descriptor(w_addr), d_desc = smem_descriptor(w_addr + S::kWeightBytes);
#pragma unroll
                for (int j = 0; j < kTcRun / kMmaK; ++j) {
                    const uint64_t step = uint64_t(j * kMmaK >> 4);
                    mma_i8(tmem_base + acc * N, w_desc + step, d_desc + step, idesc, j == 0 ? 0u : 1u);
                }
                tc_commit(bar_empty + 8 * stage);
                tc_commit(bar_acc_full + 8 * acc);
                if (++stage == kStages) { stage = 0; phase ^= 1u; }
            }
        }
    } else if (warp >= 4) {
        // ---------------- drain: one thread per output channel of the tile ----------------
        dependency_wait();  // the scales of the runs come from the split
        const int quarter = warp & 3;
        const uint32_t lane_base = uint32_t(quarter * 32) << 16;
        const int thread = quarter * 32 + lane;  // channel of the tile
        const T* bias = static_cast<const T*>(p.bias);
        const T* residual = static_cast<const T*>(p.residual);
        const T* rscale = static_cast<const T*>(p.rscale);
        T* y = static_cast<T*>(p.y);
        float* my_slots = p.slots + (long long)blockIdx.x * 2 * S::kPieceFloats;
        bool ok = true;
        long long block = 0;
        for (long long pair = begin; pair < end && ok;) {
            const int tile = int(pair / p.kblocks), kb0 = int(pair - (long long)tile * p.kblocks);
            const int kb1 = int(min((long long)p.kblocks, kb0 + (end - pair)));
            float acc[TB];
#pragma unroll
            for (int t = 0; t < TB; ++t) acc[t] = 0.f;
            for (int kb = kb0; kb < kb1 && ok; ++kb, ++block) {
                // the powers of two of this run's tokens: requested before the wait (every lane the same addresses: one transaction each)
                float4 scale4[TB / 4];
#pragma unroll
                for (int i = 0; i < TB / 4; ++i) {
                    const uint4 bits = load_16(p.scales + (long long)kb * TB + 4 * i);
                    scale4[i] = make_float4(__uint_as_float(bits.x), __uint_as_float(bits.y), __uint_as_float(bits.z), __uint_as_float(bits.w));
                }
                const int buffer = int(block % kAcc);
                if (!(ok = tc_wait(bar_acc_full + 8 * buffer, uint32_t(block / kAcc) & 1u, abort_flag))) break;
                tc_fence_after();
                const uint32_t taddr = tmem_base + lane_base + buffer * N;
                int sums[3][TB];
#pragma unroll
                for (int plane = 0; plane < 3; ++plane) {
                    if constexpr (TB == 32) tmem_load_32(taddr + plane * TB, sums[plane]);
                    else if constexpr (TB == 16) tmem_load_16(taddr + plane * TB, sums[plane]);
                    else tmem_load_8(taddr + plane * TB, sums[plane]);
                }
                tmem_load_wait();
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(bar_acc_empty + 8 * buffer);  // the sums are in registers: the buffer goes back to the MMAs
                const float* scale = reinterpret_cast<const float*>(scale4);
#pragma unroll
                for (int t = 0; t < TB; ++t) {
                    // exact INT32 sums of the run (below 2^21 in magnitude) -> FP32, planes combined, scaled by the token's power of two
                    const float combined = fmaf(float(sums[2][t]), 1.f / 16384.f, fmaf(float(sums[1][t]), 1.f / 128.f, float(sums[0][t])));
                    acc[t] = fmaf(combined, scale[t], acc[t]);
                }
            }
            if (!ok) break;
            const int channel = tile * kTcChannels + thread;
            const bool whole = kb0 == 0 && kb1 == p.kblocks;
            bool finish = whole;
            if (!whole) {
                // a piece of a tile: into this CTA's slot (0: the tile its share starts in, 1: the tile it ends in), then the tile's counter
                const int which = (long long)tile * p.kblocks <= begin ? 0 : 1;
                float* slot = my_slots + which * S::kPieceFloats;
#pragma unroll
                for (int t = 0; t < TB; ++t) __stcg(slot + t * kTcChannels + thread, acc[t]);
                __threadfence();
                asm volatile("bar.sync 1, 128;" ::: "memory");  // the four drain warps
                const long long first_pair = (long long)tile * p.kblocks;
                const int first_cta = int(cta_of_pair(first_pair, total, ctas)), last_cta = int(cta_of_pair(first_pair + p.kblocks - 1, total, ctas));
                if (thread == 0) arrival = atomicAdd(p.counters + tile, 1);
                asm volatile("bar.sync 1, 128;" ::: "memory");
                finish = arrival == last_cta - first_cta;  // the last piece to arrive finishes the tile
                asm volatile("bar.sync 1, 128;" ::: "memory");  // `arrival` may be rewritten by this CTA's next piece
                if (finish) {
                    __threadfence();
#pragma unroll
                    for (int t = 0; t < TB; ++t) acc[t] = 0.f;
                    for (int c = first_cta; c <= last_cta; ++c) {  // the pieces in CTA order: a fixed order of additions
                        const int piece = share_start(c, total, ctas) >= first_pair ? 0 : 1;
                        const float* from = p.slots + ((long long)c * 2 + piece) * S::kPieceFloats;
#pragma unroll
                        for (int t = 0; t < TB; ++t) acc[t] += __ldcg(from + t * kTcChannels + thread);
                    }
                    if (thread == 0) p.counters[tile] = 0;  // left zero for the next launch
                }
            }
            if (finish && channel < p.n) {
                const float sw = p.sw[channel], b = bias ? as_float(bias[channel]) : 0.f;
                const float rs = rscale ? as_float(rscale[channel]) : 1.f;
#pragma unroll
                for (int t = 0; t < TB; ++t) {
                    if (t < p.m) {
                        float v = fmaf(acc[t], sw, b);
                        if (residual) v = fmaf(v, rs, as_float(residual[(long long)t * p.n + channel]));
                        y[(long long)t * p.n + channel] = round_one<T>(v);
                    }
                }
            }
            pair += kb1 - kb0;
        }
    }

    tc_fence_before();
    __syncthreads();
    if (warp == 2) {
        tc_fence_after();
        tmem_dealloc(tmem_base, S::kTmemColumns);
    }
}

// ---- host side -------------------------------------------------------------------------------------------------------
bool make_swizzled_byte_map(CUtensorMap* map, const void* base, int64_t rows, int k, int box_rows);  // gemm_tc.cu

struct TcPlan { int token_slots, ctas; int64_t digit_bytes, scale_bytes, slot_bytes, counter_bytes; };

static int token_slots_of(int m) { return m <= 8 ? 8 : m <= 16 ? 16 : 32; }

// The plan of a shape, or token_slots = 0 when the shape is not this kernel's (K not a multiple of 128, more than 32 tokens).
static TcPlan plan_tc(int m, int n, int k, int sms) {
    TcPlan plan{0, 0, 0, 0, 0, 0};
    if (m <= 0 || m > 32 || n <= 0 || k <= 0 || k % kTcRun) return plan;
    if (sms <= 0) sms = 148;
    const int slots = token_slots_of(m), tiles = (n + kTcChannels - 1) / kTcChannels, kblocks = k / kTcRun;
    const int64_t pairs = int64_t(tiles) * kblocks;
    plan.token_slots = slots;
    plan.ctas = int(pairs < sms ? pairs : sms);
    const int rows = slots == 8 ? 32 : 3 * slots;
    plan.digit_bytes = int64_t(rows) * k;
    plan.scale_bytes = int64_t(kblocks) * slots * 4;
    plan.slot_bytes = int64_t(plan.ctas) * 2 * kTcChannels * slots * 4;
    plan.counter_bytes = int64_t(tiles) * 4;
    return plan;
}

template <class T, int TB>
static int launch_tc_shape(const T* x, int64_t ldx, const int8_t* w, const float* sw, const T* bias, const T* residual, const T* rscale, T* y, int m, int n,
                           int k, const TcPlan& plan, int8_t* digits, float* scales, float* slots, int* counters, cudaStream_t stream) {
    using S = TcShape<TB>;
    auto kernel = stream_tc<T, TB>;
    static bool configured[64] = {};
    int device = 0;
    cudaGetDevice(&device);
    if (device < 0 || device >= 64 || !configured[device]) {
        const cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, S::kSmemBytes);
        if (e != cudaSuccess) return int(e);
        if (device >= 0 && device < 64) configured[device] = true;
    }
    CUtensorMap map_w, map_d;
    if (!make_swizzled_byte_map(&map_w, w, n, k, kTcChannels) || !make_swizzled_byte_map(&map_d, digits, S::kDigitRows, k, S::kDigitRows))
        return int(cudaErrorNotSupported);
    const int runs = k / kTcRun, units = runs * (TB == 8 ? 16 : TB);
    const cudaError_t split = launch_after_previous(split_digits<T, TB>, dim3((units + 7) / 8), dim3(256), size_t(0), stream, x, ldx, digits, scales, m, k);
    if (split != cudaSuccess) return int(split);
    TcParams p{scales, sw, bias, residual, rscale, y, slots, counters, m, n, k, (n + kTcChannels - 1) / kTcChannels, runs};
    // behind the split: the stream kernel's set-up and first weight loads run under the split's tail
    const cudaError_t launched = launch_after_previous(kernel, dim3(plan.ctas), dim3(kTcThreads), size_t(S::kSmemBytes), stream, map_w, map_d, p);
    return int(launched != cudaSuccess ? launched : cudaGetLastError());
}

// x (m, K) in T, already transformed; workspace: digits, then scales, then slots (plan sizes, each rounded up to 256 bytes); counters zeroed.
template <class T>
static int launch_tc(const void* x, int64_t ldx, const int8_t* w, const float* sw, const void* bias, const void* residual, const void* rscale, void* y, int m,
                     int n, int k, const TcPlan& plan, void* workspace, int* counters, cudaStream_t stream) {
    auto round_up = [](int64_t v) { return (v + 255) / 256 * 256; };
    int8_t* digits = static_cast<int8_t*>(workspace);
    float* scales = reinterpret_cast<float*>(digits + round_up(plan.digit_bytes));
    float* slots = reinterpret_cast<float*>(reinterpret_cast<int8_t*>(scales) + round_up(plan.scale_bytes));
    auto xs = static_cast<const T*>(x);
    auto b = static_cast<const T*>(bias), r = static_cast<const T*>(residual), rs = static_cast<const T*>(rscale);
    auto out = static_cast<T*>(y);
    if (plan.token_slots == 8) return launch_tc_shape<T, 8>(xs, ldx, w, sw, b, r, rs, out, m, n, k, plan, digits, scales, slots, counters, stream);
    if (plan.token_slots == 16) return launch_tc_shape<T, 16>(xs, ldx, w, sw, b, r, rs, out, m, n, k, plan, digits, scales, slots, counters, stream);
    return launch_tc_shape<T, 32>(xs, ldx, w, sw, b, r, rs, out, m, n, k, plan, digits, scales, slots, counters, stream);
}

// What the entry points of stream.cu use.
int64_t stream_tc_workspace(int m, int n, int k, int sms, int64_t* counter_bytes) {
    const TcPlan plan = plan_tc(m, n, k, sms);
    if (counter_bytes) *counter_bytes = plan.token_slots ? plan.counter_bytes : 0;
    if (!plan.token_slots) return 0;
    auto round_up = [](int64_t v) { return (v + 255) / 256 * 256; };
    return round_up(plan.digit_bytes) + round_up(plan.scale_bytes) + round_up(plan.slot_bytes);
}

int stream_tc_launch(const void* x, int64_t ldx, const int8_t* w, const float* sw, const void* bias, const void* residual, const void* rscale, void* y, int m,
                     int n, int k, int dtype, int sms, void* workspace, int* counters, cudaStream_t stream) {
    const TcPlan plan = plan_tc(m, n, k, sms);
    if (!plan.token_slots || !workspace || !counters) return -2;
    if (dtype == 0) return launch_tc<__half>(x, ldx, w, sw, bias, residual, rscale, y, m, n, k, plan, workspace, counters, stream);
    if (dtype == 1) return launch_tc<bf16>(x, ldx, w, sw, bias, residual, rscale, y, m, n, k, plan, workspace, counters, stream);
    return -1;
}

// Status of this kernel on the current device: 0, or the code of a wait that gave up; clears it.
int stream_tc_status_take() {
    int code = 0;
    const int zero = 0;
    if (cudaMemcpyFromSymbol(&code, g_tc_status, sizeof(int)) != cudaSuccess) return -1;
    if (code) cudaMemcpyToSymbol(g_tc_status, &zero, sizeof(int));
    return code;
}

}  // namespace wq
