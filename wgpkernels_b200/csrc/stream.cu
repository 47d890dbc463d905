// Few-token paths ('lines': 1-4 tokens, 'small': up to 32 tokens): weight-only INT8.  The activations stay unquantized (or are rewritten
// exactly as digit planes); the INT8 weight matrix is streamed once from HBM.  HBM-bound: the design goal is bytes in flight on every
// SM and fixed-order (deterministic) reductions.  Kernels of this file:
//   stream_bulk    up to 16 tokens, no scratch: weights through per-warp TMA rings, converted exactly to BF16 / FP16 in registers for
//                  mma.sync.m16n8k16 (what wq8_gemv_lines runs, and wq8_small without scratch)
//   stream_planes  up to 8 tokens: the activations as INT8 digit planes, the weights into mma.sync.m16n8k32.s8 untouched
//   direct_rows    every other shape and alignment, on plain CUDA cores, with an optional split of K over CTAs
// and stream_tc.cu holds the tcgen05 kernel that wq8_small runs with its caller's scratch (up to 32 tokens).
// Together they replace w8a16_small / gemv_lines of the reference (wgpkernels/int8/int8_gemm.cu:1039-1151, 1772-1810): same values up
// to FP32 summation order.
#include "common.cuh"

namespace wq {

WQ_DEVICE uint32_t byte_permute(uint32_t a, uint32_t b, uint32_t selector) {
    uint32_t d;
    asm("prmt.b32 %0, %1, %2, %3;\n" : "=r"(d) : "r"(a), "r"(b), "r"(selector));
    return d;
}

// Four signed bytes -> two packed pairs of T holding exactly the same integers: pair 0 = bytes (0, 1), pair 1 = bytes (2, 3).
// BF16 (7 mantissa bits): place the low 7 bits in the mantissa of 128.0 (0x4300 | low7 = 128 + low7) and subtract 128.0 or,
// for negative bytes, 256.0 (0x4380): (128 + low7) - 256 = low7 - 128 = the signed byte.
// FP16 (10 mantissa bits): 1024.0 (0x6400) | (byte ^ 0x80) = 1024 + byte + 128; subtract 1152.0.
template <class T> WQ_DEVICE void int8x4_to_pairs(uint32_t w, uint32_t& p01, uint32_t& p23);
template <> WQ_DEVICE void int8x4_to_pairs<bf16>(uint32_t w, uint32_t& p01, uint32_t& p23) {
    const uint32_t low7 = w & 0x7f7f7f7fu, sign = w & 0x80808080u;
    uint32_t v01 = byte_permute(low7, 0x43434343u, 0x5140u), o01 = byte_permute(sign, 0x43434343u, 0x5140u);
    uint32_t v23 = byte_permute(low7, 0x43434343u, 0x5342u), o23 = byte_permute(sign, 0x43434343u, 0x5342u);
    __nv_bfloat162 r01 = __hsub2(*reinterpret_cast<__nv_bfloat162*>(&v01), *reinterpret_cast<__nv_bfloat162*>(&o01));
    __nv_bfloat162 r23 = __hsub2(*reinterpret_cast<__nv_bfloat162*>(&v23), *reinterpret_cast<__nv_bfloat162*>(&o23));
    p01 = *reinterpret_cast<uint32_t*>(&r01);
    p23 = *reinterpret_cast<uint32_t*>(&r23);
}
template <> WQ_DEVICE void int8x4_to_pairs<__half>(uint32_t w, uint32_t& p01, uint32_t& p23) {
    const uint32_t flipped = w ^ 0x80808080u;
    uint32_t v01 = byte_permute(flipped, 0x64646464u, 0x5140u), v23 = byte_permute(flipped, 0x64646464u, 0x5342u);
    const __half2 offset = __float2half2_rn(1152.f);
    __half2 r01 = __hsub2(*reinterpret_cast<__half2*>(&v01), offset), r23 = __hsub2(*reinterpret_cast<__half2*>(&v23), offset);
    p01 = *reinterpret_cast<uint32_t*>(&r01);
    p23 = *reinterpret_cast<uint32_t*>(&r23);
}

// D (16 x 8, FP32) += A (16 x 16, row) * B (16 x 8, col).
template <class T> WQ_DEVICE void mma_16x8x16(float* d, uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1);
template <> WQ_DEVICE void mma_16x8x16<bf16>(float* d, uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
template <> WQ_DEVICE void mma_16x8x16<__half>(float* d, uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

constexpr int kStreamChunk = 64;   // elements of K one warp step covers: 16 contiguous bytes per lane of each of its two rows

// ---------------------------------------------------------------------------------------------------------------------
// direct_rows: the shapes and alignments the tensor-core kernels do not take (K any multiple of 4, weights 4-byte aligned, activation
// rows 8-byte aligned, up to 32 tokens), and the K-split path of callers that bring scratch.  Plain CUDA cores, one THREAD per output
// channel: a CTA owns 32 channels (the lanes) and its 8 warps share the CTA's range of K; a thread walks its channel's row four weight
// bytes at a time (exact INT8 -> FP32), multiplying them with the tokens' activations, which every lane of the warp reads from the
// same address (one broadcast transaction).  The 8 warps' sums meet in shared memory and are added in warp order; with gridDim.y > 1
// the CTAs of a channel block split K further, each writes its sums to a slot of the caller's scratch and the last one to arrive
// (a counter per channel block, zero on entry, left zero) adds the slots in split order: every addition order is fixed.
// ---------------------------------------------------------------------------------------------------------------------
constexpr int kDirectChannels = 32, kDirectWarps = 8;

template <class T, int TOKENS>
__global__ void __launch_bounds__(32 * kDirectWarps) direct_rows(const T* __restrict__ x, int64_t ldx, const int8_t* __restrict__ w, const float* __restrict__ sw,
                                                                  const T* __restrict__ bias, const T* residual, const T* __restrict__ rscale, T* y, int m, int n,
                                                                  int k, float* __restrict__ slots, int* __restrict__ counters) {
    __shared__ float partial[kDirectWarps][TOKENS][kDirectChannels + 1];
    __shared__ int is_last;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int channel = blockIdx.x * kDirectChannels + lane;
    const int quads = k / 4, splits = gridDim.y;
    // this CTA's quads of K, then this warp's share of them
    const int cta_begin = int(int64_t(blockIdx.y) * quads / splits), cta_end = int(int64_t(blockIdx.y + 1) * quads / splits);
    const int begin = cta_begin + int(int64_t(warp) * (cta_end - cta_begin) / kDirectWarps);
    const int end = cta_begin + int(int64_t(warp + 1) * (cta_end - cta_begin) / kDirectWarps);
    const uint32_t* row = reinterpret_cast<const uint32_t*>(w + int64_t(channel < n ? channel : 0) * k);
    float acc[TOKENS];
#pragma unroll
    for (int t = 0; t < TOKENS; ++t) acc[t] = 0.f;
    for (int quad = begin; quad < end; ++quad) {
        const uint32_t packed = __ldg(row + quad);
        const float w0 = float(int(int8_t(packed))), w1 = float(int(int8_t(packed >> 8))), w2 = float(int(int8_t(packed >> 16))), w3 = float(int(packed) >> 24);
#pragma unroll
        for (int t = 0; t < TOKENS; ++t) {
            if (t < m) {  // uniform
                const uint2 raw = __ldg(reinterpret_cast<const uint2*>(x + int64_t(t) * ldx + 4 * quad));
                float x0, x1, x2, x3;
                unpack_pair<T>(raw.x, x0, x1);
                unpack_pair<T>(raw.y, x2, x3);
                acc[t] = fmaf(w3, x3, fmaf(w2, x2, fmaf(w1, x1, fmaf(w0, x0, acc[t]))));
            }
        }
    }
#pragma unroll
    for (int t = 0; t < TOKENS; ++t) partial[warp][t][lane] = acc[t];
    __syncthreads();
    // the 8 warps' sums of every (token, channel), in warp order; thread i takes outputs i, i + 256, ...
    constexpr int kOutputs = TOKENS * kDirectChannels;
    float* own = slots ? slots + (int64_t(blockIdx.x) * splits + blockIdx.y) * kOutputs : nullptr;
    for (int i = threadIdx.x; i < kOutputs; i += 32 * kDirectWarps) {
        const int t = i / kDirectChannels, c = i % kDirectChannels;
        float sum = partial[0][t][c];
#pragma unroll
        for (int part = 1; part < kDirectWarps; ++part) sum += partial[part][t][c];
        partial[0][t][c] = sum;  // each output is read and written by this thread only
        if (own) __stcg(own + i, sum);
    }
    if (splits > 1) {
        __threadfence();
        __syncthreads();
        if (threadIdx.x == 0) is_last = atomicAdd(counters + blockIdx.x, 1) == splits - 1;
        __syncthreads();
        if (!is_last) return;
        __threadfence();
        const float* pieces = slots + int64_t(blockIdx.x) * splits * kOutputs;
        for (int i = threadIdx.x; i < kOutputs; i += 32 * kDirectWarps) {
            float sum = 0.f;
            for (int piece = 0; piece < splits; ++piece) sum += __ldcg(pieces + int64_t(piece) * kOutputs + i);
            partial[0][i / kDirectChannels][i % kDirectChannels] = sum;
        }
        if (threadIdx.x == 0) counters[blockIdx.x] = 0;  // left zero for the next launch
    }
    for (int i = threadIdx.x; i < kOutputs; i += 32 * kDirectWarps) {
        const int t = i / kDirectChannels, c = i % kDirectChannels, ch = blockIdx.x * kDirectChannels + c;
        if (t < m && ch < n) {
            float v = fmaf(partial[0][t][c], sw[ch], bias ? as_float(bias[ch]) : 0.f);
            if (residual) v = fmaf(v, rscale ? as_float(rscale[ch]) : 1.f, as_float(residual[int64_t(t) * n + ch]));
            y[int64_t(t) * n + ch] = round_one<T>(v);
        }
    }
}

// ---------------------------------------------------------------------------------------------------------------------
// stream_bulk: the same linear with the weights fed by the copy engine.
//
// A kernel that loads weights straight into registers keeps a few KiB per warp in flight, and only while the warp is not computing: far
// from the bytes the HBM needs outstanding.  Here every warp owns a ring of kBulkStages stages of 4 KiB in shared memory, filled by
// the TMA unit (one cp.async.bulk.tensor box of ROWS weight rows x 128 or 256 bytes of K per stage, no multicast, completion counted by
// an mbarrier per stage; rows past N and bytes past K arrive as zeros): 16 warps x 3 stages x 4 KiB = 192 KiB per SM are requested
// before any of it is needed, whatever the warps are doing.  One persistent CTA per SM walks work items of ROWS output channels (8, 16
// or 32); the 16 warps of the CTA take the item's K segments in turn, the ring running ahead across item boundaries; a 17th warp adds
// the partial sums of the 16 in warp order from shared memory (deterministic), scales, biases and stores them while the others are
// already streaming the next item (two sets of partial sums, handed over through mbarriers).  No workspace of any kind.
// Sixteen warps because the work per stage is a long dependent chain (activation loads, byte conversions, MMAs on one accumulator):
// the SM needs that many chains in progress to keep issuing.
// A wait that runs out (about a second of SM clocks) records a status code, the warp stops computing but keeps meeting the CTA's
// mbarrier hand-overs (a warp that stopped no longer arrives, so its peers run out of time too), and the kernel ends with unspecified
// output instead of hanging.  There is no CTA-wide barrier after the start.
// ---------------------------------------------------------------------------------------------------------------------
constexpr int kBulkWarps = 16, kBulkThreads = 32 * (kBulkWarps + 1), kBulkPartials = 2;  // 16 streaming warps and the reducer warp
constexpr long long kBulkWaitLimit = 2000000000ll;
__device__ int g_stream_status = 0;

WQ_DEVICE uint32_t bulk_smem_address(const void* p) { return uint32_t(__cvta_generic_to_shared(p)); }

WQ_DEVICE bool bulk_stage_ready(uint32_t bar, uint32_t parity) {
    uint32_t done;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(done)
        : "r"(bar), "r"(parity)
        : "memory");
    return done != 0;
}

// false when the data did not arrive in time (recorded) or another warp of the CTA already gave up
WQ_DEVICE bool bulk_wait(uint32_t bar, uint32_t parity, volatile int* gave_up) {
    if (bulk_stage_ready(bar, parity)) return true;
    const long long start = clock64();
    for (uint32_t spin = 1;; ++spin) {
        if (bulk_stage_ready(bar, parity)) return true;
        if ((spin & 63u) == 0u) {
            if (*gave_up) return false;
            if (clock64() - start > kBulkWaitLimit) {
                *gave_up = 1;
                atomicCAS(&g_stream_status, 0, 1);
                return false;
            }
        }
    }
}

template <int MT, int ROWS> struct BulkShape {
    static constexpr int kSegment = ROWS >= 32 ? 128 : 256;  // bytes of K per row and stage (a TMA box is at most 256 bytes wide)
    static constexpr int kStageBytes = ROWS * kSegment;      // 2 KiB (8 rows) or 4 KiB
    static constexpr int kSub = kSegment / kStreamChunk;     // 64-byte pieces per stage and row
    static constexpr int kRowBlocks = ROWS >= 16 ? ROWS / 16 : 1;
    // the partial sums of two items (one being reduced while the next is produced), then as many ring stages per warp as fit (at most 3)
    static constexpr int kPartialBytes = kBulkPartials * kBulkWarps * MT * 8 * (ROWS + 1) * 4;
    static constexpr int kRoom = (227 * 1024 - kPartialBytes - 1024) / (kBulkWarps * kStageBytes);
    static constexpr int kStages = kRoom >= 3 ? 3 : kRoom;
    static_assert(kStages >= 2, "the rings do not fit");
    static constexpr int kRingBytes = kBulkWarps * kStages * kStageBytes;
    static constexpr int kBarrierBytes = (kBulkWarps * kStages + 2 * kBulkPartials) * 8;
    static constexpr int kSmemBytes = kRingBytes + kBarrierBytes + kPartialBytes + 16;
};

template <class T, int MT, int ROWS>
__global__ void __launch_bounds__(kBulkThreads, 1) stream_bulk(const __grid_constant__ CUtensorMap map_w, const T* __restrict__ x, int64_t ldx, const float* __restrict__ sw,
                                                      const T* __restrict__ bias, const T* residual, const T* __restrict__ rscale, T* y, int m, int n,
                                                      int k) {
    using S = BulkShape<MT, ROWS>;
    constexpr int SEG = S::kSegment, SUB = S::kSub, RB = S::kRowBlocks, kStageBytes = S::kStageBytes, kStages = S::kStages;
    constexpr bool kHalf = ROWS == 8;  // rows 8..15 of the MMA tile are empty
    extern __shared__ __align__(1024) uint8_t bulk_smem[];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, g = lane >> 2, t = lane & 3;
    const uint32_t all_bars = bulk_smem_address(bulk_smem + S::kRingBytes);
    const uint32_t sums_ready = all_bars + kBulkWarps * kStages * 8, sums_free = sums_ready + 8 * kBulkPartials;
    using Partial = float[kBulkWarps][MT * 8][ROWS + 1];
    Partial* partial = reinterpret_cast<Partial*>(bulk_smem + S::kRingBytes + S::kBarrierBytes);
    volatile int* gave_up = reinterpret_cast<volatile int*>(bulk_smem + S::kRingBytes + S::kBarrierBytes + S::kPartialBytes);
    if (threadIdx.x == 0) {
        *gave_up = 0;
        for (int s = 0; s < kBulkWarps * kStages; ++s) asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(all_bars + 8 * s));
        for (int s = 0; s < kBulkPartials; ++s) {
            asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(sums_ready + 8 * s), "r"(kBulkWarps));
            asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(sums_free + 8 * s));
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(&map_w) : "memory");
    }
    __syncthreads();

    const int items = (n + ROWS - 1) / ROWS, segments = (k + SEG - 1) / SEG;
    const int my_items = int(blockIdx.x) < items ? (items - int(blockIdx.x) + int(gridDim.x) - 1) / int(gridDim.x) : 0;

    if (warp == kBulkWarps) {
        // ---------------- reducer: adds the 16 warps' partial sums of an item in warp order, scales, adds bias / residual, stores ----------------
        bool ok = true;
        for (int round = 0; round < my_items && ok; ++round) {
            const int set = round % kBulkPartials;
            if (!(ok = __all_sync(0xffffffffu, bulk_wait(sums_ready + 8 * set, uint32_t(round / kBulkPartials) & 1u, gave_up)))) break;
            const int item = int(blockIdx.x) + round * int(gridDim.x);
            for (int i = lane; i < MT * 8 * ROWS; i += 32) {
                const int token = i / ROWS, r = i % ROWS, channel = item * ROWS + r;
                if (token < m && channel < n) {
                    float sum = 0.f;
#pragma unroll
                    for (int part = 0; part < kBulkWarps; ++part) sum += partial[set][part][token][r];
                    float v = sum * sw[channel] + (bias ? as_float(bias[channel]) : 0.f);
                    if (residual) v = fmaf(v, rscale ? as_float(rscale[channel]) : 1.f, as_float(residual[int64_t(token) * n + channel]));
                    y[int64_t(token) * n + channel] = round_one<T>(v);
                }
            }
            __syncwarp();
            if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(sums_free + 8 * set) : "memory");
        }
        return;
    }

    // ---------------- streaming warps ----------------
    uint8_t* ring = bulk_smem + warp * kStages * kStageBytes;
    const uint32_t ring_address = bulk_smem_address(ring);
    const uint32_t bars = all_bars + warp * kStages * 8;
    const int per_item = warp < segments ? (segments - warp + kBulkWarps - 1) / kBulkWarps : 0;  // this warp's stages of one item
    const long long total = (long long)my_items * per_item;

    // the next stage to request: the rows of this CTA's item number ask_round at the warp's K segment number ask_j, into ring slot ask_slot
    // (plain counters: a division per stage would cost more instructions than the stage's arithmetic)
    int ask_round = 0, ask_j = 0, ask_slot = 0;
    auto request = [&]() {
        const int item = int(blockIdx.x) + ask_round * int(gridDim.x), segment = warp + ask_j * kBulkWarps;
        const int slot = ask_slot;
        if (++ask_j == per_item) { ask_j = 0; ++ask_round; }
        if (++ask_slot == kStages) ask_slot = 0;
        const uint32_t bar = bars + 8 * slot;
        if (lane == 0) {
            // the whole box is counted, zero-filled parts included
            asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(kStageBytes) : "memory");
            asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];" ::"r"(
                             ring_address + slot * kStageBytes),
                         "l"(&map_w), "r"(bar), "r"(segment * SEG), "r"(item * ROWS)
                         : "memory");
        }
    };

    const T* x_row[MT];
    bool x_ok[MT];
#pragma unroll
    for (int mt = 0; mt < MT; ++mt) {
        const int token = mt * 8 + g;
        x_ok[mt] = token < m;
        x_row[mt] = x + int64_t(x_ok[mt] ? token : 0) * ldx + 16 * t;
    }

    long long requested = 0;
    for (; requested < total && requested < kStages; ++requested) request();
    bool ok = true;
    long long landed = 0;
    int slot = 0;
    uint32_t parity = 0;  // of the stage the warp consumes next
    for (int round = 0; round < my_items; ++round) {
        // with few outputs per lane, two chains of MMAs per output (even and odd 16-byte pieces) instead of one long dependent chain
        constexpr bool kTwoChains = RB * MT <= 2;
        float acc[RB][MT][4], odd[kTwoChains ? RB : 1][kTwoChains ? MT : 1][4];
#pragma unroll
        for (int rb = 0; rb < RB; ++rb)
#pragma unroll
            for (int mt = 0; mt < MT; ++mt) {
                acc[rb][mt][0] = acc[rb][mt][1] = acc[rb][mt][2] = acc[rb][mt][3] = 0.f;
                if (kTwoChains) odd[rb][mt][0] = odd[rb][mt][1] = odd[rb][mt][2] = odd[rb][mt][3] = 0.f;
            }
        for (int j = 0; j < per_item; ++j) {
            const int segment = warp + j * kBulkWarps;
            const int pieces = min(SUB, (k - segment * SEG) / kStreamChunk);
            // the activations of a piece: this lane's 16 values start at k0 + 16 t.  They do not depend on the stage: the first piece's are
            // requested before the wait, every other piece's while the piece before it is multiplied.
            uint4 xv[MT][2], ahead[MT][2];
            auto fetch_x = [&](int u, uint4 (&v)[MT][2]) {
                const int64_t k0 = int64_t(segment) * SEG + u * kStreamChunk;
#pragma unroll
                for (int mt = 0; mt < MT; ++mt) {
                    const T* p = x_row[mt] + k0;
                    v[mt][0] = x_ok[mt] ? __ldg(reinterpret_cast<const uint4*>(p)) : make_uint4(0u, 0u, 0u, 0u);
                    v[mt][1] = x_ok[mt] ? __ldg(reinterpret_cast<const uint4*>(p) + 1) : make_uint4(0u, 0u, 0u, 0u);
                }
            };
            fetch_x(0, ahead);
            if (ok) ok = __all_sync(0xffffffffu, bulk_wait(bars + 8 * slot, parity, gave_up));
            if (ok) {
                ++landed;
                const uint8_t* stage = ring + slot * kStageBytes;
#pragma unroll
                for (int u = 0; u < SUB; ++u) {
                    if (u < pieces) {
#pragma unroll
                        for (int mt = 0; mt < MT; ++mt) {
                            xv[mt][0] = ahead[mt][0];
                            xv[mt][1] = ahead[mt][1];
                        }
                        if (u + 1 < pieces) fetch_x(u + 1, ahead);
#pragma unroll
                        for (int rb = 0; rb < RB; ++rb) {
                            const uint4 row0 = *reinterpret_cast<const uint4*>(stage + (rb * 16 + g) * SEG + u * kStreamChunk + 16 * t);
                            const uint4 row1 = kHalf ? make_uint4(0u, 0u, 0u, 0u)
                                                     : *reinterpret_cast<const uint4*>(stage + (rb * 16 + g + 8) * SEG + u * kStreamChunk + 16 * t);
                            const uint32_t* r0 = reinterpret_cast<const uint32_t*>(&row0);
                            const uint32_t* r1 = reinterpret_cast<const uint32_t*>(&row1);
#pragma unroll
                            for (int piece = 0; piece < 4; ++piece) {
                                uint32_t a0, a1 = 0u, a2, a3 = 0u;
                                int8x4_to_pairs<T>(r0[piece], a0, a2);
                                if (!kHalf) int8x4_to_pairs<T>(r1[piece], a1, a3);
#pragma unroll
                                for (int mt = 0; mt < MT; ++mt) {
                                    const uint32_t* xs = reinterpret_cast<const uint32_t*>(&xv[mt][piece >> 1]);
                                    float* chain = kTwoChains && (piece & 1) ? odd[kTwoChains ? rb : 0][kTwoChains ? mt : 0] : acc[rb][mt];
                                    mma_16x8x16<T>(chain, a0, a1, a2, a3, xs[(piece & 1) * 2], xs[(piece & 1) * 2 + 1]);
                                }
                            }
                        }
                    }
                }
            }
            __syncwarp();  // every lane has read the stage: its slot takes the stage kStages ahead
            if (ok && requested < total) {
                request();
                ++requested;
            }
            if (++slot == kStages) { slot = 0; parity ^= 1u; }
        }
        // hand the item's partial sums to the reducer: the set of this round is free once the reducer has finished the round two before
        const int set = round % kBulkPartials;
        if (ok && round >= kBulkPartials)
            ok = __all_sync(0xffffffffu, bulk_wait(sums_free + 8 * set, uint32_t(round / kBulkPartials - 1) & 1u, gave_up));
        // acc[rb][mt] = {(row g, token 2t), (g, 2t + 1), (g + 8, 2t), (g + 8, 2t + 1)} of row block rb and token block mt
        if (ok) {
#pragma unroll
            for (int rb = 0; rb < RB; ++rb)
#pragma unroll
                for (int mt = 0; mt < MT; ++mt) {
#pragma unroll
                    for (int e = 0; e < 4; ++e)
                        if (kTwoChains) acc[rb][mt][e] += odd[kTwoChains ? rb : 0][kTwoChains ? mt : 0][e];
                    partial[set][warp][mt * 8 + 2 * t][rb * 16 + g] = acc[rb][mt][0];
                    partial[set][warp][mt * 8 + 2 * t + 1][rb * 16 + g] = acc[rb][mt][1];
                    if (!kHalf) {
                        partial[set][warp][mt * 8 + 2 * t][rb * 16 + g + 8] = acc[rb][mt][2];
                        partial[set][warp][mt * 8 + 2 * t + 1][rb * 16 + g + 8] = acc[rb][mt][3];
                    }
                }
            __syncwarp();
            if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(sums_ready + 8 * set) : "memory");
        }
    }
    // A warp that gave up may still have copies on their way into its ring: give them a bounded chance to land before the CTA's shared
    // memory goes away.
    if (!ok) {
        for (long long pending = landed; pending < requested; ++pending) {
            const long long start = clock64();
            while (!bulk_stage_ready(bars + 8 * int(pending % kStages), uint32_t(pending / kStages) & 1u) && clock64() - start < kBulkWaitLimit / 8) {
            }
        }
    }
}

// ---------------------------------------------------------------------------------------------------------------------
// stream_planes: at most 8 tokens, INT8 tensor cores on the weights as they are.
//
// stream_bulk spends most of its instructions turning weight bytes into BF16 / FP16 (8 instructions per 4 bytes): at 1-8 tokens that,
// not the HBM, bounds it.  Here the few activations are rewritten instead, once per call by split_planes: every run of 128 values of a
// token becomes three planes of signed 7-bit digits with one power of two, x = 2^(E-7) (q0 + q1 / 128 + q2 / 16384), exact for every
// value within 2^14 of the largest of its run (a BF16 / FP16 value has at most 11 significant bits; smaller values are rounded to the
// nearest multiple of 2^-21 of the run's power of two: an absolute error of at most 2^-21 of the run's largest value).  The weights then go into mma.sync.m16n8k32.s8 untouched: per plane an exact INT32 dot product over the
// run, combined and scaled in FP32.  Same rings, reducer and hand-overs as stream_bulk.
// ---------------------------------------------------------------------------------------------------------------------
constexpr int kPlaneRun = 128;   // values sharing one power of two
constexpr int kPlaneTokens = 8;  // token slots of the planes (one MMA column block); unused ones hold zeros

// planes: (8 tokens, 3, K) int8, scales: (K / 128, 8 tokens) float = 2^(E-7).  One warp per token and run, 4 values per lane.
template <class T>
__global__ void __launch_bounds__(256) split_planes(const T* x, int64_t ldx, int8_t* __restrict__ planes, float* __restrict__ scales, int m,
                                                    int k) {
    // the stream kernel behind this one may start (its set-up and its first weight requests do not depend on the planes); this kernel
    // itself may have started under the tail of the one that produced x
    dependents_may_start();
    dependency_wait();
    const int lane = threadIdx.x & 31, runs = k / kPlaneRun;
    const int unit = blockIdx.x * 8 + (threadIdx.x >> 5);
    if (unit >= runs * kPlaneTokens) return;
    const int token = unit % kPlaneTokens, run = unit / kPlaneTokens;
    float v[4] = {0.f, 0.f, 0.f, 0.f};
    if (token < m) {
        const uint2 raw = load_8(x + int64_t(token) * ldx + run * kPlaneRun + 4 * lane);
        unpack_pair<T>(raw.x, v[0], v[1]);
        unpack_pair<T>(raw.y, v[2], v[3]);
    }
    float amax = fmaxf(fmaxf(fabsf(v[0]), fabsf(v[1])), fmaxf(fabsf(v[2]), fabsf(v[3])));
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, d));
    // amax < 2^E; the digits of v / 2^E in base 128: the first two truncate toward zero (every remainder keeps the sign and is exact in
    // FP32), the last one rounds to nearest, so the rewritten value is within 2^(E-22) of v -- half a unit of the last digit, and no
    // bias toward zero; a value within 2^14 of the run's largest (BF16) has no bits below the last digit and is exact
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
    for (int p = 0; p < 3; ++p)
        *reinterpret_cast<uint32_t*>(planes + (int64_t(token) * 3 + p) * k + run * kPlaneRun + 4 * lane) = packed[p];
    if (lane == 0) scales[run * kPlaneTokens + token] = amax > 0.f ? ldexpf(1.f, exponent - 7) : 0.f;
}

WQ_DEVICE void mma_s8_16x8x32(int* d, uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+r"(d[0]), "+r"(d[1]), "+r"(d[2]), "+r"(d[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

template <class T, int ROWS>
__global__ void __launch_bounds__(kBulkThreads, 1) stream_planes(const __grid_constant__ CUtensorMap map_w, const int8_t* planes,
                                                                 const float* scales, const float* __restrict__ sw, const T* __restrict__ bias,
                                                                 const T* residual, const T* __restrict__ rscale, T* y, int m, int n, int k) {
    constexpr int MT = 1;
    using S = BulkShape<MT, ROWS>;
    constexpr int SEG = S::kSegment, RB = S::kRowBlocks, kStageBytes = S::kStageBytes, kStages = S::kStages;
    constexpr int RUNS = SEG / kPlaneRun;  // runs of 128 values per stage: 2, or 1 with 32 rows
    constexpr bool kHalf = ROWS == 8;
    extern __shared__ __align__(1024) uint8_t bulk_smem[];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, g = lane >> 2, t = lane & 3;
    const uint32_t all_bars = bulk_smem_address(bulk_smem + S::kRingBytes);
    const uint32_t sums_ready = all_bars + kBulkWarps * kStages * 8, sums_free = sums_ready + 8 * kBulkPartials;
    using Partial = float[kBulkWarps][MT * 8][ROWS + 1];
    Partial* partial = reinterpret_cast<Partial*>(bulk_smem + S::kRingBytes + S::kBarrierBytes);
    volatile int* gave_up = reinterpret_cast<volatile int*>(bulk_smem + S::kRingBytes + S::kBarrierBytes + S::kPartialBytes);
    if (threadIdx.x == 0) {
        *gave_up = 0;
        for (int s = 0; s < kBulkWarps * kStages; ++s) asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(all_bars + 8 * s));
        for (int s = 0; s < kBulkPartials; ++s) {
            asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(sums_ready + 8 * s), "r"(kBulkWarps));
            asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(sums_free + 8 * s));
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(&map_w) : "memory");
    }
    __syncthreads();

    const int items = (n + ROWS - 1) / ROWS, segments = (k + SEG - 1) / SEG;
    const int my_items = int(blockIdx.x) < items ? (items - int(blockIdx.x) + int(gridDim.x) - 1) / int(gridDim.x) : 0;

    if (warp == kBulkWarps) {
        // ---------------- reducer (as in stream_bulk) ----------------
        bool ok = true;
        for (int round = 0; round < my_items && ok; ++round) {
            const int set = round % kBulkPartials;
            if (!(ok = __all_sync(0xffffffffu, bulk_wait(sums_ready + 8 * set, uint32_t(round / kBulkPartials) & 1u, gave_up)))) break;
            const int item = int(blockIdx.x) + round * int(gridDim.x);
            for (int i = lane; i < MT * 8 * ROWS; i += 32) {
                const int token = i / ROWS, r = i % ROWS, channel = item * ROWS + r;
                if (token < m && channel < n) {
                    float sum = 0.f;
#pragma unroll
                    for (int part = 0; part < kBulkWarps; ++part) sum += partial[set][part][token][r];
                    float v = sum * sw[channel] + (bias ? as_float(bias[channel]) : 0.f);
                    if (residual) v = fmaf(v, rscale ? as_float(rscale[channel]) : 1.f, as_float(residual[int64_t(token) * n + channel]));
                    y[int64_t(token) * n + channel] = round_one<T>(v);
                }
            }
            __syncwarp();
            if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(sums_free + 8 * set) : "memory");
        }
        return;
    }

    // ---------------- streaming warps ----------------
    uint8_t* ring = bulk_smem + warp * kStages * kStageBytes;
    const uint32_t ring_address = bulk_smem_address(ring);
    const uint32_t bars = all_bars + warp * kStages * 8;
    const int per_item = warp < segments ? (segments - warp + kBulkWarps - 1) / kBulkWarps : 0;
    const long long total = (long long)my_items * per_item;
    int ask_round = 0, ask_j = 0, ask_slot = 0;  // the next stage to request (see stream_bulk)
    auto request = [&]() {
        const int item = int(blockIdx.x) + ask_round * int(gridDim.x), segment = warp + ask_j * kBulkWarps;
        const int slot = ask_slot;
        if (++ask_j == per_item) { ask_j = 0; ++ask_round; }
        if (++ask_slot == kStages) ask_slot = 0;
        const uint32_t bar = bars + 8 * slot;
        if (lane == 0) {
            asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(kStageBytes) : "memory");
            asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];" ::"r"(
                             ring_address + slot * kStageBytes),
                         "l"(&map_w), "r"(bar), "r"(segment * SEG), "r"(item * ROWS)
                         : "memory");
        }
    };
    // this lane's 16 digits of a 64-value piece start at 16 t of token g's plane; its outputs are tokens 2 t and 2 t + 1
    const int8_t* plane0 = planes + int64_t(g) * 3 * k + 16 * t;
    const float* my_scales = scales + 2 * t;

    long long requested = 0;
    for (; requested < total && requested < kStages; ++requested) request();
    // the ring's first stages of weights are on their way; the digit planes and their scales exist once the split kernel has finished
    dependency_wait();
    bool ok = true;
    long long landed = 0;
    int slot = 0;
    uint32_t parity = 0;  // of the stage the warp consumes next
    for (int round = 0; round < my_items; ++round) {
        float acc[RB][4];
#pragma unroll
        for (int rb = 0; rb < RB; ++rb) acc[rb][0] = acc[rb][1] = acc[rb][2] = acc[rb][3] = 0.f;
        for (int j = 0; j < per_item; ++j) {
            const int segment = warp + j * kBulkWarps;
            // digits and scales of the stage's runs: independent of the weights, requested before the wait
            uint4 digits[RUNS][3][2];
            float2 scale[RUNS];
#pragma unroll
            for (int run = 0; run < RUNS; ++run) {
                const int k0 = segment * SEG + run * kPlaneRun;
                const bool inside = k0 < k && g < m;  // token slots past M hold zeros: not fetched (their MMA columns are never stored)
                const uint2 scale_bits = k0 < k ? load_8(my_scales + (k0 / kPlaneRun) * kPlaneTokens) : make_uint2(0u, 0u);
                scale[run] = make_float2(__uint_as_float(scale_bits.x), __uint_as_float(scale_bits.y));
#pragma unroll
                for (int p = 0; p < 3; ++p)
#pragma unroll
                    for (int piece = 0; piece < 2; ++piece)
                        digits[run][p][piece] = inside ? load_16(plane0 + int64_t(p) * k + k0 + piece * kStreamChunk) : make_uint4(0u, 0u, 0u, 0u);
            }
            if (ok) ok = __all_sync(0xffffffffu, bulk_wait(bars + 8 * slot, parity, gave_up));
            if (ok) {
                ++landed;
                const uint8_t* stage = ring + slot * kStageBytes;
#pragma unroll
                for (int run = 0; run < RUNS; ++run) {
#pragma unroll
                    for (int rb = 0; rb < RB; ++rb) {
                        int sums[3][4];
#pragma unroll
                        for (int p = 0; p < 3; ++p) sums[p][0] = sums[p][1] = sums[p][2] = sums[p][3] = 0;
#pragma unroll
                        for (int piece = 0; piece < 2; ++piece) {
                            const int offset = run * kPlaneRun + piece * kStreamChunk + 16 * t;
                            const uint4 row0 = *reinterpret_cast<const uint4*>(stage + (rb * 16 + g) * SEG + offset);
                            const uint4 row1 = kHalf ? make_uint4(0u, 0u, 0u, 0u) : *reinterpret_cast<const uint4*>(stage + (rb * 16 + g + 8) * SEG + offset);
#pragma unroll
                            for (int p = 0; p < 3; ++p) {
                                const uint4 d = digits[run][p][piece];
                                mma_s8_16x8x32(sums[p], row0.x, row1.x, row0.y, row1.y, d.x, d.y);
                                mma_s8_16x8x32(sums[p], row0.z, row1.z, row0.w, row1.w, d.z, d.w);
                            }
                        }
                        // exact INT32 sums of the run (below 2^21 in magnitude) -> FP32, planes combined, scaled by the token's power of two
#pragma unroll
                        for (int e = 0; e < 4; ++e) {
                            const float combined = fmaf(float(sums[2][e]), 1.f / 16384.f, fmaf(float(sums[1][e]), 1.f / 128.f, float(sums[0][e])));
                            acc[rb][e] = fmaf(combined, (e & 1) ? scale[run].y : scale[run].x, acc[rb][e]);
                        }
                    }
                }
            }
            __syncwarp();
            if (ok && requested < total) {
                request();
                ++requested;
            }
            if (++slot == kStages) { slot = 0; parity ^= 1u; }
        }
        const int set = round % kBulkPartials;
        if (ok && round >= kBulkPartials)
            ok = __all_sync(0xffffffffu, bulk_wait(sums_free + 8 * set, uint32_t(round / kBulkPartials - 1) & 1u, gave_up));
        if (ok) {
#pragma unroll
            for (int rb = 0; rb < RB; ++rb) {
                partial[set][warp][2 * t][rb * 16 + g] = acc[rb][0];
                partial[set][warp][2 * t + 1][rb * 16 + g] = acc[rb][1];
                if (!kHalf) {
                    partial[set][warp][2 * t][rb * 16 + g + 8] = acc[rb][2];
                    partial[set][warp][2 * t + 1][rb * 16 + g + 8] = acc[rb][3];
                }
            }
            __syncwarp();
            if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(sums_ready + 8 * set) : "memory");
        }
    }
    if (!ok) {
        for (long long pending = landed; pending < requested; ++pending) {
            const long long start = clock64();
            while (!bulk_stage_ready(bars + 8 * int(pending % kStages), uint32_t(pending / kStages) & 1u) && clock64() - start < kBulkWaitLimit / 8) {
            }
        }
    }
}

// ---- host side ---------------------------------------------------------------------------------------------------------
struct DirectPlan { int ctas, splits, token_slots; };

static int tokens_blocks(int m) { return m <= 8 ? 1 : m <= 16 ? 2 : 4; }

// Channel blocks of 32, and as many splits of K across CTAs (only with scratch) as give every SM two CTAs, each split keeping at least
// 64 quads of K per warp; at most 1024 channel blocks can be split (the counter buffer callers keep).
static DirectPlan plan_direct(int m, int n, int k, int sms, bool may_split) {
    DirectPlan p{(n + kDirectChannels - 1) / kDirectChannels, 1, 8 * tokens_blocks(m)};
    const int target = 2 * (sms > 0 ? sms : 148);
    if (may_split && p.ctas < target && p.ctas <= 1024) {
        const int wanted = (target + p.ctas - 1) / p.ctas, most = (k / 4) / (kDirectWarps * 64);
        p.splits = wanted < most ? wanted : (most > 1 ? most : 1);
    }
    return p;
}

static int64_t direct_slot_bytes(const DirectPlan& p) { return p.splits > 1 ? int64_t(p.ctas) * p.splits * p.token_slots * kDirectChannels * 4 : 0; }

template <class T>
static int launch_direct(const void* x, int64_t ldx, const int8_t* w, const float* sw, const void* bias, const void* residual, const void* rscale,
                         void* y, int m, int n, int k, const DirectPlan& p, float* slots, int* counters, cudaStream_t stream) {
    const dim3 grid(p.ctas, p.splits);
    auto xs = static_cast<const T*>(x);
    auto b = static_cast<const T*>(bias), r = static_cast<const T*>(residual), rs = static_cast<const T*>(rscale);
    auto out = static_cast<T*>(y);
    float* sl = p.splits > 1 ? slots : nullptr;
    switch (p.token_slots) {
        case 8: direct_rows<T, 8><<<grid, 32 * kDirectWarps, 0, stream>>>(xs, ldx, w, sw, b, r, rs, out, m, n, k, sl, counters); break;
        case 16: direct_rows<T, 16><<<grid, 32 * kDirectWarps, 0, stream>>>(xs, ldx, w, sw, b, r, rs, out, m, n, k, sl, counters); break;
        default: direct_rows<T, 32><<<grid, 32 * kDirectWarps, 0, stream>>>(xs, ldx, w, sw, b, r, rs, out, m, n, k, sl, counters); break;
    }
    return int(cudaGetLastError());
}

// Rows per work item of stream_bulk / stream_planes (0: the shape is left to the other kernels).  More rows per item read the activations fewer
// times (every item reads all of x from L2), reduce less often and were the faster choice at every measured shape; fewer rows only when
// the larger items would leave more than a fifth of the SMs' time idle.
static int plan_bulk(int m, int n, int k, int sms) {
    if (sms <= 0) sms = 148;
    if (m > 16) return 0;  // 17-32 tokens: four token blocks per lane do not fit the registers of a 17-warp CTA (the tensor-core kernel's job)
    int best = 0;
    double best_balance = 0.0;
    for (int rows = 32; rows >= 8; rows /= 2) {
        const int segment = rows >= 32 ? 128 : 256;
        if (k / segment < kBulkWarps) continue;  // fewer K segments than warps: warps would idle
        const int items = (n + rows - 1) / rows, rounds = (items + sms - 1) / sms;
        const double balance = double(items) / (double(sms) * rounds);
        if (balance >= 0.8) return rows;
        if (balance > best_balance) {
            best_balance = balance;
            best = rows;
        }
    }
    return best;
}

template <class T, int MT, int ROWS>
static int launch_bulk_shape(const T* x, int64_t ldx, const int8_t* w, const float* sw, const T* bias, const T* residual, const T* rscale, T* y, int m,
                             int n, int k, int sms, cudaStream_t stream) {
    using S = BulkShape<MT, ROWS>;
    auto kernel = stream_bulk<T, MT, ROWS>;
    static bool configured[64] = {};  // the attribute belongs to a device's copy of the kernel
    int device = 0;
    cudaGetDevice(&device);
    if (device < 0 || device >= 64 || !configured[device]) {
        const cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, S::kSmemBytes);
        if (e != cudaSuccess) return int(e);
        if (device >= 0 && device < 64) configured[device] = true;
    }
    CUtensorMap map_w;
    if (!make_byte_matrix_map(&map_w, w, n, k, S::kSegment, ROWS)) return int(cudaErrorNotSupported);
    const int items = (n + ROWS - 1) / ROWS;
    kernel<<<items < sms ? items : sms, kBulkThreads, S::kSmemBytes, stream>>>(map_w, x, ldx, sw, bias, residual, rscale, y, m, n, k);
    return int(cudaGetLastError());
}

template <class T>
static int launch_bulk(const void* x, int64_t ldx, const int8_t* w, const float* sw, const void* bias, const void* residual, const void* rscale, void* y,
                       int m, int n, int k, int rows, int sms, cudaStream_t stream) {
    auto xs = static_cast<const T*>(x);
    auto b = static_cast<const T*>(bias), r = static_cast<const T*>(residual), rs = static_cast<const T*>(rscale);
    auto out = static_cast<T*>(y);
    if (sms <= 0) sms = 148;
#define WQ_BULK(MT, ROWS) return launch_bulk_shape<T, MT, ROWS>(xs, ldx, w, sw, b, r, rs, out, m, n, k, sms, stream)
    switch (tokens_blocks(m) * 100 + rows) {
        case 108: WQ_BULK(1, 8);
        case 116: WQ_BULK(1, 16);
        case 132: WQ_BULK(1, 32);
        case 208: WQ_BULK(2, 8);
        case 216: WQ_BULK(2, 16);
        case 232: WQ_BULK(2, 32);
    }
#undef WQ_BULK
    return -2;
}

template <class T, int ROWS>
static int launch_planes_shape(const int8_t* planes, const float* scales, const int8_t* w, const float* sw, const T* bias, const T* residual,
                               const T* rscale, T* y, int m, int n, int k, int sms, cudaStream_t stream) {
    using S = BulkShape<1, ROWS>;
    auto kernel = stream_planes<T, ROWS>;
    static bool configured[64] = {};
    int device = 0;
    cudaGetDevice(&device);
    if (device < 0 || device >= 64 || !configured[device]) {
        const cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, S::kSmemBytes);
        if (e != cudaSuccess) return int(e);
        if (device >= 0 && device < 64) configured[device] = true;
    }
    CUtensorMap map_w;
    if (!make_byte_matrix_map(&map_w, w, n, k, S::kSegment, ROWS)) return int(cudaErrorNotSupported);
    const int items = (n + ROWS - 1) / ROWS;
    // launched behind the split: set-up and the first weight requests run under its tail
    const cudaError_t launched = launch_after_previous(kernel, dim3(items < sms ? items : sms), dim3(kBulkThreads), size_t(S::kSmemBytes), stream, map_w, planes, scales,
                                                       sw, bias, residual, rscale, y, m, n, k);
    return int(launched != cudaSuccess ? launched : cudaGetLastError());
}

// The digit planes of the activations into `workspace`, then the INT8 tensor-core kernel.
template <class T>
static int launch_planes(const void* x, int64_t ldx, const int8_t* w, const float* sw, const void* bias, const void* residual, const void* rscale,
                         void* y, int m, int n, int k, int rows, int sms, void* workspace, cudaStream_t stream) {
    int8_t* planes = static_cast<int8_t*>(workspace);
    float* scales = reinterpret_cast<float*>(planes + int64_t(kPlaneTokens) * 3 * k);
    const int units = (k / kPlaneRun) * kPlaneTokens;
    const cudaError_t split = launch_after_previous(split_planes<T>, dim3((units + 7) / 8), dim3(256), size_t(0), stream, static_cast<const T*>(x), ldx, planes, scales, m, k);
    if (split != cudaSuccess) return int(split);
    auto b = static_cast<const T*>(bias), r = static_cast<const T*>(residual), rs = static_cast<const T*>(rscale);
    auto out = static_cast<T*>(y);
    if (sms <= 0) sms = 148;
    if (rows == 8) return launch_planes_shape<T, 8>(planes, scales, w, sw, b, r, rs, out, m, n, k, sms, stream);
    if (rows == 16) return launch_planes_shape<T, 16>(planes, scales, w, sw, b, r, rs, out, m, n, k, sms, stream);
    return launch_planes_shape<T, 32>(planes, scales, w, sw, b, r, rs, out, m, n, k, sms, stream);
}

// Status of the streaming kernels on the current device: 0, or 1 when a wait for weight data gave up; clears it.
int stream_status_take() {
    int code = 0;
    const int zero = 0;
    if (cudaMemcpyFromSymbol(&code, g_stream_status, sizeof(int)) != cudaSuccess) return -1;
    if (code) cudaMemcpyToSymbol(g_stream_status, &zero, sizeof(int));
    const int tensor_core_kernel = stream_tc_status_take();
    if (tensor_core_kernel < 0) return -1;
    return code ? code : tensor_core_kernel;
}

static int device_sms() {
    int device = 0, sms = 148;
    cudaGetDevice(&device);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device);
    return sms;
}

}  // namespace wq

using namespace wq;

// Bytes of workspace wq8_stream_planes needs for this shape, 0 when the shape is not one of its own (more than 8 tokens, K not a
// multiple of 128, or too few K segments for the 16 warps).
WQ_API int64_t wq8_stream_planes_workspace(int m, int n, int k, int sms) {
    if (m <= 0 || m > kPlaneTokens || n <= 0 || k <= 0 || k % kPlaneRun || !plan_bulk(m, n, k, sms)) return 0;
    return int64_t(kPlaneTokens) * 3 * k + int64_t(k / kPlaneRun) * kPlaneTokens * 4;
}

// Weight-only INT8 linear for at most 8 tokens with the activations split into INT8 digit planes (see stream_planes): the weights go into
// INT8 tensor-core MMAs as they are.  workspace: wq8_stream_planes_workspace() bytes, 16-byte aligned.  Values: FP32 sums of exact
// INT32 dot products per 128 values of K; an activation more than 2^14 times smaller than the largest of its 128 is rounded to the
// nearest 2^-21 of that largest value's power of two (relative error of the whole product below 2^-21 per run).
WQ_API int wq8_stream_planes(const void* x, int64_t ldx, const int8_t* w, const float* sw, const void* bias, const void* residual, const void* rscale,
                             void* y, int m, int n, int k, int dtype, int sms, void* workspace, cudaStream_t stream) {
    if (m <= 0 || n <= 0) return 0;
    if (dtype != 0 && dtype != 1) return -1;
    if (m > kPlaneTokens || k <= 0 || k % kPlaneRun || ldx % 4 || (reinterpret_cast<uintptr_t>(x) & 7) || (reinterpret_cast<uintptr_t>(w) & 15) || !workspace ||
        (reinterpret_cast<uintptr_t>(workspace) & 15))
        return -2;
    const int rows = plan_bulk(m, n, k, sms);
    if (!rows) return -2;
    if (dtype == 0) return launch_planes<__half>(x, ldx, w, sw, bias, residual, rscale, y, m, n, k, rows, sms, workspace, stream);
    return launch_planes<bf16>(x, ldx, w, sw, bias, residual, rscale, y, m, n, k, rows, sms, workspace, stream);
}

// The tensor-core kernel takes every shape with K a multiple of 128 and at most 1024 channel tiles (the counter buffer callers keep).
static int64_t tensor_core_scratch(int m, int n, int k, int sms, int64_t* counter_bytes) {
    const int64_t bytes = stream_tc_workspace(m, n, k, sms, counter_bytes);
    return bytes && *counter_bytes <= 4096 ? bytes : 0;
}

WQ_API void wq8_small_workspace(int m, int n, int k, int sms, int64_t* sizes) {
    if (const int64_t bytes = tensor_core_scratch(m, n, k, sms, &sizes[1])) {
        sizes[0] = bytes;
        return;
    }
    const DirectPlan p = plan_direct(m, n, k, sms, true);
    sizes[0] = direct_slot_bytes(p);
    sizes[1] = p.splits > 1 ? 4 * int64_t(p.ctas) : 0;
}

WQ_API int wq8_small(const void* x, int64_t ldx, const int8_t* w, const float* sw, const void* bias, const void* residual, const void* rscale, void* y,
                     int m, int n, int k, int dtype, int sms, float* slots, int* counters, cudaStream_t stream) {
    if (m <= 0 || n <= 0) return 0;
    // every kernel below reads x and w with 16-byte loads (or TMA boxes): unaligned operands are refused, never launched
    if (k <= 0 || k % 64 || m > 32 || ldx % 8 || (reinterpret_cast<uintptr_t>(x) & 15) || (reinterpret_cast<uintptr_t>(w) & 15)) return -2;
    if (dtype != 0 && dtype != 1) return -1;
    // with the caller's scratch: the tensor-core kernel (digit planes, stream-K over all SMs)
    int64_t counter_bytes = 0;
    if (slots && counters && (reinterpret_cast<uintptr_t>(slots) & 255) == 0 && tensor_core_scratch(m, n, k, sms, &counter_bytes))
        return stream_tc_launch(x, ldx, w, sw, bias, residual, rscale, y, m, n, k, dtype, sms, slots, counters, stream);
    const int rows = plan_bulk(m, n, k, sms);
    if (rows && dtype == 0) return launch_bulk<__half>(x, ldx, w, sw, bias, residual, rscale, y, m, n, k, rows, sms, stream);
    if (rows) return launch_bulk<bf16>(x, ldx, w, sw, bias, residual, rscale, y, m, n, k, rows, sms, stream);
    const DirectPlan p = plan_direct(m, n, k, sms, slots && counters);
    if (dtype == 0) return launch_direct<__half>(x, ldx, w, sw, bias, residual, rscale, y, m, n, k, p, slots, counters, stream);
    return launch_direct<bf16>(x, ldx, w, sw, bias, residual, rscale, y, m, n, k, p, slots, counters, stream);
}

WQ_API int wq8_gemv_lines(const void* x, int64_t ldx, const int8_t* w, const float* sw, const void* bias, const void* residual, const void* rscale,
                          void* y, int m, int n, int k, int dtype, cudaStream_t stream) {
    if (m <= 0 || n <= 0) return 0;
    if (m > 4 || k <= 0 || k % 4) return -2;
    if (dtype != 0 && dtype != 1) return -1;
    const bool tensor_cores = k % 64 == 0 && ldx % 8 == 0 && (reinterpret_cast<uintptr_t>(x) & 15) == 0 && (reinterpret_cast<uintptr_t>(w) & 15) == 0;
    if (tensor_cores) {
        const int sms = device_sms(), rows = plan_bulk(m, n, k, sms);
        if (rows && dtype == 0) return launch_bulk<__half>(x, ldx, w, sw, bias, residual, rscale, y, m, n, k, rows, sms, stream);
        if (rows) return launch_bulk<bf16>(x, ldx, w, sw, bias, residual, rscale, y, m, n, k, rows, sms, stream);
    }
    // the direct kernel reads four weight bytes and four activations (8 bytes) per step
    if (ldx % 4 || (reinterpret_cast<uintptr_t>(x) & 7) || (reinterpret_cast<uintptr_t>(w) & 3)) return -2;
    const DirectPlan p = plan_direct(m, n, k, 0, false);
    if (dtype == 0) return launch_direct<__half>(x, ldx, w, sw, bias, residual, rscale, y, m, n, k, p, nullptr, nullptr, stream);
    return launch_direct<bf16>(x, ldx, w, sw, bias, residual, rscale, y, m, n, k, p, nullptr, nullptr, stream);
}

// ---------------------------------------------------------------------------------------------------------------------
// wq8_small without caller scratch.
//
// wq8_small splits K across CTAs when few output channels would leave SMs idle, and the caller has to hand it the partial-sum slots
// and the tile counters for that.  Some callers have no way to provide them: a host that drives this library through plain ctypes / FFI
// with buffers it was given (no allocator of its own on the device), a serving loop that runs under a fixed memory budget and may not
// grow it per request, code that runs while a CUDA graph is being captured or inside a real-time section where cudaMalloc (which
// synchronizes and may fail) is off limits.  For them the scratch lives here, in device memory that belongs to the library: every GPU
// that loads the library holds kStaticScratchBytes (8 MiB + 4 KiB) of it until the process exits.
//
// The array's name is only a handle on the host: a kernel must be given the device address, which cudaGetSymbolAddress returns for
// the device that is current at the time.  It is looked up once per device, on the first call made with that device current -- that
// first call should therefore happen before any stream capture starts -- and cached.
// ---------------------------------------------------------------------------------------------------------------------
namespace wq {

constexpr int64_t kStaticSlotBytes = 8 << 20;     // digit planes and partial sums of the tensor-core kernel: 32 tokens, K up to 32768, 148 SMs
constexpr int64_t kStaticCounterBytes = 4 << 10;  // one counter per tile, at most 1024 tiles
constexpr int64_t kStaticScratchBytes = kStaticSlotBytes + kStaticCounterBytes;
static __device__ __align__(256) unsigned char static_scratch[kStaticScratchBytes];

// Device address of static_scratch on the current device (nullptr and *error set when the lookup fails).
static unsigned char* static_scratch_address(int* error) {
    static unsigned char* known[64] = {};
    int device = 0;
    cudaError_t code = cudaGetDevice(&device);
    if (code != cudaSuccess || device < 0 || device >= 64) {
        *error = code != cudaSuccess ? int(code) : -2;
        return nullptr;
    }
    if (!known[device]) {
        void* address = nullptr;
        code = cudaGetSymbolAddress(&address, static_scratch);
        if (code != cudaSuccess || !address) {
            *error = code != cudaSuccess ? int(code) : int(cudaErrorInvalidSymbol);
            return nullptr;
        }
        known[device] = static_cast<unsigned char*>(address);
    }
    return known[device];
}

}  // namespace wq

// Same linear as wq8_small (at most 32 tokens, K multiple of 64, x rows and w 16-byte aligned) with the same kernel choice, hence the
// same values bit for bit; no scratch arguments and no allocation of any kind: the digit planes, partial sums and tile counters that
// wq8_small takes from its caller live in the library's own static device buffer.
// Returns -5 when the shape's scratch would not fit that buffer (use wq8_small with caller scratch then); other codes as wq8_small.
// Calls share the one buffer per device: two calls whose kernels may overlap on the GPU (different streams, or one stream of a graph with
// parallel branches) race on it -- keep them on one stream, or give the others caller scratch through wq8_small.  The buffer keeps what
// the last call left in it; the counters are cleared on the stream in front of every launch, everything else is written before it is read.
WQ_API int wq8_small_static(const void* x, int64_t ldx, const int8_t* w, const float* sw, const void* bias, const void* residual, const void* rscale,
                            void* y, int m, int n, int k, int dtype, int sms, cudaStream_t stream) {
    if (m <= 0 || n <= 0) return 0;
    if (k <= 0 || k % 64 || m > 32 || ldx % 8 || (reinterpret_cast<uintptr_t>(x) & 15) || (reinterpret_cast<uintptr_t>(w) & 15)) return -2;
    if (dtype != 0 && dtype != 1) return -1;
    // how much scratch the kernel wq8_small would pick needs
    int64_t counter_bytes = 0;
    const int64_t tensor_core_bytes = tensor_core_scratch(m, n, k, sms, &counter_bytes);
    const int rows = tensor_core_bytes ? 0 : plan_bulk(m, n, k, sms);
    const DirectPlan p = plan_direct(m, n, k, sms, true);
    int64_t slot_bytes = tensor_core_bytes;
    if (!tensor_core_bytes && !rows && p.splits > 1) {
        slot_bytes = direct_slot_bytes(p);
        counter_bytes = 4 * int64_t(p.ctas);
    }
    float* slots = nullptr;
    int* counters = nullptr;
    if (slot_bytes) {
        if (slot_bytes > kStaticSlotBytes || counter_bytes > kStaticCounterBytes) return -5;
        int error = 0;
        unsigned char* scratch = static_scratch_address(&error);
        if (!scratch) return error;
        slots = reinterpret_cast<float*>(scratch);
        counters = reinterpret_cast<int*>(scratch + kStaticSlotBytes);
        const cudaError_t cleared = cudaMemsetAsync(counters, 0, size_t(counter_bytes), stream);
        if (cleared != cudaSuccess) return int(cleared);
    }
    if (tensor_core_bytes) return stream_tc_launch(x, ldx, w, sw, bias, residual, rscale, y, m, n, k, dtype, sms, slots, counters, stream);
    if (rows && dtype == 0) return launch_bulk<__half>(x, ldx, w, sw, bias, residual, rscale, y, m, n, k, rows, sms, stream);
    if (rows) return launch_bulk<bf16>(x, ldx, w, sw, bias, residual, rscale, y, m, n, k, rows, sms, stream);
    if (dtype == 0) return launch_direct<__half>(x, ldx, w, sw, bias, residual, rscale, y, m, n, k, p, slots, counters, stream);
    return launch_direct<bf16>(x, ldx, w, sw, bias, residual, rscale, y, m, n, k, p, slots, counters, stream);
}
