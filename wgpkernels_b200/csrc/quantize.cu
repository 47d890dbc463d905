// Activation preparation kernels: per-(row, 128-block) INT8 quantizer, row / hi-lo INT8 quantizer, few-token transform,
// ConvRot group rotation.  All of them stream the activation once from HBM with 16-byte loads and fuse the input operation
// (rms_norm / swiglu / gelu-tanh) in FP32.  Results are bit-for-bit those of the reference library
// (wgpkernels/int8/int8_gemm.cu:253-485, 1814-1831 of WGPKernels): same FP32 expressions, same fixed-order reductions.
#include "common.cuh"

namespace wq {

// Row window of the *_at entry points: the input rows start at row first + counter[0] * step of x, the counter being read on the GPU
// when the kernel runs (a CUDA graph replays the launch while its loop counter advances).  No counter: row 0.
struct RowShift { const long long* counter; long long first, step; };
template <class T> WQ_DEVICE const T* first_row(const T* x, int64_t ldx, const RowShift& shift) {
    return shift.counter ? x + (shift.first + __ldg(shift.counter) * shift.step) * ldx : x;
}

// ---- one 256-element chunk -> two 128-element blocks (16 lanes each): absmax, scale, INT8 codes --------------------------
template <int GROUP, bool PAIRS = false>
WQ_DEVICE void store_chunk_as_blocks(const float* v, int lane, int64_t row, int base, int k, int kblocks, int8_t* __restrict__ q,
                                     float* __restrict__ scale) {
    float amax = 0.f;
#pragma unroll
    for (int j = 0; j < 8; ++j) amax = fmaxf(amax, fabsf(v[j]));
#pragma unroll
    for (int d = 8; d > 0; d >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, d));  // stays inside each half warp
    // every lane holds its block's absmax: all of them do the division (the instructions issue once per warp either way; a branch for the
    // first lane of a block and a shuffle back would only add to them), the block's first lane stores the scale
    const float inv = amax > 0.f ? 127.f / amax : 0.f;
    const int block = base / kBlockK + (lane >> 4);
    if ((lane & 15) == 0 && block < kblocks) scale[row * kblocks + block] = amax * group_norm<GROUP>() / 127.f;
    const int col = base + lane * 8;
    if (col < k) {
        int c[8];
        if constexpr (PAIRS) {  // two-wide multiplies (each half rounds as the scalar multiply does): fewer instructions where the input
                                // operation leaves registers to pair; the row kernels, short of registers, keep the scalar form
            const float2 inverse = make_float2(inv, inv);
#pragma unroll
            for (int j = 0; j < 8; j += 2) {
                const float2 scaled = __fmul2_rn(make_float2(v[j], v[j + 1]), inverse);
                c[j] = __float2int_rn(scaled.x);
                c[j + 1] = __float2int_rn(scaled.y);
            }
        } else {
#pragma unroll
            for (int j = 0; j < 8; ++j) c[j] = __float2int_rn(v[j] * inv);
        }
        *reinterpret_cast<uint2*>(q + row * k + col) = make_uint2(pack_bytes(c[0], c[1], c[2], c[3]), pack_bytes(c[4], c[5], c[6], c[7]));
    }
}

// RMSNorm needs the row's sum of squares first: one CTA per row.  CPW > 0: the row (K <= 2048 * CPW) stays in registers, one read.
// CPW == 0: any K, the row is read twice (the second read comes from L2).
// Sum of squares: thread (warp w, lane l) accumulates fmaf(v, v, ss) over chunks w, w + 8, ... in order; then the ordered CTA sum.
template <class T, int GROUP, int CPW>
__global__ void __launch_bounds__(kRowThreads, CPW > 0 && CPW <= 4 ? 6 : 1) quantize_blocks_rms(const T* __restrict__ x, int8_t* __restrict__ q, float* __restrict__ scale, int m, int k,
                                                                   int64_t ldx, const T* __restrict__ act_weight, float eps, RowShift shift) {
    __shared__ float slots[9];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int64_t row = blockIdx.x;
    const T* src = first_row(x, ldx, shift) + row * ldx;
    const int kblocks = (k + kBlockK - 1) / kBlockK;
    float ss = 0.f;
    if constexpr (CPW > 0) {
        static_assert(sizeof(T) == 2, "rms_norm takes 16-bit inputs");
        float v[CPW][8];
#pragma unroll
        for (int i = 0; i < CPW; ++i) {
            const int col = (warp + 8 * i) * kChunk + lane * 8;
            load_eight(src + col, v[i], col < k);
        }
#pragma unroll
        for (int i = 0; i < CPW; ++i)
#pragma unroll
            for (int j = 0; j < 8; ++j) ss = fmaf(v[i][j], v[i][j], ss);
        const float inv_rms = cta_inverse_rms(ss, slots, k, eps);
#pragma unroll
        for (int i = 0; i < CPW; ++i) {
            const int base = (warp + 8 * i) * kChunk;
            if (base < k) {  // warp-uniform
                // the RMSNorm weights of the chunk come from L1 / L2 when they are needed: held from before the reduction they would cost the
                // registers that let six CTAs share an SM (the kernel is bound by instruction issue: occupancy is what it needs)
                const uint4 raw = (act_weight && base + lane * 8 < k) ? __ldg(reinterpret_cast<const uint4*>(act_weight + base + lane * 8)) : make_uint4(0u, 0u, 0u, 0u);
                float w[8];
                unpack_pair<T>(raw.x, w[0], w[1]);
                unpack_pair<T>(raw.y, w[2], w[3]);
                unpack_pair<T>(raw.z, w[4], w[5]);
                unpack_pair<T>(raw.w, w[6], w[7]);
#pragma unroll
                for (int j = 0; j < 8; ++j) v[i][j] = v[i][j] * inv_rms * (act_weight ? w[j] : 1.f);
                rotate_chunk<GROUP>(v[i]);
                store_chunk_as_blocks<GROUP>(v[i], lane, row, base, k, kblocks, q, scale);
            }
        }
    } else {
        for (int base = warp * kChunk; base < k; base += 8 * kChunk) {
            float v[8];
            load_eight(src + base + lane * 8, v, base + lane * 8 < k);
#pragma unroll
            for (int j = 0; j < 8; ++j) ss = fmaf(v[j], v[j], ss);
        }
        const float inv_rms = cta_inverse_rms(ss, slots, k, eps);
        for (int base = warp * kChunk; base < k; base += 8 * kChunk) {
            float v[8];
            const bool valid = base + lane * 8 < k;
            load_eight(src + base + lane * 8, v, valid);
            scale_by_rms(v, inv_rms, act_weight, base + lane * 8, valid);
            rotate_chunk<GROUP>(v);
            store_chunk_as_blocks<GROUP>(v, lane, row, base, k, kblocks, q, scale);
        }
    }
}

// No row statistic: every (row, 256-element chunk) is independent.  One warp per item and nothing else: the row is the grid's y
// coordinate and the chunk comes from x, so there is no loop, no division and no bookkeeping -- the input operations (the accurate
// tanhf / expf of gelu and swiglu) are what these launches spend their time on, and every register and instruction beside them
// costs occupancy.  The host launches batches of at most 65535 rows (the grid's y limit).
template <class T, int GROUP, int ACT>
__global__ void __launch_bounds__(256) quantize_blocks_items(const T* __restrict__ x, int8_t* __restrict__ q, float* __restrict__ scale, int64_t row0, int k,
                                                             int64_t ldx, RowShift shift) {
    const int lane = threadIdx.x & 31;
    const int base = (blockIdx.x * 8 + (threadIdx.x >> 5)) * kChunk;
    if (base >= k) return;
    const int kblocks = (k + kBlockK - 1) / kBlockK;
    const int64_t row = row0 + blockIdx.y;
    float v[8];
    load_op<T, ACT>(first_row(x, ldx, shift) + row * ldx, k, base + lane * 8, v, base + lane * 8 < k);
    rotate_chunk<GROUP>(v);
    store_chunk_as_blocks<GROUP, true>(v, lane, row, base, k, kblocks, q, scale);
}

// ---- row-wise INT8 (one scale per row), optional exact hi / lo split -----------------------------------------------------
template <bool HILO> WQ_DEVICE void store_row_codes(const float* v, float inv, int8_t* __restrict__ hi, int8_t* __restrict__ lo, int64_t offset) {
    int h[8], l[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
        const float t = v[j] * inv;
        h[j] = __float2int_rn(t);
        if (HILO) l[j] = __float2int_rn((t - float(h[j])) * 254.f);
    }
    *reinterpret_cast<uint2*>(hi + offset) = make_uint2(pack_bytes(h[0], h[1], h[2], h[3]), pack_bytes(h[4], h[5], h[6], h[7]));
    if (HILO) *reinterpret_cast<uint2*>(lo + offset) = make_uint2(pack_bytes(l[0], l[1], l[2], l[3]), pack_bytes(l[4], l[5], l[6], l[7]));
}

// Rows of up to 8192 values: five CTAs per SM (at most 51 registers per thread) -- these kernels are bound by instruction issue and by
// the latency of their two CTA-wide reductions, so resident warps count for more than registers.
template <class T, int GROUP, bool HILO, int ACT, int CPW>
__global__ void __launch_bounds__(kRowThreads, CPW > 0 && CPW <= 4 ? 5 : 1) quantize_rows(const T* __restrict__ x, int8_t* __restrict__ hi, int8_t* __restrict__ lo,
                                                             float* __restrict__ scale, int k, int64_t ldx, const T* __restrict__ act_weight, float eps,
                                                             RowShift shift) {
    __shared__ float sum_slots[9], max_slots[8];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int64_t row = blockIdx.x;
    const T* src = first_row(x, ldx, shift) + row * ldx;
    float amax = 0.f;
    if constexpr (CPW > 0) {
        float v[CPW][8];
#pragma unroll
        for (int i = 0; i < CPW; ++i) {
            const int col = (warp + 8 * i) * kChunk + lane * 8;
            load_op<T, ACT>(src, k, col, v[i], col < k);
        }
        if constexpr (ACT == kActRms) {
            float ss = 0.f;
#pragma unroll
            for (int i = 0; i < CPW; ++i)
#pragma unroll
                for (int j = 0; j < 8; ++j) ss = fmaf(v[i][j], v[i][j], ss);
            const float inv_rms = cta_inverse_rms(ss, sum_slots, k, eps);
#pragma unroll
            for (int i = 0; i < CPW; ++i) {
                const int col = (warp + 8 * i) * kChunk + lane * 8;
                scale_by_rms(v[i], inv_rms, act_weight, col, col < k);
            }
        }
#pragma unroll
        for (int i = 0; i < CPW; ++i) {
            rotate_chunk<GROUP>(v[i]);
#pragma unroll
            for (int j = 0; j < 8; ++j) amax = fmaxf(amax, fabsf(v[i][j]));
        }
        amax = cta_max(amax, max_slots);
        const float inv = amax > 0.f ? 127.f / amax : 0.f;
        if (threadIdx.x == 0) scale[row] = amax * group_norm<GROUP>() / 127.f;
#pragma unroll
        for (int i = 0; i < CPW; ++i) {
            const int col = (warp + 8 * i) * kChunk + lane * 8;
            if (col < k) store_row_codes<HILO>(v[i], inv, hi, lo, row * k + col);
        }
    } else {
        float inv_rms = 1.f;
        if constexpr (ACT == kActRms) {
            float ss = 0.f;
            for (int base = warp * kChunk; base < k; base += 8 * kChunk) {
                float v[8];
                load_eight(src + base + lane * 8, v, base + lane * 8 < k);
#pragma unroll
                for (int j = 0; j < 8; ++j) ss = fmaf(v[j], v[j], ss);
            }
            inv_rms = cta_inverse_rms(ss, sum_slots, k, eps);
        }
        for (int base = warp * kChunk; base < k; base += 8 * kChunk) {
            float v[8];
            const bool valid = base + lane * 8 < k;
            load_op<T, ACT>(src, k, base + lane * 8, v, valid);
            if constexpr (ACT == kActRms) scale_by_rms(v, inv_rms, act_weight, base + lane * 8, valid);
            rotate_chunk<GROUP>(v);
#pragma unroll
            for (int j = 0; j < 8; ++j) amax = fmaxf(amax, fabsf(v[j]));
        }
        amax = cta_max(amax, max_slots);
        const float inv = amax > 0.f ? 127.f / amax : 0.f;
        if (threadIdx.x == 0) scale[row] = amax * group_norm<GROUP>() / 127.f;
        for (int base = warp * kChunk; base < k; base += 8 * kChunk) {
            float v[8];
            const bool valid = base + lane * 8 < k;
            load_op<T, ACT>(src, k, base + lane * 8, v, valid);
            if constexpr (ACT == kActRms) scale_by_rms(v, inv_rms, act_weight, base + lane * 8, valid);
            rotate_chunk<GROUP>(v);
            if (valid) store_row_codes<HILO>(v, inv, hi, lo, row * k + base + lane * 8);
        }
    }
}

// ---- few-token paths: op(x), rotated, rounded once to T ---------------------------------------------------------------
template <class T, int GROUP, int ACT>
__global__ void __launch_bounds__(kRowThreads) transform_rows(const T* __restrict__ x, T* __restrict__ out, int k, int64_t ldx,
                                                              const T* __restrict__ act_weight, float eps) {
    __shared__ float slots[9];
    dependents_may_start();  // a few-token linear follows: its digit split may be set up while these rows are transformed
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int64_t row = blockIdx.x;
    const T* src = x + row * ldx;
    float inv_rms = 1.f;
    if constexpr (ACT == kActRms) {
        float ss = 0.f;
        for (int base = warp * kChunk; base < k; base += 8 * kChunk) {
            float v[8];
            load_eight(src + base + lane * 8, v, base + lane * 8 < k);
#pragma unroll
            for (int j = 0; j < 8; ++j) ss = fmaf(v[j], v[j], ss);
        }
        inv_rms = cta_inverse_rms(ss, slots, k, eps);
    }
    constexpr float norm = group_norm<GROUP>();
    // gridDim.y CTAs share a row when no row statistic is needed: with one or a few rows every warp then has one chunk and one trip to
    // memory instead of a chain of them
    for (int base = (blockIdx.y * 8 + warp) * kChunk; base < k; base += gridDim.y * 8 * kChunk) {
        float v[8];
        const bool valid = base + lane * 8 < k;
        load_op<T, ACT>(src, k, base + lane * 8, v, valid);
        if constexpr (ACT == kActRms) scale_by_rms(v, inv_rms, act_weight, base + lane * 8, valid);
        rotate_chunk<GROUP>(v);
        if (valid) {
            uint4 packed;
            packed.x = pack_pair<T>(v[0] * norm, v[1] * norm);
            packed.y = pack_pair<T>(v[2] * norm, v[3] * norm);
            packed.z = pack_pair<T>(v[4] * norm, v[5] * norm);
            packed.w = pack_pair<T>(v[6] * norm, v[7] * norm);
            *reinterpret_cast<uint4*>(out + row * k + base + lane * 8) = packed;
        }
    }
}

// Standalone rotation (a warp per 256-element chunk, persistent): out = T(rotated * 1 / sqrt(GROUP)).
template <class T, int GROUP>
__global__ void __launch_bounds__(256) rotate_groups(const T* __restrict__ x, T* __restrict__ out, int m, int k, int64_t ldx) {
    const int lane = threadIdx.x & 31;
    const int chunks = (k + kChunk - 1) / kChunk;
    const int64_t items = int64_t(m) * chunks, stride = int64_t(gridDim.x) * 8;
    constexpr float norm = group_norm<GROUP>();
    for (int64_t item = int64_t(blockIdx.x) * 8 + (threadIdx.x >> 5); item < items; item += stride) {
        const int64_t row = item / chunks;
        const int col = int(item % chunks) * kChunk + lane * 8;
        float v[8];
        load_eight(x + row * ldx + col, v, col < k);
        rotate_chunk<GROUP>(v);
        if (col < k) {
            uint4 packed;
            packed.x = pack_pair<T>(v[0] * norm, v[1] * norm);
            packed.y = pack_pair<T>(v[2] * norm, v[3] * norm);
            packed.z = pack_pair<T>(v[4] * norm, v[5] * norm);
            packed.w = pack_pair<T>(v[6] * norm, v[7] * norm);
            *reinterpret_cast<uint4*>(out + row * k + col) = packed;
        }
    }
}

// ---- host dispatch ----------------------------------------------------------------------------------------------------
static int persistent_ctas(int64_t warps_of_work) {
    int device = 0, sms = 148;
    cudaGetDevice(&device);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device);
    const int64_t ctas = (warps_of_work + 7) / 8, cap = int64_t(sms) * 8;  // 8 CTAs of 256 threads fill an SM
    return int(ctas < cap ? (ctas < 1 ? 1 : ctas) : cap);
}

template <class T, int GROUP, int ACT>
static int launch_blocks(const void* x, int8_t* q, float* scale, int m, int k, int64_t ldx, const void* act_weight, float eps, const RowShift& shift,
                         cudaStream_t stream) {
    auto src = static_cast<const T*>(x);
    auto aw = static_cast<const T*>(act_weight);
    if constexpr (ACT == kActRms) {
        if (k <= 2048) quantize_blocks_rms<T, GROUP, 1><<<m, kRowThreads, 0, stream>>>(src, q, scale, m, k, ldx, aw, eps, shift);
        else if (k <= 4096) quantize_blocks_rms<T, GROUP, 2><<<m, kRowThreads, 0, stream>>>(src, q, scale, m, k, ldx, aw, eps, shift);
        else if (k <= 8192) quantize_blocks_rms<T, GROUP, 4><<<m, kRowThreads, 0, stream>>>(src, q, scale, m, k, ldx, aw, eps, shift);
        else if (k <= 16384) quantize_blocks_rms<T, GROUP, 8><<<m, kRowThreads, 0, stream>>>(src, q, scale, m, k, ldx, aw, eps, shift);
        else quantize_blocks_rms<T, GROUP, 0><<<m, kRowThreads, 0, stream>>>(src, q, scale, m, k, ldx, aw, eps, shift);
    } else {
        const int chunks = (k + kChunk - 1) / kChunk;
        for (int64_t row0 = 0; row0 < m; row0 += 65535) {
            const dim3 grid((chunks + 7) / 8, unsigned(m - row0 < 65535 ? m - row0 : 65535));
            quantize_blocks_items<T, GROUP, ACT><<<grid, 256, 0, stream>>>(src, q, scale, row0, k, ldx, shift);
        }
    }
    return int(cudaGetLastError());
}

template <class T, int ACT>
static int blocks_by_group(const void* x, int8_t* q, float* scale, int m, int k, int64_t ldx, int group, const void* aw, float eps, const RowShift& shift,
                           cudaStream_t stream) {
    switch (group) {
        case 0: return launch_blocks<T, 0, ACT>(x, q, scale, m, k, ldx, aw, eps, shift, stream);
        case 16: return launch_blocks<T, 16, ACT>(x, q, scale, m, k, ldx, aw, eps, shift, stream);
        case 64: return launch_blocks<T, 64, ACT>(x, q, scale, m, k, ldx, aw, eps, shift, stream);
        case 256: return launch_blocks<T, 256, ACT>(x, q, scale, m, k, ldx, aw, eps, shift, stream);
    }
    return -1;
}

template <class T>
static int blocks_by_act(const void* x, int8_t* q, float* scale, int m, int k, int64_t ldx, int group, int act, const void* aw, float eps,
                         const RowShift& shift, cudaStream_t stream) {
    switch (act) {
        case kActNone: return blocks_by_group<T, kActNone>(x, q, scale, m, k, ldx, group, aw, eps, shift, stream);
        case kActRms: return blocks_by_group<T, kActRms>(x, q, scale, m, k, ldx, group, aw, eps, shift, stream);
        case kActSwiglu: return blocks_by_group<T, kActSwiglu>(x, q, scale, m, k, ldx, group, aw, eps, shift, stream);
        case kActGelu: return blocks_by_group<T, kActGelu>(x, q, scale, m, k, ldx, group, aw, eps, shift, stream);
    }
    return -1;
}

template <class T, int GROUP, bool HILO, int ACT>
static int launch_rows(const void* x, int8_t* hi, int8_t* lo, float* scale, int m, int k, int64_t ldx, const void* act_weight, float eps,
                       const RowShift& shift, cudaStream_t stream) {
    auto src = static_cast<const T*>(x);
    auto aw = static_cast<const T*>(act_weight);
    if (k <= 2048) quantize_rows<T, GROUP, HILO, ACT, 1><<<m, kRowThreads, 0, stream>>>(src, hi, lo, scale, k, ldx, aw, eps, shift);
    else if (k <= 4096) quantize_rows<T, GROUP, HILO, ACT, 2><<<m, kRowThreads, 0, stream>>>(src, hi, lo, scale, k, ldx, aw, eps, shift);
    else if (k <= 8192) quantize_rows<T, GROUP, HILO, ACT, 4><<<m, kRowThreads, 0, stream>>>(src, hi, lo, scale, k, ldx, aw, eps, shift);
    else if (k <= 16384) quantize_rows<T, GROUP, HILO, ACT, 8><<<m, kRowThreads, 0, stream>>>(src, hi, lo, scale, k, ldx, aw, eps, shift);
    else quantize_rows<T, GROUP, HILO, ACT, 0><<<m, kRowThreads, 0, stream>>>(src, hi, lo, scale, k, ldx, aw, eps, shift);
    return int(cudaGetLastError());
}

template <class T, bool HILO, int ACT>
static int rows_by_group(const void* x, int8_t* hi, int8_t* lo, float* scale, int m, int k, int64_t ldx, int group, const void* aw, float eps,
                         const RowShift& shift, cudaStream_t stream) {
    switch (group) {
        case 0: return launch_rows<T, 0, HILO, ACT>(x, hi, lo, scale, m, k, ldx, aw, eps, shift, stream);
        case 16: return launch_rows<T, 16, HILO, ACT>(x, hi, lo, scale, m, k, ldx, aw, eps, shift, stream);
        case 64: return launch_rows<T, 64, HILO, ACT>(x, hi, lo, scale, m, k, ldx, aw, eps, shift, stream);
        case 256: return launch_rows<T, 256, HILO, ACT>(x, hi, lo, scale, m, k, ldx, aw, eps, shift, stream);
    }
    return -1;
}

template <class T, bool HILO>
static int rows_by_act(const void* x, int8_t* hi, int8_t* lo, float* scale, int m, int k, int64_t ldx, int group, int act, const void* aw, float eps,
                       const RowShift& shift, cudaStream_t stream) {
    switch (act) {
        case kActNone: return rows_by_group<T, HILO, kActNone>(x, hi, lo, scale, m, k, ldx, group, aw, eps, shift, stream);
        case kActRms: return rows_by_group<T, HILO, kActRms>(x, hi, lo, scale, m, k, ldx, group, aw, eps, shift, stream);
        case kActSwiglu: return rows_by_group<T, HILO, kActSwiglu>(x, hi, lo, scale, m, k, ldx, group, aw, eps, shift, stream);
        case kActGelu: return rows_by_group<T, HILO, kActGelu>(x, hi, lo, scale, m, k, ldx, group, aw, eps, shift, stream);
    }
    return -1;
}

template <class T, int GROUP>
static int launch_transform(const void* x, void* out, int m, int k, int64_t ldx, int act, const void* act_weight, float eps, cudaStream_t stream) {
    auto src = static_cast<const T*>(x);
    auto aw = static_cast<const T*>(act_weight);
    auto dst = static_cast<T*>(out);
    // few rows: the CTAs of a row take its chunks in turn (not with rms_norm, whose row sum is formed inside one CTA)
    const int chunk_groups = (k + 8 * kChunk - 1) / (8 * kChunk);
    const dim3 grid(m, m < 64 ? (chunk_groups < 64 ? chunk_groups : 64) : 1);
    switch (act) {
        case kActNone: transform_rows<T, GROUP, kActNone><<<grid, kRowThreads, 0, stream>>>(src, dst, k, ldx, aw, eps); break;
        case kActRms: transform_rows<T, GROUP, kActRms><<<m, kRowThreads, 0, stream>>>(src, dst, k, ldx, aw, eps); break;
        case kActSwiglu: transform_rows<T, GROUP, kActSwiglu><<<grid, kRowThreads, 0, stream>>>(src, dst, k, ldx, aw, eps); break;
        case kActGelu: transform_rows<T, GROUP, kActGelu><<<grid, kRowThreads, 0, stream>>>(src, dst, k, ldx, aw, eps); break;
        default: return -1;
    }
    return int(cudaGetLastError());
}

template <class T>
static int transform_by_group(const void* x, void* out, int m, int k, int64_t ldx, int group, int act, const void* aw, float eps, cudaStream_t stream) {
    switch (group) {
        case 0: return launch_transform<T, 0>(x, out, m, k, ldx, act, aw, eps, stream);
        case 16: return launch_transform<T, 16>(x, out, m, k, ldx, act, aw, eps, stream);
        case 64: return launch_transform<T, 64>(x, out, m, k, ldx, act, aw, eps, stream);
        case 256: return launch_transform<T, 256>(x, out, m, k, ldx, act, aw, eps, stream);
    }
    return -1;
}

template <class T>
static int rotate_by_group(const void* x, void* out, int m, int k, int64_t ldx, int group, cudaStream_t stream) {
    auto src = static_cast<const T*>(x);
    auto dst = static_cast<T*>(out);
    const int ctas = persistent_ctas(int64_t(m) * ((k + kChunk - 1) / kChunk));
    if (group == 16) rotate_groups<T, 16><<<ctas, 256, 0, stream>>>(src, dst, m, k, ldx);
    else if (group == 64) rotate_groups<T, 64><<<ctas, 256, 0, stream>>>(src, dst, m, k, ldx);
    else if (group == 256) rotate_groups<T, 256><<<ctas, 256, 0, stream>>>(src, dst, m, k, ldx);
    else return -1;
    return int(cudaGetLastError());
}

}  // namespace wq

using namespace wq;

static int quantize_blocks_entry(const void* x, int8_t* q, float* scale, int m, int k, int64_t ldx, int dtype, int group, int act,
                                 const void* act_weight, float eps, const RowShift& shift, cudaStream_t stream) {
    if (m <= 0) return 0;
    if (k <= 0 || k % 8 || (group && k % group)) return -2;
    if (dtype == 0) return blocks_by_act<__half>(x, q, scale, m, k, ldx, group, act, act_weight, eps, shift, stream);
    if (dtype == 1) return blocks_by_act<bf16>(x, q, scale, m, k, ldx, group, act, act_weight, eps, shift, stream);
    if (dtype != 2 || act) return -1;
    return blocks_by_group<float, kActNone>(x, q, scale, m, k, ldx, group, nullptr, 0.f, shift, stream);
}

static int quantize_entry(const void* x, int8_t* hi, int8_t* lo, float* scale, int m, int k, int64_t ldx, int dtype, int group, int act,
                          const void* act_weight, float eps, const RowShift& shift, cudaStream_t stream) {
    if (m <= 0) return 0;
    if (k <= 0 || k % 8 || (group && k % group)) return -2;
    if (dtype == 0)
        return lo ? rows_by_act<__half, true>(x, hi, lo, scale, m, k, ldx, group, act, act_weight, eps, shift, stream)
                  : rows_by_act<__half, false>(x, hi, lo, scale, m, k, ldx, group, act, act_weight, eps, shift, stream);
    if (dtype == 1)
        return lo ? rows_by_act<bf16, true>(x, hi, lo, scale, m, k, ldx, group, act, act_weight, eps, shift, stream)
                  : rows_by_act<bf16, false>(x, hi, lo, scale, m, k, ldx, group, act, act_weight, eps, shift, stream);
    if (dtype != 2 || act) return -1;
    return lo ? rows_by_group<float, true, kActNone>(x, hi, lo, scale, m, k, ldx, group, nullptr, 0.f, shift, stream)
              : rows_by_group<float, false, kActNone>(x, hi, lo, scale, m, k, ldx, group, nullptr, 0.f, shift, stream);
}

WQ_API int wq8_quantize_blocks(const void* x, int8_t* q, float* scale, int m, int k, int64_t ldx, int dtype, int group, int act,
                               const void* act_weight, float eps, float* /*inv_rms: rows of any K are handled inside one kernel*/, cudaStream_t stream) {
    return quantize_blocks_entry(x, q, scale, m, k, ldx, dtype, group, act, act_weight, eps, RowShift{nullptr, 0, 0}, stream);
}

// wq8_quantize_blocks reading rows first + counter[0] * step ... of x (the outputs start at row 0): counter on the GPU, read at run time.
WQ_API int wq8_quantize_blocks_at(const void* x, int8_t* q, float* scale, int m, int k, int64_t ldx, int dtype, int group, int act,
                                  const void* act_weight, float eps, float* /*inv_rms*/, const long long* counter, long long first, long long step,
                                  cudaStream_t stream) {
    return quantize_blocks_entry(x, q, scale, m, k, ldx, dtype, group, act, act_weight, eps, RowShift{counter, first, step}, stream);
}

WQ_API int wq8_quantize(const void* x, int8_t* hi, int8_t* lo, float* scale, int m, int k, int64_t ldx, int dtype, int group, int act,
                        const void* act_weight, float eps, cudaStream_t stream) {
    return quantize_entry(x, hi, lo, scale, m, k, ldx, dtype, group, act, act_weight, eps, RowShift{nullptr, 0, 0}, stream);
}

// wq8_quantize reading rows first + counter[0] * step ... of x: counter on the GPU, read at run time.
WQ_API int wq8_quantize_at(const void* x, int8_t* hi, int8_t* lo, float* scale, int m, int k, int64_t ldx, int dtype, int group, int act,
                           const void* act_weight, float eps, const long long* counter, long long first, long long step, cudaStream_t stream) {
    return quantize_entry(x, hi, lo, scale, m, k, ldx, dtype, group, act, act_weight, eps, RowShift{counter, first, step}, stream);
}

WQ_API int wq8_transform_rows(const void* x, void* out, int m, int k, int64_t ldx, int dtype, int group, int act, const void* act_weight, float eps,
                              cudaStream_t stream) {
    if (m <= 0) return 0;
    if (k <= 0 || k % 8 || (group && k % group)) return -2;
    if (dtype == 0) return transform_by_group<__half>(x, out, m, k, ldx, group, act, act_weight, eps, stream);
    if (dtype == 1) return transform_by_group<bf16>(x, out, m, k, ldx, group, act, act_weight, eps, stream);
    return -1;
}

WQ_API int wq8_rotate_groups(const void* x, void* out, int m, int k, int64_t ldx, int dtype, int group, cudaStream_t stream) {
    if (m <= 0) return 0;
    if (k <= 0 || k % 8 || (group && k % group)) return -2;
    if (dtype == 0) return rotate_by_group<__half>(x, out, m, k, ldx, group, stream);
    if (dtype == 1) return rotate_by_group<bf16>(x, out, m, k, ldx, group, stream);
    return -1;
}
