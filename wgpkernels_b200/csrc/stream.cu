// Few-token paths ('lines': 1-4 tokens, 'small': up to 32 tokens): weight-only INT8.  The activations stay unquantized; the INT8
// weight matrix is streamed once from HBM with 128-bit loads, converted exactly to BF16 / FP16 in registers and multiplied on tensor
// cores with FP32 accumulation.  HBM-bound: the design goal is bytes in flight (every SM streaming, 4 x 1 KiB per warp outstanding)
// and a fixed-order (deterministic) reduction.  Replaces w8a16_small / gemv_lines of the reference (wgpkernels/int8/int8_gemm.cu:
// 1039-1151, 1772-1810): same values up to FP32 summation order.
#include "common.cuh"

namespace wq {

WQ_DEVICE uint4 load_streaming(const void* p) {
    uint4 r;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];\n" : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w) : "l"(p));
    return r;
}

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
constexpr int kStreamUnroll = 4;   // chunks in flight per warp

// Output channels are the MMA rows ("swap AB"): a warp owns 16 channels, lane (g = lane / 4, t = lane % 4) streams 16 contiguous bytes of
// rows g and g + 8 per chunk.  Any permutation of K applied to both operands leaves the product unchanged, so the bytes are used where they
// land: MMA q of a chunk takes bytes 4q..4q+3 of both rows (logical k 2t, 2t+1 | 2t+8, 2t+9) and the tokens' values at the same positions.
// The 8 warps of a CTA are wn channel blocks x wk slices of K (wn * wk = 8): many channels -> no reduction in the CTA, few channels -> the
// CTA splits K so that every SM streams.  gridDim.y splits K further across CTAs (partials through `slots`, last arriver reduces in order).
template <class T, int MT>
__global__ void __launch_bounds__(256) stream_mma(const T* __restrict__ x, int64_t ldx, const int8_t* __restrict__ w, const float* __restrict__ sw,
                                                  const T* __restrict__ bias, const T* residual, const T* __restrict__ rscale, T* y, int m, int n, int k,
                                                  int wk, float* __restrict__ slots, int* __restrict__ counters) {
    __shared__ float partial[8][MT * 8][17];
    __shared__ int is_last;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, g = lane >> 2, t = lane & 3;
    const int wn = 8 / wk, slice = warp % wk, channel_block = warp / wk;
    const int ch0 = (blockIdx.x * wn + channel_block) * 16 + g, ch1 = ch0 + 8;
    const bool ok0 = ch0 < n, ok1 = ch1 < n;
    const int chunks = k / kStreamChunk, splits = gridDim.y;
    const int c_begin = int(int64_t(blockIdx.y) * chunks / splits), c_end = int(int64_t(blockIdx.y + 1) * chunks / splits);
    const int8_t* w0 = w + int64_t(ok0 ? ch0 : 0) * k + 16 * t;
    const int8_t* w1 = w + int64_t(ok1 ? ch1 : 0) * k + 16 * t;
    const T* x_row[MT];
    bool x_ok[MT];
#pragma unroll
    for (int mt = 0; mt < MT; ++mt) {
        const int token = mt * 8 + g;
        x_ok[mt] = token < m;
        x_row[mt] = x + int64_t(x_ok[mt] ? token : 0) * ldx + 16 * t;
    }
    float acc[MT][4];
#pragma unroll
    for (int mt = 0; mt < MT; ++mt) acc[mt][0] = acc[mt][1] = acc[mt][2] = acc[mt][3] = 0.f;

    for (int c = c_begin + slice; c < c_end; c += wk * kStreamUnroll) {
        uint4 row0[kStreamUnroll], row1[kStreamUnroll];
#pragma unroll
        for (int u = 0; u < kStreamUnroll; ++u) {
            const int cc = c + wk * u;
            const bool inside = cc < c_end;
            row0[u] = inside && ok0 ? load_streaming(w0 + int64_t(cc) * kStreamChunk) : make_uint4(0u, 0u, 0u, 0u);
            row1[u] = inside && ok1 ? load_streaming(w1 + int64_t(cc) * kStreamChunk) : make_uint4(0u, 0u, 0u, 0u);
        }
#pragma unroll
        for (int u = 0; u < kStreamUnroll; ++u) {
            const int cc = c + wk * u;
            const bool inside = cc < c_end;  // chunks past the range carry zero weights: no divergent exit inside the unrolled body
            uint4 xv[MT][2];
#pragma unroll
            for (int mt = 0; mt < MT; ++mt) {
                const T* p = x_row[mt] + int64_t(cc) * kStreamChunk;
                xv[mt][0] = x_ok[mt] && inside ? __ldg(reinterpret_cast<const uint4*>(p)) : make_uint4(0u, 0u, 0u, 0u);
                xv[mt][1] = x_ok[mt] && inside ? __ldg(reinterpret_cast<const uint4*>(p) + 1) : make_uint4(0u, 0u, 0u, 0u);
            }
            const uint32_t* r0 = reinterpret_cast<const uint32_t*>(&row0[u]);
            const uint32_t* r1 = reinterpret_cast<const uint32_t*>(&row1[u]);
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                uint32_t a0, a1, a2, a3;
                int8x4_to_pairs<T>(r0[q], a0, a2);
                int8x4_to_pairs<T>(r1[q], a1, a3);
#pragma unroll
                for (int mt = 0; mt < MT; ++mt) {
                    const uint32_t* xs = reinterpret_cast<const uint32_t*>(&xv[mt][q >> 1]);
                    mma_16x8x16<T>(acc[mt], a0, a1, a2, a3, xs[(q & 1) * 2], xs[(q & 1) * 2 + 1]);
                }
            }
        }
    }
    // acc[mt] = {(channel g, token 2t), (g, 2t + 1), (g + 8, 2t), (g + 8, 2t + 1)} of token block mt
#pragma unroll
    for (int mt = 0; mt < MT; ++mt) {
        partial[warp][mt * 8 + 2 * t][g] = acc[mt][0];
        partial[warp][mt * 8 + 2 * t + 1][g] = acc[mt][1];
        partial[warp][mt * 8 + 2 * t][g + 8] = acc[mt][2];
        partial[warp][mt * 8 + 2 * t + 1][g + 8] = acc[mt][3];
    }
    __syncthreads();
    constexpr int kPerBlock = MT * 8 * 16;  // outputs of one channel block
    const int outputs = wn * kPerBlock;
    float* own = slots ? slots + (int64_t(blockIdx.x) * splits + blockIdx.y) * outputs : nullptr;
    // the K slices of the CTA, in slice order; the sum lands in the first slice's buffer
    for (int i = threadIdx.x; i < outputs; i += 256) {
        const int cb = i / kPerBlock, token = (i % kPerBlock) / 16, c = i % 16;
        float s = 0.f;
        for (int ks = 0; ks < wk; ++ks) s += partial[cb * wk + ks][token][c];
        partial[cb * wk][token][c] = s;
        if (own) __stcg(own + i, s);
    }
    if (splits > 1) {
        __threadfence();
        __syncthreads();
        if (threadIdx.x == 0) is_last = atomicAdd(counters + blockIdx.x, 1) == splits - 1;
        __syncthreads();
        if (!is_last) return;
        __threadfence();
        const float* tile = slots + int64_t(blockIdx.x) * splits * outputs;
        for (int i = threadIdx.x; i < outputs; i += 256) {
            float s = 0.f;
            for (int piece = 0; piece < splits; ++piece) s += __ldcg(tile + int64_t(piece) * outputs + i);
            partial[(i / kPerBlock) * wk][(i % kPerBlock) / 16][i % 16] = s;
        }
        if (threadIdx.x == 0) counters[blockIdx.x] = 0;  // left zeroed for the next launch
    }
    __syncthreads();
    for (int i = threadIdx.x; i < outputs; i += 256) {
        const int cb = i / kPerBlock, token = (i % kPerBlock) / 16, c = i % 16;
        const int channel = (blockIdx.x * wn + cb) * 16 + c;
        if (token < m && channel < n) {
            float v = partial[cb * wk][token][c] * sw[channel] + (bias ? as_float(bias[channel]) : 0.f);
            if (residual) v = fmaf(v, rscale ? as_float(rscale[channel]) : 1.f, as_float(residual[int64_t(token) * n + channel]));
            y[int64_t(token) * n + channel] = round_one<T>(v);
        }
    }
}

// General GEMV for one to four tokens when the tensor-core kernel's alignment does not hold (K multiple of 4 only, rows of x 8-byte
// aligned): a warp per output channel, four weight bytes per lane and step, exact INT8 -> FP32 conversion, FP32 FMA, butterfly sum.
template <class T, int ROWS>
__global__ void __launch_bounds__(256) gemv_cores(const T* __restrict__ x, int64_t ldx, const int8_t* __restrict__ w, const float* __restrict__ sw,
                                                  const T* __restrict__ bias, const T* residual, const T* __restrict__ rscale, T* y, int n, int k) {
    const int lane = threadIdx.x & 31, channel = blockIdx.x * 8 + (threadIdx.x >> 5);
    if (channel >= n) return;
    const int8_t* row = w + int64_t(channel) * k;
    float acc[ROWS];
#pragma unroll
    for (int r = 0; r < ROWS; ++r) acc[r] = 0.f;
#pragma unroll 4
    for (int base = lane * 4; base < k; base += 128) {
        const uint32_t packed = __ldg(reinterpret_cast<const uint32_t*>(row + base));
        float wf[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) wf[j] = float(int(int8_t(packed >> (8 * j))));
#pragma unroll
        for (int r = 0; r < ROWS; ++r) {
            const uint2 raw = __ldg(reinterpret_cast<const uint2*>(x + int64_t(r) * ldx + base));
            float x0, x1, x2, x3;
            unpack_pair<T>(raw.x, x0, x1);
            unpack_pair<T>(raw.y, x2, x3);
            acc[r] = fmaf(wf[0], x0, acc[r]);
            acc[r] = fmaf(wf[1], x1, acc[r]);
            acc[r] = fmaf(wf[2], x2, acc[r]);
            acc[r] = fmaf(wf[3], x3, acc[r]);
        }
    }
#pragma unroll
    for (int r = 0; r < ROWS; ++r) {
        float a = acc[r];
#pragma unroll
        for (int d = 16; d > 0; d >>= 1) a += __shfl_xor_sync(0xffffffffu, a, d);
        if (lane == 0) {
            float v = a * sw[channel] + (bias ? as_float(bias[channel]) : 0.f);
            if (residual) v = fmaf(v, rscale ? as_float(rscale[channel]) : 1.f, as_float(residual[int64_t(r) * n + channel]));
            y[int64_t(r) * n + channel] = round_one<T>(v);
        }
    }
}

// ---- host side ---------------------------------------------------------------------------------------------------------
struct StreamPlan { int wk, ctas, splits; };

// wn channel blocks per CTA: as many as still leave two CTAs per SM; then K splits across CTAs (only with a workspace) until every SM streams,
// keeping at least four chunks per warp and piece.
static StreamPlan plan_stream(int n, int k, int sms, bool may_split) {
    const int blocks = (n + 15) / 16, target = 2 * (sms > 0 ? sms : 148);
    int wn = 8;
    while (wn > 1 && (blocks + wn - 1) / wn < target) wn /= 2;
    StreamPlan p{8 / wn, (blocks + wn - 1) / wn, 1};
    if (may_split && p.ctas < target) {
        const int wanted = (target + p.ctas - 1) / p.ctas, most = (k / kStreamChunk) / (p.wk * 4);
        p.splits = wanted < most ? wanted : (most > 1 ? most : 1);
        if (p.ctas > 1024) p.splits = 1;  // the caller's counter buffer holds 1024 tiles
    }
    return p;
}

static int tokens_blocks(int m) { return m <= 8 ? 1 : m <= 16 ? 2 : 4; }

template <class T>
static int launch_stream(const void* x, int64_t ldx, const int8_t* w, const float* sw, const void* bias, const void* residual, const void* rscale,
                         void* y, int m, int n, int k, const StreamPlan& p, float* slots, int* counters, cudaStream_t stream) {
    const dim3 grid(p.ctas, p.splits);
    auto xs = static_cast<const T*>(x);
    auto b = static_cast<const T*>(bias), r = static_cast<const T*>(residual), rs = static_cast<const T*>(rscale);
    auto out = static_cast<T*>(y);
    float* sl = p.splits > 1 ? slots : nullptr;
    switch (tokens_blocks(m)) {
        case 1: stream_mma<T, 1><<<grid, 256, 0, stream>>>(xs, ldx, w, sw, b, r, rs, out, m, n, k, p.wk, sl, counters); break;
        case 2: stream_mma<T, 2><<<grid, 256, 0, stream>>>(xs, ldx, w, sw, b, r, rs, out, m, n, k, p.wk, sl, counters); break;
        default: stream_mma<T, 4><<<grid, 256, 0, stream>>>(xs, ldx, w, sw, b, r, rs, out, m, n, k, p.wk, sl, counters); break;
    }
    return int(cudaGetLastError());
}

template <class T>
static int launch_cores(const void* x, int64_t ldx, const int8_t* w, const float* sw, const void* bias, const void* residual, const void* rscale,
                        void* y, int m, int n, int k, cudaStream_t stream) {
    auto xs = static_cast<const T*>(x);
    auto b = static_cast<const T*>(bias), r = static_cast<const T*>(residual), rs = static_cast<const T*>(rscale);
    auto out = static_cast<T*>(y);
    const int grid = (n + 7) / 8;
    if (m == 1) gemv_cores<T, 1><<<grid, 256, 0, stream>>>(xs, ldx, w, sw, b, r, rs, out, n, k);
    else if (m == 2) gemv_cores<T, 2><<<grid, 256, 0, stream>>>(xs, ldx, w, sw, b, r, rs, out, n, k);
    else if (m == 3) gemv_cores<T, 3><<<grid, 256, 0, stream>>>(xs, ldx, w, sw, b, r, rs, out, n, k);
    else gemv_cores<T, 4><<<grid, 256, 0, stream>>>(xs, ldx, w, sw, b, r, rs, out, n, k);
    return int(cudaGetLastError());
}

static int device_sms() {
    int device = 0, sms = 148;
    cudaGetDevice(&device);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device);
    return sms;
}

}  // namespace wq

using namespace wq;

WQ_API void wq8_small_workspace(int m, int n, int k, int sms, int64_t* sizes) {
    const StreamPlan p = plan_stream(n, k, sms, true);
    const int64_t outputs = int64_t(8 / p.wk) * tokens_blocks(m) * 8 * 16;
    sizes[0] = p.splits > 1 ? int64_t(p.ctas) * p.splits * outputs * 4 : 0;
    sizes[1] = p.splits > 1 ? 4 * int64_t(p.ctas) : 0;
}

WQ_API int wq8_small(const void* x, int64_t ldx, const int8_t* w, const float* sw, const void* bias, const void* residual, const void* rscale, void* y,
                     int m, int n, int k, int dtype, int sms, float* slots, int* counters, cudaStream_t stream) {
    if (m <= 0 || n <= 0) return 0;
    if (k <= 0 || k % 64 || m > 32 || ldx % 8 || (reinterpret_cast<uintptr_t>(x) & 15)) return -2;
    if (dtype != 0 && dtype != 1) return -1;
    StreamPlan p = plan_stream(n, k, sms, true);
    if (p.splits > 1 && (!slots || !counters)) p.splits = 1;
    if (dtype == 0) return launch_stream<__half>(x, ldx, w, sw, bias, residual, rscale, y, m, n, k, p, slots, counters, stream);
    return launch_stream<bf16>(x, ldx, w, sw, bias, residual, rscale, y, m, n, k, p, slots, counters, stream);
}

WQ_API int wq8_gemv_lines(const void* x, int64_t ldx, const int8_t* w, const float* sw, const void* bias, const void* residual, const void* rscale,
                          void* y, int m, int n, int k, int dtype, cudaStream_t stream) {
    if (m <= 0 || n <= 0) return 0;
    if (m > 4 || k <= 0 || k % 4) return -2;
    if (dtype != 0 && dtype != 1) return -1;
    const bool tensor_cores = k % 64 == 0 && ldx % 8 == 0 && (reinterpret_cast<uintptr_t>(x) & 15) == 0 && (reinterpret_cast<uintptr_t>(w) & 15) == 0;
    if (tensor_cores) {
        const StreamPlan p = plan_stream(n, k, device_sms(), false);
        if (dtype == 0) return launch_stream<__half>(x, ldx, w, sw, bias, residual, rscale, y, m, n, k, p, nullptr, nullptr, stream);
        return launch_stream<bf16>(x, ldx, w, sw, bias, residual, rscale, y, m, n, k, p, nullptr, nullptr, stream);
    }
    if (dtype == 0) return launch_cores<__half>(x, ldx, w, sw, bias, residual, rscale, y, m, n, k, stream);
    return launch_cores<bf16>(x, ldx, w, sw, bias, residual, rscale, y, m, n, k, stream);
}

// ---------------------------------------------------------------------------------------------------------------------
// wq8_small without caller scratch.
//
// wq8_small splits K across CTAs when few output channels would leave SMs idle, and the caller has to hand it the partial-sum slots
// and the tile counters for that.  Some callers have no way to provide them: a host that drives this library through plain ctypes / FFI
// with buffers it was given (no allocator of its own on the device), a serving loop that runs under a fixed memory budget and may not
// grow it per request, code that runs while a CUDA graph is being captured or inside a real-time section where cudaMalloc (which
// synchronizes and may fail) is off limits.  For them the scratch lives here, in device memory that belongs to the library: every GPU
// that loads the library holds kStaticScratchBytes (2 MiB + 4 KiB) of it until the process exits.
//
// The array's name is only a handle on the host: a kernel must be given the device address, which cudaGetSymbolAddress returns for
// the device that is current at the time.  It is looked up once per device, on the first call made with that device current -- that
// first call should therefore happen before any stream capture starts -- and cached.
// ---------------------------------------------------------------------------------------------------------------------
namespace wq {

constexpr int64_t kStaticSlotBytes = 2 << 20;     // partial sums: enough for every plan of at most 32 tokens on up to 256 SMs
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

// Same linear as wq8_small (at most 32 tokens, K multiple of 64, x rows 16-byte aligned), same values, no scratch arguments and no
// allocation of any kind: the K-split partial sums and tile counters use the library's own static device buffer.
// Returns -5 when the shape's scratch would not fit that buffer (use wq8_small with caller scratch then); other codes as wq8_small.
// Calls share the one buffer per device: two calls whose kernels may overlap on the GPU (different streams, or one stream of a graph with
// parallel branches) race on it -- keep them on one stream, or give the others caller scratch through wq8_small.  The buffer keeps what
// the last call left in it; the counters are cleared on the stream in front of every launch, the slots are written before they are read.
WQ_API int wq8_small_static(const void* x, int64_t ldx, const int8_t* w, const float* sw, const void* bias, const void* residual, const void* rscale,
                            void* y, int m, int n, int k, int dtype, int sms, cudaStream_t stream) {
    if (m <= 0 || n <= 0) return 0;
    if (k <= 0 || k % 64 || m > 32 || ldx % 8 || (reinterpret_cast<uintptr_t>(x) & 15)) return -2;
    if (dtype != 0 && dtype != 1) return -1;
    const StreamPlan p = plan_stream(n, k, sms, true);
    float* slots = nullptr;
    int* counters = nullptr;
    if (p.splits > 1) {
        const int64_t outputs = int64_t(8 / p.wk) * tokens_blocks(m) * 8 * 16;
        const int64_t slot_bytes = int64_t(p.ctas) * p.splits * outputs * 4, counter_bytes = 4 * int64_t(p.ctas);
        if (slot_bytes > kStaticSlotBytes || counter_bytes > kStaticCounterBytes) return -5;
        int error = 0;
        unsigned char* scratch = static_scratch_address(&error);
        if (!scratch) return error;
        slots = reinterpret_cast<float*>(scratch);
        counters = reinterpret_cast<int*>(scratch + kStaticSlotBytes);
        const cudaError_t cleared = cudaMemsetAsync(counters, 0, size_t(counter_bytes), stream);
        if (cleared != cudaSuccess) return int(cleared);
    }
    if (dtype == 0) return launch_stream<__half>(x, ldx, w, sw, bias, residual, rscale, y, m, n, k, p, slots, counters, stream);
    return launch_stream<bf16>(x, ldx, w, sw, bias, residual, rscale, y, m, n, k, p, slots, counters, stream);
}
