// Shared device helpers of the INT8 weight-linear library (sm_100a).
#pragma once
#include <cuda.h>  // CUtensorMap and its enums only; cuTensorMapEncodeTiled is resolved through the runtime, libcuda is not linked
#include <cuda_runtime.h>
#include <cuda_fp16.h>
#include <cuda_bf16.h>
#include <stdint.h>
#include <type_traits>

#define WQ_DEVICE __device__ __forceinline__
#define WQ_API extern "C" __attribute__((visibility("default")))

namespace wq {

using bf16 = __nv_bfloat16;

enum Act : int { kActNone = 0, kActRms = 1, kActSwiglu = 2, kActGelu = 3 };

constexpr int kBlockK = 128;      // elements of K sharing one activation (and group-weight) scale
constexpr int kChunk = 256;       // elements of K a warp quantizes at once: 8 per lane, two scale blocks
constexpr int kRowThreads = 256;  // threads of the one-CTA-per-row kernels (8 warps)

// ---- element conversion -------------------------------------------------------------------------------------
template <class T> WQ_DEVICE float as_float(T v) { return float(v); }
template <> WQ_DEVICE float as_float<bf16>(bf16 v) { return __bfloat162float(v); }
template <> WQ_DEVICE float as_float<__half>(__half v) { return __half2float(v); }

// Two floats rounded to nearest-even into one 32-bit pair of T (element 0 in the low half).
template <class T> WQ_DEVICE uint32_t pack_pair(float lo, float hi);
template <> WQ_DEVICE uint32_t pack_pair<bf16>(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}
template <> WQ_DEVICE uint32_t pack_pair<__half>(float lo, float hi) {
    __half2 v = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}
template <class T> WQ_DEVICE T round_one(float v);
template <> WQ_DEVICE bf16 round_one<bf16>(float v) { return __float2bfloat16_rn(v); }
template <> WQ_DEVICE __half round_one<__half>(float v) { return __float2half_rn(v); }

template <class T> WQ_DEVICE void unpack_pair(uint32_t raw, float& lo, float& hi);
template <> WQ_DEVICE void unpack_pair<bf16>(uint32_t raw, float& lo, float& hi) {
    lo = __uint_as_float(raw << 16);
    hi = __uint_as_float(raw & 0xffff0000u);
}
template <> WQ_DEVICE void unpack_pair<__half>(uint32_t raw, float& lo, float& hi) {
    const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&raw));
    lo = f.x;
    hi = f.y;
}

// Eight consecutive elements at p (16-byte aligned for 16-bit types, 32 bytes for float) as floats; zeros when !valid.
template <class T> WQ_DEVICE void load_eight(const T* p, float* v, bool valid) {
    if constexpr (sizeof(T) == 2) {
        uint4 raw = make_uint4(0u, 0u, 0u, 0u);
        if (valid) raw = __ldg(reinterpret_cast<const uint4*>(p));
        unpack_pair<T>(raw.x, v[0], v[1]);
        unpack_pair<T>(raw.y, v[2], v[3]);
        unpack_pair<T>(raw.z, v[4], v[5]);
        unpack_pair<T>(raw.w, v[6], v[7]);
    } else {
        float4 a = make_float4(0.f, 0.f, 0.f, 0.f), b = a;
        if (valid) {
            a = __ldg(reinterpret_cast<const float4*>(p));
            b = __ldg(reinterpret_cast<const float4*>(p) + 1);
        }
        v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w;
        v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
    }
}

// Eight consecutive 16-bit elements at p (16-byte aligned) as floats, through an ordinary (coherent) load: for data the same
// kernel writes later.
template <class T> WQ_DEVICE void load_eight_plain(const T* p, float* v) {
    static_assert(sizeof(T) == 2, "16-bit element types only");
    const uint4 raw = *reinterpret_cast<const uint4*>(p);
    unpack_pair<T>(raw.x, v[0], v[1]);
    unpack_pair<T>(raw.y, v[2], v[3]);
    unpack_pair<T>(raw.z, v[4], v[5]);
    unpack_pair<T>(raw.w, v[6], v[7]);
}

// Four INT8 codes (each already within [-128, 127]) into one word, a in the lowest byte: two packing conversions
// (cvt.pack: the two converted values go to the low half, the third operand's low half moves up).
WQ_DEVICE uint32_t pack_bytes(int a, int b, int c, int d) {
    uint32_t high, word;
    asm("cvt.pack.sat.s8.s32.b32 %0, %1, %2, %3;" : "=r"(high) : "r"(d), "r"(c), "r"(0));
    asm("cvt.pack.sat.s8.s32.b32 %0, %1, %2, %3;" : "=r"(word) : "r"(b), "r"(a), "r"(high));
    return word;
}

// ---- input operations, FP32 (the expression shapes fix the rounding: they are part of the numerical contract) ----
WQ_DEVICE float gelu_tanh(float x) {
    const float inner = 0.7978845608028654f * (x + 0.044715f * (x * x * x));
    return 0.5f * x * (1.f + tanhf(inner));
}
WQ_DEVICE float silu_times(float gate, float value) { return gate / (1.f + expf(-gate)) * value; }

// The eight op(x) values at column `col` of a row (`k` = width of the linear; SwiGLU rows hold [gate | value]).
// RMSNorm is applied later, once the row's sum of squares is known.
template <class T, int ACT> WQ_DEVICE void load_op(const T* row, int k, int col, float* v, bool valid) {
    load_eight(row + col, v, valid);
    if constexpr (ACT == kActSwiglu) {
        float u[8];
        load_eight(row + k + col, u, valid);
#pragma unroll
        for (int j = 0; j < 8; ++j) v[j] = silu_times(v[j], u[j]);
    }
    if constexpr (ACT == kActGelu) {
#pragma unroll
        for (int j = 0; j < 8; ++j) v[j] = gelu_tanh(v[j]);
    }
}

template <class T> WQ_DEVICE void scale_by_rms(float* v, float inv_rms, const T* weight, int col, bool valid) {
    float w[8];
    if (weight) load_eight(weight + col, w, valid);
#pragma unroll
    for (int j = 0; j < 8; ++j) v[j] = v[j] * inv_rms * (weight ? w[j] : 1.f);
}

WQ_DEVICE float inverse_rms(float sum_squares, int k, float eps) { return 1.f / sqrtf(sum_squares / float(k) + eps); }

// 1 / rms of a row from the threads' partial sums of squares, summed in a fixed order (xor-butterfly inside each warp, then warps 0..7 in
// turn); the sum over the warps, the division, the square root and the reciprocal are done by the first warp alone and handed to the others through shared
// memory (slots9[8]) -- a second barrier instead of some fifty instructions in each of the other seven warps.
WQ_DEVICE float cta_inverse_rms(float v, float* slots9, int k, float eps) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) v += __shfl_xor_sync(0xffffffffu, v, d);
    if (lane == 0) slots9[warp] = v;
    __syncthreads();
    if (warp == 0) {
        float total = slots9[0];
#pragma unroll
        for (int w = 1; w < 8; ++w) total += slots9[w];
        const float result = inverse_rms(total, k, eps);
        if (lane == 0) slots9[8] = result;
    }
    __syncthreads();
    return slots9[8];
}

WQ_DEVICE float cta_max(float v, float* slots8) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, d));
    if (lane == 0) slots8[warp] = v;
    __syncthreads();
    float total = slots8[0];
#pragma unroll
    for (int w = 1; w < 8; ++w) total = fmaxf(total, slots8[w]);
    return total;
}

// ---- ConvRot rotation of a 256-element chunk held by a warp (lane l: elements 8l .. 8l+7) -----------------------
// The rotation is the Kronecker power of the regular 4x4 Hadamard matrix H4 = J - 2 * antidiag: along each base-4 digit of the
// index inside a group, out[d] = (in0 + in1) + (in2 + in3) - 2 * in[3 - d].  Unnormalised: callers fold 1 / sqrt(GROUP) in later.
// Digit 0 is bits 0-1 of the element index (inside a lane), digit 1 is bit 2 of the element and bit 0 of the lane,
// digit 2 is lane bits 1-2, digit 3 is lane bits 3-4.
WQ_DEVICE void h4_digit_in_lane(float* v) {
#pragma unroll
    for (int base = 0; base < 8; base += 4) {
        const float x0 = v[base], x1 = v[base + 1], x2 = v[base + 2], x3 = v[base + 3];
        const float s = (x0 + x1) + (x2 + x3);
        v[base] = s - 2.f * x3;
        v[base + 1] = s - 2.f * x2;
        v[base + 2] = s - 2.f * x1;
        v[base + 3] = s - 2.f * x0;
    }
}
WQ_DEVICE void h4_digit_split(float* v) {
    // digit value = (element >> 2) | ((lane & 1) << 1); the mirrored digit 3 - d sits in the neighbour lane at the other element half
    float out[8];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        const float pair = v[j] + v[j + 4];
        const float s = pair + __shfl_xor_sync(0xffffffffu, pair, 1);
        const float mirror_of_low = __shfl_xor_sync(0xffffffffu, v[j + 4], 1);
        const float mirror_of_high = __shfl_xor_sync(0xffffffffu, v[j], 1);
        out[j] = s - 2.f * mirror_of_low;
        out[j + 4] = s - 2.f * mirror_of_high;
    }
#pragma unroll
    for (int j = 0; j < 8; ++j) v[j] = out[j];
}
template <int LANE_BIT> WQ_DEVICE void h4_digit_across_lanes(float* v) {
#pragma unroll
    for (int j = 0; j < 8; ++j) {
        const float pair = v[j] + __shfl_xor_sync(0xffffffffu, v[j], LANE_BIT);
        const float s = pair + __shfl_xor_sync(0xffffffffu, pair, 2 * LANE_BIT);
        v[j] = s - 2.f * __shfl_xor_sync(0xffffffffu, v[j], 3 * LANE_BIT);
    }
}
template <int GROUP> WQ_DEVICE void rotate_chunk(float* v) {
    static_assert(GROUP == 0 || GROUP == 16 || GROUP == 64 || GROUP == 256, "ConvRot groups are 16, 64 or 256");
    if constexpr (GROUP >= 16) {
        h4_digit_in_lane(v);
        h4_digit_split(v);
    }
    if constexpr (GROUP >= 64) h4_digit_across_lanes<2>(v);
    if constexpr (GROUP >= 256) h4_digit_across_lanes<8>(v);
}
template <int GROUP> __host__ __device__ constexpr float group_norm() { return GROUP == 256 ? 0.0625f : GROUP == 64 ? 0.125f : GROUP == 16 ? 0.25f : 1.f; }

// ---- programmatic dependent launch ---------------------------------------------------------------------------------------
// A kernel launched with launch_after_previous() may start while the kernel before it on the stream is still running: what it does
// before dependency_wait() (set-up, requests for data the previous kernel does not write) overlaps that kernel's tail; after the wait the
// previous kernel has finished and its writes are visible.  The previous kernel lets the next one start early with dependents_may_start();
// without it the next one starts when the previous one ends, as usual.  Data the previous kernel wrote is read with ordinary loads (below),
// never through the read-only path, whose contract is that nobody writes the data while the kernel runs.
WQ_DEVICE void dependents_may_start() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
WQ_DEVICE void dependency_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
WQ_DEVICE uint4 load_16(const void* p) {
    uint4 v;
    asm volatile("ld.global.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
    return v;
}
WQ_DEVICE uint2 load_8(const void* p) {
    uint2 v;
    asm volatile("ld.global.v2.u32 {%0, %1}, [%2];" : "=r"(v.x), "=r"(v.y) : "l"(p) : "memory");
    return v;
}
template <class... Params, class... Args>
inline cudaError_t launch_after_previous(void (*kernel)(Params...), dim3 grid, dim3 block, size_t shared_bytes, cudaStream_t stream, Args... args) {
    cudaLaunchConfig_t config = {};
    config.gridDim = grid;
    config.blockDim = block;
    config.dynamicSmemBytes = shared_bytes;
    config.stream = stream;
    cudaLaunchAttribute attribute;
    attribute.id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attribute.val.programmaticStreamSerializationAllowed = 1;
    config.attrs = &attribute;
    config.numAttrs = 1;
    return cudaLaunchKernelEx(&config, kernel, Params(args)...);
}

// ---- device status word (bounded waits report here instead of trapping) ----------------------------------------------
// gemm_tc.cu: tensor map of a (rows, row_bytes) row-major byte matrix with boxes of box_rows rows x box_bytes bytes (at most 256), no
// swizzle, zero fill outside; false when the driver entry point is missing or refuses the description.
bool make_byte_matrix_map(CUtensorMap* map, const void* base, int rows, int row_bytes, int box_bytes, int box_rows);
int stream_status_take();  // stream.cu: status of the weight-streaming kernels on the current device (0 = fine), cleared by the call
// stream_tc.cu: the few-token linear on tcgen05 (digit planes): scratch bytes of a shape (0: not this kernel's shape; *counter_bytes: its
// tile counters), the launch (x already transformed; workspace and zeroed counters of those sizes), and its status word
int64_t stream_tc_workspace(int m, int n, int k, int sms, int64_t* counter_bytes);
int stream_tc_launch(const void* x, int64_t ldx, const int8_t* w, const float* sw, const void* bias, const void* residual, const void* rscale, void* y, int m,
                     int n, int k, int dtype, int sms, void* workspace, int* counters, cudaStream_t stream);
int stream_tc_status_take();

enum Status : int { kOk = 0, kTimeoutFull = 1, kTimeoutEmpty = 2, kTimeoutTmemFull = 3, kTimeoutTmemEmpty = 4, kTimeoutScales = 5, kTimeoutParams = 6, kStatusSharedAlignment = 7 };

}  // namespace wq
