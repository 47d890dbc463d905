// Issue-rate probe of the tensor pipe, built into a library of its own (libwgp_int8_probe.so) that only the benchmark loads: a
// measurement tool that allocates and synchronizes has no place in the product library.
//
// One CTA per SM issues `iters` groups of four M128 N256 MMAs on resident shared-memory operands (no loads, no epilogue), alternating
// two accumulator buffers.  KIND 0: kind::i8 (K = 32), 1: kind::f16 with BF16 (K = 16).
#include <cuda.h>

#include "tc_ptx.cuh"

namespace wq {

template <int KIND>
__global__ void __launch_bounds__(128, 1) mma_peak_probe(int iters, long long* cycles, long long* nanoseconds, int* status) {
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
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // the bytes above are read by the tensor cores
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
        mbar_wait(smem_u32(&bar), 0, &abort_word, 1, status, 4000000000ll);
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

}  // namespace wq

using namespace wq;

// results[0] = tera-operations per second of the whole GPU, results[1] = SM clock in MHz during the probe, results[2] = clocks per MMA
// group.  kind 0: tcgen05 kind::i8, 1: kind::f16 with BF16; iters < 0: pseudo-random operands instead of zeros.
WQ_API int wq8_probe_mma_peak(int kind, int iters, int sms, double* results) {
    if (iters == 0 || sms <= 0 || sms > 1024 || (kind != 0 && kind != 1)) return -2;
    long long* buffers = nullptr;
    if (cudaMalloc(&buffers, sizeof(long long) * (2 * sms + 1)) != cudaSuccess) return int(cudaGetLastError());
    cudaMemset(buffers, 0, sizeof(long long) * (2 * sms + 1));
    const int smem_bytes = (kBM + 256) * kStageK + 1024;
    auto kernel = kind == 0 ? mma_peak_probe<0> : mma_peak_probe<1>;
    cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes);
    for (int round = 0; round < 2; ++round) kernel<<<sms, 128, smem_bytes>>>(iters, buffers, buffers + sms, reinterpret_cast<int*>(buffers + 2 * sms));
    int code = int(cudaDeviceSynchronize());
    long long host[2049];
    if (!code) code = int(cudaMemcpy(host, buffers, sizeof(long long) * (2 * sms + 1), cudaMemcpyDeviceToHost));
    cudaFree(buffers);
    if (code) return code;
    if (host[2 * sms]) return -6;  // a probe's wait for its MMAs ran out
    double cycles = 0, ns = 0;
    for (int i = 0; i < sms; ++i) { cycles += double(host[i]); ns += double(host[sms + i]); }
    cycles /= sms; ns /= sms;
    const double ops = 2.0 * kBM * 256 * (kind == 0 ? 32 : 16) * 4.0 * (iters < 0 ? -iters : iters) * sms;
    results[0] = ops / (ns * 1e-9) / 1e12;
    results[1] = cycles / ns * 1e3;
    results[2] = cycles / (iters < 0 ? -iters : iters);
    return 0;
}
