// Measurement aid: the rate of the int8 tensor-core instruction on this GPU.
//
// The contraction's roofline needs a denominator that is measured, not quoted: every SM runs one CTA that issues
// `iters` groups of four tcgen05.mma.kind::i8 (M = 128, N = `n` columns, K = 32, u8 x s8 -> s32) on operand tiles that
// stay resident in shared memory, into two alternating tensor-memory accumulators, with one commit at the end.
// Nothing is loaded or stored in the timed region, so the figure is the issue/execute rate of the instruction
// itself: 2 * 128 * n * 32 operations per instruction.
#include <cuda.h>

#include "wf_common.cuh"

namespace wf {
__device__ int g_probe_status = 0;
}
#define WF_STATUS_WORD ::wf::g_probe_status
#include "wf_async.cuh"

namespace wf {

constexpr int PROBE_A_BYTES = 128 * 128;  // 128 rows x 128 B (one 128-byte swizzle atom of K)
constexpr int PROBE_B_BYTES = 256 * 128;  // up to 256 columns x 128 B
constexpr int PROBE_SMEM = 1024 + PROBE_A_BYTES + PROBE_B_BYTES + 64;

__device__ __forceinline__ uint64_t probe_desc_sw128(uint32_t addr) {
    uint64_t d = 0;
    d |= static_cast<uint64_t>((addr & 0x3FFFF) >> 4);
    d |= static_cast<uint64_t>(1024 >> 4) << 32;
    d |= static_cast<uint64_t>(1) << 46;
    d |= static_cast<uint64_t>(2) << 61;
    return d;
}

__global__ void __launch_bounds__(128, 1) probe_i8_mma_kernel(int iters, int n) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
    uint8_t* a_tile = smem;
    uint8_t* b_tile = smem + PROBE_A_BYTES;
    uint64_t* bar = reinterpret_cast<uint64_t*>(smem + PROBE_A_BYTES + PROBE_B_BYTES);
    uint32_t* slot = reinterpret_cast<uint32_t*>(bar + 1);
    volatile int* poisoned = reinterpret_cast<volatile int*>(slot + 1);
    const int tid = threadIdx.x, warp = tid >> 5;
    for (int i = tid; i < (PROBE_A_BYTES + PROBE_B_BYTES) / 4; i += 128) reinterpret_cast<uint32_t*>(smem)[i] = 0x01010101u;
    if (tid == 0) {
        mbar_init(bar, 1);
        *poisoned = 0;
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    }
    asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(smem_u32(slot)), "r"(512));
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::);
    }
    asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
    const uint32_t tmem = *slot;
    if (tid == 0) {
        // D = s32, A = unsigned 8-bit, B = signed 8-bit, both K-major, N = n, M = 128
        const uint32_t idesc = (2u << 4) | (0u << 7) | (1u << 10) | (static_cast<uint32_t>(n >> 3) << 17) | (static_cast<uint32_t>(128 >> 4) << 24);
        const uint64_t ad = probe_desc_sw128(smem_u32(a_tile)), bd = probe_desc_sw128(smem_u32(b_tile));
        for (int it = 0; it < iters; ++it) {
            const uint32_t d = tmem + (it & 1) * 256;
#pragma unroll
            for (int k = 0; k < 4; ++k)
                asm volatile(
                    "{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n"
                    " tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, {%5, %5, %5, %5}, p;\n}\n" ::"r"(d),
                    "l"(ad + 2 * k), "l"(bd + 2 * k), "r"(idesc), "r"((it > 1 || k) ? 1u : 0u), "r"(0u)
                    : "memory");
        }
        asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n" ::"r"(smem_u32(bar)) : "memory");
        mbar_wait(bar, 0, poisoned);
    }
    asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
    __syncthreads();
    if (warp == 0) {
        asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem), "r"(512));
    }
}

}  // namespace wf

using namespace wf;

extern "C" int wf_probe_i8_mma(int n, int iters, double* tops_out, double* ns_per_mma_out) {
    WF_REQUIRE(tops_out, "wf_probe_i8_mma: null pointer");
    WF_REQUIRE(n >= 16 && n <= 256 && n % 16 == 0, "wf_probe_i8_mma: n must be a multiple of 16 in [16, 256]");
    WF_REQUIRE(iters >= 1 && iters <= 100000, "wf_probe_i8_mma: iters out of range");
    if (int rc = require_device()) return rc;
    static PerDeviceOnce configured;
    const int dev = current_device();
    if (configured.needs(dev)) {
        WF_CUDA(cudaFuncSetAttribute(probe_i8_mma_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, PROBE_SMEM));
        configured.mark(dev);
    }
    const int sms = num_sms();
    cudaEvent_t a, b;
    WF_CUDA(cudaEventCreate(&a));
    WF_CUDA(cudaEventCreate(&b));
    probe_i8_mma_kernel<<<sms, 128, PROBE_SMEM>>>(64, n);  // warm-up
    WF_CUDA(cudaEventRecord(a));
    probe_i8_mma_kernel<<<sms, 128, PROBE_SMEM>>>(iters, n);
    WF_CUDA(cudaEventRecord(b));
    cudaError_t e = cudaDeviceSynchronize();
    float ms = 0.f;
    if (e == cudaSuccess) e = cudaEventElapsedTime(&ms, a, b);
    cudaEventDestroy(a);
    cudaEventDestroy(b);
    if (e != cudaSuccess) return cuda_fail(e, "wf_probe_i8_mma");
    int st = 0;
    WF_CUDA(cudaMemcpyFromSymbol(&st, g_probe_status, sizeof(int)));
    if (st) {
        int zero = 0;
        WF_CUDA(cudaMemcpyToSymbol(g_probe_status, &zero, sizeof(int)));
        return fail(WF_E_LIMIT, "wf_probe_i8_mma: the bounded wait for the tensor core ran out");
    }
    const double mmas = 4.0 * iters;
    *tops_out = 2.0 * 128.0 * n * 32.0 * mmas * sms / (ms * 1e-3) / 1e12;
    if (ns_per_mma_out) *ns_per_mma_out = ms * 1e6 / mmas;
    return WF_OK;
}
