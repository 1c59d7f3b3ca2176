// Device helpers for asynchronous copies and mbarriers (sm_100a inline PTX).
// The including file defines WF_STATUS_WORD, the __device__ int that records a
// bounded wait that ran out.
#pragma once

#include <stdint.h>

namespace wf {

constexpr unsigned SPIN_LIMIT = 1u << 20;
constexpr unsigned SUSPEND_HINT_NS = 20000;            // per try_wait
constexpr unsigned long long WAIT_LIMIT_NS = 400000000;  // a wait that never completes gives up after 0.4 s (or SPIN_LIMIT polls)

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }

__device__ __forceinline__ void mbar_init(uint64_t* bar, unsigned count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("{\n .reg .b64 st;\n mbarrier.arrive.shared::cta.b64 st, [%0];\n}\n" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, unsigned bytes) {
    asm volatile("{\n .reg .b64 st;\n mbarrier.arrive.expect_tx.shared::cta.b64 st, [%0], %1;\n}\n" ::"r"(smem_u32(bar)), "r"(bytes)
                 : "memory");
}
// Bounded wait.  Returns false (and poisons the CTA) when the bound is hit.
// The common case in a running pipeline is a barrier whose phase has completed already: that is answered by one
// non-blocking test (measured: ~50 cycles, against ~260 for the blocking form even when it succeeds at once).
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, unsigned parity, volatile int* poisoned) {
    const uint32_t a = smem_u32(bar);
    unsigned ok;
    asm volatile("{\n .reg .pred p;\n mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}\n"
                 : "=r"(ok)
                 : "r"(a), "r"(parity)
                 : "memory");
    if (ok) return true;
    if (*poisoned) return false;
    unsigned long long t0 = 0;
    for (unsigned it = 0; it < SPIN_LIMIT; ++it) {
        // the last operand is a suspend-time hint (ns): the warp sleeps in hardware until the phase completes or about
        // that long, instead of spinning through the issue slots of the warps that do the work
        asm volatile("{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n selp.u32 %0, 1, 0, p;\n}\n"
                     : "=r"(ok)
                     : "r"(a), "r"(parity), "r"(SUSPEND_HINT_NS)
                     : "memory");
        if (ok) return true;
        if ((it & 15) == 15) {  // bound the wait by time as well: the hint makes one iteration up to SUSPEND_HINT_NS long
            if (*poisoned) return false;
            unsigned long long now;
            asm volatile("mov.u64 %0, %%globaltimer;\n" : "=l"(now));
            if (t0 == 0) t0 = now;
            else if (now - t0 > WAIT_LIMIT_NS) break;
        }
    }
    *poisoned = 1;
    atomicExch(&WF_STATUS_WORD, WF_E_LIMIT);
    return false;
}
__device__ __forceinline__ void bulk_copy_g2s(void* dst, const void* src, unsigned bytes, uint64_t* bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];\n" ::"r"(smem_u32(dst)),
                 "l"(src), "r"(bytes), "r"(smem_u32(bar))
                 : "memory");
}
__device__ __forceinline__ void tma_load_3d(void* dst, const void* tmap, int c0, int c1, int c2, uint64_t* bar) {
    asm volatile("cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];\n" ::"r"(
                     smem_u32(dst)),
                 "l"(reinterpret_cast<uint64_t>(tmap)), "r"(c0), "r"(c1), "r"(c2), "r"(smem_u32(bar))
                 : "memory");
}
__device__ __forceinline__ void tma_load_2d(void* dst, const void* tmap, int c0, int c1, uint64_t* bar) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];\n" ::"r"(
                     smem_u32(dst)),
                 "l"(reinterpret_cast<uint64_t>(tmap)), "r"(c0), "r"(c1), "r"(smem_u32(bar))
                 : "memory");
}

}  // namespace wf
