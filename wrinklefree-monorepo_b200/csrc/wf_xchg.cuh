// The exchange of a row-parallel projection fused into the projection itself (the push side) — shared by the decode
// kernels, which push, and the reduce + residual + RMSNorm kernel, which consumes.
//
// Every rank's exchange buffer (the allocation of wf_ar_init) holds, behind the slots of the stand-alone all-reduce,
// two PUSH slots of `world` source regions each.  A projection launched with wf_problem.xchg set writes its partial
// output as usual and, when a CTA has finished its share of the work list, copies that share into the region
// [slot = step & 1][source = this rank] of EVERY rank's buffer with plain peer stores (no multicast) and then adds the
// number of elements it pushed to the counter pcount[slot][this rank] of every rank (one release-ordered reduction per
// rank; CTAs without work do nothing).  The consumer (wf_ar_reduce_add_rmsnorm) polls its own counters — local memory,
// bounded — until every source has delivered all M x N elements, sums the `world` regions of its own buffer in rank
// order in fp32, and its last block clears the slot's counters.  Nothing waits on the producer's side.
// Two slots are enough: a rank pushes step s + 2 only after it has consumed step s + 1, which every peer pushed only
// after its own consumer of step s had completed (and cleared the counters of that slot).
#pragma once

#include <stdint.h>

#include "../../include/wf_b200.h"

namespace wf {

constexpr size_t XCHG_PCOUNT_OFF = 2304;   // unsigned pcount[2][8]: elements delivered per (slot, source rank)
constexpr size_t XCHG_PSTEP_OFF = 2368;    // exchanges this rank's consumer has completed
constexpr size_t XCHG_CTICKET_OFF = 2372;  // consumer blocks of the running launch that have finished
constexpr size_t XCHG_STATUS_OFF = 2056;   // shared with the stand-alone all-reduce
constexpr size_t XCHG_DESC_OFF = 3072;     // the wf_xchg descriptor itself

__device__ __forceinline__ void xchg_red_release_sys(unsigned* p, unsigned v) {
    asm volatile("red.release.sys.global.add.u32 [%0], %1;\n" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ unsigned xchg_ld_acquire_sys(const unsigned* p) {
    unsigned v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];\n" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void xchg_st_peer32(void* p, uint32_t v) {
    asm volatile("st.relaxed.sys.global.u32 [%0], %1;\n" ::"l"(p), "r"(v) : "memory");
}

// The pushing kernels fetch the descriptor and the count of consumed exchanges into shared memory with asynchronous
// copies right after they have waited for their predecessors, and use them at their end: no round trip is left then.
// (The descriptor lives inside this rank's own buffer, so the counter's address follows from the descriptor's.)
constexpr int XCHG_SMEM_BYTES = 100;  // 96 bytes of descriptor (88 used) + the counter
__device__ __forceinline__ void xchg_fetch_async(const void* gdesc, uint8_t* sdst, int tid) {
    const uint8_t* g = static_cast<const uint8_t*>(gdesc);
    const uint32_t d = static_cast<uint32_t>(__cvta_generic_to_shared(sdst));
    if (tid < 6) asm volatile("cp.async.ca.shared.global [%0], [%1], 16;\n" ::"r"(d + 16 * tid), "l"(g + 16 * tid) : "memory");
    if (tid == 6) asm volatile("cp.async.ca.shared.global [%0], [%1], 4;\n" ::"r"(d + 96), "l"(g - XCHG_DESC_OFF + XCHG_PSTEP_OFF) : "memory");
}
__device__ __forceinline__ void xchg_fetch_wait(int tid) {
    if (tid < 7) asm volatile("cp.async.wait_all;\n" ::: "memory");
}

// The step this launch pushes: one more than the exchanges this rank has consumed.  Valid once the launch has waited for
// its predecessors in the stream (the consumer of the previous exchange among them).
__device__ __forceinline__ unsigned xchg_step(const wf_xchg* x) {
    const uint8_t* mine = static_cast<const uint8_t*>(x->peer[x->rank]);
    return *reinterpret_cast<const volatile unsigned*>(mine + XCHG_PSTEP_OFF) + 1;
}

// Copies rows [r0, r1) x tokens [m0, m1) of this rank's partial output y (16-bit elements, row stride ldy, N even, r0
// even) into the push region of every rank: two elements per thread and store.  Called by all `nthreads` threads of a group
// that have made their own stores to y visible to each other (a barrier) before.
__device__ __forceinline__ void xchg_push_block(const wf_xchg* x, unsigned step, const uint16_t* y, int64_t ldy, int N, int m0, int m1,
                                                int r0, int r1, int tid, int nthreads) {
    const int pairs = (r1 - r0) >> 1;
    const int total = (m1 - m0) * pairs;
    const uint64_t region = x->push_off + (static_cast<uint64_t>(step & 1) * x->world + x->rank) * x->slot_bytes;
    for (int w = tid; w < total; w += nthreads) {
        const int m = m0 + w / pairs, r = r0 + 2 * (w % pairs);
        const uint32_t v = *reinterpret_cast<const uint32_t*>(y + static_cast<int64_t>(m) * ldy + r);
        const uint64_t off = region + (static_cast<uint64_t>(m) * N + r) * 2;
        for (int pr = 0; pr < x->world; ++pr) xchg_st_peer32(static_cast<uint8_t*>(x->peer[pr]) + off, v);
    }
}

// After a CTA has pushed `elems` elements (all of its threads have passed a barrier since their peer stores): one thread
// reports them to every rank.  The release orders the CTA's stores, observed through the barrier, before the count.
__device__ __forceinline__ void xchg_report(const wf_xchg* x, unsigned step, unsigned elems) {
    for (int pr = 0; pr < x->world; ++pr)
        xchg_red_release_sys(reinterpret_cast<unsigned*>(static_cast<uint8_t*>(x->peer[pr]) + XCHG_PCOUNT_OFF) + (step & 1) * 8 + x->rank, elems);
}

}  // namespace wf
