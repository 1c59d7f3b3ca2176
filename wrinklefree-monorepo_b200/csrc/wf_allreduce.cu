// One-shot all-reduce over peer memory for the small tensors that follow a row-parallel projection in the decode
// step (hidden x tokens: 8 KB for one token of the 8B shape).  At that size a library all-reduce is latency: several
// launches and protocol round trips.  Here every rank
//   1. copies its partial tensor into its own exported buffer (two slots, alternating by step),
//   2. stores the step number into a flag word of its own INSIDE EVERY PEER'S buffer (after a system-scope fence),
//   3. polls the flag words in its OWN buffer until every peer has published the step (bounded; local memory, so the
//      polling crosses no link),
//   4. reads all partial tensors through peer pointers (plain loads over NVLink, no multicast) and sums them in rank
//      order in fp32, so every rank obtains bit-identical results.
// Two slots are enough: a rank overwrites slot s & 1 at step s + 2 only after it has seen every peer's flag of step
// s + 1, which a peer stores only after it has finished reading step s.
// The buffers are plain cudaMalloc allocations exported with CUDA IPC handles (one process per GPU).
#include <cuda_runtime.h>

#include <cstdint>
#include <cstring>
#include <new>

#include "wf_common.cuh"
#include "wf_xchg.cuh"
#include "wf_rowquant.cuh"

namespace wf {

constexpr int AR_MAX_RANKS = 8;
constexpr int AR_MAX_CTAS = 32;
constexpr int AR_THREADS = 512;
constexpr size_t AR_FLAG_BYTES = AR_MAX_CTAS * AR_MAX_RANKS * sizeof(unsigned);  // flags[cta][rank]
constexpr size_t AR_HEADER = 4096;  // flags, step counter, ticket, status
constexpr unsigned AR_SPIN_LIMIT = 1u << 22;

struct ArPeers {
    uint8_t* base[AR_MAX_RANKS];
};

struct ArCtx {
    int world, rank, device;
    size_t max_bytes;
    uint8_t* local;
    ArPeers peers;
    bool connected;
};

__device__ __forceinline__ unsigned ld_acquire_sys(const unsigned* p) {
    unsigned v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];\n" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void st_release_sys(unsigned* p, unsigned v) {
    asm volatile("st.release.sys.global.u32 [%0], %1;\n" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint4 ld_peer16(const void* p) {  // another GPU's memory: never served from this SM's L1
    uint4 v;
    asm volatile("ld.relaxed.sys.global.v4.u32 {%0,%1,%2,%3}, [%4];\n" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
    return v;
}

template <int DT>
__device__ __forceinline__ void accumulate8(const uint4& u, float (&acc)[8]) {
    const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        if constexpr (DT == WF_BF16) {
            acc[2 * i] += __uint_as_float(w[i] << 16);
            acc[2 * i + 1] += __uint_as_float(w[i] & 0xffff0000u);
        } else {
            const float2 v = __half22float2(*reinterpret_cast<const __half2*>(&w[i]));
            acc[2 * i] += v.x;
            acc[2 * i + 1] += v.y;
        }
    }
}

// header of a rank's buffer: flags[cta][rank] | step (at 2048) | ticket (2052) | status (2056)
// n16: 16-byte chunks of the tensor; CTA c handles the chunks c, c + grid, ...
template <int DT>
__global__ void __launch_bounds__(AR_THREADS) allreduce_kernel(ArPeers peers, int world, int rank, size_t slot_bytes,
                                                               const uint4* __restrict__ in, uint4* __restrict__ out, int64_t n16) {
    asm volatile("griddepcontrol.launch_dependents;\n" ::: "memory");
    uint8_t* mine = peers.base[rank];
    unsigned* step_word = reinterpret_cast<unsigned*>(mine + 2048);
    unsigned* ticket = reinterpret_cast<unsigned*>(mine + 2052);
    unsigned* status = reinterpret_cast<unsigned*>(mine + 2056);
    const int tid = threadIdx.x, cta = blockIdx.x;
    asm volatile("griddepcontrol.wait;\n" ::: "memory");  // the partial tensor comes from the previous kernel
    const unsigned step = *reinterpret_cast<volatile unsigned*>(step_word) + 1;
    const size_t slot = AR_HEADER + (step & 1) * slot_bytes;

    // 1. publish the partial tensor
    uint4* my_slot = reinterpret_cast<uint4*>(mine + slot);
    for (int64_t i = cta * static_cast<int64_t>(AR_THREADS) + tid; i < n16; i += static_cast<int64_t>(gridDim.x) * AR_THREADS)
        my_slot[i] = in[i];
    __threadfence_system();
    __syncthreads();
    // 2. tell every peer (and this rank itself)
    if (tid < world) st_release_sys(reinterpret_cast<unsigned*>(peers.base[tid]) + cta * AR_MAX_RANKS + rank, step);
    // 3. wait for every peer's flag of this step, in this rank's own memory
    if (tid < world) {
        const unsigned* f = reinterpret_cast<const unsigned*>(mine) + cta * AR_MAX_RANKS + tid;
        unsigned it = 0;
        // flags only grow; a difference below 2^31 means "not yet there"
        while (static_cast<int>(ld_acquire_sys(f) - step) < 0) {
            if (++it > AR_SPIN_LIMIT) {
                atomicExch(status, static_cast<unsigned>(WF_E_LIMIT));
                break;
            }
            __nanosleep(20);
        }
    }
    __syncthreads();
    // 4. sum in rank order
    for (int64_t i = cta * static_cast<int64_t>(AR_THREADS) + tid; i < n16; i += static_cast<int64_t>(gridDim.x) * AR_THREADS) {
        if constexpr (DT == WF_F32) {
            float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
            for (int r = 0; r < world; ++r) {
                const uint4 u = ld_peer16(peers.base[r] + slot + i * 16);
                acc.x += __uint_as_float(u.x); acc.y += __uint_as_float(u.y); acc.z += __uint_as_float(u.z); acc.w += __uint_as_float(u.w);
            }
            out[i] = make_uint4(__float_as_uint(acc.x), __float_as_uint(acc.y), __float_as_uint(acc.z), __float_as_uint(acc.w));
        } else {
            float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
            for (int r = 0; r < world; ++r) accumulate8<DT>(ld_peer16(peers.base[r] + slot + i * 16), acc);
            uint32_t o[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                if constexpr (DT == WF_BF16) {
                    const __nv_bfloat162 t2 = __floats2bfloat162_rn(acc[2 * j], acc[2 * j + 1]);
                    o[j] = *reinterpret_cast<const uint32_t*>(&t2);
                } else {
                    const __half2 t2 = __floats2half2_rn(acc[2 * j], acc[2 * j + 1]);
                    o[j] = *reinterpret_cast<const uint32_t*>(&t2);
                }
            }
            out[i] = make_uint4(o[0], o[1], o[2], o[3]);
        }
    }
    // 5. the last CTA to finish advances the step
    __syncthreads();
    if (tid == 0) {
        __threadfence();
        if (atomicAdd(ticket, 1u) == gridDim.x - 1) {
            *ticket = 0;
            *reinterpret_cast<volatile unsigned*>(step_word) = step;
        }
    }
}

// ---- consumer of a fused exchange: delta = sum of the pushed partial outputs, then h += delta, y = rmsnorm(h) * w ----
// One block per token row; the row stays in registers.  The arithmetic after the sum is that of the residual add +
// RMSNorm kernel of this library, the sum itself that of allreduce_kernel (fp32 in rank order, rounded to bf16).
constexpr int XR_THREADS = 512;
constexpr int XR_CHUNKS = 4;  // 8-element chunks per thread: rows up to 16384 elements

__device__ __forceinline__ float xr_lo(uint32_t w) { return __uint_as_float(w << 16); }
__device__ __forceinline__ float xr_hi(uint32_t w) { return __uint_as_float(w & 0xffff0000u); }
__device__ __forceinline__ uint32_t xr_pack(float lo, float hi) {
    const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<const uint32_t*>(&v);
}
__device__ __forceinline__ float xr_round(float v) { return __bfloat162float(__float2bfloat16_rn(v)); }

__global__ void __launch_bounds__(XR_THREADS) reduce_add_rmsnorm_kernel(const wf_xchg x, __nv_bfloat16* __restrict__ h,
                                                                        const __nv_bfloat16* __restrict__ w, __nv_bfloat16* __restrict__ y,
                                                                        int K, float eps, int8_t* __restrict__ q, float* __restrict__ q_scale,
                                                                        float q_eps) {
    __shared__ float sh[XR_THREADS / 32];
    asm volatile("griddepcontrol.launch_dependents;\n" ::: "memory");
    const int64_t m = blockIdx.x;
    const int tid = threadIdx.x;
    const int chunks = K >> 3;
    uint4 hv[XR_CHUNKS], wv[XR_CHUNKS];
#pragma unroll
    for (int c = 0; c < XR_CHUNKS; ++c) {  // the norm weights do not depend on the previous kernel
        const int i = tid + c * XR_THREADS;
        if (i < chunks) wv[c] = __ldg(reinterpret_cast<const uint4*>(w) + i);
    }
    asm volatile("griddepcontrol.wait;\n" ::: "memory");
    uint8_t* mine = static_cast<uint8_t*>(x.peer[x.rank]);
    // the count of consumed exchanges and both slots' counters are requested together: one round trip, not two
    const volatile unsigned* pstep_p = reinterpret_cast<volatile unsigned*>(mine + XCHG_PSTEP_OFF);
    unsigned* const counts0 = reinterpret_cast<unsigned*>(mine + XCHG_PCOUNT_OFF);
    unsigned first[2] = {0u, 0u};
    if (tid < x.world) {
        first[0] = xchg_ld_acquire_sys(counts0 + tid);
        first[1] = xchg_ld_acquire_sys(counts0 + 8 + tid);
    }
    const unsigned step = *pstep_p + 1;
    unsigned* counts = counts0 + (step & 1) * 8;
    // every rank has delivered all of its M x K elements of this step: poll this rank's own counters (bounded)
    if (tid < x.world) {
        const unsigned want = gridDim.x * static_cast<unsigned>(K);
        unsigned it = 0;
        while ((it == 0 ? first[step & 1] : xchg_ld_acquire_sys(counts + tid)) < want) {
            if (++it > AR_SPIN_LIMIT) {
                atomicExch(reinterpret_cast<unsigned*>(mine + XCHG_STATUS_OFF), static_cast<unsigned>(WF_E_LIMIT));
                break;
            }
            __nanosleep(20);
        }
    }
    __syncthreads();
    const uint8_t* slot = mine + x.push_off + static_cast<uint64_t>(step & 1) * x.world * x.slot_bytes;
    uint4* hrow = reinterpret_cast<uint4*>(h + m * K);
    float ss = 0.f;
#pragma unroll
    for (int c = 0; c < XR_CHUNKS; ++c) {
        const int i = tid + c * XR_THREADS;
        if (i < chunks) {
            float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
            for (int r = 0; r < x.world; ++r)  // pushed by peers: read past this SM's L1
                accumulate8<WF_BF16>(ld_peer16(slot + r * x.slot_bytes + (static_cast<uint64_t>(m) * K + 8 * static_cast<uint64_t>(i)) * 2), acc);
            const uint4 hh = hrow[i];
            uint32_t a[4] = {hh.x, hh.y, hh.z, hh.w};
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const uint32_t d = xr_pack(acc[2 * e], acc[2 * e + 1]);  // delta, rounded to bf16 like the all-reduced tensor
                a[e] = xr_pack(xr_lo(a[e]) + xr_lo(d), xr_hi(a[e]) + xr_hi(d));  // the residual stream stays bf16
                ss += xr_lo(a[e]) * xr_lo(a[e]) + xr_hi(a[e]) * xr_hi(a[e]);
            }
            hv[c] = make_uint4(a[0], a[1], a[2], a[3]);
            hrow[i] = hv[c];
        }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    if ((tid & 31) == 0) sh[tid >> 5] = ss;
    __syncthreads();
    float tot = 0.f;
#pragma unroll
    for (int i = 0; i < XR_THREADS / 32; ++i) tot += sh[i];
    const float rn = rsqrtf(tot / static_cast<float>(K) + eps);
    uint4* yrow = y ? reinterpret_cast<uint4*>(y + m * K) : nullptr;
    uint32_t o[XR_CHUNKS][4];
    float mx = 0.f;
#pragma unroll
    for (int c = 0; c < XR_CHUNKS; ++c) {
        const int i = tid + c * XR_THREADS;
        if (i < chunks) {
            const uint32_t a[4] = {hv[c].x, hv[c].y, hv[c].z, hv[c].w};
            const uint32_t g[4] = {wv[c].x, wv[c].y, wv[c].z, wv[c].w};
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                o[c][e] = xr_pack(xr_round(xr_lo(a[e]) * rn) * xr_lo(g[e]), xr_round(xr_hi(a[e]) * rn) * xr_hi(g[e]));
                mx = fmaxf(mx, fmaxf(fabsf(xr_lo(o[c][e])), fabsf(xr_hi(o[c][e]))));
            }
            if (y) yrow[i] = make_uint4(o[c][0], o[c][1], o[c][2], o[c][3]);
        }
    }
    // the per-token int8 quantization of the projections that follow, as in the residual add + RMSNorm kernel
    if (q) quantize_row_bf16<XR_THREADS, XR_CHUNKS>(o, mx, chunks, tid, sh, q + m * K, q_scale + m, q_eps);
    // the last block to finish advances this rank's count of consumed exchanges
    __syncthreads();
    if (tid == 0) {
        __threadfence();
        unsigned* ticket = reinterpret_cast<unsigned*>(mine + XCHG_CTICKET_OFF);
        if (atomicAdd(ticket, 1u) == gridDim.x - 1) {
            *ticket = 0;
            for (int r = 0; r < x.world; ++r) counts[r] = 0;  // the slot's next use is two exchanges away
            __threadfence();
            *reinterpret_cast<volatile unsigned*>(mine + XCHG_PSTEP_OFF) = step;
        }
    }
}

}  // namespace wf

using namespace wf;

extern "C" int wf_ar_handle_bytes(void) { return static_cast<int>(sizeof(cudaIpcMemHandle_t)); }

extern "C" int wf_ar_init(int world, int rank, size_t max_bytes, void** ctx_out, unsigned char* handle_out) {
    WF_REQUIRE(ctx_out && handle_out, "wf_ar_init: null pointer");
    WF_REQUIRE(world >= 2 && world <= AR_MAX_RANKS && rank >= 0 && rank < world, "wf_ar_init: 2..%d ranks", AR_MAX_RANKS);
    WF_REQUIRE(max_bytes >= 16 && max_bytes % 16 == 0 && max_bytes <= (64u << 20), "wf_ar_init: max_bytes must be a multiple of 16, at most 64 MiB");
    if (int rc = require_device()) return rc;
    ArCtx* c = new (std::nothrow) ArCtx();
    WF_REQUIRE(c, "wf_ar_init: out of host memory");
    c->world = world; c->rank = rank; c->max_bytes = max_bytes; c->connected = false;
    WF_CUDA(cudaGetDevice(&c->device));
    // header | two slots of the stand-alone all-reduce | two push slots of `world` source regions each
    const size_t total = AR_HEADER + 2 * max_bytes + 2 * static_cast<size_t>(world) * max_bytes;
    void* p = nullptr;
    cudaError_t e = cudaMalloc(&p, total);
    if (e != cudaSuccess) {
        delete c;
        return cuda_fail(e, "cudaMalloc of the exchange buffer");
    }
    c->local = static_cast<uint8_t*>(p);
    e = cudaMemset(p, 0, AR_HEADER);
    cudaIpcMemHandle_t h;
    if (e == cudaSuccess) e = cudaIpcGetMemHandle(&h, p);
    if (e != cudaSuccess) {
        cudaFree(p);
        delete c;
        return cuda_fail(e, "cudaIpcGetMemHandle");
    }
    std::memcpy(handle_out, &h, sizeof(h));
    for (int r = 0; r < AR_MAX_RANKS; ++r) c->peers.base[r] = nullptr;
    c->peers.base[rank] = c->local;
    *ctx_out = c;
    return WF_OK;
}

// handles: world x wf_ar_handle_bytes() bytes, entry r = the handle that rank r obtained from wf_ar_init
extern "C" int wf_ar_connect(void* ctx, const unsigned char* handles) {
    ArCtx* c = static_cast<ArCtx*>(ctx);
    WF_REQUIRE(c && handles, "wf_ar_connect: null pointer");
    WF_REQUIRE(!c->connected, "wf_ar_connect: already connected");
    for (int r = 0; r < c->world; ++r) {
        if (r == c->rank) continue;
        cudaIpcMemHandle_t h;
        std::memcpy(&h, handles + static_cast<size_t>(r) * sizeof(h), sizeof(h));
        void* p = nullptr;
        WF_CUDA(cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess));
        c->peers.base[r] = static_cast<uint8_t*>(p);
    }
    wf_xchg d = {};
    d.world = c->world;
    d.rank = c->rank;
    d.slot_bytes = c->max_bytes;
    d.push_off = AR_HEADER + 2 * c->max_bytes;
    for (int r = 0; r < c->world; ++r) d.peer[r] = c->peers.base[r];
    WF_CUDA(cudaMemcpy(c->local + XCHG_DESC_OFF, &d, sizeof(d), cudaMemcpyHostToDevice));
    c->connected = true;
    return WF_OK;
}

extern "C" int wf_ar_xchg(void* ctx, const void** dev_desc_out) {
    ArCtx* c = static_cast<ArCtx*>(ctx);
    WF_REQUIRE(c && dev_desc_out, "wf_ar_xchg: null pointer");
    WF_REQUIRE(c->connected, "wf_ar_xchg: wf_ar_connect has not run");
    *dev_desc_out = c->local + XCHG_DESC_OFF;
    return WF_OK;
}

extern "C" int wf_ar_reduce_add_rmsnorm_quant(void* ctx, void* h, const void* weight, void* y, int8_t* q, float* q_scale, int64_t M, int64_t K,
                                              float eps, float quant_eps, unsigned flags, void* stream);

extern "C" int wf_ar_reduce_add_rmsnorm(void* ctx, void* h, const void* weight, void* y, int64_t M, int64_t K, float eps, unsigned flags,
                                        void* stream) {
    WF_REQUIRE(y, "wf_ar_reduce_add_rmsnorm: null pointer");
    return wf_ar_reduce_add_rmsnorm_quant(ctx, h, weight, y, nullptr, nullptr, M, K, eps, 0.f, flags, stream);
}

extern "C" int wf_ar_reduce_add_rmsnorm_quant(void* ctx, void* h, const void* weight, void* y, int8_t* q, float* q_scale, int64_t M, int64_t K,
                                              float eps, float quant_eps, unsigned flags, void* stream) {
    ArCtx* c = static_cast<ArCtx*>(ctx);
    WF_REQUIRE(c && h && weight && (y || q) && (!q || q_scale), "wf_ar_reduce_add_rmsnorm: null pointer");
    WF_REQUIRE(!q || (reinterpret_cast<uintptr_t>(q) & 7) == 0, "wf_ar_reduce_add_rmsnorm: q must be 8-byte aligned");
    WF_REQUIRE(c->connected, "wf_ar_reduce_add_rmsnorm: wf_ar_connect has not run");
    WF_REQUIRE(M >= 1 && K >= 8 && K % 8 == 0 && K <= XR_THREADS * XR_CHUNKS * 8, "wf_ar_reduce_add_rmsnorm: K must be a multiple of 8, at most %d",
               XR_THREADS * XR_CHUNKS * 8);
    WF_REQUIRE(static_cast<size_t>(M) * K * 2 <= c->max_bytes, "wf_ar_reduce_add_rmsnorm: %lld x %lld exceeds the exchange's %zu bytes",
               (long long)M, (long long)K, c->max_bytes);
    WF_REQUIRE((reinterpret_cast<uintptr_t>(h) | reinterpret_cast<uintptr_t>(weight) | reinterpret_cast<uintptr_t>(y)) % 16 == 0,
               "wf_ar_reduce_add_rmsnorm: tensors must be 16-byte aligned");  // a null y passes
    cudaLaunchConfig_t lc = {};
    lc.gridDim = dim3(static_cast<unsigned>(M));
    lc.blockDim = dim3(XR_THREADS);
    lc.stream = static_cast<cudaStream_t>(stream);
    cudaLaunchAttribute attr[1];
    if (flags & WF_FLAG_PDL) {
        attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[0].val.programmaticStreamSerializationAllowed = 1;
        lc.attrs = attr;
        lc.numAttrs = 1;
    }
    wf_xchg desc = {};
    desc.world = c->world;
    desc.rank = c->rank;
    desc.slot_bytes = c->max_bytes;
    desc.push_off = AR_HEADER + 2 * c->max_bytes;
    for (int r = 0; r < c->world; ++r) desc.peer[r] = c->peers.base[r];
    WF_CUDA(cudaLaunchKernelEx(&lc, reduce_add_rmsnorm_kernel, desc, static_cast<__nv_bfloat16*>(h), static_cast<const __nv_bfloat16*>(weight),
                               static_cast<__nv_bfloat16*>(y), static_cast<int>(K), eps, q, q_scale, quant_eps));
    return WF_OK;
}

extern "C" int wf_ar_allreduce(void* ctx, const void* in, void* out, int64_t n, int dtype, unsigned flags, void* stream) {
    ArCtx* c = static_cast<ArCtx*>(ctx);
    WF_REQUIRE(c && in && out, "wf_ar_allreduce: null pointer");
    WF_REQUIRE(c->connected, "wf_ar_allreduce: wf_ar_connect has not run");
    WF_REQUIRE(dtype == WF_BF16 || dtype == WF_F16 || dtype == WF_F32, "wf_ar_allreduce: bf16, f16 or f32");
    const int64_t bytes = n * (dtype == WF_F32 ? 4 : 2);
    WF_REQUIRE(n > 0 && bytes % 16 == 0 && static_cast<size_t>(bytes) <= c->max_bytes,
               "wf_ar_allreduce: %lld bytes; need a multiple of 16, at most %zu", static_cast<long long>(bytes), c->max_bytes);
    WF_REQUIRE((reinterpret_cast<uintptr_t>(in) | reinterpret_cast<uintptr_t>(out)) % 16 == 0, "wf_ar_allreduce: tensors must be 16-byte aligned");
    const int64_t n16 = bytes / 16;
    int64_t grid = (n16 + AR_THREADS - 1) / AR_THREADS;
    if (grid > AR_MAX_CTAS) grid = AR_MAX_CTAS;
    cudaLaunchConfig_t lc = {};
    lc.gridDim = dim3(static_cast<unsigned>(grid));
    lc.blockDim = dim3(AR_THREADS);
    lc.stream = static_cast<cudaStream_t>(stream);
    cudaLaunchAttribute attr[1];
    if (flags & WF_FLAG_PDL) {
        attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[0].val.programmaticStreamSerializationAllowed = 1;
        lc.attrs = attr;
        lc.numAttrs = 1;
    }
    const uint4* in4 = static_cast<const uint4*>(in);
    uint4* out4 = static_cast<uint4*>(out);
    if (dtype == WF_BF16)
        WF_CUDA(cudaLaunchKernelEx(&lc, allreduce_kernel<WF_BF16>, c->peers, c->world, c->rank, c->max_bytes, in4, out4, n16));
    else if (dtype == WF_F16)
        WF_CUDA(cudaLaunchKernelEx(&lc, allreduce_kernel<WF_F16>, c->peers, c->world, c->rank, c->max_bytes, in4, out4, n16));
    else
        WF_CUDA(cudaLaunchKernelEx(&lc, allreduce_kernel<WF_F32>, c->peers, c->world, c->rank, c->max_bytes, in4, out4, n16));
    return WF_OK;
}

// 0 = no wait ran out; WF_E_LIMIT otherwise (the word is cleared)
extern "C" int wf_ar_status(void* ctx, int* out) {
    ArCtx* c = static_cast<ArCtx*>(ctx);
    WF_REQUIRE(c && out, "wf_ar_status: null pointer");
    unsigned v = 0;
    WF_CUDA(cudaMemcpy(&v, c->local + 2056, sizeof(v), cudaMemcpyDeviceToHost));
    if (v) WF_CUDA(cudaMemset(c->local + 2056, 0, sizeof(v)));
    *out = static_cast<int>(v);
    return WF_OK;
}

// this rank's count of completed all-reduces (waits for the device)
extern "C" int wf_ar_step(void* ctx, unsigned* out) {
    ArCtx* c = static_cast<ArCtx*>(ctx);
    WF_REQUIRE(c && out, "wf_ar_step: null pointer");
    WF_CUDA(cudaDeviceSynchronize());
    unsigned pulled = 0, pushed = 0;
    WF_CUDA(cudaMemcpy(&pulled, c->local + 2048, sizeof(unsigned), cudaMemcpyDeviceToHost));
    WF_CUDA(cudaMemcpy(&pushed, c->local + XCHG_PSTEP_OFF, sizeof(unsigned), cudaMemcpyDeviceToHost));
    *out = pulled > pushed ? pulled : pushed;  // the stand-alone all-reduce and the fused exchange count separately
    return WF_OK;
}

// Re-synchronisation after a wait that ran out: every rank sets the same step, larger than any flag published so far
// (flags only grow, so stale flags read as "not yet there"); the ticket and the status word are cleared.
extern "C" int wf_ar_set_step(void* ctx, unsigned step) {
    ArCtx* c = static_cast<ArCtx*>(ctx);
    WF_REQUIRE(c, "wf_ar_set_step: null pointer");
    WF_CUDA(cudaDeviceSynchronize());
    const unsigned words[3] = {step, 0u, 0u};  // step | ticket | status
    WF_CUDA(cudaMemcpy(c->local + 2048, words, sizeof(words), cudaMemcpyHostToDevice));
    const unsigned pwords[18] = {0u, 0u, 0u, 0u, 0u, 0u, 0u, 0u, 0u, 0u, 0u, 0u, 0u, 0u, 0u, 0u, step, 0u};  // delivered elements [2][8] | consumed exchanges | consumer ticket
    WF_CUDA(cudaMemcpy(c->local + XCHG_PCOUNT_OFF, pwords, sizeof(pwords), cudaMemcpyHostToDevice));
    return WF_OK;
}

extern "C" int wf_ar_destroy(void* ctx) {
    ArCtx* c = static_cast<ArCtx*>(ctx);
    if (!c) return WF_OK;
    for (int r = 0; r < c->world; ++r)
        if (r != c->rank && c->peers.base[r]) cudaIpcCloseMemHandle(c->peers.base[r]);
    cudaFree(c->local);
    delete c;
    return WF_OK;
}
