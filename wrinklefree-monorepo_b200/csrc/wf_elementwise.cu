// Small fused elementwise kernels around the BitLinear projections of a decoder layer (bf16 tensors):
// residual add + RMSNorm, RoPE + KV-cache write, gate activation x up.  They replace chains of framework
// kernels in the decode step.  With one token per sequence they are pure latency: every tensor is read with
// 16-byte loads that are all in flight at once, rows stay in registers between the reduction and the
// normalisation, and every kernel can be chained to its neighbours with a programmatic dependency (it lets the
// next kernel start at once and itself reads nothing that the previous kernel writes before it has waited).
#include "wf_common.cuh"
#include "wf_rowquant.cuh"

namespace wf {

__device__ __forceinline__ float bf(const __nv_bfloat16 v) { return __bfloat162float(v); }
__device__ __forceinline__ float bf_lo(uint32_t w) { return __uint_as_float(w << 16); }
__device__ __forceinline__ float bf_hi(uint32_t w) { return __uint_as_float(w & 0xffff0000u); }
__device__ __forceinline__ uint32_t pack_bf(float lo, float hi) {
    const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<const uint32_t*>(&v);
}
__device__ __forceinline__ float round_bf(float v) { return bf(__float2bfloat16_rn(v)); }
__device__ __forceinline__ void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;\n" ::: "memory"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;\n" ::: "memory"); }

constexpr int NORM_THREADS = 512;
constexpr int NORM_CHUNKS = 4;  // 8-element chunks per thread held in registers: rows up to 16384 elements

// h[m, :] += delta[m, :] (when delta != nullptr); y[m, :] = h * rsqrt(mean(h^2) + eps) * w.  One block per row.
// VEC: K % 8 == 0 and K <= NORM_THREADS * NORM_CHUNKS * 8, the row stays in registers; else two passes over global memory.
// With `q` (VEC only) the normalised row is also quantized to int8 per token, with the arithmetic of the stand-alone
// quantization kernel on the bf16 values (absmax, multiplier 127 / max rounded like torch's, round half to even): the
// projections that follow read q and q_scale and no kernel stands between the norm and them; y may then be null.
template <bool VEC>
__global__ void __launch_bounds__(NORM_THREADS) add_rmsnorm_kernel(__nv_bfloat16* __restrict__ h, const __nv_bfloat16* __restrict__ delta,
                                                                   const __nv_bfloat16* __restrict__ w, __nv_bfloat16* __restrict__ y,
                                                                   int K, float eps, int8_t* __restrict__ q, float* __restrict__ q_scale,
                                                                   float q_eps) {
    __shared__ float sh[NORM_THREADS / 32];
    pdl_trigger();
    const int64_t m = blockIdx.x;
    const int tid = threadIdx.x;
    float ss = 0.f;
    uint4 hv[NORM_CHUNKS], wv[NORM_CHUNKS];
    if constexpr (VEC) {
        const int chunks = K >> 3;
        // the norm weights do not depend on the previous kernel
#pragma unroll
        for (int c = 0; c < NORM_CHUNKS; ++c) {
            const int i = tid + c * NORM_THREADS;
            if (i < chunks) wv[c] = __ldg(reinterpret_cast<const uint4*>(w) + i);
        }
        pdl_wait();
        uint4 dv[NORM_CHUNKS];
        uint4* hrow = reinterpret_cast<uint4*>(h + m * K);
#pragma unroll
        for (int c = 0; c < NORM_CHUNKS; ++c) {
            const int i = tid + c * NORM_THREADS;
            if (i < chunks) {
                hv[c] = hrow[i];
                if (delta) dv[c] = __ldg(reinterpret_cast<const uint4*>(delta + m * K) + i);
            }
        }
#pragma unroll
        for (int c = 0; c < NORM_CHUNKS; ++c) {
            const int i = tid + c * NORM_THREADS;
            if (i < chunks) {
                uint32_t a[4] = {hv[c].x, hv[c].y, hv[c].z, hv[c].w};
                if (delta) {
                    const uint32_t d[4] = {dv[c].x, dv[c].y, dv[c].z, dv[c].w};
#pragma unroll
                    for (int e = 0; e < 4; ++e)  // the residual stream stays bf16
                        a[e] = pack_bf(bf_lo(a[e]) + bf_lo(d[e]), bf_hi(a[e]) + bf_hi(d[e]));
                    hv[c] = make_uint4(a[0], a[1], a[2], a[3]);
                    hrow[i] = hv[c];
                }
#pragma unroll
                for (int e = 0; e < 4; ++e) ss += bf_lo(a[e]) * bf_lo(a[e]) + bf_hi(a[e]) * bf_hi(a[e]);
            }
        }
    } else {
        pdl_wait();
        for (int k = tid * 2; k < K; k += NORM_THREADS * 2) {
            __nv_bfloat162 a = *reinterpret_cast<const __nv_bfloat162*>(h + m * K + k);
            if (delta) {
                const __nv_bfloat162 d = *reinterpret_cast<const __nv_bfloat162*>(delta + m * K + k);
                a = __floats2bfloat162_rn(bf(a.x) + bf(d.x), bf(a.y) + bf(d.y));
                *reinterpret_cast<__nv_bfloat162*>(h + m * K + k) = a;
            }
            ss += bf(a.x) * bf(a.x) + bf(a.y) * bf(a.y);
        }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    if ((tid & 31) == 0) sh[tid >> 5] = ss;
    __syncthreads();
    float tot = 0.f;
#pragma unroll
    for (int i = 0; i < NORM_THREADS / 32; ++i) tot += sh[i];
    const float r = rsqrtf(tot / static_cast<float>(K) + eps);
    // normalise in fp32, round to bf16, then scale by the bf16 weight (the order of the unfused operator chain)
    if constexpr (VEC) {
        const int chunks = K >> 3;
        uint4* yrow = y ? reinterpret_cast<uint4*>(y + m * K) : nullptr;
        uint32_t o[NORM_CHUNKS][4];
        float mx = 0.f;
#pragma unroll
        for (int c = 0; c < NORM_CHUNKS; ++c) {
            const int i = tid + c * NORM_THREADS;
            if (i < chunks) {
                const uint32_t a[4] = {hv[c].x, hv[c].y, hv[c].z, hv[c].w};
                const uint32_t g[4] = {wv[c].x, wv[c].y, wv[c].z, wv[c].w};
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    o[c][e] = pack_bf(round_bf(bf_lo(a[e]) * r) * bf_lo(g[e]), round_bf(bf_hi(a[e]) * r) * bf_hi(g[e]));
                    mx = fmaxf(mx, fmaxf(fabsf(bf_lo(o[c][e])), fabsf(bf_hi(o[c][e]))));
                }
                if (y) yrow[i] = make_uint4(o[c][0], o[c][1], o[c][2], o[c][3]);
            }
        }
        if (q) {
            quantize_row_bf16<NORM_THREADS, NORM_CHUNKS>(o, mx, chunks, tid, sh, q + m * K, q_scale + m, q_eps);
        }
    } else {
        for (int k = tid * 2; k < K; k += NORM_THREADS * 2) {
            const __nv_bfloat162 a = *reinterpret_cast<const __nv_bfloat162*>(h + m * K + k);
            const __nv_bfloat162 g = *reinterpret_cast<const __nv_bfloat162*>(w + k);
            *reinterpret_cast<__nv_bfloat162*>(y + m * K + k) =
                __floats2bfloat162_rn(round_bf(bf(a.x) * r) * bf(g.x), round_bf(bf(a.y) * r) * bf(g.y));
        }
    }
}

// Decode-step RoPE + cache write for one new token per sequence.  One block per (sequence, head): query heads are
// rotated in place; key heads are rotated and written to kcache[b, head, slot, :], and the same block copies the
// value head to vcache[b, head, slot, :].  cos/sin [T, D/2] fp32; the position *pos is read on the device
// (the caller keeps it below T; it is reduced modulo T only so that a stray value stays inside the tables).
__global__ void rope_kv_kernel(__nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ k, const __nv_bfloat16* __restrict__ v,
                               const float* __restrict__ cosv, const float* __restrict__ sinv, const int64_t* __restrict__ pos,
                               __nv_bfloat16* __restrict__ kcache, __nv_bfloat16* __restrict__ vcache, int nq, int nkv, int D, int T) {
    pdl_trigger();
    const int heads = nq + nkv, half = D / 2;
    const int b = blockIdx.x / heads, head = blockIdx.x % heads;
    pdl_wait();
    const int slot = static_cast<int>(*pos % T);
    const float* c = cosv + static_cast<int64_t>(slot) * half;
    const float* s = sinv + static_cast<int64_t>(slot) * half;
    if (head < nq) {
        __nv_bfloat16* p = q + (static_cast<int64_t>(b) * nq + head) * D;
        for (int j = threadIdx.x; j < half; j += blockDim.x) {
            const float x1 = bf(p[j]), x2 = bf(p[j + half]), cj = c[j], sj = s[j];
            p[j] = __float2bfloat16_rn(x1 * cj - x2 * sj);
            p[j + half] = __float2bfloat16_rn(x2 * cj + x1 * sj);
        }
    } else {
        const int hk = head - nq;
        const __nv_bfloat16* p = k + (static_cast<int64_t>(b) * nkv + hk) * D;
        const __nv_bfloat16* pv = v + (static_cast<int64_t>(b) * nkv + hk) * D;
        const int64_t at = ((static_cast<int64_t>(b) * nkv + hk) * T + slot) * D;
        for (int j = threadIdx.x; j < half; j += blockDim.x) {
            const float x1 = bf(p[j]), x2 = bf(p[j + half]), cj = c[j], sj = s[j];
            const __nv_bfloat16 v1 = pv[j], v2 = pv[j + half];
            kcache[at + j] = __float2bfloat16_rn(x1 * cj - x2 * sj);
            kcache[at + j + half] = __float2bfloat16_rn(x2 * cj + x1 * sj);
            vcache[at + j] = v1;
            vcache[at + j + half] = v2;
        }
    }
}

// out = act(g) * u, act = SiLU (mode 0) or ReLU^2 (mode 1); intermediate rounded to bf16 like the unfused chain.
__device__ __forceinline__ float act_one(float a, int mode) {
    float t;
    if (mode == 0) {
        t = a / (1.0f + __expf(-a));
    } else {
        const float rl = round_bf(fmaxf(a, 0.f));
        t = rl * rl;
    }
    return round_bf(t);
}
__global__ void __launch_bounds__(256) act_mul_kernel(const __nv_bfloat16* __restrict__ g, const __nv_bfloat16* __restrict__ u,
                                                      __nv_bfloat16* __restrict__ out, int64_t n, int mode) {
    pdl_trigger();
    pdl_wait();
    const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
    const int64_t tid = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    const int64_t n8 = n >> 3;
    for (int64_t i = tid; i < n8; i += stride) {
        const uint4 a = __ldg(reinterpret_cast<const uint4*>(g) + i), b = __ldg(reinterpret_cast<const uint4*>(u) + i);
        const uint32_t av[4] = {a.x, a.y, a.z, a.w}, bv[4] = {b.x, b.y, b.z, b.w};
        uint32_t o[4];
#pragma unroll
        for (int e = 0; e < 4; ++e)
            o[e] = pack_bf(act_one(bf_lo(av[e]), mode) * bf_lo(bv[e]), act_one(bf_hi(av[e]), mode) * bf_hi(bv[e]));
        reinterpret_cast<uint4*>(out)[i] = make_uint4(o[0], o[1], o[2], o[3]);
    }
    for (int64_t i = n8 * 8 + tid; i < n; i += stride)  // the tail of a length that is not a multiple of 8
        out[i] = __float2bfloat16_rn(act_one(bf(g[i]), mode) * bf(u[i]));
}

// act(g) * u of one token row per block, quantized to int8 per token on the way (and written as bf16 when `out` is given):
// the activation in front of down_proj together with the quantization that projection would otherwise run itself.
constexpr int AMQ_THREADS = 512;
constexpr int AMQ_CHUNKS = 4;  // rows up to 16384 elements
__global__ void __launch_bounds__(AMQ_THREADS) act_mul_quant_kernel(const __nv_bfloat16* __restrict__ g, const __nv_bfloat16* __restrict__ u,
                                                                    __nv_bfloat16* __restrict__ out, int8_t* __restrict__ q,
                                                                    float* __restrict__ q_scale, int I, int mode, float q_eps) {
    __shared__ float sh[AMQ_THREADS / 32];
    pdl_trigger();
    pdl_wait();
    const int64_t m = blockIdx.x;
    const int tid = threadIdx.x, chunks = I >> 3;
    uint32_t o[AMQ_CHUNKS][4];
    float mx = 0.f;
#pragma unroll
    for (int c = 0; c < AMQ_CHUNKS; ++c) {
        const int i = tid + c * AMQ_THREADS;
        if (i < chunks) {
            const uint4 a = __ldg(reinterpret_cast<const uint4*>(g + m * I) + i), b = __ldg(reinterpret_cast<const uint4*>(u + m * I) + i);
            const uint32_t av[4] = {a.x, a.y, a.z, a.w}, bv[4] = {b.x, b.y, b.z, b.w};
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                o[c][e] = pack_bf(act_one(bf_lo(av[e]), mode) * bf_lo(bv[e]), act_one(bf_hi(av[e]), mode) * bf_hi(bv[e]));
                mx = fmaxf(mx, fmaxf(fabsf(bf_lo(o[c][e])), fabsf(bf_hi(o[c][e]))));
            }
            if (out) reinterpret_cast<uint4*>(out + m * I)[i] = make_uint4(o[c][0], o[c][1], o[c][2], o[c][3]);
        }
    }
    quantize_row_bf16<AMQ_THREADS, AMQ_CHUNKS>(o, mx, chunks, tid, sh, q + m * I, q_scale + m, q_eps);
}

template <typename... KArgs, typename... Args>
static cudaError_t launch(void (*kernel)(KArgs...), unsigned grid, unsigned block, unsigned flags, void* stream, Args... args) {
    cudaLaunchConfig_t lc = {};
    lc.gridDim = dim3(grid);
    lc.blockDim = dim3(block);
    lc.stream = static_cast<cudaStream_t>(stream);
    cudaLaunchAttribute attr[1];
    if (flags & WF_FLAG_PDL) {
        attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[0].val.programmaticStreamSerializationAllowed = 1;
        lc.attrs = attr;
        lc.numAttrs = 1;
    }
    return cudaLaunchKernelEx(&lc, kernel, static_cast<KArgs>(args)...);
}

}  // namespace wf

using namespace wf;

extern "C" int wf_add_rmsnorm_bf16(void* h, const void* delta, const void* weight, void* y, int64_t M, int64_t K, float eps,
                                   unsigned flags, void* stream) {
    WF_REQUIRE(h && weight && y, "wf_add_rmsnorm_bf16: null pointer");
    WF_REQUIRE(M > 0 && K > 0 && K % 2 == 0 && M < (1LL << 31) && K < (1LL << 31), "wf_add_rmsnorm_bf16: need M > 0 and an even K");
    if (int rc = require_device()) return rc;
    auto al16 = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; };
    const bool vec = K % 8 == 0 && K <= static_cast<int64_t>(NORM_THREADS) * NORM_CHUNKS * 8 && al16(h) && al16(weight) && al16(y) &&
                     (!delta || al16(delta));
    WF_CUDA(launch(vec ? add_rmsnorm_kernel<true> : add_rmsnorm_kernel<false>, static_cast<unsigned>(M), NORM_THREADS, flags, stream,
                   static_cast<__nv_bfloat16*>(h), static_cast<const __nv_bfloat16*>(delta), static_cast<const __nv_bfloat16*>(weight),
                   static_cast<__nv_bfloat16*>(y), static_cast<int>(K), eps, static_cast<int8_t*>(nullptr), static_cast<float*>(nullptr), 0.f));
    return WF_OK;
}

extern "C" int wf_add_rmsnorm_quant_bf16(void* h, const void* delta, const void* weight, void* y, int8_t* q, float* q_scale, int64_t M,
                                         int64_t K, float eps, float quant_eps, unsigned flags, void* stream) {
    WF_REQUIRE(h && weight && q && q_scale, "wf_add_rmsnorm_quant_bf16: null pointer");
    auto al16 = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; };
    WF_REQUIRE(M > 0 && M < (1LL << 31) && K > 0 && K % 8 == 0 && K <= static_cast<int64_t>(NORM_THREADS) * NORM_CHUNKS * 8,
               "wf_add_rmsnorm_quant_bf16: K must be a multiple of 8, at most %d", NORM_THREADS * NORM_CHUNKS * 8);
    WF_REQUIRE(al16(h) && al16(weight) && (!y || al16(y)) && (!delta || al16(delta)) && (reinterpret_cast<uintptr_t>(q) & 7) == 0,
               "wf_add_rmsnorm_quant_bf16: tensors must be 16-byte aligned (q: 8)");
    if (int rc = require_device()) return rc;
    WF_CUDA(launch(add_rmsnorm_kernel<true>, static_cast<unsigned>(M), NORM_THREADS, flags, stream, static_cast<__nv_bfloat16*>(h),
                   static_cast<const __nv_bfloat16*>(delta), static_cast<const __nv_bfloat16*>(weight), static_cast<__nv_bfloat16*>(y),
                   static_cast<int>(K), eps, q, q_scale, quant_eps));
    return WF_OK;
}

extern "C" int wf_act_mul_quant_bf16(const void* gate, const void* up, void* out, int8_t* q, float* q_scale, int64_t M, int64_t I, int mode,
                                     float quant_eps, unsigned flags, void* stream) {
    WF_REQUIRE(gate && up && q && q_scale, "wf_act_mul_quant_bf16: null pointer");
    WF_REQUIRE(M > 0 && M < (1LL << 31) && I > 0 && I % 8 == 0 && I <= static_cast<int64_t>(AMQ_THREADS) * AMQ_CHUNKS * 8 && (mode == 0 || mode == 1),
               "wf_act_mul_quant_bf16: rows of a multiple of 8 elements, at most %d; mode 0 or 1", AMQ_THREADS * AMQ_CHUNKS * 8);
    auto al16 = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; };
    WF_REQUIRE(al16(gate) && al16(up) && (!out || al16(out)) && (reinterpret_cast<uintptr_t>(q) & 7) == 0,
               "wf_act_mul_quant_bf16: tensors must be 16-byte aligned (q: 8)");
    if (int rc = require_device()) return rc;
    WF_CUDA(launch(act_mul_quant_kernel, static_cast<unsigned>(M), static_cast<unsigned>(AMQ_THREADS), flags, stream,
                   static_cast<const __nv_bfloat16*>(gate), static_cast<const __nv_bfloat16*>(up), static_cast<__nv_bfloat16*>(out), q, q_scale,
                   static_cast<int>(I), mode, quant_eps));
    return WF_OK;
}

extern "C" int wf_rope_kv_bf16(void* q, const void* k, const void* v, const float* cos, const float* sin, const int64_t* pos,
                               void* kcache, void* vcache, int64_t B, int nq, int nkv, int D, int T, unsigned flags, void* stream) {
    WF_REQUIRE(q && k && v && cos && sin && pos && kcache && vcache, "wf_rope_kv_bf16: null pointer");
    WF_REQUIRE(B > 0 && nq > 0 && nkv > 0 && D > 0 && D % 2 == 0 && T > 0 && B * (nq + nkv) < (1LL << 31), "wf_rope_kv_bf16: bad dimensions");
    if (int rc = require_device()) return rc;
    int threads = (D / 2 + 31) / 32 * 32;
    if (threads > 256) threads = 256;
    WF_CUDA(launch(rope_kv_kernel, static_cast<unsigned>(B * (nq + nkv)), static_cast<unsigned>(threads), flags, stream,
                   static_cast<__nv_bfloat16*>(q), static_cast<const __nv_bfloat16*>(k), static_cast<const __nv_bfloat16*>(v), cos, sin, pos,
                   static_cast<__nv_bfloat16*>(kcache), static_cast<__nv_bfloat16*>(vcache), nq, nkv, D, T));
    return WF_OK;
}

extern "C" int wf_act_mul_bf16(const void* gate, const void* up, void* out, int64_t n, int mode, unsigned flags, void* stream) {
    WF_REQUIRE(gate && up && out, "wf_act_mul_bf16: null pointer");
    WF_REQUIRE(n > 0 && (mode == 0 || mode == 1), "wf_act_mul_bf16: need a positive element count and mode 0 or 1");
    auto al16 = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; };
    WF_REQUIRE(al16(gate) && al16(up) && al16(out), "wf_act_mul_bf16: tensors must be 16-byte aligned");
    if (int rc = require_device()) return rc;
    int64_t blocks = ((n + 7) / 8 + 255) / 256;
    if (blocks > 148 * 8) blocks = 148 * 8;
    WF_CUDA(launch(act_mul_kernel, static_cast<unsigned>(blocks), 256u, flags, stream, static_cast<const __nv_bfloat16*>(gate),
                   static_cast<const __nv_bfloat16*>(up), static_cast<__nv_bfloat16*>(out), n, mode));
    return WF_OK;
}
