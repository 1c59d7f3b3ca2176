// Small fused elementwise kernels around the BitLinear projections of a decoder layer (bf16 tensors):
// residual add + RMSNorm, RoPE + KV-cache write, gate activation x up.  They replace chains of framework
// kernels in the decode step; none of them is on the roofline of the path, they only remove launches.
#include "wf_common.cuh"

namespace wf {

__device__ __forceinline__ float bf(const __nv_bfloat16 v) { return __bfloat162float(v); }

// h[m, :] += delta[m, :] (when delta != nullptr); y[m, :] = h * rsqrt(mean(h^2) + eps) * w.  One block per row.
__global__ void __launch_bounds__(256) add_rmsnorm_kernel(__nv_bfloat16* __restrict__ h, const __nv_bfloat16* __restrict__ delta,
                                                          const __nv_bfloat16* __restrict__ w, __nv_bfloat16* __restrict__ y, int K,
                                                          float eps) {
    __shared__ float sh[8];
    const int64_t m = blockIdx.x;
    float ss = 0.f;
    for (int k = threadIdx.x * 2; k < K; k += 512) {
        __nv_bfloat162 a = *reinterpret_cast<const __nv_bfloat162*>(h + m * K + k);
        if (delta) {
            const __nv_bfloat162 d = *reinterpret_cast<const __nv_bfloat162*>(delta + m * K + k);
            a = __floats2bfloat162_rn(bf(a.x) + bf(d.x), bf(a.y) + bf(d.y));  // the residual stream stays bf16
            *reinterpret_cast<__nv_bfloat162*>(h + m * K + k) = a;
        }
        ss += bf(a.x) * bf(a.x) + bf(a.y) * bf(a.y);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    if ((threadIdx.x & 31) == 0) sh[threadIdx.x >> 5] = ss;
    __syncthreads();
    float tot = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) tot += sh[i];
    const float r = rsqrtf(tot / static_cast<float>(K) + eps);
    for (int k = threadIdx.x * 2; k < K; k += 512) {
        const __nv_bfloat162 a = *reinterpret_cast<const __nv_bfloat162*>(h + m * K + k);
        const __nv_bfloat162 g = *reinterpret_cast<const __nv_bfloat162*>(w + k);
        // normalise in fp32, round to bf16, then scale by the bf16 weight (the order of the unfused operator chain)
        const float n0 = bf(__float2bfloat16_rn(bf(a.x) * r)), n1 = bf(__float2bfloat16_rn(bf(a.y) * r));
        *reinterpret_cast<__nv_bfloat162*>(y + m * K + k) = __floats2bfloat162_rn(n0 * bf(g.x), n1 * bf(g.y));
    }
}

// Decode-step RoPE + cache write for one new token per sequence.
// q [B, nq*D] is rotated in place; k [B, nkv*D] is rotated and written to kcache[b, head, slot, :]; v is copied to
// vcache[b, head, slot, :].  cos/sin [T, D/2] fp32; slot = *pos % T is read on the device.
__global__ void rope_kv_kernel(__nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ k, const __nv_bfloat16* __restrict__ v,
                               const float* __restrict__ cosv, const float* __restrict__ sinv, const int64_t* __restrict__ pos,
                               __nv_bfloat16* __restrict__ kcache, __nv_bfloat16* __restrict__ vcache, int nq, int nkv, int D, int T) {
    const int b = blockIdx.x, half = D / 2;
    const int slot = static_cast<int>(*pos % T);
    const float* c = cosv + static_cast<int64_t>(slot) * half;
    const float* s = sinv + static_cast<int64_t>(slot) * half;
    for (int i = threadIdx.x; i < (nq + nkv) * half; i += blockDim.x) {
        const int head = i / half, j = i % half;
        if (head < nq) {
            __nv_bfloat16* p = q + (static_cast<int64_t>(b) * nq + head) * D;
            const float x1 = bf(p[j]), x2 = bf(p[j + half]);
            p[j] = __float2bfloat16_rn(x1 * c[j] - x2 * s[j]);
            p[j + half] = __float2bfloat16_rn(x2 * c[j] + x1 * s[j]);
        } else {
            const int hk = head - nq;
            const __nv_bfloat16* p = k + (static_cast<int64_t>(b) * nkv + hk) * D;
            __nv_bfloat16* dst = kcache + ((static_cast<int64_t>(b) * nkv + hk) * T + slot) * D;
            const float x1 = bf(p[j]), x2 = bf(p[j + half]);
            dst[j] = __float2bfloat16_rn(x1 * c[j] - x2 * s[j]);
            dst[j + half] = __float2bfloat16_rn(x2 * c[j] + x1 * s[j]);
        }
    }
    for (int i = threadIdx.x; i < nkv * D; i += blockDim.x) {
        const int hk = i / D, j = i % D;
        vcache[((static_cast<int64_t>(b) * nkv + hk) * T + slot) * D + j] = v[(static_cast<int64_t>(b) * nkv + hk) * D + j];
    }
}

// out = act(g) * u, act = SiLU (mode 0) or ReLU^2 (mode 1); intermediate rounded to bf16 like the unfused chain.
__global__ void act_mul_kernel(const __nv_bfloat16* __restrict__ g, const __nv_bfloat16* __restrict__ u, __nv_bfloat16* __restrict__ out,
                               int64_t n, int mode) {
    for (int64_t i = (static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x) * 2; i < n; i += static_cast<int64_t>(gridDim.x) * blockDim.x * 2) {
        const __nv_bfloat162 a = *reinterpret_cast<const __nv_bfloat162*>(g + i);
        const __nv_bfloat162 b = *reinterpret_cast<const __nv_bfloat162*>(u + i);
        float r[2];
        const float av[2] = {bf(a.x), bf(a.y)};
#pragma unroll
        for (int e = 0; e < 2; ++e) {
            float t;
            if (mode == 0) {
                t = av[e] / (1.0f + __expf(-av[e]));
            } else {
                const float rl = fmaxf(av[e], 0.f);
                t = bf(__float2bfloat16_rn(rl)) * bf(__float2bfloat16_rn(rl));
            }
            r[e] = bf(__float2bfloat16_rn(t));
        }
        *reinterpret_cast<__nv_bfloat162*>(out + i) = __floats2bfloat162_rn(r[0] * bf(b.x), r[1] * bf(b.y));
    }
}

}  // namespace wf

using namespace wf;

extern "C" int wf_add_rmsnorm_bf16(void* h, const void* delta, const void* weight, void* y, int64_t M, int64_t K, float eps,
                                   void* stream) {
    WF_REQUIRE(h && weight && y, "wf_add_rmsnorm_bf16: null pointer");
    WF_REQUIRE(M > 0 && K > 0 && K % 2 == 0 && M < (1LL << 31), "wf_add_rmsnorm_bf16: need M > 0 and an even K");
    if (int rc = require_device()) return rc;
    add_rmsnorm_kernel<<<static_cast<unsigned>(M), 256, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<__nv_bfloat16*>(h), static_cast<const __nv_bfloat16*>(delta), static_cast<const __nv_bfloat16*>(weight),
        static_cast<__nv_bfloat16*>(y), static_cast<int>(K), eps);
    WF_CUDA(cudaGetLastError());
    return WF_OK;
}

extern "C" int wf_rope_kv_bf16(void* q, const void* k, const void* v, const float* cos, const float* sin, const int64_t* pos,
                               void* kcache, void* vcache, int64_t B, int nq, int nkv, int D, int T, void* stream) {
    WF_REQUIRE(q && k && v && cos && sin && pos && kcache && vcache, "wf_rope_kv_bf16: null pointer");
    WF_REQUIRE(B > 0 && nq > 0 && nkv > 0 && D > 0 && D % 2 == 0 && T > 0, "wf_rope_kv_bf16: bad dimensions");
    if (int rc = require_device()) return rc;
    rope_kv_kernel<<<static_cast<unsigned>(B), 256, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<__nv_bfloat16*>(q), static_cast<const __nv_bfloat16*>(k), static_cast<const __nv_bfloat16*>(v), cos, sin, pos,
        static_cast<__nv_bfloat16*>(kcache), static_cast<__nv_bfloat16*>(vcache), nq, nkv, D, T);
    WF_CUDA(cudaGetLastError());
    return WF_OK;
}

extern "C" int wf_act_mul_bf16(const void* gate, const void* up, void* out, int64_t n, int mode, void* stream) {
    WF_REQUIRE(gate && up && out, "wf_act_mul_bf16: null pointer");
    WF_REQUIRE(n > 0 && n % 2 == 0 && (mode == 0 || mode == 1), "wf_act_mul_bf16: need an even element count and mode 0 or 1");
    if (int rc = require_device()) return rc;
    int64_t blocks = (n / 2 + 255) / 256;
    if (blocks > 148 * 8) blocks = 148 * 8;
    act_mul_kernel<<<static_cast<unsigned>(blocks), 256, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const __nv_bfloat16*>(gate), static_cast<const __nv_bfloat16*>(up), static_cast<__nv_bfloat16*>(out), n, mode);
    WF_CUDA(cudaGetLastError());
    return WF_OK;
}
