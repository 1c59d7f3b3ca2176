// Per-token int8 quantization of a row that a block holds in registers — shared by the kernels that quantize their own
// result (residual add + RMSNorm, gate activation, the consumer of a fused tensor-parallel exchange).
#pragma once

#include "wf_common.cuh"

namespace wf {

__device__ __forceinline__ float rq_lo(uint32_t w) { return __uint_as_float(w << 16); }
__device__ __forceinline__ float rq_hi(uint32_t w) { return __uint_as_float(w & 0xffff0000u); }

// Per-token int8 quantization of a row that a block holds in registers as packed bf16 pairs (chunk c of thread t = elements
// 8 * (t + c * THREADS) .. + 7): block-wide absmax, then the arithmetic of act_quant_token_kernel<bf16>.  `sh` is a
// scratch of THREADS / 32 floats that the caller no longer reads.
template <int THREADS, int CHUNKS>
__device__ __forceinline__ void quantize_row_bf16(const uint32_t (&o)[CHUNKS][4], float mx, int chunks, int tid, float* sh, int8_t* qrow,
                                                  float* scale_out, float q_eps) {
#pragma unroll
    for (int s = 16; s > 0; s >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, s));
    __syncthreads();  // the scratch is free
    if ((tid & 31) == 0) sh[tid >> 5] = mx;
    __syncthreads();
    float tot = sh[0];
#pragma unroll
    for (int i = 1; i < THREADS / 32; ++i) tot = fmaxf(tot, sh[i]);
    const float sc = act_scale_from_absmax<WF_BF16>(tot, q_eps);
#pragma unroll
    for (int c = 0; c < CHUNKS; ++c) {
        const int i = tid + c * THREADS;
        if (i < chunks) {
            uint32_t w0 = 0, w1 = 0;
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                const int a0 = quantize_one<WF_BF16>(rq_lo(o[c][e]), sc), a1 = quantize_one<WF_BF16>(rq_hi(o[c][e]), sc);
                const int b0 = quantize_one<WF_BF16>(rq_lo(o[c][2 + e]), sc), b1 = quantize_one<WF_BF16>(rq_hi(o[c][2 + e]), sc);
                w0 |= (static_cast<uint32_t>(a0 & 0xff) << (16 * e)) | (static_cast<uint32_t>(a1 & 0xff) << (16 * e + 8));
                w1 |= (static_cast<uint32_t>(b0 & 0xff) << (16 * e)) | (static_cast<uint32_t>(b1 & 0xff) << (16 * e + 8));
            }
            *reinterpret_cast<uint2*>(qrow + 8 * static_cast<int64_t>(i)) = make_uint2(w0, w1);
        }
    }
    if (tid == 0) *scale_out = sc;
}

}  // namespace wf
