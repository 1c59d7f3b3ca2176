// Stand-alone activation quantization to int8 (per token, or per tensor with the
// semantics of the reference's CPU operator).
#include "wf_common.cuh"

namespace wf {

constexpr int AQ_THREADS = 256;

__device__ __forceinline__ float block_max(float v, float* sh) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    int w = threadIdx.x >> 5, l = threadIdx.x & 31;
    if (l == 0) sh[w] = v;
    __syncthreads();
    float t = sh[0];
#pragma unroll
    for (int i = 1; i < AQ_THREADS / 32; ++i) t = fmaxf(t, sh[i]);
    __syncthreads();
    return t;
}

__device__ __forceinline__ int block_sum_int(int v, int* sh) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    int w = threadIdx.x >> 5, l = threadIdx.x & 31;
    if (l == 0) sh[w] = v;
    __syncthreads();
    int t = 0;
#pragma unroll
    for (int i = 0; i < AQ_THREADS / 32; ++i) t += sh[i];
    __syncthreads();
    return t;
}

// One block per token.  K % 8 == 0.
template <int DT>
__global__ void __launch_bounds__(AQ_THREADS)
    act_quant_token_kernel(const void* __restrict__ x, int64_t K, int64_t ldx, float eps, int8_t* __restrict__ q,
                           float* __restrict__ scale, int32_t* __restrict__ rowsum, int x_ready) {
    __shared__ float shf[AQ_THREADS / 32];
    __shared__ int shi[AQ_THREADS / 32];
    // chained with a programmatic dependency: the next kernel may start (the contraction fetches its first weights
    // meanwhile); x may come from the previous kernel and q may still be read by it, so everything else waits for it
    // -- unless the caller states that neither is the case (x_ready): then only the end of the grid waits, so that
    // whoever waits for this grid may still rely on everything ahead of it in the stream
    asm volatile("griddepcontrol.launch_dependents;\n" ::: "memory");
    if (!x_ready) asm volatile("griddepcontrol.wait;\n" ::: "memory");
    const int64_t m = blockIdx.x;
    float mx = 0.f;
    for (int64_t k = threadIdx.x * 8; k < K; k += AQ_THREADS * 8) {
        float f[8];
        load8<DT>(x, m * ldx + k, f);
#pragma unroll
        for (int i = 0; i < 8; ++i) mx = fmaxf(mx, fabsf(f[i]));
    }
    mx = block_max(mx, shf);
    const float s = act_scale_from_absmax<DT>(mx, eps);
    int sum = 0;
    for (int64_t k = threadIdx.x * 8; k < K; k += AQ_THREADS * 8) {
        float f[8];
        load8<DT>(x, m * ldx + k, f);
        uint32_t w0 = 0, w1 = 0;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            int a = quantize_one<DT>(f[i], s), b = quantize_one<DT>(f[4 + i], s);
            sum += a + b;
            w0 |= static_cast<uint32_t>(a & 0xff) << (8 * i);
            w1 |= static_cast<uint32_t>(b & 0xff) << (8 * i);
        }
        *reinterpret_cast<uint2*>(q + m * K + k) = make_uint2(w0, w1);
    }
    sum = block_sum_int(sum, shi);
    if (threadIdx.x == 0) {
        scale[m] = s;
        if (rowsum) rowsum[m] = sum;
    }
    // one block stays until the predecessor has completed, so that this grid does not end before it; the others leave
    if (x_ready && blockIdx.x == 0) asm volatile("griddepcontrol.wait;\n" ::: "memory");
}

// Per-tensor absmax: pass 1 reduces |x| into a float kept as ordered uint bits.
__global__ void __launch_bounds__(AQ_THREADS)
    tensor_absmax_kernel(const float* __restrict__ x, int64_t M, int64_t K, int64_t ldx, unsigned* __restrict__ maxbits) {
    __shared__ float shf[AQ_THREADS / 32];
    const int64_t total = M * (K / 4);
    float mx = 0.f;
    for (int64_t v = static_cast<int64_t>(blockIdx.x) * AQ_THREADS + threadIdx.x; v < total;
         v += static_cast<int64_t>(gridDim.x) * AQ_THREADS) {
        int64_t row = v / (K / 4), col = (v % (K / 4)) * 4;
        float4 f = __ldg(reinterpret_cast<const float4*>(x + row * ldx + col));
        mx = fmaxf(mx, fmaxf(fmaxf(fabsf(f.x), fabsf(f.y)), fmaxf(fabsf(f.z), fabsf(f.w))));
    }
    mx = block_max(mx, shf);
    if (threadIdx.x == 0) atomicMax(maxbits, __float_as_uint(mx));
}

// Pass 2: one block per row; scale = max/127, multiplier 127/max (both fp32 divisions), round to nearest even.
__global__ void __launch_bounds__(AQ_THREADS)
    tensor_quant_kernel(const float* __restrict__ x, int64_t K, int64_t ldx, const unsigned* __restrict__ maxbits,
                        int8_t* __restrict__ q, int32_t* __restrict__ rowsum) {
    __shared__ int shi[AQ_THREADS / 32];
    const int64_t m = blockIdx.x;
    float mx = __uint_as_float(*maxbits);
    if (mx < 1e-6f) mx = 1.0f;
    const float inv = __fdiv_rn(127.0f, mx);
    int sum = 0;
    for (int64_t k = threadIdx.x * 4; k < K; k += AQ_THREADS * 4) {
        float4 f = __ldg(reinterpret_cast<const float4*>(x + m * ldx + k));
        int a = quantize_one<WF_F32>(f.x, inv), b = quantize_one<WF_F32>(f.y, inv);
        int c = quantize_one<WF_F32>(f.z, inv), d = quantize_one<WF_F32>(f.w, inv);
        sum += a + b + c + d;
        *reinterpret_cast<uint32_t*>(q + m * K + k) = (a & 0xff) | ((b & 0xff) << 8) | ((c & 0xff) << 16) | ((d & 0xff) << 24);
    }
    sum = block_sum_int(sum, shi);
    if (threadIdx.x == 0 && rowsum) rowsum[m] = sum;
}

// Pass 3: the reduction cell held the absmax while pass 2 read it; turn it into the returned scale.
__global__ void publish_tensor_scale(float* scale) {
    float mx = scale[0];
    if (mx < 1e-6f) mx = 1.0f;
    scale[0] = __fdiv_rn(mx, 127.0f);
}

}  // namespace wf

using namespace wf;

static int act_quant_impl(const void* x, int x_dtype, int64_t M, int64_t K, int64_t ldx, int mode, float eps, int8_t* q, float* scale,
                          int32_t* rowsum, int x_ready, void* stream);

// The same with the row held in registers between the two passes (K <= 8 * AQ_THREADS * CHUNKS): x is read once, and all
// of a thread's loads are in flight together.
template <int DT, int CHUNKS>
__global__ void __launch_bounds__(AQ_THREADS)
    act_quant_token_reg_kernel(const void* __restrict__ x, int64_t K, int64_t ldx, float eps, int8_t* __restrict__ q,
                               float* __restrict__ scale, int32_t* __restrict__ rowsum, int x_ready) {
    __shared__ float shf[AQ_THREADS / 32];
    __shared__ int shi[AQ_THREADS / 32];
    asm volatile("griddepcontrol.launch_dependents;\n" ::: "memory");
    if (!x_ready) asm volatile("griddepcontrol.wait;\n" ::: "memory");
    const int64_t m = blockIdx.x;
    const int chunks = static_cast<int>(K >> 3);
    float f[CHUNKS][8];
#pragma unroll
    for (int c = 0; c < CHUNKS; ++c) {
        const int i = threadIdx.x + c * AQ_THREADS;
        if (i < chunks) {
            load8<DT>(x, m * ldx + 8 * static_cast<int64_t>(i), f[c]);
        } else {
#pragma unroll
            for (int e = 0; e < 8; ++e) f[c][e] = 0.f;
        }
    }
    float mx = 0.f;
#pragma unroll
    for (int c = 0; c < CHUNKS; ++c)
#pragma unroll
        for (int e = 0; e < 8; ++e) mx = fmaxf(mx, fabsf(f[c][e]));
    mx = block_max(mx, shf);
    const float s = act_scale_from_absmax<DT>(mx, eps);
    int sum = 0;
#pragma unroll
    for (int c = 0; c < CHUNKS; ++c) {
        const int i = threadIdx.x + c * AQ_THREADS;
        if (i < chunks) {
            uint32_t w0 = 0, w1 = 0;
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int a = quantize_one<DT>(f[c][e], s), b = quantize_one<DT>(f[c][4 + e], s);
                sum += a + b;
                w0 |= static_cast<uint32_t>(a & 0xff) << (8 * e);
                w1 |= static_cast<uint32_t>(b & 0xff) << (8 * e);
            }
            *reinterpret_cast<uint2*>(q + m * K + 8 * static_cast<int64_t>(i)) = make_uint2(w0, w1);
        }
    }
    sum = block_sum_int(sum, shi);
    if (threadIdx.x == 0) {
        scale[m] = s;
        if (rowsum) rowsum[m] = sum;
    }
    // one block stays until the predecessor has completed, so that this grid does not end before it; the others leave
    if (x_ready && blockIdx.x == 0) asm volatile("griddepcontrol.wait;\n" ::: "memory");
}

template <int DT>
static cudaError_t launch_token_quant(const cudaLaunchConfig_t& lc, const void* x, int64_t K, int64_t ldx, float eps, int8_t* q,
                                      float* scale, int32_t* rowsum, int x_ready) {
    const int64_t per_thread = ((K >> 3) + AQ_THREADS - 1) / AQ_THREADS;
    if (per_thread <= 2) return cudaLaunchKernelEx(&lc, act_quant_token_reg_kernel<DT, 2>, x, K, ldx, eps, q, scale, rowsum, x_ready);
    if (per_thread <= 4) return cudaLaunchKernelEx(&lc, act_quant_token_reg_kernel<DT, 4>, x, K, ldx, eps, q, scale, rowsum, x_ready);
    return cudaLaunchKernelEx(&lc, act_quant_token_kernel<DT>, x, K, ldx, eps, q, scale, rowsum, x_ready);
}

extern "C" int wf_act_quant_i8(const void* x, int x_dtype, int64_t M, int64_t K, int64_t ldx, int mode, float eps, int8_t* q,
                               float* scale, int32_t* rowsum, void* stream) {
    return act_quant_impl(x, x_dtype, M, K, ldx, mode, eps, q, scale, rowsum, 0, stream);
}

// Per-token quantization whose launch neither reads nor overwrites anything the kernels still running ahead of it use
// (x_ready != 0): see wf_prefill_quantize.
int wf_act_quant_token_ready(const void* x, int x_dtype, int64_t M, int64_t K, int64_t ldx, float eps, int8_t* q, float* scale,
                             int32_t* rowsum, int x_ready, void* stream) {
    return act_quant_impl(x, x_dtype, M, K, ldx, WF_ACT_PER_TOKEN, eps, q, scale, rowsum, x_ready, stream);
}

static int act_quant_impl(const void* x, int x_dtype, int64_t M, int64_t K, int64_t ldx, int mode, float eps, int8_t* q, float* scale,
                          int32_t* rowsum, int x_ready, void* stream) {
    WF_REQUIRE(x && q && scale, "wf_act_quant_i8: null pointer");
    WF_REQUIRE(M > 0 && K > 0 && K % 8 == 0, "wf_act_quant_i8: need M > 0 and K a positive multiple of 8 (M=%lld K=%lld)",
               (long long)M, (long long)K);
    WF_REQUIRE(M <= 0x7fffffff, "wf_act_quant_i8: M too large");
    WF_REQUIRE(is_float_dtype(x_dtype), "wf_act_quant_i8: unsupported dtype %d", x_dtype);
    WF_REQUIRE(ldx >= K && (ldx * dtype_size(x_dtype)) % 16 == 0 && reinterpret_cast<uintptr_t>(x) % 16 == 0,
               "wf_act_quant_i8: rows of x must be 16-byte aligned");
    WF_REQUIRE(reinterpret_cast<uintptr_t>(q) % 8 == 0, "wf_act_quant_i8: q must be 8-byte aligned");
    if (int rc = require_device()) return rc;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (mode == WF_ACT_PER_TOKEN) {
        cudaLaunchConfig_t lc = {};
        lc.gridDim = dim3(static_cast<unsigned>(M));
        lc.blockDim = dim3(AQ_THREADS);
        lc.stream = st;
        cudaLaunchAttribute attr[1];
        attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[0].val.programmaticStreamSerializationAllowed = 1;
        lc.attrs = attr;
        lc.numAttrs = 1;
        switch (x_dtype) {
            case WF_F32: WF_CUDA(launch_token_quant<WF_F32>(lc, x, K, ldx, eps, q, scale, rowsum, x_ready)); break;
            case WF_BF16: WF_CUDA(launch_token_quant<WF_BF16>(lc, x, K, ldx, eps, q, scale, rowsum, x_ready)); break;
            default: WF_CUDA(launch_token_quant<WF_F16>(lc, x, K, ldx, eps, q, scale, rowsum, x_ready)); break;
        }
    } else if (mode == WF_ACT_PER_TENSOR) {
        WF_REQUIRE(x_dtype == WF_F32, "wf_act_quant_i8: per-tensor mode takes fp32 input (as the operator it replaces)");
        // scale[0] doubles as the reduction cell: 0.0f has all-zero bits, the identity of the unsigned max
        WF_CUDA(cudaMemsetAsync(scale, 0, sizeof(float), st));
        int64_t blocks = (M * (K / 4) + AQ_THREADS - 1) / AQ_THREADS;
        if (blocks > 148 * 8) blocks = 148 * 8;
        tensor_absmax_kernel<<<(unsigned)blocks, AQ_THREADS, 0, st>>>(static_cast<const float*>(x), M, K, ldx,
                                                                     reinterpret_cast<unsigned*>(scale));
        tensor_quant_kernel<<<(unsigned)M, AQ_THREADS, 0, st>>>(static_cast<const float*>(x), K, ldx,
                                                                reinterpret_cast<const unsigned*>(scale), q, rowsum);
        publish_tensor_scale<<<1, 1, 0, st>>>(scale);
    } else {
        return fail(WF_E_ARG, "wf_act_quant_i8: unknown mode %d", mode);
    }
    WF_CUDA(cudaGetLastError());
    return WF_OK;
}
