// Weight-side kernels: absmean ternarization + 2-bit packing, layout conversion.
//
// Data layout in HBM.  Packed weights are row-major [N, K/4] bytes holding
// code = w + 1.  In WF16 every 32-bit little-endian word covers 16 consecutive
// weights k0..k0+15: byte b, bit pair j holds weight k0 + 4*j + b, so that
// (word >> 2j) & 0x03030303 is four consecutive weights as four bytes, the
// operand shape of an int8 dot product.  I2S is the 128-weight block layout of
// the reference's CPU kernels.
#include <atomic>

#include "wf_common.cuh"

namespace wf {

constexpr int PACK_THREADS = 256;
constexpr int WORDS_PER_THREAD = 4;                                      // 64 weights per thread
constexpr int PACK_WEIGHTS_PER_BLOCK = PACK_THREADS * WORDS_PER_THREAD * 16;  // 16384

__device__ __forceinline__ double block_sum(double v, double* sh) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    int w = threadIdx.x >> 5, l = threadIdx.x & 31;
    if (l == 0) sh[w] = v;
    __syncthreads();
    double t = 0.0;
    if (threadIdx.x == 0) {
        for (int i = 0; i < (blockDim.x >> 5); ++i) t += sh[i];
        sh[0] = t;
    }
    __syncthreads();
    t = sh[0];
    __syncthreads();
    return t;
}

// Pass 1: per-block sum of |w| (after the optional cast) in fp64, fixed order.
template <int WDT, int MODE>
__global__ void __launch_bounds__(PACK_THREADS) abs_sum_kernel(const void* __restrict__ w, int64_t N, int64_t K,
                                                               int64_t ldw, double* __restrict__ partial) {
    __shared__ double sh[PACK_THREADS / 32];
    const int64_t total_vec = N * (K / 8);  // units of 8 weights
    double s = 0.0;
    for (int64_t v = static_cast<int64_t>(blockIdx.x) * PACK_THREADS + threadIdx.x; v < total_vec;
         v += static_cast<int64_t>(gridDim.x) * PACK_THREADS) {
        int64_t row = v / (K / 8), col = (v % (K / 8)) * 8;
        float f[8];
        load8<WDT>(w, row * ldw + col, f);
        double a = 0.0;
#pragma unroll
        for (int i = 0; i < 8; ++i) a += static_cast<double>(fabsf(rnd<MODE>(f[i])));
        s += a;
    }
    double t = block_sum(s, sh);
    if (threadIdx.x == 0) partial[blockIdx.x] = t;
}

// Pass 2: every block re-reduces the partials in the same order, derives the
// scale, ternarizes and packs.  One thread produces four output words from 64
// consecutive weights.
template <int WDT, int MODE>
__global__ void __launch_bounds__(PACK_THREADS)
    ternarize_pack_kernel(const void* __restrict__ w, int64_t N, int64_t K, int64_t ldw, const double* __restrict__ partial,
                          int npartial, float eps, uint8_t* __restrict__ codes, float* __restrict__ scale_out) {
    __shared__ double sh[PACK_THREADS / 32];
    double s = 0.0;
    for (int i = threadIdx.x; i < npartial; i += PACK_THREADS) s += partial[i];
    // the per-thread strided sums depend only on npartial and the block size: identical in every block
    double total = block_sum(s, sh);
    float mean = static_cast<float>(total / static_cast<double>(N * K));
    float q_mul, dq;
    if constexpr (MODE == WF_F32) {
        mean = fmaxf(mean, eps);
        q_mul = mean;  // codes = rint(w / mean)
        dq = mean;
    } else {
        mean = rnd<MODE>(fmaxf(rnd<MODE>(mean), eps));
        q_mul = rnd<MODE>(__frcp_rn(mean));  // codes = rint(rnd(w * scale))
        dq = rnd<MODE>(__frcp_rn(q_mul));
    }
    if (blockIdx.x == 0 && threadIdx.x == 0) {
        scale_out[0] = dq;
        scale_out[1] = q_mul;
    }
    const int64_t chunks_per_row = K / 64;
    const int64_t total_chunks = N * chunks_per_row;
    for (int64_t c = static_cast<int64_t>(blockIdx.x) * PACK_THREADS + threadIdx.x; c < total_chunks;
         c += static_cast<int64_t>(gridDim.x) * PACK_THREADS) {
        int64_t row = c / chunks_per_row, col = (c % chunks_per_row) * 64;
        uint32_t words[4];
#pragma unroll
        for (int wd = 0; wd < 4; ++wd) {
            float f[16];
            float(&lo)[8] = *reinterpret_cast<float(*)[8]>(&f[0]);
            float(&hi)[8] = *reinterpret_cast<float(*)[8]>(&f[8]);
            load8<WDT>(w, row * ldw + col + wd * 16, lo);
            load8<WDT>(w, row * ldw + col + wd * 16 + 8, hi);
            uint32_t word = 0;
#pragma unroll
            for (int i = 0; i < 16; ++i) {
                float t;
                if constexpr (MODE == WF_F32)
                    t = rintf(__fdiv_rn(f[i], q_mul));
                else
                    t = rintf(rnd<MODE>(__fmul_rn(rnd<MODE>(f[i]), q_mul)));
                int code = static_cast<int>(fminf(fmaxf(t, -1.f), 1.f)) + 1;
                int j = i >> 2, b = i & 3;  // weight 4j + b -> byte b, bit pair j
                word |= static_cast<uint32_t>(code) << (8 * b + 2 * j);
            }
            words[wd] = word;
        }
        *reinterpret_cast<uint4*>(codes + row * (K / 4) + col / 4) = make_uint4(words[0], words[1], words[2], words[3]);
    }
}

// ---- layout conversion ----

// code (0..2) of logical weight (n, k) in a packed buffer of the given layout
__device__ __forceinline__ uint32_t fetch_code(const uint8_t* __restrict__ src, int layout, int64_t N, int64_t K, int64_t n,
                                               int64_t k) {
    switch (layout) {
        case WF_LAYOUT_WF16: {
            int r = static_cast<int>(k & 15);
            uint8_t byte = src[n * (K / 4) + (k >> 4) * 4 + (r & 3)];
            return (byte >> (2 * (r >> 2))) & 3u;
        }
        case WF_LAYOUT_I2S: {
            int r = static_cast<int>(k & 127);
            uint8_t byte = src[n * (K / 4) + (k >> 7) * 32 + (r & 31)];
            return (byte >> (6 - 2 * (r >> 5))) & 3u;
        }
        case WF_LAYOUT_SEQ_LSB:
            return (src[n * (K / 4) + (k >> 2)] >> (2 * (k & 3))) & 3u;
        case WF_LAYOUT_SEQ_MSB:
            return (src[n * (K / 4) + (k >> 2)] >> (6 - 2 * (k & 3))) & 3u;
        default: {  // WF_LAYOUT_HF: [N/4, K]
            int64_t q = N / 4;
            return (src[(n % q) * K + k] >> (2 * (n / q))) & 3u;
        }
    }
}

// logical weight (inside its row) stored at (byte, bit pair s) of a row-major destination layout
__device__ __forceinline__ int64_t dst_weight(int layout, int64_t byte, int s) {
    switch (layout) {
        case WF_LAYOUT_WF16: return (byte >> 2) * 16 + 4 * s + (byte & 3);
        case WF_LAYOUT_I2S: return (byte >> 5) * 128 + 32 * (3 - s) + (byte & 31);
        case WF_LAYOUT_SEQ_LSB: return 4 * byte + s;
        default: return 4 * byte + (3 - s);  // WF_LAYOUT_SEQ_MSB
    }
}

// one thread per output byte
__global__ void repack_kernel(const uint8_t* __restrict__ src, int src_layout, uint8_t* __restrict__ dst, int dst_layout,
                              int64_t N, int64_t K, const int8_t* __restrict__ ternary) {
    const int64_t total = N * (K / 4);
    for (int64_t o = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; o < total;
         o += static_cast<int64_t>(gridDim.x) * blockDim.x) {
        int64_t n = o / (K / 4), byte = o % (K / 4);
        uint32_t out = 0;
#pragma unroll
        for (int s = 0; s < 4; ++s) {
            const int64_t k = dst_weight(dst_layout, byte, s);
            uint32_t code = ternary ? static_cast<uint32_t>(ternary[n * K + k] + 1) : fetch_code(src, src_layout, N, K, n, k);
            out |= (code & 3u) << (2 * s);
        }
        dst[o] = static_cast<uint8_t>(out);
    }
}

// ---- the max-abs quantizers of the inference side ----
// absmax over the whole matrix: non-negative floats order like their bit patterns, one atomicMax per block
template <int WDT>
__global__ void abs_max_kernel(const void* __restrict__ w, int64_t N, int64_t K, int64_t ldw, unsigned* __restrict__ maxbits) {
    float mx = 0.f;
    const int64_t total = N * K;
    for (int64_t o = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; o < total;
         o += static_cast<int64_t>(gridDim.x) * blockDim.x)
        mx = fmaxf(mx, fabsf(load1<WDT>(w, (o / K) * ldw + o % K)));
#pragma unroll
    for (int s = 16; s > 0; s >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, s));
    if ((threadIdx.x & 31) == 0) atomicMax(maxbits, __float_as_uint(mx));
}

// one thread per output byte; rule 0: codes by thresholds at +-0.5 of w / max, rule 1: by sign with a 1e-6 dead zone
template <int WDT>
__global__ void maxabs_pack_kernel(const void* __restrict__ w, int64_t N, int64_t K, int64_t ldw, int rule, int dst_layout,
                                   const unsigned* __restrict__ maxbits, uint8_t* __restrict__ dst, float* __restrict__ scale_out) {
    float mx = __uint_as_float(*maxbits);
    if (rule == WF_MAXABS_HALF && mx < 1e-6f) mx = 1.0f;
    if (blockIdx.x == 0 && threadIdx.x == 0) *scale_out = mx;
    const int64_t total = N * (K / 4);
    for (int64_t o = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; o < total;
         o += static_cast<int64_t>(gridDim.x) * blockDim.x) {
        const int64_t n = o / (K / 4), byte = o % (K / 4);
        uint32_t out = 0;
#pragma unroll
        for (int s = 0; s < 4; ++s) {
            const float v = load1<WDT>(w, n * ldw + dst_weight(dst_layout, byte, s));
            uint32_t code = 1;
            if (rule == WF_MAXABS_HALF) {
                const float t = __fdiv_rn(v, mx);
                code = t > 0.5f ? 2u : (t < -0.5f ? 0u : 1u);
            } else if (fabs(static_cast<double>(v)) >= 1e-6) {
                code = static_cast<double>(v) * static_cast<double>(mx) > 0.0 ? 2u : 0u;
            }
            out |= code << (2 * s);
        }
        dst[o] = static_cast<uint8_t>(out);
    }
}

__global__ void unpack_kernel(const uint8_t* __restrict__ src, int layout, int8_t* __restrict__ ternary, int64_t N,
                              int64_t K) {
    const int64_t total = N * K;
    for (int64_t o = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; o < total;
         o += static_cast<int64_t>(gridDim.x) * blockDim.x)
        ternary[o] = static_cast<int8_t>(static_cast<int>(fetch_code(src, layout, N, K, o / K, o % K)) - 1);
}

constexpr int PACK_MAX_GRID = 148 * 8;  // blocks of the two packing kernels = partial sums in the scratch

static int pack_grid(int64_t N, int64_t K) {
    int64_t blocks = (N * K + PACK_WEIGHTS_PER_BLOCK - 1) / PACK_WEIGHTS_PER_BLOCK;
    if (blocks < 1) blocks = 1;
    if (blocks > PACK_MAX_GRID) blocks = PACK_MAX_GRID;
    return static_cast<int>(blocks);
}

template <int WDT>
static int launch_pack(const void* w, int64_t N, int64_t K, int64_t ldw, int mode, float eps, uint8_t* codes, float* scale,
                       double* partial, cudaStream_t st) {
    int grid = pack_grid(N, K);
    switch (mode) {
        case WF_PACK_FP32:
            abs_sum_kernel<WDT, WF_F32><<<grid, PACK_THREADS, 0, st>>>(w, N, K, ldw, partial);
            ternarize_pack_kernel<WDT, WF_F32><<<grid, PACK_THREADS, 0, st>>>(w, N, K, ldw, partial, grid, eps, codes, scale);
            break;
        case WF_PACK_CAST_BF16:
            abs_sum_kernel<WDT, WF_BF16><<<grid, PACK_THREADS, 0, st>>>(w, N, K, ldw, partial);
            ternarize_pack_kernel<WDT, WF_BF16><<<grid, PACK_THREADS, 0, st>>>(w, N, K, ldw, partial, grid, eps, codes, scale);
            break;
        default:
            abs_sum_kernel<WDT, WF_F16><<<grid, PACK_THREADS, 0, st>>>(w, N, K, ldw, partial);
            ternarize_pack_kernel<WDT, WF_F16><<<grid, PACK_THREADS, 0, st>>>(w, N, K, ldw, partial, grid, eps, codes, scale);
            break;
    }
    WF_CUDA(cudaGetLastError());
    return WF_OK;
}

}  // namespace wf

using namespace wf;

extern "C" {

size_t wf_pack_scratch_bytes(int64_t N, int64_t K) {
    if (N <= 0 || K <= 0) return 0;
    return static_cast<size_t>(pack_grid(N, K)) * sizeof(double);
}

int wf_pack_ternary(const void* w, int w_dtype, int64_t N, int64_t K, int64_t ldw, int mode, float eps, uint8_t* codes_out,
                    float* scale_out, void* scratch, size_t scratch_bytes, void* stream) {
    WF_REQUIRE(w && codes_out && scale_out && scratch, "wf_pack_ternary: null pointer");
    WF_REQUIRE(N > 0 && K > 0 && K % 64 == 0, "wf_pack_ternary: need N > 0 and K a positive multiple of 64 (N=%lld K=%lld)",
               (long long)N, (long long)K);
    WF_REQUIRE(is_float_dtype(w_dtype), "wf_pack_ternary: unsupported weight dtype %d", w_dtype);
    WF_REQUIRE(mode >= WF_PACK_FP32 && mode <= WF_PACK_CAST_F16, "wf_pack_ternary: unknown mode %d", mode);
    WF_REQUIRE(ldw >= K && (ldw * dtype_size(w_dtype)) % 16 == 0, "wf_pack_ternary: row stride must cover K and keep rows 16-byte aligned");
    WF_REQUIRE(reinterpret_cast<uintptr_t>(w) % 16 == 0 && reinterpret_cast<uintptr_t>(codes_out) % 16 == 0 &&
                   reinterpret_cast<uintptr_t>(scratch) % 8 == 0,
               "wf_pack_ternary: w and codes_out must be 16-byte aligned, scratch 8-byte aligned");
    if (scratch_bytes < wf_pack_scratch_bytes(N, K))
        return fail(WF_E_SCRATCH, "wf_pack_ternary: scratch of %zu bytes, need %zu", scratch_bytes, wf_pack_scratch_bytes(N, K));
    if (int rc = require_device()) return rc;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    double* partial = static_cast<double*>(scratch);
    switch (w_dtype) {
        case WF_F32: return launch_pack<WF_F32>(w, N, K, ldw, mode, eps, codes_out, scale_out, partial, st);
        case WF_BF16: return launch_pack<WF_BF16>(w, N, K, ldw, mode, eps, codes_out, scale_out, partial, st);
        default: return launch_pack<WF_F16>(w, N, K, ldw, mode, eps, codes_out, scale_out, partial, st);
    }
}

static int check_layout_dims(const char* who, int layout, int64_t N, int64_t K) {
    WF_REQUIRE(N > 0 && K > 0, "%s: empty matrix", who);
    switch (layout) {
        case WF_LAYOUT_WF16: WF_REQUIRE(K % 16 == 0, "%s: WF16 needs K %% 16 == 0 (K=%lld)", who, (long long)K); break;
        case WF_LAYOUT_I2S: WF_REQUIRE(K % 128 == 0, "%s: I2_S needs K %% 128 == 0 (K=%lld)", who, (long long)K); break;
        case WF_LAYOUT_SEQ_LSB:
        case WF_LAYOUT_SEQ_MSB: WF_REQUIRE(K % 4 == 0, "%s: sequential layouts need K %% 4 == 0", who); break;
        case WF_LAYOUT_HF: WF_REQUIRE(N % 4 == 0 && K % 4 == 0, "%s: HF layout needs N %% 4 == 0 and K %% 4 == 0", who); break;
        default: return fail(WF_E_ARG, "%s: unknown layout %d", who, layout);
    }
    return WF_OK;
}

static int grid_for(int64_t total) {
    int64_t b = (total + 255) / 256;
    if (b > 148 * 16) b = 148 * 16;
    return static_cast<int>(b < 1 ? 1 : b);
}

int wf_repack(const uint8_t* src, int src_layout, uint8_t* dst, int dst_layout, int64_t N, int64_t K, void* stream) {
    WF_REQUIRE(src && dst, "wf_repack: null pointer");
    WF_REQUIRE(dst_layout >= WF_LAYOUT_WF16 && dst_layout <= WF_LAYOUT_SEQ_MSB, "wf_repack: destination must be a row-major layout (not HF)");
    if (int rc = check_layout_dims("wf_repack(src)", src_layout, N, K)) return rc;
    if (int rc = check_layout_dims("wf_repack(dst)", dst_layout, N, K)) return rc;
    if (int rc = require_device()) return rc;
    repack_kernel<<<grid_for(N * (K / 4)), 256, 0, static_cast<cudaStream_t>(stream)>>>(src, src_layout, dst, dst_layout, N, K,
                                                                                     nullptr);
    WF_CUDA(cudaGetLastError());
    return WF_OK;
}

int wf_pack_codes(const int8_t* ternary, uint8_t* dst, int layout, int64_t N, int64_t K, void* stream) {
    WF_REQUIRE(ternary && dst, "wf_pack_codes: null pointer");
    WF_REQUIRE(layout >= WF_LAYOUT_WF16 && layout <= WF_LAYOUT_SEQ_MSB, "wf_pack_codes: layout must be row-major (not HF)");
    if (int rc = check_layout_dims("wf_pack_codes", layout, N, K)) return rc;
    if (int rc = require_device()) return rc;
    repack_kernel<<<grid_for(N * (K / 4)), 256, 0, static_cast<cudaStream_t>(stream)>>>(nullptr, 0, dst, layout, N, K, ternary);
    WF_CUDA(cudaGetLastError());
    return WF_OK;
}

int wf_unpack_codes(const uint8_t* src, int layout, int8_t* ternary, int64_t N, int64_t K, void* stream) {
    WF_REQUIRE(src && ternary, "wf_unpack_codes: null pointer");
    if (int rc = check_layout_dims("wf_unpack_codes", layout, N, K)) return rc;
    if (int rc = require_device()) return rc;
    unpack_kernel<<<grid_for(N * K), 256, 0, static_cast<cudaStream_t>(stream)>>>(src, layout, ternary, N, K);
    WF_CUDA(cudaGetLastError());
    return WF_OK;
}

int wf_quantize_maxabs(const void* w, int w_dtype, int64_t N, int64_t K, int64_t ldw, int rule, int dst_layout,
                       uint8_t* codes_out, float* scale_out, void* stream) {
    WF_REQUIRE(w && codes_out && scale_out, "wf_quantize_maxabs: null pointer");
    WF_REQUIRE(is_float_dtype(w_dtype), "wf_quantize_maxabs: unsupported weight dtype %d", w_dtype);
    WF_REQUIRE(rule == WF_MAXABS_HALF || rule == WF_MAXABS_SIGN, "wf_quantize_maxabs: unknown rule %d", rule);
    WF_REQUIRE(dst_layout >= WF_LAYOUT_WF16 && dst_layout <= WF_LAYOUT_SEQ_MSB, "wf_quantize_maxabs: destination must be a row-major layout");
    WF_REQUIRE(ldw >= K, "wf_quantize_maxabs: row stride must cover K");
    if (int rc = check_layout_dims("wf_quantize_maxabs", dst_layout, N, K)) return rc;
    if (int rc = require_device()) return rc;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    // the running maximum lives in the second float of scale_out until the packing kernel has read it
    unsigned* maxbits = reinterpret_cast<unsigned*>(scale_out) + 1;
    WF_CUDA(cudaMemsetAsync(maxbits, 0, sizeof(unsigned), st));
    const int g1 = grid_for(N * K), g2 = grid_for(N * (K / 4));
    switch (w_dtype) {
        case WF_F32:
            abs_max_kernel<WF_F32><<<g1, 256, 0, st>>>(w, N, K, ldw, maxbits);
            maxabs_pack_kernel<WF_F32><<<g2, 256, 0, st>>>(w, N, K, ldw, rule, dst_layout, maxbits, codes_out, scale_out);
            break;
        case WF_BF16:
            abs_max_kernel<WF_BF16><<<g1, 256, 0, st>>>(w, N, K, ldw, maxbits);
            maxabs_pack_kernel<WF_BF16><<<g2, 256, 0, st>>>(w, N, K, ldw, rule, dst_layout, maxbits, codes_out, scale_out);
            break;
        default:
            abs_max_kernel<WF_F16><<<g1, 256, 0, st>>>(w, N, K, ldw, maxbits);
            maxabs_pack_kernel<WF_F16><<<g2, 256, 0, st>>>(w, N, K, ldw, rule, dst_layout, maxbits, codes_out, scale_out);
            break;
    }
    WF_CUDA(cudaGetLastError());
    return WF_OK;
}
}

// ---------------------------------------------------------------------------------------------
// Allocation-free variant of wf_pack_ternary.
//
// Some hosts of this library may not allocate device memory at the point where they pack weights:
// a serving process whose own pool has claimed the GPU and forbids cudaMalloc inside layer code,
// or a latency-critical thread that cannot afford the implicit device synchronisation of an
// allocation.  wf_pack_ternary needs a small scratch buffer (the per-block partial sums of |w|);
// here that scratch is a fixed array that lives in the library image on every GPU that loads it
// (WF_PACK_NOALLOC_SCRATCH_BYTES, held until the process exits).  Nothing is allocated or freed by
// this entry point, neither through the CUDA runtime nor through any other library.
//
// The first call on a device looks up the device address of the array (the host-side symbol is
// only a handle, not an address a kernel may use); make that first call outside any stream capture.
// All calls on a device share the one array: two calls whose kernels overlap on the GPU (different
// streams) race on it.  Every launch overwrites the part of the array it later reads, so nothing
// has to be cleared between calls.
// ---------------------------------------------------------------------------------------------
namespace wf {

constexpr int NOALLOC_MAX_PARTIALS = PACK_MAX_GRID;  // the largest grid launch_pack ever uses
static __device__ __align__(256) double g_pack_noalloc_scratch[NOALLOC_MAX_PARTIALS];

constexpr int NOALLOC_MAX_DEVICES = 64;
static std::atomic<double*> g_noalloc_ptr[NOALLOC_MAX_DEVICES];  // device address of the array, per device (zero-initialised)

// Set-up, once per device, with that device current.
static int noalloc_scratch(double** out) {
    int dev = -1;
    WF_CUDA(cudaGetDevice(&dev));
    if (dev < 0 || dev >= NOALLOC_MAX_DEVICES) return fail(WF_E_LIMIT, "wf_pack_ternary_noalloc: device index %d not supported", dev);
    if (!g_noalloc_ptr[dev].load(std::memory_order_acquire)) {
        double* ptr = nullptr;
        cudaError_t e = cudaGetSymbolAddress(reinterpret_cast<void**>(&ptr), g_pack_noalloc_scratch);
        if (e != cudaSuccess) return cuda_fail(e, "cudaGetSymbolAddress(g_pack_noalloc_scratch)");
        if (!ptr) return fail(WF_E_DEVICE, "wf_pack_ternary_noalloc: no device address for the scratch array");
        g_noalloc_ptr[dev].store(ptr, std::memory_order_release);
    }
    *out = g_noalloc_ptr[dev].load(std::memory_order_acquire);
    return WF_OK;
}

}  // namespace wf

extern "C" size_t wf_pack_noalloc_scratch_bytes(void) { return sizeof(double) * wf::NOALLOC_MAX_PARTIALS; }

extern "C" int wf_pack_ternary_noalloc(const void* w, int w_dtype, int64_t N, int64_t K, int64_t ldw, int mode, float eps,
                                       uint8_t* codes_out, float* scale_out, void* stream) {
    WF_REQUIRE(w && codes_out && scale_out, "wf_pack_ternary_noalloc: null pointer");
    WF_REQUIRE(N > 0 && K > 0 && K % 64 == 0, "wf_pack_ternary_noalloc: need N > 0 and K a positive multiple of 64 (N=%lld K=%lld)",
               (long long)N, (long long)K);
    if (N > WF_PACK_NOALLOC_MAX_WEIGHTS / K)
        return fail(WF_E_LIMIT, "wf_pack_ternary_noalloc: %lld x %lld weights exceed the maximum of %lld for the allocation-free "
                                "entry point; use wf_pack_ternary with caller scratch",
                    (long long)N, (long long)K, (long long)WF_PACK_NOALLOC_MAX_WEIGHTS);
    WF_REQUIRE(is_float_dtype(w_dtype), "wf_pack_ternary_noalloc: unsupported weight dtype %d", w_dtype);
    WF_REQUIRE(mode >= WF_PACK_FP32 && mode <= WF_PACK_CAST_F16, "wf_pack_ternary_noalloc: unknown mode %d", mode);
    WF_REQUIRE(ldw >= K && (ldw * dtype_size(w_dtype)) % 16 == 0, "wf_pack_ternary_noalloc: row stride must cover K and keep rows 16-byte aligned");
    WF_REQUIRE(reinterpret_cast<uintptr_t>(w) % 16 == 0 && reinterpret_cast<uintptr_t>(codes_out) % 16 == 0,
               "wf_pack_ternary_noalloc: w and codes_out must be 16-byte aligned");
    if (int rc = require_device()) return rc;
    double* partial = nullptr;
    if (int rc = noalloc_scratch(&partial)) return rc;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    switch (w_dtype) {
        case WF_F32: return launch_pack<WF_F32>(w, N, K, ldw, mode, eps, codes_out, scale_out, partial, st);
        case WF_BF16: return launch_pack<WF_BF16>(w, N, K, ldw, mode, eps, codes_out, scale_out, partial, st);
        default: return launch_pack<WF_F16>(w, N, K, ldw, mode, eps, codes_out, scale_out, partial, st);
    }
}
