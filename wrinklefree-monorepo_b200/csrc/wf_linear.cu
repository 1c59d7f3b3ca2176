// Dense bf16 linear layer for the one full-precision matrix of a ternary decoder: the output head (and the embedding
// tied to it).  y[M, N] = x[M, K] · w[N, K]^T with bf16 operands and fp32 accumulation in tensor memory.
//
// In the decode step the head is read once per token batch (1.05 GB for a 128 k vocabulary of width 4096) and is
// bound by HBM: the weights sit on the MMA's M side (a tile = 128 rows of w), the tokens on its N side (up to 256 per
// tile), so one pass over w serves the whole batch.  Persistent CTAs, one per SM, walk the row tiles; K advances in
// stages of 128 (two 128-byte swizzle atoms per operand):
//   * warp 0 (one lane): TMA of the stage's rows of w (2 x 128 rows x 128 bytes) and of the token tile (2 x NTOK rows x
//     128 bytes) into a ring of shared-memory stages, one mbarrier per stage counting the bytes of both;
//   * warp 1 (one lane): eight tcgen05.mma.cta_group::1.kind::f16 per stage (M = 128, N = NTOK, K = 16, both operands from
//     shared memory), one commit per stage, two accumulator buffers of NTOK columns;
//   * warps 2-5: epilogue, thread = row of w (tensor-memory lane): tcgen05.ld, conversion, store of y[token][row].
// The rows of w are requested before griddepcontrol.wait (they never depend on the previous kernel), the token tiles after it.
// Every mbarrier wait is bounded.
#include <cuda.h>

#include "wf_common.cuh"

namespace wf {
__device__ int g_linear_status = 0;
}
#define WF_STATUS_WORD ::wf::g_linear_status
#include "wf_async.cuh"

namespace wf {

constexpr int LN_BM = 128;        // rows of w per tile
constexpr int LN_ATOM_K = 64;     // bf16 elements per 128-byte swizzle atom
constexpr int LN_ATOMS = 2;       // atoms per stage
constexpr int LN_THREADS = 6 * 32;
constexpr int LN_A_BYTES = LN_ATOMS * LN_BM * 128;  // 32 KB of w per stage
constexpr int LN_MAX_STAGES = 8;

struct LinearParams {
    void* y;
    int y_dtype;
    int64_t ldy;
    int M, N, K;
    int ntok;      // token columns per tile: a multiple of 16, at most 256
    int stages;    // ring depth
    int tiles_n, tiles_m;
    int pdl;
};

__device__ __forceinline__ void ln_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory"); }
__device__ __forceinline__ void ln_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory"); }
__device__ __forceinline__ void ln_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n" ::"r"(smem_u32(bar)) : "memory");
}
// K-major operand tile with 128-byte swizzle: rows of 128 bytes, 8-row groups 1024 bytes apart.
__device__ __forceinline__ uint64_t ln_desc_sw128(uint32_t addr) {
    uint64_t d = 0;
    d |= static_cast<uint64_t>((addr & 0x3FFFF) >> 4);
    d |= static_cast<uint64_t>(1024 >> 4) << 32;
    d |= static_cast<uint64_t>(1) << 46;
    d |= static_cast<uint64_t>(2) << 61;
    return d;
}
// the four MMAs of one swizzle atom (K = 16 each: 32 bytes, 2 in descriptor units)
__device__ __forceinline__ void ln_mma_x4(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate_first) {
    asm volatile(
        "{\n .reg .pred p, q;\n .reg .b64 a1, a2, a3, b1, b2, b3;\n"
        " setp.ne.b32 p, %4, 0;\n setp.eq.b32 q, %5, %5;\n"
        " add.u64 a1, %1, 2;\n add.u64 a2, %1, 4;\n add.u64 a3, %1, 6;\n"
        " add.u64 b1, %2, 2;\n add.u64 b2, %2, 4;\n add.u64 b3, %2, 6;\n"
        " tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, {%5, %5, %5, %5}, p;\n"
        " tcgen05.mma.cta_group::1.kind::f16 [%0], a1, b1, %3, {%5, %5, %5, %5}, q;\n"
        " tcgen05.mma.cta_group::1.kind::f16 [%0], a2, b2, %3, {%5, %5, %5, %5}, q;\n"
        " tcgen05.mma.cta_group::1.kind::f16 [%0], a3, b3, %3, {%5, %5, %5, %5}, q;\n}\n" ::"r"(d_tmem),
        "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate_first), "r"(0u)
        : "memory");
}
__device__ __forceinline__ void ln_tmem_ld16(uint32_t addr, uint32_t (&v)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];\n"
        : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]), "=r"(v[9]),
          "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15])
        : "r"(addr));
    asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory");
}

__global__ void __launch_bounds__(LN_THREADS, 1)
    linear_bf16_kernel(const __grid_constant__ CUtensorMap tmap_w, const __grid_constant__ CUtensorMap tmap_x, const LinearParams p) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
    const int x_atom = p.ntok * 128;                 // bytes of one atom of the token tile
    const int stage_bytes = LN_A_BYTES + LN_ATOMS * x_atom;  // a multiple of 1024: ntok is a multiple of 16
    uint8_t* ring = smem;
    uint64_t* full = reinterpret_cast<uint64_t*>(ring + static_cast<size_t>(p.stages) * stage_bytes);
    uint64_t* empty = full + LN_MAX_STAGES;
    uint64_t* acc_full = empty + LN_MAX_STAGES;
    uint64_t* acc_empty = acc_full + 2;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);
    volatile int* poisoned = reinterpret_cast<volatile int*>(tmem_slot + 1);

    asm volatile("griddepcontrol.launch_dependents;\n" ::: "memory");
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int S = p.stages;
    const int kstages = (p.K + LN_ATOMS * LN_ATOM_K - 1) / (LN_ATOMS * LN_ATOM_K);  // a stage past K is zero-filled by the TMA unit
    const int total_tiles = p.tiles_n * p.tiles_m;  // row tiles vary fastest: neighbouring CTAs read the same token tile

    if (tid == 0) {
        for (int s = 0; s < S; ++s) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], 1);
        }
        for (int a = 0; a < 2; ++a) {
            mbar_init(&acc_full[a], 1);
            mbar_init(&acc_empty[a], 4);
        }
        *poisoned = 0;
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(smem_u32(tmem_slot)), "r"(512));
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::);
    }
    ln_fence_before();
    __syncthreads();
    ln_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        if (lane == 0) {
            // The first ring of stages: rows of w at once, token tiles after the previous kernel has finished.
            const long long total_stages = static_cast<long long>((total_tiles - blockIdx.x + gridDim.x - 1) / gridDim.x) * kstages;
            auto coords = [&](long long sit, int& row_w, int& row_x, int& k0) {
                const int t = blockIdx.x + static_cast<int>(sit / kstages) * gridDim.x;
                row_w = (t % p.tiles_n) * LN_BM;
                row_x = (t / p.tiles_n) * p.ntok;
                k0 = static_cast<int>(sit % kstages) * (LN_ATOMS * LN_ATOM_K);
            };
            const int head = static_cast<int>(total_stages < S ? total_stages : S);
            for (int sit = 0; sit < head; ++sit) {
                int row_w, row_x, k0;
                coords(sit, row_w, row_x, k0);
                uint8_t* st = ring + static_cast<size_t>(sit) * stage_bytes;
                mbar_expect_tx(&full[sit], stage_bytes);
#pragma unroll
                for (int j = 0; j < LN_ATOMS; ++j) tma_load_2d(st + j * (LN_BM * 128), &tmap_w, k0 + j * LN_ATOM_K, row_w, &full[sit]);
            }
            if (p.pdl) asm volatile("griddepcontrol.wait;\n" ::: "memory");
            for (int sit = 0; sit < head; ++sit) {
                int row_w, row_x, k0;
                coords(sit, row_w, row_x, k0);
                uint8_t* st = ring + static_cast<size_t>(sit) * stage_bytes + LN_A_BYTES;
#pragma unroll
                for (int j = 0; j < LN_ATOMS; ++j) tma_load_2d(st + j * x_atom, &tmap_x, k0 + j * LN_ATOM_K, row_x, &full[sit]);
            }
            for (long long sit = head; sit < total_stages; ++sit) {
                const int s = static_cast<int>(sit % S);
                int row_w, row_x, k0;
                coords(sit, row_w, row_x, k0);
                mbar_wait(&empty[s], static_cast<unsigned>((sit / S) - 1) & 1, poisoned);
                uint8_t* st = ring + static_cast<size_t>(s) * stage_bytes;
                mbar_expect_tx(&full[s], stage_bytes);
#pragma unroll
                for (int j = 0; j < LN_ATOMS; ++j) tma_load_2d(st + j * (LN_BM * 128), &tmap_w, k0 + j * LN_ATOM_K, row_w, &full[s]);
#pragma unroll
                for (int j = 0; j < LN_ATOMS; ++j) tma_load_2d(st + LN_A_BYTES + j * x_atom, &tmap_x, k0 + j * LN_ATOM_K, row_x, &full[s]);
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            // D = f32, A = B = bf16, both K-major, N = ntok, M = 128
            const uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | (static_cast<uint32_t>(p.ntok >> 3) << 17) |
                                   (static_cast<uint32_t>(LN_BM >> 4) << 24);
            long long sit = 0;
            int nt = 0;
            for (int t = blockIdx.x; t < total_tiles; t += gridDim.x, ++nt) {
                const int a = nt & 1;
                if (nt >= 2) mbar_wait(&acc_empty[a], ((nt >> 1) - 1) & 1, poisoned);
                ln_fence_after();
                const uint32_t d_tmem = tmem_base + a * 256;
                for (int g = 0; g < kstages; ++g, ++sit) {
                    const int s = static_cast<int>(sit % S);
                    mbar_wait(&full[s], static_cast<unsigned>(sit / S) & 1, poisoned);
                    ln_fence_after();
                    const uint32_t st = smem_u32(ring + static_cast<size_t>(s) * stage_bytes);
#pragma unroll
                    for (int j = 0; j < LN_ATOMS; ++j)
                        ln_mma_x4(d_tmem, ln_desc_sw128(st + j * (LN_BM * 128)), ln_desc_sw128(st + LN_A_BYTES + j * x_atom), idesc,
                                  (g | j) ? 1u : 0u);
                    ln_commit(&empty[s]);
                }
                ln_commit(&acc_full[a]);
            }
        }
    } else {
        // ---- epilogue: thread = row of w (tensor-memory lane), registers = tokens
        const int quarter = warp & 3;  // the lanes this warp may read
        const int r = quarter * 32 + lane;
        if (p.pdl) asm volatile("griddepcontrol.wait;\n" ::: "memory");  // y may still be read by the previous kernel
        int nt = 0;
        for (int t = blockIdx.x; t < total_tiles; t += gridDim.x, ++nt) {
            const int a = nt & 1;
            const int nrow = (t % p.tiles_n) * LN_BM + r;
            const int tok0 = (t / p.tiles_n) * p.ntok;
            const int mtok = min(p.ntok, p.M - tok0);
            const bool row_ok = nrow < p.N;
            mbar_wait(&acc_full[a], (nt >> 1) & 1, poisoned);
            ln_fence_after();
            for (int c0 = 0; c0 < p.ntok; c0 += 16) {
                uint32_t v[16];
                ln_tmem_ld16(tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + a * 256 + c0, v);
                if (c0 + 16 >= p.ntok) {  // every column of this warp's lanes is in registers: hand the buffer back
                    ln_fence_before();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(&acc_empty[a]);
                }
                if (!row_ok) continue;
#pragma unroll
                for (int jt = 0; jt < 16; ++jt) {
                    const int tok_in = c0 + jt;
                    if (tok_in < mtok) {
                        const float o = __uint_as_float(v[jt]);
                        const int64_t off = static_cast<int64_t>(tok0 + tok_in) * p.ldy + nrow;
                        if (p.y_dtype == WF_F32)
                            static_cast<float*>(p.y)[off] = o;
                        else if (p.y_dtype == WF_BF16)
                            static_cast<__nv_bfloat16*>(p.y)[off] = __float2bfloat16_rn(o);
                        else
                            static_cast<__half*>(p.y)[off] = __float2half_rn(o);
                    }
                }
            }
        }
    }
    ln_fence_before();
    __syncthreads();
    if (warp == 1) {
        ln_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem_base), "r"(512));
    }
}

typedef CUresult (*LnEncodeFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                               const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                               CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static LnEncodeFn ln_encode_fn() {
    static LnEncodeFn fn = nullptr;
    if (!fn) {
        void* q = nullptr;
        cudaDriverEntryPointQueryResult r;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &q, cudaEnableDefault, &r) == cudaSuccess && r == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<LnEncodeFn>(q);
    }
    return fn;
}

}  // namespace wf

using namespace wf;

extern "C" int wf_linear_bf16(const void* x, int64_t ldx, const void* w, int64_t ldw, void* y, int y_dtype, int64_t ldy, int64_t M,
                              int64_t N, int64_t K, unsigned flags, void* stream) {
    WF_REQUIRE(x && w && y, "wf_linear_bf16: null pointer");
    WF_REQUIRE(M >= 1 && N >= 1 && K >= 8 && K % 8 == 0, "wf_linear_bf16: M, N >= 1 and K a positive multiple of 8 (K = %lld)", (long long)K);
    WF_REQUIRE(M <= 0x7fffffffLL && N <= 0x7fffffffLL && K <= 0x7fffffffLL, "wf_linear_bf16: sizes beyond 2^31");
    WF_REQUIRE(ldx >= K && ldw >= K && ldx % 8 == 0 && ldw % 8 == 0, "wf_linear_bf16: row strides must be multiples of 8 elements, at least K");
    WF_REQUIRE(ldy >= N, "wf_linear_bf16: ldy < N");
    WF_REQUIRE(y_dtype == WF_F32 || y_dtype == WF_BF16 || y_dtype == WF_F16, "wf_linear_bf16: y must be f32, bf16 or f16");
    WF_REQUIRE((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(w)) % 16 == 0, "wf_linear_bf16: x and w must be 16-byte aligned");
    if (int rc = require_device()) return rc;
    LnEncodeFn enc = ln_encode_fn();
    if (!enc) return fail(WF_E_DEVICE, "cuTensorMapEncodeTiled is not available in this driver");
    LinearParams p;
    p.y = y; p.y_dtype = y_dtype; p.ldy = ldy;
    p.M = static_cast<int>(M); p.N = static_cast<int>(N); p.K = static_cast<int>(K);
    const int64_t m16 = (M + 15) / 16 * 16;
    p.ntok = static_cast<int>(m16 < 256 ? m16 : 256);
    p.tiles_n = static_cast<int>((N + LN_BM - 1) / LN_BM);
    p.tiles_m = static_cast<int>((M + p.ntok - 1) / p.ntok);
    p.pdl = (flags & WF_FLAG_PDL) ? 1 : 0;
    const size_t stage_bytes = LN_A_BYTES + static_cast<size_t>(LN_ATOMS) * p.ntok * 128;
    const size_t budget = 227 * 1024 - 1024 - 1024;  // alignment slack, barriers
    int stages = static_cast<int>(budget / stage_bytes);
    if (stages > LN_MAX_STAGES) stages = LN_MAX_STAGES;
    p.stages = stages;  // >= 2: a stage is at most 96 KB
    const size_t smem = 1024 + stages * stage_bytes + 1024;
    alignas(64) CUtensorMap tmap_w, tmap_x;
    const cuuint32_t ones[2] = {1, 1};
    {
        const cuuint64_t dims[2] = {static_cast<cuuint64_t>(K), static_cast<cuuint64_t>(N)};
        const cuuint64_t strides[1] = {static_cast<cuuint64_t>(ldw) * 2};
        const cuuint32_t box[2] = {LN_ATOM_K, LN_BM};
        CUresult r = enc(&tmap_w, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(w), dims, strides, box, ones,
                         CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                         CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (r != CUDA_SUCCESS) return fail(WF_E_DEVICE, "cuTensorMapEncodeTiled (weights) failed with %d", (int)r);
    }
    {
        const cuuint64_t dims[2] = {static_cast<cuuint64_t>(K), static_cast<cuuint64_t>(M)};
        const cuuint64_t strides[1] = {static_cast<cuuint64_t>(ldx) * 2};
        const cuuint32_t box[2] = {LN_ATOM_K, static_cast<cuuint32_t>(p.ntok)};
        CUresult r = enc(&tmap_x, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(x), dims, strides, box, ones,
                         CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                         CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (r != CUDA_SUCCESS) return fail(WF_E_DEVICE, "cuTensorMapEncodeTiled (activations) failed with %d", (int)r);
    }
    static PerDeviceOnce configured;
    const int dev = current_device();
    if (configured.needs(dev)) {
        WF_CUDA(cudaFuncSetAttribute(linear_bf16_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024));
        configured.mark(dev);
    }
    const int sms = num_sms();
    const long long tiles = static_cast<long long>(p.tiles_n) * p.tiles_m;
    cudaLaunchConfig_t lc = {};
    lc.gridDim = dim3(static_cast<unsigned>(tiles < sms ? tiles : sms));
    lc.blockDim = dim3(LN_THREADS);
    lc.dynamicSmemBytes = smem;
    lc.stream = static_cast<cudaStream_t>(stream);
    cudaLaunchAttribute attr[1];
    if (p.pdl) {
        attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[0].val.programmaticStreamSerializationAllowed = 1;
        lc.attrs = attr;
        lc.numAttrs = 1;
    }
    WF_CUDA(cudaLaunchKernelEx(&lc, linear_bf16_kernel, tmap_w, tmap_x, p));
    return WF_OK;
}

// read-out for wf_device_status: the status word of this file's kernel (cleared when set)
extern "C" int wf_linear_status_fetch(int* out) {
    WF_CUDA(cudaMemcpyFromSymbol(out, g_linear_status, sizeof(int)));
    if (*out) {
        int zero = 0;
        WF_CUDA(cudaMemcpyToSymbol(g_linear_status, &zero, sizeof(int)));
    }
    return WF_OK;
}
